// Small row-wise / element-wise ops a Llama graph needs between the mat-muls so
// that no node leaves the device: RMS_NORM, NORM, ADD/SUB/MUL/DIV with
// broadcasting, unary activations, SCALE, CLAMP, ROPE (normal + NeoX, YaRN,
// frequency factors), CPY/DUP/CONT with type conversion (incl. F32 -> Q8_0/Q4_0
// for a quantized KV cache), GET_ROWS with on-the-fly dequantization, SOFT_MAX.
//
// Semantics follow the reference CPU ops (ggml/src/ggml-cpu/ggml-cpu.c:
// rms_norm 7015, rope 9366, get_rows 8464, soft_max 8900ff, dup 3390ff) and the
// behaviour of ggml/src/ggml-cuda/{norm,binbcast,unary,rope,cpy,getrows,softmax}.cu.
// All of these are HBM-bound; they are fused where the graph allows
// (rms_norm*weight, silu*up, both optionally emitting the int8 activation
// blocks the following mat-vec consumes).
#include "common.cuh"
#include "kernels.h"
#include <math.h>

namespace b200 {

#define B200_LAUNCH_CHECK() cudaGetLastError()

__device__ __forceinline__ float block_sum(float v, float * sh /* >= 32 floats */) {
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    if (lane == 0) sh[w] = v;
    __syncthreads();
    float r = (threadIdx.x < nw) ? sh[threadIdx.x] : 0.0f;
    if (w == 0) { r = warp_sum(r); if (lane == 0) sh[0] = r; }
    __syncthreads();
    r = sh[0];
    __syncthreads();
    return r;
}
__device__ __forceinline__ float block_max(float v, float * sh) {
    v = warp_max(v);
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    if (lane == 0) sh[w] = v;
    __syncthreads();
    float r = (threadIdx.x < nw) ? sh[threadIdx.x] : -INFINITY;
    if (w == 0) { r = warp_max(r); if (lane == 0) sh[0] = r; }
    __syncthreads();
    r = sh[0];
    __syncthreads();
    return r;
}

__device__ __forceinline__ float ld_f(const void * p, int type) {
    if (type == T_F32) return *(const float *) p;
    if (type == T_F16) return __half2float(*(const __half *) p);
    return __bfloat162float(*(const __nv_bfloat16 *) p);
}
__device__ __forceinline__ void st_f(void * p, int type, float v) {
    if (type == T_F32) *(float *) p = v;
    else if (type == T_F16) *(__half *) p = __float2half(v);
    else *(__nv_bfloat16 *) p = __float2bfloat16(v);
}

// quantize four values that are already scaled and write one blk_act128 group
// (used by the fused producers below): each thread owns 4 consecutive values of
// a row, 8 threads form one 32-value group
__device__ __forceinline__ void emit_act128(const float (&v)[4], int64_t k0, int64_t K, blk_act128 * col) {
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float d  = amax / 127.0f;
    const float id = amax > 0.0f ? 127.0f / amax : 0.0f;
    int q[4], qsum = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) { q[i] = __float2int_rn(v[i] * id); qsum += q[i]; }
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) qsum += __shfl_xor_sync(0xffffffffu, qsum, o);
    if (k0 < K) {
        blk_act128 * yb = col + (k0 >> 7);
        const uint32_t packed = (uint32_t) (q[0] & 0xff) | ((uint32_t) (q[1] & 0xff) << 8) |
                                ((uint32_t) (q[2] & 0xff) << 16) | ((uint32_t) (q[3] & 0xff) << 24);
        ((uint32_t *) yb->q)[(k0 & 127) >> 2] = packed;
        if (((k0 >> 2) & 7) == 0) yb->ds[(k0 & 127) >> 5] = make_float2(d, d * (float) qsum);
    }
}

// ---------------------------------------------------------------------------
// RMS_NORM (+ optional weight multiply, + optional activation quantization)
// ---------------------------------------------------------------------------
template <bool HAS_W, bool EMIT>
__global__ void rms_norm_kernel(const TensorD src, const TensorD w, const TensorD dst, float eps, blk_act128 * act, float * norm_out,
                                const float * addend, float * sum_out, __half * h16) {
    pdl_enter();
    __shared__ float sh[32];
    const int64_t row = blockIdx.x;
    const int64_t i1 = row % src.ne[1], i2 = (row / src.ne[1]) % src.ne[2], i3 = row / (src.ne[1] * src.ne[2]);
    const float * x = (const float *) ((const char *) src.data + i1 * src.nb[1] + i2 * src.nb[2] + i3 * src.nb[3]);
    float *       y = (float *) ((char *) dst.data + i1 * dst.nb[1] + i2 * dst.nb[2] + i3 * dst.nb[3]);
    const int64_t n = src.ne[0];
    const float * wr = nullptr;
    if (HAS_W) wr = (const float *) ((const char *) w.data + (i1 % w.ne[1]) * w.nb[1] + (i2 % w.ne[2]) * w.nb[2] + (i3 % w.ne[3]) * w.nb[3]);
    float * yn = norm_out ? norm_out + row * n : nullptr;
    const int64_t npad = (n + 127) & ~(int64_t) 127;
    blk_act128 * col = EMIT ? act + row * (npad >> 7) : nullptr;

    // fast path (the usual case: one row of a few thousand values): every thread keeps its values (up to four groups of
    // four) in registers between the reduction and the output, so the row is read exactly once
    constexpr int MAXV = 4;
    const int nv = (int) ((npad / 4 + blockDim.x - 1) / blockDim.x);
    const bool fast = (n & 3) == 0 && nv <= MAXV && (!HAS_W || w.ne[0] == n) &&
                      (((uintptr_t) x | (uintptr_t) y | (uintptr_t) wr | (uintptr_t) yn | (uintptr_t) addend | (uintptr_t) sum_out) & 15) == 0;
    if (fast) {
        float4 v[MAXV];
        float part = 0.0f;
#pragma unroll
        for (int j = 0; j < MAXV; ++j) {
            v[j] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            const int64_t k0 = ((int64_t) j * blockDim.x + threadIdx.x) * 4;
            if (j < nv && k0 < n) {
                v[j] = *(const float4 *) (x + k0);
                if (addend) {
                    const float4 a4 = *(const float4 *) (addend + row * n + k0);
                    v[j].x += a4.x; v[j].y += a4.y; v[j].z += a4.z; v[j].w += a4.w;
                    *(float4 *) (sum_out + row * n + k0) = v[j];
                }
                part += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
            }
        }
        const float ss = block_sum(part, sh);
        const float scale = rsqrtf(ss / (float) n + eps);
#pragma unroll
        for (int j = 0; j < MAXV; ++j) {
            const int64_t k0 = ((int64_t) j * blockDim.x + threadIdx.x) * 4;
            if (j >= nv) break;
            const bool in = k0 < n;
            float o[4] = {v[j].x * scale, v[j].y * scale, v[j].z * scale, v[j].w * scale};
            if (in && yn) *(float4 *) (yn + k0) = make_float4(o[0], o[1], o[2], o[3]);
            if (HAS_W && in) { const float4 wv = *(const float4 *) (wr + k0); o[0] *= wv.x; o[1] *= wv.y; o[2] *= wv.z; o[3] *= wv.w; }
            if (in) *(float4 *) (y + k0) = make_float4(o[0], o[1], o[2], o[3]);
            if (in && h16) {                                          // F16 copy for a tensor-core mat-mul (dense rows of n)
                __half2 h0 = __floats2half2_rn(o[0], o[1]), h1 = __floats2half2_rn(o[2], o[3]);
                *(uint2 *) (h16 + row * n + k0) = make_uint2(*(uint32_t *) &h0, *(uint32_t *) &h1);
            }
            if (EMIT && k0 < npad) emit_act128(o, k0, npad, col);     // whole warps take this branch together (npad % 128 == 0)
        }
        return;
    }

    float ss = 0.0f;
    if (addend) {
        // fused residual add: x + addend is written to sum_out (contiguous rows) and normalised from there
        float * so = sum_out + row * n;
        const float * ad = addend + row * n;
        for (int64_t i = threadIdx.x; i < n; i += blockDim.x) { const float v = x[i] + ad[i]; so[i] = v; ss += v * v; }
        x = so;
    } else {
        for (int64_t i = threadIdx.x; i < n; i += blockDim.x) { const float v = x[i]; ss += v * v; }
    }
    ss = block_sum(ss, sh);                        // (its barriers also make the sums written above visible to the block)
    const float scale = rsqrtf(ss / (float) n + eps);
    if (!EMIT) {
        for (int64_t i = threadIdx.x; i < n; i += blockDim.x) {
            float v = x[i] * scale;
            if (yn) yn[i] = v;
            if (HAS_W) v *= wr[i % w.ne[0]];
            y[i] = v;
            if (h16) h16[row * n + i] = __float2half_rn(v);
        }
    } else {
        // 4 consecutive values per thread so that 8 threads cover one 32-value group
        for (int64_t k0 = (int64_t) threadIdx.x * 4; k0 < npad; k0 += (int64_t) blockDim.x * 4) {
            float v[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                v[i] = 0.0f;
                if (k0 + i < n) {
                    v[i] = x[k0 + i] * scale;
                    if (yn) yn[k0 + i] = v[i];
                    if (HAS_W) v[i] *= wr[(k0 + i) % w.ne[0]];
                    y[k0 + i] = v[i];
                    if (h16) h16[row * n + k0 + i] = __float2half_rn(v[i]);
                }
            }
            emit_act128(v, k0, npad, col);
        }
    }
}

// threads per row: 16 values each where the row allows it (more rows resident per SM, one short reduction)
static int row_block(int64_t n) { const int64_t b = ((n + 15) / 16 + 31) & ~(int64_t) 31; return (int) (b < 128 ? 128 : (b > 1024 ? 1024 : b)); }

cudaError_t launch_rms_norm(const TensorD & src, const TensorD & dst, float eps, const LaunchCtx & c) {
    const int64_t rows = src.ne[1] * src.ne[2] * src.ne[3];
    if (rows == 0 || src.ne[0] == 0) return cudaSuccess;
    (void) (launch_err = launch_k(c.use_pdl, c.stream, rms_norm_kernel<false, false>, dim3((unsigned) rows), dim3(row_block(src.ne[0])), 0, src, src, dst, eps, nullptr, nullptr, nullptr, nullptr, nullptr));
    return B200_LAUNCH_CHECK();
}
cudaError_t launch_rms_norm_mul(const TensorD & src, const TensorD & w, const TensorD & dst, float eps, void * act, float * norm_out,
                                const float * addend, float * sum_out, const LaunchCtx & c, void * f16_out) {
    const int64_t rows = src.ne[1] * src.ne[2] * src.ne[3];
    if (rows == 0 || src.ne[0] == 0) return cudaSuccess;
    if (act) (void) (launch_err = launch_k(c.use_pdl, c.stream, rms_norm_kernel<true, true>, dim3((unsigned) rows), dim3(row_block(src.ne[0])), 0, src, w, dst, eps, (blk_act128 *) act, norm_out, addend, sum_out, (__half *) f16_out));
    else     (void) (launch_err = launch_k(c.use_pdl, c.stream, rms_norm_kernel<true, false>, dim3((unsigned) rows), dim3(row_block(src.ne[0])), 0, src, w, dst, eps, nullptr, norm_out, addend, sum_out, (__half *) f16_out));
    return B200_LAUNCH_CHECK();
}

// NORM: (x - mean) / sqrt(var + eps)
__global__ void norm_kernel(const TensorD src, const TensorD dst, float eps) {
    pdl_enter();
    __shared__ float sh[32];
    const int64_t row = blockIdx.x;
    const int64_t i1 = row % src.ne[1], i2 = (row / src.ne[1]) % src.ne[2], i3 = row / (src.ne[1] * src.ne[2]);
    const float * x = (const float *) ((const char *) src.data + i1 * src.nb[1] + i2 * src.nb[2] + i3 * src.nb[3]);
    float *       y = (float *) ((char *) dst.data + i1 * dst.nb[1] + i2 * dst.nb[2] + i3 * dst.nb[3]);
    const int64_t n = src.ne[0];
    float s = 0.0f;
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) s += x[i];
    const float mean = block_sum(s, sh) / (float) n;
    float v2 = 0.0f;
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) { const float d = x[i] - mean; v2 += d * d; }
    const float var = block_sum(v2, sh) / (float) n;
    const float scale = rsqrtf(var + eps);
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) y[i] = (x[i] - mean) * scale;
}
cudaError_t launch_norm(const TensorD & src, const TensorD & dst, float eps, const LaunchCtx & c) {
    const int64_t rows = src.ne[1] * src.ne[2] * src.ne[3];
    if (rows == 0 || src.ne[0] == 0) return cudaSuccess;
    (void) (launch_err = launch_k(c.use_pdl, c.stream, norm_kernel, dim3((unsigned) rows), dim3(row_block(src.ne[0])), 0, src, dst, eps));
    return B200_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------
// broadcasting binary ops
// ---------------------------------------------------------------------------
template <int OP> __device__ __forceinline__ float bin_apply(float a, float b) {
    if (OP == BIN_ADD) return a + b;
    if (OP == BIN_SUB) return a - b;
    if (OP == BIN_MUL) return a * b;
    return a / b;
}

template <int OP>
__global__ void bin_bcast_kernel(const TensorD a, const TensorD b, const TensorD d, int64_t total) {
    pdl_enter();
    for (int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t) gridDim.x * blockDim.x) {
        const int64_t i0 = i % d.ne[0], r1 = i / d.ne[0];
        const int64_t i1 = r1 % d.ne[1], r2 = r1 / d.ne[1];
        const int64_t i2 = r2 % d.ne[2], i3 = r2 / d.ne[2];
        const char * pa = (const char *) a.data + (i0 % a.ne[0]) * a.nb[0] + (i1 % a.ne[1]) * a.nb[1] + (i2 % a.ne[2]) * a.nb[2] + (i3 % a.ne[3]) * a.nb[3];
        const char * pb = (const char *) b.data + (i0 % b.ne[0]) * b.nb[0] + (i1 % b.ne[1]) * b.nb[1] + (i2 % b.ne[2]) * b.nb[2] + (i3 % b.ne[3]) * b.nb[3];
        char *       pd = (char *) d.data + i0 * d.nb[0] + i1 * d.nb[1] + i2 * d.nb[2] + i3 * d.nb[3];
        st_f(pd, d.type, bin_apply<OP>(ld_f(pa, a.type), ld_f(pb, b.type)));
    }
}

// fast path: all F32, a and dst contiguous with identical shape, b contiguous with
// shape either identical or a single row [ne0]; 4 elements per thread
template <int OP>
__global__ void bin_fast_kernel(const float4 * __restrict__ a, const float4 * __restrict__ b, float4 * __restrict__ d,
                                int64_t n4, int64_t b_n4 /* elements/4 of b (row or full) */) {
    pdl_enter();
    for (int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (int64_t) gridDim.x * blockDim.x) {
        const float4 x = a[i], y = b[i % b_n4];
        d[i] = make_float4(bin_apply<OP>(x.x, y.x), bin_apply<OP>(x.y, y.y), bin_apply<OP>(x.z, y.z), bin_apply<OP>(x.w, y.w));
    }
}

static bool is_contig(const TensorD & t) {
    int64_t s = type_block_bytes(t.type);
    if (type_block_elems(t.type) != 1) return false;
    for (int i = 0; i < 4; ++i) { if (t.ne[i] != 1 && t.nb[i] != s) return false; s *= t.ne[i]; }
    return true;
}
static int64_t nelem(const TensorD & t) { return t.ne[0] * t.ne[1] * t.ne[2] * t.ne[3]; }
static unsigned grid_for(int64_t n, int block, int sm) {
    int64_t g = (n + block - 1) / block;
    const int64_t cap = (int64_t) sm * 16;
    if (g > cap) g = cap;
    return (unsigned) (g < 1 ? 1 : g);
}

template <int OP>
static cudaError_t bin_dispatch(const TensorD & a, const TensorD & b, const TensorD & d, const LaunchCtx & c) {
    const int64_t total = nelem(d);
    if (total == 0) return cudaSuccess;
    const bool f32 = a.type == T_F32 && b.type == T_F32 && d.type == T_F32;
    bool same_a = true;
    for (int i = 0; i < 4; ++i) same_a = same_a && a.ne[i] == d.ne[i];
    const int64_t nb_ = nelem(b);
    const bool b_full = nb_ == total, b_row = nb_ == b.ne[0] && b.ne[0] == d.ne[0];
    if (f32 && same_a && is_contig(a) && is_contig(b) && is_contig(d) && (b_full || b_row) && d.ne[0] % 4 == 0 &&
        ((uintptr_t) a.data % 16 == 0) && ((uintptr_t) b.data % 16 == 0) && ((uintptr_t) d.data % 16 == 0)) {
        bool same_b = true;
        if (b_full) for (int i = 0; i < 4; ++i) same_b = same_b && b.ne[i] == d.ne[i];
        if (same_b) {
            (void) (launch_err = launch_k(c.use_pdl, c.stream, bin_fast_kernel<OP>, dim3(grid_for(total / 4, 256, c.sm_count)), dim3(256), 0, 
                (const float4 *) a.data, (const float4 *) b.data, (float4 *) d.data, total / 4, nb_ / 4));
            return B200_LAUNCH_CHECK();
        }
    }
    (void) (launch_err = launch_k(c.use_pdl, c.stream, bin_bcast_kernel<OP>, dim3(grid_for(total, 256, c.sm_count)), dim3(256), 0, a, b, d, total));
    return B200_LAUNCH_CHECK();
}

cudaError_t launch_bin_bcast(int op, const TensorD & a, const TensorD & b, const TensorD & d, const LaunchCtx & c) {
    switch (op) {
        case BIN_ADD: return bin_dispatch<BIN_ADD>(a, b, d, c);
        case BIN_SUB: return bin_dispatch<BIN_SUB>(a, b, d, c);
        case BIN_MUL: return bin_dispatch<BIN_MUL>(a, b, d, c);
        case BIN_DIV: return bin_dispatch<BIN_DIV>(a, b, d, c);
    }
    return cudaErrorInvalidValue;
}

// ---------------------------------------------------------------------------
// unary ops (contiguous F32)
// ---------------------------------------------------------------------------
__device__ __forceinline__ float un_apply(int op, float x) {
    switch (op) {
        case UN_SILU:        return x / (1.0f + expf(-x));
        case UN_GELU:        return 0.5f * x * (1.0f + tanhf(0.79788456080286535587989211986876f * x * (1.0f + 0.044715f * x * x)));
        case UN_GELU_QUICK:  return x * (1.0f / (1.0f + expf(-1.702f * x)));
        case UN_RELU:        return fmaxf(x, 0.0f);
        case UN_TANH:        return tanhf(x);
        case UN_SIGMOID:     return 1.0f / (1.0f + expf(-x));
        case UN_NEG:         return -x;
        case UN_EXP:         return expf(x);
        case UN_ABS:         return fabsf(x);
        case UN_SGN:         return x > 0.0f ? 1.0f : (x < 0.0f ? -1.0f : 0.0f);
        case UN_STEP:        return x > 0.0f ? 1.0f : 0.0f;
        case UN_ELU:         return x > 0.0f ? x : expm1f(x);
        case UN_HARDSIGMOID: return fminf(1.0f, fmaxf(0.0f, (x + 3.0f) / 6.0f));
        case UN_HARDSWISH:   return x * fminf(1.0f, fmaxf(0.0f, (x + 3.0f) / 6.0f));
        case UN_SQR:         return x * x;
        case UN_SQRT:        return sqrtf(x);
        case UN_SIN:         return sinf(x);
        case UN_COS:         return cosf(x);
        case UN_LOG:         return logf(x);
    }
    return x;
}
__global__ void unary_kernel(int op, const float * __restrict__ x, float * __restrict__ y, int64_t n) {
    pdl_enter();
    for (int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t) gridDim.x * blockDim.x) y[i] = un_apply(op, x[i]);
}
cudaError_t launch_unary(int op, const TensorD & src, const TensorD & dst, const LaunchCtx & c) {
    const int64_t n = nelem(src);
    if (n == 0) return cudaSuccess;
    (void) (launch_err = launch_k(c.use_pdl, c.stream, unary_kernel, dim3(grid_for(n, 256, c.sm_count)), dim3(256), 0, op, (const float *) src.data, (float *) dst.data, n));
    return B200_LAUNCH_CHECK();
}

__global__ void scale_kernel(const float * __restrict__ x, float * __restrict__ y, float s, int64_t n) {
    pdl_enter();
    for (int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t) gridDim.x * blockDim.x) y[i] = x[i] * s;
}
cudaError_t launch_scale(const TensorD & src, const TensorD & dst, float s, const LaunchCtx & c) {
    const int64_t n = nelem(src);
    if (n == 0) return cudaSuccess;
    (void) (launch_err = launch_k(c.use_pdl, c.stream, scale_kernel, dim3(grid_for(n, 256, c.sm_count)), dim3(256), 0, (const float *) src.data, (float *) dst.data, s, n));
    return B200_LAUNCH_CHECK();
}
__global__ void clamp_kernel(const float * __restrict__ x, float * __restrict__ y, float lo, float hi, int64_t n) {
    pdl_enter();
    for (int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t) gridDim.x * blockDim.x) y[i] = fminf(fmaxf(x[i], lo), hi);
}
cudaError_t launch_clamp(const TensorD & src, const TensorD & dst, float lo, float hi, const LaunchCtx & c) {
    const int64_t n = nelem(src);
    if (n == 0) return cudaSuccess;
    (void) (launch_err = launch_k(c.use_pdl, c.stream, clamp_kernel, dim3(grid_for(n, 256, c.sm_count)), dim3(256), 0, (const float *) src.data, (float *) dst.data, lo, hi, n));
    return B200_LAUNCH_CHECK();
}

// silu(gate) * up on contiguous F32 rows, optionally emitting activation blocks
template <bool EMIT>
// (no __restrict__: graph allocators compute silu in place of gate and the product in place of either operand)
__global__ void silu_mul_kernel(const float * g, const float * u, float * y,
                                int64_t n0, int64_t rows, blk_act128 * act, float * silu_out, __half * h16) {
    pdl_enter();
    const int64_t npad = (n0 + 127) & ~(int64_t) 127;
    const int64_t per_row = npad / 4;
    const int64_t total = per_row * rows;
    // rows that are whole 128-value blocks at 16-byte aligned addresses: 128-bit loads and stores, no row arithmetic
    if (n0 == npad && ((((uintptr_t) g | (uintptr_t) u | (uintptr_t) y | (uintptr_t) silu_out) & 15) == 0) && (((uintptr_t) h16 & 7) == 0)) {
        for (int64_t t = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t) gridDim.x * blockDim.x) {
            const float4 a4 = ((const float4 *) g)[t], u4 = ((const float4 *) u)[t];
            const float4 s4 = make_float4(a4.x / (1.0f + expf(-a4.x)), a4.y / (1.0f + expf(-a4.y)), a4.z / (1.0f + expf(-a4.z)), a4.w / (1.0f + expf(-a4.w)));
            float v[4] = {s4.x * u4.x, s4.y * u4.y, s4.z * u4.z, s4.w * u4.w};
            if (silu_out) ((float4 *) silu_out)[t] = s4;
            ((float4 *) y)[t] = make_float4(v[0], v[1], v[2], v[3]);
            if (h16) {
                __half2 h0 = __floats2half2_rn(v[0], v[1]), h1 = __floats2half2_rn(v[2], v[3]);
                ((uint2 *) h16)[t] = make_uint2(*(uint32_t *) &h0, *(uint32_t *) &h1);
            }
            if (EMIT) { const int64_t row = t / per_row; emit_act128(v, (t - row * per_row) * 4, npad, act + row * (npad >> 7)); }
        }
        return;
    }
    // whole warps stay together (emit_act128 shuffles), so loop bounds are warp-uniform
    const int64_t total_w = (total + 31) & ~(int64_t) 31;
    for (int64_t t = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; t < total_w; t += (int64_t) gridDim.x * blockDim.x) {
        const int64_t row = t / per_row, k0 = (t % per_row) * 4;
        float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        if (t < total) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (k0 + i < n0) {
                    const float a = g[row * n0 + k0 + i];
                    const float sa = a / (1.0f + expf(-a));
                    if (silu_out) silu_out[row * n0 + k0 + i] = sa;
                    v[i] = sa * u[row * n0 + k0 + i];
                    y[row * n0 + k0 + i] = v[i];
                    if (h16) h16[row * n0 + k0 + i] = __float2half_rn(v[i]);
                }
            }
        }
        if (EMIT) emit_act128(v, t < total ? k0 : npad, npad, act + (t < total ? row : 0) * (npad >> 7));
    }
}
cudaError_t launch_silu_mul(const TensorD & gate, const TensorD & up, const TensorD & dst, void * act, float * silu_out, const LaunchCtx & c, void * f16_out) {
    const int64_t n0 = gate.ne[0], rows = nelem(gate) / (n0 ? n0 : 1);
    if (n0 == 0 || rows == 0) return cudaSuccess;
    const int64_t threads = ((n0 + 127) / 128 * 32) * rows;
    if (act) (void) (launch_err = launch_k(c.use_pdl, c.stream, silu_mul_kernel<true>, dim3(grid_for(threads, 256, c.sm_count)), dim3(256), 0, 
                 (const float *) gate.data, (const float *) up.data, (float *) dst.data, n0, rows, (blk_act128 *) act, silu_out, (__half *) f16_out));
    else     (void) (launch_err = launch_k(c.use_pdl, c.stream, silu_mul_kernel<false>, dim3(grid_for(threads, 256, c.sm_count)), dim3(256), 0, 
                 (const float *) gate.data, (const float *) up.data, (float *) dst.data, n0, rows, nullptr, silu_out, (__half *) f16_out));
    return B200_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------
// ROPE
// ---------------------------------------------------------------------------
struct RopeK {
    int n_dims, neox;
    float freq_scale, ext_factor, attn_factor, theta_scale, corr0, corr1;
};
__device__ __forceinline__ void rope_cs(const RopeK & r, float theta_extrap, int i0, float & c, float & s) {
    // YaRN mix of interpolated and extrapolated angles (ggml-cpu.c:9275-9306)
    const float theta_interp = r.freq_scale * theta_extrap;
    float theta = theta_interp, mscale = r.attn_factor;
    if (r.ext_factor != 0.0f) {
        const float y = ((float) (i0 / 2) - r.corr0) / fmaxf(0.001f, r.corr1 - r.corr0);
        const float ramp_mix = (1.0f - fminf(1.0f, fmaxf(0.0f, y))) * r.ext_factor;
        theta = theta_interp * (1.0f - ramp_mix) + theta_extrap * ramp_mix;
        mscale *= 1.0f + 0.1f * logf(1.0f / r.freq_scale);
    }
    c = cosf(theta) * mscale;
    s = sinf(theta) * mscale;
}
template <typename T>
__global__ void rope_kernel(const TensorD src, const int32_t * __restrict__ pos, const float * __restrict__ ff,
                            const TensorD dst, const RopeK r, int64_t total_pairs) {
    pdl_enter();
    const int64_t half0 = src.ne[0] / 2;
    for (int64_t t = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; t < total_pairs; t += (int64_t) gridDim.x * blockDim.x) {
        const int64_t ip = t % half0, r1 = t / half0;
        const int64_t i1 = r1 % src.ne[1], r2 = r1 / src.ne[1];
        const int64_t i2 = r2 % src.ne[2], i3 = r2 / src.ne[2];
        const char * xs = (const char *) src.data + i1 * src.nb[1] + i2 * src.nb[2] + i3 * src.nb[3];
        char *       yd = (char *) dst.data + i1 * dst.nb[1] + i2 * dst.nb[2] + i3 * dst.nb[3];
        const int i0 = (int) (2 * ip);
        if (i0 >= r.n_dims) {
            ((T *) yd)[i0] = ((const T *) xs)[i0];
            ((T *) yd)[i0 + 1] = ((const T *) xs)[i0 + 1];
            continue;
        }
        const float theta_base = (float) pos[i2] * powf(r.theta_scale, (float) ip);
        const float f = ff ? ff[ip] : 1.0f;
        float c, s;
        rope_cs(r, theta_base / f, i0, c, s);
        const int64_t ia = r.neox ? ip : i0, ib = r.neox ? ip + r.n_dims / 2 : i0 + 1;
        const float x0 = (float) ((const T *) xs)[ia], x1 = (float) ((const T *) xs)[ib];
        ((T *) yd)[ia] = (T) (x0 * c - x1 * s);
        ((T *) yd)[ib] = (T) (x0 * s + x1 * c);
    }
}
cudaError_t launch_rope(const TensorD & src, const int32_t * pos, const float * ff, const TensorD & dst,
                        const RopeParams & rp, const LaunchCtx & c) {
    const int64_t total = nelem(src) / 2;
    if (total == 0) return cudaSuccess;
    RopeK r;
    r.n_dims = rp.n_dims; r.neox = (rp.mode & 2) ? 1 : 0;
    r.freq_scale = rp.freq_scale; r.ext_factor = rp.ext_factor; r.attn_factor = rp.attn_factor;
    r.theta_scale = powf(rp.freq_base, -2.0f / (float) rp.n_dims);
    // correction range of YaRN (ggml_rope_yarn_corr_dims, ggml/src/ggml.c)
    auto corr_dim = [&](float n_rot) {
        return (float) rp.n_dims * logf((float) rp.n_ctx_orig / (n_rot * 2.0f * 3.14159265358979323846f)) / (2.0f * logf(rp.freq_base));
    };
    const float start = floorf(corr_dim(rp.beta_fast)), end = ceilf(corr_dim(rp.beta_slow));
    r.corr0 = fmaxf(0.0f, start);
    r.corr1 = fminf((float) rp.n_dims - 1.0f, end);
    if (src.type == T_F32)      (void) (launch_err = launch_k(c.use_pdl, c.stream, rope_kernel<float>, dim3(grid_for(total, 256, c.sm_count)), dim3(256), 0, src, pos, ff, dst, r, total));
    else if (src.type == T_F16) (void) (launch_err = launch_k(c.use_pdl, c.stream, rope_kernel<__half>, dim3(grid_for(total, 256, c.sm_count)), dim3(256), 0, src, pos, ff, dst, r, total));
    else return cudaErrorInvalidValue;
    return B200_LAUNCH_CHECK();
}

// ROPE of the query and key projections plus the KV-cache store of one layer in a single launch
// (src/llama.cpp:157-199 and :1511-1531 emit ROPE, ROPE, CPY, CPY): work items are rotation pairs of Q,
// rotation pairs of K (written as F32 and, rounded to F16, into the cache rows), then pairs of V values
// (F32 -> F16 into the cache rows).  Q, K, V are contiguous [hd, n_head, n_tok] F32; the cache row
// offsets are read from device memory so that a captured launch stays valid from token to token.
struct RopeKvArgs {
    const float * q_src; float * q_dst; int64_t q_pairs;      // n_tok * n_head   * hd / 2
    const float * k_src; float * k_dst; int64_t k_pairs;      // n_tok * n_head_kv * hd / 2
    const float * v_src; int64_t v_pairs;
    __half * k_cache; __half * v_cache;                        // bases of the viewed cache tensors
    const int64_t * k_off; const int64_t * v_off;             // byte offsets of the views (device memory) or null
    int64_t k_off_imm, v_off_imm;                             // ... used when the pointers are null
    const int32_t * pos; const float * ff;
    int hd, n_head, n_head_kv;
    RopeK r;
};
// Block layout: blocks [0, n_tok * hb) take one token and ROPE_HPB heads of the combined list (query heads, then key
// heads): the cos / sin pair of every rotation index is computed once per block into shared memory and applied to all its
// heads.  The blocks after those convert V.
static constexpr int ROPE_HPB = 8;          // heads per block
static constexpr int ROPE_MAX_HALF = 256;   // head sizes up to 512
__global__ void rope_kv_kernel(const RopeKvArgs a, int64_t n_tok, int hb) {
    pdl_enter();
    __shared__ float2 cs[ROPE_MAX_HALF];
    const int half_hd = a.hd / 2;
    __half * kc = (__half *) ((char *) a.k_cache + (a.k_off ? *a.k_off : a.k_off_imm));
    __half * vc = (__half *) ((char *) a.v_cache + (a.v_off ? *a.v_off : a.v_off_imm));
    const int64_t rope_blocks = n_tok * hb;
    if ((int64_t) blockIdx.x >= rope_blocks) {
        // V: F32 -> F16 into the cache rows
        const int64_t nvb = (int64_t) gridDim.x - rope_blocks;
        const int64_t quads = a.v_pairs / 2;
        for (int64_t i = ((int64_t) blockIdx.x - rope_blocks) * blockDim.x + threadIdx.x; i < quads; i += nvb * blockDim.x) {
            const float4 v = ((const float4 *) a.v_src)[i];
            __half2 h0 = __floats2half2_rn(v.x, v.y), h1 = __floats2half2_rn(v.z, v.w);
            ((uint2 *) vc)[i] = make_uint2(*(uint32_t *) &h0, *(uint32_t *) &h1);
        }
        if ((a.v_pairs & 1) && blockIdx.x == rope_blocks && threadIdx.x == 0) {
            const float2 v = ((const float2 *) a.v_src)[a.v_pairs - 1];
            ((__half2 *) vc)[a.v_pairs - 1] = __floats2half2_rn(v.x, v.y);
        }
        return;
    }
    const int64_t tok = blockIdx.x / hb;
    const int h0 = (int) (blockIdx.x % hb) * ROPE_HPB;
    const int h1 = min(h0 + ROPE_HPB, a.n_head + a.n_head_kv);
    const int half_rot = min(a.r.n_dims / 2, half_hd);
    const float p = (float) a.pos[tok];
    for (int ip = threadIdx.x; ip < half_rot; ip += blockDim.x) {
        const float theta_base = p * powf(a.r.theta_scale, (float) ip);
        const float f = a.ff ? a.ff[ip] : 1.0f;
        float c, sn;
        rope_cs(a.r, theta_base / f, 2 * ip, c, sn);
        cs[ip] = make_float2(c, sn);
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < (h1 - h0) * half_hd; idx += blockDim.x) {
        const int head = h0 + idx / half_hd, ip = idx % half_hd;
        const bool is_k = head >= a.n_head;
        const int64_t rowi = is_k ? tok * a.n_head_kv + (head - a.n_head) : tok * a.n_head + head;
        const float * xs = (is_k ? a.k_src : a.q_src) + rowi * a.hd;
        float *       yd = (is_k ? a.k_dst : a.q_dst) + rowi * a.hd;
        const int i0 = 2 * ip;
        float o0, o1; int ia, ib;
        if (i0 >= a.r.n_dims) { ia = i0; ib = i0 + 1; o0 = xs[ia]; o1 = xs[ib]; }
        else {
            const float2 c = cs[ip];
            ia = a.r.neox ? ip : i0; ib = a.r.neox ? ip + a.r.n_dims / 2 : i0 + 1;
            const float x0 = xs[ia], x1 = xs[ib];
            o0 = x0 * c.x - x1 * c.y; o1 = x0 * c.y + x1 * c.x;
        }
        if (ib == ia + 1) *(float2 *) (yd + ia) = make_float2(o0, o1);      // (hd is even and rows are 8-byte aligned)
        else { yd[ia] = o0; yd[ib] = o1; }
        if (is_k) {
            if (ib == ia + 1) *(__half2 *) (kc + rowi * a.hd + ia) = __floats2half2_rn(o0, o1);
            else { kc[rowi * a.hd + ia] = __float2half_rn(o0); kc[rowi * a.hd + ib] = __float2half_rn(o1); }
        }
    }
}
static RopeK make_ropek(const RopeParams & rp) {
    RopeK r;
    r.n_dims = rp.n_dims; r.neox = (rp.mode & 2) ? 1 : 0;
    r.freq_scale = rp.freq_scale; r.ext_factor = rp.ext_factor; r.attn_factor = rp.attn_factor;
    r.theta_scale = powf(rp.freq_base, -2.0f / (float) rp.n_dims);
    auto corr_dim = [&](float n_rot) {
        return (float) rp.n_dims * logf((float) rp.n_ctx_orig / (n_rot * 2.0f * 3.14159265358979323846f)) / (2.0f * logf(rp.freq_base));
    };
    r.corr0 = fmaxf(0.0f, floorf(corr_dim(rp.beta_fast)));
    r.corr1 = fminf((float) rp.n_dims - 1.0f, ceilf(corr_dim(rp.beta_slow)));
    return r;
}
cudaError_t launch_rope_kv(const RopeKvLaunch & l, const RopeParams & rp, const LaunchCtx & c) {
    RopeKvArgs a;
    a.q_src = l.q_src; a.q_dst = l.q_dst; a.q_pairs = l.n_tok * l.n_head * l.hd / 2;
    a.k_src = l.k_src; a.k_dst = l.k_dst; a.k_pairs = l.n_tok * l.n_head_kv * l.hd / 2;
    a.v_src = l.v_src; a.v_pairs = l.v_elems / 2;
    a.k_cache = (__half *) l.k_cache; a.v_cache = (__half *) l.v_cache;
    a.k_off = l.k_off_dev; a.v_off = l.v_off_dev; a.k_off_imm = l.k_off; a.v_off_imm = l.v_off;
    a.pos = l.pos; a.ff = l.ff; a.hd = (int) l.hd; a.n_head = (int) l.n_head; a.n_head_kv = (int) l.n_head_kv;
    a.r = make_ropek(rp);
    const int64_t total = a.q_pairs + a.k_pairs + a.v_pairs;
    if (total == 0) return cudaSuccess;
    if (l.hd / 2 > ROPE_MAX_HALF || (l.hd & 1)) return cudaErrorInvalidValue;
    const int hb = (int) ((l.n_head + l.n_head_kv + ROPE_HPB - 1) / ROPE_HPB);
    int64_t vblocks = (a.v_pairs / 2 + 1023) / 1024; if (vblocks > 4 * c.sm_count) vblocks = 4 * c.sm_count; if (a.v_pairs && vblocks < 1) vblocks = 1;
    (void) (launch_err = launch_k(c.use_pdl, c.stream, rope_kv_kernel, dim3((unsigned) (l.n_tok * hb + vblocks)), dim3(256), 0, a, (int64_t) l.n_tok, hb));
    return B200_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------
// CPY / DUP / CONT
// ---------------------------------------------------------------------------
__global__ void cpy_elem_kernel(const TensorD s, const TensorD d, int64_t total, const int64_t * __restrict__ dyn_off) {
    pdl_enter();
    const int64_t doff = dyn_off ? *dyn_off : 0;   // byte offset of the destination view, kept in device memory so a captured launch stays valid
    for (int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t) gridDim.x * blockDim.x) {
        int64_t r = i;
        const int64_t s0 = r % s.ne[0]; r /= s.ne[0];
        const int64_t s1 = r % s.ne[1]; r /= s.ne[1];
        const int64_t s2 = r % s.ne[2]; const int64_t s3 = r / s.ne[2];
        r = i;
        const int64_t d0 = r % d.ne[0]; r /= d.ne[0];
        const int64_t d1 = r % d.ne[1]; r /= d.ne[1];
        const int64_t d2 = r % d.ne[2]; const int64_t d3 = r / d.ne[2];
        const char * ps = (const char *) s.data + s0 * s.nb[0] + s1 * s.nb[1] + s2 * s.nb[2] + s3 * s.nb[3];
        char *       pd = (char *) d.data + doff + d0 * d.nb[0] + d1 * d.nb[1] + d2 * d.nb[2] + d3 * d.nb[3];
        if (s.type == d.type) {
            if (s.type == T_F32 || s.type == T_I32) *(uint32_t *) pd = *(const uint32_t *) ps;
            else *(uint16_t *) pd = *(const uint16_t *) ps;
        } else {
            st_f(pd, d.type, ld_f(ps, s.type));
        }
    }
}

// F32 -> quantized block (32 values): one thread per block, restating
// quantize_row_q8_0_ref / q4_0_ref / q4_1_ref / q5_0_ref / q5_1_ref
// (ggml/src/ggml-quants.c:31-217) operation by operation (no fused multiply-add)
// blocks are 2-byte aligned; scales are stored with one explicit 16-bit store
__device__ __forceinline__ void st_h(uint8_t * p, float v) { *(uint16_t *) p = __half_as_ushort(__float2half_rn(v)); }

template <int QT>
__device__ void quantize_block32(const float * x, uint8_t * out) {
    if (QT == T_Q8_0) {
        float amax = 0.0f;
        for (int j = 0; j < 32; ++j) amax = fmaxf(amax, fabsf(x[j]));
        const float d = __fdiv_rn(amax, 127.0f);
        const float id = d ? __fdiv_rn(1.0f, d) : 0.0f;
        blk_q8_0 * b = (blk_q8_0 *) out;
        st_h(out, d);
        for (int j = 0; j < 32; ++j) b->qs[j] = (int8_t) roundf(__fmul_rn(x[j], id));
    } else if (QT == T_Q4_0 || QT == T_Q5_0) {
        float amax = 0.0f, mx = 0.0f;
        for (int j = 0; j < 32; ++j) { const float v = x[j]; if (amax < fabsf(v)) { amax = fabsf(v); mx = v; } }
        const float d = __fdiv_rn(mx, QT == T_Q4_0 ? -8.0f : -16.0f);
        const float id = d ? __fdiv_rn(1.0f, d) : 0.0f;
        if (QT == T_Q4_0) {
            blk_q4_0 * b = (blk_q4_0 *) out;
            st_h(out, d);
            for (int j = 0; j < 16; ++j) {
                const float x0 = __fmul_rn(x[j], id), x1 = __fmul_rn(x[16 + j], id);
                const uint8_t q0 = (uint8_t) min(15, (int) (int8_t) __fadd_rn(x0, 8.5f));
                const uint8_t q1 = (uint8_t) min(15, (int) (int8_t) __fadd_rn(x1, 8.5f));
                b->qs[j] = q0 | (q1 << 4);
            }
        } else {
            blk_q5_0 * b = (blk_q5_0 *) out;
            st_h(out, d);
            uint32_t qh = 0;
            for (int j = 0; j < 16; ++j) {
                const float x0 = __fmul_rn(x[j], id), x1 = __fmul_rn(x[16 + j], id);
                const uint8_t q0 = (uint8_t) min(31, (int) (int8_t) __fadd_rn(x0, 16.5f));
                const uint8_t q1 = (uint8_t) min(31, (int) (int8_t) __fadd_rn(x1, 16.5f));
                b->qs[j] = (q0 & 0x0F) | ((q1 & 0x0F) << 4);
                qh |= ((q0 & 0x10u) >> 4) << (j + 0);
                qh |= ((q1 & 0x10u) >> 4) << (j + 16);
            }
            b->qh[0] = qh & 0xff; b->qh[1] = (qh >> 8) & 0xff; b->qh[2] = (qh >> 16) & 0xff; b->qh[3] = (qh >> 24) & 0xff;
        }
    } else {   // Q4_1 / Q5_1
        float mn = INFINITY, mx = -INFINITY;
        for (int j = 0; j < 32; ++j) { mn = fminf(mn, x[j]); mx = fmaxf(mx, x[j]); }
        const int levels = QT == T_Q4_1 ? 15 : 31;
        const float d = __fdiv_rn(__fsub_rn(mx, mn), (float) levels);
        const float id = d ? __fdiv_rn(1.0f, d) : 0.0f;
        if (QT == T_Q4_1) {
            blk_q4_1 * b = (blk_q4_1 *) out;
            st_h(out, d); st_h(out + 2, mn);
            for (int j = 0; j < 16; ++j) {
                const float x0 = __fmul_rn(__fsub_rn(x[j], mn), id), x1 = __fmul_rn(__fsub_rn(x[16 + j], mn), id);
                const uint8_t q0 = (uint8_t) min(15, (int) (int8_t) __fadd_rn(x0, 0.5f));
                const uint8_t q1 = (uint8_t) min(15, (int) (int8_t) __fadd_rn(x1, 0.5f));
                b->qs[j] = q0 | (q1 << 4);
            }
        } else {
            blk_q5_1 * b = (blk_q5_1 *) out;
            st_h(out, d); st_h(out + 2, mn);
            uint32_t qh = 0;
            for (int j = 0; j < 16; ++j) {
                const float x0 = __fmul_rn(__fsub_rn(x[j], mn), id), x1 = __fmul_rn(__fsub_rn(x[16 + j], mn), id);
                const uint8_t q0 = (uint8_t) (int8_t) __fadd_rn(x0, 0.5f);
                const uint8_t q1 = (uint8_t) (int8_t) __fadd_rn(x1, 0.5f);
                b->qs[j] = (q0 & 0x0F) | ((q1 & 0x0F) << 4);
                qh |= ((q0 & 0x10u) >> 4) << (j + 0);
                qh |= ((q1 & 0x10u) >> 4) << (j + 16);
            }
            b->qh[0] = qh & 0xff; b->qh[1] = (qh >> 8) & 0xff; b->qh[2] = (qh >> 16) & 0xff; b->qh[3] = (qh >> 24) & 0xff;
        }
    }
}

template <int QT>
__global__ void cpy_f32_q_kernel(const TensorD s, const TensorD d, int64_t nblocks, const int64_t * __restrict__ dyn_off) {
    pdl_enter();
    const int bb = type_block_bytes(QT);
    const int64_t doff = dyn_off ? *dyn_off : 0;
    for (int64_t ib = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; ib < nblocks; ib += (int64_t) gridDim.x * blockDim.x) {
        // element index of the first value of this block, in src order
        int64_t r = ib * 32;
        const int64_t s0 = r % s.ne[0]; r /= s.ne[0];
        const int64_t s1 = r % s.ne[1]; r /= s.ne[1];
        const int64_t s2 = r % s.ne[2]; const int64_t s3 = r / s.ne[2];
        r = ib * 32;
        const int64_t d0 = r % d.ne[0]; r /= d.ne[0];
        const int64_t d1 = r % d.ne[1]; r /= d.ne[1];
        const int64_t d2 = r % d.ne[2]; const int64_t d3 = r / d.ne[2];
        const char * ps = (const char *) s.data + s0 * s.nb[0] + s1 * s.nb[1] + s2 * s.nb[2] + s3 * s.nb[3];
        char *       pd = (char *) d.data + doff + (d0 / 32) * bb + d1 * d.nb[1] + d2 * d.nb[2] + d3 * d.nb[3];
        float v[32];
        for (int j = 0; j < 32; ++j) v[j] = *(const float *) (ps + j * s.nb[0]);
        quantize_block32<QT>(v, (uint8_t *) pd);
    }
}

bool cpy_supported(int st, int dt) {
    auto flt = [](int t) { return t == T_F32 || t == T_F16 || t == T_BF16; };
    if (flt(st) && flt(dt)) return true;
    if (st == T_I32 && dt == T_I32) return true;
    if (st == T_F32 && (dt == T_Q8_0 || dt == T_Q4_0 || dt == T_Q4_1 || dt == T_Q5_0 || dt == T_Q5_1)) return true;
    return false;
}

cudaError_t launch_cpy(const TensorD & s, const TensorD & d, const LaunchCtx & c, const int64_t * dyn_off) {
    const int64_t total = nelem(s);
    if (total == 0) return cudaSuccess;
    if (type_block_elems(d.type) == 32) {
        const int64_t nb = total / 32;
        const unsigned g = grid_for(nb, 128, c.sm_count);
        switch (d.type) {
            case T_Q8_0: (void) (launch_err = launch_k(c.use_pdl, c.stream, cpy_f32_q_kernel<T_Q8_0>, dim3(g), dim3(128), 0, s, d, nb, dyn_off)); break;
            case T_Q4_0: (void) (launch_err = launch_k(c.use_pdl, c.stream, cpy_f32_q_kernel<T_Q4_0>, dim3(g), dim3(128), 0, s, d, nb, dyn_off)); break;
            case T_Q4_1: (void) (launch_err = launch_k(c.use_pdl, c.stream, cpy_f32_q_kernel<T_Q4_1>, dim3(g), dim3(128), 0, s, d, nb, dyn_off)); break;
            case T_Q5_0: (void) (launch_err = launch_k(c.use_pdl, c.stream, cpy_f32_q_kernel<T_Q5_0>, dim3(g), dim3(128), 0, s, d, nb, dyn_off)); break;
            case T_Q5_1: (void) (launch_err = launch_k(c.use_pdl, c.stream, cpy_f32_q_kernel<T_Q5_1>, dim3(g), dim3(128), 0, s, d, nb, dyn_off)); break;
            default: return cudaErrorInvalidValue;
        }
        return B200_LAUNCH_CHECK();
    }
    (void) (launch_err = launch_k(c.use_pdl, c.stream, cpy_elem_kernel, dim3(grid_for(total, 256, c.sm_count)), dim3(256), 0, s, d, total, dyn_off));
    return B200_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------
// GET_ROWS
// ---------------------------------------------------------------------------
template <int T>
__global__ void get_rows_kernel(const TensorD src, const TensorD idx, const TensorD dst) {
    pdl_enter();
    // grid: x over chunks of the row, y = index position, z = batch (i11 + i12*ne11)
    const int64_t i10 = blockIdx.y;
    const int64_t i11 = blockIdx.z % idx.ne[1], i12 = blockIdx.z / idx.ne[1];
    const int32_t row = *(const int32_t *) ((const char *) idx.data + i10 * idx.nb[0] + i11 * idx.nb[1] + i12 * idx.nb[2]);
    const uint8_t * sr = (const uint8_t *) src.data + (int64_t) row * src.nb[1] + i11 * src.nb[2] + i12 * src.nb[3];
    float * dr = (float *) ((char *) dst.data + i10 * dst.nb[1] + i11 * dst.nb[2] + i12 * dst.nb[3]);
    for (int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; i < src.ne[0]; i += (int64_t) gridDim.x * blockDim.x)
        dr[i] = dequant_elem<T>(sr, i);
}
bool get_rows_supported(int t) {
    switch (t) {
        case T_F32: case T_F16: case T_BF16: case T_Q4_0: case T_Q4_1: case T_Q5_0: case T_Q5_1: case T_Q8_0: case T_IQ4_NL: case T_IQ4_XS:
        case T_Q2_K: case T_Q3_K: case T_Q4_K: case T_Q5_K: case T_Q6_K: return true;
        default: return false;
    }
}
cudaError_t launch_get_rows(const TensorD & src, const TensorD & idx, const TensorD & dst, const LaunchCtx & c) {
    if (nelem(dst) == 0) return cudaSuccess;
    const int block = 256;
    int64_t gx = (src.ne[0] + block - 1) / block; if (gx > 64) gx = 64;
    dim3 grid((unsigned) gx, (unsigned) idx.ne[0], (unsigned) (idx.ne[1] * idx.ne[2]));
#define GR(T) case T: (void) (launch_err = launch_k(c.use_pdl, c.stream, get_rows_kernel<T>, dim3(grid), dim3(block), 0, src, idx, dst)); break;
    switch (src.type) {
        GR(T_F32) GR(T_F16) GR(T_BF16) GR(T_Q4_0) GR(T_Q4_1) GR(T_Q5_0) GR(T_Q5_1) GR(T_Q8_0) GR(T_Q4_K) GR(T_Q5_K) GR(T_Q6_K) GR(T_Q2_K) GR(T_Q3_K) GR(T_IQ4_NL) GR(T_IQ4_XS)
        default: return cudaErrorInvalidValue;
    }
#undef GR
    return B200_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------
// SOFT_MAX: y = softmax(x*scale + slope(head)*mask) per row
// ---------------------------------------------------------------------------
__global__ void soft_max_kernel(const TensorD src, const TensorD mask, int has_mask, const TensorD dst,
                                float scale, float max_bias, float m0, float m1, int n_head_log2) {
    pdl_enter();
    extern __shared__ float row_cache[];
    __shared__ float sh[32];
    const int64_t row = blockIdx.x;
    const int64_t ne0 = src.ne[0], ne1 = src.ne[1];
    const int64_t i1 = row % ne1, h = (row / ne1) % src.ne[2];
    const float * x = (const float *) src.data + row * ne0;
    float *       y = (float *) dst.data + row * ne0;
    float slope = 1.0f;
    if (max_bias > 0.0f) slope = h < n_head_log2 ? powf(m0, (float) (h + 1)) : powf(m1, (float) (2 * (h - n_head_log2) + 1));
    const char * mrow = has_mask ? (const char *) mask.data + i1 * mask.nb[1] : nullptr;
    float mx = -INFINITY;
    for (int64_t i = threadIdx.x; i < ne0; i += blockDim.x) {
        float v = x[i] * scale;
        if (has_mask) v += slope * ld_f(mrow + i * mask.nb[0], mask.type);
        row_cache[i] = v;
        mx = fmaxf(mx, v);
    }
    mx = block_max(mx, sh);
    float sum = 0.0f;
    for (int64_t i = threadIdx.x; i < ne0; i += blockDim.x) {
        const float e = expf(row_cache[i] - mx);
        row_cache[i] = e;
        sum += e;
    }
    sum = block_sum(sum, sh);
    const float inv = 1.0f / sum;
    for (int64_t i = threadIdx.x; i < ne0; i += blockDim.x) y[i] = row_cache[i] * inv;
}
cudaError_t launch_soft_max(const TensorD & src, const TensorD * mask, const TensorD & dst, float scale, float max_bias, const LaunchCtx & c) {
    const int64_t rows = src.ne[1] * src.ne[2] * src.ne[3];
    if (rows == 0 || src.ne[0] == 0) return cudaSuccess;
    const int n_head = (int) src.ne[2];
    int n_head_log2 = 1; while (n_head_log2 * 2 <= n_head) n_head_log2 *= 2;
    const float m0 = powf(2.0f, -max_bias / (float) n_head_log2), m1 = powf(2.0f, -(max_bias / 2.0f) / (float) n_head_log2);
    const size_t smem = (size_t) src.ne[0] * sizeof(float);
    static unsigned attr_mask = 0;
    if (smem > 48 * 1024 && !(attr_mask & (1u << c.device))) {
        cudaError_t e = cudaFuncSetAttribute(soft_max_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return e;
        attr_mask |= 1u << c.device;
    }
    if (smem > 200 * 1024) return cudaErrorInvalidValue;
    (void) (launch_err = launch_k(c.use_pdl, c.stream, soft_max_kernel, dim3((unsigned) rows), dim3(row_block(src.ne[0])), smem, src, mask ? *mask : src, mask ? 1 : 0, dst,
                                                                               scale, max_bias, m0, m1, n_head_log2));
    return B200_LAUNCH_CHECK();
}

}  // namespace b200
