// FLASH_ATTN_EXT over an F16 K/V cache (ggml_flash_attn_ext, ggml/src/ggml.c:4306-4345;
// CPU semantics ggml/src/ggml-cpu/ggml-cpu.c:10916-11129):
//
//   O[d, h, q] = sum_k softmax_k( scale * K[k, h/g] . Q[q, h]  (softcap)  + slope_h * mask[q, k] ) * V[k, h/g][d]
//
// with Q F32 [D, n_q, n_head, n3], K/V F16 [D, n_kv, n_head_kv, n3] as arbitrary
// strided views of the cache, mask F16 [n_kv, >= n_q] and dst F32 [D, n_head, n_q, n3].
//
// Split-KV ("flash decoding"): the KV range of one (query, head) is divided over
// CTAs so that a single decode token at 32K context still fills every SM;
// partial (max, sum, O) triples go to a workspace and are merged by a second
// kernel.  Softmax statistics and the PV accumulation are FP32 (libllama asks for
// GGML_PREC_F32 on this op, src/llama.cpp:595).
#include "common.cuh"
#include "kernels.h"
#include <math.h>

namespace b200 {

static constexpr int FA_WARPS = 4;

struct FaK {
    const char * q; int64_t q_nb1, q_nb2, q_nb3;
    const char * k; int64_t k_nb1, k_nb2, k_nb3;
    const char * v; int64_t v_nb1, v_nb2, v_nb3;
    const char * mask; int64_t m_nb1;
    float * dst;
    float * ws;               // [rows][n_splits][D + 2]
    int n_q, n_kv, n_head, gqa, q3_per_k3;
    int n_splits, kv_per_split;
    float scale, softcap, max_bias, m0, m1; int n_head_log2;
};

template <int D, int KT, int VT>
__global__ void __launch_bounds__(FA_WARPS * 32) fattn_vec_kernel(const FaK p) {
    pdl_enter();
    constexpr int DPL = (D + 31) / 32;            // head-dim elements per lane
    __shared__ float qs[D];
    __shared__ float mg_m[FA_WARPS], mg_l[FA_WARPS];
    __shared__ float mg_o[FA_WARPS][D];

    const int split = blockIdx.x, head = blockIdx.y;
    const int iq = blockIdx.z % p.n_q, i3 = blockIdx.z / p.n_q;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    const float * qrow = (const float *) (p.q + (int64_t) iq * p.q_nb1 + (int64_t) head * p.q_nb2 + (int64_t) i3 * p.q_nb3);
    for (int d = threadIdx.x; d < D; d += blockDim.x) qs[d] = qrow[d];
    __syncthreads();

    const int hk = head / p.gqa, k3 = i3 / p.q3_per_k3;
    const char * kbase = p.k + (int64_t) hk * p.k_nb2 + (int64_t) k3 * p.k_nb3;
    const char * vbase = p.v + (int64_t) hk * p.v_nb2 + (int64_t) k3 * p.v_nb3;
    const __half * mrow = p.mask ? (const __half *) (p.mask + (int64_t) iq * p.m_nb1) : nullptr;

    float slope = 1.0f;
    if (p.max_bias > 0.0f)
        slope = head < p.n_head_log2 ? powf(p.m0, (float) (head + 1)) : powf(p.m1, (float) (2 * (head - p.n_head_log2) + 1));

    const int kv0 = split * p.kv_per_split;
    const int kv1 = min(p.n_kv, kv0 + p.kv_per_split);

    float m = -INFINITY, l = 0.0f, o[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) o[i] = 0.0f;

    for (int base = kv0 + warp * 32; base < kv1; base += FA_WARPS * 32) {
        const int j = base + lane;
        float s = -INFINITY;
        if (j < kv1) {
            const float mv = mrow ? slope * __half2float(mrow[j]) : 0.0f;
            if (mv != -INFINITY) {
                float acc = 0.0f;
                if (KT == T_F16) {
                    const __half2 * kr = (const __half2 *) (kbase + (int64_t) j * p.k_nb1);
#pragma unroll 8
                    for (int d2 = 0; d2 < D / 2; ++d2) {
                        const float2 kk = __half22float2(kr[d2]);
                        acc += kk.x * qs[2 * d2] + kk.y * qs[2 * d2 + 1];
                    }
                } else {
                    // quantized K cache (Q8_0 / Q4_0 blocks of 32 along the head dimension): dequantized on the fly
                    const uint8_t * kr = (const uint8_t *) (kbase + (int64_t) j * p.k_nb1);
#pragma unroll 8
                    for (int d = 0; d < D; ++d) acc += dequant_elem<KT>(kr, d) * qs[d];
                }
                s = acc * p.scale;
                if (p.softcap != 0.0f) s = p.softcap * tanhf(s);
                s += mv;
            }
        }
        const float m_new = fmaxf(m, warp_max(s));
        if (m_new == -INFINITY) continue;         // everything so far is masked out
        const float pj   = (s == -INFINITY) ? 0.0f : expf(s - m_new);
        const float corr = (m == -INFINITY) ? 0.0f : expf(m - m_new);
        l = l * corr + warp_sum(pj);
        m = m_new;
#pragma unroll
        for (int i = 0; i < DPL; ++i) o[i] *= corr;
        for (int jj = 0; jj < 32; ++jj) {
            const float pp = __shfl_sync(0xffffffffu, pj, jj);
            if (pp == 0.0f) continue;             // warp-uniform; also covers rows past kv1
            const uint8_t * vr = (const uint8_t *) (vbase + (int64_t) (base + jj) * p.v_nb1);
#pragma unroll
            for (int i = 0; i < DPL; ++i) {
                const int d = lane + 32 * i;
                if (d < D) o[i] += pp * dequant_elem<VT>(vr, d);
            }
        }
    }

    // merge the warps of this CTA
    if (lane == 0) { mg_m[warp] = m; mg_l[warp] = l; }
#pragma unroll
    for (int i = 0; i < DPL; ++i) { const int d = lane + 32 * i; if (d < D) mg_o[warp][d] = o[i]; }
    __syncthreads();
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < FA_WARPS; ++w) M = fmaxf(M, mg_m[w]);
    float L = 0.0f;
#pragma unroll
    for (int w = 0; w < FA_WARPS; ++w) L += (mg_m[w] == -INFINITY) ? 0.0f : mg_l[w] * expf(mg_m[w] - M);

    const int64_t row = ((int64_t) i3 * p.n_q + iq) * p.n_head + head;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float acc = 0.0f;
#pragma unroll
        for (int w = 0; w < FA_WARPS; ++w) acc += (mg_m[w] == -INFINITY) ? 0.0f : mg_o[w][d] * expf(mg_m[w] - M);
        if (p.n_splits == 1) p.dst[row * D + d] = acc / L;
        else                 p.ws[(row * p.n_splits + split) * (D + 2) + d] = acc;
    }
    if (p.n_splits > 1 && threadIdx.x == 0) {
        p.ws[(row * p.n_splits + split) * (D + 2) + D]     = M;
        p.ws[(row * p.n_splits + split) * (D + 2) + D + 1] = L;
    }
}

// merges the per-split partials of one (query, head) row
template <int D>
__global__ void fattn_combine_kernel(const float * __restrict__ ws, float * __restrict__ dst, int n_splits) {
    pdl_enter();
    const int64_t row = blockIdx.x;
    const float * w = ws + row * n_splits * (D + 2);
    float M = -INFINITY;
    for (int s = 0; s < n_splits; ++s) M = fmaxf(M, w[s * (D + 2) + D]);
    float L = 0.0f;
    for (int s = 0; s < n_splits; ++s) {
        const float ms = w[s * (D + 2) + D];
        L += (ms == -INFINITY) ? 0.0f : w[s * (D + 2) + D + 1] * expf(ms - M);
    }
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float acc = 0.0f;
        for (int s = 0; s < n_splits; ++s) {
            const float ms = w[s * (D + 2) + D];
            if (ms != -INFINITY) acc += w[s * (D + 2) + d] * expf(ms - M);
        }
        dst[row * D + d] = acc / L;
    }
}

static inline bool t_is_q(int t) { return t == T_Q8_0 || t == T_Q4_0; }
// F16 K/V everywhere; a quantized KV cache (-ctk/-ctv q8_0, q4_0: 32-value blocks along the head dimension,
// reference kernels ggml/src/ggml-cuda/fattn-common.cuh:55-...) goes through the vec kernel
bool fattn_supported(int64_t D, int kt, int vt) {
    auto ok = [](int t) { return t == T_F16 || t == T_BF16 || t == T_Q8_0 || t == T_Q4_0; };
    if (!ok(kt) || !ok(vt)) return false;
    if ((kt == T_BF16 || vt == T_BF16) && kt != vt) return false;
    if ((t_is_q(kt) || t_is_q(vt)) && D % 32 != 0) return false;
    return D == 64 || D == 80 || D == 96 || D == 112 || D == 128 || D == 256;
}

static int fattn_pick_splits(int64_t rows, int64_t n_kv, int sm_count) {
    // enough CTAs for ~4 per SM, at least 256 KV positions per CTA
    int64_t want = ((int64_t) sm_count * 4 + rows - 1) / rows;
    int64_t max_by_kv = (n_kv + 255) / 256;
    int64_t s = want < max_by_kv ? want : max_by_kv;
    if (s < 1) s = 1;
    if (s > 128) s = 128;
    return (int) s;
}

size_t fattn_workspace_bytes(const TensorD & q, const TensorD & k, int sm_count) {
    const int64_t rows = q.ne[1] * q.ne[2] * q.ne[3];
    const int splits = fattn_pick_splits(rows, k.ne[1], sm_count);
    const size_t vec = splits > 1 ? (size_t) rows * splits * (q.ne[0] + 2) * sizeof(float) : 0;
    const size_t mma = fattn_mma_workspace_bytes(q, k), dec = fattn_dec_workspace_bytes(q, k, sm_count);
    const size_t m = vec > mma ? vec : mma;
    return m > dec ? m : dec;
}

template <int D>
static cudaError_t fattn_launch_d(const FaK & p, int kt, int vt, int64_t rows, int n3, const LaunchCtx & c) {
    dim3 grid((unsigned) p.n_splits, (unsigned) p.n_head, (unsigned) (p.n_q * n3));
    void (*kern)(FaK) = nullptr;
#define FA_PICK(K_, V_) if (kt == K_ && vt == V_) kern = fattn_vec_kernel<D, K_, V_>
    FA_PICK(T_F16, T_F16); FA_PICK(T_BF16, T_BF16);
    if (D % 32 == 0) {
        FA_PICK(T_Q8_0, T_Q8_0); FA_PICK(T_Q4_0, T_Q4_0); FA_PICK(T_Q8_0, T_F16); FA_PICK(T_F16, T_Q8_0);
        FA_PICK(T_Q4_0, T_F16); FA_PICK(T_F16, T_Q4_0); FA_PICK(T_Q8_0, T_Q4_0); FA_PICK(T_Q4_0, T_Q8_0);
    }
#undef FA_PICK
    if (!kern) return cudaErrorInvalidValue;
    (void) (launch_err = launch_k(c.use_pdl, c.stream, kern, dim3(grid), dim3(FA_WARPS * 32), 0, p));
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    if (p.n_splits > 1) {
        (void) (launch_err = launch_k(c.use_pdl, c.stream, fattn_combine_kernel<D>, dim3((unsigned) rows), dim3(D >= 128 ? 128 : 64), 0, p.ws, p.dst, p.n_splits));
        e = cudaGetLastError();
    }
    return e;
}

cudaError_t launch_fattn(const TensorD & q, const TensorD & k, const TensorD & v, const TensorD * mask, const TensorD & dst,
                         const FattnParams & fp, void * workspace, const LaunchCtx & c, int * n_kernels, void * act128_out) {
    const int64_t D = q.ne[0], rows = q.ne[1] * q.ne[2] * q.ne[3];
    if (rows == 0) return cudaSuccess;
    const bool f16_kv = k.type == T_F16 && v.type == T_F16;          // the two fast kernels stream F16 only
    if (f16_kv && c.fa_tickets && fattn_dec_applicable(q, k, v, mask)) {
        if (n_kernels) *n_kernels = 1;
        return launch_fattn_dec(q, k, v, mask, dst, fp, c.fa_tickets, workspace, c, act128_out);
    }
    static const int use_tc = getenv("GGML_B200_FA_TC") ? atoi(getenv("GGML_B200_FA_TC")) : 1;        // 0: keep the mma.sync kernel
    if (f16_kv && use_tc && fattn_tc_applicable(q, k, v, mask, fp)) {
        if (n_kernels) *n_kernels = mask ? 2 : 1;
        return launch_fattn_tc(q, k, v, mask, dst, fp, workspace, c);
    }
    if (f16_kv && fattn_mma_applicable(q, k, v, mask)) {
        if (n_kernels) *n_kernels = mask ? 2 : 1;
        return launch_fattn_mma(q, k, v, mask, dst, fp, workspace, c);
    }
    FaK p = {};
    p.q = (const char *) q.data; p.q_nb1 = q.nb[1]; p.q_nb2 = q.nb[2]; p.q_nb3 = q.nb[3];
    p.k = (const char *) k.data; p.k_nb1 = k.nb[1]; p.k_nb2 = k.nb[2]; p.k_nb3 = k.nb[3];
    p.v = (const char *) v.data; p.v_nb1 = v.nb[1]; p.v_nb2 = v.nb[2]; p.v_nb3 = v.nb[3];
    p.mask = mask ? (const char *) mask->data : nullptr; p.m_nb1 = mask ? mask->nb[1] : 0;
    p.dst = (float *) dst.data; p.ws = (float *) workspace;
    p.n_q = (int) q.ne[1]; p.n_kv = (int) k.ne[1]; p.n_head = (int) q.ne[2];
    p.gqa = (int) (q.ne[2] / k.ne[2]); p.q3_per_k3 = (int) (q.ne[3] / k.ne[3]);
    p.n_splits = fattn_pick_splits(rows, k.ne[1], c.sm_count);
    p.kv_per_split = (int) (((k.ne[1] + p.n_splits - 1) / p.n_splits + 31) / 32 * 32);
    if (n_kernels) *n_kernels = p.n_splits > 1 ? 2 : 1;
    p.scale = fp.scale; p.softcap = fp.logit_softcap; p.max_bias = fp.max_bias;
    if (p.softcap != 0.0f) p.scale /= p.softcap;
    int nh2 = 1; while (nh2 * 2 <= p.n_head) nh2 *= 2;
    p.n_head_log2 = nh2;
    p.m0 = powf(2.0f, -fp.max_bias / (float) nh2);
    p.m1 = powf(2.0f, -(fp.max_bias / 2.0f) / (float) nh2);
    const int n3 = (int) q.ne[3];
    switch (D) {
        case 64:  return fattn_launch_d<64>(p, k.type, v.type, rows, n3, c);
        case 80:  return fattn_launch_d<80>(p, k.type, v.type, rows, n3, c);
        case 96:  return fattn_launch_d<96>(p, k.type, v.type, rows, n3, c);
        case 112: return fattn_launch_d<112>(p, k.type, v.type, rows, n3, c);
        case 128: return fattn_launch_d<128>(p, k.type, v.type, rows, n3, c);
        case 256: return fattn_launch_d<256>(p, k.type, v.type, rows, n3, c);
    }
    return cudaErrorInvalidValue;
}

}  // namespace b200
