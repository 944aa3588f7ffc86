// FLASH_ATTN_EXT for batches of queries (prefill): tensor-core QK^T and PV with online softmax.
//
// One CTA = 4 warps = 64 query rows of one head; each warp owns 16 rows.  K/V tiles of 64 keys are
// staged in shared memory with cp.async (double buffered, rows padded by 16 bytes so ldmatrix is
// conflict free); S = Q K^T and O += P V run on mma.sync m16n8k16 (F16 in, FP32 accumulate), the
// softmax statistics and O stay in FP32 registers (libllama requests GGML_PREC_F32, src/llama.cpp:595).
// Replaces flash_attn_ext_f16 (ggml/src/ggml-cuda/fattn-mma-f16.cuh:13-689), with two differences the
// reference lacks: whole 64x64 tiles that the mask sets to -inf (everything above the causal diagonal)
// are skipped without loading K/V, using per-tile flags computed from the mask by a tiny pre-pass,
// and tiles the mask leaves at zero skip the mask read.  Semantics: ggml_compute_forward_flash_attn_ext_f16
// (ggml/src/ggml-cpu/ggml-cpu.c:10916-11129) incl. scale, logit softcap and ALiBi slopes.
#include "common.cuh"
#include "kernels.h"
#include <math.h>

namespace b200 {

static constexpr int FM_BM = 64, FM_BN = 64, FM_WARPS = 4;

struct FmParams {
    const char * q; int64_t q_nb1, q_nb2, q_nb3;
    const char * k; int64_t k_nb1, k_nb2, k_nb3;
    const char * v; int64_t v_nb1, v_nb2, v_nb3;
    const char * mask; int64_t m_nb1;
    const uint8_t * flags; int flags_stride;        // [q tiles][kv tiles]: 0 mixed, 1 all -inf, 2 all zero
    float * dst;
    int n_q, n_kv, n_head, gqa, q3_per_k3;
    float scale, softcap, max_bias, m0, m1; int n_head_log2;
};

// classifies each 64x64 tile of the mask
__global__ void fattn_mask_flags_kernel(const char * mask, int64_t m_nb1, int n_q, int n_kv, uint8_t * flags, int flags_stride) {
    pdl_enter();
    __shared__ int any_finite, any_nonzero;
    if (threadIdx.x == 0) { any_finite = 0; any_nonzero = 0; }
    __syncthreads();
    const int kv0 = blockIdx.x * FM_BN, q0 = blockIdx.y * FM_BM;
    int fin = 0, nz = 0;
    for (int i = threadIdx.x; i < FM_BM * FM_BN; i += blockDim.x) {
        const int qi = q0 + i / FM_BN, ki = kv0 + i % FM_BN;
        if (qi < n_q && ki < n_kv) {
            const float m = __half2float(*(const __half *) (mask + (int64_t) qi * m_nb1 + (int64_t) ki * 2));
            if (m != -INFINITY) fin = 1;
            if (m != 0.0f) nz = 1;
        }
    }
    if (fin) any_finite = 1;
    if (nz) any_nonzero = 1;
    __syncthreads();
    if (threadIdx.x == 0) flags[blockIdx.y * flags_stride + blockIdx.x] = !any_finite ? 1 : (!any_nonzero ? 2 : 0);
}

__device__ __forceinline__ void cp_async16(void * smem, const void * gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(smem_u32(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" :: "n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void * p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void * p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2(float a, float b) { __half2 h = __floats2half2_rn(a, b); return *(uint32_t *) &h; }

template <int D>
__global__ void __launch_bounds__(FM_WARPS * 32, 2) fattn_mma_kernel(const FmParams p) {
    pdl_enter();
    constexpr int ROWB = D * 2 + 16;                   // padded smem row (bytes)
    constexpr int TILE = FM_BN * ROWB;
    extern __shared__ __align__(16) uint8_t smem[];
    uint8_t * sK[2] = {smem, smem + TILE};
    uint8_t * sV[2] = {smem + 2 * TILE, smem + 3 * TILE};
    uint8_t * sQ = smem + 4 * TILE;                    // 64 x ROWB, used once

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int qt = blockIdx.x, head = blockIdx.y, i3 = blockIdx.z;
    const int q0 = qt * FM_BM;
    const int hk = head / p.gqa, k3 = i3 / p.q3_per_k3;
    const char * kbase = p.k + (int64_t) hk * p.k_nb2 + (int64_t) k3 * p.k_nb3;
    const char * vbase = p.v + (int64_t) hk * p.v_nb2 + (int64_t) k3 * p.v_nb3;
    const int n_kv_tiles = (p.n_kv + FM_BN - 1) / FM_BN;
    const uint8_t * flags = p.flags ? p.flags + qt * p.flags_stride : nullptr;

    float slope = 1.0f;
    if (p.max_bias > 0.0f)
        slope = head < p.n_head_log2 ? powf(p.m0, (float) (head + 1)) : powf(p.m1, (float) (2 * (head - p.n_head_log2) + 1));

    // ---- Q tile: F32 global -> F16 smem -> A fragments (kept in registers for the whole kernel) ----
    for (int i = tid; i < FM_BM * (D / 2); i += blockDim.x) {
        const int r = i / (D / 2), c2 = i % (D / 2);
        float2 v = make_float2(0.0f, 0.0f);
        if (q0 + r < p.n_q) v = *(const float2 *) (p.q + (int64_t) (q0 + r) * p.q_nb1 + (int64_t) head * p.q_nb2 + (int64_t) i3 * p.q_nb3 + c2 * 8);
        *(uint32_t *) (sQ + r * ROWB + c2 * 4) = pack2(v.x, v.y);
    }
    __syncthreads();
    uint32_t qf[D / 16][4];
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk)
        ldmatrix_x4(qf[kk], sQ + (warp * 16 + (lane & 15)) * ROWB + (kk * 16 + (lane >> 4) * 8) * 2);

    auto load_tile = [&](int buf, int jt) {
        const int kv0 = jt * FM_BN;
        constexpr int CH = D * 2 / 16;                  // 16-byte chunks per row
        for (int i = tid; i < FM_BN * CH; i += blockDim.x) {
            const int r = i / CH, c = i % CH;
            const int kv = min(kv0 + r, p.n_kv - 1);    // rows past n_kv are clamped; their scores are masked below
            cp_async16(sK[buf] + r * ROWB + c * 16, kbase + (int64_t) kv * p.k_nb1 + c * 16);
            cp_async16(sV[buf] + r * ROWB + c * 16, vbase + (int64_t) kv * p.v_nb1 + c * 16);
        }
        cp_async_commit();
    };
    // tiles to visit: all that are not entirely masked out
    auto next_tile = [&](int jt) { while (jt < n_kv_tiles && flags && flags[jt] == 1) ++jt; return jt; };

    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
    float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.0f, 0.0f};

    int jt = next_tile(0), buf = 0;
    if (jt < n_kv_tiles) load_tile(0, jt);
    while (jt < n_kv_tiles) {
        const int jn = next_tile(jt + 1);
        if (jn < n_kv_tiles) load_tile(buf ^ 1, jn);
        if (jn < n_kv_tiles) cp_async_wait<1>(); else cp_async_wait<0>();
        __syncthreads();

        // ---- S = Q K^T for this warp's 16 rows x 64 keys ----
        float s[FM_BN / 8][4];
#pragma unroll
        for (int i = 0; i < FM_BN / 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f; }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
            for (int nt = 0; nt < FM_BN / 16; ++nt) {   // two 8-key tiles per ldmatrix
                uint32_t b[4];
                ldmatrix_x4(b, sK[buf] + (nt * 16 + (lane & 7) + ((lane >> 4) << 3)) * ROWB + (kk * 16 + ((lane >> 3) & 1) * 8) * 2);
                mma16816(s[2 * nt], qf[kk], b[0], b[1]);
                mma16816(s[2 * nt + 1], qf[kk], b[2], b[3]);
            }
        }
        // ---- scale, softcap, mask; online softmax ----
        const int kv0 = jt * FM_BN;
        const bool need_mask = p.mask && (!flags || flags[jt] == 0);
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < FM_BN / 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int r = q0 + warp * 16 + g + (e >> 1) * 8, c = kv0 + nt * 8 + 2 * t + (e & 1);
                float v = s[nt][e] * p.scale;
                if (p.softcap != 0.0f) v = p.softcap * tanhf(v);
                if (need_mask && r < p.n_q && c < p.n_kv) v += slope * __half2float(*(const __half *) (p.mask + (int64_t) r * p.m_nb1 + (int64_t) c * 2));
                if (c >= p.n_kv) v = -INFINITY;
                s[nt][e] = v;
                mx[e >> 1] = fmaxf(mx[e >> 1], v);
            }
        }
        float corr[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
            const float mnew = fmaxf(mrow[h], mx[h]);
            corr[h] = (mrow[h] == -INFINITY) ? 0.0f : expf(mrow[h] - mnew);
            mrow[h] = mnew;
        }
        float rs[2] = {0.0f, 0.0f};
        uint32_t pf[FM_BN / 16][4];                     // P as A fragments (two 8-key tiles = one 16-deep k step)
#pragma unroll
        for (int nt = 0; nt < FM_BN / 8; ++nt) {
            float e0 = (mrow[0] == -INFINITY) ? 0.0f : expf(s[nt][0] - mrow[0]);
            float e1 = (mrow[0] == -INFINITY) ? 0.0f : expf(s[nt][1] - mrow[0]);
            float e2 = (mrow[1] == -INFINITY) ? 0.0f : expf(s[nt][2] - mrow[1]);
            float e3 = (mrow[1] == -INFINITY) ? 0.0f : expf(s[nt][3] - mrow[1]);
            rs[0] += e0 + e1; rs[1] += e2 + e3;
            pf[nt >> 1][(nt & 1) * 2]     = pack2(e0, e1);   // a0 / a2: row g
            pf[nt >> 1][(nt & 1) * 2 + 1] = pack2(e2, e3);   // a1 / a3: row g+8
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            rs[h] += __shfl_xor_sync(0xffffffffu, rs[h], 1);
            rs[h] += __shfl_xor_sync(0xffffffffu, rs[h], 2);
            lrow[h] = lrow[h] * corr[h] + rs[h];
        }
#pragma unroll
        for (int i = 0; i < D / 8; ++i) { o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1]; }
        // ---- O += P V ----
#pragma unroll
        for (int kk = 0; kk < FM_BN / 16; ++kk) {
#pragma unroll
            for (int dt = 0; dt < D / 16; ++dt) {       // two 8-wide d tiles per ldmatrix
                uint32_t b[4];
                ldmatrix_x4_trans(b, sV[buf] + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ROWB + (dt * 16 + (lane >> 4) * 8) * 2);
                mma16816(o[2 * dt], pf[kk], b[0], b[1]);
                mma16816(o[2 * dt + 1], pf[kk], b[2], b[3]);
            }
        }
        __syncthreads();                                // everyone is done with this buffer before it is refilled
        jt = jn; buf ^= 1;
    }

    // ---- write O / l: dst is [D, n_head, n_q] ----
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = q0 + warp * 16 + g + h * 8;
        if (r >= p.n_q) continue;
        const float inv = 1.0f / lrow[h];
        float * out = p.dst + (((int64_t) i3 * p.n_q + r) * p.n_head + head) * D;
#pragma unroll
        for (int i = 0; i < D / 8; ++i) *(float2 *) (out + i * 8 + 2 * t) = make_float2(o[i][2 * h] * inv, o[i][2 * h + 1] * inv);
    }
}

bool fattn_mma_applicable(const TensorD & q, const TensorD & k, const TensorD & v, const TensorD * mask) {
    const int64_t D = q.ne[0];
    if (D != 64 && D != 128) return false;
    if (q.ne[1] <= 8) return false;                                    // small batches take the split-KV vector kernel
    auto al16 = [](const TensorD & t) { return ((uintptr_t) t.data & 15) == 0 && (t.nb[1] & 15) == 0 && (t.nb[2] & 15) == 0 && (t.nb[3] & 15) == 0; };
    if (!al16(k) || !al16(v)) return false;
    if (((uintptr_t) q.data & 7) || (q.nb[1] & 7) || (q.nb[2] & 7) || (q.nb[3] & 7)) return false;
    if (mask && (((uintptr_t) mask->data & 1) || (mask->nb[1] & 1))) return false;
    return true;
}

size_t fattn_mma_workspace_bytes(const TensorD & q, const TensorD & k) {
    return (size_t) ((q.ne[1] + FM_BM - 1) / FM_BM) * (size_t) ((k.ne[1] + FM_BN - 1) / FM_BN) + 16;
}

template <int D>
static cudaError_t fattn_mma_launch(const FmParams & p, int n3, const LaunchCtx & c) {
    constexpr int ROWB = D * 2 + 16;
    const size_t smem = (size_t) 5 * FM_BN * ROWB;
    auto kern = fattn_mma_kernel<D>;
    static unsigned attr_mask = 0;
    if (smem > 48 * 1024 && !(attr_mask & (1u << c.device))) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem);
        if (e != cudaSuccess) return e;
        attr_mask |= 1u << c.device;
    }
    dim3 grid((unsigned) ((p.n_q + FM_BM - 1) / FM_BM), (unsigned) p.n_head, (unsigned) n3);
    (void) (launch_err = launch_k(c.use_pdl, c.stream, kern, dim3(grid), dim3(FM_WARPS * 32), smem, p));
    return cudaGetLastError();
}

cudaError_t launch_fattn_mask_flags(const char * mask, int64_t m_nb1, int n_q, int n_kv, uint8_t * flags, int flags_stride, const LaunchCtx & c) {
    const int qt = (n_q + FM_BM - 1) / FM_BM, kt = (n_kv + FM_BN - 1) / FM_BN;
    (void) (launch_err = launch_k(c.use_pdl, c.stream, fattn_mask_flags_kernel, dim3(dim3((unsigned) kt, (unsigned) qt)), dim3(256), 0, mask, m_nb1, n_q, n_kv, flags, flags_stride));
    return cudaGetLastError();
}

cudaError_t launch_fattn_mma(const TensorD & q, const TensorD & k, const TensorD & v, const TensorD * mask, const TensorD & dst,
                             const FattnParams & fp, void * workspace, const LaunchCtx & c) {
    FmParams p = {};
    p.q = (const char *) q.data; p.q_nb1 = q.nb[1]; p.q_nb2 = q.nb[2]; p.q_nb3 = q.nb[3];
    p.k = (const char *) k.data; p.k_nb1 = k.nb[1]; p.k_nb2 = k.nb[2]; p.k_nb3 = k.nb[3];
    p.v = (const char *) v.data; p.v_nb1 = v.nb[1]; p.v_nb2 = v.nb[2]; p.v_nb3 = v.nb[3];
    p.mask = mask ? (const char *) mask->data : nullptr; p.m_nb1 = mask ? mask->nb[1] : 0;
    p.dst = (float *) dst.data;
    p.n_q = (int) q.ne[1]; p.n_kv = (int) k.ne[1]; p.n_head = (int) q.ne[2];
    p.gqa = (int) (q.ne[2] / k.ne[2]); p.q3_per_k3 = (int) (q.ne[3] / k.ne[3]);
    p.scale = fp.scale; p.softcap = fp.logit_softcap; p.max_bias = fp.max_bias;
    if (p.softcap != 0.0f) p.scale /= p.softcap;
    int nh2 = 1; while (nh2 * 2 <= p.n_head) nh2 *= 2;
    p.n_head_log2 = nh2;
    p.m0 = powf(2.0f, -fp.max_bias / (float) nh2);
    p.m1 = powf(2.0f, -(fp.max_bias / 2.0f) / (float) nh2);
    if (mask) {
        const int qt = (p.n_q + FM_BM - 1) / FM_BM, kt = (p.n_kv + FM_BN - 1) / FM_BN;
        p.flags = (const uint8_t *) workspace; p.flags_stride = kt;
        (void) (launch_err = launch_k(c.use_pdl, c.stream, fattn_mask_flags_kernel, dim3(dim3((unsigned) kt, (unsigned) qt)), dim3(256), 0, p.mask, p.m_nb1, p.n_q, p.n_kv, (uint8_t *) workspace, kt));
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return e;
    }
    const int n3 = (int) q.ne[3];
    if (q.ne[0] == 64) return fattn_mma_launch<64>(p, n3, c);
    return fattn_mma_launch<128>(p, n3, c);
}

}  // namespace b200
