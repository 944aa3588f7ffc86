// Decode mat-vec for the K-quants whose super-blocks are 16-byte multiples
// (Q4_K 144 B, Q5_K 176 B): 128-bit coalesced loads straight from HBM.
//
// A row is a run of super-blocks {16 B header | [32 B qh] | 128 B qs}.  A lane owns one
// 32-byte qs run (64 weights: low nibbles = sub-block 2j, high nibbles = sub-block 2j+1) of
// one super-block: lane l takes run j = l & 3 of super-block l >> 2, so a warp-wide load
// covers 8 consecutive super-blocks; the 16-byte header (and Q5_K's high-bit bytes) comes
// with a second 128-bit load shared by the four lanes of a super-block.  One warp owns one
// weight row at a time and keeps two units (96 bytes) per lane in flight; 24 warps per SM
// give the bytes in flight HBM needs, with no shared-memory staging of weights at all.
// The int8 activations (blk_act128) of all columns sit in shared memory.  Everything that
// depends only on the lane (nibble run, scale bit positions, activation offsets) is
// computed once, outside the row loop.
//
// Arithmetic: the integer dot products and scale/min handling of
// vec_dot_q4_K_q8_1 / vec_dot_q5_K_q8_1 (ggml/src/ggml-cuda/vecdotq.cuh:357-442,
// 671-761), restated for this chunking: per chunk, low nibbles belong to
// sub-block 2j and high nibbles to sub-block 2j+1 (ggml-quants.c:1280-1302).
// Weight loads are issued before griddepcontrol.wait, activations after.
#include "common.cuh"
#include "kernels.h"

namespace b200 {

static constexpr int MK_WARPS = 8;
static constexpr int MK_BATCH = 2;          // 64-weight units per lane in flight (2 x 48 bytes of loads)

// Up to three weight matrices that share the activation operand (wq/wk/wv, gate/up) are served by one
// launch: their rows are concatenated into one row space of M = m_end[nmat-1] rows.
struct MkParams {
    const uint8_t * W[3];  int64_t w_nb1;
    const uint8_t * Xq;    int64_t xq_col_bytes;
    float * dst[3];        int64_t dst_nb1[3];
    int m_end[3], nmat;
    int M, K;
    int x_col0;
};
__device__ __forceinline__ const uint8_t * mk_row_ptr(const MkParams & p, int row, int & mat, int & local) {
    mat = (row >= p.m_end[0]) + (row >= p.m_end[1] && p.nmat > 2);
    local = row - (mat ? p.m_end[mat - 1] : 0);
    return p.W[mat] + (int64_t) local * p.w_nb1;
}

__device__ __forceinline__ uint4 ldg128(const void * p) { return __ldg((const uint4 *) p); }

template <int T, int N>
__global__ void __launch_bounds__(MK_WARPS * 32, 3) mmvq_k_kernel(const MkParams p) {
    constexpr int BLK = (T == T_Q4_K) ? 144 : 176;
    constexpr int QS_OFF = (T == T_Q4_K) ? 16 : 48;
    extern __shared__ __align__(16) uint8_t acts[];           // [N][nblk128 * 160]
    pdl_launch_dependents();          // the next kernel may start its prologue (its weight prefetch) right away

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nsb = p.K >> 8;                                  // super-blocks per row
    const int col_bytes = ((p.K + 127) >> 7) * 160;
    const int row_stride = gridDim.x * MK_WARPS;
    int row = blockIdx.x * MK_WARPS + warp;

    // lane constants: a unit is the 32-byte qs run j of super-block lb (+8 per iteration):
    // low nibbles = sub-block 2j, high nibbles = sub-block 2j+1
    const int j = lane & 3, lb = lane >> 2;
    const uint32_t w_off = lb * BLK + QS_OFF + 32 * j;
    const uint32_t h_off = lb * BLK;
    const uint32_t a_off = lb * 320 + (j >> 1) * 160 + (j & 1) * 64;          // 64 int8 of groups 2j, 2j+1
    const uint32_t d_off = lb * 320 + (j >> 1) * 160 + 128 + (j & 1) * 16;    // {d, s} of the two groups
    // 6-bit scale/min extraction (get_scale_min_k4, ggml/src/ggml-quants.c:631-638) with the shifts fixed per lane
    const bool low = j < 2;
    const int sh_a = low ? 16 * j : 8 * (2 * j - 4);          // byte position of sub-block 2j's entry
    const int sh_b = sh_a + 8;                                 // ... and of sub-block 2j+1

    uint4 q0[MK_BATCH], q1[MK_BATCH], hd[MK_BATCH], qh0[MK_BATCH], qh1[MK_BATCH];
    auto load_batch = [&](const uint8_t * wr, int it0) {
#pragma unroll
        for (int b = 0; b < MK_BATCH; ++b) {
            const int sb = (it0 + b) * 8 + lb;
            if (sb < nsb) {
                const uint8_t * base = wr + (uint32_t) (it0 + b) * (8 * BLK);
                q0[b] = ldg128(base + w_off);
                q1[b] = ldg128(base + w_off + 16);
                hd[b] = ldg128(base + h_off);
                if (T == T_Q5_K) { qh0[b] = ldg128(base + h_off + 16); qh1[b] = ldg128(base + h_off + 32); }
            }
        }
    };
    int mat = 0, lrow = 0;
    const uint8_t * wr = p.W[0];
    if (row < p.M) { wr = mk_row_ptr(p, row, mat, lrow); load_batch(wr, 0); }        // weights do not depend on the previous kernel: fetch before waiting

    pdl_wait();
    for (int n = 0; n < N; ++n) {
        const uint4 * src = (const uint4 *) (p.Xq + (int64_t) (p.x_col0 + n) * p.xq_col_bytes);
        uint4 * dstp = (uint4 *) (acts + n * col_bytes);
        for (int i = threadIdx.x; i < col_bytes / 16; i += blockDim.x) dstp[i] = src[i];
    }
    __syncthreads();

    const int niter = (nsb + 7) >> 3;
    for (; row < p.M; row += row_stride) {
        float acc[N];
#pragma unroll
        for (int n = 0; n < N; ++n) acc[n] = 0.0f;
        for (int it0 = 0; it0 < niter; it0 += MK_BATCH) {
            if (it0 > 0) load_batch(wr, it0);
#pragma unroll
            for (int b = 0; b < MK_BATCH; ++b) {
                const int sb = (it0 + b) * 8 + lb;
                if (sb >= nsb) continue;
                const uint32_t w[8] = {q0[b].x, q0[b].y, q0[b].z, q0[b].w, q1[b].x, q1[b].y, q1[b].z, q1[b].w};
                uint32_t lo[8], hi[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) { lo[i] = w[i] & 0x0F0F0F0Fu; hi[i] = (w[i] >> 4) & 0x0F0F0F0Fu; }
                if (T == T_Q5_K) {
                    const uint32_t hb[8] = {qh0[b].x, qh0[b].y, qh0[b].z, qh0[b].w, qh1[b].x, qh1[b].y, qh1[b].z, qh1[b].w};
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const uint32_t t = hb[i] >> (2 * j);       // bit 0: sub-block 2j, bit 1: 2j+1
                        lo[i] |= (t << 4) & 0x10101010u;
                        hi[i] |= (t << 3) & 0x10101010u;
                    }
                }
                const float2 dm = __half22float2(*(const __half2 *) &hd[b].x);      // {d, dmin}
                const uint32_t s0 = hd[b].y, s1 = hd[b].z, s2 = hd[b].w;
                int sc0, sc1, m0, m1;
                if (low) {
                    sc0 = (s0 >> sh_a) & 63; sc1 = (s0 >> sh_b) & 63;
                    m0  = (s1 >> sh_a) & 63; m1  = (s1 >> sh_b) & 63;
                } else {
                    sc0 = ((s2 >> sh_a) & 0xF)       | (((s0 >> (sh_a + 6)) & 3) << 4);
                    sc1 = ((s2 >> sh_b) & 0xF)       | (((s0 >> (sh_b + 6)) & 3) << 4);
                    m0  = ((s2 >> (sh_a + 4)) & 0xF) | (((s1 >> (sh_a + 6)) & 3) << 4);
                    m1  = ((s2 >> (sh_b + 4)) & 0xF) | (((s1 >> (sh_b + 6)) & 3) << 4);
                }
                const float fs0 = dm.x * (float) sc0, fs1 = dm.x * (float) sc1;
                const float fm0 = dm.y * (float) m0,  fm1 = dm.y * (float) m1;
                const uint32_t it_a = (uint32_t) (it0 + b) * (8 * 320);
#pragma unroll
                for (int n = 0; n < N; ++n) {
                    const uint8_t * ab = acts + n * col_bytes + it_a;
                    const uint4 xa = *(const uint4 *) (ab + a_off);
                    const uint4 xb = *(const uint4 *) (ab + a_off + 16);
                    const uint4 xc = *(const uint4 *) (ab + a_off + 32);
                    const uint4 xd = *(const uint4 *) (ab + a_off + 48);
                    const float4 ds = *(const float4 *) (ab + d_off);            // {d0, s0, d1, s1}
                    int t0 = __dp4a((int) lo[0], (int) xa.x, 0); t0 = __dp4a((int) lo[1], (int) xa.y, t0);
                    t0 = __dp4a((int) lo[2], (int) xa.z, t0);    t0 = __dp4a((int) lo[3], (int) xa.w, t0);
                    t0 = __dp4a((int) lo[4], (int) xb.x, t0);    t0 = __dp4a((int) lo[5], (int) xb.y, t0);
                    t0 = __dp4a((int) lo[6], (int) xb.z, t0);    t0 = __dp4a((int) lo[7], (int) xb.w, t0);
                    int t1 = __dp4a((int) hi[0], (int) xc.x, 0); t1 = __dp4a((int) hi[1], (int) xc.y, t1);
                    t1 = __dp4a((int) hi[2], (int) xc.z, t1);    t1 = __dp4a((int) hi[3], (int) xc.w, t1);
                    t1 = __dp4a((int) hi[4], (int) xd.x, t1);    t1 = __dp4a((int) hi[5], (int) xd.y, t1);
                    t1 = __dp4a((int) hi[6], (int) xd.z, t1);    t1 = __dp4a((int) hi[7], (int) xd.w, t1);
                    acc[n] += fs0 * ds.x * (float) t0 + fs1 * ds.z * (float) t1 - fm0 * ds.y - fm1 * ds.w;
                }
            }
        }
        const int cur_mat = mat, cur_row = lrow;
        if (row + row_stride < p.M) { wr = mk_row_ptr(p, row + row_stride, mat, lrow); load_batch(wr, 0); }
#pragma unroll
        for (int n = 0; n < N; ++n) acc[n] = warp_sum(acc[n]);
        if (lane == 0) {
#pragma unroll
            for (int n = 0; n < N; ++n) ((float *) ((uint8_t *) p.dst[cur_mat] + (int64_t) n * p.dst_nb1[cur_mat]))[cur_row] = acc[n];
        }
    }
}

template <int T, int N>
static cudaError_t launch_mk_tn(const MkParams & p, int sm_count, int device, int use_pdl, cudaStream_t stream) {
    const size_t smem = (size_t) N * ((p.K + 127) / 128) * 160;
    auto kern = mmvq_k_kernel<T, N>;
    static unsigned attr_mask = 0;
    if (smem > 48 * 1024 && !(attr_mask & (1u << device))) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return e;
        attr_mask |= 1u << device;
    }
    if (smem > 200 * 1024) return cudaErrorInvalidValue;
    const int64_t rows = p.M;
    int ctas_per_sm = 3;
    if (smem) { const int by_smem = (int) ((220 * 1024) / (smem + 1024)); if (by_smem < ctas_per_sm) ctas_per_sm = by_smem < 1 ? 1 : by_smem; }
    int64_t grid = (int64_t) sm_count * ctas_per_sm;
    const int64_t need = (rows + MK_WARPS - 1) / MK_WARPS;
    if (grid > need) grid = need;
    if (grid < 1) grid = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned) grid); cfg.blockDim = dim3(MK_WARPS * 32);
    cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = use_pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, p);
}

template <int T>
static cudaError_t launch_mk_t(const MkParams & p, int N, int sm, int dev, int pdl, cudaStream_t st) {
    switch (N) {
        case 1: return launch_mk_tn<T, 1>(p, sm, dev, pdl, st);
        case 2: return launch_mk_tn<T, 2>(p, sm, dev, pdl, st);
        case 3: return launch_mk_tn<T, 3>(p, sm, dev, pdl, st);
        case 4: return launch_mk_tn<T, 4>(p, sm, dev, pdl, st);
        case 5: return launch_mk_tn<T, 5>(p, sm, dev, pdl, st);
        case 6: return launch_mk_tn<T, 6>(p, sm, dev, pdl, st);
        case 7: return launch_mk_tn<T, 7>(p, sm, dev, pdl, st);
        case 8: return launch_mk_tn<T, 8>(p, sm, dev, pdl, st);
    }
    return cudaErrorInvalidValue;
}

// the direct kernel needs 16-byte aligned rows and no expert indirection
bool mmvq_k_applicable(const MmvqArgs & a) {
    if (a.type != T_Q4_K && a.type != T_Q5_K) return false;
    if (a.ids || a.ne12 * a.ne13 != 1) return false;
    if (((uintptr_t) a.W & 15) || (a.w_nb1 & 15)) return false;
    for (int i = 0; i < a.n_extra; ++i) if ((uintptr_t) a.extra_W[i] & 15) return false;
    if ((size_t) a.N * ((a.K + 127) / 128) * 160 > 200 * 1024) return false;
    return true;
}

cudaError_t launch_mmvq_k(const MmvqArgs & a, cudaStream_t stream) {
    MkParams p = {};
    p.W[0] = (const uint8_t *) a.W; p.w_nb1 = a.w_nb1;
    p.Xq = (const uint8_t *) a.Xq; p.xq_col_bytes = (int64_t) ((a.K + 127) / 128) * 160;
    p.dst[0] = a.dst; p.dst_nb1[0] = a.dst_nb1;
    p.m_end[0] = a.M; p.nmat = 1 + a.n_extra;
    for (int i = 0; i < 2; ++i) {
        const bool on = i < a.n_extra;
        p.W[i + 1] = on ? (const uint8_t *) a.extra_W[i] : p.W[0];
        p.dst[i + 1] = on ? a.extra_dst[i] : a.dst; p.dst_nb1[i + 1] = on ? a.extra_dst_nb1[i] : a.dst_nb1;
        p.m_end[i + 1] = p.m_end[i] + (on ? a.extra_M[i] : 0);
    }
    if (p.nmat < 2) p.m_end[1] = 0x7fffffff;        // row >= m_end[1] never holds
    p.M = p.m_end[p.nmat - 1]; p.K = a.K; p.x_col0 = a.x_col0;
    if (a.type == T_Q4_K) return launch_mk_t<T_Q4_K>(p, a.N, a.sm_count, a.device, a.use_pdl, stream);
    return launch_mk_t<T_Q5_K>(p, a.N, a.sm_count, a.device, a.use_pdl, stream);
}

}  // namespace b200
