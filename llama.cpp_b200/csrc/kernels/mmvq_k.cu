// Decode mat-vec for the K-quants whose super-blocks are 16-byte multiples
// (Q4_K 144 B, Q5_K 176 B): 128-bit coalesced loads straight from HBM.
//
// A row is a run of super-blocks {16 B header | [32 B qh] | 128 B qs}.  Lane l of
// a warp takes the 16-byte qs chunk l of every group of 32 chunks (4 super-blocks),
// so one warp-wide load fetches four contiguous 128-byte runs; the 16-byte header
// (and Q5_K's high-bit chunk) is fetched with a second 128-bit load that the
// eight lanes of a super-block share.  One warp owns one weight row at a time and
// keeps up to four such loads per lane in flight; 8..16 warps per SM give the
// bytes in flight HBM needs, with no shared-memory staging of weights at all.
// The int8 activations (blk_act128) of all columns sit in shared memory, laid
// out so that the 8 lanes of each 128-bit phase read 8 distinct bank groups.
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
static constexpr int MK_BATCH = 4;          // 16-byte chunks per lane in flight

struct MkParams {
    const uint8_t * W;  int64_t w_nb1, w_nb2, w_nb3;
    const uint8_t * Xq; int64_t xq_col_bytes;
    float * dst;        int64_t dst_nb1, dst_nb2, dst_nb3;
    int M, K, ne12, ne13, r2, r3;
    int x_col0, x_ncols, xq_ne12;
};

__device__ __forceinline__ uint4 ldg128(const void * p) { return __ldg((const uint4 *) p); }
// streaming load: weights are read once, keep them from displacing the activations in L1
__device__ __forceinline__ uint4 ldg128_stream(const void * p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// 6-bit scale and min of sub-block sb from the 12 scale bytes held in three registers
// (get_scale_min_k4, ggml/src/ggml-quants.c:631-638)
__device__ __forceinline__ void k4_scale_min_reg(int sb, uint32_t s0, uint32_t s1, uint32_t s2, int & sc, int & m) {
    if (sb < 4) {
        sc = (s0 >> (8 * sb)) & 63;
        m  = (s1 >> (8 * sb)) & 63;
    } else {
        const int t = sb - 4;
        sc = ((s2 >> (8 * t)) & 0xF)       | (((s0 >> (8 * t + 6)) & 3) << 4);
        m  = ((s2 >> (8 * t + 4)) & 0xF)   | (((s1 >> (8 * t + 6)) & 3) << 4);
    }
}

template <int T, int N>
__global__ void __launch_bounds__(MK_WARPS * 32) mmvq_k_kernel(const MkParams p) {
    constexpr int BLK = (T == T_Q4_K) ? 144 : 176;
    constexpr int QS_OFF = (T == T_Q4_K) ? 16 : 48;
    extern __shared__ __align__(16) uint8_t acts[];           // [N][nblk128 * 160]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nsb = p.K >> 8;                                  // super-blocks per row
    const int nq  = nsb * 8;                                   // 16-byte qs chunks per row
    const int col_bytes = ((p.K + 127) >> 7) * 160;
    const int64_t nrows_total = (int64_t) p.M * p.ne12 * p.ne13;
    const int64_t row_stride = (int64_t) gridDim.x * MK_WARPS;
    int64_t gr = (int64_t) blockIdx.x * MK_WARPS + warp;

    // chunk q -> byte offsets inside the row
    auto qoff = [&](int q) { return (q >> 3) * BLK + QS_OFF + (q & 7) * 16; };

    // prefetch the first batch of weight chunks of this warp's first row before waiting for the
    // producer of the activations (programmatic dependent launch)
    uint4 wq[MK_BATCH], hd[MK_BATCH], qh[MK_BATCH];
    auto row_ptr = [&](int64_t r, int & i12, int & i13, int & row) {
        const int64_t z = r / p.M; row = (int) (r - z * p.M);
        i12 = (int) (z % p.ne12); i13 = (int) (z / p.ne12);
        return p.W + (int64_t) (i13 / p.r3) * p.w_nb3 + (int64_t) (i12 / p.r2) * p.w_nb2 + (int64_t) row * p.w_nb1;
    };
    auto load_batch = [&](const uint8_t * wr, int q0) {
#pragma unroll
        for (int b = 0; b < MK_BATCH; ++b) {
            const int q = q0 + b * 32 + lane;
            if (q < nq) {
                wq[b] = ldg128_stream(wr + qoff(q));
                hd[b] = ldg128(wr + (q >> 3) * BLK);
                if (T == T_Q5_K) qh[b] = ldg128(wr + (q >> 3) * BLK + 16 + (q & 1) * 16);
            }
        }
    };
    int i12 = 0, i13 = 0, row = 0;
    const uint8_t * wr = nullptr;
    if (gr < nrows_total) { wr = row_ptr(gr, i12, i13, row); load_batch(wr, 0); }

    pdl_wait();
    // stage the activations: all columns of batch (i12, i13) -- the batch index is the same for
    // every row this CTA touches only when ne12*ne13 == 1; otherwise they are staged per row below
    const bool single_batch = (p.ne12 * p.ne13 == 1);
    if (single_batch) {
        for (int n = 0; n < N; ++n) {
            const uint4 * src = (const uint4 *) (p.Xq + (int64_t) (p.x_col0 + n) * p.xq_col_bytes);
            uint4 * dstp = (uint4 *) (acts + n * col_bytes);
            for (int i = threadIdx.x; i < col_bytes / 16; i += blockDim.x) dstp[i] = src[i];
        }
    }
    __syncthreads();

    for (; gr < nrows_total; gr += row_stride) {
        // (with broadcast batch dims the activations are read from global memory / L2 per row instead)
        float acc[N];
#pragma unroll
        for (int n = 0; n < N; ++n) acc[n] = 0.0f;
        for (int q0 = 0; q0 < nq; q0 += MK_BATCH * 32) {
            if (q0 > 0) load_batch(wr, q0);
#pragma unroll
            for (int b = 0; b < MK_BATCH; ++b) {
                const int q = q0 + b * 32 + lane;
                if (q >= nq) continue;
                const int sbk = q >> 3, cc = q & 7, j = cc >> 1, h = cc & 1;
                const uint32_t w[4] = {wq[b].x, wq[b].y, wq[b].z, wq[b].w};
                uint32_t lo[4], hi[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) { lo[i] = w[i] & 0x0F0F0F0Fu; hi[i] = (w[i] >> 4) & 0x0F0F0F0Fu; }
                if (T == T_Q5_K) {
                    const uint32_t hb[4] = {qh[b].x, qh[b].y, qh[b].z, qh[b].w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint32_t t = hb[i] >> (2 * j);       // bit 0: sub-block 2j, bit 1: 2j+1
                        lo[i] |= (t << 4) & 0x10101010u;
                        hi[i] |= (t << 3) & 0x10101010u;
                    }
                }
                const float d    = __half2float(__ushort_as_half((unsigned short) (hd[b].x & 0xffff)));
                const float dmin = __half2float(__ushort_as_half((unsigned short) (hd[b].x >> 16)));
                int sc0, m0, sc1, m1;
                k4_scale_min_reg(2 * j, hd[b].y, hd[b].z, hd[b].w, sc0, m0);
                k4_scale_min_reg(2 * j + 1, hd[b].y, hd[b].z, hd[b].w, sc1, m1);
                const int g = sbk * 8 + 2 * j;                     // activation group of the low nibbles
                const int a_off = (g >> 2) * 160 + (g & 3) * 32;   // g, g+1 are in the same 128-block (g even)
#pragma unroll
                for (int n = 0; n < N; ++n) {
                    const uint8_t * ab = single_batch ? acts + n * col_bytes
                        : p.Xq + (((int64_t) i13 * p.xq_ne12 + (i12 % p.xq_ne12)) * p.x_ncols + p.x_col0 + n) * p.xq_col_bytes;
                    const uint4 x0 = *(const uint4 *) (ab + a_off + 16 * h);
                    const uint4 x1 = *(const uint4 *) (ab + a_off + 32 + 16 * h);
                    const float4 ds = *(const float4 *) (ab + (g >> 2) * 160 + 128 + (g & 3) * 8);   // {d0, s0, d1, s1}
                    int s0 = __dp4a((int) lo[0], (int) x0.x, 0); s0 = __dp4a((int) lo[1], (int) x0.y, s0);
                    s0 = __dp4a((int) lo[2], (int) x0.z, s0);    s0 = __dp4a((int) lo[3], (int) x0.w, s0);
                    int s1 = __dp4a((int) hi[0], (int) x1.x, 0); s1 = __dp4a((int) hi[1], (int) x1.y, s1);
                    s1 = __dp4a((int) hi[2], (int) x1.z, s1);    s1 = __dp4a((int) hi[3], (int) x1.w, s1);
                    float v = d * ((float) (sc0 * s0) * ds.x + (float) (sc1 * s1) * ds.z);
                    if (h == 0) v -= dmin * ((float) m0 * ds.y + (float) m1 * ds.w);   // min term once per sub-block
                    acc[n] += v;
                }
            }
        }
        // next row's first batch goes out before this row's reduction
        const int cur_row = row, cur_i12 = i12, cur_i13 = i13;
        const int64_t nxt = gr + row_stride;
        if (nxt < nrows_total) { wr = row_ptr(nxt, i12, i13, row); load_batch(wr, 0); }
#pragma unroll
        for (int n = 0; n < N; ++n) acc[n] = warp_sum(acc[n]);
        if (lane == 0) {
            uint8_t * o = (uint8_t *) p.dst + (int64_t) cur_i13 * p.dst_nb3 + (int64_t) cur_i12 * p.dst_nb2;
#pragma unroll
            for (int n = 0; n < N; ++n) ((float *) (o + (int64_t) n * p.dst_nb1))[cur_row] = acc[n];
        }
    }
    pdl_launch_dependents();
}

template <int T, int N>
static cudaError_t launch_mk_tn(const MkParams & p, int sm_count, int device, int use_pdl, cudaStream_t stream) {
    const bool single_batch = p.ne12 * p.ne13 == 1;
    const size_t smem = single_batch ? (size_t) N * ((p.K + 127) / 128) * 160 : 0;
    auto kern = mmvq_k_kernel<T, N>;
    static unsigned attr_mask = 0;
    if (smem > 48 * 1024 && !(attr_mask & (1u << device))) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return e;
        attr_mask |= 1u << device;
    }
    if (smem > 200 * 1024) return cudaErrorInvalidValue;
    const int64_t rows = (int64_t) p.M * p.ne12 * p.ne13;
    int ctas_per_sm = 4;
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
    if (a.ids) return false;
    if (((uintptr_t) a.W & 15) || (a.w_nb1 & 15) || (a.w_nb2 & 15) || (a.w_nb3 & 15)) return false;
    if ((size_t) a.N * ((a.K + 127) / 128) * 160 > 200 * 1024 && a.ne12 * a.ne13 == 1) return false;
    return true;
}

cudaError_t launch_mmvq_k(const MmvqArgs & a, cudaStream_t stream) {
    MkParams p = {};
    p.W = (const uint8_t *) a.W; p.w_nb1 = a.w_nb1; p.w_nb2 = a.w_nb2; p.w_nb3 = a.w_nb3;
    p.Xq = (const uint8_t *) a.Xq; p.xq_col_bytes = (int64_t) ((a.K + 127) / 128) * 160;
    p.dst = a.dst; p.dst_nb1 = a.dst_nb1; p.dst_nb2 = a.dst_nb2; p.dst_nb3 = a.dst_nb3;
    p.M = a.M; p.K = a.K; p.ne12 = a.ne12; p.ne13 = a.ne13; p.r2 = a.r2; p.r3 = a.r3;
    p.x_col0 = a.x_col0; p.x_ncols = a.x_ncols; p.xq_ne12 = a.xq_ne12 > 0 ? a.xq_ne12 : a.ne12;
    if (a.type == T_Q4_K) return launch_mk_t<T_Q4_K>(p, a.N, a.sm_count, a.device, a.use_pdl, stream);
    return launch_mk_t<T_Q5_K>(p, a.N, a.sm_count, a.device, a.use_pdl, stream);
}

}  // namespace b200
