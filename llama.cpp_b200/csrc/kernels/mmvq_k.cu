// Decode mat-vec for the K-quants whose super-blocks are 16-byte multiples
// (Q4_K 144 B, Q5_K 176 B): 128-bit coalesced loads straight from HBM.
//
// A row is a run of super-blocks {16 B header | [32 B qh] | 128 B qs}.  A lane owns one
// 32-byte qs run (64 weights: low nibbles = sub-block 2j, high nibbles = sub-block 2j+1) of
// one super-block: lane l takes run j = l & 3 of super-block l >> 2, so a warp-wide load
// covers 8 consecutive super-blocks; the 16-byte header (and Q5_K's high-bit bytes) comes
// with a second 128-bit load shared by the four lanes of a super-block.  One warp owns one
// weight row at a time and holds two register buffers of two units (96 bytes) each per lane
// in ping-pong, so the loads of the next batch are in flight while one is consumed; 16-24
// warps per SM give the bytes in flight HBM needs, with no shared-memory staging of weights.
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
    int n_peer; int64_t peer_delta[MAX_PEERS - 1];   // row-split: results also go to dst + peer_delta[i]
};
// (no dynamic indexing into the parameter arrays: that would move them to local memory)
__device__ __forceinline__ const uint8_t * mk_row_ptr(const MkParams & p, int row, int & mat, int & local) {
    mat = (row >= p.m_end[0]) + (row >= p.m_end[1] && p.nmat > 2);
    local = row - (mat == 0 ? 0 : (mat == 1 ? p.m_end[0] : p.m_end[1]));
    const uint8_t * w = mat == 0 ? p.W[0] : (mat == 1 ? p.W[1] : p.W[2]);
    return w + (int64_t) local * p.w_nb1;
}

__device__ __forceinline__ uint4 ldg128(const void * p) { return __ldg((const uint4 *) p); }
// unsigned bytes x signed bytes (the high nibbles are kept in place as value * 16, up to 240)
__device__ __forceinline__ int dp4a_us(uint32_t a, int b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

template <int T> struct MkBuf {                       // raw bytes of MK_BATCH units of one lane
    uint4 q0[MK_BATCH], q1[MK_BATCH], hd[MK_BATCH], qh0[T == T_Q5_K ? MK_BATCH : 1], qh1[T == T_Q5_K ? MK_BATCH : 1];
};

template <int T, int N, int OCC>
__global__ void __launch_bounds__(MK_WARPS * 32, OCC) mmvq_k_kernel(const MkParams p) {
    constexpr int BLK = (T == T_Q4_K) ? 144 : 176;
    constexpr int QS_OFF = (T == T_Q4_K) ? 16 : 48;
    extern __shared__ __align__(16) uint8_t acts[];           // [N][nblk128 * 160]
    pdl_launch_dependents();          // the next kernel may start its prologue (its weight prefetch) right away

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nsb = p.K >> 8;                                  // super-blocks per row
    const int col_bytes = ((p.K + 127) >> 7) * 160;
    const int row_stride = gridDim.x * MK_WARPS;
    const int row0 = blockIdx.x * MK_WARPS + warp;

    // lane constants: a unit is the 32-byte qs run j of super-block lb (+8 per iteration):
    // low nibbles = sub-block 2j, high nibbles = sub-block 2j+1
    const int j = lane & 3, lb = lane >> 2;
    const uint32_t w_off = lb * BLK + QS_OFF + 32 * j;
    const uint32_t h_off = lb * BLK;
    const uint32_t a_off = lb * 320 + (j >> 1) * 160 + (j & 1) * 64;          // 64 int8 of groups 2j, 2j+1
    const uint32_t d_off = lb * 320 + (j >> 1) * 160 + 128 + (j & 1) * 16;    // {d, s} of the two groups
    // 6-bit scale/min extraction (get_scale_min_k4, ggml/src/ggml-quants.c:631-638), branch-free: the entries
    // of sub-blocks 2j and 2j+1 are adjacent bytes, so both are handled as one 16-bit pair.  With the three
    // 32-bit words S0 S1 S2 of the 12 scale bytes shifted right by 16 * (j & 1):
    //   j < 2 : scales = S0 & 0x3F3F                          mins = S1 & 0x3F3F
    //   j >= 2: scales = (S2 & 0x0F0F) | ((S0 >> 2) & 0x3030) mins = ((S2 >> 4) & 0x0F0F) | ((S1 >> 2) & 0x3030)
    const bool low = j < 2;
    const int sh16 = 16 * (j & 1);
    const uint32_t mk1 = low ? 0x3F3Fu : 0x0F0Fu, mk2 = low ? 0u : 0x3030u;
    const int niter = (nsb + 7) >> 3;
    // result stores: lane 0 writes this GPU's dst, lane q + 1 the copy in peer q's arena (row-split)
    bool storer = lane == 0; int64_t st_delta = 0;
#pragma unroll
    for (int q = 0; q < MAX_PEERS - 1; ++q) if (q < p.n_peer && lane == q + 1) { storer = true; st_delta = p.peer_delta[q]; }

    auto load = [&](MkBuf<T> & B, int row, int it0) {
        int mat, lrow;
        const uint8_t * wr = mk_row_ptr(p, row, mat, lrow) + (uint32_t) it0 * (8 * BLK);
#pragma unroll
        for (int b = 0; b < MK_BATCH; ++b) {
            if (it0 + b < niter && (it0 + b) * 8 + lb < nsb) {
                const uint8_t * base = wr + b * (8 * BLK);
                B.q0[b] = ldg128(base + w_off);
                B.q1[b] = ldg128(base + w_off + 16);
                B.hd[b] = ldg128(base + h_off);
                if (T == T_Q5_K) { B.qh0[b] = ldg128(base + h_off + 16); B.qh1[b] = ldg128(base + h_off + 32); }
            }
        }
    };

    float acc[N];
#pragma unroll
    for (int n = 0; n < N; ++n) acc[n] = 0.0f;

    auto compute = [&](const MkBuf<T> & B, int row, int it0) {
#pragma unroll
        for (int b = 0; b < MK_BATCH; ++b) {
            if (it0 + b >= niter || (it0 + b) * 8 + lb >= nsb) continue;
            const uint32_t w[8] = {B.q0[b].x, B.q0[b].y, B.q0[b].z, B.q0[b].w, B.q1[b].x, B.q1[b].y, B.q1[b].z, B.q1[b].w};
            // Q4_K: high nibbles stay in place (value * 16): the unsigned x signed dp4a is exact and the
            // factor 16 is folded into the activation scale, which saves a shift per word
            uint32_t lo[8], hi[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) { lo[i] = w[i] & 0x0F0F0F0Fu; hi[i] = (T == T_Q5_K) ? (w[i] >> 4) & 0x0F0F0F0Fu : w[i] & 0xF0F0F0F0u; }
            if (T == T_Q5_K) {
                const uint32_t hb[8] = {B.qh0[b].x, B.qh0[b].y, B.qh0[b].z, B.qh0[b].w, B.qh1[b].x, B.qh1[b].y, B.qh1[b].z, B.qh1[b].w};
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const uint32_t t = hb[i] >> (2 * j);           // bit 0: sub-block 2j, bit 1: 2j+1
                    lo[i] |= (t << 4) & 0x10101010u;
                    hi[i] |= (t << 3) & 0x10101010u;
                }
            }
            const float2 dm = __half22float2(*(const __half2 *) &B.hd[b].x);      // {d, dmin}
            const uint32_t sa = B.hd[b].y >> sh16, sb_ = B.hd[b].z >> sh16, sc_ = B.hd[b].w >> sh16;
            const uint32_t scp = ((low ? sa : sc_) & mk1) | ((sa >> 2) & mk2);
            const uint32_t mnp = ((low ? sb_ : (sc_ >> 4)) & mk1) | ((sb_ >> 2) & mk2);
            const int sc0 = scp & 0xFF, sc1 = (scp >> 8) & 0xFF;
            const float fm0 = dm.y * (float) (mnp & 0xFF), fm1 = dm.y * (float) ((mnp >> 8) & 0xFF);
            const float dhi = (T == T_Q5_K) ? dm.x : dm.x * 0.0625f;
            const uint8_t * ab = acts + (uint32_t) (it0 + b) * (8 * 320);
#pragma unroll
            for (int n = 0; n < N; ++n, ab += col_bytes) {
                const uint4 xa = *(const uint4 *) (ab + a_off);
                const uint4 xb = *(const uint4 *) (ab + a_off + 16);
                const uint4 xc = *(const uint4 *) (ab + a_off + 32);
                const uint4 xd = *(const uint4 *) (ab + a_off + 48);
                const float4 ds = *(const float4 *) (ab + d_off);            // {d0, s0, d1, s1}
                int t0 = dp4a_us(lo[0], (int) xa.x, 0); t0 = dp4a_us(lo[1], (int) xa.y, t0);
                t0 = dp4a_us(lo[2], (int) xa.z, t0);    t0 = dp4a_us(lo[3], (int) xa.w, t0);
                t0 = dp4a_us(lo[4], (int) xb.x, t0);    t0 = dp4a_us(lo[5], (int) xb.y, t0);
                t0 = dp4a_us(lo[6], (int) xb.z, t0);    t0 = dp4a_us(lo[7], (int) xb.w, t0);
                int t1 = dp4a_us(hi[0], (int) xc.x, 0); t1 = dp4a_us(hi[1], (int) xc.y, t1);
                t1 = dp4a_us(hi[2], (int) xc.z, t1);    t1 = dp4a_us(hi[3], (int) xc.w, t1);
                t1 = dp4a_us(hi[4], (int) xd.x, t1);    t1 = dp4a_us(hi[5], (int) xd.y, t1);
                t1 = dp4a_us(hi[6], (int) xd.z, t1);    t1 = dp4a_us(hi[7], (int) xd.w, t1);
                // |sc * t| <= 63 * 32 * 240 * 127 < 2^26: the products are exact in int32
                const float u = dm.x * ds.x * (float) (sc0 * t0) + dhi * ds.z * (float) (sc1 * t1);
                acc[n] += u - fm0 * ds.y - fm1 * ds.w;
            }
        }
        if (it0 + MK_BATCH >= niter) {                          // row finished: reduce and store
            int mat, lrow;
            mk_row_ptr(p, row, mat, lrow);
            float * d0 = mat == 0 ? p.dst[0] : (mat == 1 ? p.dst[1] : p.dst[2]);
            const int64_t nb1 = mat == 0 ? p.dst_nb1[0] : (mat == 1 ? p.dst_nb1[1] : p.dst_nb1[2]);
#pragma unroll
            for (int n = 0; n < N; ++n) {
                const float v = warp_sum(acc[n]);
                if (storer) ((float *) ((uint8_t *) d0 + (int64_t) n * nb1 + st_delta))[lrow] = v;
                acc[n] = 0.0f;
            }
        }
    };

    // Work items of this warp are (row, batch of MK_BATCH iterations) with rows row0, row0 + row_stride, ...
    // Two register buffers in ping-pong: the loads of the next item are in flight while one is consumed.
    auto advance = [&](int & row, int & it0) { it0 += MK_BATCH; if (it0 >= niter) { it0 = 0; row += row_stride; } };
    MkBuf<T> A, B;
    int lrow_ = row0, lit = 0;            // position of the load stream
    int crow = row0, cit = 0;             // position of the compute stream
    if (lrow_ < p.M) { load(A, lrow_, lit); advance(lrow_, lit); }   // weights do not depend on the previous kernel
    pdl_wait();
    for (int n = 0; n < N; ++n) {
        const uint4 * src = (const uint4 *) (p.Xq + (int64_t) (p.x_col0 + n) * p.xq_col_bytes);
        uint4 * dstp = (uint4 *) (acts + n * col_bytes);
        for (int i = threadIdx.x; i < col_bytes / 16; i += blockDim.x) dstp[i] = src[i];
    }
    __syncthreads();
    while (crow < p.M) {
        if (lrow_ < p.M) { load(B, lrow_, lit); advance(lrow_, lit); }
        compute(A, crow, cit); advance(crow, cit);
        if (crow >= p.M) break;
        if (lrow_ < p.M) { load(A, lrow_, lit); advance(lrow_, lit); }
        compute(B, crow, cit); advance(crow, cit);
    }
}

template <int T, int N>
static cudaError_t launch_mk_tn(const MkParams & p, int sm_count, int device, int use_pdl, cudaStream_t stream) {
    const size_t smem = (size_t) N * ((p.K + 127) / 128) * 160;
    constexpr int occ = (T == T_Q4_K && N <= 2) ? 3 : 2;      // the wider variants would spill at 80 registers
    auto kern = mmvq_k_kernel<T, N, occ>;
    static unsigned attr_mask = 0;
    if (smem > 48 * 1024 && !(attr_mask & (1u << device))) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return e;
        attr_mask |= 1u << device;
    }
    if (smem > 200 * 1024) return cudaErrorInvalidValue;
    const int64_t rows = p.M;
    int ctas_per_sm = occ;
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
    p.n_peer = a.n_peer; for (int i = 0; i < a.n_peer; ++i) p.peer_delta[i] = a.peer_delta[i];
    if (a.type == T_Q4_K) return launch_mk_t<T_Q4_K>(p, a.N, a.sm_count, a.device, a.use_pdl, stream);
    return launch_mk_t<T_Q5_K>(p, a.N, a.sm_count, a.device, a.use_pdl, stream);
}

}  // namespace b200
