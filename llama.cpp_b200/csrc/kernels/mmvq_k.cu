// Decode mat-vec for the K-quants whose super-blocks are 16-byte multiples
// (Q4_K 144 B, Q5_K 176 B): 128-bit coalesced loads straight from HBM.
//
// A row is a run of super-blocks {16 B header | [32 B qh] | 128 B qs}.  A lane owns one
// 32-byte qs run (64 weights: low nibbles = sub-block 2j, high nibbles = sub-block 2j+1) of
// one super-block: lane l takes run j = l & 3 of super-block l >> 2, so a warp-wide load
// covers 8 consecutive super-blocks; the 16-byte header (and Q5_K's high-bit bytes) comes
// with a second 128-bit load shared by the four lanes of a super-block.  One warp owns one
// weight row at a time and keeps P units (48 bytes of loads each) per lane in flight in a rotating
// set of register buffers that runs across row boundaries; 16-32 warps per SM give the bytes in
// flight HBM needs, with no shared-memory staging of weights.
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

// Up to three weight matrices that share the activation operand (wq/wk/wv, gate/up) are served by one
// launch: their rows are concatenated into one row space of M = m_end[nmat-1] rows.  Wadj / dst_adj are
// the matrix and result bases moved back by the matrix's first row, so that row r of the row space is at
// Wadj[i] + r * w_nb1 and its results at dst_adj[i][r] (+ n * dst_nb1[i] bytes for column n).
struct MkParams {
    const uint8_t * Wadj[3];  int64_t w_nb1;
    const uint8_t * Xq;       int64_t xq_col_bytes;
    float * dst_adj[3];       int64_t dst_nb1[3];
    int m_end[3];
    int M, K;
    int x_col0;
    int n_peer; int64_t peer_delta[MAX_PEERS - 1];   // row-split: results also go to dst + peer_delta[i]
};

__device__ __forceinline__ uint4 ldg128(const void * p) { return __ldg((const uint4 *) p); }
// unsigned bytes x signed bytes (the high nibbles are kept in place as value * 16, up to 240)
__device__ __forceinline__ int dp4a_us(uint32_t a, int b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

template <int T> struct MkUnit { uint4 hd, q0, q1, qh0, qh1; };      // raw bytes of one 64-weight unit of a lane

// P units per lane are in flight (a rotating set of register buffers: the unit consumed is reloaded with the
// one P steps ahead, across row boundaries).  FULL: K is a multiple of 2048, so every lane has a unit in
// every iteration.  All positions (row, iteration, addresses) are carried incrementally; nothing in the loop
// divides or re-derives a pointer from the row index except once per row.
template <int T, int N, bool FULL, int P, int OCC>
__global__ void __launch_bounds__(MK_WARPS * 32, OCC) mmvq_k_kernel(const __grid_constant__ MkParams p) {
    constexpr int BLK = (T == T_Q4_K) ? 144 : 176;
    constexpr int QS_OFF = (T == T_Q4_K) ? 16 : 48;
    extern __shared__ __align__(16) uint8_t acts[];           // [N][nblk128 * 160]
    pdl_launch_dependents();          // the next kernel may start its prologue (its weight prefetch) right away

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nsb = p.K >> 8;                                  // super-blocks per row
    const int col_bytes = ((p.K + 127) >> 7) * 160;
    const int row_stride = gridDim.x * MK_WARPS;
    const int row0 = blockIdx.x * MK_WARPS + warp;
    const int M = p.M;

    // lane constants: a unit is the 32-byte qs run j of super-block lb (+8 per iteration):
    // low nibbles = sub-block 2j, high nibbles = sub-block 2j+1
    const int j = lane & 3, lb = lane >> 2;
    const uint32_t h_off = lb * BLK;                                           // header of the lane's super-block
    const uint32_t q_off = QS_OFF + 32 * j;                                    // its qs run, from the header
    const uint32_t a_off = lb * 320 + (j >> 1) * 160 + (j & 1) * 64;          // 64 int8 of groups 2j, 2j+1
    const uint32_t ds_rel = 128 - (j & 1) * 48;                                // {d, s} of the two groups, from a_off
    // 6-bit scale/min extraction (get_scale_min_k4, ggml/src/ggml-quants.c:631-638), branch-free: the entries
    // of sub-blocks 2j and 2j+1 are adjacent bytes, so both are handled as one 16-bit pair.  With the three
    // 32-bit words S0 S1 S2 of the 12 scale bytes shifted right by 16 * (j & 1):
    //   j < 2 : scales = S0 & 0x3F3F                          mins = S1 & 0x3F3F
    //   j >= 2: scales = (S2 & 0x0F0F) | ((S0 >> 2) & 0x3030) mins = ((S2 >> 4) & 0x0F0F) | ((S1 >> 2) & 0x3030)
    const bool low = j < 2;
    const int sh16 = 16 * (j & 1);
    const uint32_t mk1 = low ? 0x3F3Fu : 0x0F0Fu, mk2 = low ? 0u : 0x3030u;
    const int niter = (nsb + 7) >> 3;
    const bool tail_ok = FULL || (nsb & 7) == 0 || lb < (nsb & 7);             // has a unit in the last iteration
    // result stores: lane 0 writes this GPU's dst, lane q + 1 the copy in peer q's arena (row-split)
    bool storer = lane == 0; int64_t st_delta = 0;
#pragma unroll
    for (int q = 0; q < MAX_PEERS - 1; ++q) if (q < p.n_peer && lane == q + 1) { storer = true; st_delta = p.peer_delta[q]; }

    // ---- load stream ----
    int l_row = row0, l_it = 0, l_end = p.m_end[0];
    const uint8_t * l_w = p.Wadj[0];
    const uint8_t * l_ptr = nullptr;                           // header address of the lane's next unit
    auto l_enter_row = [&]() {
        if (l_row >= l_end) {                                  // the next matrix of a grouped launch
            if (l_row >= p.m_end[1]) { l_w = p.Wadj[2]; l_end = 0x7fffffff; } else { l_w = p.Wadj[1]; l_end = p.m_end[1]; }
        }
        l_ptr = l_w + (int64_t) l_row * p.w_nb1 + h_off;
    };
    auto load = [&](MkUnit<T> & u) {
        if (FULL || l_it < niter - 1 || tail_ok) {
            u.hd = ldg128(l_ptr);
            u.q0 = ldg128(l_ptr + q_off);
            u.q1 = ldg128(l_ptr + q_off + 16);
            if (T == T_Q5_K) { u.qh0 = ldg128(l_ptr + 16); u.qh1 = ldg128(l_ptr + 32); }
        }
        l_ptr += 8 * BLK;
        if (++l_it == niter) { l_it = 0; l_row += row_stride; if (l_row < M) l_enter_row(); }
    };

    // ---- compute stream ----
    int c_row = row0, c_it = 0, c_end = p.m_end[0];
    float * c_dst = p.dst_adj[0]; int64_t c_nb1 = p.dst_nb1[0];
    const uint8_t * c_a = acts + a_off;                        // the lane's activations of the current unit
    float acc[N];
#pragma unroll
    for (int n = 0; n < N; ++n) acc[n] = 0.0f;

    auto consume = [&](const MkUnit<T> & u) {
        if (FULL || c_it < niter - 1 || tail_ok) {
            const uint32_t w[8] = {u.q0.x, u.q0.y, u.q0.z, u.q0.w, u.q1.x, u.q1.y, u.q1.z, u.q1.w};
            // Q4_K: high nibbles stay in place (value * 16): the unsigned x signed dp4a is exact and the
            // factor 16 is folded into the scale, which saves a shift per word
            uint32_t lo[8], hi[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) { lo[i] = w[i] & 0x0F0F0F0Fu; hi[i] = (T == T_Q5_K) ? (w[i] >> 4) & 0x0F0F0F0Fu : w[i] & 0xF0F0F0F0u; }
            if (T == T_Q5_K) {
                const uint32_t hb[8] = {u.qh0.x, u.qh0.y, u.qh0.z, u.qh0.w, u.qh1.x, u.qh1.y, u.qh1.z, u.qh1.w};
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const uint32_t t = hb[i] >> (2 * j);           // bit 0: sub-block 2j, bit 1: 2j+1
                    lo[i] |= (t << 4) & 0x10101010u;
                    hi[i] |= (t << 3) & 0x10101010u;
                }
            }
            const float2 dm = __half22float2(*(const __half2 *) &u.hd.x);         // {d, dmin}
            const uint32_t sa = u.hd.y >> sh16, sb_ = u.hd.z >> sh16, sc_ = u.hd.w >> sh16;
            const uint32_t scp = ((low ? sa : sc_) & mk1) | ((sa >> 2) & mk2);
            const uint32_t mnp = ((low ? sb_ : (sc_ >> 4)) & mk1) | ((sb_ >> 2) & mk2);
            const int sc0 = scp & 0xFF, sc1 = (scp >> 8) & 0xFF;
            const float fm0 = dm.y * (float) (mnp & 0xFF), fm1 = dm.y * (float) ((mnp >> 8) & 0xFF);
            const float dhi = (T == T_Q5_K) ? dm.x : dm.x * 0.0625f;
            const uint8_t * ab = c_a;
#pragma unroll
            for (int n = 0; n < N; ++n, ab += col_bytes) {
                const uint4 xa = *(const uint4 *) (ab);
                const uint4 xb = *(const uint4 *) (ab + 16);
                const uint4 xc = *(const uint4 *) (ab + 32);
                const uint4 xd = *(const uint4 *) (ab + 48);
                const float4 ds = *(const float4 *) (ab + ds_rel);           // {d0, s0, d1, s1}
                int t0 = dp4a_us(lo[0], (int) xa.x, 0); t0 = dp4a_us(lo[1], (int) xa.y, t0);
                t0 = dp4a_us(lo[2], (int) xa.z, t0);    t0 = dp4a_us(lo[3], (int) xa.w, t0);
                t0 = dp4a_us(lo[4], (int) xb.x, t0);    t0 = dp4a_us(lo[5], (int) xb.y, t0);
                t0 = dp4a_us(lo[6], (int) xb.z, t0);    t0 = dp4a_us(lo[7], (int) xb.w, t0);
                int t1 = dp4a_us(hi[0], (int) xc.x, 0); t1 = dp4a_us(hi[1], (int) xc.y, t1);
                t1 = dp4a_us(hi[2], (int) xc.z, t1);    t1 = dp4a_us(hi[3], (int) xc.w, t1);
                t1 = dp4a_us(hi[4], (int) xd.x, t1);    t1 = dp4a_us(hi[5], (int) xd.y, t1);
                t1 = dp4a_us(hi[6], (int) xd.z, t1);    t1 = dp4a_us(hi[7], (int) xd.w, t1);
                // |sc * t| <= 63 * 32 * 240 * 127 < 2^26: the products are exact in int32
                const float uu = dm.x * ds.x * (float) (sc0 * t0) + dhi * ds.z * (float) (sc1 * t1);
                acc[n] += uu - fm0 * ds.y - fm1 * ds.w;
            }
        }
        c_a += 8 * 320;
        if (++c_it == niter) {                                  // row finished: reduce and store
            if (c_row >= c_end) {
                if (c_row >= p.m_end[1]) { c_dst = p.dst_adj[2]; c_nb1 = p.dst_nb1[2]; c_end = 0x7fffffff; }
                else                     { c_dst = p.dst_adj[1]; c_nb1 = p.dst_nb1[1]; c_end = p.m_end[1]; }
            }
#pragma unroll
            for (int n = 0; n < N; ++n) {
                const float v = warp_sum(acc[n]);
                if (storer) ((float *) ((uint8_t *) c_dst + (int64_t) n * c_nb1 + st_delta))[c_row] = v;
                acc[n] = 0.0f;
            }
            c_it = 0; c_a = acts + a_off; c_row += row_stride;
        }
    };

    MkUnit<T> u0, u1, u2, u3;
    if (l_row < M) l_enter_row();
    // weights do not depend on the previous kernel: the first P units are requested before waiting for it
    if (l_row < M) load(u0);
    if (P > 1 && l_row < M) load(u1);
    if (P > 2 && l_row < M) load(u2);
    if (P > 3 && l_row < M) load(u3);
    pdl_wait();
    for (int n = 0; n < N; ++n) {
        const uint4 * src = (const uint4 *) (p.Xq + (int64_t) (p.x_col0 + n) * p.xq_col_bytes);
        uint4 * dstp = (uint4 *) (acts + n * col_bytes);
        for (int i = threadIdx.x; i < col_bytes / 16; i += blockDim.x) dstp[i] = src[i];
    }
    __syncthreads();
    for (;;) {
        if (c_row >= M) break;
        consume(u0); if (l_row < M) load(u0);
        if (P > 1) { if (c_row >= M) break; consume(u1); if (l_row < M) load(u1); }
        if (P > 2) { if (c_row >= M) break; consume(u2); if (l_row < M) load(u2); }
        if (P > 3) { if (c_row >= M) break; consume(u3); if (l_row < M) load(u3); }
    }
}

template <int T, int N, bool FULL, int P, int OCC>
static cudaError_t launch_mk_cfg(const MkParams & p, int sm_count, int device, int use_pdl, cudaStream_t stream) {
    const size_t smem = (size_t) N * ((p.K + 127) / 128) * 160;
    auto kern = mmvq_k_kernel<T, N, FULL, P, OCC>;
    static unsigned attr_mask = 0;
    if (smem > 48 * 1024 && !(attr_mask & (1u << device))) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return e;
        attr_mask |= 1u << device;
    }
    if (smem > 200 * 1024) return cudaErrorInvalidValue;
    int ctas_per_sm = OCC;
    if (smem) { const int by_smem = (int) ((220 * 1024) / (smem + 1024)); if (by_smem < ctas_per_sm) ctas_per_sm = by_smem < 1 ? 1 : by_smem; }
    int64_t grid = (int64_t) sm_count * ctas_per_sm;
    const int64_t need = ((int64_t) p.M + MK_WARPS - 1) / MK_WARPS;
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

template <int T, int N>
static cudaError_t launch_mk_tn(const MkParams & p, int sm_count, int device, int use_pdl, cudaStream_t stream) {
    const bool full = (p.K & 2047) == 0;
    // measured on B200: for one column of Q4_K, two units in flight per lane at 64 registers (4 CTAs = 32 warps
    // per SM) beats deeper pipelines at lower occupancy; the wider variants need the registers
    constexpr int OCC = (N == 1 && T == T_Q4_K) ? 4 : 2;
    if (full) return launch_mk_cfg<T, N, true, 2, OCC>(p, sm_count, device, use_pdl, stream);
    return launch_mk_cfg<T, N, false, 2, OCC>(p, sm_count, device, use_pdl, stream);
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
    p.w_nb1 = a.w_nb1;
    p.Xq = (const uint8_t *) a.Xq; p.xq_col_bytes = (int64_t) ((a.K + 127) / 128) * 160;
    const void * W[3] = {a.W, a.n_extra > 0 ? a.extra_W[0] : a.W, a.n_extra > 1 ? a.extra_W[1] : a.W};
    float * dst[3] = {a.dst, a.n_extra > 0 ? a.extra_dst[0] : a.dst, a.n_extra > 1 ? a.extra_dst[1] : a.dst};
    const int64_t nb1[3] = {a.dst_nb1, a.n_extra > 0 ? a.extra_dst_nb1[0] : a.dst_nb1, a.n_extra > 1 ? a.extra_dst_nb1[1] : a.dst_nb1};
    const int rows[3] = {a.M, a.n_extra > 0 ? a.extra_M[0] : 0, a.n_extra > 1 ? a.extra_M[1] : 0};
    int start = 0;
    for (int i = 0; i < 3; ++i) {
        // integer arithmetic: the adjusted bases may lie before the allocation, they are only ever
        // used with a row index >= start
        p.Wadj[i] = (const uint8_t *) ((intptr_t) W[i] - (intptr_t) start * a.w_nb1);
        p.dst_adj[i] = (float *) ((intptr_t) dst[i] - (intptr_t) start * 4);
        p.dst_nb1[i] = nb1[i];
        start += rows[i];
        p.m_end[i] = start;
    }
    for (int i = 1 + a.n_extra; i < 3; ++i) p.m_end[i] = 0x7fffffff;     // unused slots: never entered
    p.M = start; p.K = a.K; p.x_col0 = a.x_col0;
    p.n_peer = a.n_peer; for (int i = 0; i < a.n_peer; ++i) p.peer_delta[i] = a.peer_delta[i];
    if (a.type == T_Q4_K) return launch_mk_t<T_Q4_K>(p, a.N, a.sm_count, a.device, a.use_pdl, stream);
    return launch_mk_t<T_Q5_K>(p, a.N, a.sm_count, a.device, a.use_pdl, stream);
}

}  // namespace b200
