// MUL_MAT for a few activation columns (3 .. 8 by default: parallel sequences, speculative batches): HBM-bound like the mat-vec,
// but with every weight used N times.
//
// The mat-vec kernels give a lane a run of one weight row and repeat their dp4a chain (and the shared-memory reads of the
// int8 activations) per column: at 8 columns they are bound by shared-memory traffic, 4x slower than at one column.  The
// tcgen05 GEMM dequantizes whole 128-row tiles to F16 whatever N is and cannot go below the time of that.  Between the
// two, the integer tensor-core instruction does the job: mma.sync m16n8k32 (u8/s8 x s8 -> s32) multiplies 16 weight rows
// by 8 activation columns over one 32-value quant block, and the block scales are applied to the four int32 results a
// thread holds -- a cost per (16 rows x 8 columns x 32 values), not per weight.  The arithmetic is that of the mat-vec
// path: int8 activations with a scale per 32 values (blk_act128), integer dot products per quant block, FP32 scaling
// (ggml/src/ggml-cuda/vecdotq.cuh:357-442 for Q4_K; :235-259 for Q8_0).
//
// One CTA owns 16 weight rows and all columns; its 8 warps divide K (a warp takes every 8th run of 256 values) and add
// their partial sums through shared memory at the end.  Operand fragments are fetched straight from global memory: which
// of a block's 32 values sits in which k-slot of the instruction is free as long as both operands agree, so thread t of
// a quad takes 8 consecutive values (bytes 8t .. 8t+7 of the quant run and of the activation column), one 64-bit load
// each.  The weights of the next run are requested before the current one is multiplied.
#include "common.cuh"
#include "kernels.h"
#include <stdlib.h>

namespace b200 {

static constexpr int MS_WARPS = 8;

struct MsParams {
    const uint8_t * W;  int64_t w_nb1;
    const uint8_t * Xq; int64_t xq_col_bytes;       // blk_act128 columns
    float * dst;        int64_t dst_nb1;
    int M, K, N;
};

__device__ __forceinline__ void ms_mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ms_mma_s8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ---- raw bytes of one run of 256 values of the two rows (g, g + 8) a thread feeds, per weight type ----
template <int T> struct MsRun;

// Q4_K: super-block {d, dmin, 12 bytes of 6-bit scales | 128 bytes qs}; bytes 32j .. 32j+31 of qs hold sub-block 2j in
// the low and 2j+1 in the high nibbles (ggml-quants.c:1280-1302).  Thread t reads bytes 8t .. 8t+7 of every 32-byte run.
template <> struct MsRun<T_Q4_K> {
    static constexpr int BYTES = 144;
    uint4 hd[2]; uint2 qs[2][4];
    __device__ __forceinline__ void load(const uint8_t * r0, const uint8_t * r1, int t) {
        hd[0] = __ldg((const uint4 *) r0); hd[1] = __ldg((const uint4 *) r1);
#pragma unroll
        for (int j = 0; j < 4; ++j) { qs[0][j] = __ldg((const uint2 *) (r0 + 16 + 32 * j + 8 * t)); qs[1][j] = __ldg((const uint2 *) (r1 + 16 + 32 * j + 8 * t)); }
    }
};

// Q8_0: eight blocks {f16 d | 32 int8} = 272 bytes; a block's quants start 2 bytes after a 2-byte aligned address, so the
// 8 bytes of a thread come as aligned 32-bit words (three and a funnel shift where the run is not 4-byte aligned).
template <> struct MsRun<T_Q8_0> {
    static constexpr int BYTES = 272;
    uint32_t q[2][8][2]; uint32_t d[2][4];          // d: two f16 per word
    __device__ __forceinline__ void load(const uint8_t * r0, const uint8_t * r1, int t) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const uint8_t * p = r ? r1 : r0;
#pragma unroll
            for (int b = 0; b < 8; ++b) {
                const int off = 34 * b + 2 + 8 * t;                    // 34 b + 2 is a multiple of 4 for odd b
                if (b & 1) {
                    q[r][b][0] = __ldg((const uint32_t *) (p + off)); q[r][b][1] = __ldg((const uint32_t *) (p + off + 4));
                } else {
                    const uint32_t w0 = __ldg((const uint32_t *) (p + off - 2)), w1 = __ldg((const uint32_t *) (p + off + 2)), w2 = __ldg((const uint32_t *) (p + off + 6));
                    q[r][b][0] = __funnelshift_r(w0, w1, 16); q[r][b][1] = __funnelshift_r(w1, w2, 16);
                }
            }
            // d of block 2i: bytes 68 i, 68 i + 1; of block 2i+1: bytes 68 i + 34, + 35 = the high half of the word at 68 i + 32
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t lo = __ldg((const uint32_t *) (p + 68 * i)), hi = __ldg((const uint32_t *) (p + 68 * i + 32));
                d[r][i] = (lo & 0xffffu) | (hi & 0xffff0000u);
            }
        }
    }
};

template <int T, int NT>
__global__ void __launch_bounds__(MS_WARPS * 32, 2) mmq_s8_kernel(const __grid_constant__ MsParams p) {
    pdl_launch_dependents();
    constexpr int RB = MsRun<T>::BYTES;
    constexpr int CP = 8 * NT + 1;                                  // padded row of the reduction buffer
    __shared__ float red[MS_WARPS][16][CP];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int m0 = blockIdx.x * 16;
    const int nrun = p.K / 256;

    const uint8_t * rowp[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) rowp[r] = p.W + (int64_t) min(m0 + g + 8 * r, p.M - 1) * p.w_nb1;
    // activation columns of this thread: column g of every column tile as the B operand (clamped: columns past N are computed, not stored)
    const uint8_t * xcol[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) xcol[nt] = p.Xq + (int64_t) min(8 * nt + g, p.N - 1) * p.xq_col_bytes;
    // ... and columns 2t, 2t+1 of every tile for the scales of the results it holds
    const uint8_t * scol[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int c = 0; c < 2; ++c) scol[nt][c] = p.Xq + (int64_t) min(8 * nt + 2 * t + c, p.N - 1) * p.xq_col_bytes;

    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[nt][c] = 0.0f;

    MsRun<T> cur, nxt;
    if (warp < nrun) cur.load(rowp[0] + (int64_t) warp * RB, rowp[1] + (int64_t) warp * RB, t);
    pdl_wait();                                                     // the weights above do not depend on the previous kernel, the activations do
#pragma unroll 1
    for (int run = warp; run < nrun; run += MS_WARPS) {
        if (run + MS_WARPS < nrun) nxt.load(rowp[0] + (int64_t) (run + MS_WARPS) * RB, rowp[1] + (int64_t) (run + MS_WARPS) * RB, t);
        // the activation blocks of this run: two blk_act128 per column
        const int64_t xoff = (int64_t) run * 2 * (int64_t) sizeof(blk_act128);
#pragma unroll
        for (int sb = 0; sb < 8; ++sb) {
            // B operands and activation scales of sub-block sb for every column tile
            const int64_t boff = xoff + (sb >> 2) * (int64_t) sizeof(blk_act128);
            uint2 bq[NT];
            float2 ds[NT][2];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                bq[nt] = __ldg((const uint2 *) (xcol[nt] + boff + 32 * (sb & 3) + 8 * t));
                ds[nt][0] = __ldg((const float2 *) (scol[nt][0] + boff + 128 + 8 * (sb & 3)));
                ds[nt][1] = __ldg((const float2 *) (scol[nt][1] + boff + 128 + 8 * (sb & 3)));
            }
            uint32_t a0, a1, a2, a3;
            float wsc[2], wmn[2];                                    // per row: scale and (Q4_K) min term of this sub-block
            if constexpr (T == T_Q4_K) {
                const int j = sb >> 1, sh = (sb & 1) * 4;
                a0 = (cur.qs[0][j].x >> sh) & 0x0F0F0F0Fu; a1 = (cur.qs[1][j].x >> sh) & 0x0F0F0F0Fu;
                a2 = (cur.qs[0][j].y >> sh) & 0x0F0F0F0Fu; a3 = (cur.qs[1][j].y >> sh) & 0x0F0F0F0Fu;
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    const uint4 h = cur.hd[r];
                    const float2 dm = __half22float2(*(const __half2 *) &h.x);
                    // 6-bit scales and mins (get_scale_min_k4, ggml-quants.c:631-638)
                    uint32_t sc, mn;
                    if (sb < 4) { sc = (h.y >> (8 * sb)) & 63u; mn = (h.z >> (8 * sb)) & 63u; }
                    else { const int u = sb - 4; sc = ((h.w >> (8 * u)) & 0xFu) | (((h.y >> (8 * u + 6)) & 3u) << 4); mn = ((h.w >> (8 * u + 4)) & 0xFu) | (((h.z >> (8 * u + 6)) & 3u) << 4); }
                    wsc[r] = dm.x * (float) sc; wmn[r] = dm.y * (float) mn;
                }
            } else {
                a0 = cur.q[0][sb][0]; a1 = cur.q[1][sb][0]; a2 = cur.q[0][sb][1]; a3 = cur.q[1][sb][1];
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    const uint32_t w = cur.d[r][sb >> 1];
                    wsc[r] = __half2float(__ushort_as_half((unsigned short) ((sb & 1) ? (w >> 16) : (w & 0xffffu)))); wmn[r] = 0.0f;
                }
            }
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                int c[4] = {0, 0, 0, 0};
                if constexpr (T == T_Q4_K) ms_mma_u8s8(c, a0, a1, a2, a3, bq[nt].x, bq[nt].y);
                else                       ms_mma_s8s8(c, a0, a1, a2, a3, bq[nt].x, bq[nt].y);
                // c0: (row g, col 2t), c1: (row g, col 2t+1), c2, c3: row g + 8
                acc[nt][0] += wsc[0] * ds[nt][0].x * (float) c[0] - wmn[0] * ds[nt][0].y;
                acc[nt][1] += wsc[0] * ds[nt][1].x * (float) c[1] - wmn[0] * ds[nt][1].y;
                acc[nt][2] += wsc[1] * ds[nt][0].x * (float) c[2] - wmn[1] * ds[nt][0].y;
                acc[nt][3] += wsc[1] * ds[nt][1].x * (float) c[3] - wmn[1] * ds[nt][1].y;
            }
        }
        cur = nxt;
    }

    // ---- add the 8 warps' parts ----
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        red[warp][g][8 * nt + 2 * t]         = acc[nt][0];
        red[warp][g][8 * nt + 2 * t + 1]     = acc[nt][1];
        red[warp][g + 8][8 * nt + 2 * t]     = acc[nt][2];
        red[warp][g + 8][8 * nt + 2 * t + 1] = acc[nt][3];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 16 * 8 * NT; i += MS_WARPS * 32) {
        const int n = i >> 4, m = i & 15;                           // consecutive threads: consecutive rows of one result column
        if (n >= p.N || m0 + m >= p.M) continue;
        float s = 0.0f;
#pragma unroll
        for (int w = 0; w < MS_WARPS; ++w) s += red[w][m][n];
        *(float *) ((char *) p.dst + (int64_t) n * p.dst_nb1 + (int64_t) (m0 + m) * 4) = s;
    }
}

// Where it wins (measured on 4096 x 14336, whole MUL_MAT): Q4_K with 3 .. 8 columns (N = 4: 24.7 against 30.8 us for the
// mat-vec, N = 8: 28.2 against 47.1 us).  At 2 columns the mat-vec is faster (20.6 against 22.7 us), at 16 the tcgen05 GEMM
// (35 against 42 us), and Q8_0 gains nothing (49.8 against 48.9 us at N = 8: its 2-byte aligned blocks cost three 32-bit
// loads per fragment), so those stay where they were unless GGML_B200_MMQ_S8 widens the range (the largest column count,
// up to 16; 1 adds Q8_0 at the default range; 0 turns the kernel off).
bool mmq_s8_shape_ok(int type, int64_t n_cols, int64_t K) {
    static const int knob = [] { const char * e = getenv("GGML_B200_MMQ_S8"); return e ? atoi(e) : -1; }();
    if (knob == 0) return false;
    if (type != T_Q4_K && !(type == T_Q8_0 && knob >= 1)) return false;
    const int64_t max_cols = knob > 8 ? (knob > 16 ? 16 : knob) : 8, min_cols = knob >= 1 ? 2 : 3;
    return n_cols >= min_cols && n_cols <= max_cols && K % 256 == 0 && K >= 256;
}
bool mmq_s8_applicable(const MmvqArgs & a, int64_t n_cols) {
    if (!mmq_s8_shape_ok(a.type, n_cols, a.K)) return false;
    if (a.ne12 != 1 || a.ne13 != 1 || a.ids || a.n_peer) return false;
    if (((uintptr_t) a.W & 15) || (a.w_nb1 & 15) || ((uintptr_t) a.Xq & 15) || (a.dst_nb1 & 3) || ((uintptr_t) a.dst & 3)) return false;
    for (int i = 0; i < a.n_extra; ++i) if (((uintptr_t) a.extra_W[i] & 15) || (a.extra_dst_nb1[i] & 3) || ((uintptr_t) a.extra_dst[i] & 3)) return false;
    return true;
}

template <int T, int NT>
static cudaError_t ms_launch(const MsParams & p, int use_pdl, cudaStream_t stream) {
    cudaError_t launch_err = cudaSuccess;
    (void) (launch_err = launch_k(use_pdl, stream, mmq_s8_kernel<T, NT>, dim3((unsigned) ((p.M + 15) / 16)), dim3(MS_WARPS * 32), 0, p));
    (void) launch_err;
    return cudaGetLastError();
}

static cudaError_t ms_launch_one(const MmvqArgs & a, int64_t n_cols, cudaStream_t stream) {
    MsParams p = {};
    p.W = (const uint8_t *) a.W; p.w_nb1 = a.w_nb1;
    p.xq_col_bytes = (int64_t) (a.K / 128) * (int64_t) sizeof(blk_act128);
    p.Xq = (const uint8_t *) a.Xq + (int64_t) a.x_col0 * p.xq_col_bytes;
    p.dst = a.dst; p.dst_nb1 = a.dst_nb1;
    p.M = a.M; p.K = a.K; p.N = (int) n_cols;
    const bool two = n_cols > 8;
    if (a.type == T_Q4_K) return two ? ms_launch<T_Q4_K, 2>(p, a.use_pdl, stream) : ms_launch<T_Q4_K, 1>(p, a.use_pdl, stream);
    return two ? ms_launch<T_Q8_0, 2>(p, a.use_pdl, stream) : ms_launch<T_Q8_0, 1>(p, a.use_pdl, stream);
}

// all n_cols columns (a.x_col0 .. + n_cols) in one launch per weight matrix
cudaError_t launch_mmq_s8(const MmvqArgs & a, int64_t n_cols, cudaStream_t stream) {
    cudaError_t e = ms_launch_one(a, n_cols, stream);
    for (int i = 0; i < a.n_extra && e == cudaSuccess; ++i) {
        MmvqArgs b = a;
        b.W = a.extra_W[i]; b.dst = a.extra_dst[i]; b.dst_nb1 = a.extra_dst_nb1[i]; b.M = a.extra_M[i]; b.n_extra = 0;
        e = ms_launch_one(b, n_cols, stream);
    }
    return e;
}

}  // namespace b200
