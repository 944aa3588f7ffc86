// FLASH_ATTN_EXT for decode (at most 8 queries): HBM-bound streaming of the F16 K/V cache.
//
// One CTA serves one KV head and one slice of the KV range for ALL query heads that share that KV
// head (GQA) and all queries of the batch, so K and V are read from HBM once per KV head instead of
// once per query head (the reference's flash_attn_vec_ext kernels re-read them per query head,
// ggml/src/ggml-cuda/fattn-vec-f32.cuh).  The KV range is split over enough CTAs to fill the GPU;
// partial (max, sum, O) results go to a workspace and the last CTA of each KV head to finish (an
// atomic ticket) merges them in a fixed order, so there is no second launch and the result is
// deterministic.
//
// Inside a CTA each of the 4 warps takes a contiguous run of keys: scores with 8 lanes per key
// (two 128-bit loads of the K row each), FP32 softmax over the warp's keys, then P.V with the lanes
// across the head dimension (coalesced V rows).  Rows (query, head) are processed four at a time.
#include "common.cuh"
#include "kernels.h"
#include <math.h>
#include <stdlib.h>

namespace b200 {

static constexpr int FD_WARPS = 4, FD_RT = 4, FD_MAX_KEYS_PER_WARP = 256, FD_VROWS = 16;
static constexpr int FD_MERGE_FLOATS = FD_WARPS * FD_MAX_KEYS_PER_WARP * FD_RT;      // shared memory of the split merge: weights and sums of R x n_splits pairs

struct FdParams {
    const char * q; int64_t q_nb1, q_nb2, q_nb3;
    const char * k; int64_t k_nb1, k_nb2, k_nb3;
    const char * v; int64_t v_nb1, v_nb2, v_nb3;
    const char * mask; int64_t m_nb1;
    float * dst;
    float * ws;              // partials: [n3][n_head_kv][n_splits][R][D + 2]
    unsigned * tickets;      // [n3 * n_head_kv], zero between launches
    int n_q, n_kv, n_head, n_head_kv, gqa, q3_per_k3;
    int n_splits, kv_per_split;
    float scale, softcap, max_bias, m0, m1; int n_head_log2;
    blk_act128 * act_out;    // optional (D = 128, one query batch): int8 blocks of dst for the MUL_MAT that reads it
    int mask_al8;            // the mask's rows may be read 8 bytes at a time
    int v_t; int64_t v_nbd;  // V stored transposed (the cache layout without FLASH_ATTN_EXT): keys contiguous, v_nbd bytes between head-dim rows
};

// One output row (query iq, head) of D = 128 values is exactly one blk_act128 of the [n_head * D] activation
// column iq; thread d holds value v.  Same arithmetic as quantize_act128_kernel: a scale per 32 values (a warp).
__device__ __forceinline__ void fd_emit_act(blk_act128 * blk, int d, float v) {
    const float amax = warp_max(fabsf(v));
    const float dd = amax / 127.0f, id = amax > 0.0f ? 127.0f / amax : 0.0f;
    const int q = __float2int_rn(v * id);
    int qsum = q;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) qsum += __shfl_xor_sync(0xffffffffu, qsum, o);
    blk->q[d] = (int8_t) q;
    if ((d & 31) == 0) blk->ds[d >> 5] = make_float2(dd, dd * (float) qsum);
}

// The last CTA of a KV head to finish (an atomic ticket) merges the partial results of all splits, in split order.
// `wgt`: FD_MERGE_FLOATS floats of shared memory that no warp uses any more.
template <int D>
__device__ __forceinline__ void fd_merge_splits(const FdParams & p, int R, int i3, int hk, float * wgt, unsigned * ticket_sh) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (p.n_splits > 1) {
        // ---- the last CTA of this KV head merges all splits ----
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) *ticket_sh = atomicAdd(&p.tickets[i3 * p.n_head_kv + hk], 1u);
        __syncthreads();
        if (*ticket_sh == (unsigned) p.n_splits - 1) {
            __threadfence();
            const float * base = p.ws + (((int64_t) i3 * p.n_head_kv + hk) * p.n_splits) * R * (D + 2);
            // per (row, split) weights exp(m_s - M) / L in shared memory (`wgt`, FD_MERGE_FLOATS floats): all (max, sum) pairs are
            // fetched in one parallel pass, then one warp per row reduces over the splits
            float * wl = wgt + FD_MERGE_FLOATS / 2;                  // the sums, same indexing, in the upper half
            const int RS = R * p.n_splits;
            for (int idx = threadIdx.x; idx < RS; idx += blockDim.x) {
                const int s_ = idx / R, r = idx - s_ * R;
                const float * ps_ = base + ((int64_t) s_ * R + r) * (D + 2);
                wgt[r * p.n_splits + s_] = ps_[D];
                wl[r * p.n_splits + s_]  = ps_[D + 1];
            }
            __syncthreads();
            for (int r = warp; r < R; r += FD_WARPS) {
                float M = -INFINITY;
                for (int s_ = lane; s_ < p.n_splits; s_ += 32) M = fmaxf(M, wgt[r * p.n_splits + s_]);
                M = warp_max(M);
                float L = 0.0f;
                for (int s_ = lane; s_ < p.n_splits; s_ += 32) {
                    const float m_s = wgt[r * p.n_splits + s_];
                    const float f = (m_s == -INFINITY) ? 0.0f : expf(m_s - M);
                    wgt[r * p.n_splits + s_] = f; L += wl[r * p.n_splits + s_] * f;
                }
                L = warp_sum(L);
                const float inv = 1.0f / L;
                for (int s_ = lane; s_ < p.n_splits; s_ += 32) wgt[r * p.n_splits + s_] *= inv;
            }
            __syncthreads();
            // The partial tiles lie in L2: a load takes several hundred cycles, so a thread keeps the loads of 8 splits for
            // each of its 4 outputs in flight at a time (one load after the other made this loop the longest part of the
            // kernel at 64 and more splits).
            constexpr int MI = 4, MS = 8;
            for (int ib = 0; ib < R * D; ib += MI * (int) blockDim.x) {
                int r[MI], d[MI];
                bool live[MI];
                float acc[MI];
#pragma unroll
                for (int j = 0; j < MI; ++j) {
                    const int i = ib + j * (int) blockDim.x + (int) threadIdx.x;
                    live[j] = i < R * D;                                // uniform over a warp: R * D is a multiple of 64
                    r[j] = live[j] ? i / D : 0; d[j] = i % D; acc[j] = 0.0f;
                }
                for (int s0 = 0; s0 < p.n_splits; s0 += MS) {
                    float v[MI][MS];
#pragma unroll
                    for (int j = 0; j < MI; ++j)
#pragma unroll
                        for (int u = 0; u < MS; ++u) {
                            const int s_ = min(s0 + u, p.n_splits - 1);
                            v[j][u] = __ldcg(base + ((int64_t) s_ * R + r[j]) * (D + 2) + d[j]);
                        }
#pragma unroll
                    for (int j = 0; j < MI; ++j)
#pragma unroll
                        for (int u = 0; u < MS; ++u)
                            if (s0 + u < p.n_splits) acc[j] += v[j][u] * wgt[r[j] * p.n_splits + s0 + u];
                }
#pragma unroll
                for (int j = 0; j < MI; ++j) {
                    if (!live[j]) continue;
                    const int iq = r[j] / p.gqa, head = hk * p.gqa + r[j] % p.gqa;
                    p.dst[(((int64_t) i3 * p.n_q + iq) * p.n_head + head) * D + d[j]] = acc[j];
                    if (D == 128 && p.act_out) fd_emit_act(p.act_out + (int64_t) iq * p.n_head + head, d[j], acc[j]);
                }
            }
            if (threadIdx.x == 0) p.tickets[i3 * p.n_head_kv + hk] = 0;      // ready for the next launch
        }
    }
}

template <int D>
__global__ void __launch_bounds__(FD_WARPS * 32, 4) fattn_dec_kernel(const FdParams p) {
    pdl_enter();
    constexpr int DPL = D / 32;                                   // head-dim values per lane in the P.V phase
    __shared__ __align__(16) float qs[FD_RT][D];
    __shared__ __align__(16) float ps[FD_WARPS][FD_MAX_KEYS_PER_WARP][FD_RT];   // scores, then probabilities
    __shared__ float w_m[FD_WARPS][FD_RT], w_l[FD_WARPS][FD_RT];
    __shared__ __align__(16) float w_o[FD_WARPS][FD_RT][D];
    __shared__ unsigned ticket_sh;

    const int split = blockIdx.x, hk = blockIdx.y, i3 = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int R = p.n_q * p.gqa;                                  // rows served by this CTA
    const int k3 = i3 / p.q3_per_k3;
    const char * kbase = p.k + (int64_t) hk * p.k_nb2 + (int64_t) k3 * p.k_nb3;
    const char * vbase = p.v + (int64_t) hk * p.v_nb2 + (int64_t) k3 * p.v_nb3;

    const int kv0 = split * p.kv_per_split, kv1 = min(p.n_kv, kv0 + p.kv_per_split);
    int per_warp = (max(kv1 - kv0, 0) + FD_WARPS - 1) / FD_WARPS;
    if (p.v_t) per_warp = (per_warp + 7) & ~7;                     // 16-byte aligned runs of keys in the transposed V rows
    const int kw0 = kv0 + warp * per_warp, kw1 = min(kv1, kw0 + per_warp);
    const int nkeys = max(kw1 - kw0, 0);

    float * part = p.ws + ((((int64_t) i3 * p.n_head_kv + hk) * p.n_splits + split) * R) * (D + 2);

    for (int r0 = 0; r0 < R; r0 += FD_RT) {
        // rows r0 .. r0+3: row r = iq * gqa + hg  ->  query iq, head hk * gqa + hg
        __syncthreads();
        {
            constexpr int NT = FD_WARPS * 32, QI = FD_RT * D / NT;      // all loads are issued before the first store
            float qv[QI];
#pragma unroll
            for (int it = 0; it < QI; ++it) {
                const int i = threadIdx.x + it * NT, rr = i / D, d = i % D, r = r0 + rr;
                qv[it] = 0.0f;
                if (r < R) {
                    const int iq = r / p.gqa, head = hk * p.gqa + r % p.gqa;
                    qv[it] = *(const float *) (p.q + (int64_t) iq * p.q_nb1 + (int64_t) head * p.q_nb2 + (int64_t) i3 * p.q_nb3 + d * 4);
                }
            }
#pragma unroll
            for (int it = 0; it < QI; ++it) { const int i = threadIdx.x + it * NT; qs[i / D][i % D] = qv[it]; }
        }
        __syncthreads();

        // ---- scores: 8 lanes per key, 4 keys per step ----
        const int sub = lane & 7, kq = lane >> 3;
        float slope[FD_RT];
        const __half * mrow[FD_RT];
#pragma unroll
        for (int rr = 0; rr < FD_RT; ++rr) {
            const int r = min(r0 + rr, R - 1), iq = r / p.gqa, head = hk * p.gqa + r % p.gqa;
            slope[rr] = 1.0f;
            if (p.max_bias > 0.0f) slope[rr] = head < p.n_head_log2 ? powf(p.m0, (float) (head + 1)) : powf(p.m1, (float) (2 * (head - p.n_head_log2) + 1));
            mrow[rr] = p.mask ? (const __half *) (p.mask + (int64_t) iq * p.m_nb1) : nullptr;
        }
        float mx[FD_RT];
#pragma unroll
        for (int rr = 0; rr < FD_RT; ++rr) mx[rr] = -INFINITY;
        // 16 keys per step: each 8-lane group fetches its 4 keys' chunks before any arithmetic, so four
        // K rows per lane are in flight instead of one
        for (int kb = 0; kb < nkeys; kb += 16) {
            uint4 kreg[4][D / 64];
            __half mval[4][FD_RT];                                // mask values of the same keys, fetched with them
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int kl = kb + u * 4 + kq;
                if (kl < nkeys) {
                    const char * kr = kbase + (int64_t) (kw0 + kl) * p.k_nb1;
#pragma unroll
                    for (int c = 0; c < D / 64; ++c) kreg[u][c] = __ldg((const uint4 *) (kr + (c * 8 + sub) * 16));
#pragma unroll
                    for (int rr = 0; rr < FD_RT; ++rr) mval[u][rr] = mrow[rr] ? mrow[rr][kw0 + kl] : __float2half(0.0f);
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int kl = kb + u * 4 + kq;
                if (kb + u * 4 >= nkeys) break;                   // warp-uniform
                float acc[FD_RT] = {0.0f, 0.0f, 0.0f, 0.0f};
                if (kl < nkeys) {
#pragma unroll
                    for (int c = 0; c < D / 64; ++c) {            // D/8 16-byte chunks per row, 8 lanes -> D/64 chunks each
                        const int chunk = c * 8 + sub;
                        const __half2 * kh = (const __half2 *) &kreg[u][c];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float2 kf = __half22float2(kh[e]);
                            const int d = chunk * 8 + 2 * e;
#pragma unroll
                            for (int rr = 0; rr < FD_RT; ++rr) acc[rr] += kf.x * qs[rr][d] + kf.y * qs[rr][d + 1];
                        }
                    }
                }
#pragma unroll
                for (int rr = 0; rr < FD_RT; ++rr) {
                    acc[rr] += __shfl_xor_sync(0xffffffffu, acc[rr], 1);
                    acc[rr] += __shfl_xor_sync(0xffffffffu, acc[rr], 2);
                    acc[rr] += __shfl_xor_sync(0xffffffffu, acc[rr], 4);
                }
                if (sub == 0 && kl < nkeys) {
                    float4 sv;
                    float * s4 = (float *) &sv;
#pragma unroll
                    for (int rr = 0; rr < FD_RT; ++rr) {
                        float s = acc[rr] * p.scale;
                        if (p.softcap != 0.0f) s = p.softcap * tanhf(s);
                        if (mrow[rr]) s += slope[rr] * __half2float(mval[u][rr]);
                        s4[rr] = s;
                        mx[rr] = fmaxf(mx[rr], s);
                    }
                    *(float4 *) ps[warp][kl] = sv;
                }
            }
        }
        __syncwarp();
        // ---- softmax over this warp's keys ----
        float lsum[FD_RT];
#pragma unroll
        for (int rr = 0; rr < FD_RT; ++rr) { mx[rr] = warp_max(mx[rr]); lsum[rr] = 0.0f; }
        for (int kl = lane; kl < nkeys; kl += 32) {
            float4 sv = *(float4 *) ps[warp][kl];
            float * s4 = (float *) &sv;
#pragma unroll
            for (int rr = 0; rr < FD_RT; ++rr) {
                const float e = (mx[rr] == -INFINITY || s4[rr] == -INFINITY) ? 0.0f : expf(s4[rr] - mx[rr]);
                s4[rr] = e; lsum[rr] += e;
            }
            *(float4 *) ps[warp][kl] = sv;
        }
#pragma unroll
        for (int rr = 0; rr < FD_RT; ++rr) lsum[rr] = warp_sum(lsum[rr]);
        __syncwarp();
        // ---- O = P V: lanes across the head dimension ----
        float o[FD_RT][DPL];
#pragma unroll
        for (int rr = 0; rr < FD_RT; ++rr)
#pragma unroll
            for (int i = 0; i < DPL; ++i) o[rr][i] = 0.0f;
        if (p.v_t) {
            // transposed V: row d of the cache holds the keys contiguously; a lane streams its DPL rows, 8 keys per load
            for (int kb = 0; kb < nkeys; kb += 8) {
                uint4 raw[DPL];
#pragma unroll
                for (int i = 0; i < DPL; ++i) raw[i] = __ldg((const uint4 *) (vbase + (int64_t) (lane * DPL + i) * p.v_nbd + (int64_t) (kw0 + kb) * 2));
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    if (kb + u >= nkeys) break;                     // (what lies past the last key of the cache row is not touched)
                    const float4 pv = *(const float4 *) ps[warp][kb + u];
                    if (pv.x == 0.0f && pv.y == 0.0f && pv.z == 0.0f && pv.w == 0.0f) continue;   // masked key (warp-uniform)
                    const float pr[FD_RT] = {pv.x, pv.y, pv.z, pv.w};
#pragma unroll
                    for (int i = 0; i < DPL; ++i) {
                        const float vf = __half2float(((const __half *) &raw[i])[u]);
#pragma unroll
                        for (int rr = 0; rr < FD_RT; ++rr) o[rr][i] += pr[rr] * vf;
                    }
                }
            }
        } else
        for (int kb = 0; kb < nkeys; kb += FD_VROWS) {              // 16 V rows (4 KB per warp) in flight per lane
            uint2 raw[FD_VROWS];
#pragma unroll
            for (int u = 0; u < FD_VROWS; ++u) {
                const int kl = min(kb + u, nkeys - 1);
                const char * vr = vbase + (int64_t) (kw0 + kl) * p.v_nb1 + lane * DPL * 2;
                if (DPL == 4) raw[u] = __ldg((const uint2 *) vr);
                else { raw[u].x = __ldg((const uint32_t *) vr); raw[u].y = 0; }
            }
#pragma unroll
            for (int u = 0; u < FD_VROWS; ++u) {
                if (kb + u >= nkeys) break;
                const float4 pv = *(const float4 *) ps[warp][kb + u];
                if (pv.x == 0.0f && pv.y == 0.0f && pv.z == 0.0f && pv.w == 0.0f) continue;   // masked key (warp-uniform)
                const float2 a = __half22float2(*(const __half2 *) &raw[u].x), b2 = __half22float2(*(const __half2 *) &raw[u].y);
                const float vf[4] = {a.x, a.y, b2.x, b2.y};
                const float pr[FD_RT] = {pv.x, pv.y, pv.z, pv.w};
#pragma unroll
                for (int rr = 0; rr < FD_RT; ++rr)
#pragma unroll
                    for (int i = 0; i < DPL; ++i) o[rr][i] += pr[rr] * vf[i];
            }
        }
        // ---- merge the 4 warps ----
        if (lane == 0) {
#pragma unroll
            for (int rr = 0; rr < FD_RT; ++rr) { w_m[warp][rr] = mx[rr]; w_l[warp][rr] = lsum[rr]; }
        }
#pragma unroll
        for (int rr = 0; rr < FD_RT; ++rr)
#pragma unroll
            for (int i = 0; i < DPL; ++i) w_o[warp][rr][lane * DPL + i] = o[rr][i];
        __syncthreads();
        for (int i = threadIdx.x; i < FD_RT * D; i += blockDim.x) {
            const int rr = i / D, d = i % D, r = r0 + rr;
            if (r >= R) continue;
            float M = -INFINITY;
#pragma unroll
            for (int w = 0; w < FD_WARPS; ++w) M = fmaxf(M, w_m[w][rr]);
            float L = 0.0f, acc = 0.0f;
#pragma unroll
            for (int w = 0; w < FD_WARPS; ++w) {
                const float f = (w_m[w][rr] == -INFINITY) ? 0.0f : expf(w_m[w][rr] - M);
                L += w_l[w][rr] * f; acc += w_o[w][rr][d] * f;
            }
            if (p.n_splits == 1) {
                const int iq = r / p.gqa, head = hk * p.gqa + r % p.gqa;
                const float val = acc / L;
                p.dst[(((int64_t) i3 * p.n_q + iq) * p.n_head + head) * D + d] = val;
                if (D == 128 && p.act_out) fd_emit_act(p.act_out + (int64_t) iq * p.n_head + head, d, val);   // r is uniform per pass
            } else {
                part[(int64_t) r * (D + 2) + d] = acc;
                if (d == 0) { part[(int64_t) r * (D + 2) + D] = M; part[(int64_t) r * (D + 2) + D + 1] = L; }
            }
        }
    }

    fd_merge_splits<D>(p, R, i3, hk, &ps[0][0][0], &ticket_sh);
}

// ---------------------------------------------------------------------------
// Tensor-core variant.  The kernel above spends about 140 warp instructions per key (FP32 dot products with the query in
// shared memory) and is bound by instruction issue long before HBM.  Here a warp takes 16 keys per step and computes
//   S[8 rows x 16 keys] = Q K^T   as mma.sync m16n8k16 (the 8 (query, head) rows in the upper half of the 16-row operand),
//   O^T[D x 8 rows]    += V^T P^T as mma.sync m16n8k16 with the head dimension as the 16-row operand,
// so the probabilities leave the first product in exactly the register layout the second one wants (no shuffles, no
// shared memory), with an online softmax per step.  Every operand fragment is fetched straight from global memory with
// 128-bit loads: which head-dimension index (and which key) a fragment slot stands for is free as long as both
// operands of a product agree, so the slots are numbered to make each thread's data contiguous:
//   Q.K:  k-slot (2t, 2t+1, 2t+8, 2t+9) of step (blk, j) <-> d = 32 blk + 8 t + 4 j + (0, 1, 2, 3)
//   keys: column c of key tile nt <-> key 4 (c / 2) + 2 nt + c % 2, so thread (g, t) ends up with the scores of its row
//         for keys 4t .. 4t+3, the four keys whose V rows (or 8-byte run of a transposed V row) it loads
//   P.V:  operand row m of tile mt <-> d = (D / 8) (m % 8) + (D / 16) (m / 8) + mt: thread g reads 32 contiguous bytes of a V row
// RG = 2 handles 16 rows per pass (both halves of the query operand, two probability operands).
// ---------------------------------------------------------------------------
__device__ __forceinline__ void fd_mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t fd_pack_h2(float a, float b) { const __half2 h = __floats2half2_rn(a, b); return *(const uint32_t *) &h; }

template <int D, int RG>
__global__ void __launch_bounds__(FD_WARPS * 32, RG == 1 ? 3 : 2) fattn_dec_mma_kernel(const FdParams p) {
    pdl_enter();
    constexpr int NR = 8 * RG;                                    // rows per pass
    constexpr int KS = D / 16;                                    // k-steps of Q.K; 16-value tiles of the head dimension in P.V
    constexpr int WPR = D / 16;                                   // 32-bit words of a V row held by one thread (D / 8 halfs)
    constexpr int DP = D + 8;                                     // a row of w_o: one pad float after every D / 8 values (the stores below would hit two banks otherwise)
    constexpr int SB = FD_WARPS * NR * DP > FD_MERGE_FLOATS ? FD_WARPS * NR * DP : FD_MERGE_FLOATS;
    __shared__ __align__(16) float sbuf[SB];                      // w_o[warp][row][DP]; the split merge's scratch at the end
    __shared__ float w_m[FD_WARPS][NR], w_l[FD_WARPS][NR];
    __shared__ unsigned ticket_sh;

    const int split = blockIdx.x, hk = blockIdx.y, i3 = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int R = p.n_q * p.gqa;
    const int k3 = i3 / p.q3_per_k3;
    const char * kbase = p.k + (int64_t) hk * p.k_nb2 + (int64_t) k3 * p.k_nb3;
    const char * vbase = p.v + (int64_t) hk * p.v_nb2 + (int64_t) k3 * p.v_nb3;

    const int kv0 = split * p.kv_per_split, kv1 = min(p.n_kv, kv0 + p.kv_per_split);           // kv_per_split is a multiple of 16
    const int per_warp = (((max(kv1 - kv0, 0) + FD_WARPS - 1) / FD_WARPS) + 15) & ~15;
    const int kw0 = kv0 + warp * per_warp, kw1 = min(kv1, kw0 + per_warp);
    const int nkeys = max(kw1 - kw0, 0);
    float * part = p.ws + ((((int64_t) i3 * p.n_head_kv + hk) * p.n_splits + split) * R) * (D + 2);

    for (int r0 = 0; r0 < R; r0 += NR) {
        __syncthreads();                                          // the previous pass has read sbuf
        // ---- this thread's rows: r0 + g (+ 8): query fragments, mask row, ALiBi slope ----
        uint32_t qa[KS][2 * RG];
        float slope[RG];
        const __half * mrow[RG];
#pragma unroll
        for (int rg = 0; rg < RG; ++rg) {
            const int r = r0 + g + 8 * rg;
            const bool live = r < R;
            const int rc = live ? r : R - 1, iq = rc / p.gqa, head = hk * p.gqa + rc % p.gqa;
            const char * qp = p.q + (int64_t) iq * p.q_nb1 + (int64_t) head * p.q_nb2 + (int64_t) i3 * p.q_nb3;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                const int d = 32 * (ks >> 1) + 8 * t + 4 * (ks & 1);
                const float4 f = live ? *(const float4 *) (qp + d * 4) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                qa[ks][2 * rg] = fd_pack_h2(f.x, f.y); qa[ks][2 * rg + 1] = fd_pack_h2(f.z, f.w);
            }
            slope[rg] = 1.0f;
            if (p.max_bias > 0.0f) slope[rg] = head < p.n_head_log2 ? powf(p.m0, (float) (head + 1)) : powf(p.m1, (float) (2 * (head - p.n_head_log2) + 1));
            mrow[rg] = p.mask ? (const __half *) (p.mask + (int64_t) iq * p.m_nb1) : nullptr;
        }
        float m_run[RG], l_run[RG], o[RG][KS][4];
#pragma unroll
        for (int rg = 0; rg < RG; ++rg) {
            m_run[rg] = -INFINITY; l_run[rg] = 0.0f;
#pragma unroll
            for (int mt = 0; mt < KS; ++mt)
#pragma unroll
                for (int c = 0; c < 4; ++c) o[rg][mt][c] = 0.0f;
        }

#pragma unroll 1
        for (int kb = 0; kb < nkeys; kb += 16) {
            // ---- all loads of the step first: two K rows (the columns g of the two key tiles) and this thread's share of V ----
            const int kc = kb + (g >> 1) * 4 + (g & 1);
            const char * kr0 = kbase + (int64_t) (kw0 + min(kc, nkeys - 1)) * p.k_nb1 + t * 16;
            const char * kr1 = kbase + (int64_t) (kw0 + min(kc + 2, nkeys - 1)) * p.k_nb1 + t * 16;
            uint4 k0[D / 32], k1[D / 32];
#pragma unroll
            for (int b = 0; b < D / 32; ++b) { k0[b] = __ldg((const uint4 *) (kr0 + b * 64)); k1[b] = __ldg((const uint4 *) (kr1 + b * 64)); }
            uint32_t vr[4 * WPR];
            if (p.v_t) {
                // transposed cache: keys 4t .. 4t+3 of head-dimension row (D / 8) g + e are 8 contiguous bytes
                const int kk = kb + 4 * t, nv = nkeys - kk;                        // valid keys of this thread's four
#pragma unroll
                for (int e = 0; e < D / 8; ++e) {
                    uint2 x = make_uint2(0u, 0u);
                    if (nv > 0) x = __ldg((const uint2 *) (vbase + (int64_t) ((D / 8) * g + e) * p.v_nbd + (int64_t) (kw0 + kk) * 2));
                    if (nv < 4) {                                 // what lies past the last key may be anything: it must not reach the product
                        x.x &= nv >= 2 ? 0xffffffffu : (nv == 1 ? 0x0000ffffu : 0u);
                        x.y &= nv >= 4 ? 0xffffffffu : (nv == 3 ? 0x0000ffffu : 0u);
                    }
                    vr[2 * e] = x.x; vr[2 * e + 1] = x.y;
                }
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const char * vp = vbase + (int64_t) (kw0 + min(kb + 4 * t + i, nkeys - 1)) * p.v_nb1 + (D / 8) * g * 2;
#pragma unroll
                    for (int w4 = 0; w4 < D / 64; ++w4) {
                        const uint4 x = __ldg((const uint4 *) (vp + 16 * w4));
                        vr[i * WPR + 4 * w4] = x.x; vr[i * WPR + 4 * w4 + 1] = x.y; vr[i * WPR + 4 * w4 + 2] = x.z; vr[i * WPR + 4 * w4 + 3] = x.w;
                    }
                }
            }
            // mask values of this thread's keys (4t .. 4t+3 of the step) for its rows
            float mv[RG][4];
#pragma unroll
            for (int rg = 0; rg < RG; ++rg) {
#pragma unroll
                for (int i = 0; i < 4; ++i) mv[rg][i] = 0.0f;
                if (mrow[rg]) {
                    const __half * mp = mrow[rg] + kw0 + kb + 4 * t;
                    if (p.mask_al8 && kb + 4 * t + 3 < nkeys) {
                        const uint2 x = __ldg((const uint2 *) mp);
                        const float2 a = __half22float2(*(const __half2 *) &x.x), b = __half22float2(*(const __half2 *) &x.y);
                        mv[rg][0] = a.x; mv[rg][1] = a.y; mv[rg][2] = b.x; mv[rg][3] = b.y;
                    } else {
#pragma unroll
                        for (int i = 0; i < 4; ++i) if (kb + 4 * t + i < nkeys) mv[rg][i] = __half2float(__ldg(mp + i));
                    }
                }
            }

            // ---- S = Q K^T ----
            float sc[2][4];
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int c = 0; c < 4; ++c) sc[nt][c] = 0.0f;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                const uint4 a = k0[ks >> 1], b = k1[ks >> 1];
                const uint32_t a1 = RG == 2 ? qa[ks][2] : 0u, a3 = RG == 2 ? qa[ks][3] : 0u;
                fd_mma16816(sc[0], qa[ks][0], a1, qa[ks][1], a3, (ks & 1) ? a.z : a.x, (ks & 1) ? a.w : a.y);
                fd_mma16816(sc[1], qa[ks][0], a1, qa[ks][1], a3, (ks & 1) ? b.z : b.x, (ks & 1) ? b.w : b.y);
            }

            // ---- online softmax: this thread has keys 4t .. 4t+3 of row g (+ 8) ----
            uint32_t pb[RG][2];
            float fac[RG];
            bool same = true;
#pragma unroll
            for (int rg = 0; rg < RG; ++rg) {
                float sv[4] = {sc[0][2 * rg], sc[0][2 * rg + 1], sc[1][2 * rg], sc[1][2 * rg + 1]};
                float cm = -INFINITY;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float x = sv[i] * p.scale;
                    if (p.softcap != 0.0f) x = p.softcap * tanhf(x);
                    x += slope[rg] * mv[rg][i];
                    if (kb + 4 * t + i >= nkeys) x = -INFINITY;
                    sv[i] = x; cm = fmaxf(cm, x);
                }
                cm = fmaxf(cm, __shfl_xor_sync(0xffffffffu, cm, 1));
                cm = fmaxf(cm, __shfl_xor_sync(0xffffffffu, cm, 2));
                const float m_new = fmaxf(m_run[rg], cm);
                fac[rg] = (m_run[rg] == m_new) ? 1.0f : ((m_run[rg] == -INFINITY) ? 0.0f : expf(m_run[rg] - m_new));
                same = same && fac[rg] == 1.0f;
                float pr[4], ls = 0.0f;
#pragma unroll
                for (int i = 0; i < 4; ++i) { pr[i] = (m_new == -INFINITY || sv[i] == -INFINITY) ? 0.0f : expf(sv[i] - m_new); ls += pr[i]; }
                l_run[rg] = l_run[rg] * fac[rg] + ls;             // this thread's part of the row sum
                m_run[rg] = m_new;
                pb[rg][0] = fd_pack_h2(pr[0], pr[1]); pb[rg][1] = fd_pack_h2(pr[2], pr[3]);
            }
            if (!__all_sync(0xffffffffu, same)) {
                // the accumulators of this thread belong to rows 2t and 2t+1 (+ 8): their factors live in the lanes of those rows
#pragma unroll
                for (int rg = 0; rg < RG; ++rg) {
                    const float f0 = __shfl_sync(0xffffffffu, fac[rg], 8 * t), f1 = __shfl_sync(0xffffffffu, fac[rg], 8 * t + 4);
#pragma unroll
                    for (int mt = 0; mt < KS; ++mt) { o[rg][mt][0] *= f0; o[rg][mt][1] *= f1; o[rg][mt][2] *= f0; o[rg][mt][3] *= f1; }
                }
            }

            // ---- O^T += V^T P^T ----
#pragma unroll
            for (int mt = 0; mt < KS; ++mt) {
                uint32_t a0, a1, a2, a3;
                if (p.v_t) {
                    a0 = vr[2 * mt]; a2 = vr[2 * mt + 1]; a1 = vr[2 * (D / 16 + mt)]; a3 = vr[2 * (D / 16 + mt) + 1];
                } else {
                    const uint32_t sel = (mt & 1) ? 0x7632u : 0x5410u;
                    const int wl = mt >> 1, wh = (D / 16 + mt) >> 1;
                    a0 = __byte_perm(vr[wl], vr[WPR + wl], sel);           a1 = __byte_perm(vr[wh], vr[WPR + wh], sel);
                    a2 = __byte_perm(vr[2 * WPR + wl], vr[3 * WPR + wl], sel); a3 = __byte_perm(vr[2 * WPR + wh], vr[3 * WPR + wh], sel);
                }
#pragma unroll
                for (int rg = 0; rg < RG; ++rg) fd_mma16816(o[rg][mt], a0, a1, a2, a3, pb[rg][0], pb[rg][1]);
            }
        }

        // ---- the warp's result to shared memory ----
        float * w_o = sbuf + (size_t) warp * NR * DP;
#pragma unroll
        for (int rg = 0; rg < RG; ++rg) {
            float l = l_run[rg];
            l += __shfl_xor_sync(0xffffffffu, l, 1);
            l += __shfl_xor_sync(0xffffffffu, l, 2);
            if (t == 0) { w_m[warp][g + 8 * rg] = m_run[rg]; w_l[warp][g + 8 * rg] = l; }
#pragma unroll
            for (int mt = 0; mt < KS; ++mt)
#pragma unroll
                for (int c = 0; c < 4; ++c)
                    w_o[(8 * rg + 2 * t + (c & 1)) * DP + (D / 8) * g + g + (c >> 1) * (D / 16) + mt] = o[rg][mt][c];
        }
        __syncthreads();
        // ---- merge the 4 warps ----
        for (int i = threadIdx.x; i < NR * D; i += blockDim.x) {
            const int rr = i / D, d = i % D, r = r0 + rr;
            if (r >= R) continue;                                 // (uniform over a warp)
            float M = -INFINITY;
#pragma unroll
            for (int w = 0; w < FD_WARPS; ++w) M = fmaxf(M, w_m[w][rr]);
            float L = 0.0f, acc = 0.0f;
#pragma unroll
            for (int w = 0; w < FD_WARPS; ++w) {
                const float f = (w_m[w][rr] == -INFINITY) ? 0.0f : expf(w_m[w][rr] - M);
                L += w_l[w][rr] * f; acc += sbuf[((size_t) w * NR + rr) * DP + d + d / (D / 8)] * f;
            }
            if (p.n_splits == 1) {
                const int iq = r / p.gqa, head = hk * p.gqa + r % p.gqa;
                const float val = acc / L;
                p.dst[(((int64_t) i3 * p.n_q + iq) * p.n_head + head) * D + d] = val;
                if (D == 128 && p.act_out) fd_emit_act(p.act_out + (int64_t) iq * p.n_head + head, d, val);
            } else {
                part[(int64_t) r * (D + 2) + d] = acc;
                if (d == 0) { part[(int64_t) r * (D + 2) + D] = M; part[(int64_t) r * (D + 2) + D + 1] = L; }
            }
        }
    }
    fd_merge_splits<D>(p, R, i3, hk, sbuf, &ticket_sh);
}

static constexpr int FD_TICKETS = FATTN_DEC_TICKETS;

bool fattn_dec_applicable(const TensorD & q, const TensorD & k, const TensorD & v, const TensorD * mask) {
    const int64_t D = q.ne[0];
    if (D != 64 && D != 128) return false;
    if (q.ne[1] > 8 || q.ne[2] % k.ne[2] != 0 || k.ne[1] > 65536) return false;
    if ((q.ne[2] / k.ne[2]) * q.ne[1] > 64) return false;
    if (k.ne[2] * q.ne[3] > FD_TICKETS) return false;
    auto al16 = [](const TensorD & t) { return ((uintptr_t) t.data & 15) == 0 && (t.nb[1] & 15) == 0 && (t.nb[2] & 15) == 0 && (t.nb[3] & 15) == 0; };
    if (!al16(k)) return false;
    if (v.nb[0] == 2) { if (!al16(v)) return false; }
    else if (v.nb[1] != 2 || ((uintptr_t) v.data & 15) || (v.nb[0] & 15) || (v.nb[2] & 15) || (v.nb[3] & 15)) return false;   // transposed V
    if (((uintptr_t) q.data & 3) || (q.nb[1] & 3) || (q.nb[2] & 3) || (q.nb[3] & 3)) return false;
    (void) mask;
    return true;
}

static int fd_pick_splits(int64_t n_head_kv_total, int64_t n_kv, int sm_count, int64_t R, int per_sm = 4) {
    int64_t want = per_sm == 4 ? ((int64_t) sm_count * 4 + n_head_kv_total - 1) / n_head_kv_total : ((int64_t) sm_count * per_sm) / n_head_kv_total;   // (fewer CTAs per SM: one full wave)
    const int64_t max_by_kv = (n_kv + 63) / 64;                       // at least 64 keys per CTA (16 per warp: one score step)
    int64_t s = want < max_by_kv ? want : max_by_kv;
    const int64_t min_by_cap = (n_kv + FD_WARPS * FD_MAX_KEYS_PER_WARP - 1) / (FD_WARPS * FD_MAX_KEYS_PER_WARP);
    if (s < min_by_cap) s = min_by_cap;
    if (s > 128) s = s > min_by_cap ? (min_by_cap > 128 ? min_by_cap : 128) : s;
    const int64_t cap_by_wgt = (FD_MERGE_FLOATS / 2) / (R > 0 ? R : 1);   // merge weights and sums share ps[]
    if (s > cap_by_wgt) s = cap_by_wgt > min_by_cap ? cap_by_wgt : min_by_cap;
    if (s < 1) s = 1;
    return (int) s;
}

size_t fattn_dec_workspace_bytes(const TensorD & q, const TensorD & k, int sm_count) {
    const int64_t R = (q.ne[2] / k.ne[2]) * q.ne[1];
    const int splits = fd_pick_splits(k.ne[2] * q.ne[3], k.ne[1], sm_count, R);
    return (size_t) q.ne[3] * k.ne[2] * splits * R * (q.ne[0] + 2) * 4 + 256;
}

cudaError_t launch_fattn_dec(const TensorD & q, const TensorD & k, const TensorD & v, const TensorD * mask, const TensorD & dst,
                             const FattnParams & fp, void * tickets, void * partials, const LaunchCtx & c, void * act128_out) {
    FdParams p = {};
    p.act_out = (q.ne[0] == 128 && q.ne[3] == 1) ? (blk_act128 *) act128_out : nullptr;
    p.q = (const char *) q.data; p.q_nb1 = q.nb[1]; p.q_nb2 = q.nb[2]; p.q_nb3 = q.nb[3];
    p.k = (const char *) k.data; p.k_nb1 = k.nb[1]; p.k_nb2 = k.nb[2]; p.k_nb3 = k.nb[3];
    p.v = (const char *) v.data; p.v_nb1 = v.nb[1]; p.v_nb2 = v.nb[2]; p.v_nb3 = v.nb[3];
    p.v_t = v.nb[0] != 2 ? 1 : 0; p.v_nbd = v.nb[0];
    p.mask = mask ? (const char *) mask->data : nullptr; p.m_nb1 = mask ? mask->nb[1] : 0;
    p.dst = (float *) dst.data; p.ws = (float *) partials; p.tickets = (unsigned *) tickets;
    p.n_q = (int) q.ne[1]; p.n_kv = (int) k.ne[1]; p.n_head = (int) q.ne[2]; p.n_head_kv = (int) k.ne[2];
    p.gqa = (int) (q.ne[2] / k.ne[2]); p.q3_per_k3 = (int) (q.ne[3] / k.ne[3]);
    const int64_t R = (int64_t) p.gqa * p.n_q;
    // the tensor-core kernel wants 128-bit loads of the query rows; GGML_B200_FA_DEC_MMA=0 keeps the FP32 kernel (for comparisons)
    static const bool mma_on = [] { const char * e = getenv("GGML_B200_FA_DEC_MMA"); return !(e && e[0] == '0'); }();
    const bool use_mma = mma_on && ((uintptr_t) q.data & 15) == 0 && (q.nb[1] & 15) == 0 && (q.nb[2] & 15) == 0 && (q.nb[3] & 15) == 0;
    p.mask_al8 = mask && ((uintptr_t) mask->data & 7) == 0 && (mask->nb[1] & 7) == 0;
    p.n_splits = fd_pick_splits(k.ne[2] * q.ne[3], k.ne[1], c.sm_count, R, use_mma ? (R > 8 ? 2 : 3) : 4);
    p.kv_per_split = (int) (((k.ne[1] + p.n_splits - 1) / p.n_splits + 15) & ~(int64_t) 15);       // 16 keys: one tensor-core step; aligned runs of a transposed V row
    if (use_mma) {
        // whole steps for every warp: 64 keys per CTA and step; the number of splits follows from that
        p.kv_per_split = (p.kv_per_split + 16 * FD_WARPS - 1) / (16 * FD_WARPS) * (16 * FD_WARPS);
        p.n_splits = (int) ((k.ne[1] + p.kv_per_split - 1) / p.kv_per_split);
    }
    p.scale = fp.scale; p.softcap = fp.logit_softcap; p.max_bias = fp.max_bias;
    if (p.softcap != 0.0f) p.scale /= p.softcap;
    int nh2 = 1; while (nh2 * 2 <= p.n_head) nh2 *= 2;
    p.n_head_log2 = nh2;
    p.m0 = powf(2.0f, -fp.max_bias / (float) nh2);
    p.m1 = powf(2.0f, -(fp.max_bias / 2.0f) / (float) nh2);
    dim3 grid((unsigned) p.n_splits, (unsigned) p.n_head_kv, (unsigned) q.ne[3]);
    if (use_mma) {
        if (q.ne[0] == 64) {
            if (R > 8) (void) (launch_err = launch_k(c.use_pdl, c.stream, fattn_dec_mma_kernel<64, 2>, dim3(grid), dim3(FD_WARPS * 32), 0, p));
            else       (void) (launch_err = launch_k(c.use_pdl, c.stream, fattn_dec_mma_kernel<64, 1>, dim3(grid), dim3(FD_WARPS * 32), 0, p));
        } else {
            if (R > 8) (void) (launch_err = launch_k(c.use_pdl, c.stream, fattn_dec_mma_kernel<128, 2>, dim3(grid), dim3(FD_WARPS * 32), 0, p));
            else       (void) (launch_err = launch_k(c.use_pdl, c.stream, fattn_dec_mma_kernel<128, 1>, dim3(grid), dim3(FD_WARPS * 32), 0, p));
        }
        return cudaGetLastError();
    }
    if (q.ne[0] == 64) (void) (launch_err = launch_k(c.use_pdl, c.stream, fattn_dec_kernel<64>, dim3(grid), dim3(FD_WARPS * 32), 0, p));
    else               (void) (launch_err = launch_k(c.use_pdl, c.stream, fattn_dec_kernel<128>, dim3(grid), dim3(FD_WARPS * 32), 0, p));
    return cudaGetLastError();
}

}  // namespace b200
