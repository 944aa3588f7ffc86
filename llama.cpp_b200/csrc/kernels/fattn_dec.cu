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

namespace b200 {

static constexpr int FD_WARPS = 4, FD_RT = 4, FD_MAX_KEYS_PER_WARP = 256;

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

template <int D>
__global__ void __launch_bounds__(FD_WARPS * 32) fattn_dec_kernel(const FdParams p) {
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
        for (int kb = 0; kb < nkeys; kb += 8) {                     // 8 V rows in flight per lane
            uint2 raw[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int kl = min(kb + u, nkeys - 1);
                const char * vr = vbase + (int64_t) (kw0 + kl) * p.v_nb1 + lane * DPL * 2;
                if (DPL == 4) raw[u] = __ldg((const uint2 *) vr);
                else { raw[u].x = __ldg((const uint32_t *) vr); raw[u].y = 0; }
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
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

    if (p.n_splits > 1) {
        // ---- the last CTA of this KV head merges all splits ----
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) ticket_sh = atomicAdd(&p.tickets[i3 * p.n_head_kv + hk], 1u);
        __syncthreads();
        if (ticket_sh == (unsigned) p.n_splits - 1) {
            __threadfence();
            const float * base = p.ws + (((int64_t) i3 * p.n_head_kv + hk) * p.n_splits) * R * (D + 2);
            // per (row, split) weights exp(m_s - M) / L in shared memory (reusing ps): all (max, sum) pairs are
            // fetched in one parallel pass, then one warp per row reduces over the splits
            float * wgt = &ps[0][0][0];                               // R * n_splits floats, at most half of ps[] (fd_pick_splits)
            float * wl  = wgt + FD_WARPS * FD_MAX_KEYS_PER_WARP * FD_RT / 2;   // the sums, same indexing, in the upper half
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
            for (int i = threadIdx.x; i < R * D; i += blockDim.x) {
                const int r = i / D, d = i % D;
                float acc0 = 0.0f, acc1 = 0.0f, acc2 = 0.0f, acc3 = 0.0f;
                int s = 0;
                for (; s + 4 <= p.n_splits; s += 4) {                  // four independent loads per step
                    acc0 += base[((int64_t) (s + 0) * R + r) * (D + 2) + d] * wgt[r * p.n_splits + s + 0];
                    acc1 += base[((int64_t) (s + 1) * R + r) * (D + 2) + d] * wgt[r * p.n_splits + s + 1];
                    acc2 += base[((int64_t) (s + 2) * R + r) * (D + 2) + d] * wgt[r * p.n_splits + s + 2];
                    acc3 += base[((int64_t) (s + 3) * R + r) * (D + 2) + d] * wgt[r * p.n_splits + s + 3];
                }
                for (; s < p.n_splits; ++s) acc0 += base[((int64_t) s * R + r) * (D + 2) + d] * wgt[r * p.n_splits + s];
                const int iq = r / p.gqa, head = hk * p.gqa + r % p.gqa;
                const float val = (acc0 + acc1) + (acc2 + acc3);
                p.dst[(((int64_t) i3 * p.n_q + iq) * p.n_head + head) * D + d] = val;
                if (D == 128 && p.act_out) fd_emit_act(p.act_out + (int64_t) iq * p.n_head + head, d, val);
            }
            if (threadIdx.x == 0) p.tickets[i3 * p.n_head_kv + hk] = 0;      // ready for the next launch
        }
    }
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

static int fd_pick_splits(int64_t n_head_kv_total, int64_t n_kv, int sm_count, int64_t R) {
    int64_t want = ((int64_t) sm_count * 4 + n_head_kv_total - 1) / n_head_kv_total;
    const int64_t max_by_kv = (n_kv + 63) / 64;                       // at least 64 keys per CTA (16 per warp: one score step)
    int64_t s = want < max_by_kv ? want : max_by_kv;
    const int64_t min_by_cap = (n_kv + FD_WARPS * FD_MAX_KEYS_PER_WARP - 1) / (FD_WARPS * FD_MAX_KEYS_PER_WARP);
    if (s < min_by_cap) s = min_by_cap;
    if (s > 128) s = s > min_by_cap ? (min_by_cap > 128 ? min_by_cap : 128) : s;
    const int64_t cap_by_wgt = (FD_WARPS * FD_MAX_KEYS_PER_WARP * FD_RT / 2) / (R > 0 ? R : 1);   // merge weights and sums share ps[]
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
    p.n_splits = fd_pick_splits(k.ne[2] * q.ne[3], k.ne[1], c.sm_count, (int64_t) p.gqa * p.n_q);
    p.kv_per_split = (int) ((k.ne[1] + p.n_splits - 1) / p.n_splits);
    p.scale = fp.scale; p.softcap = fp.logit_softcap; p.max_bias = fp.max_bias;
    if (p.softcap != 0.0f) p.scale /= p.softcap;
    int nh2 = 1; while (nh2 * 2 <= p.n_head) nh2 *= 2;
    p.n_head_log2 = nh2;
    p.m0 = powf(2.0f, -fp.max_bias / (float) nh2);
    p.m1 = powf(2.0f, -(fp.max_bias / 2.0f) / (float) nh2);
    dim3 grid((unsigned) p.n_splits, (unsigned) p.n_head_kv, (unsigned) q.ne[3]);
    if (q.ne[0] == 64) (void) (launch_err = launch_k(c.use_pdl, c.stream, fattn_dec_kernel<64>, dim3(grid), dim3(FD_WARPS * 32), 0, p));
    else               (void) (launch_err = launch_k(c.use_pdl, c.stream, fattn_dec_kernel<128>, dim3(grid), dim3(FD_WARPS * 32), 0, p));
    return cudaGetLastError();
}

}  // namespace b200
