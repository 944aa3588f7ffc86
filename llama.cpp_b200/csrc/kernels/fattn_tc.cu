// FLASH_ATTN_EXT for batches of queries (prefill) on the sm_100a tensor cores: head size 128, F16 K and V.
//
// One CTA = 128 query rows of one head.  Roles:
//   warps 0-3  softmax: thread = query row.  They convert the Q tile to F16 into shared memory (K-major, 128-byte
//              swizzle) once, then per KV tile read the row of S = Q K^T from tensor memory (tcgen05.ld), apply scale and
//              mask, keep the running maximum and sum in FP32 (libllama requests GGML_PREC_F32, src/llama.cpp:595),
//              write P as F16 back to tensor memory (tcgen05.st), rescale the O accumulator in tensor memory when the
//              maximum moved, and at the end divide O by the sum and store it.
//   warp 4     one thread issues the MMAs: S(j) = Q K(j)^T (operands from shared-memory descriptors, 128 x 128 x 16, eight
//              per tile) into one of two S buffers, and O += P(j) V(j) with P from tensor memory and V as the N-contiguous
//              operand (V rows are [key][d] in the cache: d is contiguous); tcgen05.commit publishes S, frees K/V stages,
//              and tells the softmax warps that O may be touched.
//   warp 5     one thread loads K and V tiles (128 keys x 128 values, two 64-value boxes each) with tiled tensor copies
//              (cp.async.bulk.tensor.3d, no multicast) into two-stage rings.
// Tensor memory (512 columns): S0 [0,128) S1 [128,256) O [256,384) P0 [384,448) P1 [448,512).
// Whole 128 x 128 tiles that the mask sets to -inf (everything above the causal diagonal) are skipped by all roles, tiles
// the mask leaves at zero skip the mask read (per-tile flags from fattn_mask_flags_kernel, 64 x 64 granularity).
// Every wait is bounded; a role that gives up sets the CTA's abort flag and the status word.
// Replaces flash_attn_ext_f16 (ggml/src/ggml-cuda/fattn-mma-f16.cuh:69-529) for this shape; semantics of
// ggml_compute_forward_flash_attn_ext_f16 (ggml/src/ggml-cpu/ggml-cpu.c:10916-11129) without ALiBi and soft-capping
// (those, other head sizes and layouts stay on fattn_mma.cu / fattn.cu).
#include "common.cuh"
#include "kernels.h"
#include "tcgen05.cuh"
#include <math.h>

namespace b200 {

static constexpr int FT_BM = 128, FT_BN = 128, FT_D = 128;
static constexpr int FT_THREADS = 192;
static constexpr int FT_TILE_BYTES = FT_BN * FT_D * 2;             // 32 KB: two [128][64] F16 boxes
static constexpr int FT_SMEM = 5 * FT_TILE_BYTES + 1024;            // Q, 2 x K, 2 x V (+ alignment)

struct FtParams {
    const char * q; int64_t q_nb1, q_nb2;
    const char * mask; int64_t m_nb1;
    const uint8_t * flags; int flags_stride;        // [64-row q tiles][64-key kv tiles]: 0 mixed, 1 all -inf, 2 all zero
    float * dst;
    int n_q, n_kv, n_head, gqa;
    float scale_log2;                               // scale * log2(e)
    int v_t;                                        // V stored transposed (keys contiguous): the cache layout without FLASH_ATTN_EXT
    int * status;
};

// 0: mixed (read the mask), 1: skip the tile, 2: no mask needed
__device__ __forceinline__ int ft_tile_class(const FtParams & p, int qt128, int kt128) {
    if (!p.mask) return 2;
    int all1 = 1, all2 = 1;
#pragma unroll
    for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int b = 0; b < 2; ++b) {
            const int qi = 2 * qt128 + a, ki = 2 * kt128 + b;
            if (qi * 64 >= p.n_q || ki * 64 >= p.n_kv) continue;
            const int f = p.flags[qi * p.flags_stride + ki];
            if (f != 1) all1 = 0;
            if (f != 2) all2 = 0;
        }
    return all1 ? 1 : (all2 ? 2 : 0);
}

__global__ void __launch_bounds__(FT_THREADS, 1) fattn_tc_kernel(const FtParams p, const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    pdl_enter();
    uint8_t * smem = (uint8_t *) (((uintptr_t) smem_raw + 1023) & ~(uintptr_t) 1023);
    uint8_t * q_s = smem, * k_s = smem + FT_TILE_BYTES, * v_s = smem + 3 * FT_TILE_BYTES;
    __shared__ uint64_t q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], p_full[2], o_done;
    __shared__ uint32_t tmem_base_sh;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    const int qt = blockIdx.x, head = blockIdx.y, head_kv = head / p.gqa;
    const int q0 = qt * FT_BM;
    const int n_kt = (p.n_kv + FT_BN - 1) / FT_BN;

    if (tid == 0) {
        mbar_init(&q_full, 4);
        for (int s = 0; s < 2; ++s) {
            mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
            mbar_init(&s_full[s], 1); mbar_init(&p_full[s], 4);
        }
        mbar_init(&o_done, 1);
        abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 4) tmem_alloc(&tmem_base_sh, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_base_sh;
    constexpr uint32_t COL_S = 0, COL_O = 256, COL_P = 384;

    if (warp < 4) {
        // ------------------------------ softmax warps ------------------------------
        const int r = tid;                                             // row of the tile = tensor-memory lane
        const bool row_ok = q0 + r < p.n_q;
        const uint32_t lane_addr = tmem + ((uint32_t) (warp * 32) << 16);
        {   // Q tile: F32 -> F16, K-major rows of 128 bytes per 64-value half, 16-byte chunks XOR-swizzled by the row
            const float * qrow = (const float *) (p.q + (int64_t) (q0 + (row_ok ? r : 0)) * p.q_nb1 + (int64_t) head * p.q_nb2);
#pragma unroll
            for (int c = 0; c < FT_D / 8; ++c) {
                uint4 w = make_uint4(0, 0, 0, 0);
                if (row_ok) {
                    const float4 a = *(const float4 *) (qrow + c * 8), b = *(const float4 *) (qrow + c * 8 + 4);
                    __half2 h0 = __floats2half2_rn(a.x, a.y), h1 = __floats2half2_rn(a.z, a.w), h2 = __floats2half2_rn(b.x, b.y), h3 = __floats2half2_rn(b.z, b.w);
                    w = make_uint4(*(uint32_t *) &h0, *(uint32_t *) &h1, *(uint32_t *) &h2, *(uint32_t *) &h3);
                }
                const int atom = c >> 3, cc = c & 7;
                *(uint4 *) (q_s + atom * (FT_BM * 128) + r * 128 + ((cc ^ (r & 7)) << 4)) = w;
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(&q_full);
        }
        float m_run = -INFINITY, l_run = 0.0f;
        bool ok = true;
        int j = 0;                                                     // ordinal among the tiles that are processed
        for (int kt = 0; kt < n_kt && ok; ++kt) {
            const int cls = ft_tile_class(p, qt, kt);
            if (cls == 1) continue;
            const int b = j & 1;
            if (!mbar_wait_or_abort(smem_u32(&s_full[b]), (uint32_t) (j >> 1) & 1, &abort_flag)) { ok = false; break; }
            tc_fence_after();
            float s[FT_BN];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t v[32];
                tmem_ld32(lane_addr + COL_S + (uint32_t) (b * 128 + c * 32), v);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) s[c * 32 + i] = __uint_as_float(v[i]) * p.scale_log2;
            }
            const int kv0 = kt * FT_BN;
            if (cls == 0 && row_ok) {
                const uint4 * mrow = (const uint4 *) (p.mask + (int64_t) (q0 + r) * p.m_nb1 + (int64_t) kv0 * 2);
#pragma unroll
                for (int c = 0; c < FT_BN / 8; ++c) {
                    if (kv0 + c * 8 >= p.n_kv) break;
                    const uint4 mw = mrow[c];
                    const uint32_t w4[4] = {mw.x, mw.y, mw.z, mw.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float2 f = __half22float2(*(const __half2 *) &w4[i]);
                        s[c * 8 + 2 * i] += f.x * 1.4426950408889634f; s[c * 8 + 2 * i + 1] += f.y * 1.4426950408889634f;
                    }
                }
            }
            if (kv0 + FT_BN > p.n_kv) {                                // keys past the end (their K rows were zero-filled)
#pragma unroll
                for (int i = 0; i < FT_BN; ++i) if (kv0 + i >= p.n_kv) s[i] = -INFINITY;
            }
            float mx = m_run;
#pragma unroll
            for (int i = 0; i < FT_BN; ++i) mx = fmaxf(mx, s[i]);
            const float m_use = mx == -INFINITY ? 0.0f : mx;           // a row with nothing visible yet
            const float alpha = exp2f(m_run - m_use);                  // (exp2f(-inf) = 0 for the first tile)
            float sum = 0.0f;
            uint32_t pk[FT_BN / 2];
#pragma unroll
            for (int i = 0; i < FT_BN / 2; ++i) {
                const float a = exp2f(s[2 * i] - m_use), c2 = exp2f(s[2 * i + 1] - m_use);
                const __half2 h = __floats2half2_rn(a, c2);
                const float2 back = __half22float2(h);                // the sum of what the tensor core will see
                sum += back.x + back.y;
                pk[i] = *(const uint32_t *) &h;
            }
            l_run = l_run * alpha + sum;
            m_run = mx;
            // P(j) may be written once P(j-2) has been consumed and O rescaled once PV(j-1) is complete: both follow from
            // the completion of PV(j-1)
            if (j > 0) {
                if (!mbar_wait_or_abort(smem_u32(&o_done), (uint32_t) (j - 1) & 1, &abort_flag)) { ok = false; break; }
                tc_fence_after();
                if (__any_sync(0xffffffffu, alpha != 1.0f)) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        uint32_t v[32];
                        tmem_ld32(lane_addr + COL_O + (uint32_t) (c * 32), v);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
                        tmem_st32(lane_addr + COL_O + (uint32_t) (c * 32), v);
                    }
                }
            }
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t v[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = pk[c * 32 + i];
                tmem_st32(lane_addr + COL_P + (uint32_t) (b * 64 + c * 32), v);
            }
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_full[b]);
            ++j;
        }
        if (!ok && lane == 0) { atomicExch(p.status, ERR_MBAR_TIMEOUT); abort_flag = 1; }
        // ------------------------------ output ------------------------------
        if (ok && j > 0 && !mbar_wait_or_abort(smem_u32(&o_done), (uint32_t) (j - 1) & 1, &abort_flag)) {
            ok = false;
            if (lane == 0) { atomicExch(p.status, ERR_MBAR_TIMEOUT); abort_flag = 1; }
        }
        if (ok) {
            tc_fence_after();
            const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
            float * out = p.dst + ((int64_t) (q0 + r) * p.n_head + head) * FT_D;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t v[32];
                if (j > 0) { tmem_ld32(lane_addr + COL_O + (uint32_t) (c * 32), v); tmem_ld_wait(); }
                if (row_ok) {
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        *(float4 *) (out + c * 32 + i * 4) = j > 0 ? make_float4(__uint_as_float(v[4 * i]) * inv, __uint_as_float(v[4 * i + 1]) * inv,
                                                                               __uint_as_float(v[4 * i + 2]) * inv, __uint_as_float(v[4 * i + 3]) * inv)
                                                                   : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                }
            }
        }
    } else if (warp == 4) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc_s = umma_idesc_f16(FT_BM, FT_BN), idesc_o = umma_idesc_f16_bmn(FT_BM, FT_D), idesc_ot = umma_idesc_f16(FT_BM, FT_D);
            bool ok = mbar_wait_or_abort(smem_u32(&q_full), 0, &abort_flag);
            // S(j) = Q K(j)^T over the head size: 8 x (128 x 128 x 16); the two 64-value halves are separate swizzle atoms
            auto issue_s = [&](int j) -> bool {
                const int b = j & 1;
                if (!mbar_wait_or_abort(smem_u32(&k_full[b]), (uint32_t) (j >> 1) & 1, &abort_flag)) return false;
                tc_fence_after();
                const uint32_t qa = smem_u32(q_s), ka = smem_u32(k_s + b * FT_TILE_BYTES);
#pragma unroll
                for (int kk = 0; kk < FT_D / 16; ++kk) {
                    const uint32_t off = (uint32_t) ((kk >> 2) * (FT_BM * 128) + (kk & 3) * 32);
                    umma_f16(tmem + COL_S + (uint32_t) (b * 128), umma_smem_desc(qa + off), umma_smem_desc(ka + off), idesc_s, kk != 0);
                }
                umma_commit(&k_empty[b]);
                umma_commit(&s_full[b]);
                return true;
            };
            // which tiles are processed is the same list for every role
            int n_proc = 0;
            for (int kt = 0; kt < n_kt; ++kt) if (ft_tile_class(p, qt, kt) != 1) ++n_proc;
            if (ok && n_proc > 0) ok = issue_s(0);
            for (int j = 0; j < n_proc && ok; ++j) {
                const int b = j & 1;
                if (j + 1 < n_proc && !issue_s(j + 1)) { ok = false; break; }
                if (!mbar_wait_or_abort(smem_u32(&p_full[b]), (uint32_t) (j >> 1) & 1, &abort_flag)) { ok = false; break; }
                if (!mbar_wait_or_abort(smem_u32(&v_full[b]), (uint32_t) (j >> 1) & 1, &abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t va = smem_u32(v_s + b * FT_TILE_BYTES);
                if (p.v_t) {
                    // V^T tile [d][64 keys] x 2: K-major like the K tile (16 keys = 32 bytes inside the swizzle atom)
#pragma unroll
                    for (int kk = 0; kk < FT_BN / 16; ++kk)
                        umma_f16_ts(tmem + COL_O, tmem + COL_P + (uint32_t) (b * 64 + kk * 8), umma_smem_desc(va + (kk >> 2) * (FT_D * 128) + (kk & 3) * 32), idesc_ot, (j | kk) != 0);
                } else {
#pragma unroll
                    for (int kk = 0; kk < FT_BN / 16; ++kk)           // 16 keys: 8 columns of P, 16 rows (2048 bytes) of V
                        umma_f16_ts(tmem + COL_O, tmem + COL_P + (uint32_t) (b * 64 + kk * 8), umma_smem_desc_mn(va + kk * 2048, FT_BN * 128), idesc_o, (j | kk) != 0);
                }
                umma_commit(&v_empty[b]);
                umma_commit(&o_done);
            }
            if (!ok) { atomicExch(p.status, ERR_MBAR_TIMEOUT); abort_flag = 1; }
        }
        __syncwarp();
    } else {
        // ------------------------------ loader ------------------------------
        if (lane == 0) {
            bool ok = true;
            int j = 0;
            for (int kt = 0; kt < n_kt && ok; ++kt) {
                if (ft_tile_class(p, qt, kt) == 1) continue;
                const int b = j & 1;
                if (j >= 2 && !mbar_wait_or_abort(smem_u32(&k_empty[b]), (uint32_t) ((j >> 1) - 1) & 1, &abort_flag)) { ok = false; break; }
                mbar_arrive_expect_tx(&k_full[b], FT_TILE_BYTES);
                tma_load_3d(k_s + b * FT_TILE_BYTES, &kmap, 0, kt * FT_BN, head_kv, &k_full[b]);
                tma_load_3d(k_s + b * FT_TILE_BYTES + FT_BN * 128, &kmap, 64, kt * FT_BN, head_kv, &k_full[b]);
                if (j >= 2 && !mbar_wait_or_abort(smem_u32(&v_empty[b]), (uint32_t) ((j >> 1) - 1) & 1, &abort_flag)) { ok = false; break; }
                mbar_arrive_expect_tx(&v_full[b], FT_TILE_BYTES);
                if (p.v_t) {                                           // boxes of 64 keys x 128 rows of V^T
                    tma_load_3d(v_s + b * FT_TILE_BYTES, &vmap, kt * FT_BN, 0, head_kv, &v_full[b]);
                    tma_load_3d(v_s + b * FT_TILE_BYTES + FT_D * 128, &vmap, kt * FT_BN + 64, 0, head_kv, &v_full[b]);
                } else {
                    tma_load_3d(v_s + b * FT_TILE_BYTES, &vmap, 0, kt * FT_BN, head_kv, &v_full[b]);
                    tma_load_3d(v_s + b * FT_TILE_BYTES + FT_BN * 128, &vmap, 64, kt * FT_BN, head_kv, &v_full[b]);
                }
                ++j;
            }
            if (!ok) { atomicExch(p.status, ERR_MBAR_TIMEOUT); abort_flag = 1; }
            // when the kernel gives up, the last copies may still be in flight: wait (bounded) for them before the CTA's
            // shared memory is released; in a normal run the MMA thread has waited for every tile
            if (!ok || *(volatile int *) &abort_flag) {
                for (int jj = max(0, j - 2); jj < j; ++jj) {
                    mbar_wait(&k_full[jj & 1], (uint32_t) (jj >> 1) & 1, 1 << 16);
                    mbar_wait(&v_full[jj & 1], (uint32_t) (jj >> 1) & 1, 1 << 16);
                }
            }
        }
        __syncwarp();
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 4) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

bool fattn_tc_applicable(const TensorD & q, const TensorD & k, const TensorD & v, const TensorD * mask, const FattnParams & fp) {
    const bool v_t = v.nb[0] != 2;                  // transposed V: keys contiguous, nb[0] bytes between head-dim rows
    if (q.ne[0] != FT_D || v.ne[0] != FT_D || q.ne[1] < (v_t ? 9 : 64) || q.ne[3] != 1 || k.ne[3] != 1 || v.ne[3] != 1) return false;
    if (q.type != T_F32 || k.type != T_F16 || v.type != T_F16 || fp.max_bias != 0.0f || fp.logit_softcap != 0.0f) return false;
    if (k.ne[2] != v.ne[2] || k.ne[2] == 0 || q.ne[2] % k.ne[2] != 0 || k.ne[1] != v.ne[1]) return false;
    auto al16 = [](const TensorD & t) { return ((uintptr_t) t.data & 15) == 0 && (t.nb[1] & 15) == 0 && (t.nb[2] & 15) == 0; };
    if (!al16(k) || !al16(q) || k.nb[0] != 2 || q.nb[0] != 4) return false;
    if (!v_t) { if (!al16(v)) return false; }
    else if (v.nb[1] != 2 || ((uintptr_t) v.data & 15) || (v.nb[0] & 15) || (v.nb[2] & 15)) return false;
    if (mask && (mask->type != T_F16 || ((uintptr_t) mask->data & 15) || (mask->nb[1] & 15) || mask->ne[2] != 1 || mask->ne[3] != 1)) return false;
    return true;
}

// `workspace`: fattn_mma_workspace_bytes() of scratch for the mask-tile flags
cudaError_t launch_fattn_tc(const TensorD & q, const TensorD & k, const TensorD & v, const TensorD * mask, const TensorD & dst,
                            const FattnParams & fp, void * workspace, const LaunchCtx & c) {
    encode_tiled_fn enc = get_encode_tiled();
    if (!enc) return cudaErrorNotSupported;
    FtParams p = {};
    p.q = (const char *) q.data; p.q_nb1 = q.nb[1]; p.q_nb2 = q.nb[2];
    p.mask = mask ? (const char *) mask->data : nullptr; p.m_nb1 = mask ? mask->nb[1] : 0;
    p.dst = (float *) dst.data;
    p.n_q = (int) q.ne[1]; p.n_kv = (int) k.ne[1]; p.n_head = (int) q.ne[2]; p.gqa = (int) (q.ne[2] / k.ne[2]);
    p.scale_log2 = fp.scale * 1.4426950408889634f;
    p.status = c.status;
    p.v_t = v.nb[0] != 2 ? 1 : 0;
    if (mask) {
        const int kt = (p.n_kv + 63) / 64;                        // flags: one byte per 64 x 64 tile of the mask
        p.flags = (const uint8_t *) workspace; p.flags_stride = kt;
        cudaError_t e = launch_fattn_mask_flags(p.mask, p.m_nb1, p.n_q, p.n_kv, (uint8_t *) workspace, kt, c);
        if (e != cudaSuccess) return e;
    }
    // K and V as [d][key][kv head] F16 tensors: boxes of 64 values x 128 keys of one head, 128-byte swizzle, zero fill
    CUtensorMap maps[2];
    const TensorD * kv[2] = {&k, &v};
    for (int i = 0; i < 2; ++i) {
        const bool tr = i == 1 && p.v_t;            // V^T: [key][d][kv head], boxes of 64 keys x 128 rows
        const cuuint64_t gdim[3] = {(cuuint64_t) (tr ? kv[i]->ne[1] : FT_D), (cuuint64_t) (tr ? FT_D : kv[i]->ne[1]), (cuuint64_t) kv[i]->ne[2]};
        const cuuint64_t gstr[2] = {(cuuint64_t) (tr ? kv[i]->nb[0] : kv[i]->nb[1]), (cuuint64_t) kv[i]->nb[2]};
        const cuuint32_t box[3] = {64, FT_BN, 1}, estr[3] = {1, 1, 1};
        if (enc(&maps[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, kv[i]->data, gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    static unsigned attr_mask = 0;
    if (!(attr_mask & (1u << c.device))) {
        cudaError_t e = cudaFuncSetAttribute(fattn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FT_SMEM);
        if (e != cudaSuccess) return e;
        attr_mask |= 1u << c.device;
    }
    dim3 grid((unsigned) ((p.n_q + FT_BM - 1) / FT_BM), (unsigned) p.n_head);
    (void) (launch_err = launch_k(c.use_pdl, c.stream, fattn_tc_kernel, grid, dim3(FT_THREADS), (size_t) FT_SMEM, p, maps[0], maps[1]));
    return cudaGetLastError();
}

}  // namespace b200
