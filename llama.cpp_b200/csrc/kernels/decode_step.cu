// Persistent decode step: a run of Llama layers for ONE token in a single cooperative launch.
//
// The node-per-launch walk of a decode graph (the reference's ggml_backend_cuda_graph_compute,
// ggml/src/ggml-cuda/ggml-cuda.cu:2691-2765, and this backend's own per-node path) spends most of a
// token in launch ramps and tails: each of the ~300 kernels streams a few MB and the next one cannot
// start fetching until it is scheduled.  Here one CTA per SM stays resident for the whole token and
// walks a list of phases prepared by the host (csrc/host/decode_plan.cpp):
//
//   mat-vec phase   every CTA first builds the int8 activation blocks of the shared input in its own
//                   shared memory -- directly from x, or from rms_norm(x [+ residual]) * w -- then each
//                   warp computes whole weight rows.  Results are stored, or consumed in registers:
//                   adjacent row pairs of wq/wk are rotated (ROPE) and K/V rows go straight into the
//                   F16 cache; row r of gate and row r of up are computed by the same warp, which
//                   stores silu(gate) * up.
//   attention phase (KV head, KV slice) work items as in fattn_dec.cu: all query heads of a KV head
//                   share the K/V reads; the last CTA of a head merges the slices in a fixed order.
//
// Phases are separated by grid-wide barriers (bounded spins; a give-up sets the status word and the
// kernel drains and returns).  Weight streaming does not stop at a barrier: every warp owns a ring of
// DS_NSLOT shared-memory slots filled by cp.async.bulk (plain, non-multicast, local memory) and keeps
// requesting the units of its FUTURE rows -- across phase boundaries, because the schedule of a warp
// is a pure function of the phase list -- while it waits for activations.  HBM therefore sees one
// nearly continuous stream of weight reads per token instead of ~150 separate ramps.
//
// Arithmetic of the dot products: vec_dot_q4_K_q8_1 / q5_K / q6_K (ggml/src/ggml-cuda/vecdotq.cuh:357-496,
// 671-787) restated for these layouts, identical to mmvq_k.cu / mmvq_q6k.cu; activation blocks as
// quantize_act128_kernel (mmvq.cu); rms_norm, rope and silu as in glue.cu; attention as fattn_dec.cu.
#include "common.cuh"
#include "kernels.h"
#include <math.h>
#include <string.h>
#include <vector>

namespace b200 {

static constexpr int DS_WARPS = 16, DS_THREADS = DS_WARPS * 32;
static constexpr int DS_NSLOT = 2, DS_SLOT = 4608;               // per-warp ring: slots of 32 Q4_K super-blocks (one being computed on, the rest in flight)
static constexpr int DS_ACT_STRIDE = 336;                         // shared-memory bytes per 256 activation values: 256 int8, 8 x {d, s}, 16 pad
static constexpr int DS_MAX_K = 28672;
static constexpr int DS_BS16_OFF = DS_MAX_K / 256 * DS_ACT_STRIDE;    // int16 sums of 16 activations each (the -32 of Q6_K weights folds into them)
static constexpr int DS_ACT_BYTES = (DS_BS16_OFF + DS_MAX_K / 8 + 255) / 256 * 256;   // activation blocks of one column / attention scratch
static constexpr int DS_PSTRIDE = 132;                            // floats per (head, slice, row) attention partial: O[128], max, sum, pad
static constexpr int DS_SPIN_LIMIT = 1 << 22;

// The rows of all mat-vec phases of a launch as a flat list of parts: one part per weight matrix of a phase (the
// gate/up pair is one part).  A group is the work item of a warp: one row, or two rows (adjacent rows of a matrix, or
// row r of gate and row r of up).  Group g of a phase belongs to warp g mod (warps of the grid).
struct alignas(16) DsPart {
    uint64_t W0, W1;            // the matrix; W1: the partner matrix of a gate/up pair
    uint32_t nb1;               // row stride in bytes
    uint32_t g_begin, g_end;    // groups of this part, in the numbering of its phase
    uint32_t first_mod;         // g_begin mod (warps of the grid): a warp finds its first group without a division
    uint16_t seg_b, last_b;     // bytes of a full / of the last segment of a row
    uint8_t  type, nseg, seg_blk, last_blk;   // segments per row, super-blocks per full / last segment
    uint8_t  mode;              // bit 0: gate/up pair; bit 1: two rows per group; bit 2: both rows travel in one ring slot
    uint8_t  mat;               // index of the matrix within its phase
    uint16_t phase;             // index of the mat-vec phase within the launch
};
static_assert(sizeof(DsPart) == 48, "part size");

// shared-memory layout
static constexpr int DS_OFF_RING = DS_ACT_BYTES;
static constexpr int DS_OFF_BAR  = DS_OFF_RING + DS_WARPS * DS_NSLOT * DS_SLOT;
static constexpr int DS_OFF_OP   = DS_OFF_BAR + DS_WARPS * DS_NSLOT * 8;
static constexpr int DS_OP_BYTES = (int) sizeof(DsOp);
static_assert(sizeof(DsOp) % 16 == 0, "phase parameters are copied in 16-byte pieces");
static constexpr int DS_OFF_MISC = DS_OFF_OP + 2 * DS_OP_BYTES;     // two copies: the next phase's parameters are fetched during the current one
struct DsMisc {
    float red[32];
    float2 rope_cs[64];
    __half * kc; __half * vc;
    volatile int dead;
    unsigned ticket;
};
static constexpr int DS_OFF_DESC = DS_OFF_MISC + (int) ((sizeof(DsMisc) + 15) / 16 * 16);
static constexpr int DS_SMEM_LIMIT = 232448;                      // 227 KB opt-in maximum per CTA

struct DsParams {
    const DsOp * ops; int n_ops;
    const DsPart * parts; int n_parts;
    unsigned * sync;            // [0] barrier arrivals, [1] exit arrivals, [2] give-up flag
    int * status;
    unsigned long long * timing;   // optional: per phase {start, input stage done, rows done, barrier passed} of CTA 0, in ns
};

__device__ __forceinline__ unsigned long long ds_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ unsigned ds_ld_acquire(const unsigned * p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void ds_red_release(unsigned * p, unsigned v) {
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" :: "l"(p), "r"(v) : "memory");
}
// mbarrier / bulk-copy operations on shared-memory addresses that were converted once
__device__ __forceinline__ bool ds_try_wait(uint32_t bar_s, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar_s), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ void ds_expect_tx(uint32_t bar_s, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar_s), "r"(bytes) : "memory");
}
__device__ __forceinline__ void ds_bulk(uint32_t dst_s, const void * src, uint32_t bytes, uint32_t bar_s) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :: "r"(dst_s), "l"(src), "r"(bytes), "r"(bar_s) : "memory");
}
__device__ __forceinline__ void ds_fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void ds_give_up(const DsParams & p, DsMisc * misc, int code) {
    misc->dead = 1;
    atomicExch(&p.sync[2], 1u);
    atomicCAS(p.status, ERR_NONE, code);
}

// Grid-wide barrier: arrival number `target` of the monotonically increasing counter releases the phase.
__device__ __forceinline__ void ds_grid_barrier(const DsParams & p, DsMisc * misc, unsigned target) {
    __syncthreads();
    if (threadIdx.x == 0) {
        // The release is cumulative: what the other threads of the CTA wrote before the bar.sync above happens before it,
        // and the acquiring load below orders the next phase's reads after the other CTAs' releases.  No separate fences.
        ds_red_release(&p.sync[0], 1u);
        if (!misc->dead) {
            int spins = 0;
            while (ds_ld_acquire(&p.sync[0]) < target) {
                if (++spins >= DS_SPIN_LIMIT) { ds_give_up(p, misc, ERR_MBAR_TIMEOUT); break; }
                if ((spins & 255) == 0 && ds_ld_acquire(&p.sync[2])) { misc->dead = 1; break; }
            }
        }
    }
    __syncthreads();
}

__device__ __forceinline__ int ds_blk_bytes(int type) { return (type == T_Q4_K || type == T_Q4_0) ? 144 : (type == T_Q5_K ? 176 : (type == T_Q8_0 ? 272 : 210)); }

// ---------------------------------------------------------------------------
// dot products of one ring slot (a run of super-blocks of one weight row) with the activation blocks
// ---------------------------------------------------------------------------
__device__ __forceinline__ int ds_dp4a_us(uint32_t a, int b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// Q4_K / Q5_K: one lane per super-block (256 weights).  The 12 scale bytes are decoded once per block, every
// load is 128 bits wide, and with a lane stride of 144 / 176 bytes (weights) and DS_ACT_STRIDE (activations) the
// eight lanes of a quarter warp hit eight different bank groups.  `ab` is the activation block of the same 256 values.
template <int T>
__device__ __forceinline__ float ds_dot_blk(const uint8_t * blk, const uint8_t * ab) {
    constexpr int QS_OFF = (T == T_Q4_K) ? 16 : 48;
    const uint4 hd = *(const uint4 *) blk;
    const float2 dm = __half22float2(*(const __half2 *) &hd.x);                 // {d, dmin}
    // 6-bit scales and mins of the 8 sub-blocks as bytes (get_scale_min_k4, ggml/src/ggml-quants.c:631-638)
    const uint32_t sc_lo = hd.y & 0x3f3f3f3fu, mn_lo = hd.z & 0x3f3f3f3fu;
    const uint32_t sc_hi = (hd.w & 0x0f0f0f0fu) | ((hd.y >> 2) & 0x30303030u);
    const uint32_t mn_hi = ((hd.w >> 4) & 0x0f0f0f0fu) | ((hd.z >> 2) & 0x30303030u);
    uint32_t hb[8];
    if (T == T_Q5_K) {
        const uint4 h0 = *(const uint4 *) (blk + 16), h1 = *(const uint4 *) (blk + 32);
        hb[0] = h0.x; hb[1] = h0.y; hb[2] = h0.z; hb[3] = h0.w; hb[4] = h1.x; hb[5] = h1.y; hb[6] = h1.z; hb[7] = h1.w;
    }
    float accE = 0.0f, accO = 0.0f, accM = 0.0f;
#pragma unroll
    for (int r = 0; r < 4; ++r) {                      // 64 weights: low nibbles = sub-block 2r, high nibbles = 2r+1
        const uint4 q0 = *(const uint4 *) (blk + QS_OFF + 32 * r), q1 = *(const uint4 *) (blk + QS_OFF + 32 * r + 16);
        const uint4 xa = *(const uint4 *) (ab + 64 * r), xb = *(const uint4 *) (ab + 64 * r + 16);
        const uint4 xc = *(const uint4 *) (ab + 64 * r + 32), xd = *(const uint4 *) (ab + 64 * r + 48);
        const float4 ds = *(const float4 *) (ab + 256 + 16 * r);              // {d, s} of sub-blocks 2r, 2r+1
        const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
        uint32_t lo[8], hi[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) { lo[i] = w[i] & 0x0F0F0F0Fu; hi[i] = (T == T_Q5_K) ? (w[i] >> 4) & 0x0F0F0F0Fu : w[i] & 0xF0F0F0F0u; }
        if (T == T_Q5_K) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const uint32_t t = hb[i] >> (2 * r);
                lo[i] |= (t << 4) & 0x10101010u;
                hi[i] |= (t << 3) & 0x10101010u;
            }
        }
        // four independent chains of four dependent dp4a each
        int t0 = ds_dp4a_us(lo[0], (int) xa.x, 0), u0 = ds_dp4a_us(lo[4], (int) xb.x, 0);
        int t1 = ds_dp4a_us(hi[0], (int) xc.x, 0), u1 = ds_dp4a_us(hi[4], (int) xd.x, 0);
        t0 = ds_dp4a_us(lo[1], (int) xa.y, t0); u0 = ds_dp4a_us(lo[5], (int) xb.y, u0);
        t1 = ds_dp4a_us(hi[1], (int) xc.y, t1); u1 = ds_dp4a_us(hi[5], (int) xd.y, u1);
        t0 = ds_dp4a_us(lo[2], (int) xa.z, t0); u0 = ds_dp4a_us(lo[6], (int) xb.z, u0);
        t1 = ds_dp4a_us(hi[2], (int) xc.z, t1); u1 = ds_dp4a_us(hi[6], (int) xd.z, u1);
        t0 = ds_dp4a_us(lo[3], (int) xa.w, t0); u0 = ds_dp4a_us(lo[7], (int) xb.w, u0);
        t1 = ds_dp4a_us(hi[3], (int) xc.w, t1); u1 = ds_dp4a_us(hi[7], (int) xd.w, u1);
        t0 += u0; t1 += u1;
        const uint32_t scw = (r < 2 ? sc_lo : sc_hi) >> (16 * (r & 1)), mnw = (r < 2 ? mn_lo : mn_hi) >> (16 * (r & 1));
        // |sc * t| <= 63 * 32 * 240 * 127 < 2^26: exact in int32 (Q4_K keeps the high nibbles in place, value * 16)
        accE += ds.x * (float) ((int) (scw & 0xff) * t0);
        accO += ds.z * (float) ((int) ((scw >> 8) & 0xff) * t1);
        accM += ds.y * (float) (mnw & 0xff) + ds.w * (float) ((mnw >> 8) & 0xff);
    }
    return dm.x * (accE + (T == T_Q5_K ? 1.0f : 0.0625f) * accO) - dm.y * accM;
}

// Q4_0 / Q8_0: eight consecutive 32-value blocks (256 values, 144 / 272 bytes: 16-byte multiples) are one lane's unit, like
// a super-block of the K types.  Inside, the 18- / 34-byte blocks sit at 2-byte aligned offsets; words are rebuilt with
// funnel shifts whose amounts are compile-time constants once the loop over the blocks is unrolled.
// x = d * (q - 8): dot = d * (d_a * sum(q * a) - 8 * d_a * sum(a)), the activation block carries both factors per 32 values.
__device__ __forceinline__ float ds_dot_q4_0(const uint8_t * grp, const uint8_t * ab) {
    uint32_t w[36];
#pragma unroll
    for (int i = 0; i < 9; ++i) { const uint4 v = *(const uint4 *) (grp + 16 * i); w[4 * i] = v.x; w[4 * i + 1] = v.y; w[4 * i + 2] = v.z; w[4 * i + 3] = v.w; }
    float acc = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int o = 18 * j, wi = o >> 2, sh = (o & 3) * 8;            // sh is 0 (even j) or 16 (odd j)
        const uint32_t dbits = (w[wi] >> sh) & 0xffffu;
        uint32_t q[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) q[k] = sh == 0 ? __funnelshift_r(w[wi + k], w[wi + k + 1], 16) : w[wi + 1 + k];
        const uint4 xa = *(const uint4 *) (ab + 32 * j), xb = *(const uint4 *) (ab + 32 * j + 16);      // values 0..15 and 16..31 of the block
        const float2 ds = *(const float2 *) (ab + 256 + 8 * j);
        const int xl[4] = {(int) xa.x, (int) xa.y, (int) xa.z, (int) xa.w}, xh[4] = {(int) xb.x, (int) xb.y, (int) xb.z, (int) xb.w};
        int s0 = 0, s1 = 0;
#pragma unroll
        for (int k = 0; k < 4; ++k) { s0 = ds_dp4a_us(q[k] & 0x0F0F0F0Fu, xl[k], s0); s1 = ds_dp4a_us((q[k] >> 4) & 0x0F0F0F0Fu, xh[k], s1); }
        acc += __half2float(__ushort_as_half((unsigned short) dbits)) * (ds.x * (float) (s0 + s1) - 8.0f * ds.y);
    }
    return acc;
}
__device__ __forceinline__ float ds_dot_q8_0(const uint8_t * grp, const uint8_t * ab) {
    float acc = 0.0f;
#pragma unroll
    for (int h = 0; h < 2; ++h) {                      // blocks 4h .. 4h+3 lie inside bytes [128 h, 128 h + 144): nine 128-bit loads
        uint32_t w[36];
#pragma unroll
        for (int i = 0; i < 9; ++i) { const uint4 v = *(const uint4 *) (grp + 128 * h + 16 * i); w[4 * i] = v.x; w[4 * i + 1] = v.y; w[4 * i + 2] = v.z; w[4 * i + 3] = v.w; }
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
            const int j = 4 * h + jj, o = 34 * j - 128 * h, wi = o >> 2, sh = (o & 3) * 8;      // sh is 0 or 16
            const uint32_t dbits = (w[wi] >> sh) & 0xffffu;
            const uint4 xa = *(const uint4 *) (ab + 32 * j), xb = *(const uint4 *) (ab + 32 * j + 16);
            const float2 ds = *(const float2 *) (ab + 256 + 8 * j);
            const int x[8] = {(int) xa.x, (int) xa.y, (int) xa.z, (int) xa.w, (int) xb.x, (int) xb.y, (int) xb.z, (int) xb.w};
            int s0 = 0, s1 = 0;
#pragma unroll
            for (int k = 0; k < 8; k += 2) {
                const uint32_t q0 = sh == 0 ? __funnelshift_r(w[wi + k], w[wi + k + 1], 16) : w[wi + k + 1];
                const uint32_t q1 = sh == 0 ? __funnelshift_r(w[wi + k + 1], w[wi + k + 2], 16) : w[wi + k + 2];
                s0 = __dp4a((int) q0, x[k], s0); s1 = __dp4a((int) q1, x[k + 1], s1);
            }
            acc += __half2float(__ushort_as_half((unsigned short) dbits)) * ds.x * (float) (s0 + s1);
        }
    }
    return acc;
}

// NW consecutive 32-bit words at a 2-byte aligned shared-memory address
template <int NW>
__device__ __forceinline__ void ds_lds_run(const uint8_t * p, uint32_t (&out)[NW]) {
    const uint32_t * base = (const uint32_t *) ((uintptr_t) p & ~(uintptr_t) 3);
    const uint32_t sh = ((uint32_t) (uintptr_t) p & 3u) * 8u;
    uint32_t prev = base[0];
#pragma unroll
    for (int i = 0; i < NW; ++i) {
        const uint32_t next = base[i + 1];
        out[i] = __funnelshift_r(prev, next, sh);
        prev = next;
    }
}

// Q6_K: lane l owns half (l & 1) of super-block l >> 1 (a slot holds at most 16 super-blocks).  The 6-bit values
// stay unsigned (0..63): sum (q - 32) x = sum q x - 32 sum x, and the sums of x over the 16-value sub-blocks come
// ready-made from the input stage (bs16), so no per-byte subtraction is needed.
__device__ __forceinline__ float ds_dot_q6k(const uint8_t * slot, int nblk, const uint8_t * acts, const uint8_t * bs16, int lane) {
    const int b = lane >> 1, n128 = lane & 1;
    float acc = 0.0f;
    if (b < nblk) {
        const uint8_t * blk = slot + b * 210;
        uint32_t ql[16], qh[8], scw[2];
        ds_lds_run<16>(blk + n128 * 64, ql);
        ds_lds_run<8>(blk + 128 + n128 * 32, qh);
        ds_lds_run<2>(blk + 192 + n128 * 8, scw);
        const float d = h2f(*(const uint16_t *) (blk + 208));
        const uint8_t * ab = acts + b * DS_ACT_STRIDE + n128 * 128;       // 128 int8 of this half; its {d, s} pairs follow the block's 256 int8
        const uint8_t * dsb = acts + b * DS_ACT_STRIDE + 256 + n128 * 32;
        const uint4 bsv = *(const uint4 *) (bs16 + b * 32 + n128 * 16);   // eight int16 sums
        const uint32_t bsw[4] = {bsv.x, bsv.y, bsv.z, bsv.w};
#pragma unroll
        for (int t = 0; t < 4; ++t) {                                     // 32 values: words 0..3 sub-block 2t, words 4..7 sub-block 2t+1
            uint32_t q[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const uint32_t L = (t & 1) ? ql[8 + i] : ql[i];
                const uint32_t nib = (t & 2) ? (L >> 4) & 0x0F0F0F0Fu : L & 0x0F0F0F0Fu;
                const uint32_t hb = t == 0 ? (qh[i] << 4) : t == 1 ? (qh[i] << 2) : t == 2 ? qh[i] : (qh[i] >> 2);
                q[i] = nib | (hb & 0x30303030u);
            }
            const int sc_lo = (int) (int8_t) ((scw[(2 * t) >> 2] >> (8 * ((2 * t) & 3))) & 0xff);
            const int sc_hi = (int) (int8_t) ((scw[(2 * t + 1) >> 2] >> (8 * ((2 * t + 1) & 3))) & 0xff);
            const uint4 x0 = *(const uint4 *) (ab + t * 32);
            const uint4 x1 = *(const uint4 *) (ab + t * 32 + 16);
            const float dx = *(const float *) (dsb + t * 8);
            int s0 = ds_dp4a_us(q[0], (int) x0.x, 0); s0 = ds_dp4a_us(q[1], (int) x0.y, s0);
            s0 = ds_dp4a_us(q[2], (int) x0.z, s0);    s0 = ds_dp4a_us(q[3], (int) x0.w, s0);
            int s1 = ds_dp4a_us(q[4], (int) x1.x, 0); s1 = ds_dp4a_us(q[5], (int) x1.y, s1);
            s1 = ds_dp4a_us(q[6], (int) x1.z, s1);    s1 = ds_dp4a_us(q[7], (int) x1.w, s1);
            const int b0 = (int) (int16_t) (bsw[t] & 0xffffu), b1 = (int) bsw[t] >> 16;
            acc += dx * (float) (sc_lo * (s0 - 32 * b0) + sc_hi * (s1 - 32 * b1));
        }
        acc *= d;
    }
    return acc;
}

// ---------------------------------------------------------------------------
// input stage of a mat-vec phase: x (+ residual) [-> rms_norm * w] -> int8 activation blocks in shared memory
// ---------------------------------------------------------------------------
__device__ __forceinline__ float ds_block_sum(float v, float * red) {
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) red[w] = v;
    __syncthreads();
    float r = lane < DS_WARPS ? red[lane] : 0.0f;
    return warp_sum(r);
}

// Input stage: the shared input vector of a mat-vec phase becomes int8 activation blocks in shared memory.  A thread
// handles four consecutive values at a time (one 128-bit load per operand), eight neighbouring threads form a
// 32-value quantization group.  Quad q of a pass belongs to thread q mod DS_THREADS.
__device__ __forceinline__ float4 ds_ld4(const float * p) { return __ldcg((const float4 *) p); }

// quantizes the quad y (values i .. i+3) and stores it; all 32 lanes of a warp call this together
__device__ __forceinline__ void ds_quant_quad(const float4 y, int i, uint8_t * acts) {
    const int tid = threadIdx.x;
    float amax = fmaxf(fmaxf(fabsf(y.x), fabsf(y.y)), fmaxf(fabsf(y.z), fabsf(y.w)));
#pragma unroll
    for (int s = 4; s > 0; s >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, s));
    const float d = amax * (1.0f / 127.0f), id = amax > 0.0f ? __fdividef(127.0f, amax) : 0.0f;
    const int q0 = __float2int_rn(y.x * id), q1 = __float2int_rn(y.y * id), q2 = __float2int_rn(y.z * id), q3 = __float2int_rn(y.w * id);
    int qsum = q0 + q1 + q2 + q3;
    qsum += __shfl_xor_sync(0xffffffffu, qsum, 1);
    qsum += __shfl_xor_sync(0xffffffffu, qsum, 2);                // 16 values: what a Q6_K sub-block multiplies
    if ((tid & 3) == 0) *(int16_t *) (acts + DS_BS16_OFF + (i >> 4) * 2) = (int16_t) qsum;
    qsum += __shfl_xor_sync(0xffffffffu, qsum, 4);
    uint8_t * blk = acts + (i >> 8) * DS_ACT_STRIDE;
    *(uint32_t *) (blk + (i & 255)) = (uint32_t) (q0 & 0xff) | ((uint32_t) (q1 & 0xff) << 8) | ((uint32_t) (q2 & 0xff) << 16) | ((uint32_t) (q3 & 0xff) << 24);
    if ((tid & 7) == 0) *(float2 *) (blk + 256 + ((i & 255) >> 5) * 8) = make_float2(d, d * (float) qsum);
}

// x = in0 (+ in1), optionally rms-normalised and weighted.  NORM: the whole vector (K <= VQ * 4 * DS_THREADS) is
// held in registers between the sum of squares and the output, so it is read once.  Otherwise the vector is
// processed in passes of VQ quads per thread.
template <int VQ, bool NORM>
__device__ __forceinline__ void ds_input_x(const DsOp & o, uint8_t * acts, float * red) {
    const int tid = threadIdx.x, K = o.K;
    const bool writer = blockIdx.x == 0;
    const float * __restrict__ in0 = o.in0;
    const float * __restrict__ in1 = o.in1;
    const bool one_pass = K <= VQ * DS_THREADS * 4;
    float scale = 1.0f;
    if (NORM && !one_pass) {                     // longer than the registers hold: sum of squares first, second read below
        float ss = 0.0f;
#pragma unroll 1
        for (int base = 0; base < K; base += VQ * DS_THREADS * 4) {
#pragma unroll
            for (int k = 0; k < VQ; ++k) {
                const int i = base + (k * DS_THREADS + tid) * 4;
                if (i < K) {
                    float4 x = ds_ld4(in0 + i);
                    if (in1) { const float4 r = ds_ld4(in1 + i); x.x += r.x; x.y += r.y; x.z += r.z; x.w += r.w; }
                    ss += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
                }
            }
        }
        ss = ds_block_sum(ss, red);
        scale = rsqrtf(ss / (float) K + o.eps);
    }
#pragma unroll 1
    for (int base = 0; base < K; base += VQ * DS_THREADS * 4) {
        float4 xv[VQ], wv[NORM ? VQ : 1];
#pragma unroll
        for (int k = 0; k < VQ; ++k) {
            const int i = base + (k * DS_THREADS + tid) * 4;
            xv[k] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (i < K) { xv[k] = ds_ld4(in0 + i); if (NORM) wv[k] = __ldg((const float4 *) (o.norm_w + i)); }
        }
        if (in1) {
#pragma unroll
            for (int k = 0; k < VQ; ++k) {
                const int i = base + (k * DS_THREADS + tid) * 4;
                if (i < K) {
                    const float4 r = ds_ld4(in1 + i);
                    xv[k].x += r.x; xv[k].y += r.y; xv[k].z += r.z; xv[k].w += r.w;
                    if (writer && o.sum_out) *(float4 *) (o.sum_out + i) = xv[k];
                }
            }
        }
        if (NORM && one_pass) {
            float ss = 0.0f;
#pragma unroll
            for (int k = 0; k < VQ; ++k) ss += xv[k].x * xv[k].x + xv[k].y * xv[k].y + xv[k].z * xv[k].z + xv[k].w * xv[k].w;
            ss = ds_block_sum(ss, red);
            scale = rsqrtf(ss / (float) K + o.eps);
        }
#pragma unroll
        for (int k = 0; k < VQ; ++k) {
            const int i = base + (k * DS_THREADS + tid) * 4;
            if (base + (k * DS_THREADS + (tid & ~31)) * 4 < K) {          // warp-uniform: K is a multiple of 128
                float4 y = xv[k];
                if (NORM) { y.x = y.x * scale * wv[k].x; y.y = y.y * scale * wv[k].y; y.z = y.z * scale * wv[k].z; y.w = y.w * scale * wv[k].w; }
                if (writer && o.y_out) *(float4 *) (o.y_out + i) = y;
                ds_quant_quad(y, i, acts);
            }
        }
    }
}

// The input is the attention output, still in KV slices: (max, sum, unnormalised O) per (head, slice), merged here in
// slice order (what the last CTA of a head would otherwise do after a fence and a ticket).
__device__ __forceinline__ void ds_input_attn(const DsOp & o, uint8_t * acts) {
    constexpr int D = 128, MAXS = DS_MAX_MERGE_SLICES;
    const int tid = threadIdx.x, K = o.K, ns = o.in_slices, gqa = o.in_gqa;
    const bool writer = blockIdx.x == 0;
#pragma unroll 1
    for (int base = 0; base < K; base += DS_THREADS * 4) {
        const int i = base + tid * 4;
        if (base + (tid & ~31) * 4 < K) {                                  // warp-uniform
            const int h = i / D, d = i - h * D, hk = h / gqa, r = h - hk * gqa;
            const float * p0 = o.in0 + ((int64_t) hk * ns * gqa + r) * DS_PSTRIDE;
            float ms[MAXS]; float M = -INFINITY;
#pragma unroll
            for (int s = 0; s < MAXS; ++s) { ms[s] = s < ns ? __ldcg(p0 + (int64_t) s * gqa * DS_PSTRIDE + D) : -INFINITY; M = fmaxf(M, ms[s]); }
            float L = 0.0f; float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
            for (int s = 0; s < MAXS; ++s) {
                if (s < ns) {
                    const float * ps = p0 + (int64_t) s * gqa * DS_PSTRIDE;
                    const float f = (ms[s] == -INFINITY) ? 0.0f : expf(ms[s] - M);
                    const float4 v = ds_ld4(ps + d);
                    L += __ldcg(ps + D + 1) * f;
                    acc.x += v.x * f; acc.y += v.y * f; acc.z += v.z * f; acc.w += v.w * f;
                }
            }
            const float inv = 1.0f / L;
            const float4 y = make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
            if (writer && o.y_out) *(float4 *) (o.y_out + i) = y;
            ds_quant_quad(y, i, acts);
        }
    }
}

__device__ __forceinline__ void ds_input_stage(const DsOp & o, uint8_t * acts, float * red) {
    if (o.in_kind == DS_IN_NORM) ds_input_x<3, true>(o, acts, red);
    else if (o.in_kind == DS_IN_ATTN) ds_input_attn(o, acts);
    else ds_input_x<7, false>(o, acts, red);                        // 14336 values (Llama-3-8B's feed-forward width) in one pass
}

__device__ __forceinline__ void ds_rope_cs(const DsOp & o, float theta_extrap, int i0, float & c, float & s) {
    // YaRN mix of interpolated and extrapolated angles (ggml-cpu.c:9275-9306), as rope_cs in glue.cu
    const float theta_interp = o.freq_scale * theta_extrap;
    float theta = theta_interp, mscale = o.attn_factor;
    if (o.ext_factor != 0.0f) {
        const float y = ((float) (i0 / 2) - o.corr0) / fmaxf(0.001f, o.corr1 - o.corr0);
        const float ramp_mix = (1.0f - fminf(1.0f, fmaxf(0.0f, y))) * o.ext_factor;
        theta = theta_interp * (1.0f - ramp_mix) + theta_extrap * ramp_mix;
        mscale *= 1.0f + 0.1f * logf(1.0f / o.freq_scale);
    }
    c = cosf(theta) * mscale;
    s = sinf(theta) * mscale;
}

__device__ __forceinline__ void ds_prefetch_l2(const char * p, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" :: "l"(p), "r"(bytes) : "memory");
}

__device__ __forceinline__ void ds_matvec_input(const DsOp & o, uint8_t * acts, DsMisc * misc) {
    if (o.epilogue == DS_EP_ROPE_KV) {
        const int tid = threadIdx.x;
        // The attention phase that follows reads this layer's K/V rows while the weight stream keeps HBM's queues
        // full; asking for them now, two barriers ahead, puts them into L2 by then.
        if ((tid & 31) == 0 && o.pf_bytes > 0) {
            const int64_t CH = 4096, step = (int64_t) gridDim.x * DS_WARPS * CH;
            for (int64_t off = ((int64_t) (tid >> 5) * gridDim.x + blockIdx.x) * CH; off < o.pf_bytes; off += step) {
                const uint32_t n = (uint32_t) (o.pf_bytes - off < CH ? o.pf_bytes - off : CH);
                ds_prefetch_l2(o.pf_k + off, n);
                ds_prefetch_l2(o.pf_v + off, n);
            }
        }
        if (tid < o.n_dims / 2 && tid < 64) {
            const float theta_base = (float) __ldg(o.pos) * powf(o.theta_scale, (float) tid);
            const float f = o.ff ? __ldg(o.ff + tid) : 1.0f;
            float c, s;
            ds_rope_cs(o, theta_base / f, 2 * tid, c, s);
            misc->rope_cs[tid] = make_float2(c, s);
        }
        if (tid == 64) {
            misc->kc = (__half *) ((char *) o.k_cache + (o.k_off_dev ? __ldg(o.k_off_dev) : o.k_off));
            misc->vc = (__half *) ((char *) o.v_cache + (o.v_off_dev ? __ldg(o.v_off_dev) : o.v_off));
        }
    }
    ds_input_stage(o, acts, misc->red);
    __syncthreads();
}

// ---------------------------------------------------------------------------
// weight streaming: the schedule of one warp over all mat-vec phases of the launch
// ---------------------------------------------------------------------------
// A unit is what one ring slot holds: a run of super-blocks of one weight row, or (mode bit 2) both rows of a group
// back to back.  Both cursors of a warp -- the one that requests units and the one that computes on them -- walk the
// parts in the same order; everything they need of the current part sits in registers.
struct DsCursor {
    int part;                   // current part (n_parts: nothing left)
    uint32_t g, g_end;          // current group of this warp, end of the part
    int j, s;                   // row of the group, segment of the row
    const uint8_t * row;        // first row of the current group
    const uint8_t * src;        // next unit
    uint64_t g_stride;          // bytes from a group of this warp to its next one
    int64_t  pair_off;          // from the first to the second row of a group
    uint32_t seg_b, last_b; int nseg, mode;
};

// loads part `c.part` and positions the cursor on this warp's first group in it; false if the warp has none
__device__ __forceinline__ bool ds_cursor_enter(DsCursor & c, const DsPart * parts, uint32_t gw, uint32_t G) {
    const DsPart & P = parts[c.part];
    const uint4 a = *(const uint4 *) &P, b = *(const uint4 *) ((const uint8_t *) &P + 16), d = *(const uint4 *) ((const uint8_t *) &P + 32);
    const uint64_t W0 = (uint64_t) a.x | ((uint64_t) a.y << 32), W1 = (uint64_t) a.z | ((uint64_t) a.w << 32);
    const uint32_t nb1 = b.x, g_begin = b.y, first_mod = b.w;
    c.g_end = b.z;
    c.g = g_begin + (gw >= first_mod ? gw - first_mod : gw + G - first_mod);
    if (c.g >= c.g_end) return false;
    c.seg_b = d.x & 0xffffu; c.last_b = d.x >> 16;
    c.nseg = (d.y >> 8) & 0xff; c.mode = d.z & 0xff;
    const uint32_t rows_per_group = (c.mode & 3) == 2 ? 2u : 1u;           // adjacent rows of one matrix
    c.g_stride = (uint64_t) G * rows_per_group * nb1;
    c.pair_off = (c.mode & 1) ? (int64_t) (W1 - W0) : (int64_t) nb1;
    c.row = (const uint8_t *) W0 + (uint64_t) (c.g - g_begin) * rows_per_group * nb1;
    c.src = c.row; c.j = 0; c.s = 0;
    return true;
}
__device__ __forceinline__ void ds_cursor_seek(DsCursor & c, const DsPart * parts, int n_parts, uint32_t gw, uint32_t G) {
    while (c.part < n_parts && !ds_cursor_enter(c, parts, gw, G)) ++c.part;
}
// steps to the next unit of this warp
__device__ __forceinline__ void ds_cursor_advance(DsCursor & c, const DsPart * parts, int n_parts, uint32_t gw, uint32_t G) {
    if (++c.s < c.nseg) { c.src += c.seg_b; return; }
    c.s = 0;
    if ((c.mode & 6) == 2 && c.j == 0) { c.j = 1; c.src = c.row + c.pair_off; return; }
    c.j = 0;
    c.g += G;
    if (c.g < c.g_end) { c.row += c.g_stride; c.src = c.row; return; }
    ++c.part;
    ds_cursor_seek(c, parts, n_parts, gw, G);
}

// ---------------------------------------------------------------------------
// attention phase (one query token, head size 128, F16 K/V), after fattn_dec.cu
// ---------------------------------------------------------------------------
__device__ __forceinline__ void ds_attention(const DsOp & o, uint8_t * scratch, DsMisc * misc) {
    constexpr int D = 128, RT = 4, CH = 4, KU = CH / 4, DPL = 4;
    float (*qs)[D] = (float (*)[D]) scratch;                                     // [RT][D]
    float * ps_all = (float *) (scratch + RT * D * 4);                           // [DS_WARPS][CH][RT]
    float * w_m = ps_all + DS_WARPS * CH * RT;                                   // [DS_WARPS][RT]
    float * w_l = w_m + DS_WARPS * RT;
    float * w_o = w_l + DS_WARPS * RT;                                           // [DS_WARPS][RT][D]
    static_assert((RT * D + DS_WARPS * CH * RT + 2 * DS_WARPS * RT + DS_WARPS * RT * D) * 4 <= DS_ACT_BYTES, "attention scratch");
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gqa = o.n_head / o.n_head_kv;
    const int n_items = o.n_head_kv * o.n_slices;
    float * ps = ps_all + warp * CH * RT;
    const __half * mrow = (const __half *) o.mask;

#pragma unroll 1
    for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
        const int hk = item / o.n_slices, split = item - hk * o.n_slices;
        const char * kbase = o.k + (int64_t) hk * o.k_nb2;
        const char * vbase = o.v + (int64_t) hk * o.v_nb2;
        const int kv0 = split * o.kv_per_slice, kv1 = min(o.n_kv, kv0 + o.kv_per_slice);
        int per_warp = (max(kv1 - kv0, 0) + DS_WARPS - 1) / DS_WARPS;
        if (o.v_t) per_warp = (per_warp + 3) & ~3;                     // 8-byte aligned runs of keys in the transposed V rows
        const int kw0 = kv0 + warp * per_warp, kw1 = min(kv1, kw0 + per_warp);
        const int nkeys = max(kw1 - kw0, 0);
        float * part = o.partials + ((int64_t) hk * o.n_slices + split) * gqa * DS_PSTRIDE;

#pragma unroll 1
        for (int r0 = 0; r0 < gqa; r0 += RT) {
            __syncthreads();
            for (int i = threadIdx.x; i < RT * D; i += DS_THREADS) {
                const int rr = i / D, d = i % D, r = r0 + rr;
                qs[rr][d] = r < gqa ? __ldcg(o.q + (int64_t) (hk * gqa + r) * D + d) : 0.0f;
            }
            __syncthreads();

            const int sub = lane & 7, kq = lane >> 3;
            float m_run[RT], l_part[RT], oacc[RT][DPL];
#pragma unroll
            for (int rr = 0; rr < RT; ++rr) {
                m_run[rr] = -INFINITY; l_part[rr] = 0.0f;
#pragma unroll
                for (int i = 0; i < DPL; ++i) oacc[rr][i] = 0.0f;
            }
#pragma unroll 1
            for (int kb = 0; kb < nkeys; kb += CH) {
                const int nk = min(CH, nkeys - kb);
                // the K rows of this 8-lane group and this lane's part of all V rows of the chunk are requested together
                uint4 kreg[KU][2];
                float mval[KU];
                uint2 vreg[CH];
#pragma unroll
                for (int u = 0; u < KU; ++u) {
                    const int kl = kb + u * 4 + kq;
                    mval[u] = 0.0f;
                    if (kl < nkeys) {
                        const char * kr = kbase + (int64_t) (kw0 + kl) * o.k_nb1;
                        kreg[u][0] = __ldcg((const uint4 *) (kr + sub * 16));
                        kreg[u][1] = __ldcg((const uint4 *) (kr + (8 + sub) * 16));
                        if (mrow) mval[u] = o.mask_f32 ? __ldg((const float *) o.mask + kw0 + kl) : __half2float(__ldg(mrow + kw0 + kl));
                    }
                }
                if (o.v_t) {
                    // transposed cache: vreg[i] = the chunk's four keys of head-size row lane * 4 + i
#pragma unroll
                    for (int i = 0; i < DPL; ++i) vreg[i] = __ldcg((const uint2 *) (vbase + (int64_t) (lane * DPL + i) * o.v_nbd + (int64_t) (kw0 + kb) * 2));
                } else {
#pragma unroll
                    for (int t = 0; t < CH; ++t) {
                        const int kl = min(kb + t, nkeys - 1);
                        vreg[t] = __ldcg((const uint2 *) (vbase + (int64_t) (kw0 + kl) * o.v_nb1 + lane * 8));
                    }
                }
                float cmax[RT];
#pragma unroll
                for (int rr = 0; rr < RT; ++rr) cmax[rr] = -INFINITY;
#pragma unroll
                for (int u = 0; u < KU; ++u) {
                    const int kl = kb + u * 4 + kq;
                    float acc[RT] = {0.0f, 0.0f, 0.0f, 0.0f};
                    if (kl < nkeys) {
#pragma unroll
                        for (int c = 0; c < 2; ++c) {
                            const int chunk = c * 8 + sub;
                            const __half2 * kh = (const __half2 *) &kreg[u][c];
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const float2 kf = __half22float2(kh[e]);
                                const int d = chunk * 8 + 2 * e;
#pragma unroll
                                for (int rr = 0; rr < RT; ++rr) acc[rr] += kf.x * qs[rr][d] + kf.y * qs[rr][d + 1];
                            }
                        }
                    }
#pragma unroll
                    for (int rr = 0; rr < RT; ++rr) {
                        acc[rr] += __shfl_xor_sync(0xffffffffu, acc[rr], 1);
                        acc[rr] += __shfl_xor_sync(0xffffffffu, acc[rr], 2);
                        acc[rr] += __shfl_xor_sync(0xffffffffu, acc[rr], 4);
                    }
                    if (kl < nkeys) {
                        float4 sv;
                        float * s4 = (float *) &sv;
#pragma unroll
                        for (int rr = 0; rr < RT; ++rr) {
                            const float s = acc[rr] * o.scale + mval[u];
                            s4[rr] = s;
                            cmax[rr] = fmaxf(cmax[rr], s);
                        }
                        if (sub == 0) *(float4 *) (ps + (u * 4 + kq) * RT) = sv;
                    }
                }
                float fac[RT], m_new[RT];
#pragma unroll
                for (int rr = 0; rr < RT; ++rr) {
                    cmax[rr] = warp_max(cmax[rr]);
                    m_new[rr] = fmaxf(m_run[rr], cmax[rr]);
                    fac[rr] = (m_run[rr] == -INFINITY) ? 0.0f : expf(m_run[rr] - m_new[rr]);
                    m_run[rr] = m_new[rr];
                }
                __syncwarp();
                // lane t turns the scores of key t into probabilities
                {
                    float4 sv = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                    if (lane < nk) sv = *(float4 *) (ps + lane * RT);
                    float * s4 = (float *) &sv;
#pragma unroll
                    for (int rr = 0; rr < RT; ++rr) {
                        const float e = (lane >= nk || m_new[rr] == -INFINITY || s4[rr] == -INFINITY) ? 0.0f : expf(s4[rr] - m_new[rr]);
                        s4[rr] = e;
                        l_part[rr] = l_part[rr] * fac[rr] + e;
                    }
                    if (lane < nk) *(float4 *) (ps + lane * RT) = sv;
                }
                __syncwarp();
#pragma unroll
                for (int rr = 0; rr < RT; ++rr)
#pragma unroll
                    for (int i = 0; i < DPL; ++i) oacc[rr][i] *= fac[rr];
#pragma unroll
                for (int t = 0; t < CH; ++t) {
                    if (t < nk) {                                // (keys past the chunk's end are not touched: the cache row may hold anything there)
                        const float4 pv = *(const float4 *) (ps + t * RT);
                        float vf[4];
                        if (o.v_t) {
#pragma unroll
                            for (int i = 0; i < DPL; ++i) vf[i] = __half2float(((const __half *) &vreg[i])[t]);
                        } else {
                            const float2 a = __half22float2(*(const __half2 *) &vreg[t].x), b2 = __half22float2(*(const __half2 *) &vreg[t].y);
                            vf[0] = a.x; vf[1] = a.y; vf[2] = b2.x; vf[3] = b2.y;
                        }
                        const float pr[RT] = {pv.x, pv.y, pv.z, pv.w};
#pragma unroll
                        for (int rr = 0; rr < RT; ++rr)
#pragma unroll
                            for (int i = 0; i < DPL; ++i) oacc[rr][i] += pr[rr] * vf[i];
                    }
                }
                __syncwarp();
            }
            // ---- merge the warps of the CTA ----
#pragma unroll
            for (int rr = 0; rr < RT; ++rr) {
                const float l = warp_sum(l_part[rr]);
                if (lane == 0) { w_m[warp * RT + rr] = m_run[rr]; w_l[warp * RT + rr] = l; }
#pragma unroll
                for (int i = 0; i < DPL; ++i) w_o[(warp * RT + rr) * D + lane * DPL + i] = oacc[rr][i];
            }
            __syncthreads();
            for (int i = threadIdx.x; i < RT * D; i += DS_THREADS) {
                const int rr = i / D, d = i % D, r = r0 + rr;
                if (r >= gqa) continue;
                float M = -INFINITY;
#pragma unroll
                for (int w = 0; w < DS_WARPS; ++w) M = fmaxf(M, w_m[w * RT + rr]);
                float L = 0.0f, acc = 0.0f;
#pragma unroll
                for (int w = 0; w < DS_WARPS; ++w) {
                    const float f = (w_m[w * RT + rr] == -INFINITY) ? 0.0f : expf(w_m[w * RT + rr] - M);
                    L += w_l[w * RT + rr] * f; acc += w_o[(w * RT + rr) * D + d] * f;
                }
                if (o.n_slices == 1) {
                    o.out[(int64_t) (hk * gqa + r) * D + d] = acc / L;
                } else {
                    part[(int64_t) r * DS_PSTRIDE + d] = acc;
                    if (d == 0) { part[(int64_t) r * DS_PSTRIDE + D] = M; part[(int64_t) r * DS_PSTRIDE + D + 1] = L; }
                }
            }
        }

        if (o.n_slices > 1 && !o.consumer_merge) {
            // ---- the last CTA of this KV head merges the slices, in slice order ----
            __threadfence();
            __syncthreads();
            if (threadIdx.x == 0) misc->ticket = atomicAdd(&o.tickets[hk], 1u);
            __syncthreads();
            if (misc->ticket == (unsigned) o.n_slices - 1) {
                __threadfence();
                const float * base = o.partials + (int64_t) hk * o.n_slices * gqa * DS_PSTRIDE;
                for (int i = threadIdx.x; i < gqa * D; i += DS_THREADS) {
                    const int r = i / D, d = i % D;
                    float M = -INFINITY;
                    for (int s = 0; s < o.n_slices; ++s) M = fmaxf(M, __ldcg(base + ((int64_t) s * gqa + r) * DS_PSTRIDE + D));
                    float L = 0.0f, acc = 0.0f;
                    for (int s = 0; s < o.n_slices; ++s) {
                        const float * ps_ = base + ((int64_t) s * gqa + r) * DS_PSTRIDE;
                        const float m_s = __ldcg(ps_ + D);
                        const float f = (m_s == -INFINITY) ? 0.0f : expf(m_s - M);
                        L += __ldcg(ps_ + D + 1) * f; acc += __ldcg(ps_ + d) * f;
                    }
                    o.out[(int64_t) (hk * gqa + r) * D + d] = acc / L;
                }
                if (threadIdx.x == 0) o.tickets[hk] = 0;                    // ready for the next use
            }
        }
    }
}

// ---------------------------------------------------------------------------
// the kernel
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(DS_THREADS, 1) decode_step_kernel(const __grid_constant__ DsParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t *  acts  = smem;
    uint64_t * bars  = (uint64_t *) (smem + DS_OFF_BAR);
    DsOp *     s_op  = (DsOp *) (smem + DS_OFF_OP);
    DsMisc *   misc  = (DsMisc *) (smem + DS_OFF_MISC);
    DsPart *   parts = (DsPart *) (smem + DS_OFF_DESC);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    uint8_t *  ring = smem + DS_OFF_RING + warp * DS_NSLOT * DS_SLOT;
    uint64_t * bar  = bars + warp * DS_NSLOT;
    const uint32_t G = gridDim.x * DS_WARPS, gw = (uint32_t) warp * gridDim.x + blockIdx.x;
    const int n_parts = p.n_parts;

    for (int i = tid; i < n_parts * (int) (sizeof(DsPart) / 16); i += DS_THREADS) ((uint4 *) parts)[i] = __ldg((const uint4 *) p.parts + i);
    for (int i = tid; i < DS_OP_BYTES / 16; i += DS_THREADS) ((uint4 *) s_op)[i] = __ldg((const uint4 *) p.ops + i);
    if (tid == 0) { misc->dead = 0; misc->ticket = 0; }
    if (lane == 0) for (int s = 0; s < DS_NSLOT; ++s) mbar_init(&bar[s], 1);
    mbar_fence_init();
    __syncthreads();

    // ---- the weight stream of this warp: f requests units, c (below) computes on them, in the same order ----
    DsCursor f;
    f.part = 0;
    ds_cursor_seek(f, parts, n_parts, gw, G);
    const uint32_t ring_s = smem_u32(ring), bar_s = smem_u32(bar);
    uint32_t f_off = 0, f_bar = bar_s;          // slot being filled next: byte offset in the ring, its mbarrier
    unsigned n_fetched = 0, n_done = 0;
    bool warp_dead = false;                     // this warp gave up a wait: it neither requests nor waits any more
    auto fetch_issue = [&]() {
        if (f.part >= n_parts) return;
        const uint32_t bytes = (f.s == f.nseg - 1) ? f.last_b : f.seg_b;
        if (lane == 0) {
            ds_fence_proxy_async();
            if (f.mode & 4) {                   // both rows of the group: adjacent in memory (one copy) or not (two)
                ds_expect_tx(f_bar, 2 * bytes);
                if (f.pair_off == (int64_t) bytes) ds_bulk(ring_s + f_off, f.src, 2 * bytes, f_bar);
                else { ds_bulk(ring_s + f_off, f.src, bytes, f_bar); ds_bulk(ring_s + f_off + bytes, f.src + f.pair_off, bytes, f_bar); }
            } else {
                ds_expect_tx(f_bar, bytes);
                ds_bulk(ring_s + f_off, f.src, bytes, f_bar);
            }
        }
        ++n_fetched;
        f_off += DS_SLOT; f_bar += 8;
        if (f_off == DS_NSLOT * DS_SLOT) { f_off = 0; f_bar = bar_s; }
        ds_cursor_advance(f, parts, n_parts, gw, G);
    };
#pragma unroll
    for (int s = 0; s < DS_NSLOT; ++s) fetch_issue();

    uint32_t c_off = 0, c_bar = bar_s, c_par = 0;   // slot being consumed; parities of all slots (bit = slot)
    uint32_t c_bit = 1;
    // waits for the unit in the current slot; returns its address
    auto unit_wait = [&]() -> const uint8_t * {
        if (!ds_try_wait(c_bar, (c_par & c_bit) ? 1u : 0u) && !warp_dead) {
            bool ok = false;
            for (int it = 0; it < DS_SPIN_LIMIT && !ok; ++it) ok = ds_try_wait(c_bar, (c_par & c_bit) ? 1u : 0u);
            if (!ok) { ds_give_up(p, misc, ERR_MBAR_TIMEOUT); warp_dead = true; f.part = n_parts; }
        }
        return ring + c_off;
    };
    // hands the slot back to the stream
    auto unit_done = [&]() {
        if (!warp_dead) { c_par ^= c_bit; ++n_done; }
        c_off += DS_SLOT; c_bar += 8; c_bit <<= 1;
        if (c_off == DS_NSLOT * DS_SLOT) { c_off = 0; c_bar = bar_s; c_bit = 1; }
        __syncwarp();
        fetch_issue();
    };

    DsCursor c;                                 // only part / g / g_end of it are used: the compute loop has its own nest
    c.part = 0;
    int mv = 0;
    unsigned phase = 0;
#pragma unroll 1
    for (int op = 0; op < p.n_ops; ++op) {
        const DsOp & o = s_op[op & 1];
        // the next phase's parameters travel while this phase runs (they become visible at the phase's barrier)
        uint4 next_op = make_uint4(0, 0, 0, 0);
        const bool carries = op + 1 < p.n_ops && tid < DS_OP_BYTES / 16;
        if (carries) next_op = __ldg((const uint4 *) (p.ops + op + 1) + tid);
        const bool stamp = p.timing && blockIdx.x == 0 && tid == 0;
        if (stamp) p.timing[op * 4 + 0] = ds_now();
        if (o.kind == DS_OP_MATVEC) {
            ds_matvec_input(o, acts, misc);
            if (stamp) p.timing[op * 4 + 1] = ds_now();
            const int epilogue = o.epilogue;
#pragma unroll 1
            for (; c.part < n_parts && parts[c.part].phase == mv; ++c.part) {
                if (!ds_cursor_enter(c, parts, gw, G)) continue;
                const DsPart & P = parts[c.part];
                const int type = P.type, nseg = P.nseg, seg_blk = P.seg_blk, last_blk = P.last_blk, mode = P.mode, mat = P.mat;
                const uint32_t g_begin = P.g_begin, g_end = c.g_end;
                const bool both = (mode & 4) != 0;
                const int n_member = both ? 1 : ((mode & 2) ? 2 : 1);
                float * const dst = o.dst[mat];
#pragma unroll 1
                for (uint32_t g = c.g; g < g_end; g += G) {
                    float acc0 = 0.0f, acc1 = 0.0f;
#pragma unroll 1
                    for (int j = 0; j < n_member; ++j) {
                        float a = 0.0f;
#pragma unroll 1
                        for (int sg = 0; sg < nseg; ++sg) {
                            const int nblk = sg == nseg - 1 ? last_blk : seg_blk;
                            const uint8_t * slot = unit_wait();
                            const uint8_t * ap = acts + sg * seg_blk * DS_ACT_STRIDE;
                            if (type == T_Q6_K) a += ds_dot_q6k(slot, nblk, ap, acts + DS_BS16_OFF + sg * seg_blk * 32, lane);
                            else if (lane < (both ? 2 * nblk : nblk)) {
                                // `both`: lanes [0, nblk) take the first row of the group, [nblk, 2 nblk) the second
                                const uint8_t * al = ap + ((both && lane >= nblk) ? lane - nblk : lane) * DS_ACT_STRIDE;
                                if (type == T_Q4_K)      a += ds_dot_blk<T_Q4_K>(slot + lane * 144, al);
                                else if (type == T_Q5_K) a += ds_dot_blk<T_Q5_K>(slot + lane * 176, al);
                                else if (type == T_Q4_0) a += ds_dot_q4_0(slot + lane * 144, al);
                                else                     a += ds_dot_q8_0(slot + lane * 272, al);
                            }
                            unit_done();
                        }
                        if (both) {
                            if (last_blk == 16) {           // halves of the warp: four butterfly steps, then lane 0 fetches the other half's sum
                                a += __shfl_xor_sync(0xffffffffu, a, 8); a += __shfl_xor_sync(0xffffffffu, a, 4);
                                a += __shfl_xor_sync(0xffffffffu, a, 2); a += __shfl_xor_sync(0xffffffffu, a, 1);
                                acc0 = a; acc1 = __shfl_sync(0xffffffffu, a, 16);
                            } else { acc0 = warp_sum(lane < last_blk ? a : 0.0f); acc1 = warp_sum(lane < last_blk ? 0.0f : a); }
                        } else if (j == 0) acc0 = warp_sum(a);
                        else acc1 = warp_sum(a);
                    }
                    if (lane == 0) {
                        const uint32_t lg = g - g_begin;
                        if (epilogue == DS_EP_STORE) {
                            if (mode & 2) { dst[2 * lg] = acc0; dst[2 * lg + 1] = acc1; }
                            else dst[lg] = acc0;
                        } else if (epilogue == DS_EP_SILU_MUL) {
                            const float sa = acc0 / (1.0f + expf(-acc0));
                            if (o.dst[0]) o.dst[0][lg] = acc0;
                            if (o.dst[1]) o.dst[1][lg] = acc1;
                            if (o.silu_out) o.silu_out[lg] = sa;
                            o.act_out[lg] = sa * acc1;
                        } else {
                            const uint32_t row0 = 2 * lg;
                            if (dst) { dst[row0] = acc0; dst[row0 + 1] = acc1; }
                            if (mat == 2) {
                                if (o.v_t) {                    // transposed cache: value j of the row is element [j][token]
                                    char * vb = (char *) misc->vc + (int64_t) row0 * o.v_nbd;
                                    *(__half *) vb = __float2half_rn(acc0);
                                    *(__half *) (vb + o.v_nbd) = __float2half_rn(acc1);
                                } else ((__half2 *) misc->vc)[lg] = __floats2half2_rn(acc0, acc1);
                            } else {
                                const int ip = (int) (row0 % (uint32_t) o.head_dim) >> 1;
                                float o0 = acc0, o1 = acc1;
                                if (2 * ip < o.n_dims) {
                                    const float2 cs = misc->rope_cs[ip];
                                    o0 = acc0 * cs.x - acc1 * cs.y; o1 = acc0 * cs.y + acc1 * cs.x;
                                }
                                if (mat == 0) { o.q_rope[row0] = o0; o.q_rope[row0 + 1] = o1; }
                                else {
                                    if (o.k_rope) { o.k_rope[row0] = o0; o.k_rope[row0 + 1] = o1; }
                                    ((__half2 *) misc->kc)[lg] = __floats2half2_rn(o0, o1);
                                }
                            }
                        }
                    }
                }
            }
            ++mv;
        } else if (o.kind == DS_OP_ATTN) {
            if (stamp) p.timing[op * 4 + 1] = ds_now();
            ds_attention(o, acts, misc);
        }
        if (carries) ((uint4 *) (s_op + ((op + 1) & 1)))[tid] = next_op;
        if (stamp) p.timing[op * 4 + 2] = ds_now();
        ds_grid_barrier(p, misc, ++phase * gridDim.x);
        if (stamp) p.timing[op * 4 + 3] = ds_now();
    }

    // ---- drain: nothing may still be writing into this CTA's shared memory when it exits ----
    for (; n_done < n_fetched; ++n_done) {
        bool ok = false;
        for (int it = 0; it < (1 << 20) && !ok; ++it) ok = ds_try_wait(c_bar, (c_par & c_bit) ? 1u : 0u);
        c_par ^= c_bit;
        c_off += DS_SLOT; c_bar += 8; c_bit <<= 1;
        if (c_off == DS_NSLOT * DS_SLOT) { c_off = 0; c_bar = bar_s; c_bit = 1; }
    }
    __syncthreads();
    if (tid == 0) {
        const unsigned n = atomicAdd(&p.sync[1], 1u);
        if (n == gridDim.x - 1) {                 // everyone is past the last barrier: reset for the next launch
            p.sync[0] = 0; p.sync[2] = 0;
            __threadfence();
            p.sync[1] = 0;
        }
    }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
int64_t decode_step_max_k() { return DS_MAX_K; }

bool decode_step_type_ok(int type, int64_t K, int64_t w_nb1, const void * W) {
    if (type != T_Q4_K && type != T_Q5_K && type != T_Q6_K && type != T_Q4_0 && type != T_Q8_0) return false;
    if (K <= 0 || K > DS_MAX_K || K % 256) return false;
    if (type == T_Q6_K && K % 2048) return false;                 // runs of 8 super-blocks are the 16-byte multiples
    if (((uintptr_t) W & 15) || (w_nb1 & 15) || w_nb1 <= 0 || w_nb1 > 0xffffffffll) return false;
    return true;
}

static size_t ds_smem_bytes(int n_parts) { return (size_t) DS_OFF_DESC + (size_t) n_parts * sizeof(DsPart); }

int decode_step_max_matvecs(int) { return (int) ((DS_SMEM_LIMIT - DS_OFF_DESC) / sizeof(DsPart) / 3); }

size_t decode_step_work_bytes(int n_ops) { return (size_t) (n_ops > 0 ? n_ops : 1) * 3 * sizeof(DsPart); }

static int ds_host_blk_bytes(int type) { return (type == T_Q4_K || type == T_Q4_0) ? 144 : (type == T_Q5_K ? 176 : (type == T_Q8_0 ? 272 : 210)); }
static int ds_host_cap(int type) { return (type == T_Q4_K || type == T_Q4_0) ? 32 : (type == T_Q5_K ? 24 : 16); }      // 256-value units per 4608-byte ring slot
// the parts of one mat-vec phase (at most three)
static bool ds_make_parts(const DsOp & o, int phase, uint32_t grid_warps, std::vector<DsPart> & out) {
    const bool zip = o.epilogue == DS_EP_SILU_MUL;
    // plain results are computed two rows at a time as well when every matrix has an even number of rows
    bool pair = o.epilogue != DS_EP_STORE;
    if (!pair) {
        pair = true;
        for (int i = 0; i < o.nmat; ++i) if ((o.M[i] & 1) || o.type[i] == T_Q6_K || o.K / 256 > ds_host_cap(o.type[i]) / 2) pair = false;   // only rows that share a slot
    }
    if (o.nmat < 1 || o.nmat > 3 || (zip && (o.nmat != 2 || o.M[0] != o.M[1]))) return false;
    uint32_t g = 0;
    for (int i = 0; i < (zip ? 1 : o.nmat); ++i) {
        const int type = o.type[i];
        if (!decode_step_type_ok(type, o.K, o.w_nb1[i], o.W[i]) || o.M[i] <= 0) return false;
        if (zip && (!decode_step_type_ok(o.type[1], o.K, o.w_nb1[1], o.W[1]) || o.type[1] != type || o.w_nb1[1] != o.w_nb1[0])) return false;
        if (pair && !zip && (o.M[i] & 1)) return false;
        const int nblk = o.K / 256, bb = ds_host_blk_bytes(type);
        const int cap = ds_host_cap(type);                                      // super-blocks per ring slot
        const int nseg = (nblk + cap - 1) / cap;
        DsPart P; memset(&P, 0, sizeof(P));
        P.W0 = (uint64_t) (uintptr_t) o.W[i]; P.W1 = zip ? (uint64_t) (uintptr_t) o.W[1] : 0;
        P.nb1 = (uint32_t) o.w_nb1[i];
        P.g_begin = g; g += (uint32_t) (pair && !zip ? o.M[i] / 2 : o.M[i]); P.g_end = g;
        P.first_mod = P.g_begin % grid_warps;
        P.type = (uint8_t) type; P.nseg = (uint8_t) nseg;
        P.seg_blk = (uint8_t) (nseg > 1 ? cap : nblk); P.last_blk = (uint8_t) (nblk - (nseg - 1) * cap);
        P.seg_b = (uint16_t) (P.seg_blk * bb); P.last_b = (uint16_t) (P.last_blk * bb);
        // short rows of the one-lane-per-block types: both rows of a pair share a ring slot
        const bool both = pair && type != T_Q6_K && nblk <= cap / 2;
        P.mode = (uint8_t) ((zip ? 1 : 0) | (pair ? 2 : 0) | (both ? 4 : 0));
        P.mat = (uint8_t) i; P.phase = (uint16_t) phase;
        out.push_back(P);
    }
    return true;
}

static bool ds_all_parts(const DsOp * ops, int n_ops, int sm_count, std::vector<DsPart> & parts) {
    int phase = 0;
    for (int i = 0; i < n_ops; ++i) {
        if (ops[i].kind != DS_OP_MATVEC) continue;
        if (!ds_make_parts(ops[i], phase++, (uint32_t) sm_count * DS_WARPS, parts)) return false;
    }
    return phase < 65536;
}

cudaError_t decode_step_prepare(const DsOp * ops, int n_ops, int sm_count, void * work, cudaStream_t copy_stream) {
    std::vector<DsPart> parts;
    if (!ds_all_parts(ops, n_ops, sm_count, parts)) return cudaErrorInvalidValue;
    if (ds_smem_bytes((int) parts.size()) > (size_t) DS_SMEM_LIMIT) return cudaErrorInvalidValue;
    if (parts.empty()) return cudaSuccess;
    // synchronous with respect to the host buffer: the vector dies at return
    cudaError_t e = cudaMemcpyAsync(work, parts.data(), parts.size() * sizeof(DsPart), cudaMemcpyHostToDevice, copy_stream);
    if (e != cudaSuccess) return e;
    return cudaStreamSynchronize(copy_stream);
}

cudaError_t launch_decode_step(const DsOp * ops_dev, const DsOp * ops, int n_ops, const void * work, unsigned * sync, const LaunchCtx & c,
                               unsigned long long * timing) {
    DsParams p = {};
    p.ops = ops_dev; p.n_ops = n_ops;
    p.parts = (const DsPart *) work;
    {
        std::vector<DsPart> parts;
        if (!ds_all_parts(ops, n_ops, c.sm_count, parts)) return cudaErrorInvalidValue;
        p.n_parts = (int) parts.size();
    }
    p.sync = sync; p.status = c.status; p.timing = timing;
    const size_t smem = ds_smem_bytes(p.n_parts);
    if (smem > (size_t) DS_SMEM_LIMIT) return cudaErrorInvalidValue;
    static unsigned long long attr_mask = 0;
    if (!(attr_mask & (1ull << (c.device & 63)))) {
        cudaError_t e = cudaFuncSetAttribute(decode_step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DS_SMEM_LIMIT);
        if (e != cudaSuccess) return e;
        attr_mask |= 1ull << (c.device & 63);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned) c.sm_count); cfg.blockDim = dim3(DS_THREADS);
    cfg.dynamicSmemBytes = smem; cfg.stream = c.stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeCooperative;
    at[0].val.cooperative = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, decode_step_kernel, p);
}

}  // namespace b200
