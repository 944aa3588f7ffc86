// Prefill-time quantized GEMM on the 5th-generation tensor cores (tcgen05 + TMEM).
//
//   dst[n][m] = sum_k W[m][k] * X[n][k]      W quantized (ggml blocks), X F32, dst F32
//
// Replaces the reference's mul_mat_q (ggml/src/ggml-cuda/mmq.cuh:2501-2911: mma.sync int8 tiles with
// an FP32 scale epilogue per 32-deep MMA).  ggml's scales change every 32 (16 for Q6_K) values along
// K on the weight side, so an integer accumulator would have to be drained from TMEM and scaled after
// every MMA; on tcgen05 that epilogue costs several times the MMA itself.  Instead the weight tile is
// dequantized to F16 on its way into shared memory (exact up to the F16 rounding of d*q), and one
// FP32 accumulator in TMEM runs over the whole K with tcgen05.mma kind::f16.
//
// CTA = 9 warps, one 128 (weight rows) x 128 or 256 (tokens) output tile (256 when that still gives every SM a CTA:
// a weight tile is then dequantized half as often):
//   warps 0-7  producers: thread (r, h) dequantizes 32 consecutive weights of weight row r per k-step
//              (raw quant bytes of the next k-step are prefetched into registers first) and writes them
//              as F16 in the canonical K-major SWIZZLE_128B layout (row r at r*128 B, 16-byte chunk c at
//              position c ^ (r & 7)); then fence.proxy.async + mbarrier arrive.  The activation tile
//              (128 tokens x 64 F16, pre-converted) is fetched by one plain, non-multicast TMA tile load
//              with the same swizzle, completing on the same barrier.  After the K loop the producer
//              warps become the epilogue: tcgen05.ld of the accumulator (lane = weight row, column =
//              token; warps w and w+4 share a lane quadrant and split the columns) and coalesced stores.
//   warp 8     one elected thread issues 4 x tcgen05.mma (M128 N128 K16) per k-step from shared-memory
//              matrix descriptors; tcgen05.commit frees the stage / publishes the accumulator.
//   warp 9     loader (types whose 256-value row chunks are 16-byte multiples: Q4_K, Q5_K, Q8_0, Q4_0, ...): brings the
//              raw quant bytes of the tile's 128 rows, one 256-deep K chunk at a time, into a double-buffered
//              shared-memory tile with cp.async.bulk (plain, non-multicast), one copy per row.  The producers then
//              read their bytes with shared-memory loads: a warp-wide global load of one row per thread touched 32
//              sectors and the load/store unit, not the tensor core, set the pace.  The other types keep the
//              producers' own global loads.
// Ring of 32 KB / 48 KB operand stages; every mbarrier wait is bounded and failure is reported through the
// status word; TMEM is allocated and released by warp 8 on every path.
#include "common.cuh"
#include "kernels.h"
#include "tcgen05.cuh"

namespace b200 {

static constexpr int TC_BM = 128, TC_BN = 128, TC_BK = 64;
static constexpr int TC_GROUP = 256;                                  // threads that dequantize one k-step: 128 rows x two 32-value halves
static constexpr int TC_PRODUCERS = 2 * TC_GROUP;                      // two groups work on different k-steps at the same time
static constexpr int TC_THREADS = TC_PRODUCERS + 64;                  // + the MMA warp and the loader warp
static constexpr int TC_CHUNK_K = 256;                                // K values per staged raw chunk (4 k-steps)
static constexpr int TC_PF = 4;                                        // k-steps of raw weight bytes in flight per producer thread

// ---- weight dequantization: 32 consecutive values of one row as F16 ---------------------------
// Raw<T> holds the quant bytes a thread needs for its 32 values of one k-step; load() only issues the
// loads (so the next k-step can be in flight while the current one is converted), get() converts.
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *(uint32_t *) &h;
}
__device__ __forceinline__ __half2 u32_as_h2(uint32_t v) { return *(__half2 *) &v; }
__device__ __forceinline__ uint32_t h2_as_u32(__half2 v) { return *(uint32_t *) &v; }
// bytes (b0, b1) or (b2, b3) of v, each 0..255, as half2 (exact): 0x6400 | b is the F16 number 1024 + b
__device__ __forceinline__ __half2 bytes01_h2(uint32_t v) { return __hsub2(u32_as_h2(__byte_perm(v, 0x64646464u, 0x4140)), u32_as_h2(0x64006400u)); }
__device__ __forceinline__ __half2 bytes23_h2(uint32_t v) { return __hsub2(u32_as_h2(__byte_perm(v, 0x64646464u, 0x4342)), u32_as_h2(0x64006400u)); }

template <int T> struct Deq32 {                     // generic path: element-wise through the bit-exact dequantizer
    static constexpr int KPR = 1;                                   // k-steps covered by one Raw
    struct Raw { const uint8_t * row; int k; };
    static __device__ __forceinline__ void load(const uint8_t * row, int k, Raw & r) { r.row = row; r.k = k; }
    static __device__ __forceinline__ void load_s(const uint8_t * b, int k, Raw & r) { r.row = b; r.k = k; }   // dequant_elem reads with plain loads
    static __device__ __forceinline__ void get(const Raw & r, uint32_t (&out)[16]) {
#pragma unroll 4
        for (int i = 0; i < 16; ++i) out[i] = pack_h2(dequant_elem<T>(r.row, r.k + 2 * i), dequant_elem<T>(r.row, r.k + 2 * i + 1));
    }
};

// Q4_K: k .. k+31 is one sub-block sb = (k >> 5) & 7: nibble (sb & 1) of qs bytes [32 (sb >> 1), +32)
template <> struct Deq32<T_Q4_K> {
    static constexpr int KPR = 1;                                   // k-steps covered by one Raw
    struct Raw { uint4 hd, qa, qb; int sb; };
    static __device__ __forceinline__ void load(const uint8_t * row, int k, Raw & r) {
        const uint8_t * b = row + (k >> 8) * 144;
        r.sb = (k >> 5) & 7;
        r.hd = __ldg((const uint4 *) b);
        r.qa = __ldg((const uint4 *) (b + 16 + 32 * (r.sb >> 1)));
        r.qb = __ldg((const uint4 *) (b + 32 + 32 * (r.sb >> 1)));
    }
    static __device__ __forceinline__ void load_s(const uint8_t * b, int k, Raw & r) {       // b: the row's chunk in shared memory
        r.sb = (k >> 5) & 7;
        r.hd = *(const uint4 *) b;
        r.qa = *(const uint4 *) (b + 16 + 32 * (r.sb >> 1));
        r.qb = *(const uint4 *) (b + 32 + 32 * (r.sb >> 1));
    }
    static __device__ __forceinline__ void get(const Raw & r, uint32_t (&out)[16]) {
        const float2 dm = __half22float2(u32_as_h2(r.hd.x));
        const uint32_t s0 = r.hd.y, s1 = r.hd.z, s2 = r.hd.w;
        int sc, m;
        if (r.sb < 4) { sc = (s0 >> (8 * r.sb)) & 63; m = (s1 >> (8 * r.sb)) & 63; }
        else { const int t = r.sb - 4; sc = ((s2 >> (8 * t)) & 0xF) | (((s0 >> (8 * t + 6)) & 3) << 4); m = ((s2 >> (8 * t + 4)) & 0xF) | (((s1 >> (8 * t + 6)) & 3) << 4); }
        const __half2 ds = __float2half2_rn(dm.x * (float) sc), nm = __float2half2_rn(-dm.y * (float) m);
        const uint32_t w[8] = {r.qa.x, r.qa.y, r.qa.z, r.qa.w, r.qb.x, r.qb.y, r.qb.z, r.qb.w};
        const int sh = (r.sb & 1) * 4;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t v = (w[i] >> sh) & 0x0F0F0F0Fu;
            out[2 * i]     = h2_as_u32(__hfma2(bytes01_h2(v), ds, nm));
            out[2 * i + 1] = h2_as_u32(__hfma2(bytes23_h2(v), ds, nm));
        }
    }
};

// Q5_K: as Q4_K plus bit sb of qh[l] as the fifth bit.  A thread's consecutive k-steps are sub-blocks sb and sb + 2 of
// the same super-block: they share the header and the 32 qh bytes, so one Raw is loaded per pair of k-steps.
template <> struct Deq32<T_Q5_K> {
    static constexpr int KPR = 2;
    struct Raw { uint4 hd, ha, hb, qa[2], qb[2]; int sb0; };
    static __device__ __forceinline__ void load(const uint8_t * row, int k, Raw & r) {      // k: first k-step of the pair
        const uint8_t * b = row + (k >> 8) * 176;
        r.sb0 = (k >> 5) & 7;
        r.hd = __ldg((const uint4 *) b);
        r.ha = __ldg((const uint4 *) (b + 16));
        r.hb = __ldg((const uint4 *) (b + 32));
#pragma unroll
        for (int s = 0; s < 2; ++s) {
            const int o = 48 + 32 * ((r.sb0 + 2 * s) >> 1);
            r.qa[s] = __ldg((const uint4 *) (b + o));
            r.qb[s] = __ldg((const uint4 *) (b + o + 16));
        }
    }
    static __device__ __forceinline__ void load_s(const uint8_t * b, int k, Raw & r) {
        r.sb0 = (k >> 5) & 7;
        r.hd = *(const uint4 *) b;
        r.ha = *(const uint4 *) (b + 16);
        r.hb = *(const uint4 *) (b + 32);
#pragma unroll
        for (int s = 0; s < 2; ++s) {
            const int o = 48 + 32 * ((r.sb0 + 2 * s) >> 1);
            r.qa[s] = *(const uint4 *) (b + o);
            r.qb[s] = *(const uint4 *) (b + o + 16);
        }
    }
    static __device__ __forceinline__ void get(const Raw & r, int sub, uint32_t (&out)[16]) {
        const int sb = r.sb0 + 2 * sub;
        const float2 dm = __half22float2(u32_as_h2(r.hd.x));
        const uint32_t s0 = r.hd.y, s1 = r.hd.z, s2 = r.hd.w;
        int sc, m;
        if (sb < 4) { sc = (s0 >> (8 * sb)) & 63; m = (s1 >> (8 * sb)) & 63; }
        else { const int t = sb - 4; sc = ((s2 >> (8 * t)) & 0xF) | (((s0 >> (8 * t + 6)) & 3) << 4); m = ((s2 >> (8 * t + 4)) & 0xF) | (((s1 >> (8 * t + 6)) & 3) << 4); }
        const __half2 ds = __float2half2_rn(dm.x * (float) sc), nm = __float2half2_rn(-dm.y * (float) m);
        const uint4 qa = sub ? r.qa[1] : r.qa[0], qb = sub ? r.qb[1] : r.qb[0];
        const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
        const uint32_t h[8] = {r.ha.x, r.ha.y, r.ha.z, r.ha.w, r.hb.x, r.hb.y, r.hb.z, r.hb.w};
        const int sh = (sb & 1) * 4;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t v = ((w[i] >> sh) & 0x0F0F0F0Fu) | (((h[i] >> sb) & 0x01010101u) << 4);      // 4 values 0..31
            out[2 * i]     = h2_as_u32(__hfma2(bytes01_h2(v), ds, nm));
            out[2 * i + 1] = h2_as_u32(__hfma2(bytes23_h2(v), ds, nm));
        }
    }
};

// Q6_K: k .. k+31 is group t = (k >> 5) & 3 of half n128 = (k >> 7) & 1 (ggml-quants.c:1690-1719);
// blocks are only 2-byte aligned, so the bytes come in as aligned words plus a funnel shift
// Q6_K: the 32 ql bytes and 32 qh bytes a thread reads hold its weights of TWO k-steps (sub-block groups t and
// t + 2 are the low and high nibbles of the same bytes), so one Raw is loaded per pair of k-steps.
template <> struct Deq32<T_Q6_K> {
    static constexpr int KPR = 2;
    struct Raw { uint32_t ql[9], qh[9], sc[2], d; uint32_t sh; int t0; };
    static __device__ __forceinline__ void load(const uint8_t * row, int k, Raw & r) {      // k: first k-step of the pair
        const uint8_t * b = row + (k >> 8) * 210;
        const int n128 = (k >> 7) & 1;
        r.t0 = (k >> 5) & 1;                                            // the pair is (t0, t0 + 2)
        const uint8_t * pl = b + n128 * 64 + r.t0 * 32;                 // 32 bytes of ql
        const uint8_t * ph = b + 128 + n128 * 32;                       // 32 bytes of qh
        const uint32_t * al = (const uint32_t *) ((uintptr_t) pl & ~(uintptr_t) 3);
        const uint32_t * ah = (const uint32_t *) ((uintptr_t) ph & ~(uintptr_t) 3);
        r.sh = ((uint32_t) (uintptr_t) pl & 3u) * 8u;                   // pl and ph have the same alignment (offsets differ by a multiple of 4)
#pragma unroll
        for (int i = 0; i < 9; ++i) { r.ql[i] = __ldg(al + i); r.qh[i] = __ldg(ah + i); }
        const uint8_t * ps = b + 192 + n128 * 8 + 2 * r.t0;            // scales[2t], scales[2t+1] for t = t0 and t0 + 2; d at b+208
        r.sc[0] = *(const uint16_t *) ps;
        r.sc[1] = *(const uint16_t *) (ps + 4);
        r.d = *(const uint16_t *) (b + 208);
    }
    static __device__ __forceinline__ void load_s(const uint8_t * b, int k, Raw & r) {       // b: the row's super-block in shared memory
        const int n128 = (k >> 7) & 1;
        r.t0 = (k >> 5) & 1;
        const uint8_t * pl = b + n128 * 64 + r.t0 * 32;
        const uint8_t * ph = b + 128 + n128 * 32;
        const uint32_t * al = (const uint32_t *) ((uintptr_t) pl & ~(uintptr_t) 3);
        const uint32_t * ah = (const uint32_t *) ((uintptr_t) ph & ~(uintptr_t) 3);
        r.sh = ((uint32_t) (uintptr_t) pl & 3u) * 8u;
#pragma unroll
        for (int i = 0; i < 9; ++i) { r.ql[i] = al[i]; r.qh[i] = ah[i]; }
        const uint8_t * ps = b + 192 + n128 * 8 + 2 * r.t0;
        r.sc[0] = *(const uint16_t *) ps;
        r.sc[1] = *(const uint16_t *) (ps + 4);
        r.d = *(const uint16_t *) (b + 208);
    }
    static __device__ __forceinline__ void get(const Raw & r, int sub, uint32_t (&out)[16]) {
        const float d = __half2float(__ushort_as_half((unsigned short) r.d));
        const uint32_t scw = sub ? r.sc[1] : r.sc[0];
        const __half2 dlo = __float2half2_rn(d * (float) (int) (int8_t) (scw & 0xff));
        const __half2 dhi = __float2half2_rn(d * (float) (int) (int8_t) (scw >> 8));
        const __half2 off = u32_as_h2(0x50005000u);                     // 32.0 in F16
        const int hs = 2 * (r.t0 + 2 * sub), ns = sub ? 4 : 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t L = __funnelshift_r(r.ql[i], r.ql[i + 1], r.sh), H = __funnelshift_r(r.qh[i], r.qh[i + 1], r.sh);
            const uint32_t q = ((L >> ns) & 0x0F0F0F0Fu) | (((H >> hs) & 0x03030303u) << 4);     // 4 values 0..63
            const __half2 sd = i < 4 ? dlo : dhi;                       // l < 16 uses scales[2t], l >= 16 scales[2t+1]
            out[2 * i]     = h2_as_u32(__hmul2(__hsub2(bytes01_h2(q), off), sd));
            out[2 * i + 1] = h2_as_u32(__hmul2(__hsub2(bytes23_h2(q), off), sd));
        }
    }
};

// Q4_0 / Q8_0: one 32-value block per thread and k-step
// A block {fp16 d, NQ words of quants} at a 2-byte aligned address: read as aligned 32-bit words (at most two bytes past the
// block; every buffer has tail slack) and realigned with one funnel shift per word.
template <int NQ>
__device__ __forceinline__ void load_block32(const uint8_t * pb, uint32_t (&q)[NQ], uint32_t & d) {
    const uint32_t * al = (const uint32_t *) ((uintptr_t) pb & ~(uintptr_t) 3);
    const bool odd = ((uintptr_t) pb & 2) != 0;                     // block starts in the upper half of al[0]
    uint32_t w[NQ + 1];
#pragma unroll
    for (int i = 0; i < NQ + 1; ++i) w[i] = __ldg(al + i);
    d = odd ? (w[0] >> 16) : (w[0] & 0xffffu);
#pragma unroll
    for (int i = 0; i < NQ; ++i) q[i] = odd ? w[i + 1] : __funnelshift_r(w[i], w[i + 1], 16);
}

template <int NQ>
__device__ __forceinline__ void load_block32_s(const uint8_t * pb, uint32_t (&q)[NQ], uint32_t & d) {       // shared memory
    const uint32_t * al = (const uint32_t *) ((uintptr_t) pb & ~(uintptr_t) 3);
    const bool odd = ((uintptr_t) pb & 2) != 0;
    uint32_t w[NQ + 1];
#pragma unroll
    for (int i = 0; i < NQ + 1; ++i) w[i] = al[i];
    d = odd ? (w[0] >> 16) : (w[0] & 0xffffu);
#pragma unroll
    for (int i = 0; i < NQ; ++i) q[i] = odd ? w[i + 1] : __funnelshift_r(w[i], w[i + 1], 16);
}

template <> struct Deq32<T_Q4_0> {
    static constexpr int KPR = 1;                                   // k-steps covered by one Raw
    struct Raw { uint32_t w[4]; uint32_t d; };
    static __device__ __forceinline__ void load(const uint8_t * row, int k, Raw & r) { load_block32<4>(row + (k >> 5) * 18, r.w, r.d); }
    static __device__ __forceinline__ void load_s(const uint8_t * b, int k, Raw & r) { load_block32_s<4>(b + (k >> 5) * 18, r.w, r.d); }
    static __device__ __forceinline__ void get(const Raw & r, uint32_t (&out)[16]) {
        const __half2 d = __half2half2(__ushort_as_half((unsigned short) r.d)), off = u32_as_h2(0x48004800u);   // 8.0
#pragma unroll
        for (int i = 0; i < 4; ++i) {                                   // low nibbles: elements 4i..4i+3, high: 16+4i..
            const uint32_t lo = r.w[i] & 0x0F0F0F0Fu, hi = (r.w[i] >> 4) & 0x0F0F0F0Fu;
            out[2 * i]         = h2_as_u32(__hmul2(__hsub2(bytes01_h2(lo), off), d));
            out[2 * i + 1]     = h2_as_u32(__hmul2(__hsub2(bytes23_h2(lo), off), d));
            out[8 + 2 * i]     = h2_as_u32(__hmul2(__hsub2(bytes01_h2(hi), off), d));
            out[8 + 2 * i + 1] = h2_as_u32(__hmul2(__hsub2(bytes23_h2(hi), off), d));
        }
    }
};
template <> struct Deq32<T_Q8_0> {
    static constexpr int KPR = 1;                                   // k-steps covered by one Raw
    struct Raw { uint32_t w[8]; uint32_t d; };
    static __device__ __forceinline__ void load(const uint8_t * row, int k, Raw & r) { load_block32<8>(row + (k >> 5) * 34, r.w, r.d); }
    static __device__ __forceinline__ void load_s(const uint8_t * b, int k, Raw & r) { load_block32_s<8>(b + (k >> 5) * 34, r.w, r.d); }
    static __device__ __forceinline__ void get(const Raw & r, uint32_t (&out)[16]) {
        const __half2 d = __half2half2(__ushort_as_half((unsigned short) r.d)), off = u32_as_h2(0x58005800u);   // 128.0
#pragma unroll
        for (int i = 0; i < 8; ++i) {                                   // signed byte + 128 = unsigned byte
            const uint32_t u = r.w[i] ^ 0x80808080u;
            out[2 * i]     = h2_as_u32(__hmul2(__hsub2(bytes01_h2(u), off), d));
            out[2 * i + 1] = h2_as_u32(__hmul2(__hsub2(bytes23_h2(u), off), d));
        }
    }
};

// IQ4_NL: the Q4_0 block with its nibbles mapped through the code book; table values are signed bytes
template <> struct Deq32<T_IQ4_NL> {
    static constexpr int KPR = 1;
    struct Raw { uint32_t w[4]; uint32_t d; };
    static __device__ __forceinline__ void load(const uint8_t * row, int k, Raw & r) { load_block32<4>(row + (k >> 5) * 18, r.w, r.d); }
    static __device__ __forceinline__ void load_s(const uint8_t * b, int k, Raw & r) { load_block32_s<4>(b + (k >> 5) * 18, r.w, r.d); }
    static __device__ __forceinline__ void get(const Raw & r, uint32_t (&out)[16]) {
        const __half2 d = __half2half2(__ushort_as_half((unsigned short) r.d)), off = u32_as_h2(0x58005800u);   // 128.0
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t lo = iq4nl_lut4(r.w[i] & 0x0F0F0F0Fu) ^ 0x80808080u, hi = iq4nl_lut4((r.w[i] >> 4) & 0x0F0F0F0Fu) ^ 0x80808080u;
            out[2 * i]         = h2_as_u32(__hmul2(__hsub2(bytes01_h2(lo), off), d));
            out[2 * i + 1]     = h2_as_u32(__hmul2(__hsub2(bytes23_h2(lo), off), d));
            out[8 + 2 * i]     = h2_as_u32(__hmul2(__hsub2(bytes01_h2(hi), off), d));
            out[8 + 2 * i + 1] = h2_as_u32(__hmul2(__hsub2(bytes23_h2(hi), off), d));
        }
    }
};
// IQ4_XS: blocks of 136 bytes are 8-byte aligned; a k-step is sub-block ib: 16 qs bytes and a 6-bit scale
template <> struct Deq32<T_IQ4_XS> {
    static constexpr int KPR = 1;
    struct Raw { uint2 hd, q0, q1; int ib; };
    static __device__ __forceinline__ void load(const uint8_t * row, int k, Raw & r) {
        const uint8_t * b = row + (k >> 8) * 136;
        r.ib = (k >> 5) & 7;
        r.hd = __ldg((const uint2 *) b);
        r.q0 = __ldg((const uint2 *) (b + 8 + 16 * r.ib));
        r.q1 = __ldg((const uint2 *) (b + 16 + 16 * r.ib));
    }
    static __device__ __forceinline__ void get(const Raw & r, uint32_t (&out)[16]) {
        const int ls = (int) (((r.hd.y >> (4 * r.ib)) & 0xF) | ((((r.hd.x >> 16) >> (2 * r.ib)) & 3) << 4)) - 32;   // scales_l nibble, scales_h pair
        const __half2 d = __float2half2_rn(__half2float(__ushort_as_half((unsigned short) (r.hd.x & 0xffffu))) * (float) ls);
        const __half2 off = u32_as_h2(0x58005800u);
        const uint32_t w[4] = {r.q0.x, r.q0.y, r.q1.x, r.q1.y};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t lo = iq4nl_lut4(w[i] & 0x0F0F0F0Fu) ^ 0x80808080u, hi = iq4nl_lut4((w[i] >> 4) & 0x0F0F0F0Fu) ^ 0x80808080u;
            out[2 * i]         = h2_as_u32(__hmul2(__hsub2(bytes01_h2(lo), off), d));
            out[2 * i + 1]     = h2_as_u32(__hmul2(__hsub2(bytes23_h2(lo), off), d));
            out[8 + 2 * i]     = h2_as_u32(__hmul2(__hsub2(bytes01_h2(hi), off), d));
            out[8 + 2 * i + 1] = h2_as_u32(__hmul2(__hsub2(bytes23_h2(hi), off), d));
        }
    }
};
// Q2_K: blocks of 84 bytes are 4-byte aligned.  A thread's consecutive k-steps are bit pairs j and j + 2 of the same 32
// qs bytes (128-half n128), so one Raw serves a pair of k-steps; each k-step has two 16-weight sub-blocks with a 4-bit
// scale and a 4-bit min.
template <> struct Deq32<T_Q2_K> {
    static constexpr int KPR = 2;
    struct Raw { uint32_t q[8], sc[2], dm; int j0; };
    static __device__ __forceinline__ void load(const uint8_t * row, int k, Raw & r) {      // k: first k-step of the pair
        const uint8_t * b = row + (k >> 8) * 84;
        const int n128 = (k >> 7) & 1;
        r.j0 = (k >> 5) & 1;                                            // the pair is (j0, j0 + 2)
        const uint32_t * pq = (const uint32_t *) (b + 16 + 32 * n128);
#pragma unroll
        for (int i = 0; i < 8; ++i) r.q[i] = __ldg(pq + i);
        r.sc[0] = *(const uint16_t *) (b + 8 * n128 + 2 * r.j0);        // scales[8 n + 2 j], [.. + 1]
        r.sc[1] = *(const uint16_t *) (b + 8 * n128 + 2 * r.j0 + 4);
        r.dm = __ldg((const uint32_t *) (b + 80));
    }
    static __device__ __forceinline__ void get(const Raw & r, int sub, uint32_t (&out)[16]) {
        const float2 dm = __half22float2(u32_as_h2(r.dm));
        const uint32_t scw = sub ? r.sc[1] : r.sc[0];
        const __half2 d0 = __float2half2_rn(dm.x * (float) (scw & 0xF)),        m0 = __float2half2_rn(-dm.y * (float) ((scw >> 4) & 0xF));
        const __half2 d1 = __float2half2_rn(dm.x * (float) ((scw >> 8) & 0xF)), m1 = __float2half2_rn(-dm.y * (float) (scw >> 12));
        const int sh = 2 * (r.j0 + 2 * sub);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t v = (r.q[i] >> sh) & 0x03030303u;
            out[2 * i]     = h2_as_u32(__hfma2(bytes01_h2(v), i < 4 ? d0 : d1, i < 4 ? m0 : m1));
            out[2 * i + 1] = h2_as_u32(__hfma2(bytes23_h2(v), i < 4 ? d0 : d1, i < 4 ? m0 : m1));
        }
    }
};
// Q3_K: blocks of 110 bytes are 2-byte aligned: the 32 qs bytes and the 32 hmask bytes come in as aligned words plus a
// funnel shift (both at the same alignment: their offsets differ by a multiple of 4).  Pairs of k-steps as for Q2_K.
template <> struct Deq32<T_Q3_K> {
    static constexpr int KPR = 2;
    struct Raw { uint32_t q[9], hm[9]; uint32_t s0, s1, s2; uint32_t d, sh; int j0, n128; };
    static __device__ __forceinline__ void load(const uint8_t * row, int k, Raw & r) {
        const uint8_t * b = row + (k >> 8) * 110;
        r.n128 = (k >> 7) & 1;
        r.j0 = (k >> 5) & 1;
        const uint8_t * pq = b + 32 + 32 * r.n128;
        const uint32_t * aq = (const uint32_t *) ((uintptr_t) pq & ~(uintptr_t) 3);
        const uint32_t * ah = (const uint32_t *) ((uintptr_t) b & ~(uintptr_t) 3);
        r.sh = ((uint32_t) (uintptr_t) b & 3u) * 8u;
#pragma unroll
        for (int i = 0; i < 9; ++i) { r.q[i] = __ldg(aq + i); r.hm[i] = __ldg(ah + i); }
        const uint16_t * ps = (const uint16_t *) (b + 96);              // the 12 scale bytes as three words
        r.s0 = ps[0] | ((uint32_t) ps[1] << 16); r.s1 = ps[2] | ((uint32_t) ps[3] << 16); r.s2 = ps[4] | ((uint32_t) ps[5] << 16);
        r.d = ps[6];
    }
    static __device__ __forceinline__ int scale6(const Raw & r, int s) {
        auto byte = [&](int t) { return ((t < 4 ? r.s0 : (t < 8 ? r.s1 : r.s2)) >> (8 * (t & 3))) & 0xFFu; };
        const uint32_t lo = s < 8 ? (byte(s) & 0xF) : (byte(s - 8) >> 4);
        return (int) (lo | (((byte(8 + (s & 3)) >> (2 * (s >> 2))) & 3) << 4)) - 32;
    }
    static __device__ __forceinline__ void get(const Raw & r, int sub, uint32_t (&out)[16]) {
        const int j = r.j0 + 2 * sub;
        const float d = __half2float(__ushort_as_half((unsigned short) r.d));
        const __half2 d0 = __float2half2_rn(d * (float) scale6(r, 8 * r.n128 + 2 * j)), d1 = __float2half2_rn(d * (float) scale6(r, 8 * r.n128 + 2 * j + 1));
        const __half2 off = u32_as_h2(0x44004400u);                     // 4.0
        const int hb = 4 * r.n128 + j;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t Q = __funnelshift_r(r.q[i], r.q[i + 1], r.sh), H = __funnelshift_r(r.hm[i], r.hm[i + 1], r.sh);
            const uint32_t v = ((Q >> (2 * j)) & 0x03030303u) | (((H >> hb) & 0x01010101u) << 2);          // 0..7, value = v - 4
            out[2 * i]     = h2_as_u32(__hmul2(__hsub2(bytes01_h2(v), off), i < 4 ? d0 : d1));
            out[2 * i + 1] = h2_as_u32(__hmul2(__hsub2(bytes23_h2(v), off), i < 4 ? d0 : d1));
        }
    }
};

// Staging of raw blocks through shared memory.  SRC: bytes of one row's 256-value chunk; BYTES: bytes per row of the box
// that is copied (0: not staged).  A tensor copy starts on a 16-byte boundary, so where SRC is not a multiple of 16 the
// box starts at the boundary below the chunk and is wide enough for every remainder; readers add the remainder.
template <int T> struct TcChunk { static constexpr int SRC = 0, BYTES = 0; };
template <> struct TcChunk<T_Q4_K>   { static constexpr int SRC = 144, BYTES = 144; };
template <> struct TcChunk<T_Q5_K>   { static constexpr int SRC = 176, BYTES = 176; };
template <> struct TcChunk<T_Q6_K>   { static constexpr int SRC = 210, BYTES = 240; };    // 210 + 14 = 224; 240 spreads rows over 8 banks
template <> struct TcChunk<T_Q8_0>   { static constexpr int SRC = 272, BYTES = 272; };
template <> struct TcChunk<T_Q4_0>   { static constexpr int SRC = 144, BYTES = 144; };
template <> struct TcChunk<T_IQ4_NL> { static constexpr int SRC = 144, BYTES = 144; };
template <> struct TcChunk<T_Q4_1>   { static constexpr int SRC = 160, BYTES = 160; };
template <> struct TcChunk<T_Q5_0>   { static constexpr int SRC = 176, BYTES = 176; };
template <> struct TcChunk<T_Q5_1>   { static constexpr int SRC = 192, BYTES = 192; };

// ---- F32 -> F16 activations (pre-pass) --------------------------------------------------------
__global__ void tc_convert_x_kernel(const float * __restrict__ x, int64_t x_nb1 /*bytes*/, __half * __restrict__ y, int64_t K, int64_t N) {
    pdl_enter();
    const int64_t total = N * K / 2;
    for (int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t) gridDim.x * blockDim.x) {
        const int64_t n = (2 * i) / K, k = (2 * i) % K;
        const float2 v = *(const float2 *) ((const char *) x + n * x_nb1 + k * 4);
        ((__half2 *) y)[i] = __floats2half2_rn(v.x, v.y);
    }
}

// ---- the GEMM kernel ---------------------------------------------------------------------------
static constexpr int TC_MAX_MATS = 3;
struct TcParams {
    int staged;                 // raw blocks come through shared memory by tensor copies (needs 16-byte aligned rows)
    // Up to three weight matrices of one type and row length that share the activations (wq/wk/wv, gate/up) run as one
    // launch: their 128-row tiles are numbered consecutively, matrix j owning m-tiles [mt0[j], mt0[j + 1]).
    int n_mats;
    const uint8_t * W[TC_MAX_MATS]; int64_t w_nb1;
    float * dst[TC_MAX_MATS]; int64_t dst_nb1[TC_MAX_MATS];      // bytes between token columns
    int M[TC_MAX_MATS], mt0[TC_MAX_MATS + 1];
    const __half * Xh;                 // [N][K] F16 (read through the tensor map)
    int N, K;
    int * status;
    // Tiles are numbered with the token tile fastest (neighbouring CTAs share a weight tile in L2).  CTAs [0, n_direct)
    // compute one whole tile each.  The tiles after those (the part of the output that would not fill another wave of
    // CTAs, or every tile of a small output) are divided along K: CTA n_direct + r * ksplit + z computes k-steps
    // [z * kps, z * kps + kps) of tile n_direct + r into the partial tile part + (r * ksplit + z) * 128 * BN, and
    // tc_reduce_kernel sums the splits in order.
    int n_tiles_n, n_direct, ksplit, kps; float * part;
    // MUL_MAT_ID over many (slot, token) pairs: the pairs are sorted by expert (tc_moe_sort_kernel), their activations
    // gathered into Xh in that order, and a token tile is a run of up to BN sorted rows of ONE expert, listed on the device:
    // moe_tiles[t] = {expert, first row, end row, 0}.  CTA = (m-tile, tile slot); slots past *moe_n_tiles leave at once.
    // Row r of the sorted order is stored at dst + moe_row_off[r].  W[0] is expert 0, w_nb2 bytes between experts.
    const int4 * moe_tiles; const int * moe_n_tiles; const int64_t * moe_row_off; int moe_nt_max, moe_n_expert; int64_t w_nb2;
};


// BN: token columns per CTA, 128 or 256.  The wide tile halves the number of times a weight tile is dequantized (the
// producers, not the tensor core, bound this kernel) and is used when it still leaves every SM a CTA.
template <int BN> struct TcCfg {
    static constexpr int STAGES = 4;
    static constexpr int TMEM_COLS = BN == 256 ? 512 : 256;          // accumulator (BN columns) + the ring of weight tiles (32 columns each)
    // (+16: the readers of 2-byte aligned blocks look one word past the last block of a row)
    template <int T> static __host__ __device__ constexpr int raw_bytes() { return (TC_BM * TcChunk<T>::BYTES + 16 + 127) & ~127; }
    template <int T> static __host__ __device__ constexpr int raw_bufs() {
        return TcChunk<T>::BYTES == 0 ? 0 : ((size_t) STAGES * BN * TC_BK * 2 + 3 * (size_t) raw_bytes<T>() + 2048 <= 232448 ? 3 : 2);
    }
    template <int T> static __host__ __device__ constexpr size_t smem_bytes() { return (size_t) STAGES * BN * TC_BK * 2 + (size_t) raw_bufs<T>() * raw_bytes<T>() + 1024; }
};

template <int T, int BN>
__global__ void __launch_bounds__(TC_THREADS, 1) mmq_tc_kernel(const TcParams p, const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap wmap0,
                                                                const __grid_constant__ CUtensorMap wmap1, const __grid_constant__ CUtensorMap wmap2) {
    constexpr int STAGES = TcCfg<BN>::STAGES;
    constexpr int STAGE_BYTES = BN * TC_BK * 2;                       // activation tile: 16 KB / 32 KB
    constexpr uint32_t A_COL0 = BN;                                   // tensor-memory column of the first weight tile
    constexpr int CB = TcChunk<T>::BYTES;                             // raw bytes of one row's 256-value chunk (0: not staged)
    constexpr bool STAGED = CB > 0;
    constexpr int RAW_BYTES = TcCfg<BN>::template raw_bytes<T>();     // one raw tile [128 rows][CB], padded to the 128-byte TMA alignment
    constexpr int NRB = TcCfg<BN>::template raw_bufs<T>();            // raw tiles in flight
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    pdl_launch_dependents();          // the next kernel may start its prologue (its weight prefetch) right away
    // operand stages must be 1024-byte aligned for the 128-byte swizzle pattern
    uint8_t * smem = (uint8_t *) (((uintptr_t) smem_raw + 1023) & ~(uintptr_t) 1023);
    uint8_t * rawbuf = smem + (size_t) STAGES * STAGE_BYTES;          // the raw tiles
    __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], accum_bar, raw_full[3], raw_empty[3];
    __shared__ uint32_t tmem_base_sh;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    // which tile, which part of K
    const int cta = (int) blockIdx.x;
    const bool moe = p.moe_tiles != nullptr;
    int moe_expert = 0, moe_row0 = 0, moe_row_end = 0;
    if (moe) {
        const int slot = cta % p.moe_nt_max;
        if (slot >= *p.moe_n_tiles) return;                         // (before any barrier or tensor-memory set-up; uniform over the CTA)
        const int4 t = p.moe_tiles[slot];
        moe_expert = t.x; moe_row0 = t.y; moe_row_end = t.z;
    }
    const bool is_split = !moe && cta >= p.n_direct;
    const int tile = is_split ? p.n_direct + (cta - p.n_direct) / p.ksplit : cta;
    const int zsplit = is_split ? (cta - p.n_direct) % p.ksplit : 0;
    const int mt = moe ? cta / p.moe_nt_max : tile / p.n_tiles_n, n0 = moe ? moe_row0 : (tile - mt * p.n_tiles_n) * BN;
    const int mat = (p.n_mats > 2 && mt >= p.mt0[2]) ? 2 : ((p.n_mats > 1 && mt >= p.mt0[1]) ? 1 : 0);
    const int m0 = (mt - p.mt0[mat]) * TC_BM;
    const int M = p.M[mat];
    const uint8_t * Wm = p.W[mat] + (int64_t) moe_expert * p.w_nb2;
    const CUtensorMap * wmap = mat == 0 ? &wmap0 : (mat == 1 ? &wmap1 : &wmap2);
    const int ks_begin = is_split ? zsplit * p.kps : 0;             // this CTA's range of k-steps
    const int ksteps = is_split ? min(p.kps, p.K / TC_BK - ks_begin) : p.K / TC_BK;
    const int k_base = ks_begin * TC_BK;
    constexpr int MMA_WARP = TC_PRODUCERS / 32;                       // the warp after it is the loader

    if (tid == 0) {
        // per stage: one arrival per warp of the producing group + 1 arrive.expect_tx for the activation tile
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], TC_GROUP / 32 + 1); mbar_init(&empty_bar[s], 1); }
        for (int s = 0; s < 3; ++s) { mbar_init(&raw_full[s], 1); mbar_init(&raw_empty[s], TC_PRODUCERS / 32); }
        mbar_init(&accum_bar, 1);
        abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == MMA_WARP) tmem_alloc(&tmem_base_sh, TcCfg<BN>::TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_sh;

    if (warp < MMA_WARP) {
        // ------------------------------ producers ------------------------------
        // Two groups of 8 warps: group g takes the k-step pairs (4c + 2g, 4c + 2g + 1) of every 256-value chunk c, so two
        // k-steps are being dequantized at any time (one group alone leaves each scheduler two warps and is bound by
        // instruction latency).  A group is never more than 3 k-steps past its previous one, which keeps its parity waits
        // on the stage ring within one phase of the tensor core's progress.
        const int r = tid & 127, h = (tid >> 7) & 1, g = tid >> 8;      // operand row, which 32 of the 64 k-values, group
        const bool wrow_ok = m0 + r < M;
        const uint8_t * wrow = Wm + (int64_t) (wrow_ok ? m0 + r : 0) * p.w_nb1;
        constexpr int KPR = Deq32<T>::KPR;                              // k-steps covered by one Raw
        bool ok = true;
        // one k-step: the F16 values `wv` of this thread go into stage s, then the warp arrives
        auto emit = [&](int ks, uint32_t (&wv)[16]) -> bool {
            const int s = ks % STAGES;
            const uint32_t round = (uint32_t) (ks / STAGES);
            if (ks >= STAGES && !mbar_wait_or_abort(smem_u32(&empty_bar[s]), (round - 1) & 1, &abort_flag)) return false;
            tc_fence_after();                                           // the tensor core has finished reading this stage
            if ((tid & (TC_GROUP - 1)) == 0) {                          // B: activations BN x 64 F16 by TMA (rows past N read as zero)
                mbar_arrive_expect_tx(&full_bar[s], BN * TC_BK * 2);
                tma_load_2d(smem + (size_t) s * STAGE_BYTES, &xmap, k_base + ks * TC_BK, n0, &full_bar[s]);
            }
            // A: this thread's 32 F16 weights are 16 columns of its row's lane in tensor memory (two values per column)
            tmem_st16(tmem_base + ((uint32_t) ((warp & 3) * 32) << 16) + A_COL0 + (uint32_t) (s * (TC_BK / 2) + h * 16), wv);
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&full_bar[s]);                   // one arrival per warp: 257 arrivals on one barrier serialise
            return true;
        };
        if constexpr (STAGED) if (p.staged) {
            // raw quant bytes arrive in shared memory, one 256-deep chunk (4 k-steps) of all 128 rows at a time
            pdl_wait();
            for (int c = 0; c * 4 < ksteps && ok; ++c) {
                const int buf = c % NRB;
                if (!mbar_wait_or_abort(smem_u32(&raw_full[buf]), (uint32_t) (c / NRB) & 1, &abort_flag)) { ok = false; break; }
                const uint8_t * rrow = rawbuf + (size_t) buf * RAW_BYTES + r * CB + (((k_base / TC_CHUNK_K + c) * TcChunk<T>::SRC) & 15);
                typename Deq32<T>::Raw raw;
#pragma unroll
                for (int uu = 0; uu < 2; ++uu) {
                    const int u = 2 * g + uu, ks = c * 4 + u;
                    if (ks >= ksteps || !ok) break;
                    uint32_t wv[16];
                    if (uu % KPR == 0) Deq32<T>::load_s(rrow, u * TC_BK + h * 32, raw);
                    if constexpr (KPR == 1) Deq32<T>::get(raw, wv); else Deq32<T>::get(raw, uu % KPR, wv);
                    if (!emit(ks, wv)) ok = false;
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&raw_empty[buf]);            // this warp has read the chunk
            }
        }
        if ((!STAGED || !p.staged) && g == 0) {
            // (one group only on this path) raw quant bytes of the next TC_PF k-steps are kept in flight in registers (HBM latency is several
            // k-steps long); weights do not depend on the previous kernel, so the first loads precede the wait
            constexpr int NRAW = TC_PF / KPR;
            typename Deq32<T>::Raw raw[NRAW];
#pragma unroll
            for (int u = 0; u < NRAW; ++u) if (u * KPR < ksteps) Deq32<T>::load(wrow, k_base + u * KPR * TC_BK + h * 32, raw[u]);
            pdl_wait();
            for (int ks0 = 0; ks0 < ksteps && ok; ks0 += TC_PF) {
#pragma unroll
                for (int u = 0; u < TC_PF; ++u) {
                    const int ks = ks0 + u;
                    if (ks >= ksteps || !ok) break;
                    uint32_t wv[16];
                    const int ru = u / KPR, sub = u % KPR;        // constants once the loop is unrolled
                    if constexpr (KPR == 1) Deq32<T>::get(raw[ru], wv); else Deq32<T>::get(raw[ru], sub, wv);
                    if (!wrow_ok) {                     // (this path reads row 0 in place of rows past M)
#pragma unroll
                        for (int i = 0; i < 16; ++i) wv[i] = 0;
                    }
                    // the Raw is free after its last k-step: refill it with the one NRAW pairs ahead
                    if (sub == KPR - 1 && ks + 1 + (NRAW - 1) * KPR < ksteps) Deq32<T>::load(wrow, k_base + (ks + 1 + (NRAW - 1) * KPR) * TC_BK + h * 32, raw[ru]);
                    if (!emit(ks, wv)) ok = false;
                }
            }
        }
        if (!ok && lane == 0) { atomicExch(p.status, ERR_MBAR_TIMEOUT); abort_flag = 1; }

        // ------------------------------ epilogue ------------------------------
        if (ok && mbar_wait(&accum_bar, 0)) {
            tc_fence_after();
            const int quad = warp & 3, cq = warp >> 2;                  // lane quadrant; which quarter of the BN columns
            const int m = m0 + quad * 32 + lane;
            // a whole tile goes to its place in the result, a K part to its partial tile [BN][128]
            char * out = is_split ? (char *) (p.part + (int64_t) (cta - p.n_direct) * TC_BM * BN) - (int64_t) n0 * TC_BM * 4 - (int64_t) m0 * 4
                                  : (char *) p.dst[mat];
            const int64_t out_nb1 = is_split ? (int64_t) TC_BM * 4 : p.dst_nb1[mat];
            const int n_end = is_split ? n0 + BN : (moe ? moe_row_end : p.N), m_end = is_split ? m0 + TC_BM : M;
#pragma unroll 1
            for (int c0 = cq * (BN / 4); c0 < cq * (BN / 4) + BN / 4; c0 += 32) {
                uint32_t v[32];
                tmem_ld32(tmem_base + ((uint32_t) (quad * 32) << 16) + (uint32_t) c0, v);
                tmem_ld_wait();
                if (m < m_end) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int n = n0 + c0 + i;
                        if (n < n_end) {
                            if (moe) *(float *) (out + p.moe_row_off[n] + (int64_t) m * 4) = __uint_as_float(v[i]);
                            else     *(float *) (out + (int64_t) n * out_nb1 + (int64_t) m * 4) = __uint_as_float(v[i]);
                        }
                    }
                }
            }
        } else if (ok && lane == 0) {
            atomicExch(p.status, ERR_MBAR_TIMEOUT);
        }
    } else if (warp == MMA_WARP) {
        // ------------------------------ MMA issuer ------------------------------
        // One thread runs this loop, and every k-step has to pass through it: it is kept to a wait, a fence, four
        // tcgen05.mma and a commit, with the stage's descriptors derived by one addition (the address field of a
        // shared-memory descriptor counts 16-byte units, and shared memory is smaller than the field).
        constexpr uint32_t idesc = umma_idesc_f16(TC_BM, BN);
        if (lane == 0) {
            bool ok = true;
            // every descriptor and address of the loop is a register set up here
            uint64_t bd[STAGES][TC_BK / 16];
            uint32_t ta[STAGES][TC_BK / 16];
#pragma unroll
            for (int s = 0; s < STAGES; ++s)
#pragma unroll
                for (int kk = 0; kk < TC_BK / 16; ++kk) {               // 16 K-elements: 8 columns of A, 32 bytes of B inside the 128-byte swizzle atom
                    bd[s][kk] = umma_smem_desc(smem_u32(smem) + s * STAGE_BYTES + kk * 32);
                    ta[s][kk] = tmem_base + A_COL0 + (uint32_t) (s * (TC_BK / 2) + 8 * kk);
                }
            const uint32_t full0 = smem_u32(&full_bar[0]), empty0 = smem_u32(&empty_bar[0]);
            uint32_t ph = 0, acc = 0;
            for (int ks0 = 0; ks0 < ksteps && ok; ks0 += STAGES, ph ^= 1) {
#pragma unroll
                for (int s = 0; s < STAGES; ++s) {
                    if (ks0 + s >= ksteps) break;
                    if (!mbar_wait_or_abort(full0 + 8 * s, ph, &abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    umma_f16_ts(tmem_base, ta[s][0], bd[s][0], idesc, acc);
                    acc = 1;
#pragma unroll
                    for (int kk = 1; kk < TC_BK / 16; ++kk) umma_f16_ts(tmem_base, ta[s][kk], bd[s][kk], idesc, 1);
                    umma_commit_addr(empty0 + 8 * s);                   // frees the stage once these MMAs have read it
                }
            }
            if (ok) umma_commit(&accum_bar);                            // accumulator complete
            else { atomicExch(p.status, ERR_MBAR_TIMEOUT); abort_flag = 1; }
        }
        __syncwarp();
    } else {
        // ------------------------------ loader ------------------------------
        // One tensor copy per chunk: the box is CB bytes (as 32-bit words) of 128 consecutive rows, laid down densely;
        // rows past M read as zero.  Weights do not depend on the kernel launched before this one, so the first
        // chunks are requested right away.
        if constexpr (STAGED) if (p.staged) {
            const int nchunks = (ksteps + 3) / 4;
            bool ok = true;
            if (lane == 0) {
                int c = 0;
                for (; c < nchunks; ++c) {
                    const int buf = c % NRB;
                    if (c >= NRB && !mbar_wait(&raw_empty[buf], (uint32_t) (c / NRB - 1) & 1)) { ok = false; break; }
                    if (*(volatile int *) &abort_flag) break;
                    mbar_arrive_expect_tx(&raw_full[buf], TC_BM * CB);
                    const int wx = (((k_base / TC_CHUNK_K + c) * TcChunk<T>::SRC) >> 4) * 4;
                    if (moe) tma_load_3d(rawbuf + (size_t) buf * RAW_BYTES, wmap, wx, m0, moe_expert, &raw_full[buf]);      // (the map then has the expert as third dimension)
                    else     tma_load_2d(rawbuf + (size_t) buf * RAW_BYTES, wmap, wx, m0, &raw_full[buf]);
                }
                if (!ok) { atomicExch(p.status, ERR_MBAR_TIMEOUT); abort_flag = 1; }
                // When the kernel gives up, the last copies of this thread may still be in flight: wait (bounded) for
                // each of them before the CTA's shared memory is released.  In a normal run the producers have waited
                // for every chunk.
                if (!ok || *(volatile int *) &abort_flag) {
                    for (int cc = max(0, c - NRB); cc < c; ++cc) mbar_wait(&raw_full[cc % NRB], (uint32_t) (cc / NRB) & 1);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == MMA_WARP) { tc_fence_after(); tmem_dealloc(tmem_base, TcCfg<BN>::TMEM_COLS); }
}

bool mmq_tc_supported(int type, int64_t M, int64_t N, int64_t K) {
    if (!mmvq_type_supported(type)) return false;
    // from 9 columns on; for large matrices already from 6 (measured: the dp4a mat-vec needs about 5 us per column on a
    // 4096 x 14336 matrix, the GEMM about 33 us for any column count up to 128)
    const bool wide_enough = N > 8 || (N >= 6 && M * K >= (int64_t) 32 << 20);
    return wide_enough && K % TC_BK == 0 && K >= TC_BK;
}
size_t mmq_tc_workspace_bytes(int64_t N, int64_t K) { return (size_t) N * K * 2 + 256; }
// the fast dequantizers read headers / nibble runs with aligned vector loads
bool mmq_tc_ptr_ok(int type, const void * W, int64_t w_nb1, const void * X, int64_t x_nb1) {
    if (((uintptr_t) X & 7) || (x_nb1 & 7)) return false;
    if (type == T_Q4_K || type == T_Q5_K) return ((uintptr_t) W & 15) == 0 && (w_nb1 & 15) == 0;
    return ((uintptr_t) W & 1) == 0 && (w_nb1 & 1) == 0;
}
// Raw blocks can be staged by tensor copies when whole 256-value chunks tile K, rows start on 16-byte boundaries and a
// row is a whole number of 32-bit words.
template <int T> static bool tc_can_stage(const TcParams & p) {
    if (TcChunk<T>::BYTES == 0 || p.K % TC_CHUNK_K) return false;
    const int64_t row_bytes = (int64_t) (p.K / TC_CHUNK_K) * TcChunk<T>::SRC;
    for (int j = 0; j < p.n_mats; ++j) if ((uintptr_t) p.W[j] & 15) return false;
    if (p.moe_tiles && (p.w_nb2 & 15)) return false;
    return (p.w_nb1 & 15) == 0 && (row_bytes & 3) == 0 && p.w_nb1 >= row_bytes;
}

// sums the K parts of the divided tiles in split order (deterministic) into their place in the result
template <int BN>
__global__ void tc_reduce_kernel(const TcParams p, int n_split_tiles) {
    pdl_enter();
    const int64_t per_tile = (int64_t) TC_BM * BN, total = per_tile * n_split_tiles;
    for (int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t) gridDim.x * blockDim.x) {
        const int r = (int) (i / per_tile);
        const int e = (int) (i - (int64_t) r * per_tile), nl = e / TC_BM, ml = e - nl * TC_BM;
        const int tile = p.n_direct + r, mt = tile / p.n_tiles_n, n = (tile - mt * p.n_tiles_n) * BN + nl;
        const int mat = (p.n_mats > 2 && mt >= p.mt0[2]) ? 2 : ((p.n_mats > 1 && mt >= p.mt0[1]) ? 1 : 0);
        const int m = (mt - p.mt0[mat]) * TC_BM + ml;
        if (n >= p.N || m >= p.M[mat]) continue;
        const float * src = p.part + (int64_t) r * p.ksplit * per_tile + e;
        float acc = src[0];
        for (int z = 1; z < p.ksplit; ++z) acc += src[(int64_t) z * per_tile];
        *(float *) ((char *) p.dst[mat] + (int64_t) n * p.dst_nb1[mat] + (int64_t) m * 4) = acc;
    }
}

// How a product of `m_tiles` 128-row tiles by N tokens is laid over the SMs.  The K range of a tile is divided over several
// CTAs where whole tiles would leave SMs idle: every tile of a small output, or the tiles left over after the last full
// wave of a large one (a part keeps at least 8 k-steps, and whole 256-value chunks).
struct TcPlan { int bn, n_tiles_n, tiles, n_direct, ksplit, kps; double cost; };
static TcPlan tc_plan_bn(int bn, int64_t m_tiles, int64_t N, int64_t K, int sm_count, bool allow_split) {
    TcPlan pl;
    pl.bn = bn; pl.n_tiles_n = (int) ((N + bn - 1) / bn); pl.tiles = (int) (m_tiles * pl.n_tiles_n);
    const int ksteps = (int) (K / TC_BK);
    const int full = pl.tiles / sm_count * sm_count, rest = pl.tiles - full;
    int s = 1;
    if (allow_split && rest > 0 && rest * 4 < sm_count * 3) {
        s = sm_count / rest; if (s > 8) s = 8;
        while (s > 1 && ksteps / s < 8) --s;
    }
    pl.kps = ((ksteps + s - 1) / s + 3) & ~3;
    pl.ksplit = (ksteps + pl.kps - 1) / pl.kps;
    if (pl.ksplit < 2) { pl.ksplit = 1; pl.kps = ksteps; pl.n_direct = pl.tiles; }
    else pl.n_direct = full;
    // estimated time in microseconds, from measurements on B200: a k-step of a CTA (a 128-token tile is bound by the issue
    // rate of its MMAs, not by their size), a fixed part per wave (set-up, accumulator read-out), and what dividing K adds
    // (partial tiles written and read back, the summation launch)
    const double t_k = bn == 256 ? 0.47 : 0.45, fixed = 6.0, split_extra = 15.0;
    pl.cost = (pl.n_direct + sm_count - 1) / sm_count * (ksteps * t_k + fixed);
    if (pl.ksplit > 1) pl.cost += pl.kps * t_k + fixed + split_extra;
    return pl;
}
static TcPlan tc_plan(int64_t m_tiles, int64_t N, int64_t K, int sm_count, bool allow_split) {
    const char * e_bn = getenv("GGML_B200_TC_BN"), * e_ns = getenv("GGML_B200_TC_NO_SPLIT");            // tuning and test aids (read per call)
    const int force_bn = e_bn ? atoi(e_bn) : 0, no_tail = e_ns ? atoi(e_ns) : 0;
    if (no_tail) allow_split = false;
    const TcPlan a = tc_plan_bn(128, m_tiles, N, K, sm_count, allow_split);
    if (N < 256 || force_bn == 128) return a;
    const TcPlan b = tc_plan_bn(256, m_tiles, N, K, sm_count, allow_split);
    return (force_bn == 256 || b.cost <= a.cost) ? b : a;
}
static int64_t m_tiles_of(int n_mats, const int64_t * M) {
    int64_t t = 0;
    for (int j = 0; j < n_mats; ++j) t += (M[j] + TC_BM - 1) / TC_BM;
    return t;
}
size_t mmq_tc_group_partial_bytes(int n_mats, const int64_t * M, int64_t N, int64_t K, int sm_count) {
    const TcPlan pl = tc_plan(m_tiles_of(n_mats, M), N, K, sm_count, true);
    return pl.ksplit > 1 ? (size_t) (pl.tiles - pl.n_direct) * pl.ksplit * TC_BM * pl.bn * 4 + 256 : 0;
}
size_t mmq_tc_partial_bytes(int64_t M, int64_t N, int64_t K, int sm_count) { return mmq_tc_group_partial_bytes(1, &M, N, K, sm_count); }

template <int T, int BN>
static cudaError_t launch_tc_tb(const TcParams & p_in, int device, int use_pdl, cudaStream_t stream) {
    auto kern = mmq_tc_kernel<T, BN>;
    const size_t smem = TcCfg<BN>::template smem_bytes<T>();
    static unsigned attr_mask = 0;
    if (!(attr_mask & (1u << device))) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem);
        if (e != cudaSuccess) return e;
        attr_mask |= 1u << device;
    }
    // tensor map of the F16 activations [N][K]: boxes of 64 (k) x BN (tokens), 128-byte swizzle, zero fill
    encode_tiled_fn enc = get_encode_tiled();
    if (!enc) return cudaErrorNotSupported;
    TcParams p = p_in;
    p.staged = tc_can_stage<T>(p) ? 1 : 0;
    CUtensorMap xmap;
    const cuuint64_t gdim[2] = {(cuuint64_t) p.K, (cuuint64_t) p.N};
    const cuuint64_t gstr[1] = {(cuuint64_t) p.K * 2};
    const cuuint32_t box[2] = {TC_BK, BN}, estr[2] = {1, 1};
    if (enc(&xmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void *) p.Xh, gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return cudaErrorInvalidValue;
    // per matrix, a tensor map of the raw weight rows as 32-bit words [M][row bytes / 4]: boxes of one 256-value chunk x 128 rows
    CUtensorMap wmap[TC_MAX_MATS] = {xmap, xmap, xmap};
    if (p.staged && p.moe_tiles) {
        // the experts' matrices as one [row words][M][expert] tensor
        constexpr cuuint32_t CW = TcChunk<T>::BYTES / 4;
        const cuuint64_t wdim[3] = {(cuuint64_t) (p.K / TC_CHUNK_K) * TcChunk<T>::SRC / 4, (cuuint64_t) p.M[0], (cuuint64_t) p.moe_n_expert};
        const cuuint64_t wstr[2] = {(cuuint64_t) p.w_nb1, (cuuint64_t) p.w_nb2};
        const cuuint32_t wbox[3] = {CW, TC_BM, 1}, estr3[3] = {1, 1, 1};
        if (enc(&wmap[0], CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, (void *) p.W[0], wdim, wstr, wbox, estr3, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    } else if (p.staged) for (int j = 0; j < p.n_mats; ++j) {
        constexpr cuuint32_t CW = TcChunk<T>::BYTES / 4;
        const cuuint64_t wdim[2] = {(cuuint64_t) (p.K / TC_CHUNK_K) * TcChunk<T>::SRC / 4, (cuuint64_t) p.M[j]};
        const cuuint64_t wstr[1] = {(cuuint64_t) p.w_nb1};
        const cuuint32_t wbox[2] = {CW, TC_BM};
        if (enc(&wmap[j], CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, (void *) p.W[j], wdim, wstr, wbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    if (p.moe_tiles) {
        // the tables are written by the kernel launched just before: no early start
        const unsigned g = (unsigned) (p.moe_nt_max * p.mt0[p.n_mats]);
        return launch_k(0, stream, kern, dim3(g), dim3(TC_THREADS), smem, p, xmap, wmap[0], wmap[1], wmap[2]);
    }
    const int n_split_tiles = p.mt0[p.n_mats] * p.n_tiles_n - p.n_direct;
    const unsigned grid = (unsigned) (p.n_direct + n_split_tiles * (p.ksplit > 1 ? p.ksplit : 0));
    cudaError_t e = launch_k(use_pdl, stream, kern, dim3(grid), dim3(TC_THREADS), smem, p, xmap, wmap[0], wmap[1], wmap[2]);
    if (e != cudaSuccess || p.ksplit == 1) return e;
    const int64_t total = (int64_t) n_split_tiles * TC_BM * BN;
    int64_t g = (total + 255) / 256; if (g > 148 * 8) g = 148 * 8;
    return launch_k(use_pdl, stream, tc_reduce_kernel<BN>, dim3((unsigned) g), dim3(256), 0, p, n_split_tiles);
}

template <int T>
static cudaError_t launch_tc_t(const TcParams & p, int bn, int device, int use_pdl, cudaStream_t stream) {
    if (bn == 256) return launch_tc_tb<T, 256>(p, device, use_pdl, stream);
    return launch_tc_tb<T, TC_BN>(p, device, use_pdl, stream);
}

// ---- MUL_MAT_ID over many (slot, token) pairs ------------------------------------------------------------------------
// Sorts the pairs by expert (one CTA; every pair's place is found by the thread of its expert walking the pairs in order, so
// the result does not depend on timing), lists the token tiles and records where each sorted row's result goes.
__global__ void __launch_bounds__(1024) tc_moe_sort_kernel(const int32_t * ids, int64_t ids_s1 /*elements between tokens*/, int n_used, int n_tok, int n_expert,
                                                           int bn, int64_t dst_nb1, int64_t dst_nb2, int * row_pair, int64_t * row_off, int4 * tiles, int * n_tiles) {
    pdl_enter();
    extern __shared__ int sh[];                                     // counts[n_expert], offsets[n_expert + 1]
    int * counts = sh, * off = sh + n_expert;
    const int P = n_used * n_tok;
    for (int e = threadIdx.x; e < n_expert; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < P; p += blockDim.x) {
        const int e = ids[(int64_t) (p / n_used) * ids_s1 + p % n_used];
        if (e >= 0 && e < n_expert) atomicAdd(&counts[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int acc = 0, t = 0;
        for (int e = 0; e < n_expert; ++e) {
            off[e] = acc;
            for (int r0 = acc; r0 < acc + counts[e]; r0 += bn) tiles[t++] = make_int4(e, r0, min(acc + counts[e], r0 + bn), 0);
            acc += counts[e];
        }
        off[n_expert] = acc;
        *n_tiles = t;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n_expert; e += blockDim.x) {
        int r = off[e];
        for (int p = 0; p < P; ++p) {
            const int it = p / n_used, iu = p - it * n_used;
            if (ids[(int64_t) it * ids_s1 + iu] != e) continue;
            row_pair[r] = p;
            row_off[r] = (int64_t) iu * dst_nb1 + (int64_t) it * dst_nb2;
            ++r;
        }
    }
}
// activations of the sorted rows as F16: row r = column (slot iu % ne11, token it) of src1
__global__ void tc_moe_gather_kernel(const char * __restrict__ x, int64_t x_nb1, int64_t x_nb2, int ne11, int n_used, const int * __restrict__ row_pair,
                                     __half * __restrict__ y, int64_t K, int64_t P) {
    pdl_enter();
    const int64_t total = P * K / 2;
    for (int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t) gridDim.x * blockDim.x) {
        const int64_t r = (2 * i) / K, k = (2 * i) % K;
        const int p = row_pair[r], it = p / n_used, iu = p - it * n_used;
        const float2 v = *(const float2 *) (x + (int64_t) (iu % ne11) * x_nb1 + (int64_t) it * x_nb2 + k * 4);
        ((__half2 *) y)[i] = __floats2half2_rn(v.x, v.y);
    }
}

static size_t moe_align(size_t v) { return (v + 255) & ~(size_t) 255; }
bool mmq_tc_moe_supported(int type, int64_t M, int64_t K, int64_t n_expert, int64_t n_pairs) {
    return mmq_tc_supported(type, M, n_pairs > 8 ? n_pairs : 9, K) && n_expert >= 1 && n_expert <= 1024 && n_pairs >= 1 && n_pairs <= (1 << 20);
}
size_t mmq_tc_moe_workspace_bytes(int64_t n_pairs, int64_t K, int64_t n_expert) {
    const int64_t nt_max = (n_pairs + TC_BN - 1) / TC_BN + n_expert;
    return moe_align((size_t) n_pairs * K * 2) + moe_align((size_t) n_pairs * 4) + moe_align((size_t) n_pairs * 8) + moe_align((size_t) nt_max * 16) + 256 + 256;
}
template <int T> static cudaError_t launch_moe_t(const TcParams & p, const LaunchCtx & c) { return launch_tc_tb<T, TC_BN>(p, c.device, 0, c.stream); }

// dst[:, iu, it] = W[:, :, ids[iu, it]] x src1[:, iu % ne11, it] for all pairs at once (ggml_mul_mat_id, ggml/src/ggml.c:2735-2759;
// the reference sorts on the host after copying ids back, ggml/src/ggml-cuda/ggml-cuda.cu:1956-2092; here nothing leaves the device)
cudaError_t launch_mmq_tc_moe(int type, const void * W, int64_t w_nb1, int64_t w_nb2, int64_t n_expert, int64_t M, int64_t K,
                              const float * X, int64_t x_nb1, int64_t x_nb2, int64_t ne11,
                              const int32_t * ids, int64_t ids_nb1, int64_t n_used, int64_t n_tok,
                              float * dst, int64_t dst_nb1, int64_t dst_nb2, void * workspace, const LaunchCtx & c) {
    const int64_t P = n_used * n_tok;
    const int nt_max = (int) ((P + TC_BN - 1) / TC_BN + n_expert);
    char * ws = (char *) workspace;
    __half * xh = (__half *) ws;                 ws += moe_align((size_t) P * K * 2);
    int * row_pair = (int *) ws;                 ws += moe_align((size_t) P * 4);
    int64_t * row_off = (int64_t *) ws;          ws += moe_align((size_t) P * 8);
    int4 * tiles = (int4 *) ws;                  ws += moe_align((size_t) nt_max * 16);
    int * n_tiles = (int *) ws;
    cudaError_t e = launch_k(c.use_pdl, c.stream, tc_moe_sort_kernel, dim3(1), dim3(1024), (size_t) (2 * n_expert + 1) * sizeof(int), ids, ids_nb1 / 4,
                             (int) n_used, (int) n_tok, (int) n_expert, (int) TC_BN, dst_nb1, dst_nb2, row_pair, row_off, tiles, n_tiles);
    if (e != cudaSuccess) return e;
    {
        const int64_t total = P * K / 2;
        int64_t g = (total + 255) / 256; if (g > (int64_t) c.sm_count * 8) g = (int64_t) c.sm_count * 8;
        e = launch_k(c.use_pdl, c.stream, tc_moe_gather_kernel, dim3((unsigned) g), dim3(256), 0, (const char *) X, x_nb1, x_nb2, (int) ne11, (int) n_used,
                     (const int *) row_pair, xh, K, P);
        if (e != cudaSuccess) return e;
    }
    TcParams p = {};
    p.n_mats = 1; p.w_nb1 = w_nb1; p.Xh = xh; p.N = (int) P; p.K = (int) K; p.status = c.status;
    p.W[0] = (const uint8_t *) W; p.dst[0] = dst; p.dst_nb1[0] = dst_nb1; p.M[0] = (int) M;
    p.mt0[0] = 0; for (int j = 1; j <= TC_MAX_MATS; ++j) p.mt0[j] = (int) ((M + TC_BM - 1) / TC_BM);
    p.n_tiles_n = 1; p.n_direct = 1 << 30; p.ksplit = 1; p.kps = (int) (K / TC_BK); p.part = nullptr;
    p.moe_tiles = tiles; p.moe_n_tiles = n_tiles; p.moe_row_off = row_off; p.moe_nt_max = nt_max; p.moe_n_expert = (int) n_expert; p.w_nb2 = w_nb2;
    switch (type) {
        case T_Q4_0: return launch_moe_t<T_Q4_0>(p, c);
        case T_Q4_1: return launch_moe_t<T_Q4_1>(p, c);
        case T_Q5_0: return launch_moe_t<T_Q5_0>(p, c);
        case T_Q5_1: return launch_moe_t<T_Q5_1>(p, c);
        case T_Q8_0: return launch_moe_t<T_Q8_0>(p, c);
        case T_Q4_K: return launch_moe_t<T_Q4_K>(p, c);
        case T_Q5_K: return launch_moe_t<T_Q5_K>(p, c);
        case T_Q6_K: return launch_moe_t<T_Q6_K>(p, c);
        case T_Q2_K: return launch_moe_t<T_Q2_K>(p, c);
        case T_Q3_K: return launch_moe_t<T_Q3_K>(p, c);
        case T_IQ4_NL: return launch_moe_t<T_IQ4_NL>(p, c);
        case T_IQ4_XS: return launch_moe_t<T_IQ4_XS>(p, c);
    }
    return cudaErrorInvalidValue;
}

cudaError_t launch_mmq_tc_group(int type, int n_mats, const void * const * W, int64_t w_nb1, const int64_t * M, float * const * dst,
                                const int64_t * dst_nb1, const float * X, int64_t x_nb1, int64_t N, int64_t K, void * workspace,
                                const LaunchCtx & c, bool preconverted, void * partials) {
    if (n_mats < 1 || n_mats > TC_MAX_MATS) return cudaErrorInvalidValue;
    __half * xh = (__half *) workspace;
    if (!preconverted) {                 // (the caller may keep the F16 copy of X for the next mat-mul on the same activations)
        const int64_t total = N * K / 2;
        int64_t g = (total + 255) / 256; if (g > (int64_t) c.sm_count * 8) g = (int64_t) c.sm_count * 8;
        cudaError_t e = launch_k(c.use_pdl, c.stream, tc_convert_x_kernel, dim3((unsigned) g), dim3(256), 0, X, x_nb1, xh, K, N);
        if (e != cudaSuccess) return e;
    }
    TcParams p = {};
    p.n_mats = n_mats; p.w_nb1 = w_nb1; p.Xh = xh; p.N = (int) N; p.K = (int) K; p.status = c.status;
    int mt = 0;
    for (int j = 0; j < n_mats; ++j) {
        p.W[j] = (const uint8_t *) W[j]; p.dst[j] = dst[j]; p.dst_nb1[j] = dst_nb1[j]; p.M[j] = (int) M[j];
        p.mt0[j] = mt; mt += (int) ((M[j] + TC_BM - 1) / TC_BM);
    }
    for (int j = n_mats; j <= TC_MAX_MATS; ++j) p.mt0[j] = mt;
    const TcPlan pl = tc_plan(mt, N, K, c.sm_count, partials != nullptr);
    p.n_tiles_n = pl.n_tiles_n; p.n_direct = pl.n_direct; p.ksplit = pl.ksplit; p.kps = pl.kps;
    p.part = (float *) partials;
    switch (type) {
        case T_Q4_0: return launch_tc_t<T_Q4_0>(p, pl.bn, c.device, c.use_pdl, c.stream);
        case T_Q4_1: return launch_tc_t<T_Q4_1>(p, pl.bn, c.device, c.use_pdl, c.stream);
        case T_Q5_0: return launch_tc_t<T_Q5_0>(p, pl.bn, c.device, c.use_pdl, c.stream);
        case T_Q5_1: return launch_tc_t<T_Q5_1>(p, pl.bn, c.device, c.use_pdl, c.stream);
        case T_Q8_0: return launch_tc_t<T_Q8_0>(p, pl.bn, c.device, c.use_pdl, c.stream);
        case T_Q4_K: return launch_tc_t<T_Q4_K>(p, pl.bn, c.device, c.use_pdl, c.stream);
        case T_Q5_K: return launch_tc_t<T_Q5_K>(p, pl.bn, c.device, c.use_pdl, c.stream);
        case T_Q6_K: return launch_tc_t<T_Q6_K>(p, pl.bn, c.device, c.use_pdl, c.stream);
        case T_Q2_K: return launch_tc_t<T_Q2_K>(p, pl.bn, c.device, c.use_pdl, c.stream);
        case T_Q3_K: return launch_tc_t<T_Q3_K>(p, pl.bn, c.device, c.use_pdl, c.stream);
        case T_IQ4_NL: return launch_tc_t<T_IQ4_NL>(p, pl.bn, c.device, c.use_pdl, c.stream);
        case T_IQ4_XS: return launch_tc_t<T_IQ4_XS>(p, pl.bn, c.device, c.use_pdl, c.stream);
    }
    return cudaErrorInvalidValue;
}
cudaError_t launch_mmq_tc(int type, const void * W, int64_t w_nb1, const float * X, int64_t x_nb1, float * dst, int64_t dst_nb1,
                          int64_t M, int64_t N, int64_t K, void * workspace, const LaunchCtx & c, bool preconverted, void * partials) {
    return launch_mmq_tc_group(type, 1, &W, w_nb1, &M, &dst, &dst_nb1, X, x_nb1, N, K, workspace, c, preconverted, partials);
}

}  // namespace b200
