// Decode-time quantized mat-vec / skinny mat-mat (1..8 activation columns).
//
//   dst[col][row] = sum_k W[row][k] * X[col][k]
//
// Replaces, for the B200, the reference's separate quantize_q8_1 +
// mul_mat_vec_q launches (ggml/src/ggml-cuda/quantize.cu:4-38,
// ggml/src/ggml-cuda/mmvq.cu:50-130) and restates the integer-dot arithmetic of
// ggml/src/ggml-cuda/vecdotq.cuh per weight type.  The kernel is HBM-bound, so
// the design is about bytes in flight rather than math:
//
//  * the weight matrix is streamed as raw quant bytes by one producer warp using
//    plain (non-multicast) cp.async.bulk copies into a multi-stage shared-memory
//    ring, completed on mbarriers; quant blocks of 18/34/210 bytes are only
//    2-byte aligned, so a row segment is copied from its 16-byte-aligned
//    superset and indexed from the remainder in shared memory;
//  * eight consumer warps take one weight row each per tile, unpack nibbles and
//    run dp4a against int8 activations, and reduce with warp shuffles;
//  * weight copies for the first stages are issued before griddepcontrol.wait,
//    so under programmatic dependent launch they overlap the previous kernel.
//
// Every mbarrier wait is bounded; on expiry the kernel records ERR_MBAR_TIMEOUT
// in the status word and drains instead of spinning.
#include "common.cuh"
#include "kernels.h"

namespace b200 {

// ---------------------------------------------------------------------------
// activation quantizer: F32 column (contiguous along k) -> blk_act128
// one warp per 128 values; 8 lanes share one 32-value group
// ---------------------------------------------------------------------------
__global__ void quantize_act128_kernel(const float * __restrict__ x, int64_t ne11, int64_t ne12,
                                       int64_t s11, int64_t s12, int64_t s13 /* element strides of dims 1,2,3 */,
                                       blk_act128 * __restrict__ y, int K, int nblk /*per column*/, int64_t ncols) {
    pdl_enter();
    const int64_t gw   = (int64_t) blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int     lane = threadIdx.x & 31;
    if (gw >= ncols * nblk) return;
    const int64_t col = gw / nblk;                 // columns are ordered [i13][i12][i11]
    const int     b   = (int) (gw - col * nblk);
    const int64_t i11 = col % ne11, i12 = (col / ne11) % ne12, i13 = col / (ne11 * ne12);
    const float * xc  = x + i11 * s11 + i12 * s12 + i13 * s13;
    const int     k0  = b * 128 + lane * 4;

    float v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = (k0 + i < K) ? xc[k0 + i] : 0.0f;
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float d  = amax / 127.0f;
    const float id = amax > 0.0f ? 127.0f / amax : 0.0f;
    int q[4], qsum = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) { q[i] = __float2int_rn(v[i] * id); qsum += q[i]; }
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) qsum += __shfl_xor_sync(0xffffffffu, qsum, o);
    blk_act128 * yb = y + col * nblk + b;
    const uint32_t packed = (uint32_t) (q[0] & 0xff) | ((uint32_t) (q[1] & 0xff) << 8) |
                            ((uint32_t) (q[2] & 0xff) << 16) | ((uint32_t) (q[3] & 0xff) << 24);
    ((uint32_t *) yb->q)[lane] = packed;
    if ((lane & 7) == 0) yb->ds[lane >> 3] = make_float2(d, d * (float) qsum);
}

// ---------------------------------------------------------------------------
// per-type integer dot products on one "unit" of a weight row held in smem
// ---------------------------------------------------------------------------
// A view of the activation chunk in shared memory: column n starts at
// base + n*col_bytes and holds consecutive blk_act128 starting at the chunk's k0.
struct ActView {
    const uint8_t * base;
    int col_bytes;
    __device__ __forceinline__ const int * q32(int n, int g32) const {   // 8 ints of 32-value group g32
        return (const int *) (base + n * col_bytes + (g32 >> 2) * 160 + (g32 & 3) * 32);
    }
    __device__ __forceinline__ float2 ds(int n, int g32) const {
        return *(const float2 *) (base + n * col_bytes + (g32 >> 2) * 160 + 128 + (g32 & 3) * 8);
    }
};

// 32-bit load from shared memory at 2-byte alignment
__device__ __forceinline__ uint32_t lds_u32_a2(const uint8_t * p) {
    const uint16_t * h = (const uint16_t *) p;
    return (uint32_t) h[0] | ((uint32_t) h[1] << 16);
}
// NW consecutive 32-bit words starting at a 2-byte aligned shared-memory address: NW+1 aligned
// loads and a funnel shift each instead of 2*NW 16-bit loads (the slot keeps 16 bytes of slack)
template <int NW>
__device__ __forceinline__ void lds_words(const uint8_t * p, uint32_t (&out)[NW]) {
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

template <int T> struct WT;   // weight-type traits: UNIT = weights per unit, dot() accumulates one unit

template <> struct WT<T_Q4_0> {
    static constexpr int UNIT = 32, BLK_ELEMS = 32, BLK_BYTES = 18;
    template <int N> static __device__ __forceinline__ void dot(const uint8_t * row, int u, const ActView & xv, float (&acc)[N]) {
        const uint8_t * b = row + u * 18;
        const float dw = h2f(*(const uint16_t *) b);
        uint32_t w[4], lo[4], hi[4];
        lds_words<4>(b + 2, w);
#pragma unroll
        for (int i = 0; i < 4; ++i) { lo[i] = w[i] & 0x0F0F0F0Fu; hi[i] = (w[i] >> 4) & 0x0F0F0F0Fu; }
#pragma unroll
        for (int n = 0; n < N; ++n) {
            const int * xq = xv.q32(n, u);
            int s = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) { s = __dp4a((int) lo[i], xq[i], s); s = __dp4a((int) hi[i], xq[i + 4], s); }
            const float2 ds = xv.ds(n, u);
            acc[n] += dw * ((float) s * ds.x - 8.0f * ds.y);
        }
    }
};

template <> struct WT<T_Q4_1> {
    static constexpr int UNIT = 32, BLK_ELEMS = 32, BLK_BYTES = 20;
    template <int N> static __device__ __forceinline__ void dot(const uint8_t * row, int u, const ActView & xv, float (&acc)[N]) {
        const uint8_t * b = row + u * 20;
        const float dw = h2f(*(const uint16_t *) b), mw = h2f(*(const uint16_t *) (b + 2));
        uint32_t lo[4], hi[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t w = lds_u32_a2(b + 4 + 4 * i);
            lo[i] = w & 0x0F0F0F0Fu; hi[i] = (w >> 4) & 0x0F0F0F0Fu;
        }
#pragma unroll
        for (int n = 0; n < N; ++n) {
            const int * xq = xv.q32(n, u);
            int s = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) { s = __dp4a((int) lo[i], xq[i], s); s = __dp4a((int) hi[i], xq[i + 4], s); }
            const float2 ds = xv.ds(n, u);
            acc[n] += dw * (float) s * ds.x + mw * ds.y;
        }
    }
};

// expands the 5th bits of Q5_0/Q5_1 (bit j of qh belongs to element j) into byte lanes
__device__ __forceinline__ uint32_t spread4(uint32_t bits4) {   // 4 low bits -> 0x10 in each byte
    return ((bits4 & 1) << 4) | ((bits4 & 2) << 11) | ((bits4 & 4) << 18) | ((bits4 & 8) << 25);
}

template <> struct WT<T_Q5_0> {
    static constexpr int UNIT = 32, BLK_ELEMS = 32, BLK_BYTES = 22;
    template <int N> static __device__ __forceinline__ void dot(const uint8_t * row, int u, const ActView & xv, float (&acc)[N]) {
        const uint8_t * b = row + u * 22;
        const float dw = h2f(*(const uint16_t *) b);
        const uint32_t qh = lds_u32_a2(b + 2);
        uint32_t lo[4], hi[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t w = lds_u32_a2(b + 6 + 4 * i);
            lo[i] = (w & 0x0F0F0F0Fu)        | spread4(qh >> (4 * i));
            hi[i] = ((w >> 4) & 0x0F0F0F0Fu) | spread4(qh >> (16 + 4 * i));
        }
#pragma unroll
        for (int n = 0; n < N; ++n) {
            const int * xq = xv.q32(n, u);
            int s = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) { s = __dp4a((int) lo[i], xq[i], s); s = __dp4a((int) hi[i], xq[i + 4], s); }
            const float2 ds = xv.ds(n, u);
            acc[n] += dw * ((float) s * ds.x - 16.0f * ds.y);
        }
    }
};

template <> struct WT<T_Q5_1> {
    static constexpr int UNIT = 32, BLK_ELEMS = 32, BLK_BYTES = 24;
    template <int N> static __device__ __forceinline__ void dot(const uint8_t * row, int u, const ActView & xv, float (&acc)[N]) {
        const uint8_t * b = row + u * 24;
        const float dw = h2f(*(const uint16_t *) b), mw = h2f(*(const uint16_t *) (b + 2));
        const uint32_t qh = lds_u32_a2(b + 4);
        uint32_t lo[4], hi[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t w = lds_u32_a2(b + 8 + 4 * i);
            lo[i] = (w & 0x0F0F0F0Fu)        | spread4(qh >> (4 * i));
            hi[i] = ((w >> 4) & 0x0F0F0F0Fu) | spread4(qh >> (16 + 4 * i));
        }
#pragma unroll
        for (int n = 0; n < N; ++n) {
            const int * xq = xv.q32(n, u);
            int s = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) { s = __dp4a((int) lo[i], xq[i], s); s = __dp4a((int) hi[i], xq[i + 4], s); }
            const float2 ds = xv.ds(n, u);
            acc[n] += dw * (float) s * ds.x + mw * ds.y;
        }
    }
};

template <> struct WT<T_Q8_0> {
    static constexpr int UNIT = 32, BLK_ELEMS = 32, BLK_BYTES = 34;
    template <int N> static __device__ __forceinline__ void dot(const uint8_t * row, int u, const ActView & xv, float (&acc)[N]) {
        const uint8_t * b = row + u * 34;
        const float dw = h2f(*(const uint16_t *) b);
        uint32_t wu[8];
        lds_words<8>(b + 2, wu);
        int w[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) w[i] = (int) wu[i];
#pragma unroll
        for (int n = 0; n < N; ++n) {
            const int * xq = xv.q32(n, u);
            int s = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) s = __dp4a(w[i], xq[i], s);
            acc[n] += dw * xv.ds(n, u).x * (float) s;
        }
    }
};

// Q4_K / Q5_K: a unit is one 32-byte run of qs = 64 weights: low nibbles are
// sub-block 2j, high nibbles sub-block 2j+1 (ggml-quants.c:1280-1302).
template <> struct WT<T_Q4_K> {
    static constexpr int UNIT = 64, BLK_ELEMS = 256, BLK_BYTES = 144;
    template <int N> static __device__ __forceinline__ void dot(const uint8_t * row, int u, const ActView & xv, float (&acc)[N]) {
        const uint8_t * b = row + (u >> 2) * 144;
        const int j = u & 3;
        const float d = h2f(*(const uint16_t *) b), dmin = h2f(*(const uint16_t *) (b + 2));
        int sc0, m0, sc1, m1;
        k4_scale_min(2 * j, b + 4, sc0, m0);
        k4_scale_min(2 * j + 1, b + 4, sc1, m1);
        uint32_t lo[8], hi[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t w = lds_u32_a2(b + 16 + 32 * j + 4 * i);
            lo[i] = w & 0x0F0F0F0Fu; hi[i] = (w >> 4) & 0x0F0F0F0Fu;
        }
        const int g = (u >> 2) * 8 + 2 * j;   // first 32-value activation group
#pragma unroll
        for (int n = 0; n < N; ++n) {
            const int * x0 = xv.q32(n, g);
            const int * x1 = xv.q32(n, g + 1);
            int s0 = 0, s1 = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) { s0 = __dp4a((int) lo[i], x0[i], s0); s1 = __dp4a((int) hi[i], x1[i], s1); }
            const float2 a0 = xv.ds(n, g), a1 = xv.ds(n, g + 1);
            acc[n] += d * ((float) (sc0 * s0) * a0.x + (float) (sc1 * s1) * a1.x)
                    - dmin * ((float) m0 * a0.y + (float) m1 * a1.y);
        }
    }
};

template <> struct WT<T_Q5_K> {
    static constexpr int UNIT = 64, BLK_ELEMS = 256, BLK_BYTES = 176;
    template <int N> static __device__ __forceinline__ void dot(const uint8_t * row, int u, const ActView & xv, float (&acc)[N]) {
        const uint8_t * b = row + (u >> 2) * 176;
        const int j = u & 3;
        const float d = h2f(*(const uint16_t *) b), dmin = h2f(*(const uint16_t *) (b + 2));
        int sc0, m0, sc1, m1;
        k4_scale_min(2 * j, b + 4, sc0, m0);
        k4_scale_min(2 * j + 1, b + 4, sc1, m1);
        uint32_t lo[8], hi[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t w  = lds_u32_a2(b + 48 + 32 * j + 4 * i);
            const uint32_t qh = lds_u32_a2(b + 16 + 4 * i) >> (2 * j);     // bit 0: sub-block 2j, bit 1: 2j+1
            lo[i] = (w & 0x0F0F0F0Fu)        | ((qh << 4) & 0x10101010u);
            hi[i] = ((w >> 4) & 0x0F0F0F0Fu) | ((qh << 3) & 0x10101010u);
        }
        const int g = (u >> 2) * 8 + 2 * j;
#pragma unroll
        for (int n = 0; n < N; ++n) {
            const int * x0 = xv.q32(n, g);
            const int * x1 = xv.q32(n, g + 1);
            int s0 = 0, s1 = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) { s0 = __dp4a((int) lo[i], x0[i], s0); s1 = __dp4a((int) hi[i], x1[i], s1); }
            const float2 a0 = xv.ds(n, g), a1 = xv.ds(n, g + 1);
            acc[n] += d * ((float) (sc0 * s0) * a0.x + (float) (sc1 * s1) * a1.x)
                    - dmin * ((float) m0 * a0.y + (float) m1 * a1.y);
        }
    }
};

// Q6_K: a unit is 8 consecutive l-positions of one 128-half: 2 words of
// ql[l], ql[l+32] and qh[l] give 32 weights in four 32-value activation groups
// (ggml-quants.c:1690-1719).
template <> struct WT<T_Q6_K> {
    static constexpr int UNIT = 32, BLK_ELEMS = 256, BLK_BYTES = 210;
    template <int N> static __device__ __forceinline__ void dot(const uint8_t * row, int u, const ActView & xv, float (&acc)[N]) {
        const uint8_t * b = row + (u >> 3) * 210;
        const int n128 = (u >> 2) & 1, g8 = u & 3;
        const float d = h2f(*(const uint16_t *) (b + 208));
        const int8_t * sc = (const int8_t *) (b + 192) + n128 * 8 + (g8 >> 1);
        int q[4][2];
        uint32_t Aw[2], Bw[2], Hw[2];
        lds_words<2>(b + n128 * 64 + g8 * 8, Aw);
        lds_words<2>(b + n128 * 64 + 32 + g8 * 8, Bw);
        lds_words<2>(b + 128 + n128 * 32 + g8 * 8, Hw);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const uint32_t A = Aw[i], B = Bw[i], H = Hw[i];
            q[0][i] = (int) __vsubss4((A & 0x0F0F0F0Fu)        | ((H << 4) & 0x30303030u), 0x20202020u);
            q[1][i] = (int) __vsubss4((B & 0x0F0F0F0Fu)        | ((H << 2) & 0x30303030u), 0x20202020u);
            q[2][i] = (int) __vsubss4(((A >> 4) & 0x0F0F0F0Fu) | ( H       & 0x30303030u), 0x20202020u);
            q[3][i] = (int) __vsubss4(((B >> 4) & 0x0F0F0F0Fu) | ((H >> 2) & 0x30303030u), 0x20202020u);
        }
        const int gbase = (u >> 3) * 8 + n128 * 4;
#pragma unroll
        for (int n = 0; n < N; ++n) {
            float part = 0.0f;
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                const int * xq = xv.q32(n, gbase + t) + g8 * 2;
                int s = __dp4a(q[t][0], xq[0], 0);
                s     = __dp4a(q[t][1], xq[1], s);
                part += (float) ((int) sc[2 * t] * s) * xv.ds(n, gbase + t).x;
            }
            acc[n] += d * part;
        }
    }
};

// Q2_K: a unit is the 32 weights of (128-half n, bit pair j): bits [2j, 2j+2) of 32 consecutive qs bytes, two
// 16-weight sub-blocks with a 4-bit scale and a 4-bit min each (ggml-quants.c:712-744); the mins need the
// activation sums of the two 16-value halves, taken here with a dot against ones.
template <> struct WT<T_Q2_K> {
    static constexpr int UNIT = 32, BLK_ELEMS = 256, BLK_BYTES = 84;
    template <int N> static __device__ __forceinline__ void dot(const uint8_t * row, int u, const ActView & xv, float (&acc)[N]) {
        const uint8_t * b = row + (u >> 3) * 84;
        const int n128 = (u >> 2) & 1, j = u & 3;
        const int sc0 = b[n128 * 8 + 2 * j], sc1 = b[n128 * 8 + 2 * j + 1];
        const float d = h2f(*(const uint16_t *) (b + 80)), dmin = h2f(*(const uint16_t *) (b + 82));
        uint32_t w[8];
        lds_words<8>(b + 16 + n128 * 32, w);
#pragma unroll
        for (int i = 0; i < 8; ++i) w[i] = (w[i] >> (2 * j)) & 0x03030303u;
#pragma unroll
        for (int n = 0; n < N; ++n) {
            const int * xq = xv.q32(n, u);
            int s0 = 0, s1 = 0, x0 = 0, x1 = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                s0 = __dp4a((int) w[i], xq[i], s0);         x0 = __dp4a(0x01010101, xq[i], x0);
                s1 = __dp4a((int) w[i + 4], xq[i + 4], s1); x1 = __dp4a(0x01010101, xq[i + 4], x1);
            }
            acc[n] += xv.ds(n, u).x * (d * (float) ((sc0 & 15) * s0 + (sc1 & 15) * s1) - dmin * (float) ((sc0 >> 4) * x0 + (sc1 >> 4) * x1));
        }
    }
};

// Q3_K: the same unit; the third bit of weight l is bit (4 n + j) of hmask[l], a clear bit subtracts 4, and the
// 6-bit scales carry an offset of 32 (ggml-quants.c:1056-1106)
template <> struct WT<T_Q3_K> {
    static constexpr int UNIT = 32, BLK_ELEMS = 256, BLK_BYTES = 110;
    template <int N> static __device__ __forceinline__ void dot(const uint8_t * row, int u, const ActView & xv, float (&acc)[N]) {
        const uint8_t * b = row + (u >> 3) * 110;
        const int n128 = (u >> 2) & 1, j = u & 3;
        const int sc0 = q3k_scale(b + 96, n128 * 8 + 2 * j) - 32, sc1 = q3k_scale(b + 96, n128 * 8 + 2 * j + 1) - 32;
        const float d = h2f(*(const uint16_t *) (b + 108));
        uint32_t w[8], h[8];
        lds_words<8>(b + 32 + n128 * 32, w);
        lds_words<8>(b, h);
#pragma unroll
        for (int i = 0; i < 8; ++i)
            w[i] = __vsub4(((w[i] >> (2 * j)) & 0x03030303u) | (((h[i] >> (4 * n128 + j)) & 0x01010101u) << 2), 0x04040404u);
#pragma unroll
        for (int n = 0; n < N; ++n) {
            const int * xq = xv.q32(n, u);
            int s0 = 0, s1 = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) { s0 = __dp4a((int) w[i], xq[i], s0); s1 = __dp4a((int) w[i + 4], xq[i + 4], s1); }
            acc[n] += d * xv.ds(n, u).x * (float) (sc0 * s0 + sc1 * s1);
        }
    }
};

// IQ4_NL: Q4_0 layout, nibbles looked up in the 16-entry table of the format with iq4nl_lut4
template <> struct WT<T_IQ4_NL> {
    static constexpr int UNIT = 32, BLK_ELEMS = 32, BLK_BYTES = 18;
    template <int N> static __device__ __forceinline__ void dot(const uint8_t * row, int u, const ActView & xv, float (&acc)[N]) {
        const uint8_t * b = row + u * 18;
        const float dw = h2f(*(const uint16_t *) b);
        uint32_t w[4], lo[4], hi[4];
        lds_words<4>(b + 2, w);
#pragma unroll
        for (int i = 0; i < 4; ++i) { lo[i] = iq4nl_lut4(w[i] & 0x0F0F0F0Fu); hi[i] = iq4nl_lut4((w[i] >> 4) & 0x0F0F0F0Fu); }
#pragma unroll
        for (int n = 0; n < N; ++n) {
            const int * xq = xv.q32(n, u);
            int s = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) { s = __dp4a((int) lo[i], xq[i], s); s = __dp4a((int) hi[i], xq[i + 4], s); }
            acc[n] += dw * xv.ds(n, u).x * (float) s;
        }
    }
};

// IQ4_XS: a unit is one 32-weight sub-block (16 qs bytes) with its own 6-bit scale (ggml-quants.c:2453-2475)
template <> struct WT<T_IQ4_XS> {
    static constexpr int UNIT = 32, BLK_ELEMS = 256, BLK_BYTES = 136;
    template <int N> static __device__ __forceinline__ void dot(const uint8_t * row, int u, const ActView & xv, float (&acc)[N]) {
        const uint8_t * b = row + (u >> 3) * 136;
        const int ib = u & 7;
        const float dl = h2f(*(const uint16_t *) b) * (float) iq4xs_scale(b, ib);
        uint32_t w[4], lo[4], hi[4];
        lds_words<4>(b + 8 + ib * 16, w);
#pragma unroll
        for (int i = 0; i < 4; ++i) { lo[i] = iq4nl_lut4(w[i] & 0x0F0F0F0Fu); hi[i] = iq4nl_lut4((w[i] >> 4) & 0x0F0F0F0Fu); }
#pragma unroll
        for (int n = 0; n < N; ++n) {
            const int * xq = xv.q32(n, u);
            int s = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) { s = __dp4a((int) lo[i], xq[i], s); s = __dp4a((int) hi[i], xq[i + 4], s); }
            acc[n] += dl * xv.ds(n, u).x * (float) s;
        }
    }
};

// ---------------------------------------------------------------------------
// the streaming kernel
// ---------------------------------------------------------------------------
static constexpr int MMVQ_WARPS  = 8;                    // consumer warps = rows per tile
static constexpr int MMVQ_STAGES = 4;
static constexpr int MMVQ_THREADS = (MMVQ_WARPS + 1) * 32;

struct MmvqParams {
    const uint8_t * W;  int64_t w_nb1, w_nb2, w_nb3;     // weight byte strides (row, dim2, dim3)
    const uint8_t * Xq; int64_t xq_col_bytes;            // quantized activations, columns ordered [i13][i12][n]
    int x_col0, x_ncols, xq_ne12;                        // first column of this launch, columns per batch, dim-2 extent of Xq
    const int32_t * ids; int64_t ids_s12, ids_s13;       // MUL_MAT_ID: expert index per (i12, i13), element strides
    float * dst;        int64_t dst_nb1, dst_nb2, dst_nb3;   // byte strides
    int M, K, N;                                         // rows, reduction length, columns of this launch's matrix
    int ne12, ne13, r2, r3;                              // batch dims of src1 and broadcast ratios
    int chunk_units;                                     // units (WT::UNIT weights) per k-chunk
    int slot_bytes;                                      // smem bytes reserved per row segment
    int xslot_bytes;                                     // smem bytes per activation column chunk
    int * status;
    int device, use_pdl;
};

__device__ __forceinline__ const uint8_t * weight_base(const MmvqParams & p, int i12, int i13) {
    if (p.ids) return p.W + (int64_t) p.ids[i12 * p.ids_s12 + i13 * p.ids_s13] * p.w_nb2;
    return p.W + (int64_t) (i13 / p.r3) * p.w_nb3 + (int64_t) (i12 / p.r2) * p.w_nb2;
}

template <int T, int N>
__global__ void __launch_bounds__(MMVQ_THREADS, 1) mmvq_kernel(const MmvqParams p) {
    using W = WT<T>;
    extern __shared__ __align__(128) uint8_t smem[];
    pdl_launch_dependents();          // the next kernel may start its prologue (its weight prefetch) right away
    __shared__ uint64_t full_bar[MMVQ_STAGES], empty_bar[MMVQ_STAGES];
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int stage_bytes = MMVQ_WARPS * p.slot_bytes + N * p.xslot_bytes;

    if (threadIdx.x == 0) {
        for (int s = 0; s < MMVQ_STAGES; ++s) { mbar_init(&full_bar[s], 2); mbar_init(&empty_bar[s], MMVQ_WARPS); }
        abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();

    // work decomposition: tile = (batch z, row group g, k chunk c); a CTA walks
    // row groups g = blockIdx.x, blockIdx.x + gridDim.x, ... and all chunks of each
    const int units_total = p.K / W::UNIT;
    const int nchunks     = (units_total + p.chunk_units - 1) / p.chunk_units;
    const int ngroups     = (p.M + MMVQ_WARPS - 1) / MMVQ_WARPS;
    const int nbatch      = p.ne12 * p.ne13;
    const int64_t total_groups = (int64_t) ngroups * nbatch;
    const int64_t my_groups = total_groups > blockIdx.x ? (total_groups - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    const int64_t my_tiles  = my_groups * nchunks;
    const int unit_bytes_num = W::BLK_BYTES * W::UNIT;   // bytes of u units = u * unit_bytes_num / BLK_ELEMS

    if (warp == MMVQ_WARPS) {
        // ---------------- producer warp ----------------
        // full_bar[s] takes two arrivals per tile: one carries the weight bytes
        // (lanes 0..7, one row segment each), one the activation bytes (lanes
        // 8..8+N-1, one column chunk each).  Weights do not depend on the previous
        // kernel in the stream, so the first ring-full of weight copies is issued
        // before the dependency wait.
        auto issue = [&](int64_t t, bool weights) {
            const int s = (int) (t % MMVQ_STAGES);
            const int64_t gi = blockIdx.x + (t / nchunks) * gridDim.x;
            const int c   = (int) (t % nchunks);
            const int z   = (int) (gi / ngroups), g = (int) (gi % ngroups);
            const int i12 = z % p.ne12, i13 = z / p.ne12;
            const int u0  = c * p.chunk_units;
            const int un  = min(p.chunk_units, units_total - u0);
            uint8_t * st = smem + (size_t) s * stage_bytes;
            const uint8_t * src = nullptr; uint8_t * dstp = nullptr; uint32_t bytes = 0;
            if (weights) {
                const int row = g * MMVQ_WARPS + lane;
                if (lane < MMVQ_WARPS && row < p.M) {
                    const int64_t seg_off   = (int64_t) u0 * unit_bytes_num / W::BLK_ELEMS;
                    const int     seg_bytes = un * unit_bytes_num / W::BLK_ELEMS;
                    const uint8_t * a = weight_base(p, i12, i13) + (int64_t) row * p.w_nb1 + seg_off;
                    const uintptr_t mis = (uintptr_t) a & 15;
                    src   = a - mis;
                    bytes = (uint32_t) ((mis + seg_bytes + 15) & ~(uintptr_t) 15);
                    dstp  = st + lane * p.slot_bytes;
                }
            } else if (lane >= MMVQ_WARPS && lane < MMVQ_WARPS + N) {
                const int n = lane - MMVQ_WARPS;
                const int64_t col = ((int64_t) i13 * p.xq_ne12 + (i12 % p.xq_ne12)) * p.x_ncols + p.x_col0 + n;
                const int b0 = u0 * W::UNIT / 128;
                const int b1 = ((u0 + un) * W::UNIT + 127) / 128;
                src   = p.Xq + col * p.xq_col_bytes + (int64_t) b0 * 160;
                bytes = (uint32_t) (b1 - b0) * 160;
                dstp  = st + MMVQ_WARPS * p.slot_bytes + n * p.xslot_bytes;
            }
            uint32_t total = bytes;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
            if (lane == 0) mbar_arrive_expect_tx(&full_bar[s], total);
            __syncwarp();
            if (bytes) bulk_g2s(dstp, src, bytes, &full_bar[s]);
        };
        const int64_t pre = my_tiles < MMVQ_STAGES ? my_tiles : MMVQ_STAGES;
        for (int64_t t = 0; t < pre; ++t) issue(t, true);
        pdl_wait();                                   // activations come from the previous kernel
        for (int64_t t = 0; t < pre; ++t) issue(t, false);
        for (int64_t t = pre; t < my_tiles; ++t) {
            const int s = (int) (t % MMVQ_STAGES);
            const uint32_t round = (uint32_t) (t / MMVQ_STAGES);
            if (!mbar_wait(&empty_bar[s], (round - 1) & 1)) {
                if (lane == 0) { atomicExch(p.status, ERR_MBAR_TIMEOUT); abort_flag = 1; }
                break;
            }
            issue(t, true);
            issue(t, false);
        }
    } else {
        // ---------------- consumer warps ----------------
        float acc[N];
#pragma unroll
        for (int n = 0; n < N; ++n) acc[n] = 0.0f;
        pdl_wait();                                   // dst may alias memory the previous kernel still uses
        for (int64_t t = 0; t < my_tiles; ++t) {
            const int s = (int) (t % MMVQ_STAGES);
            const uint32_t round = (uint32_t) (t / MMVQ_STAGES);
            if (!mbar_wait(&full_bar[s], round & 1)) { if (lane == 0) { atomicExch(p.status, ERR_MBAR_TIMEOUT); abort_flag = 1; } break; }
            if (*(volatile int *) &abort_flag) break;
            const int64_t gi = blockIdx.x + (t / nchunks) * gridDim.x;
            const int c   = (int) (t % nchunks);
            const int z   = (int) (gi / ngroups), g = (int) (gi % ngroups);
            const int row = g * MMVQ_WARPS + warp;
            const int u0  = c * p.chunk_units;
            const int un  = min(p.chunk_units, units_total - u0);
            const uint8_t * st = smem + (size_t) s * stage_bytes;
            if (row < p.M) {
                const int i12 = z % p.ne12, i13 = z / p.ne12;
                const uint8_t * a = weight_base(p, i12, i13) + (int64_t) row * p.w_nb1 + (int64_t) u0 * unit_bytes_num / W::BLK_ELEMS;
                const uint8_t * wrow = st + warp * p.slot_bytes + ((uintptr_t) a & 15);
                ActView xv { st + MMVQ_WARPS * p.slot_bytes, p.xslot_bytes };
                for (int u = lane; u < un; u += 32) W::template dot<N>(wrow, u, xv, acc);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[s]);
            if (c == nchunks - 1) {
#pragma unroll
                for (int n = 0; n < N; ++n) acc[n] = warp_sum(acc[n]);
                if (lane == 0 && row < p.M) {
                    const int i12 = z % p.ne12, i13 = z / p.ne12;
                    uint8_t * o = (uint8_t *) p.dst + (int64_t) i13 * p.dst_nb3 + (int64_t) i12 * p.dst_nb2;
#pragma unroll
                    for (int n = 0; n < N; ++n) ((float *) (o + (int64_t) n * p.dst_nb1))[row] = acc[n];
                }
#pragma unroll
                for (int n = 0; n < N; ++n) acc[n] = 0.0f;
            }
        }
    }
}

template <int T, int N>
static cudaError_t launch_mmvq_tn(const MmvqParams & p0, int sm_count, cudaStream_t stream) {
    using W = WT<T>;
    MmvqParams p = p0;
    // k-chunk: whole 256-weight groups, a multiple of 32 units when the row is
    // long enough, sized so one ring stage (8 row segments + N activation column
    // chunks) stays near 44 KB and 4 stages fit one CTA
    const int units_total   = p.K / W::UNIT;
    const int units_per_256 = 256 / W::UNIT;
    const int unit_w_bytes  = (W::BLK_BYTES * W::UNIT + W::BLK_ELEMS - 1) / W::BLK_ELEMS;   // Q2_K, Q3_K, Q6_K: fractional, rounded up
    const int per_unit      = MMVQ_WARPS * unit_w_bytes + N * (W::UNIT * 160 / 128);
    int cu = (44 * 1024 - MMVQ_WARPS * 48) / per_unit;
    const int cu_cap = 2304 / unit_w_bytes;            // ~2.25 KB per row segment is plenty
    if (cu > cu_cap) cu = cu_cap;
    cu = (cu / 32) * 32;
    if (cu < 32) cu = 32;
    if (cu > units_total) cu = ((units_total + units_per_256 - 1) / units_per_256) * units_per_256;
    p.chunk_units = cu;
    const int seg_bytes = (cu * W::BLK_BYTES * W::UNIT + W::BLK_ELEMS - 1) / W::BLK_ELEMS;
    p.slot_bytes  = ((seg_bytes + 15 + 15) & ~15) + 16;
    p.xslot_bytes = ((cu * W::UNIT + 127) / 128) * 160;
    const size_t smem = (size_t) MMVQ_STAGES * (MMVQ_WARPS * p.slot_bytes + N * p.xslot_bytes);

    static unsigned attr_mask = 0;                     // per-device: the attribute belongs to the context
    auto kern = mmvq_kernel<T, N>;
    if (!(attr_mask & (1u << p.device))) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return e;
        attr_mask |= 1u << p.device;
    }
    if (smem > 200 * 1024) return cudaErrorInvalidValue;
    const int64_t groups = (int64_t) ((p.M + MMVQ_WARPS - 1) / MMVQ_WARPS) * p.ne12 * p.ne13;
    int ctas_per_sm = (int) ((220 * 1024) / (smem + 2048));
    if (ctas_per_sm < 1) ctas_per_sm = 1;
    if (ctas_per_sm > 4) ctas_per_sm = 4;
    int64_t grid = (int64_t) sm_count * ctas_per_sm;
    if (grid > groups) grid = groups;
    if (grid < 1) grid = 1;

    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned) grid); cfg.blockDim = dim3(MMVQ_THREADS);
    cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = p.use_pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, p);
}

template <int T>
static cudaError_t launch_mmvq_t(const MmvqParams & p, int sm, cudaStream_t st) {
    switch (p.N) {
        case 1: return launch_mmvq_tn<T, 1>(p, sm, st);
        case 2: return launch_mmvq_tn<T, 2>(p, sm, st);
        case 3: return launch_mmvq_tn<T, 3>(p, sm, st);
        case 4: return launch_mmvq_tn<T, 4>(p, sm, st);
        case 5: return launch_mmvq_tn<T, 5>(p, sm, st);
        case 6: return launch_mmvq_tn<T, 6>(p, sm, st);
        case 7: return launch_mmvq_tn<T, 7>(p, sm, st);
        case 8: return launch_mmvq_tn<T, 8>(p, sm, st);
        default: return cudaErrorInvalidValue;
    }
}

// ---------------------------------------------------------------------------
// warp-staged kernel for the K-block types without a kernel of their own (Q2_K, Q3_K, IQ4_XS)
// ---------------------------------------------------------------------------
// One warp per weight row at a time, no block-wide barriers in the loop: the warp fetches a run of up to 32
// super-blocks of its row with coalesced 128-bit loads from the enclosing 16-byte aligned window into registers,
// parks it in a warp-private shared-memory buffer, and every lane takes units (32 weights) from there with the same
// WT<T>::dot as the ring kernel.  The next run (of this row or of the warp's next row) is loaded while the
// current one is decoded; weight loads are issued before the dependency wait.  All activation columns sit in
// shared memory for the life of the CTA.
static constexpr int STG_WARPS = 8;
static constexpr int STG_RUN_BLOCKS = 32;

struct StagedParams {
    const uint8_t * W;  int64_t w_nb1;
    const uint8_t * Xq; int64_t xq_col_bytes;
    float * dst;        int64_t dst_nb1;
    int M, K, x_col0;
    int n_peer; int64_t peer_delta[MAX_PEERS - 1];                 // row-split: results also go to dst + peer_delta[i]
};

template <int T, int N>
__global__ void __launch_bounds__(STG_WARPS * 32, 2) mmvq_staged_kernel(const StagedParams p) {
    using W = WT<T>;
    constexpr int BB = W::BLK_BYTES;
    constexpr int RUN_BYTES = STG_RUN_BLOCKS * BB;
    constexpr int STAGE_BYTES = (RUN_BYTES + 15 + 15) / 16 * 16 + 16;      // misalignment in front, 16 bytes of slack behind
    constexpr int VPL = (STAGE_BYTES / 16 + 31) / 32;                      // uint4 per lane
    constexpr int UPB = 256 / W::UNIT;                                     // units per super-block
    extern __shared__ __align__(128) uint8_t smem[];
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nblk = p.K >> 8;
    const int col_bytes = ((p.K + 127) >> 7) * 160;
    uint8_t * acts  = smem;                                                // [N][col_bytes]
    uint8_t * stage = smem + (size_t) N * col_bytes + (size_t) warp * STAGE_BYTES;

    const int nruns = (nblk + STG_RUN_BLOCKS - 1) / STG_RUN_BLOCKS;
    const int row_stride = gridDim.x * STG_WARPS;
    int row = blockIdx.x * STG_WARPS + warp;
    bool storer = lane == 0; int64_t st_delta = 0;
#pragma unroll
    for (int q = 0; q < MAX_PEERS - 1; ++q) if (q < p.n_peer && lane == q + 1) { storer = true; st_delta = p.peer_delta[q]; }

    uint4 v[VPL];
    auto run_src = [&](int r, int run) { return p.W + (int64_t) r * p.w_nb1 + (int64_t) run * RUN_BYTES; };
    auto run_vecs = [&](const uint8_t * a, int run) {
        const int bytes = min(STG_RUN_BLOCKS, nblk - run * STG_RUN_BLOCKS) * BB;
        return (int) ((((uintptr_t) a & 15) + bytes + 15) >> 4);
    };
    auto load_run = [&](int r, int run) {
        const uint8_t * a = run_src(r, run);
        const uint4 * src = (const uint4 *) ((uintptr_t) a & ~(uintptr_t) 15);
        const int nvec = run_vecs(a, run);
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            const int idx = i * 32 + lane;
            if (idx < nvec) v[i] = __ldg(src + idx);
        }
    };
    auto store_run = [&](int r, int run) {
        const int nvec = run_vecs(run_src(r, run), run);
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            const int idx = i * 32 + lane;
            if (idx < nvec) ((uint4 *) stage)[idx] = v[i];
        }
    };

    if (row < p.M) load_run(row, 0);
    pdl_wait();
    for (int n = 0; n < N; ++n) {
        const uint4 * src = (const uint4 *) (p.Xq + (int64_t) (p.x_col0 + n) * p.xq_col_bytes);
        uint4 * dstp = (uint4 *) (acts + n * col_bytes);
        for (int i = threadIdx.x; i < col_bytes / 16; i += blockDim.x) dstp[i] = src[i];
    }
    __syncthreads();
    const ActView xv { acts, col_bytes };

    while (row < p.M) {
        float acc[N];
#pragma unroll
        for (int n = 0; n < N; ++n) acc[n] = 0.0f;
        for (int run = 0; run < nruns; ++run) {
            __syncwarp();
            store_run(row, run);
            __syncwarp();
            if (run + 1 < nruns) load_run(row, run + 1);
            else if (row + row_stride < p.M) load_run(row + row_stride, 0);
            // dot() addresses units from the start of the row: hand it the address the row would have if all of it were staged
            const uint8_t * vrow = stage + ((uintptr_t) run_src(row, run) & 15) - (size_t) run * RUN_BYTES;
            const int u_end = min((run + 1) * STG_RUN_BLOCKS, nblk) * UPB;
            for (int u = run * STG_RUN_BLOCKS * UPB + lane; u < u_end; u += 32) W::template dot<N>(vrow, u, xv, acc);
        }
#pragma unroll
        for (int n = 0; n < N; ++n) acc[n] = warp_sum(acc[n]);
        if (storer) {                     // lane 0: this GPU's dst; lane q + 1: the copy in peer q's arena
#pragma unroll
            for (int n = 0; n < N; ++n) ((float *) ((uint8_t *) p.dst + (int64_t) n * p.dst_nb1 + st_delta))[row] = acc[n];
        }
        row += row_stride;
    }
}

template <int T>
static size_t staged_smem_bytes(int N, int K) {
    constexpr int STAGE_BYTES = (STG_RUN_BLOCKS * WT<T>::BLK_BYTES + 15 + 15) / 16 * 16 + 16;
    return (size_t) N * ((K + 127) / 128) * 160 + (size_t) STG_WARPS * STAGE_BYTES;
}

template <int T, int N>
static cudaError_t launch_staged_tn(const StagedParams & p, int sm_count, int device, int use_pdl, cudaStream_t stream) {
    const size_t smem = staged_smem_bytes<T>(N, p.K);
    auto kern = mmvq_staged_kernel<T, N>;
    static unsigned attr_mask = 0;
    if (smem > 48 * 1024 && !(attr_mask & (1u << device))) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return e;
        attr_mask |= 1u << device;
    }
    if (smem > 200 * 1024) return cudaErrorInvalidValue;
    int ctas_per_sm = (int) ((220 * 1024) / (smem + 1024));
    if (ctas_per_sm > 3) ctas_per_sm = 3;
    if (ctas_per_sm < 1) ctas_per_sm = 1;
    int64_t grid = (int64_t) sm_count * ctas_per_sm;
    const int64_t need = ((int64_t) p.M + STG_WARPS - 1) / STG_WARPS;
    if (grid > need) grid = need;
    if (grid < 1) grid = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned) grid); cfg.blockDim = dim3(STG_WARPS * 32);
    cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = use_pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, p);
}

template <int T>
static cudaError_t launch_staged_t(const StagedParams & p, int N, int sm, int dev, int pdl, cudaStream_t st) {
    switch (N) {
        case 1: return launch_staged_tn<T, 1>(p, sm, dev, pdl, st);
        case 2: return launch_staged_tn<T, 2>(p, sm, dev, pdl, st);
        case 3: return launch_staged_tn<T, 3>(p, sm, dev, pdl, st);
        case 4: return launch_staged_tn<T, 4>(p, sm, dev, pdl, st);
        case 5: return launch_staged_tn<T, 5>(p, sm, dev, pdl, st);
        case 6: return launch_staged_tn<T, 6>(p, sm, dev, pdl, st);
        case 7: return launch_staged_tn<T, 7>(p, sm, dev, pdl, st);
        case 8: return launch_staged_tn<T, 8>(p, sm, dev, pdl, st);
    }
    return cudaErrorInvalidValue;
}

// plain 2-D weights (no batching, no expert indirection), whole super-blocks, activations that fit shared memory
static bool mmvq_staged_applicable(const MmvqArgs & a) {
    if ((a.type != T_Q2_K && a.type != T_Q3_K && a.type != T_IQ4_XS) || a.ids || a.ne12 * a.ne13 != 1) return false;
    if ((a.K % 256) != 0 || a.N < 1 || a.N > 8) return false;
    const size_t smem = a.type == T_Q2_K ? staged_smem_bytes<T_Q2_K>(a.N, a.K) : a.type == T_Q3_K ? staged_smem_bytes<T_Q3_K>(a.N, a.K) : staged_smem_bytes<T_IQ4_XS>(a.N, a.K);
    return smem <= 200 * 1024;
}

static cudaError_t launch_mmvq_staged(const MmvqArgs & a, cudaStream_t stream) {
    StagedParams p = {};
    p.W = (const uint8_t *) a.W; p.w_nb1 = a.w_nb1;
    p.Xq = (const uint8_t *) a.Xq; p.xq_col_bytes = (int64_t) ((a.K + 127) / 128) * 160;
    p.dst = a.dst; p.dst_nb1 = a.dst_nb1;
    p.M = a.M; p.K = a.K; p.x_col0 = a.x_col0;
    p.n_peer = a.n_peer; for (int i = 0; i < a.n_peer; ++i) p.peer_delta[i] = a.peer_delta[i];
    if (a.type == T_Q2_K) return launch_staged_t<T_Q2_K>(p, a.N, a.sm_count, a.device, a.use_pdl, stream);
    if (a.type == T_Q3_K) return launch_staged_t<T_Q3_K>(p, a.N, a.sm_count, a.device, a.use_pdl, stream);
    return launch_staged_t<T_IQ4_XS>(p, a.N, a.sm_count, a.device, a.use_pdl, stream);
}

bool mmvq_type_supported(int type) {
    switch (type) {
        case T_Q4_0: case T_Q4_1: case T_Q5_0: case T_Q5_1: case T_Q8_0: case T_IQ4_NL: case T_IQ4_XS:
        case T_Q2_K: case T_Q3_K: case T_Q4_K: case T_Q5_K: case T_Q6_K: return true;
        default: return false;
    }
}

size_t act128_bytes(int64_t K, int64_t ncols) { return (size_t) ((K + 127) / 128) * 160 * (size_t) ncols; }

cudaError_t launch_quantize_act128(const float * x, int64_t ne11, int64_t ne12, int64_t ne13,
                                   int64_t s11, int64_t s12, int64_t s13, void * y, int K, cudaStream_t stream, int use_pdl) {
    const int nblk = (K + 127) / 128;
    const int64_t ncols = ne11 * ne12 * ne13;
    const int64_t warps = ncols * nblk;
    if (warps == 0) return cudaSuccess;
    const int wpb = 8;
    return launch_k(use_pdl, stream, quantize_act128_kernel, dim3((unsigned) ((warps + wpb - 1) / wpb)), dim3(wpb * 32), 0,
                    x, ne11, ne12, s11, s12, s13, (blk_act128 *) y, K, nblk, ncols);
}

// do the kernels launch_mmvq picks for these arguments honour n_peer / peer_delta?
bool mmvq_stores_to_peers(const MmvqArgs & a) { return mmvq_k_applicable(a) || mmvq_q6k_applicable(a) || mmvq_q32_applicable(a) || mmvq_staged_applicable(a); }

cudaError_t launch_mmvq(const MmvqArgs & a, cudaStream_t stream) {
    if (mmvq_k_applicable(a)) return launch_mmvq_k(a, stream);
    if (mmvq_q6k_applicable(a)) return launch_mmvq_q6k(a, stream);
    if (mmvq_q32_applicable(a)) return launch_mmvq_q32(a, stream);
    if (mmvq_staged_applicable(a)) return launch_mmvq_staged(a, stream);
    MmvqParams p = {};
    p.W = (const uint8_t *) a.W; p.w_nb1 = a.w_nb1; p.w_nb2 = a.w_nb2; p.w_nb3 = a.w_nb3;
    p.Xq = (const uint8_t *) a.Xq; p.xq_col_bytes = (int64_t) ((a.K + 127) / 128) * 160;
    p.dst = a.dst; p.dst_nb1 = a.dst_nb1; p.dst_nb2 = a.dst_nb2; p.dst_nb3 = a.dst_nb3;
    p.M = a.M; p.K = a.K; p.N = a.N; p.ne12 = a.ne12; p.ne13 = a.ne13; p.r2 = a.r2; p.r3 = a.r3;
    p.status = a.status; p.device = a.device; p.use_pdl = a.use_pdl;
    p.x_col0 = a.x_col0; p.x_ncols = a.x_ncols; p.xq_ne12 = a.xq_ne12 > 0 ? a.xq_ne12 : a.ne12;
    p.ids = a.ids; p.ids_s12 = a.ids_s12; p.ids_s13 = a.ids_s13;
    switch (a.type) {
        case T_Q4_0: return launch_mmvq_t<T_Q4_0>(p, a.sm_count, stream);
        case T_Q4_1: return launch_mmvq_t<T_Q4_1>(p, a.sm_count, stream);
        case T_Q5_0: return launch_mmvq_t<T_Q5_0>(p, a.sm_count, stream);
        case T_Q5_1: return launch_mmvq_t<T_Q5_1>(p, a.sm_count, stream);
        case T_Q8_0: return launch_mmvq_t<T_Q8_0>(p, a.sm_count, stream);
        case T_Q4_K: return launch_mmvq_t<T_Q4_K>(p, a.sm_count, stream);
        case T_Q5_K: return launch_mmvq_t<T_Q5_K>(p, a.sm_count, stream);
        case T_Q6_K: return launch_mmvq_t<T_Q6_K>(p, a.sm_count, stream);
        case T_Q2_K: return launch_mmvq_t<T_Q2_K>(p, a.sm_count, stream);
        case T_Q3_K: return launch_mmvq_t<T_Q3_K>(p, a.sm_count, stream);
        case T_IQ4_NL: return launch_mmvq_t<T_IQ4_NL>(p, a.sm_count, stream);
        case T_IQ4_XS: return launch_mmvq_t<T_IQ4_XS>(p, a.sm_count, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace b200
