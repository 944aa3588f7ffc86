/*
 * CPU restatement of the reference's algorithms for the hot path, in plain C.
 * TEST INFRASTRUCTURE ONLY: it is the checker the CUDA kernels are compared
 * with (tests/, the smoke test and the CPU-baseline leg of bench.py); nothing
 * in the product path may call it.
 *
 * Parity pin: every function here is checked by tests/test_oracle.py against
 * tests/golden/golden.bin, which holds outputs of the unmodified reference
 * (quantizers, dequantizers and the ggml CPU backend) on seeded inputs, and,
 * when oracle/_ref is present, against the reference libraries directly.
 *
 * Each function cites the reference code it follows (paths within the
 * reference project).  Scalar C, one thread, no SIMD: results equal the
 * reference's up to floating-point summation order.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define EXPORT __attribute__((visibility("default")))

enum { T_F32 = 0, T_F16 = 1, T_Q4_0 = 2, T_Q4_1 = 3, T_Q5_0 = 6, T_Q5_1 = 7, T_Q8_0 = 8, T_Q2_K = 10, T_Q3_K = 11, T_Q4_K = 12, T_Q5_K = 13, T_Q6_K = 14, T_IQ4_NL = 20, T_IQ4_XS = 23 };

/* ---- IEEE half <-> float (ggml_compute_fp16_to_fp32 / fp32_to_fp16, ggml/src/ggml-impl.h:330-400) ---- */
static float h2f(uint16_t h) {
    const uint32_t sign = (uint32_t) (h & 0x8000) << 16;
    uint32_t exp = (h >> 10) & 0x1F, man = h & 0x3FF, bits;
    if (exp == 0) {
        if (man == 0) { bits = sign; }
        else {                                  /* subnormal */
            int e = -1;
            do { e++; man <<= 1; } while (!(man & 0x400));
            bits = sign | ((uint32_t) (127 - 15 - e) << 23) | ((man & 0x3FF) << 13);
        }
    } else if (exp == 31) { bits = sign | 0x7F800000u | (man << 13); }
    else { bits = sign | ((exp + 112) << 23) | (man << 13); }
    float f; memcpy(&f, &bits, 4); return f;
}
static uint16_t f2h(float f) {                 /* round to nearest even */
    uint32_t x; memcpy(&x, &f, 4);
    const uint16_t sign = (uint16_t) ((x >> 16) & 0x8000);
    const uint32_t ax = x & 0x7FFFFFFFu;
    if (ax >= 0x7F800000u) return (uint16_t) (sign | 0x7C00 | ((ax > 0x7F800000u) ? 0x200 : 0));
    if (ax >= 0x477FF000u) return (uint16_t) (sign | 0x7C00);            /* overflows to inf after rounding */
    if (ax < 0x33000001u) return sign;                                    /* rounds to zero */
    int32_t exp = (int32_t) (ax >> 23) - 127;
    uint32_t man = (ax & 0x7FFFFFu) | 0x800000u;
    if (exp < -14) {                                                       /* subnormal half */
        const int shift = -14 - exp + 13;
        const uint32_t halfway = 1u << (shift - 1), mask = (1u << shift) - 1;
        uint32_t r = man >> shift;
        const uint32_t rem = man & mask;
        if (rem > halfway || (rem == halfway && (r & 1))) r++;
        return (uint16_t) (sign | r);
    }
    uint32_t r = ((uint32_t) (exp + 15) << 10) | ((man >> 13) & 0x3FF);
    const uint32_t rem = man & 0x1FFF;
    if (rem > 0x1000 || (rem == 0x1000 && (r & 1))) r++;
    return (uint16_t) (sign | r);
}
EXPORT void oracle_f32_to_f16(const float * x, uint16_t * y, int64_t n) { for (int64_t i = 0; i < n; ++i) y[i] = f2h(x[i]); }
EXPORT void oracle_f16_to_f32(const uint16_t * x, float * y, int64_t n) { for (int64_t i = 0; i < n; ++i) y[i] = h2f(x[i]); }

/* ---- block layouts (ggml/src/ggml-common.h:161-328) ---- */
#pragma pack(push, 1)
typedef struct { uint16_t d; uint8_t qs[16]; } blk_q4_0;
typedef struct { uint16_t d, m; uint8_t qs[16]; } blk_q4_1;
typedef struct { uint16_t d; uint8_t qh[4]; uint8_t qs[16]; } blk_q5_0;
typedef struct { uint16_t d, m; uint8_t qh[4]; uint8_t qs[16]; } blk_q5_1;
typedef struct { uint16_t d; int8_t qs[32]; } blk_q8_0;
typedef struct { uint16_t d, s; int8_t qs[32]; } blk_q8_1;
typedef struct { uint16_t d, dmin; uint8_t scales[12]; uint8_t qs[128]; } blk_q4_K;
typedef struct { uint16_t d, dmin; uint8_t scales[12]; uint8_t qh[32]; uint8_t qs[128]; } blk_q5_K;
typedef struct { uint8_t ql[128]; uint8_t qh[64]; int8_t scales[16]; uint16_t d; } blk_q6_K;
typedef struct { uint8_t scales[16]; uint8_t qs[64]; uint16_t d, dmin; } blk_q2_K;
typedef struct { uint8_t hmask[32]; uint8_t qs[64]; uint8_t scales[12]; uint16_t d; } blk_q3_K;
typedef struct { uint16_t d; uint8_t qs[16]; } blk_iq4_nl;
typedef struct { uint16_t d, scales_h; uint8_t scales_l[4]; uint8_t qs[128]; } blk_iq4_xs;
typedef struct { float d; int8_t qs[256]; int16_t bsums[16]; } blk_q8_K;
#pragma pack(pop)

EXPORT int64_t oracle_row_size(int type, int64_t k) {      /* ggml_row_size, ggml/src/ggml.c:1204 */
    switch (type) {
        case T_F32: return 4 * k; case T_F16: return 2 * k;
        case T_Q4_0: return k / 32 * 18; case T_Q4_1: return k / 32 * 20; case T_Q5_0: return k / 32 * 22;
        case T_Q5_1: return k / 32 * 24; case T_Q8_0: return k / 32 * 34;
        case T_Q4_K: return k / 256 * 144; case T_Q5_K: return k / 256 * 176; case T_Q6_K: return k / 256 * 210;
        case T_Q2_K: return k / 256 * 84; case T_Q3_K: return k / 256 * 110; case T_IQ4_NL: return k / 32 * 18; case T_IQ4_XS: return k / 256 * 136;
    }
    return 0;
}

/* get_scale_min_k4, ggml/src/ggml-quants.c:631-638 */
static void scale_min_k4(int j, const uint8_t * q, uint8_t * d, uint8_t * m) {
    if (j < 4) { *d = q[j] & 63; *m = q[j + 4] & 63; }
    else { *d = (uint8_t) ((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4)); *m = (uint8_t) ((q[j + 4] >> 4) | ((q[j] >> 6) << 4)); }
}

/* 6-bit scale s of a Q3_K super-block before its offset of 32: low nibble from scales[0..7], two high bits from
 * scales[8..11] (what the word shuffle at ggml/src/ggml-quants.c:1075-1080 produces, element by element) */
static int q3k_scale6(const uint8_t * sc, int s) {
    const int lo = s < 8 ? (sc[s] & 0xF) : (sc[s - 8] >> 4);
    return lo | (((sc[8 + (s & 3)] >> (2 * (s >> 2))) & 3) << 4);
}
/* the non-linear 4-bit code book of IQ4_NL (kvalues_iq4nl, ggml/src/ggml-quants.c:2434) */
static const int8_t iq4nl_values[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};

/* 6-bit scale of sub-block ib of an IQ4_XS super-block, offset removed (ggml/src/ggml-quants.c:2465) */
static int iq4xs_scale(const blk_iq4_xs * b, int ib) {
    return (((b->scales_l[ib / 2] >> (4 * (ib % 2))) & 0xF) | (((b->scales_h >> (2 * ib)) & 3) << 4)) - 32;
}

/* ---- dequantize_row_* (ggml/src/ggml-quants.c: q2_K 712, q3_K 1056, iq4_nl 2436, iq4_xs 2453, q4_0 255, q4_1 275, q5_0 296, q5_1 322, q8_0 349,
 *      q4_K 1280, q5_K 1482, q6_K 1690) ---- */
EXPORT int oracle_dequantize_row(int type, const void * src, float * y, int64_t k) {
    switch (type) {
        case T_F32: memcpy(y, src, (size_t) k * 4); return 0;
        case T_F16: oracle_f16_to_f32((const uint16_t *) src, y, k); return 0;
        case T_Q4_0: { const blk_q4_0 * x = src;
            for (int64_t i = 0; i < k / 32; ++i) { const float d = h2f(x[i].d);
                for (int j = 0; j < 16; ++j) { y[i*32 + j] = (float) ((x[i].qs[j] & 0x0F) - 8) * d; y[i*32 + j + 16] = (float) ((x[i].qs[j] >> 4) - 8) * d; } }
            return 0; }
        case T_Q4_1: { const blk_q4_1 * x = src;
            for (int64_t i = 0; i < k / 32; ++i) { const float d = h2f(x[i].d), m = h2f(x[i].m);
                for (int j = 0; j < 16; ++j) { y[i*32 + j] = (float) (x[i].qs[j] & 0x0F) * d + m; y[i*32 + j + 16] = (float) (x[i].qs[j] >> 4) * d + m; } }
            return 0; }
        case T_Q5_0: { const blk_q5_0 * x = src;
            for (int64_t i = 0; i < k / 32; ++i) { const float d = h2f(x[i].d); uint32_t qh; memcpy(&qh, x[i].qh, 4);
                for (int j = 0; j < 16; ++j) {
                    const uint8_t xh0 = (uint8_t) (((qh >> (j + 0)) << 4) & 0x10), xh1 = (uint8_t) ((qh >> (j + 12)) & 0x10);
                    y[i*32 + j] = (float) (((x[i].qs[j] & 0x0F) | xh0) - 16) * d; y[i*32 + j + 16] = (float) (((x[i].qs[j] >> 4) | xh1) - 16) * d; } }
            return 0; }
        case T_Q5_1: { const blk_q5_1 * x = src;
            for (int64_t i = 0; i < k / 32; ++i) { const float d = h2f(x[i].d), m = h2f(x[i].m); uint32_t qh; memcpy(&qh, x[i].qh, 4);
                for (int j = 0; j < 16; ++j) {
                    const uint8_t xh0 = (uint8_t) (((qh >> (j + 0)) << 4) & 0x10), xh1 = (uint8_t) ((qh >> (j + 12)) & 0x10);
                    y[i*32 + j] = (float) ((x[i].qs[j] & 0x0F) | xh0) * d + m; y[i*32 + j + 16] = (float) ((x[i].qs[j] >> 4) | xh1) * d + m; } }
            return 0; }
        case T_Q8_0: { const blk_q8_0 * x = src;
            for (int64_t i = 0; i < k / 32; ++i) { const float d = h2f(x[i].d); for (int j = 0; j < 32; ++j) y[i*32 + j] = (float) x[i].qs[j] * d; }
            return 0; }
        case T_Q2_K: { const blk_q2_K * x = src;
            for (int64_t i = 0; i < k / 256; ++i) { const float d = h2f(x[i].d), min = h2f(x[i].dmin);
                for (int e = 0; e < 256; ++e) { const int n = e >> 7, j = (e & 127) >> 5, l = e & 31;
                    const uint8_t sc = x[i].scales[n * 8 + 2 * j + (l >> 4)];
                    const float dl = d * (float) (sc & 0xF), ml = min * (float) (sc >> 4);
                    y[i*256 + e] = dl * (float) ((x[i].qs[n * 32 + l] >> (2 * j)) & 3) - ml; } }
            return 0; }
        case T_Q3_K: { const blk_q3_K * x = src;
            for (int64_t i = 0; i < k / 256; ++i) { const float d = h2f(x[i].d);
                for (int e = 0; e < 256; ++e) { const int n = e >> 7, j = (e & 127) >> 5, l = e & 31;
                    const float dl = d * (float) (q3k_scale6(x[i].scales, n * 8 + 2 * j + (l >> 4)) - 32);
                    const int q = ((x[i].qs[n * 32 + l] >> (2 * j)) & 3) - (((x[i].hmask[l] >> (4 * n + j)) & 1) ? 0 : 4);
                    y[i*256 + e] = dl * (float) q; } }
            return 0; }
        case T_IQ4_NL: { const blk_iq4_nl * x = src;
            for (int64_t i = 0; i < k / 32; ++i) { const float d = h2f(x[i].d);
                for (int j = 0; j < 16; ++j) { y[i*32 + j] = d * (float) iq4nl_values[x[i].qs[j] & 0xF]; y[i*32 + j + 16] = d * (float) iq4nl_values[x[i].qs[j] >> 4]; } }
            return 0; }
        case T_IQ4_XS: { const blk_iq4_xs * x = src;
            for (int64_t i = 0; i < k / 256; ++i) { const float d = h2f(x[i].d);
                for (int ib = 0; ib < 8; ++ib) { const float dl = d * (float) iq4xs_scale(&x[i], ib); const uint8_t * qs = x[i].qs + 16 * ib;
                    for (int j = 0; j < 16; ++j) { y[i*256 + ib*32 + j] = dl * (float) iq4nl_values[qs[j] & 0xF]; y[i*256 + ib*32 + j + 16] = dl * (float) iq4nl_values[qs[j] >> 4]; } } }
            return 0; }
        case T_Q4_K: { const blk_q4_K * x = src;
            for (int64_t i = 0; i < k / 256; ++i) { const uint8_t * q = x[i].qs; const float d = h2f(x[i].d), min = h2f(x[i].dmin);
                int is = 0; uint8_t sc, m;
                for (int j = 0; j < 256; j += 64) {
                    scale_min_k4(is + 0, x[i].scales, &sc, &m); const float d1 = d * sc, m1 = min * m;
                    scale_min_k4(is + 1, x[i].scales, &sc, &m); const float d2 = d * sc, m2 = min * m;
                    for (int l = 0; l < 32; ++l) *y++ = d1 * (float) (q[l] & 0xF) - m1;
                    for (int l = 0; l < 32; ++l) *y++ = d2 * (float) (q[l] >> 4) - m2;
                    q += 32; is += 2; } }
            return 0; }
        case T_Q5_K: { const blk_q5_K * x = src;
            for (int64_t i = 0; i < k / 256; ++i) { const uint8_t * ql = x[i].qs; const uint8_t * qh = x[i].qh; const float d = h2f(x[i].d), min = h2f(x[i].dmin);
                int is = 0; uint8_t sc, m, u1 = 1, u2 = 2;
                for (int j = 0; j < 256; j += 64) {
                    scale_min_k4(is + 0, x[i].scales, &sc, &m); const float d1 = d * sc, m1 = min * m;
                    scale_min_k4(is + 1, x[i].scales, &sc, &m); const float d2 = d * sc, m2 = min * m;
                    for (int l = 0; l < 32; ++l) *y++ = d1 * (float) ((ql[l] & 0xF) + ((qh[l] & u1) ? 16 : 0)) - m1;
                    for (int l = 0; l < 32; ++l) *y++ = d2 * (float) ((ql[l] >> 4) + ((qh[l] & u2) ? 16 : 0)) - m2;
                    ql += 32; is += 2; u1 <<= 2; u2 <<= 2; } }
            return 0; }
        case T_Q6_K: { const blk_q6_K * x = src;
            for (int64_t i = 0; i < k / 256; ++i) { const float d = h2f(x[i].d); const uint8_t * ql = x[i].ql; const uint8_t * qh = x[i].qh; const int8_t * sc = x[i].scales;
                for (int n = 0; n < 256; n += 128) {
                    for (int l = 0; l < 32; ++l) { const int is = l / 16;
                        const int8_t q1 = (int8_t) ((ql[l] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32, q2 = (int8_t) ((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
                        const int8_t q3 = (int8_t) ((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32, q4 = (int8_t) ((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
                        y[l] = d * sc[is] * q1; y[l + 32] = d * sc[is + 2] * q2; y[l + 64] = d * sc[is + 4] * q3; y[l + 96] = d * sc[is + 6] * q4; }
                    y += 128; ql += 64; qh += 32; sc += 8; } }
            return 0; }
    }
    return -1;
}

/* ---- quantize_row_*_ref for the 32-value formats (ggml/src/ggml-quants.c:31-217) ---- */
#define MINI(a, b) ((a) < (b) ? (a) : (b))
EXPORT int oracle_quantize_row(int type, const float * x, void * dst, int64_t k) {
    const int64_t nb = k / 32;
    switch (type) {
        case T_Q4_0: { blk_q4_0 * y = dst;
            for (int64_t i = 0; i < nb; ++i) { float amax = 0.0f, max = 0.0f;
                for (int j = 0; j < 32; ++j) { const float v = x[i*32 + j]; if (amax < fabsf(v)) { amax = fabsf(v); max = v; } }
                const float d = max / -8; const float id = d ? 1.0f / d : 0.0f; y[i].d = f2h(d);
                for (int j = 0; j < 16; ++j) { const float x0 = x[i*32 + j] * id, x1 = x[i*32 + 16 + j] * id;
                    const uint8_t xi0 = (uint8_t) MINI(15, (int8_t) (x0 + 8.5f)), xi1 = (uint8_t) MINI(15, (int8_t) (x1 + 8.5f)); y[i].qs[j] = (uint8_t) (xi0 | (xi1 << 4)); } }
            return 0; }
        case T_Q4_1: { blk_q4_1 * y = dst;
            for (int64_t i = 0; i < nb; ++i) { float min = INFINITY, max = -INFINITY;
                for (int j = 0; j < 32; ++j) { const float v = x[i*32 + j]; if (v < min) min = v; if (v > max) max = v; }
                const float d = (max - min) / 15; const float id = d ? 1.0f / d : 0.0f; y[i].d = f2h(d); y[i].m = f2h(min);
                for (int j = 0; j < 16; ++j) { const float x0 = (x[i*32 + j] - min) * id, x1 = (x[i*32 + 16 + j] - min) * id;
                    const uint8_t xi0 = (uint8_t) MINI(15, (int8_t) (x0 + 0.5f)), xi1 = (uint8_t) MINI(15, (int8_t) (x1 + 0.5f)); y[i].qs[j] = (uint8_t) (xi0 | (xi1 << 4)); } }
            return 0; }
        case T_Q5_0: { blk_q5_0 * y = dst;
            for (int64_t i = 0; i < nb; ++i) { float amax = 0.0f, max = 0.0f;
                for (int j = 0; j < 32; ++j) { const float v = x[i*32 + j]; if (amax < fabsf(v)) { amax = fabsf(v); max = v; } }
                const float d = max / -16; const float id = d ? 1.0f / d : 0.0f; y[i].d = f2h(d); uint32_t qh = 0;
                for (int j = 0; j < 16; ++j) { const float x0 = x[i*32 + j] * id, x1 = x[i*32 + 16 + j] * id;
                    const uint8_t xi0 = (uint8_t) MINI(31, (int8_t) (x0 + 16.5f)), xi1 = (uint8_t) MINI(31, (int8_t) (x1 + 16.5f));
                    y[i].qs[j] = (uint8_t) ((xi0 & 0x0F) | ((xi1 & 0x0F) << 4)); qh |= ((xi0 & 0x10u) >> 4) << (j + 0); qh |= ((xi1 & 0x10u) >> 4) << (j + 16); }
                memcpy(y[i].qh, &qh, 4); }
            return 0; }
        case T_Q5_1: { blk_q5_1 * y = dst;
            for (int64_t i = 0; i < nb; ++i) { float min = INFINITY, max = -INFINITY;
                for (int j = 0; j < 32; ++j) { const float v = x[i*32 + j]; if (v < min) min = v; if (v > max) max = v; }
                const float d = (max - min) / 31; const float id = d ? 1.0f / d : 0.0f; y[i].d = f2h(d); y[i].m = f2h(min); uint32_t qh = 0;
                for (int j = 0; j < 16; ++j) { const float x0 = (x[i*32 + j] - min) * id, x1 = (x[i*32 + 16 + j] - min) * id;
                    const uint8_t xi0 = (uint8_t) (x0 + 0.5f), xi1 = (uint8_t) (x1 + 0.5f);
                    y[i].qs[j] = (uint8_t) ((xi0 & 0x0F) | ((xi1 & 0x0F) << 4)); qh |= ((xi0 & 0x10u) >> 4) << (j + 0); qh |= ((xi1 & 0x10u) >> 4) << (j + 16); }
                memcpy(y[i].qh, &qh, 4); }
            return 0; }
        case T_Q8_0: { blk_q8_0 * y = dst;
            for (int64_t i = 0; i < nb; ++i) { float amax = 0.0f;
                for (int j = 0; j < 32; ++j) { const float v = fabsf(x[i*32 + j]); if (v > amax) amax = v; }
                const float d = amax / 127; const float id = d ? 1.0f / d : 0.0f; y[i].d = f2h(d);
                for (int j = 0; j < 32; ++j) y[i].qs[j] = (int8_t) roundf(x[i*32 + j] * id); }
            return 0; }
    }
    return -1;
}

/* ---- activation quantizers used by the CPU mat-mul (vec_dot_type of each weight type,
 *      ggml/src/ggml-cpu/ggml-cpu.c:252-340): q8_0 above; q8_1 ggml-quants.c:219-252; q8_K :2479-2516 ---- */
static void quantize_row_q8_1(const float * x, blk_q8_1 * y, int64_t k) {
    for (int64_t i = 0; i < k / 32; ++i) {
        float amax = 0.0f;
        for (int j = 0; j < 32; ++j) { const float v = fabsf(x[i*32 + j]); if (v > amax) amax = v; }
        const float d = amax / 127; const float id = d ? 1.0f / d : 0.0f;
        y[i].d = f2h(d);
        int sum = 0;
        for (int j = 0; j < 32; ++j) { y[i].qs[j] = (int8_t) roundf(x[i*32 + j] * id); sum += y[i].qs[j]; }
        y[i].s = f2h((float) sum * d);
    }
}
static int nearest_int(float fval) { float val = fval + 12582912.f; int i; memcpy(&i, &val, sizeof(int)); return (i & 0x007fffff) - 0x00400000; }
static void quantize_row_q8_K(const float * x, blk_q8_K * y, int64_t k) {
    for (int64_t i = 0; i < k / 256; ++i, x += 256) {
        float max = 0, amax = 0;
        for (int j = 0; j < 256; ++j) { const float ax = fabsf(x[j]); if (ax > amax) { amax = ax; max = x[j]; } }
        if (!amax) { y[i].d = 0; memset(y[i].qs, 0, 256); memset(y[i].bsums, 0, sizeof(y[i].bsums)); continue; }
        const float iscale = -127.f / max;
        for (int j = 0; j < 256; ++j) { const int v = nearest_int(iscale * x[j]); y[i].qs[j] = (int8_t) MINI(127, v); }
        for (int j = 0; j < 16; ++j) { int sum = 0; for (int ii = 0; ii < 16; ++ii) sum += y[i].qs[j*16 + ii]; y[i].bsums[j] = (int16_t) sum; }
        y[i].d = 1 / iscale;
    }
}

/* ---- vec_dot, scalar forms (ggml/src/ggml-cpu/ggml-cpu-quants.c: q4_0 1842 (tail :2360-2378),
 *      q4_1 2380, q5_0 2700, q5_1 3080, q8_0 3533, q4_K 6115 (scalar :6800-6858), q5_K 6859, q6_K 7594) ---- */
static float vec_dot(int type, int64_t k, const void * vx, const void * vy) {
    float sumf = 0.0f;
    switch (type) {
        case T_Q4_0: { const blk_q4_0 * x = vx; const blk_q8_0 * y = vy;
            for (int64_t i = 0; i < k / 32; ++i) { int s0 = 0, s1 = 0;
                for (int j = 0; j < 16; ++j) { s0 += ((x[i].qs[j] & 0x0F) - 8) * y[i].qs[j]; s1 += ((x[i].qs[j] >> 4) - 8) * y[i].qs[j + 16]; }
                sumf += (float) (s0 + s1) * h2f(x[i].d) * h2f(y[i].d); }
            return sumf; }
        case T_Q4_1: { const blk_q4_1 * x = vx; const blk_q8_1 * y = vy;
            for (int64_t i = 0; i < k / 32; ++i) { int s0 = 0, s1 = 0;
                for (int j = 0; j < 16; ++j) { s0 += (x[i].qs[j] & 0x0F) * y[i].qs[j]; s1 += (x[i].qs[j] >> 4) * y[i].qs[j + 16]; }
                sumf += (h2f(x[i].d) * h2f(y[i].d)) * (float) (s0 + s1) + h2f(x[i].m) * h2f(y[i].s); }
            return sumf; }
        case T_Q5_0: { const blk_q5_0 * x = vx; const blk_q8_0 * y = vy;
            for (int64_t i = 0; i < k / 32; ++i) { uint32_t qh; memcpy(&qh, x[i].qh, 4); int s0 = 0, s1 = 0;
                for (int j = 0; j < 16; ++j) { const uint8_t xh0 = (uint8_t) (((qh & (1u << (j + 0))) >> (j + 0)) << 4), xh1 = (uint8_t) ((qh & (1u << (j + 16))) >> (j + 12));
                    s0 += (int8_t) (((x[i].qs[j] & 0x0F) | xh0) - 16) * y[i].qs[j]; s1 += (int8_t) (((x[i].qs[j] >> 4) | xh1) - 16) * y[i].qs[j + 16]; }
                sumf += (h2f(x[i].d) * h2f(y[i].d)) * (float) (s0 + s1); }
            return sumf; }
        case T_Q5_1: { const blk_q5_1 * x = vx; const blk_q8_1 * y = vy;
            for (int64_t i = 0; i < k / 32; ++i) { uint32_t qh; memcpy(&qh, x[i].qh, 4); int s0 = 0, s1 = 0;
                for (int j = 0; j < 16; ++j) { const uint8_t xh0 = (uint8_t) (((qh >> (j + 0)) << 4) & 0x10), xh1 = (uint8_t) ((qh >> (j + 12)) & 0x10);
                    s0 += ((x[i].qs[j] & 0xF) | xh0) * y[i].qs[j]; s1 += ((x[i].qs[j] >> 4) | xh1) * y[i].qs[j + 16]; }
                sumf += (h2f(x[i].d) * h2f(y[i].d)) * (float) (s0 + s1) + h2f(x[i].m) * h2f(y[i].s); }
            return sumf; }
        case T_Q8_0: { const blk_q8_0 * x = vx; const blk_q8_0 * y = vy;
            for (int64_t i = 0; i < k / 32; ++i) { int s = 0; for (int j = 0; j < 32; ++j) s += x[i].qs[j] * y[i].qs[j];
                sumf += (float) s * (h2f(x[i].d) * h2f(y[i].d)); }
            return sumf; }
        case T_Q2_K: { const blk_q2_K * x = vx; const blk_q8_K * y = vy;            /* scalar form, ggml-cpu-quants.c:5058-5096 */
            for (int64_t i = 0; i < k / 256; ++i) {
                int mins = 0, isum = 0;
                for (int sb = 0; sb < 16; ++sb) mins += y[i].bsums[sb] * (x[i].scales[sb] >> 4);
                for (int sb = 0; sb < 16; ++sb) { const int n = sb >> 3, j = (sb & 7) >> 1, half = sb & 1;
                    int part = 0;
                    for (int l = 0; l < 16; ++l) part += y[i].qs[sb * 16 + l] * ((x[i].qs[n * 32 + half * 16 + l] >> (2 * j)) & 3);
                    isum += (x[i].scales[sb] & 0xF) * part; }
                const float dall = y[i].d * h2f(x[i].d), dmin = y[i].d * h2f(x[i].dmin);
                sumf += dall * (float) isum - dmin * (float) mins; }
            return sumf; }
        case T_Q3_K: { const blk_q3_K * x = vx; const blk_q8_K * y = vy;            /* scalar form, ggml-cpu-quants.c:6041-6108: eight running sums */
            float sums[8] = {0};
            for (int64_t i = 0; i < k / 256; ++i) {
                int32_t part[8] = {0};
                for (int e = 0; e < 256; ++e) { const int n = e >> 7, j = (e & 127) >> 5, l = e & 31;
                    const int q = ((x[i].qs[n * 32 + l] >> (2 * j)) & 3) - (((x[i].hmask[l] >> (4 * n + j)) & 1) ? 0 : 4);
                    part[e & 7] += (q3k_scale6(x[i].scales, e >> 4) - 32) * (y[i].qs[e] * q); }
                const float d = h2f(x[i].d) * y[i].d;
                for (int l = 0; l < 8; ++l) sums[l] += d * (float) part[l]; }
            for (int l = 0; l < 8; ++l) sumf += sums[l];
            return sumf; }
        case T_IQ4_NL: { const blk_iq4_nl * x = vx; const blk_q8_0 * y = vy;        /* ggml-cpu-quants.c:11188 (scalar tail) */
            for (int64_t i = 0; i < k / 32; ++i) { int s0 = 0, s1 = 0;
                for (int j = 0; j < 16; ++j) { s0 += y[i].qs[j] * iq4nl_values[x[i].qs[j] & 0xF]; s1 += y[i].qs[j + 16] * iq4nl_values[x[i].qs[j] >> 4]; }
                sumf += h2f(y[i].d) * h2f(x[i].d) * (float) (s0 + s1); }
            return sumf; }
        case T_IQ4_XS: { const blk_iq4_xs * x = vx; const blk_q8_K * y = vy;        /* scalar form, ggml-cpu-quants.c:11646-11676 */
            for (int64_t i = 0; i < k / 256; ++i) { const float dd = h2f(x[i].d) * y[i].d;
                for (int ib = 0; ib < 8; ++ib) { const uint8_t * qs = x[i].qs + 16 * ib; const int8_t * q8 = y[i].qs + 32 * ib; int s0 = 0, s1 = 0;
                    for (int j = 0; j < 16; ++j) { s0 += q8[j] * iq4nl_values[qs[j] & 0xF]; s1 += q8[j + 16] * iq4nl_values[qs[j] >> 4]; }
                    sumf += dd * (float) iq4xs_scale(&x[i], ib) * (float) (s0 + s1); } }
            return sumf; }
        case T_Q4_K: case T_Q5_K: {
            const blk_q8_K * y = vy;
            for (int64_t i = 0; i < k / 256; ++i) {
                const uint8_t * scales; const uint8_t * qs; const uint8_t * qh = NULL; uint16_t dh, dmh;
                if (type == T_Q4_K) { const blk_q4_K * x = (const blk_q4_K *) vx + i; scales = x->scales; qs = x->qs; dh = x->d; dmh = x->dmin; }
                else { const blk_q5_K * x = (const blk_q5_K *) vx + i; scales = x->scales; qs = x->qs; qh = x->qh; dh = x->d; dmh = x->dmin; }
                int32_t sum_sc = 0, sum_min = 0;
                for (int sb = 0; sb < 8; ++sb) {
                    uint8_t sc, m; scale_min_k4(sb, scales, &sc, &m);
                    int s = 0;
                    for (int l = 0; l < 32; ++l) {
                        const uint8_t byte = qs[(sb >> 1) * 32 + l];
                        int q = (sb & 1) ? (byte >> 4) : (byte & 0xF);
                        if (qh && ((qh[l] >> sb) & 1)) q += 16;
                        s += q * y[i].qs[sb * 32 + l];
                    }
                    sum_sc += (int32_t) sc * s;
                    sum_min += (int32_t) m * (y[i].bsums[2 * sb] + y[i].bsums[2 * sb + 1]);
                }
                sumf += h2f(dh) * y[i].d * (float) sum_sc - h2f(dmh) * y[i].d * (float) sum_min;
            }
            return sumf; }
        case T_Q6_K: { const blk_q6_K * x = vx; const blk_q8_K * y = vy;
            for (int64_t i = 0; i < k / 256; ++i) {
                int32_t acc = 0;
                for (int n = 0; n < 2; ++n) for (int l = 0; l < 32; ++l) {
                    const uint8_t * ql = x[i].ql + 64 * n; const uint8_t * qh = x[i].qh + 32 * n; const int8_t * sc = x[i].scales + 8 * n; const int8_t * q8 = y[i].qs + 128 * n;
                    const int is = l / 16;
                    const int q1 = (int8_t) ((ql[l] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32, q2 = (int8_t) ((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
                    const int q3 = (int8_t) ((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32, q4 = (int8_t) ((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
                    acc += sc[is] * q1 * q8[l] + sc[is + 2] * q2 * q8[l + 32] + sc[is + 4] * q3 * q8[l + 64] + sc[is + 6] * q4 * q8[l + 96];
                }
                sumf += h2f(x[i].d) * y[i].d * (float) acc;
            }
            return sumf; }
    }
    return NAN;
}

/* ---- GGML_OP_MUL_MAT as the CPU backend computes it (ggml_compute_forward_mul_mat,
 *      ggml/src/ggml-cpu/ggml-cpu.c:7443-7635): src1 rows are quantized to the weight type's
 *      vec_dot_type, then dst[n][m] = vec_dot(W row m, quantized X row n) ---- */
EXPORT int oracle_mul_mat(int type, const void * W, int64_t M, int64_t K, const float * X, int64_t N, float * dst) {
    const int64_t wrs = oracle_row_size(type, K);
    if (!wrs) return -1;
    int64_t yrs;
    if (type == T_Q4_0 || type == T_Q5_0 || type == T_Q8_0 || type == T_IQ4_NL) yrs = K / 32 * (int64_t) sizeof(blk_q8_0);
    else if (type == T_Q4_1 || type == T_Q5_1) yrs = K / 32 * (int64_t) sizeof(blk_q8_1);
    else yrs = K / 256 * (int64_t) sizeof(blk_q8_K);
    uint8_t * yq = malloc((size_t) yrs);
    if (!yq) return -2;
    for (int64_t n = 0; n < N; ++n) {
        if (type == T_Q4_0 || type == T_Q5_0 || type == T_Q8_0 || type == T_IQ4_NL) oracle_quantize_row(T_Q8_0, X + n * K, yq, K);
        else if (type == T_Q4_1 || type == T_Q5_1) quantize_row_q8_1(X + n * K, (blk_q8_1 *) yq, K);
        else quantize_row_q8_K(X + n * K, (blk_q8_K *) yq, K);
        for (int64_t m = 0; m < M; ++m) dst[n * M + m] = vec_dot(type, K, (const uint8_t *) W + m * wrs, yq);
    }
    free(yq);
    return 0;
}

/* plain float product of dequantized weights (what the quantized product approximates) */
EXPORT int oracle_mul_mat_f32(int type, const void * W, int64_t M, int64_t K, const float * X, int64_t N, float * dst) {
    const int64_t wrs = oracle_row_size(type, K);
    float * row = malloc((size_t) K * 4);
    if (!wrs || !row) { free(row); return -1; }
    for (int64_t m = 0; m < M; ++m) {
        oracle_dequantize_row(type, (const uint8_t *) W + m * wrs, row, K);
        for (int64_t n = 0; n < N; ++n) { double s = 0; for (int64_t k = 0; k < K; ++k) s += (double) row[k] * X[n * K + k]; dst[n * M + m] = (float) s; }
    }
    free(row);
    return 0;
}

/* ---- GGML_OP_FLASH_ATTN_EXT as the CPU backend computes it for F16 K/V
 *      (ggml_compute_forward_flash_attn_ext_f16, ggml/src/ggml-cpu/ggml-cpu.c:10916-11129):
 *      per query row, Q is rounded to F16 (K's vec_dot_type), s = scale * K.Q (+softcap) + slope*mask,
 *      rows with mask -inf are skipped, online softmax with the V accumulator kept in F16.
 *      q f32 [n_head][n_q][D], k/v f16 [n_head_kv][n_kv][D], mask f16 [n_q][n_kv] or NULL,
 *      dst f32 [n_q][n_head][D] ---- */
EXPORT int oracle_flash_attn(const float * q, const uint16_t * k, const uint16_t * v, const uint16_t * mask, float * dst,
                             int64_t D, int64_t n_q, int64_t n_head, int64_t n_kv, int64_t n_head_kv,
                             float scale, float max_bias, float softcap) {
    const int64_t gqa = n_head / n_head_kv;
    uint32_t n_head_log2 = 1; while (n_head_log2 * 2 <= (uint32_t) n_head) n_head_log2 *= 2;
    const float m0 = powf(2.0f, -max_bias / (float) n_head_log2), m1 = powf(2.0f, -(max_bias / 2.0f) / (float) n_head_log2);
    if (softcap != 0.0f) scale /= softcap;
    uint16_t * q16 = malloc((size_t) D * 2), * acc16 = malloc((size_t) D * 2);
    if (!q16 || !acc16) { free(q16); free(acc16); return -1; }
    for (int64_t h = 0; h < n_head; ++h) for (int64_t iq = 0; iq < n_q; ++iq) {
        const float slope = max_bias > 0.0f ? (h < (int64_t) n_head_log2 ? powf(m0, (float) (h + 1)) : powf(m1, (float) (2 * (h - n_head_log2) + 1))) : 1.0f;
        oracle_f32_to_f16(q + (h * n_q + iq) * D, q16, D);
        for (int64_t d = 0; d < D; ++d) acc16[d] = 0;
        float S = 0.0f, Mx = -INFINITY;
        const uint16_t * kh = k + (h / gqa) * n_kv * D, * vh = v + (h / gqa) * n_kv * D;
        for (int64_t ic = 0; ic < n_kv; ++ic) {
            const float mv = mask ? slope * h2f(mask[iq * n_kv + ic]) : 0.0f;
            if (mv == -INFINITY) continue;
            float s = 0.0f;
            for (int64_t d = 0; d < D; ++d) s += h2f(kh[ic * D + d]) * h2f(q16[d]);
            s = s * scale;
            if (softcap != 0.0f) s = softcap * tanhf(s);
            s += mv;
            const float Mold = Mx;
            float ms = 1.0f, vs = 1.0f;
            if (s > Mx) { Mx = s; ms = expf(Mold - Mx); for (int64_t d = 0; d < D; ++d) acc16[d] = f2h(h2f(acc16[d]) * ms); }
            else { vs = expf(s - Mx); }
            for (int64_t d = 0; d < D; ++d) acc16[d] = f2h(fmaf(h2f(vh[ic * D + d]), vs, h2f(acc16[d])));
            S = S * ms + vs;
        }
        const float Sinv = 1.0f / S;
        for (int64_t d = 0; d < D; ++d) dst[(iq * n_head + h) * D + d] = h2f(acc16[d]) * Sinv;
    }
    free(q16); free(acc16);
    return 0;
}

/* ---- glue ops ---- */
/* ggml_compute_forward_rms_norm_f32, ggml/src/ggml-cpu/ggml-cpu.c:7015-7061 (sum in double) */
EXPORT void oracle_rms_norm(const float * x, int64_t rows, int64_t k, float eps, const float * w, float * y) {
    for (int64_t r = 0; r < rows; ++r) {
        double sum = 0.0;
        for (int64_t i = 0; i < k; ++i) sum += (double) x[r*k + i] * x[r*k + i];
        const float mean = (float) (sum / (double) k), scale = 1.0f / sqrtf(mean + eps);
        for (int64_t i = 0; i < k; ++i) { float v = x[r*k + i] * scale; if (w) v *= w[i]; y[r*k + i] = v; }
    }
}
/* silu then mul: ggml_compute_forward_silu_f32 (ggml-cpu.c:6360ff), x/(1+exp(-x)) */
EXPORT void oracle_silu_mul(const float * g, const float * u, int64_t n, float * y) {
    for (int64_t i = 0; i < n; ++i) y[i] = (g[i] / (1.0f + expf(-g[i]))) * u[i];
}
/* ggml_compute_forward_soft_max_f32, ggml-cpu.c:8900ff (no ALiBi) */
EXPORT void oracle_soft_max(const float * x, int64_t rows, int64_t k, const uint16_t * mask, float scale, float * y) {
    for (int64_t r = 0; r < rows; ++r) {
        float mx = -INFINITY;
        for (int64_t i = 0; i < k; ++i) { float v = x[r*k + i] * scale + (mask ? h2f(mask[r*k + i]) : 0.0f); y[r*k + i] = v; if (v > mx) mx = v; }
        double sum = 0.0;
        for (int64_t i = 0; i < k; ++i) { const float e = expf(y[r*k + i] - mx); y[r*k + i] = e; sum += e; }
        const float inv = (float) (1.0 / sum);
        for (int64_t i = 0; i < k; ++i) y[r*k + i] *= inv;
    }
}
/* ggml_compute_forward_rope_f32 with YaRN (ggml-cpu.c:9275-9306, 9366-9540; corr dims ggml.c ggml_rope_yarn_corr_dims).
 * x, y: [n_tok][n_head][head_dim]; mode 0 = adjacent pairs, 2 = NeoX halves */
EXPORT void oracle_rope(const float * x, int64_t hd, int64_t n_head, int64_t n_tok, const int32_t * pos, const float * ff,
                        int n_dims, int mode, int n_ctx_orig, float freq_base, float freq_scale, float ext_factor,
                        float attn_factor, float beta_fast, float beta_slow, float * y) {
    const float theta_scale = powf(freq_base, -2.0f / (float) n_dims);
    const float c0 = (float) n_dims * logf((float) n_ctx_orig / (beta_fast * 2.0f * (float) M_PI)) / (2.0f * logf(freq_base));
    const float c1 = (float) n_dims * logf((float) n_ctx_orig / (beta_slow * 2.0f * (float) M_PI)) / (2.0f * logf(freq_base));
    const float corr0 = fmaxf(0.0f, floorf(c0)), corr1 = fminf((float) n_dims - 1.0f, ceilf(c1));
    for (int64_t t = 0; t < n_tok; ++t) for (int64_t h = 0; h < n_head; ++h) {
        const float * xs = x + (t * n_head + h) * hd; float * yd = y + (t * n_head + h) * hd;
        float theta = (float) pos[t];
        for (int64_t i0 = 0; i0 < hd; i0 += 2) {
            if (i0 >= n_dims) { yd[i0] = xs[i0]; yd[i0 + 1] = xs[i0 + 1]; continue; }
            const float f = ff ? ff[i0 / 2] : 1.0f;
            const float theta_extrap = theta / f, theta_interp = freq_scale * theta_extrap;
            float th = theta_interp, mscale = attn_factor;
            if (ext_factor != 0.0f) {
                const float yy = ((float) (i0 / 2) - corr0) / fmaxf(0.001f, corr1 - corr0);
                const float ramp = (1.0f - fminf(1.0f, fmaxf(0.0f, yy))) * ext_factor;
                th = theta_interp * (1.0f - ramp) + theta_extrap * ramp;
                mscale *= 1.0f + 0.1f * logf(1.0f / freq_scale);
            }
            const float c = cosf(th) * mscale, s = sinf(th) * mscale;
            const int64_t ia = (mode & 2) ? i0 / 2 : i0, ib = (mode & 2) ? i0 / 2 + n_dims / 2 : i0 + 1;
            yd[ia] = xs[ia] * c - xs[ib] * s; yd[ib] = xs[ia] * s + xs[ib] * c;
            theta *= theta_scale;
        }
    }
}
