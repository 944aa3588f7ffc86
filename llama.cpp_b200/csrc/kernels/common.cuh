// Shared device-side definitions for the B200 ggml backend kernels.
//
// Block layouts restate the on-disk/in-memory quantization formats of ggml
// (ggml/src/ggml-common.h:161-328).  They are byte-for-byte contracts, so the
// sizes are pinned with static_asserts.  Nothing in this directory includes a
// ggml header: the kernels take plain pointers, sizes and byte strides.
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace b200 {

// ggml_type values used by the kernels (ggml/include/ggml.h:351-392).
enum : int {
    T_F32 = 0, T_F16 = 1, T_Q4_0 = 2, T_Q4_1 = 3, T_Q5_0 = 6, T_Q5_1 = 7, T_Q8_0 = 8,
    T_Q2_K = 10, T_Q3_K = 11, T_Q4_K = 12, T_Q5_K = 13, T_Q6_K = 14,
    T_IQ4_NL = 20, T_IQ4_XS = 23, T_I32 = 26, T_BF16 = 30,
};

#pragma pack(push, 1)
struct blk_q4_0 { uint16_t d; uint8_t qs[16]; };                                            // 18 B / 32 w
struct blk_q4_1 { uint16_t d; uint16_t m; uint8_t qs[16]; };                                // 20 B / 32 w
struct blk_q5_0 { uint16_t d; uint8_t qh[4]; uint8_t qs[16]; };                             // 22 B / 32 w
struct blk_q5_1 { uint16_t d; uint16_t m; uint8_t qh[4]; uint8_t qs[16]; };                 // 24 B / 32 w
struct blk_q8_0 { uint16_t d; int8_t qs[32]; };                                             // 34 B / 32 w
struct blk_q4_K { uint16_t d; uint16_t dmin; uint8_t scales[12]; uint8_t qs[128]; };        // 144 B / 256 w
struct blk_q5_K { uint16_t d; uint16_t dmin; uint8_t scales[12]; uint8_t qh[32]; uint8_t qs[128]; }; // 176 B
struct blk_q6_K { uint8_t ql[128]; uint8_t qh[64]; int8_t scales[16]; uint16_t d; };        // 210 B / 256 w
struct blk_q2_K { uint8_t scales[16]; uint8_t qs[64]; uint16_t d; uint16_t dmin; };         // 84 B / 256 w
struct blk_q3_K { uint8_t hmask[32]; uint8_t qs[64]; uint8_t scales[12]; uint16_t d; };     // 110 B / 256 w
struct blk_iq4_nl { uint16_t d; uint8_t qs[16]; };                                          // 18 B / 32 w
struct blk_iq4_xs { uint16_t d; uint16_t scales_h; uint8_t scales_l[4]; uint8_t qs[128]; }; // 136 B / 256 w
#pragma pack(pop)
static_assert(sizeof(blk_q4_0) == 18 && sizeof(blk_q4_1) == 20 && sizeof(blk_q5_0) == 22, "block size");
static_assert(sizeof(blk_q5_1) == 24 && sizeof(blk_q8_0) == 34, "block size");
static_assert(sizeof(blk_q4_K) == 144 && sizeof(blk_q5_K) == 176 && sizeof(blk_q6_K) == 210, "block size");
static_assert(sizeof(blk_q2_K) == 84 && sizeof(blk_q3_K) == 110 && sizeof(blk_iq4_nl) == 18 && sizeof(blk_iq4_xs) == 136, "block size");

// Activation blocks produced on the device for the integer dot products:
// 128 consecutive values of one activation column = 4 groups of 32 int8 plus,
// per group, {d, s} with d = amax/127 and s = d * sum(q).  160 bytes, so every
// block (and any run of blocks) is a legal bulk-copy source (16-byte multiple).
struct blk_act128 { int8_t q[128]; float2 ds[4]; };
static_assert(sizeof(blk_act128) == 160, "activation block size");

__host__ __device__ inline int type_block_elems(int t) {
    switch (t) {
        case T_F32: case T_F16: case T_BF16: case T_I32: return 1;
        case T_Q4_0: case T_Q4_1: case T_Q5_0: case T_Q5_1: case T_Q8_0: case T_IQ4_NL: return 32;
        case T_Q2_K: case T_Q3_K: case T_Q4_K: case T_Q5_K: case T_Q6_K: case T_IQ4_XS: return 256;
        default: return 0;
    }
}
__host__ __device__ inline int type_block_bytes(int t) {
    switch (t) {
        case T_F32: case T_I32: return 4;
        case T_F16: case T_BF16: return 2;
        case T_Q4_0: return 18; case T_Q4_1: return 20; case T_Q5_0: return 22; case T_Q5_1: return 24;
        case T_Q8_0: return 34; case T_Q4_K: return 144; case T_Q5_K: return 176; case T_Q6_K: return 210;
        case T_Q2_K: return 84; case T_Q3_K: return 110; case T_IQ4_NL: return 18; case T_IQ4_XS: return 136;
        default: return 0;
    }
}

__device__ __forceinline__ float h2f(uint16_t h) { return __half2float(__ushort_as_half(h)); }

// 6-bit scale / min of sub-block j of a Q4_K / Q5_K super-block
// (get_scale_min_k4, ggml/src/ggml-quants.c:631-638).
__device__ __forceinline__ void k4_scale_min(int j, const uint8_t * q, int & sc, int & m) {
    if (j < 4) {
        sc = q[j] & 63;
        m  = q[j + 4] & 63;
    } else {
        sc = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4);
        m  = (q[j + 4] >> 4)  | ((q[j]     >> 6) << 4);
    }
}

// Value of element `i` (0 <= i < K) of a quantized row, computed with exactly
// the operation order of the reference dequantize_row_* functions and with no
// fused multiply-add, so that results are bit-identical to the CPU code:
//   q4_0 ggml-quants.c:255-273   q4_1 :275-294   q5_0 :296-320   q5_1 :322-347
//   q8_0 :349-363   q4_K :1280-1302   q5_K :1482-1507   q6_K :1690-1719
//   q2_K :712-744   q3_K :1056-1106   iq4_nl :2434-2451   iq4_xs :2453-2475
template <int T> __device__ __forceinline__ float dequant_elem(const uint8_t * row, int64_t i);

template <> __device__ __forceinline__ float dequant_elem<T_F32>(const uint8_t * row, int64_t i) {
    return ((const float *) row)[i];
}
template <> __device__ __forceinline__ float dequant_elem<T_F16>(const uint8_t * row, int64_t i) {
    return __half2float(((const __half *) row)[i]);
}
template <> __device__ __forceinline__ float dequant_elem<T_BF16>(const uint8_t * row, int64_t i) {
    return __bfloat162float(((const __nv_bfloat16 *) row)[i]);
}
template <> __device__ __forceinline__ float dequant_elem<T_Q4_0>(const uint8_t * row, int64_t i) {
    const blk_q4_0 * b = (const blk_q4_0 *) row + (i >> 5);
    const int j = i & 31;
    const int q = j < 16 ? (b->qs[j] & 0x0F) : (b->qs[j - 16] >> 4);
    return __fmul_rn((float) (q - 8), h2f(b->d));
}
template <> __device__ __forceinline__ float dequant_elem<T_Q4_1>(const uint8_t * row, int64_t i) {
    const blk_q4_1 * b = (const blk_q4_1 *) row + (i >> 5);
    const int j = i & 31;
    const int q = j < 16 ? (b->qs[j] & 0x0F) : (b->qs[j - 16] >> 4);
    return __fadd_rn(__fmul_rn((float) q, h2f(b->d)), h2f(b->m));
}
template <> __device__ __forceinline__ float dequant_elem<T_Q5_0>(const uint8_t * row, int64_t i) {
    const blk_q5_0 * b = (const blk_q5_0 *) row + (i >> 5);
    const int j = i & 31;
    const uint32_t qh = b->qh[0] | (b->qh[1] << 8) | (b->qh[2] << 16) | ((uint32_t) b->qh[3] << 24);
    const int lo = j < 16 ? (b->qs[j] & 0x0F) : (b->qs[j - 16] >> 4);
    const int q  = lo | (((qh >> j) & 1) << 4);
    return __fmul_rn((float) (q - 16), h2f(b->d));
}
template <> __device__ __forceinline__ float dequant_elem<T_Q5_1>(const uint8_t * row, int64_t i) {
    const blk_q5_1 * b = (const blk_q5_1 *) row + (i >> 5);
    const int j = i & 31;
    const uint32_t qh = b->qh[0] | (b->qh[1] << 8) | (b->qh[2] << 16) | ((uint32_t) b->qh[3] << 24);
    const int lo = j < 16 ? (b->qs[j] & 0x0F) : (b->qs[j - 16] >> 4);
    const int q  = lo | (((qh >> j) & 1) << 4);
    return __fadd_rn(__fmul_rn((float) q, h2f(b->d)), h2f(b->m));
}
template <> __device__ __forceinline__ float dequant_elem<T_Q8_0>(const uint8_t * row, int64_t i) {
    const blk_q8_0 * b = (const blk_q8_0 *) row + (i >> 5);
    return __fmul_rn((float) b->qs[i & 31], h2f(b->d));
}
template <> __device__ __forceinline__ float dequant_elem<T_Q4_K>(const uint8_t * row, int64_t i) {
    const blk_q4_K * b = (const blk_q4_K *) row + (i >> 8);
    const int r = i & 255, sub = r >> 5, l = r & 31;
    int sc, m; k4_scale_min(sub, b->scales, sc, m);
    const float d1 = __fmul_rn(h2f(b->d), (float) sc);
    const float m1 = __fmul_rn(h2f(b->dmin), (float) m);
    const uint8_t byte = b->qs[(sub >> 1) * 32 + l];
    const int q = (sub & 1) ? (byte >> 4) : (byte & 0xF);
    return __fsub_rn(__fmul_rn(d1, (float) q), m1);
}
template <> __device__ __forceinline__ float dequant_elem<T_Q5_K>(const uint8_t * row, int64_t i) {
    const blk_q5_K * b = (const blk_q5_K *) row + (i >> 8);
    const int r = i & 255, sub = r >> 5, l = r & 31;
    int sc, m; k4_scale_min(sub, b->scales, sc, m);
    const float d1 = __fmul_rn(h2f(b->d), (float) sc);
    const float m1 = __fmul_rn(h2f(b->dmin), (float) m);
    const uint8_t byte = b->qs[(sub >> 1) * 32 + l];
    const int q = ((sub & 1) ? (byte >> 4) : (byte & 0xF)) + (((b->qh[l] >> sub) & 1) ? 16 : 0);
    return __fsub_rn(__fmul_rn(d1, (float) q), m1);
}
template <> __device__ __forceinline__ float dequant_elem<T_Q6_K>(const uint8_t * row, int64_t i) {
    const blk_q6_K * b = (const blk_q6_K *) row + (i >> 8);
    const int r = i & 255, n = r >> 7, rr = r & 127, grp = rr >> 5, l = rr & 31;
    const uint8_t qlb = b->ql[n * 64 + (grp & 1) * 32 + l];
    const int lo = (grp & 2) ? (qlb >> 4) : (qlb & 0xF);
    const int hi = (b->qh[n * 32 + l] >> (2 * grp)) & 3;
    const int q  = (int) (int8_t) (lo | (hi << 4)) - 32;
    const int sc = b->scales[n * 8 + (l >> 4) + 2 * grp];
    return __fmul_rn(__fmul_rn(h2f(b->d), (float) sc), (float) q);
}

// Q2_K: 16 sub-blocks of 16 weights; scales[s] = 4-bit scale | 4-bit min << 4; weight l of the 128-half n, 32-run j
// is bits [2j, 2j+2) of qs[32 n + l]
template <> __device__ __forceinline__ float dequant_elem<T_Q2_K>(const uint8_t * row, int64_t i) {
    const blk_q2_K * b = (const blk_q2_K *) row + (i >> 8);
    const int r = i & 255, n = r >> 7, j = (r & 127) >> 5, l = r & 31;
    const uint8_t sc = b->scales[n * 8 + 2 * j + (l >> 4)];
    const float dl = __fmul_rn(h2f(b->d), (float) (sc & 0xF));
    const float ml = __fmul_rn(h2f(b->dmin), (float) (sc >> 4));
    const int q = (b->qs[n * 32 + l] >> (2 * j)) & 3;
    return __fsub_rn(__fmul_rn(dl, (float) q), ml);
}
// 6-bit scale s (0..15) of a Q3_K super-block, before the -32 offset (the aux[] shuffle of ggml-quants.c:1075-1080)
__device__ __forceinline__ int q3k_scale(const uint8_t * scales, int s) {
    const int lo = s < 8 ? (scales[s] & 0xF) : (scales[s - 8] >> 4);
    const int hi = (scales[8 + (s & 3)] >> (2 * (s >> 2))) & 3;
    return lo | (hi << 4);
}
// Q3_K: low 2 bits as Q2_K, third bit in hmask[l] bit (4 n + j); a clear bit subtracts 4
template <> __device__ __forceinline__ float dequant_elem<T_Q3_K>(const uint8_t * row, int64_t i) {
    const blk_q3_K * b = (const blk_q3_K *) row + (i >> 8);
    const int r = i & 255, n = r >> 7, j = (r & 127) >> 5, l = r & 31;
    const float dl = __fmul_rn(h2f(b->d), (float) (q3k_scale(b->scales, n * 8 + 2 * j + (l >> 4)) - 32));
    const int q = ((b->qs[n * 32 + l] >> (2 * j)) & 3) - (((b->hmask[l] >> (4 * n + j)) & 1) ? 0 : 4);
    return __fmul_rn(dl, (float) q);
}
// IQ4_NL: Q4_0 layout with the nibble mapped through the 16-entry non-linear table of the format
// (kvalues_iq4nl, ggml-quants.c:2434), held here as two 64-bit words of int8
__device__ __forceinline__ int iq4nl_value(int idx) {
    const uint64_t t = idx < 8 ? 0xF6EADDCFBFAD9881ull : 0x7159453526190D01ull;
    return (int) (int8_t) (t >> (8 * (idx & 7)));
}
// four table lookups at once: two byte permutes over the table halves and a select on bit 3 of each index
__device__ __forceinline__ uint32_t iq4nl_lut4(uint32_t idx) {          // idx: four byte lanes, each 0..15
    const uint32_t s = idx & 0x07070707u, t = s | (s >> 4);
    const uint32_t sel = (t & 0xFFu) | ((t >> 8) & 0xFF00u);
    const uint32_t lo = __byte_perm(0xBFAD9881u, 0xF6EADDCFu, sel), hi = __byte_perm(0x26190D01u, 0x71594535u, sel);
    const uint32_t m = ((idx >> 3) & 0x01010101u) * 0xFFu;
    return (lo & ~m) | (hi & m);
}
template <> __device__ __forceinline__ float dequant_elem<T_IQ4_NL>(const uint8_t * row, int64_t i) {
    const blk_iq4_nl * b = (const blk_iq4_nl *) row + (i >> 5);
    const int j = i & 31;
    const int q = j < 16 ? (b->qs[j] & 0x0F) : (b->qs[j - 16] >> 4);
    return __fmul_rn(h2f(b->d), (float) iq4nl_value(q));
}

// IQ4_XS: eight 32-weight sub-blocks in IQ4_NL coding, each with a 6-bit scale (offset 32): low nibble in
// scales_l, two high bits in scales_h
__device__ __forceinline__ int iq4xs_scale(const uint8_t * blk, int ib) {
    const int h = blk[2] | (blk[3] << 8);
    return (((blk[4 + (ib >> 1)] >> (4 * (ib & 1))) & 0xF) | (((h >> (2 * ib)) & 3) << 4)) - 32;
}
template <> __device__ __forceinline__ float dequant_elem<T_IQ4_XS>(const uint8_t * row, int64_t i) {
    const uint8_t * b = row + (i >> 8) * 136;
    const int r = i & 255, ib = r >> 5, j = r & 31;
    const float dl = __fmul_rn(h2f(*(const uint16_t *) b), (float) iq4xs_scale(b, ib));
    const uint8_t byte = b[8 + ib * 16 + (j & 15)];
    return __fmul_rn(dl, (float) iq4nl_value(j < 16 ? (byte & 0x0F) : (byte >> 4)));
}

// ---------------------------------------------------------------------------
// Asynchronous bulk copies (global -> shared) completed on an mbarrier.  Only
// the plain, non-multicast form is used anywhere in this backend.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void * p) { return (uint32_t) __cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t * bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t * bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t * bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t * bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: gives up after `limit` polls (each poll itself blocks for a
// hardware-defined time slice) and reports failure instead of spinning forever.
__device__ __forceinline__ bool mbar_wait(uint64_t * bar, uint32_t parity, int limit = (1 << 22)) {
    for (int i = 0; i < limit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
    }
    return false;
}
__device__ __forceinline__ void bulk_g2s(void * dst_smem, const void * src_gmem, uint32_t bytes, uint64_t * bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        :: "r"(smem_u32(dst_smem)), "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

// programmatic dependent launch: everything before pdl_wait() may overlap the
// tail of the previous kernel in the stream (it must not read that kernel's output)
__device__ __forceinline__ void pdl_wait()              { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Both halves of programmatic dependent launch at the top of a kernel that has nothing to prefetch:
// let the next kernel in the stream start its own prologue now, then wait until everything this
// kernel depends on has completed and is visible.  No-ops when launched without the attribute.
__device__ __forceinline__ void pdl_enter() { pdl_launch_dependents(); pdl_wait(); }

// error codes written to the device status word by kernels that give up a wait
enum : int { ERR_NONE = 0, ERR_MBAR_TIMEOUT = 1, ERR_BAD_ARG = 2, ERR_PEER_TIMEOUT = 3 };

static thread_local cudaError_t launch_err = cudaSuccess;   // result of the most recent launch_k in this translation unit

// host-side launch through cudaLaunchKernelEx so that the programmatic-serialization attribute can be set
template <typename... KArgs, typename... Args>
inline cudaError_t launch_k(int use_pdl, cudaStream_t stream, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, Args &&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = use_pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

}  // namespace b200
