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
// CTA = 5 warps, one 128 (weight rows) x 128 (tokens) output tile:
//   warps 0-3  producers: thread r dequantizes 64 consecutive weights of weight row r and copies 64
//              F16 activations of token r per k-step, writing both operand tiles in the canonical
//              K-major SWIZZLE_128B layout (row r at r*128 B, 16-byte chunk c at position c ^ (r & 7));
//              then fence.proxy.async + mbarrier arrive.  After the K loop they become the epilogue:
//              tcgen05.ld of the accumulator (lane = weight row, column = token) and coalesced stores.
//   warp 4     one elected thread issues 4 x tcgen05.mma (M128 N128 K16) per k-step from shared-memory
//              matrix descriptors, tcgen05.commit frees the stage / publishes the accumulator.
// 4-stage ring of 32 KB stages; every mbarrier wait is bounded and failure is reported through the
// status word; TMEM (128 columns) is allocated and released by warp 4 on every path.
#include "common.cuh"
#include "kernels.h"

namespace b200 {

static constexpr int TC_BM = 128, TC_BN = 128, TC_BK = 64;
static constexpr int TC_STAGES = 4;
static constexpr int TC_STAGE_BYTES = (TC_BM + TC_BN) * TC_BK * 2;      // 32 KB
static constexpr int TC_THREADS = 160;
static constexpr int TC_TMEM_COLS = 128;

// ---- tcgen05 wrappers -------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t * smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(smem_dst)), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after()  { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        :: "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t * bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// shared-memory matrix descriptor: K-major operand, 128-byte swizzle, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t) ((smem_addr & 0x3FFFF) >> 4);          // start address
    d |= (uint64_t) 1 << 16;                               // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t) (1024 >> 4) << 32;                     // stride byte offset between 8-row groups
    d |= (uint64_t) 1 << 46;                               // descriptor version of this architecture
    d |= (uint64_t) 2 << 61;                               // SWIZZLE_128B
    return d;
}
// instruction descriptor: F16 x F16 -> F32, both operands K-major, M = 128, N = 128
__device__ __forceinline__ constexpr uint32_t umma_idesc_f16(int M, int N) {
    return (1u << 4) | (0u << 7) | (0u << 10) | ((uint32_t) (N >> 3) << 17) | ((uint32_t) (M >> 4) << 24);
}

// ---- weight dequantization: 64 consecutive values of one row as F16 ---------------------------
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *(uint32_t *) &h;
}

template <int T> struct Deq64;     // get(row, k0, out[32]): out = 64 F16 values k0 .. k0+63 (k0 % 64 == 0)

template <> struct Deq64<T_Q4_K> {
    static __device__ __forceinline__ void get(const uint8_t * row, int k0, uint32_t (&out)[32]) {
        const uint8_t * b = row + (k0 >> 8) * 144;
        const int j = (k0 >> 6) & 3;
        const uint4 hd = __ldg((const uint4 *) b);
        const float2 dm = __half22float2(*(const __half2 *) &hd.x);
        const uint8_t * sc = (const uint8_t *) &hd.y;
        int s0, m0, s1, m1;
        k4_scale_min(2 * j, sc, s0, m0);
        k4_scale_min(2 * j + 1, sc, s1, m1);
        const float d0 = dm.x * s0, n0 = dm.y * m0, d1 = dm.x * s1, n1 = dm.y * m1;
        const uint4 qa = __ldg((const uint4 *) (b + 16 + 32 * j)), qb = __ldg((const uint4 *) (b + 32 + 32 * j));
        const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {       // word i: bytes 4i..4i+3 -> low nibbles k0+4i.., high nibbles k0+32+4i..
            const uint32_t v = w[i];
            out[2 * i]          = pack_h2(d0 * (float) (v & 0xF) - n0,         d0 * (float) ((v >> 8) & 0xF) - n0);
            out[2 * i + 1]      = pack_h2(d0 * (float) ((v >> 16) & 0xF) - n0, d0 * (float) ((v >> 24) & 0xF) - n0);
            out[16 + 2 * i]     = pack_h2(d1 * (float) ((v >> 4) & 0xF) - n1,  d1 * (float) ((v >> 12) & 0xF) - n1);
            out[16 + 2 * i + 1] = pack_h2(d1 * (float) ((v >> 20) & 0xF) - n1, d1 * (float) ((v >> 28) & 0xF) - n1);
        }
    }
};

// generic path: element-wise through the bit-exact dequantizer
template <int T> struct Deq64 {
    static __device__ __forceinline__ void get(const uint8_t * row, int k0, uint32_t (&out)[32]) {
#pragma unroll 4
        for (int i = 0; i < 32; ++i) out[i] = pack_h2(dequant_elem<T>(row, k0 + 2 * i), dequant_elem<T>(row, k0 + 2 * i + 1));
    }
};

template <> struct Deq64<T_Q6_K> {
    static __device__ __forceinline__ void get(const uint8_t * row, int k0, uint32_t (&out)[32]) {
        // 64 values = groups t0, t0+1 (32 each) of half n128; blocks are only 2-byte aligned
        const uint8_t * b = row + (k0 >> 8) * 210;
        const int n128 = (k0 >> 7) & 1, t0 = (k0 >> 5) & 3;            // t0 is 0 or 2
        const float d = h2f(*(const uint16_t *) (b + 208));
        const uint16_t * ql = (const uint16_t *) (b + n128 * 64);
        const uint16_t * qh = (const uint16_t *) (b + 128 + n128 * 32);
        const int8_t * sc = (const int8_t *) (b + 192 + n128 * 8);
#pragma unroll
        for (int tt = 0; tt < 2; ++tt) {
            const int t = t0 + tt;                                      // group: elements l + 32 t
            const float dlo = d * (float) sc[2 * t], dhi = d * (float) sc[2 * t + 1];
#pragma unroll
            for (int l2 = 0; l2 < 16; ++l2) {                           // two l values per 16-bit load
                const uint32_t L = ql[(t & 1) * 16 + l2], H = qh[l2];
                const uint32_t nib0 = (t & 2) ? (L >> 4) & 0xF : L & 0xF, nib1 = (t & 2) ? (L >> 12) & 0xF : (L >> 8) & 0xF;
                const uint32_t h0 = (H >> (2 * t)) & 3, h1 = (H >> (8 + 2 * t)) & 3;
                const float sd = l2 < 8 ? dlo : dhi;
                out[tt * 16 + l2] = pack_h2(sd * (float) ((int) (nib0 | (h0 << 4)) - 32), sd * (float) ((int) (nib1 | (h1 << 4)) - 32));
            }
        }
    }
};

// ---- F32 -> F16 activations (pre-pass) --------------------------------------------------------
__global__ void tc_convert_x_kernel(const float * __restrict__ x, int64_t x_nb1 /*bytes*/, __half * __restrict__ y, int64_t K, int64_t N) {
    const int64_t total = N * K / 2;
    for (int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t) gridDim.x * blockDim.x) {
        const int64_t n = (2 * i) / K, k = (2 * i) % K;
        const float2 v = *(const float2 *) ((const char *) x + n * x_nb1 + k * 4);
        ((__half2 *) y)[i] = __floats2half2_rn(v.x, v.y);
    }
}

// ---- the GEMM kernel ---------------------------------------------------------------------------
struct TcParams {
    const uint8_t * W; int64_t w_nb1;
    const __half * Xh;                 // [N][K] F16
    float * dst; int64_t dst_nb1;      // bytes between token columns
    int M, N, K;
    int * status;
};

template <int T>
__global__ void __launch_bounds__(TC_THREADS, 1) mmq_tc_kernel(const TcParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // operand stages must be 1024-byte aligned for the 128-byte swizzle pattern
    uint8_t * smem = (uint8_t *) (((uintptr_t) smem_raw + 1023) & ~(uintptr_t) 1023);
    __shared__ uint64_t full_bar[TC_STAGES], empty_bar[TC_STAGES], accum_bar;
    __shared__ uint32_t tmem_base_sh;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    const int m0 = blockIdx.x * TC_BM, n0 = blockIdx.y * TC_BN;
    const int ksteps = p.K / TC_BK;

    if (tid == 0) {
        for (int s = 0; s < TC_STAGES; ++s) { mbar_init(&full_bar[s], 128); mbar_init(&empty_bar[s], 1); }
        mbar_init(&accum_bar, 1);
        abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 4) tmem_alloc(&tmem_base_sh, TC_TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_sh;

    if (warp < 4) {
        // ------------------------------ producers ------------------------------
        const int r = tid;                                              // operand row handled by this thread
        const bool wrow_ok = m0 + r < p.M, xrow_ok = n0 + r < p.N;
        const uint8_t * wrow = p.W + (int64_t) (wrow_ok ? m0 + r : 0) * p.w_nb1;
        const __half * xrow = p.Xh + (int64_t) (xrow_ok ? n0 + r : 0) * p.K;
        pdl_wait();
        bool ok = true;
        for (int ks = 0; ks < ksteps; ++ks) {
            const int s = ks % TC_STAGES;
            const uint32_t round = (uint32_t) (ks / TC_STAGES);
            if (ks >= TC_STAGES && !mbar_wait(&empty_bar[s], (round - 1) & 1)) { ok = false; break; }
            if (*(volatile int *) &abort_flag) { ok = false; break; }
            uint8_t * sa = smem + (size_t) s * TC_STAGE_BYTES;          // A: weights 128 x 64 F16
            uint8_t * sb = sa + TC_BM * TC_BK * 2;                      // B: activations 128 x 64 F16
            uint32_t wv[32];
            if (wrow_ok) Deq64<T>::get(wrow, ks * TC_BK, wv);
            else {
#pragma unroll
                for (int i = 0; i < 32; ++i) wv[i] = 0;
            }
#pragma unroll
            for (int c = 0; c < 8; ++c)
                *(uint4 *) (sa + r * 128 + ((c ^ (r & 7)) << 4)) = make_uint4(wv[4 * c], wv[4 * c + 1], wv[4 * c + 2], wv[4 * c + 3]);
            const uint4 * xs = (const uint4 *) (xrow + ks * TC_BK);
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const uint4 v = xrow_ok ? __ldg(xs + c) : make_uint4(0, 0, 0, 0);
                *(uint4 *) (sb + r * 128 + ((c ^ (r & 7)) << 4)) = v;
            }
            fence_async_smem();                                         // make the generic-proxy stores visible to the tensor core
            mbar_arrive(&full_bar[s]);
        }
        if (!ok && lane == 0) { atomicExch(p.status, ERR_MBAR_TIMEOUT); abort_flag = 1; }

        // ------------------------------ epilogue ------------------------------
        if (ok && mbar_wait(&accum_bar, 0)) {
            tc_fence_after();
            const int m = m0 + warp * 32 + lane;
#pragma unroll 1
            for (int c0 = 0; c0 < TC_BN; c0 += 32) {
                uint32_t v[32];
                tmem_ld32(tmem_base + ((uint32_t) (warp * 32) << 16) + (uint32_t) c0, v);
                tmem_ld_wait();
                if (m < p.M) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int n = n0 + c0 + i;
                        if (n < p.N) *(float *) ((char *) p.dst + (int64_t) n * p.dst_nb1 + (int64_t) m * 4) = __uint_as_float(v[i]);
                    }
                }
            }
        } else if (ok && lane == 0) {
            atomicExch(p.status, ERR_MBAR_TIMEOUT);
        }
    } else {
        // ------------------------------ MMA issuer ------------------------------
        constexpr uint32_t idesc = umma_idesc_f16(TC_BM, TC_BN);
        bool ok = true;
        for (int ks = 0; ks < ksteps && ok; ++ks) {
            const int s = ks % TC_STAGES;
            const uint32_t round = (uint32_t) (ks / TC_STAGES);
            if (!mbar_wait(&full_bar[s], round & 1)) { ok = false; break; }
            if (*(volatile int *) &abort_flag) { ok = false; break; }
            tc_fence_after();
            if (lane == 0) {
                const uint32_t a_addr = smem_u32(smem + (size_t) s * TC_STAGE_BYTES);
                const uint32_t b_addr = a_addr + TC_BM * TC_BK * 2;
#pragma unroll
                for (int kk = 0; kk < TC_BK / 16; ++kk) {
                    // advancing 16 K-elements = 32 bytes inside the 128-byte swizzle atom
                    umma_f16(tmem_base, umma_smem_desc(a_addr + kk * 32), umma_smem_desc(b_addr + kk * 32), idesc, (ks | kk) != 0);
                }
                umma_commit(&empty_bar[s]);                             // frees the stage once these MMAs have read it
                if (ks == ksteps - 1) umma_commit(&accum_bar);          // accumulator complete
            }
            __syncwarp();
        }
        if (!ok && lane == 0) { atomicExch(p.status, ERR_MBAR_TIMEOUT); abort_flag = 1; }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 4) { tc_fence_after(); tmem_dealloc(tmem_base, TC_TMEM_COLS); }
    pdl_launch_dependents();
}

bool mmq_tc_supported(int type, int64_t M, int64_t N, int64_t K) {
    (void) M;
    if (!mmvq_type_supported(type)) return false;
    return N > 8 && K % TC_BK == 0 && K >= TC_BK;
}
size_t mmq_tc_workspace_bytes(int64_t N, int64_t K) { return (size_t) N * K * 2 + 256; }
// the fast dequantizers read headers / nibble runs with aligned vector loads
bool mmq_tc_ptr_ok(int type, const void * W, int64_t w_nb1, const void * X, int64_t x_nb1) {
    if (((uintptr_t) X & 7) || (x_nb1 & 7)) return false;
    if (type == T_Q4_K || type == T_Q5_K) return ((uintptr_t) W & 15) == 0 && (w_nb1 & 15) == 0;
    return ((uintptr_t) W & 1) == 0 && (w_nb1 & 1) == 0;
}

template <int T>
static cudaError_t launch_tc_t(const TcParams & p, int device, cudaStream_t stream) {
    auto kern = mmq_tc_kernel<T>;
    const size_t smem = (size_t) TC_STAGES * TC_STAGE_BYTES + 1024;
    static unsigned attr_mask = 0;
    if (!(attr_mask & (1u << device))) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem);
        if (e != cudaSuccess) return e;
        attr_mask |= 1u << device;
    }
    dim3 grid((unsigned) ((p.M + TC_BM - 1) / TC_BM), (unsigned) ((p.N + TC_BN - 1) / TC_BN));
    kern<<<grid, TC_THREADS, smem, stream>>>(p);
    return cudaGetLastError();
}

cudaError_t launch_mmq_tc(int type, const void * W, int64_t w_nb1, const float * X, int64_t x_nb1, float * dst, int64_t dst_nb1,
                          int64_t M, int64_t N, int64_t K, void * workspace, const LaunchCtx & c) {
    __half * xh = (__half *) workspace;
    {
        const int64_t total = N * K / 2;
        int64_t g = (total + 255) / 256; if (g > (int64_t) c.sm_count * 8) g = (int64_t) c.sm_count * 8;
        tc_convert_x_kernel<<<(unsigned) g, 256, 0, c.stream>>>(X, x_nb1, xh, K, N);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return e;
    }
    TcParams p;
    p.W = (const uint8_t *) W; p.w_nb1 = w_nb1; p.Xh = xh; p.dst = dst; p.dst_nb1 = dst_nb1;
    p.M = (int) M; p.N = (int) N; p.K = (int) K; p.status = c.status;
    switch (type) {
        case T_Q4_0: return launch_tc_t<T_Q4_0>(p, c.device, c.stream);
        case T_Q4_1: return launch_tc_t<T_Q4_1>(p, c.device, c.stream);
        case T_Q5_0: return launch_tc_t<T_Q5_0>(p, c.device, c.stream);
        case T_Q5_1: return launch_tc_t<T_Q5_1>(p, c.device, c.stream);
        case T_Q8_0: return launch_tc_t<T_Q8_0>(p, c.device, c.stream);
        case T_Q4_K: return launch_tc_t<T_Q4_K>(p, c.device, c.stream);
        case T_Q5_K: return launch_tc_t<T_Q5_K>(p, c.device, c.stream);
        case T_Q6_K: return launch_tc_t<T_Q6_K>(p, c.device, c.stream);
    }
    return cudaErrorInvalidValue;
}

}  // namespace b200
