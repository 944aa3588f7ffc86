// MUL_MAT for F16 / BF16 weight matrices (unquantized models, float side matrices) on the fast paths:
//   mm16_tc_kernel   more than 4 activation columns: tcgen05 GEMM.  Both operands are 16-bit K-major tiles brought in by
//                    tiled tensor copies with the 128-byte swizzle (weights straight from the model's rows, activations
//                    from the F16 / BF16 copy the caller's workspace holds), `tcgen05.mma kind::f16` 128 x 128 x 16 from
//                    shared-memory descriptors into an FP32 tensor-memory accumulator, six stages; one thread loads, one
//                    issues, four warps read the accumulator back and store.
//   mv16_kernel      at most 4 columns: one warp per weight row, 128-bit loads, FP32 accumulation (HBM-bound).
// What the reference does with cuBLAS for these types (ggml_cuda_op_mul_mat_cublas, ggml/src/ggml-cuda/ggml-cuda.cu:1180-1290:
// 16-bit operands, FP32 result) and with mul_mat_vec (ggml/src/ggml-cuda/mmv.cu:5-91).  Strided / batched / F32-weight
// products stay on matmul_f_kernel (matmul_f.cu).  Every mbarrier wait is bounded.
#include "common.cuh"
#include "kernels.h"
#include "tcgen05.cuh"
#include <cuda_bf16.h>

namespace b200 {

static constexpr int MF_BM = 128, MF_BN = 128, MF_BK = 64, MF_STAGES = 6;
static constexpr int MF_STAGE_BYTES = (MF_BM + MF_BN) * MF_BK * 2;          // 32 KB
static constexpr int MF_THREADS = 192;

struct MfParams { float * dst; int64_t dst_nb1; int M, N, K; int * status; int bf16; };

__global__ void __launch_bounds__(MF_THREADS, 1) mm16_tc_kernel(const MfParams p, const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap xmap) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t * smem = (uint8_t *) (((uintptr_t) smem_raw + 1023) & ~(uintptr_t) 1023);
    __shared__ uint64_t full_bar[MF_STAGES], empty_bar[MF_STAGES], accum_bar;
    __shared__ uint32_t tmem_base_sh;
    __shared__ int abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    const int n0 = blockIdx.x * MF_BN, m0 = blockIdx.y * MF_BM;
    const int ksteps = p.K / MF_BK;
    if (tid == 0) {
        for (int s = 0; s < MF_STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        mbar_init(&accum_bar, 1);
        abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc(&tmem_base_sh, MF_BN);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_base_sh;

    if (warp == 0) {
        // ---- loader: weights do not depend on the kernel before this one, the activation copy does ----
        if (lane == 0) {
            bool ok = true;
            int ks = 0;
            for (; ks < ksteps; ++ks) {
                const int s = ks % MF_STAGES;
                if (ks >= MF_STAGES && !mbar_wait_or_abort(smem_u32(&empty_bar[s]), (uint32_t) (ks / MF_STAGES - 1) & 1, &abort_flag)) { ok = false; break; }
                uint8_t * st = smem + (size_t) s * MF_STAGE_BYTES;
                mbar_arrive_expect_tx(&full_bar[s], MF_STAGE_BYTES);
                tma_load_2d(st, &wmap, ks * MF_BK, m0, &full_bar[s]);
                if (ks == 0) pdl_wait();
                tma_load_2d(st + MF_BM * MF_BK * 2, &xmap, ks * MF_BK, n0, &full_bar[s]);
            }
            if (!ok) { atomicExch(p.status, ERR_MBAR_TIMEOUT); abort_flag = 1; }
            // copies still in flight when the kernel gives up are waited for (bounded) before shared memory is released
            if (!ok || *(volatile int *) &abort_flag)
                for (int kj = max(0, ks - MF_STAGES); kj < ks; ++kj) mbar_wait(&full_bar[kj % MF_STAGES], (uint32_t) (kj / MF_STAGES) & 1, 1 << 16);
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---- MMA issuer ----
        if (lane == 0) {
            // instruction descriptor: 16-bit x 16-bit -> F32, both operands K-major; format 1 = BF16
            const uint32_t fmt = p.bf16 ? 1u : 0u;
            const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t) (MF_BN >> 3) << 17) | ((uint32_t) (MF_BM >> 4) << 24);
            bool ok = true;
            for (int ks = 0; ks < ksteps; ++ks) {
                const int s = ks % MF_STAGES;
                if (!mbar_wait_or_abort(smem_u32(&full_bar[s]), (uint32_t) (ks / MF_STAGES) & 1, &abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t a = smem_u32(smem + (size_t) s * MF_STAGE_BYTES), b = a + MF_BM * MF_BK * 2;
#pragma unroll
                for (int kk = 0; kk < MF_BK / 16; ++kk) umma_f16(tmem, umma_smem_desc(a + kk * 32), umma_smem_desc(b + kk * 32), idesc, (ks | kk) != 0);
                umma_commit(&empty_bar[s]);
            }
            if (ok) umma_commit(&accum_bar);
            else { atomicExch(p.status, ERR_MBAR_TIMEOUT); abort_flag = 1; }
        }
        __syncwarp();
    } else {
        // ---- epilogue: warps 2..5 own the lane quadrants 2, 3, 0, 1 ----
        if (mbar_wait_or_abort(smem_u32(&accum_bar), 0, &abort_flag)) {
            tc_fence_after();
            const int quad = warp & 3;
            const int m = m0 + quad * 32 + lane;
#pragma unroll 1
            for (int c0 = 0; c0 < MF_BN; c0 += 32) {
                uint32_t v[32];
                tmem_ld32(tmem + ((uint32_t) (quad * 32) << 16) + (uint32_t) c0, v);
                tmem_ld_wait();
                if (m < p.M) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int n = n0 + c0 + i;
                        if (n < p.N) *(float *) ((char *) p.dst + (int64_t) n * p.dst_nb1 + (int64_t) m * 4) = __uint_as_float(v[i]);
                    }
                }
            }
        } else if (lane == 0) {
            atomicExch(p.status, ERR_MBAR_TIMEOUT);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, MF_BN); }
}

// F32 -> BF16 activations [N][K] (the F16 form is tc_convert_x_kernel in mmq_tc.cu)
__global__ void mf_convert_bf16_kernel(const float * __restrict__ x, int64_t x_nb1, __nv_bfloat16 * __restrict__ y, int64_t K, int64_t N) {
    pdl_enter();
    const int64_t total = N * K / 2;
    for (int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t) gridDim.x * blockDim.x) {
        const int64_t n = (2 * i) / K, k = (2 * i) % K;
        const float2 v = *(const float2 *) ((const char *) x + n * x_nb1 + k * 4);
        ((__nv_bfloat162 *) y)[i] = __floats2bfloat162_rn(v.x, v.y);
    }
}
__global__ void mf_convert_f16_kernel(const float * __restrict__ x, int64_t x_nb1, __half * __restrict__ y, int64_t K, int64_t N) {
    pdl_enter();
    const int64_t total = N * K / 2;
    for (int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t) gridDim.x * blockDim.x) {
        const int64_t n = (2 * i) / K, k = (2 * i) % K;
        const float2 v = *(const float2 *) ((const char *) x + n * x_nb1 + k * 4);
        ((__half2 *) y)[i] = __floats2half2_rn(v.x, v.y);
    }
}

bool mm16_tc_applicable(const TensorD & W, const TensorD & X, const TensorD & dst) {
    if ((W.type != T_F16 && W.type != T_BF16) || X.type != T_F32 || dst.type != T_F32) return false;
    if (W.ne[2] != 1 || W.ne[3] != 1 || X.ne[2] != 1 || X.ne[3] != 1) return false;
    if (X.ne[1] <= 4 || W.ne[0] % MF_BK != 0 || W.ne[0] < MF_BK) return false;
    if (W.nb[0] != 2 || (W.nb[1] & 15) || ((uintptr_t) W.data & 15)) return false;
    if (X.nb[0] != 4 || (X.nb[1] & 7) || ((uintptr_t) X.data & 7) || dst.nb[0] != 4) return false;
    return true;
}
size_t mm16_tc_workspace_bytes(int64_t N, int64_t K) { return (size_t) N * K * 2 + 256; }

cudaError_t launch_mm16_tc(const TensorD & W, const TensorD & X, const TensorD & dst, void * workspace, const LaunchCtx & c) {
    encode_tiled_fn enc = get_encode_tiled();
    if (!enc) return cudaErrorNotSupported;
    const int64_t M = W.ne[1], N = X.ne[1], K = W.ne[0];
    const bool bf16 = W.type == T_BF16;
    {
        const int64_t total = N * K / 2;
        int64_t g = (total + 255) / 256; if (g > (int64_t) c.sm_count * 8) g = (int64_t) c.sm_count * 8;
        cudaError_t e = bf16 ? launch_k(c.use_pdl, c.stream, mf_convert_bf16_kernel, dim3((unsigned) g), dim3(256), 0, (const float *) X.data, X.nb[1], (__nv_bfloat16 *) workspace, K, N)
                             : launch_k(c.use_pdl, c.stream, mf_convert_f16_kernel, dim3((unsigned) g), dim3(256), 0, (const float *) X.data, X.nb[1], (__half *) workspace, K, N);
        if (e != cudaSuccess) return e;
    }
    const CUtensorMapDataType dt = bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUtensorMap wmap, xmap;
    const cuuint32_t estr[2] = {1, 1};
    {
        const cuuint64_t gdim[2] = {(cuuint64_t) K, (cuuint64_t) M};
        const cuuint64_t gstr[1] = {(cuuint64_t) W.nb[1]};
        const cuuint32_t box[2] = {MF_BK, MF_BM};
        if (enc(&wmap, dt, 2, W.data, gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) return cudaErrorInvalidValue;
    }
    {
        const cuuint64_t gdim[2] = {(cuuint64_t) K, (cuuint64_t) N};
        const cuuint64_t gstr[1] = {(cuuint64_t) K * 2};
        const cuuint32_t box[2] = {MF_BK, MF_BN};
        if (enc(&xmap, dt, 2, workspace, gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) return cudaErrorInvalidValue;
    }
    const size_t smem = (size_t) MF_STAGES * MF_STAGE_BYTES + 1024;
    static unsigned attr_mask = 0;
    if (!(attr_mask & (1u << c.device))) {
        cudaError_t e = cudaFuncSetAttribute(mm16_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem);
        if (e != cudaSuccess) return e;
        attr_mask |= 1u << c.device;
    }
    MfParams p = {(float *) dst.data, dst.nb[1], (int) M, (int) N, (int) K, c.status, bf16 ? 1 : 0};
    dim3 grid((unsigned) ((N + MF_BN - 1) / MF_BN), (unsigned) ((M + MF_BM - 1) / MF_BM));
    return launch_k(c.use_pdl, c.stream, mm16_tc_kernel, grid, dim3(MF_THREADS), smem, p, wmap, xmap);
}

// ---- at most 4 columns (the template takes up to 8): warp per row ----
template <int N, bool BF>
__global__ void __launch_bounds__(256) mv16_kernel(const char * __restrict__ W, int64_t w_nb1, const float * __restrict__ X, int64_t x_nb1 /*bytes*/,
                                                   float * dst, int64_t dst_nb1, int M, int K) {
    pdl_enter();
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= M) return;
    const uint4 * wr = (const uint4 *) (W + (int64_t) row * w_nb1);
    float acc[N];
#pragma unroll
    for (int n = 0; n < N; ++n) acc[n] = 0.0f;
    for (int c = lane; c < K / 8; c += 32) {                          // 8 weights per 128-bit load
        const uint4 w4 = __ldg(wr + c);
        const uint32_t ww[4] = {w4.x, w4.y, w4.z, w4.w};
        float wf[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 f;
            if (BF) f = __bfloat1622float2(*(const __nv_bfloat162 *) &ww[i]); else f = __half22float2(*(const __half2 *) &ww[i]);
            wf[2 * i] = f.x; wf[2 * i + 1] = f.y;
        }
#pragma unroll
        for (int n = 0; n < N; ++n) {
            const float4 * xr = (const float4 *) ((const char *) X + (int64_t) n * x_nb1) + 2 * c;
            const float4 a = __ldg(xr), b = __ldg(xr + 1);
            acc[n] += wf[0] * a.x + wf[1] * a.y + wf[2] * a.z + wf[3] * a.w + wf[4] * b.x + wf[5] * b.y + wf[6] * b.z + wf[7] * b.w;
        }
    }
#pragma unroll
    for (int n = 0; n < N; ++n) {
        float v = acc[n];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0) *(float *) ((char *) dst + (int64_t) n * dst_nb1 + (int64_t) row * 4) = v;
    }
}

bool mv16_applicable(const TensorD & W, const TensorD & X, const TensorD & dst) {
    if ((W.type != T_F16 && W.type != T_BF16) || X.type != T_F32 || dst.type != T_F32) return false;
    if (W.ne[2] != 1 || W.ne[3] != 1 || X.ne[2] != 1 || X.ne[3] != 1 || X.ne[1] > 4 || X.ne[1] < 1) return false;     // (from 5 columns on the GEMM is faster)
    if (W.ne[0] % 8 != 0 || W.nb[0] != 2 || (W.nb[1] & 15) || ((uintptr_t) W.data & 15)) return false;
    return X.nb[0] == 4 && (X.nb[1] & 15) == 0 && ((uintptr_t) X.data & 15) == 0 && dst.nb[0] == 4;
}

template <bool BF>
static cudaError_t mv16_launch(const TensorD & W, const TensorD & X, const TensorD & dst, const LaunchCtx & c) {
    const int M = (int) W.ne[1], K = (int) W.ne[0];
    const dim3 grid((unsigned) ((M + 7) / 8)), block(256);
#define MV16(NN) case NN: return launch_k(c.use_pdl, c.stream, mv16_kernel<NN, BF>, grid, block, 0, (const char *) W.data, W.nb[1], (const float *) X.data, X.nb[1], (float *) dst.data, dst.nb[1], M, K)
    switch ((int) X.ne[1]) { MV16(1); MV16(2); MV16(3); MV16(4); MV16(5); MV16(6); MV16(7); MV16(8); }
#undef MV16
    return cudaErrorInvalidValue;
}
cudaError_t launch_mv16(const TensorD & W, const TensorD & X, const TensorD & dst, const LaunchCtx & c) {
    return W.type == T_BF16 ? mv16_launch<true>(W, X, dst, c) : mv16_launch<false>(W, X, dst, c);
}

}  // namespace b200
