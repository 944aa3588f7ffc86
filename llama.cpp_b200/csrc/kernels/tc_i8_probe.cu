// Measurement of the design alternative for the prefill GEMM: int8 tensor-core products with the block scales applied
// outside the MMA, the way mul_mat_q does on mma.sync (ggml/src/ggml-cuda/mmq.cuh:649-727: one int8 MMA per 32-deep
// step, then `sum += d_w * d_x * acc` in FP32).  ggml's scales change every 32 values along K (every 16 for Q6_K), so an
// int32 accumulator cannot run across K: every 128 x 256 x 32 `tcgen05.mma kind::i8` has to be read back from tensor
// memory, converted and folded into FP32 sums before the next one may reuse the accumulator.
//
// This kernel does exactly that and nothing else (operands stay fixed in shared memory: no loads, no dequantization): one
// thread issues the MMAs into two alternating 256-column int32 accumulators, eight warps (thread = row x half of the
// columns, 128 FP32 sums in registers) drain them with tcgen05.ld, I2F and FMA with a per-row and a per-column scale.
// The time per 32-deep step is the floor of the int8 form; b200_tc_i8_probe reports it beside a value of the result so the
// caller can see that the products were really computed.  Not on any product path.
#include "common.cuh"
#include "kernels.h"
#include "tcgen05.cuh"

namespace b200 {

static constexpr int IP_BM = 128, IP_BN = 256;
static constexpr int IP_THREADS = 256 + 32;

// instruction descriptor: S8 x S8 -> S32, both operands K-major
__device__ __forceinline__ constexpr uint32_t umma_idesc_i8(int M, int N) {
    return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t) (N >> 3) << 17) | ((uint32_t) (M >> 4) << 24);
}
__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        :: "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

__global__ void __launch_bounds__(IP_THREADS, 1) tc_i8_probe_kernel(int kblocks, float * out, int * status) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t * smem = (uint8_t *) (((uintptr_t) smem_raw + 1023) & ~(uintptr_t) 1023);
    uint8_t * a_s = smem, * b_s = smem + IP_BM * 128;               // [rows][128 int8], 128-byte swizzle; 4 steps of K = 32
    __shared__ uint64_t acc_full[2], acc_free[2];
    __shared__ uint32_t tmem_base_sh;
    __shared__ int abort_flag;
    __shared__ float col_scale[IP_BN];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    if (tid == 0) {
        for (int s = 0; s < 2; ++s) { mbar_init(&acc_full[s], 1); mbar_init(&acc_free[s], 8); }
        abort_flag = 0;
        mbar_fence_init();
    }
    // operands: A[r][k] = (r % 7) - 3, B[n][k] = (n % 5) - 2, written through the swizzle (16-byte chunk c of row r at c ^ (r & 7))
    for (int i = tid; i < (IP_BM + IP_BN) * 8; i += IP_THREADS) {
        const int r = i >> 3, c = i & 7;
        const int val = r < IP_BM ? (r % 7) - 3 : ((r - IP_BM) % 5) - 2;
        const uint32_t w = (uint32_t) (val & 0xff) * 0x01010101u;
        *(uint4 *) (smem + r * 128 + ((c ^ (r & 7)) << 4)) = make_uint4(w, w, w, w);
    }
    for (int i = tid; i < IP_BN; i += IP_THREADS) col_scale[i] = 1.0f + 0.001f * (float) i;
    fence_async_smem();
    if (warp == 8) tmem_alloc(&tmem_base_sh, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_base_sh;

    if (warp < 8) {
        // drain: thread = (row, half of the columns); 128 FP32 sums in registers
        const int r = tid & 127, half = tid >> 7;
        const uint32_t lane_addr = tmem + ((uint32_t) ((warp & 3) * 32) << 16);
        const float row_scale = 0.5f + 0.01f * (float) r;
        float sum[128];
#pragma unroll
        for (int i = 0; i < 128; ++i) sum[i] = 0.0f;
        bool ok = true;
        for (int j = 0; j < kblocks && ok; ++j) {
            const int b = j & 1;
            if (!mbar_wait_or_abort(smem_u32(&acc_full[b]), (uint32_t) (j >> 1) & 1, &abort_flag)) { ok = false; break; }
            tc_fence_after();
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t v[32];
                tmem_ld32(lane_addr + (uint32_t) (b * 256 + half * 128 + c * 32), v);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) sum[c * 32 + i] += (float) (int) v[i] * row_scale * col_scale[half * 128 + c * 32 + i];
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_free[b]);
        }
        if (!ok && lane == 0) { atomicExch(status, ERR_MBAR_TIMEOUT); abort_flag = 1; }
        float total = 0.0f;
#pragma unroll
        for (int i = 0; i < 128; ++i) total += sum[i];
        if (blockIdx.x == 0) out[tid] = total;                       // (row r, half) of CTA 0
        if (blockIdx.x == 0 && tid == 5) out[256] = sum[3];          // one element: row 5, column 3
    } else if (lane == 0) {
        constexpr uint32_t idesc = umma_idesc_i8(IP_BM, IP_BN);
        const uint64_t ad = umma_smem_desc(smem_u32(a_s)), bd = umma_smem_desc(smem_u32(b_s));
        bool ok = true;
        for (int j = 0; j < kblocks && ok; ++j) {
            const int b = j & 1;
            if (j >= 2 && !mbar_wait_or_abort(smem_u32(&acc_free[b]), (uint32_t) ((j >> 1) - 1) & 1, &abort_flag)) { ok = false; break; }
            tc_fence_after();
            umma_i8(tmem + (uint32_t) (b * 256), ad + 2 * (j & 3), bd + 2 * (j & 3), idesc, 0);     // K = 32 int8 = 32 bytes inside the swizzle atom
            umma_commit(&acc_full[b]);
        }
        if (!ok) { atomicExch(status, ERR_MBAR_TIMEOUT); abort_flag = 1; }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 8) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

// Runs `reps` launches of `kblocks` 32-deep steps on every SM; us_per_kblock receives the time of one step of one CTA,
// check the value of element (row 5, column 3) of CTA 0 (expected: kblocks * 32 * (5 % 7 - 3) * (3 % 5 - 2) * row scale *
// column scale).
cudaError_t launch_tc_i8_probe(int kblocks, int reps, float * us_per_kblock, float * check, float * expected, const LaunchCtx & c) {
    float * out = nullptr;
    cudaError_t e = cudaMalloc(&out, 512 * sizeof(float));
    if (e != cudaSuccess) return e;
    const size_t smem = (size_t) (IP_BM + IP_BN) * 128 + 1024;
    e = cudaFuncSetAttribute(tc_i8_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem);
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    if (e == cudaSuccess) e = cudaEventCreate(&e0);
    if (e == cudaSuccess) e = cudaEventCreate(&e1);
    if (e == cudaSuccess) {
        tc_i8_probe_kernel<<<c.sm_count, IP_THREADS, smem, c.stream>>>(kblocks, out, c.status);      // warm-up
        cudaEventRecord(e0, c.stream);
        for (int i = 0; i < reps; ++i) tc_i8_probe_kernel<<<c.sm_count, IP_THREADS, smem, c.stream>>>(kblocks, out, c.status);
        cudaEventRecord(e1, c.stream);
        e = cudaStreamSynchronize(c.stream);
    }
    if (e == cudaSuccess) {
        float ms = 0.0f;
        cudaEventElapsedTime(&ms, e0, e1);
        *us_per_kblock = ms * 1e3f / (float) reps / (float) kblocks;
        e = cudaMemcpy(check, out + 256, sizeof(float), cudaMemcpyDeviceToHost);
        *expected = (float) kblocks * 32.0f * (float) ((5 % 7 - 3) * (3 % 5 - 2)) * (0.5f + 0.01f * 5.0f) * (1.0f + 0.001f * 3.0f);
    }
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    cudaFree(out);
    return e;
}

}  // namespace b200
