// MUL_MAT for floating-point weights (F32 / F16 / BF16) with F32 or F16
// activations, any strides, broadcast over dims 2 and 3 (ggml_mul_mat,
// ggml/src/ggml.c:2694-2709).  This is the general path the non-flash attention
// graph (K.q and V.p products on cache views) and small float matrices take; it
// accumulates in FP32.  Quantized weights never come here.
#include "common.cuh"
#include "kernels.h"

namespace b200 {

__device__ __forceinline__ float ldx(const char * p, int type) {
    if (type == T_F32) return *(const float *) p;
    if (type == T_F16) return __half2float(*(const __half *) p);
    return __bfloat162float(*(const __nv_bfloat16 *) p);
}

__global__ void __launch_bounds__(256) matmul_f_kernel(const TensorD W, const TensorD X, const TensorD dst) {
    pdl_enter();
    __shared__ float Ws[32][33], Xs[32][33];
    const int tx = threadIdx.x, ty = threadIdx.y;
    const int64_t m0 = (int64_t) blockIdx.x * 32, n0 = (int64_t) blockIdx.y * 32;
    const int64_t i12 = blockIdx.z % X.ne[2], i13 = blockIdx.z / X.ne[2];
    const int64_t i02 = i12 / (X.ne[2] / W.ne[2]), i03 = i13 / (X.ne[3] / W.ne[3]);
    const int64_t M = W.ne[1], N = X.ne[1], K = W.ne[0];
    const char * wb = (const char *) W.data + i02 * W.nb[2] + i03 * W.nb[3];
    const char * xb = (const char *) X.data + i12 * X.nb[2] + i13 * X.nb[3];
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (int64_t k0 = 0; k0 < K; k0 += 32) {
        for (int r = ty; r < 32; r += 8) {
            const int64_t k = k0 + tx;
            Ws[r][tx] = (m0 + r < M && k < K) ? ldx(wb + (m0 + r) * W.nb[1] + k * W.nb[0], W.type) : 0.0f;
            Xs[r][tx] = (n0 + r < N && k < K) ? ldx(xb + (n0 + r) * X.nb[1] + k * X.nb[0], X.type) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 32; ++kk) {
            const float w = Ws[tx][kk];
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[i] += w * Xs[ty + 8 * i][kk];
        }
        __syncthreads();
    }
    char * db = (char *) dst.data + i12 * dst.nb[2] + i13 * dst.nb[3];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int64_t m = m0 + tx, n = n0 + ty + 8 * i;
        if (m < M && n < N) *(float *) (db + n * dst.nb[1] + m * dst.nb[0]) = acc[i];
    }
}

cudaError_t launch_matmul_f(const TensorD & W, const TensorD & X, const TensorD & dst, const LaunchCtx & c) {
    const int64_t M = W.ne[1], N = X.ne[1], batch = X.ne[2] * X.ne[3];
    if (M == 0 || N == 0 || batch == 0) return cudaSuccess;
    dim3 grid((unsigned) ((M + 31) / 32), (unsigned) ((N + 31) / 32), (unsigned) batch);
    (void) (launch_err = launch_k(c.use_pdl, c.stream, matmul_f_kernel, dim3(grid), dim3(dim3(32, 8)), 0, W, X, dst));
    return cudaGetLastError();
}

}  // namespace b200
