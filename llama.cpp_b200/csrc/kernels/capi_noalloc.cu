// b200_mul_mat_q_noalloc: the quantized MUL_MAT of b200_mul_mat_q for callers that must not
// allocate device memory.  Its int8 activation scratch (and the kernels' status word) live in
// file-scope __device__ arrays, so the call performs no cudaMalloc / cudaFree and uses no
// allocating library routine.  See include/b200_kernels.h for the contract.
#include "common.cuh"
#include "kernels.h"
#include "b200_kernels.h"

#include <climits>
#include <mutex>
#include <string>

using namespace b200;

// Scratch for the activation blocks: 160 bytes per 128 activation values.  Every GPU that loads
// this library holds the array until the process exits.
static __device__ __align__(256) unsigned char g_noalloc_scratch[B200_NOALLOC_SCRATCH_BYTES];
static __device__ __align__(256) int g_noalloc_status[64];

namespace {
constexpr int NA_MAX_DEVICES = 64;
struct NoAllocDev { std::mutex mu; void * scratch = nullptr; int * status = nullptr; int sm_count = 0; bool ready = false; };
NoAllocDev g_na[NA_MAX_DEVICES];
thread_local std::string g_na_err;
int na_fail(int code, const std::string & msg) { g_na_err = msg; return code; }

// One-time set-up for the current device (ordinal `dev`), under the slot's lock so that two host threads
// making their first call at the same time do it once.  In host code the array's name is only a handle; the
// kernels need the device address the runtime maps it to, looked up with that device current.
int na_device(int dev, NoAllocDev ** out) {
    if (dev < 0 || dev >= NA_MAX_DEVICES) return na_fail(B200_E_NO_DEVICE, "device ordinal beyond what this entry point tracks (64)");
    NoAllocDev & d = g_na[dev];
    std::lock_guard<std::mutex> lock(d.mu);
    if (!d.ready) {
        cudaError_t e;
        int major = 0, sm = 0;
        if ((e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev)) != cudaSuccess)
            return na_fail((int) e, std::string("cudaDeviceGetAttribute: ") + cudaGetErrorString(e));
        if (major != 10) return na_fail(B200_E_NO_DEVICE, "current device is not sm_100");
        if ((e = cudaDeviceGetAttribute(&sm, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess)
            return na_fail((int) e, std::string("cudaDeviceGetAttribute: ") + cudaGetErrorString(e));
        void * sc = nullptr, * st = nullptr;
        if ((e = cudaGetSymbolAddress(&sc, g_noalloc_scratch)) != cudaSuccess)
            return na_fail((int) e, std::string("cudaGetSymbolAddress(scratch): ") + cudaGetErrorString(e));
        if ((e = cudaGetSymbolAddress(&st, g_noalloc_status)) != cudaSuccess)
            return na_fail((int) e, std::string("cudaGetSymbolAddress(status): ") + cudaGetErrorString(e));
        if ((e = cudaMemset(st, 0, sizeof(int))) != cudaSuccess)
            return na_fail((int) e, std::string("cudaMemset(status): ") + cudaGetErrorString(e));
        d.scratch = sc; d.status = (int *) st; d.sm_count = sm;
        d.ready = true;
    }
    *out = &d;
    return 0;
}
}  // namespace

extern "C" __attribute__((visibility("default"))) const char * b200_noalloc_last_error(void) { return g_na_err.c_str(); }

extern "C" __attribute__((visibility("default")))
int b200_mul_mat_q_noalloc(int type, const void * W, int64_t w_nb1, int64_t M, int64_t K, const float * X, int64_t x_stride,
                           int64_t N, float * dst, int64_t dst_stride, void * stream) {
    if (!mmvq_type_supported(type)) return na_fail(B200_E_UNSUPPORTED, "weight type not supported");
    if (K <= 0 || M <= 0 || N <= 0 || K % type_block_elems(type) != 0) return na_fail(B200_E_BAD_ARG, "bad shape");
    if (N > 8) return na_fail(B200_E_UNSUPPORTED, "b200_mul_mat_q_noalloc handles at most 8 activation columns");
    // nothing is launched on arguments the kernels would fault on
    if (M > INT_MAX || K > INT_MAX || x_stride < K || dst_stride < M || w_nb1 < (int64_t) (K / type_block_elems(type)) * type_block_bytes(type))
        return na_fail(B200_E_BAD_ARG, "strides smaller than a row / column, or a dimension beyond 2^31-1");
    if (!W || !X || !dst || ((uintptr_t) W & 1) || (w_nb1 & 1) || ((uintptr_t) X & 3) || ((uintptr_t) dst & 3))
        return na_fail(B200_E_BAD_ARG, "null or misaligned pointer (weights 2-byte, activations and results 4-byte aligned)");
    const size_t need = act128_bytes(K, N);
    if (need > (size_t) B200_NOALLOC_SCRATCH_BYTES)
        return na_fail(B200_E_SCRATCH, "K*N too large for the built-in scratch: " + std::to_string(need) + " bytes needed, " +
                                           std::to_string((size_t) B200_NOALLOC_SCRATCH_BYTES) + " available");
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) { cudaGetLastError(); return na_fail(B200_E_NO_DEVICE, "no CUDA device"); }
    NoAllocDev * dp = nullptr;
    if (int rc = na_device(dev, &dp)) return rc;
    NoAllocDev & d = *dp;
    cudaStream_t s = (cudaStream_t) stream;
    // the activation blocks of all N columns are rewritten in full by this launch: nothing of the
    // previous call's contents is read
    if ((e = launch_quantize_act128(X, N, 1, 1, x_stride, 0, 0, d.scratch, (int) K, s)) != cudaSuccess)
        return na_fail((int) e, std::string("activation quantizer: ") + cudaGetErrorString(e));
    MmvqArgs a = {};
    a.type = type; a.W = W; a.w_nb1 = w_nb1; a.Xq = d.scratch; a.M = (int) M; a.K = (int) K; a.N = (int) N;
    a.ne12 = 1; a.ne13 = 1; a.r2 = 1; a.r3 = 1; a.x_ncols = (int) N; a.xq_ne12 = 1; a.x_col0 = 0;
    a.dst = dst; a.dst_nb1 = dst_stride * 4;
    a.status = d.status; a.sm_count = d.sm_count; a.device = dev; a.use_pdl = 0;
    if ((e = launch_mmvq(a, s)) != cudaSuccess) return na_fail((int) e, std::string("mat-vec kernel: ") + cudaGetErrorString(e));
    return 0;
}

// Reads back (and clears) the status word the kernels of b200_mul_mat_q_noalloc write when they give up a
// bounded wait.  Synchronises `stream`; copies four bytes to the host; allocates nothing.
extern "C" __attribute__((visibility("default")))
int b200_noalloc_status(void * stream) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); return na_fail(B200_E_NO_DEVICE, "no CUDA device"); }
    NoAllocDev * dp = nullptr;
    if (int rc = na_device(dev, &dp)) return rc;
    cudaStream_t s = (cudaStream_t) stream;
    int st = 0;
    cudaError_t e = cudaMemcpyAsync(&st, dp->status, sizeof(int), cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) { cudaGetLastError(); return na_fail((int) e, std::string("reading the status word: ") + cudaGetErrorString(e)); }
    if (st == 0) return 0;
    cudaMemsetAsync(dp->status, 0, sizeof(int), s);
    return na_fail(B200_E_DEVICE_WAIT, "a kernel of an earlier b200_mul_mat_q_noalloc call gave up a bounded wait (status " + std::to_string(st) + "): its results are not valid");
}
