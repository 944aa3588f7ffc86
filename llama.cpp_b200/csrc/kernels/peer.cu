// Row-split exchange between the GPUs of one node, one process per GPU.
//
// With the weight rows of a MUL_MAT split across ranks (the reference's split buffers,
// ggml/src/ggml-cuda/ggml-cuda.cu:714-1040, gather of dst slices :1520-1660) every rank computes the
// rows [row_low, row_high) of dst and all ranks need all of it.  Every rank maps the activation arena
// of every other rank (CUDA IPC), at the same offsets, so the exchange is plain stores into peer
// memory over NVLink:
//   peer_push_kernel     copies this rank's slab of dst into the same place of every peer's arena
//                        (the decode mat-vec kernels store to the peers themselves and skip this)
//   peer_barrier_kernel  publishes "my slabs are written" to every peer and waits until every peer has
//                        published the same epoch; kernels after it may read the whole dst
// Flags are 32-bit epochs: rank r writes its epoch into slot r of every peer's flag array; the epoch
// counter lives in device memory and is advanced by the kernel itself, so a captured CUDA graph can be
// replayed.  The wait is bounded: after PEER_SPIN_LIMIT polls the kernel records ERR_PEER_TIMEOUT in
// the status word and returns, leaving the context usable.
// No loads from peer memory, no multicast: stores only.
#include "common.cuh"
#include "kernels.h"

namespace b200 {

static constexpr int PEER_SPIN_LIMIT = 4000000;      // x ~1 us per poll: a few seconds

__global__ void __launch_bounds__(256) peer_push_kernel(const PeerPush p) {
    pdl_enter();
    char * dst = p.peer_dst[blockIdx.y];
    const int64_t per_col = p.col_bytes >> p.shift;                  // elements of 4 or 16 bytes per column
    const int64_t total = per_col * p.ncols;
    for (int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t) gridDim.x * blockDim.x) {
        const int64_t c = i / per_col, r = i - c * per_col;
        const int64_t off = c * p.col_stride + (r << p.shift);
        if (p.shift == 4) *(uint4 *) (dst + off) = *(const uint4 *) (p.src + off);
        else              *(uint32_t *) (dst + off) = *(const uint32_t *) (p.src + off);
    }
}

__global__ void __launch_bounds__(32) peer_barrier_kernel(const PeerBarrier b) {
    pdl_enter();                                   // everything launched before (the slab stores) has completed
    const int t = threadIdx.x;
    unsigned ep = 0;
    if (t == 0) { ep = *b.epoch + 1; *b.epoch = ep; }
    ep = __shfl_sync(0xffffffffu, ep, 0);
    __threadfence_system();
    if (t < b.n_ranks && t != b.rank) {
        asm volatile("st.release.sys.global.u32 [%0], %1;" :: "l"(b.peer_flags[t] + b.rank), "r"(ep) : "memory");
        const unsigned * mine = b.local_flags + t;
        unsigned seen = 0;
        int spins = 0;
        for (;;) {
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
            if ((int) (seen - ep) >= 0) break;
            if (++spins > (b.spin_limit > 0 ? b.spin_limit : PEER_SPIN_LIMIT)) { atomicMax(b.status, (int) ERR_PEER_TIMEOUT); break; }
            __nanosleep(200);
        }
    }
    __syncwarp();
    __threadfence_system();
}

cudaError_t launch_peer_push(const PeerPush & p, const LaunchCtx & c) {
    if (p.n_peer <= 0 || p.col_bytes <= 0 || p.ncols <= 0) return cudaSuccess;
    const int64_t total = (p.col_bytes >> p.shift) * p.ncols;
    int64_t blocks = (total + 255) / 256;
    const int64_t cap = (int64_t) c.sm_count * 4 / p.n_peer + 1;
    if (blocks > cap) blocks = cap;
    (void) (launch_err = launch_k(c.use_pdl, c.stream, peer_push_kernel, dim3((unsigned) blocks, (unsigned) p.n_peer), dim3(256), 0, p));
    return launch_err;
}

cudaError_t launch_peer_barrier(const PeerBarrier & b, const LaunchCtx & c) {
    (void) (launch_err = launch_k(c.use_pdl, c.stream, peer_barrier_kernel, dim3(1), dim3(32), 0, b));
    return launch_err;
}

}  // namespace b200
