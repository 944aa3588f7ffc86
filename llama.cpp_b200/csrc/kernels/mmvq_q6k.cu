// Decode mat-vec for Q6_K weights (210-byte super-blocks: ql[128] qh[64] scales[16] d,
// ggml/src/ggml-common.h:314-320).  The blocks are only 2-byte aligned, but sixteen of them
// (4096 weights, 3360 bytes) are a 16-byte multiple, so a warp fetches such a run with
// fully coalesced 128-bit loads into registers, parks it in a warp-private shared-memory
// buffer and then each lane decodes one half super-block (128 weights) from there with
// 32-bit loads and funnel shifts.  Loads for the next run are issued before the current one
// is decoded, there are no block-wide barriers in the loop, and weight loads are issued
// before griddepcontrol.wait.
//
// Arithmetic: vec_dot_q6_K_q8_1 (ggml/src/ggml-cuda/vecdotq.cuh:476-496, 763-787) restated
// for this chunking; element layout as in dequantize_row_q6_K (ggml-quants.c:1690-1719).
#include "common.cuh"
#include "kernels.h"

namespace b200 {

static constexpr int Q6_WARPS = 8;
static constexpr int Q6_RUN_BLOCKS = 16;                        // super-blocks per run
static constexpr int Q6_RUN_BYTES = Q6_RUN_BLOCKS * 210;        // 3360 = 210 * 16
static constexpr int Q6_RUN_VECS = Q6_RUN_BYTES / 16;           // 210 uint4
static constexpr int Q6_VECS_PER_LANE = (Q6_RUN_VECS + 31) / 32;   // 7

struct Q6Params {
    const uint8_t * W;  int64_t w_nb1;
    const uint8_t * Xq; int64_t xq_col_bytes;
    float * dst;        int64_t dst_nb1;
    int M, K, x_col0;
    int n_peer; int64_t peer_delta[MAX_PEERS - 1];   // row-split: results also go to dst + peer_delta[i]
};

// NW consecutive 32-bit words at a 2-byte aligned shared-memory address
template <int NW>
__device__ __forceinline__ void lds_run(const uint8_t * p, uint32_t (&out)[NW]) {
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

template <int N>
__global__ void __launch_bounds__(Q6_WARPS * 32, 2) mmvq_q6k_kernel(const Q6Params p) {
    extern __shared__ __align__(16) uint8_t smem[];
    pdl_launch_dependents();          // the next kernel may start its prologue (its weight prefetch) right away
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nsb = p.K >> 8;
    const int col_bytes = ((p.K + 127) >> 7) * 160;
    uint8_t * acts  = smem;                                                  // [N][col_bytes]
    uint8_t * stage = smem + (size_t) N * col_bytes + (size_t) warp * (Q6_RUN_BYTES + 16);   // +16: funnel loads read one word past

    const int nruns = (nsb + Q6_RUN_BLOCKS - 1) / Q6_RUN_BLOCKS;
    const int row_stride = gridDim.x * Q6_WARPS;
    int row = blockIdx.x * Q6_WARPS + warp;
    bool storer = lane == 0; int64_t st_delta = 0;
#pragma unroll
    for (int q = 0; q < MAX_PEERS - 1; ++q) if (q < p.n_peer && lane == q + 1) { storer = true; st_delta = p.peer_delta[q]; }

    uint4 v[Q6_VECS_PER_LANE];
    auto load_run = [&](int r, int run) {
        const uint8_t * src = p.W + (int64_t) r * p.w_nb1 + (int64_t) run * Q6_RUN_BYTES;
        const int nvec = min(Q6_RUN_BLOCKS, nsb - run * Q6_RUN_BLOCKS) * 210 / 16;
#pragma unroll
        for (int i = 0; i < Q6_VECS_PER_LANE; ++i) {
            const int idx = i * 32 + lane;
            if (idx < nvec) v[i] = __ldg((const uint4 *) src + idx);
        }
    };
    auto store_run = [&](int run) {
        const int nvec = min(Q6_RUN_BLOCKS, nsb - run * Q6_RUN_BLOCKS) * 210 / 16;
#pragma unroll
        for (int i = 0; i < Q6_VECS_PER_LANE; ++i) {
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

    // lane -> half super-block (b, n128) of the run
    const int b = lane >> 1, n128 = lane & 1;
    const uint8_t * blk = stage + b * 210;

    while (row < p.M) {
        float acc[N];
#pragma unroll
        for (int n = 0; n < N; ++n) acc[n] = 0.0f;
        for (int run = 0; run < nruns; ++run) {
            __syncwarp();
            store_run(run);
            __syncwarp();
            // prefetch the next run (of this row, or the first of the warp's next row)
            if (run + 1 < nruns) load_run(row, run + 1);
            else if (row + row_stride < p.M) load_run(row + row_stride, 0);

            if (run * Q6_RUN_BLOCKS + b < nsb) {
                uint32_t ql[16], qh[8];
                lds_run<16>(blk + n128 * 64, ql);
                lds_run<8>(blk + 128 + n128 * 32, qh);
                uint32_t scw[2];
                lds_run<2>(blk + 192 + n128 * 8, scw);                      // 8 signed scales of this half
                const float d = h2f(*(const uint16_t *) (blk + 208));
                const uint32_t a_base = (uint32_t) ((run * Q6_RUN_BLOCKS + b) * 2 + n128) * 160;   // blk_act128 of this half
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    // weights of 32-value group t: l = 0..31 -> words i = 0..7
                    int q[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const uint32_t L = (t & 1) ? ql[8 + i] : ql[i];
                        const uint32_t nib = (t & 2) ? (L >> 4) & 0x0F0F0F0Fu : L & 0x0F0F0F0Fu;
                        const uint32_t hb = t == 0 ? (qh[i] << 4) : t == 1 ? (qh[i] << 2) : t == 2 ? qh[i] : (qh[i] >> 2);
                        q[i] = (int) __vsubss4(nib | (hb & 0x30303030u), 0x20202020u);
                    }
                    const int sc_lo = (int) (int8_t) ((scw[(2 * t) >> 2] >> (8 * ((2 * t) & 3))) & 0xff);         // scales[2t]   (l < 16)
                    const int sc_hi = (int) (int8_t) ((scw[(2 * t + 1) >> 2] >> (8 * ((2 * t + 1) & 3))) & 0xff); // scales[2t+1] (l >= 16)
#pragma unroll
                    for (int n = 0; n < N; ++n) {
                        const uint8_t * ab = acts + n * col_bytes + a_base;
                        const uint4 x0 = *(const uint4 *) (ab + t * 32);
                        const uint4 x1 = *(const uint4 *) (ab + t * 32 + 16);
                        const float dx = *(const float *) (ab + 128 + t * 8);
                        int s0 = __dp4a(q[0], (int) x0.x, 0); s0 = __dp4a(q[1], (int) x0.y, s0);
                        s0 = __dp4a(q[2], (int) x0.z, s0);    s0 = __dp4a(q[3], (int) x0.w, s0);
                        int s1 = __dp4a(q[4], (int) x1.x, 0); s1 = __dp4a(q[5], (int) x1.y, s1);
                        s1 = __dp4a(q[6], (int) x1.z, s1);    s1 = __dp4a(q[7], (int) x1.w, s1);
                        acc[n] += d * dx * (float) (sc_lo * s0 + sc_hi * s1);
                    }
                }
            }
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

template <int N>
static cudaError_t launch_q6k_n(const Q6Params & p, int sm_count, int device, int use_pdl, cudaStream_t stream) {
    const size_t smem = (size_t) N * ((p.K + 127) / 128) * 160 + (size_t) Q6_WARPS * (Q6_RUN_BYTES + 16);
    auto kern = mmvq_q6k_kernel<N>;
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
    const int64_t need = ((int64_t) p.M + Q6_WARPS - 1) / Q6_WARPS;
    if (grid > need) grid = need;
    if (grid < 1) grid = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned) grid); cfg.blockDim = dim3(Q6_WARPS * 32);
    cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = use_pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, p);
}

// needs 16-byte aligned rows made of whole 8-block (1680-byte) groups, no batching / expert indirection
bool mmvq_q6k_applicable(const MmvqArgs & a) {
    if (a.type != T_Q6_K || a.ids || a.ne12 * a.ne13 != 1) return false;
    if (((uintptr_t) a.W & 15) || (a.w_nb1 & 15) || (a.K % 2048) != 0) return false;
    if ((size_t) a.N * ((a.K + 127) / 128) * 160 + (size_t) Q6_WARPS * (Q6_RUN_BYTES + 16) > 200 * 1024) return false;
    return true;
}

cudaError_t launch_mmvq_q6k(const MmvqArgs & a, cudaStream_t stream) {
    Q6Params p = {};
    p.W = (const uint8_t *) a.W; p.w_nb1 = a.w_nb1;
    p.Xq = (const uint8_t *) a.Xq; p.xq_col_bytes = (int64_t) ((a.K + 127) / 128) * 160;
    p.dst = a.dst; p.dst_nb1 = a.dst_nb1;
    p.M = a.M; p.K = a.K; p.x_col0 = a.x_col0;
    p.n_peer = a.n_peer; for (int i = 0; i < a.n_peer; ++i) p.peer_delta[i] = a.peer_delta[i];
    switch (a.N) {
        case 1: return launch_q6k_n<1>(p, a.sm_count, a.device, a.use_pdl, stream);
        case 2: return launch_q6k_n<2>(p, a.sm_count, a.device, a.use_pdl, stream);
        case 3: return launch_q6k_n<3>(p, a.sm_count, a.device, a.use_pdl, stream);
        case 4: return launch_q6k_n<4>(p, a.sm_count, a.device, a.use_pdl, stream);
        case 5: return launch_q6k_n<5>(p, a.sm_count, a.device, a.use_pdl, stream);
        case 6: return launch_q6k_n<6>(p, a.sm_count, a.device, a.use_pdl, stream);
        case 7: return launch_q6k_n<7>(p, a.sm_count, a.device, a.use_pdl, stream);
        case 8: return launch_q6k_n<8>(p, a.sm_count, a.device, a.use_pdl, stream);
    }
    return cudaErrorInvalidValue;
}

}  // namespace b200
