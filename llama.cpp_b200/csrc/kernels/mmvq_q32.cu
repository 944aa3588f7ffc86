// Decode mat-vec for the 32-weight block formats Q4_0 (18-byte blocks: fp16 d + 16 nibble bytes,
// ggml/src/ggml-common.h:161-166), Q8_0 (34-byte blocks: fp16 d + 32 int8, :203-208) and IQ4_NL (the Q4_0 layout with
// the nibbles mapped through the format's 16-entry code book, :398-403).
//
// The blocks are only 2-byte aligned, but 128 of them (4096 weights; 2304 or 4352 bytes) are a 16-byte multiple,
// so a warp fetches such a run of its weight row with fully coalesced 128-bit loads into registers, parks it in a
// warp-private shared-memory buffer, and each lane decodes four consecutive blocks from there: four blocks start
// at a multiple of 8 bytes (72 l or 136 l), so the lane reads plain 32-bit words and every shift that realigns a
// block inside them is a compile-time constant.  Four blocks are exactly one 128-value activation block
// (blk_act128).  Loads of the next run are issued before the current one is decoded, there are no block-wide
// barriers in the loop, and weight loads are issued before griddepcontrol.wait.
//
// Arithmetic: vec_dot_q4_0_q8_1 / vec_dot_q8_0_q8_1 (ggml/src/ggml-cuda/vecdotq.cuh:78-96, 190-205):
//   Q4_0: d_w (d_x sum(nib q) - 8 d_x sum(q)),   Q8_0: d_w d_x sum(q_w q)
// with d_x and d_x sum(q) taken from the activation block.  Element order of Q4_0: byte j holds weight j in its
// low and weight j + 16 in its high nibble (dequantize_row_q4_0, ggml/src/ggml-quants.c:255-273).
#include "common.cuh"
#include "kernels.h"
#include <type_traits>

namespace b200 {

static constexpr int Q32_WARPS = 8;
static constexpr int Q32_RUN_BLOCKS = 128;                         // blocks per run = 4 per lane

struct Q32Params {
    const uint8_t * W;  int64_t w_nb1;
    const uint8_t * Xq; int64_t xq_col_bytes;
    float * dst;        int64_t dst_nb1;
    int M, K, x_col0;
    int n_peer; int64_t peer_delta[MAX_PEERS - 1];                 // row-split: results also go to dst + peer_delta[i]
};

// word i of the byte string that starts OFF bytes into the 4-byte aligned word array w (OFF known at compile time)
template <int OFF>
__device__ __forceinline__ uint32_t word_at(const uint32_t * w, int i) {
    constexpr int base = OFF / 4, sh = (OFF % 4) * 8;
    if (sh == 0) return w[base + i];
    return __funnelshift_r(w[base + i], w[base + i + 1], sh);
}
__device__ __forceinline__ int dp4a_us32(uint32_t a, int b, int c) {   // unsigned bytes x signed bytes
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

template <int T, int N>
__global__ void __launch_bounds__(Q32_WARPS * 32, 2) mmvq_q32_kernel(const Q32Params p) {
    constexpr int BS = (T == T_Q8_0) ? 34 : 18;                    // block bytes (Q4_0 and IQ4_NL: 18)
    constexpr int RUN_BYTES = Q32_RUN_BLOCKS * BS;                 // 2304 / 4352
    constexpr int VPL = (RUN_BYTES / 16 + 31) / 32;                // uint4 per lane: 5 / 9
    constexpr int LW = 4 * BS / 4;                                 // 32-bit words of a lane's four blocks: 18 / 34
    extern __shared__ __align__(16) uint8_t smem[];
    pdl_launch_dependents();          // the next kernel may start its prologue (its weight prefetch) right away
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nblk = p.K >> 5;                                     // blocks per row (a multiple of 8)
    const int col_bytes = ((p.K + 127) >> 7) * 160;
    uint8_t * acts  = smem;                                        // [N][col_bytes]
    uint8_t * stage = smem + (size_t) N * col_bytes + (size_t) warp * (RUN_BYTES + 16);

    const int nruns = (nblk + Q32_RUN_BLOCKS - 1) / Q32_RUN_BLOCKS;
    const int row_stride = gridDim.x * Q32_WARPS;
    int row = blockIdx.x * Q32_WARPS + warp;
    bool storer = lane == 0; int64_t st_delta = 0;
#pragma unroll
    for (int q = 0; q < MAX_PEERS - 1; ++q) if (q < p.n_peer && lane == q + 1) { storer = true; st_delta = p.peer_delta[q]; }

    uint4 v[VPL];
    auto load_run = [&](int r, int run) {
        const uint8_t * src = p.W + (int64_t) r * p.w_nb1 + (int64_t) run * RUN_BYTES;
        const int nvec = min(Q32_RUN_BLOCKS, nblk - run * Q32_RUN_BLOCKS) * BS / 16;
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            const int idx = i * 32 + lane;
            if (idx < nvec) v[i] = __ldg((const uint4 *) src + idx);
        }
    };
    auto store_run = [&](int run) {
        const int nvec = min(Q32_RUN_BLOCKS, nblk - run * Q32_RUN_BLOCKS) * BS / 16;
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

    const uint32_t * mine = (const uint32_t *) (stage + lane * 4 * BS);       // 72 l or 136 l bytes: 8-byte aligned

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

            if (run * Q32_RUN_BLOCKS + 4 * lane < nblk) {         // K is a multiple of 128: all four blocks exist
                uint32_t w[LW];
#pragma unroll
                for (int i = 0; i < LW; ++i) w[i] = mine[i];
                const uint32_t a_base = (uint32_t) (run * (Q32_RUN_BLOCKS / 4) + lane) * 160;   // blk_act128 of these four blocks
                auto block = [&](auto BC) {
                    constexpr int b = decltype(BC)::value;
                    constexpr int OFF = b * BS;                    // byte offset of block b in the lane's words
                    const uint32_t dw = word_at<OFF>(w, 0);        // fp16 d in the low half
                    const float d = __half2float(__ushort_as_half((unsigned short) (dw & 0xffffu)));
                    uint32_t q[(BS - 2) / 4];
#pragma unroll
                    for (int i = 0; i < (BS - 2) / 4; ++i) q[i] = word_at<OFF + 2>(w, i);
                    uint32_t nl[8];                                // IQ4_NL: the nibbles mapped through the code book, once per block
                    if (T == T_IQ4_NL) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) { nl[i] = iq4nl_lut4(q[i] & 0x0F0F0F0Fu); nl[4 + i] = iq4nl_lut4((q[i] >> 4) & 0x0F0F0F0Fu); }
                    }
#pragma unroll
                    for (int n = 0; n < N; ++n) {
                        const uint8_t * ab = acts + n * col_bytes + a_base;
                        const uint4 x0 = *(const uint4 *) (ab + b * 32);
                        const uint4 x1 = *(const uint4 *) (ab + b * 32 + 16);
                        const float2 ds = *(const float2 *) (ab + 128 + b * 8);      // {d_x, d_x sum(q)}
                        if (T == T_Q4_0) {
                            int s = 0;
                            s = dp4a_us32(q[0] & 0x0F0F0F0Fu, (int) x0.x, s); s = dp4a_us32(q[1] & 0x0F0F0F0Fu, (int) x0.y, s);
                            s = dp4a_us32(q[2] & 0x0F0F0F0Fu, (int) x0.z, s); s = dp4a_us32(q[3] & 0x0F0F0F0Fu, (int) x0.w, s);
                            s = dp4a_us32((q[0] >> 4) & 0x0F0F0F0Fu, (int) x1.x, s); s = dp4a_us32((q[1] >> 4) & 0x0F0F0F0Fu, (int) x1.y, s);
                            s = dp4a_us32((q[2] >> 4) & 0x0F0F0F0Fu, (int) x1.z, s); s = dp4a_us32((q[3] >> 4) & 0x0F0F0F0Fu, (int) x1.w, s);
                            acc[n] += d * (ds.x * (float) s - 8.0f * ds.y);
                        } else if (T == T_IQ4_NL) {
                            int s = 0;
                            s = __dp4a((int) nl[0], (int) x0.x, s); s = __dp4a((int) nl[1], (int) x0.y, s);
                            s = __dp4a((int) nl[2], (int) x0.z, s); s = __dp4a((int) nl[3], (int) x0.w, s);
                            s = __dp4a((int) nl[4], (int) x1.x, s); s = __dp4a((int) nl[5], (int) x1.y, s);
                            s = __dp4a((int) nl[6], (int) x1.z, s); s = __dp4a((int) nl[7], (int) x1.w, s);
                            acc[n] += d * ds.x * (float) s;
                        } else {
                            int s = 0;
                            s = __dp4a((int) q[0], (int) x0.x, s); s = __dp4a((int) q[1], (int) x0.y, s);
                            s = __dp4a((int) q[2], (int) x0.z, s); s = __dp4a((int) q[3], (int) x0.w, s);
                            s = __dp4a((int) q[4 % ((BS - 2) / 4)], (int) x1.x, s); s = __dp4a((int) q[5 % ((BS - 2) / 4)], (int) x1.y, s);
                            s = __dp4a((int) q[6 % ((BS - 2) / 4)], (int) x1.z, s); s = __dp4a((int) q[7 % ((BS - 2) / 4)], (int) x1.w, s);
                            acc[n] += d * ds.x * (float) s;
                        }
                    }
                };
                block(std::integral_constant<int, 0>{}); block(std::integral_constant<int, 1>{});
                block(std::integral_constant<int, 2>{}); block(std::integral_constant<int, 3>{});
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

template <int T, int N>
static cudaError_t launch_q32_tn(const Q32Params & p, int sm_count, int device, int use_pdl, cudaStream_t stream) {
    constexpr int BS = (T == T_Q8_0) ? 34 : 18;
    const size_t smem = (size_t) N * ((p.K + 127) / 128) * 160 + (size_t) Q32_WARPS * (Q32_RUN_BLOCKS * BS + 16);
    auto kern = mmvq_q32_kernel<T, N>;
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
    const int64_t need = ((int64_t) p.M + Q32_WARPS - 1) / Q32_WARPS;
    if (grid > need) grid = need;
    if (grid < 1) grid = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned) grid); cfg.blockDim = dim3(Q32_WARPS * 32);
    cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = use_pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, p);
}

template <int T>
static cudaError_t launch_q32_t(const Q32Params & p, int N, int sm, int dev, int pdl, cudaStream_t st) {
    switch (N) {
        case 1: return launch_q32_tn<T, 1>(p, sm, dev, pdl, st);
        case 2: return launch_q32_tn<T, 2>(p, sm, dev, pdl, st);
        case 3: return launch_q32_tn<T, 3>(p, sm, dev, pdl, st);
        case 4: return launch_q32_tn<T, 4>(p, sm, dev, pdl, st);
        case 5: return launch_q32_tn<T, 5>(p, sm, dev, pdl, st);
        case 6: return launch_q32_tn<T, 6>(p, sm, dev, pdl, st);
        case 7: return launch_q32_tn<T, 7>(p, sm, dev, pdl, st);
        case 8: return launch_q32_tn<T, 8>(p, sm, dev, pdl, st);
    }
    return cudaErrorInvalidValue;
}

// needs 16-byte aligned rows made of whole 8-block groups and whole activation blocks, no batching / expert indirection
bool mmvq_q32_applicable(const MmvqArgs & a) {
    if ((a.type != T_Q4_0 && a.type != T_Q8_0 && a.type != T_IQ4_NL) || a.ids || a.ne12 * a.ne13 != 1) return false;
    if (((uintptr_t) a.W & 15) || (a.w_nb1 & 15) || (a.K % 256) != 0) return false;
    const int bs = a.type == T_Q8_0 ? 34 : 18;
    if ((size_t) a.N * ((a.K + 127) / 128) * 160 + (size_t) Q32_WARPS * (Q32_RUN_BLOCKS * bs + 16) > 200 * 1024) return false;
    return true;
}

cudaError_t launch_mmvq_q32(const MmvqArgs & a, cudaStream_t stream) {
    Q32Params p = {};
    p.W = (const uint8_t *) a.W; p.w_nb1 = a.w_nb1;
    p.Xq = (const uint8_t *) a.Xq; p.xq_col_bytes = (int64_t) ((a.K + 127) / 128) * 160;
    p.dst = a.dst; p.dst_nb1 = a.dst_nb1;
    p.M = a.M; p.K = a.K; p.x_col0 = a.x_col0;
    p.n_peer = a.n_peer; for (int i = 0; i < a.n_peer; ++i) p.peer_delta[i] = a.peer_delta[i];
    if (a.type == T_Q4_0) return launch_q32_t<T_Q4_0>(p, a.N, a.sm_count, a.device, a.use_pdl, stream);
    if (a.type == T_IQ4_NL) return launch_q32_t<T_IQ4_NL>(p, a.N, a.sm_count, a.device, a.use_pdl, stream);
    return launch_q32_t<T_Q8_0>(p, a.N, a.sm_count, a.device, a.use_pdl, stream);
}

}  // namespace b200
