// Internal C++ interface between the host layer and the CUDA kernels.
// No ggml types here: tensors are described by a plain descriptor that mirrors
// ggml's ne[]/nb[] convention (element counts, byte strides; dim 0 innermost).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stddef.h>

namespace b200 {

struct TensorD {
    void *  data;
    int     type;        // ggml_type value
    int64_t ne[4];
    int64_t nb[4];
};

// launch context shared by all kernels of one backend instance
struct LaunchCtx {
    cudaStream_t stream;
    int   device;
    int   sm_count;
    int * status;        // device status word (ERR_* codes), never reset by kernels
    int   use_pdl;       // launch with programmatic stream serialization where supported
    unsigned * fa_tickets;   // FATTN_DEC_TICKETS zero-initialised counters for the decode attention kernel (or null)
};
static constexpr int FATTN_DEC_TICKETS = 4096;

// ---- row-split exchange over peer memory (peer.cu) ----
static constexpr int MAX_PEERS = 8;                    // ranks per node
struct PeerPush {                                      // copy a [ncols][col_bytes] slab (column stride col_stride) to every peer
    const char * src; char * peer_dst[MAX_PEERS - 1]; int n_peer;
    int64_t col_bytes, col_stride, ncols; int shift;   // shift: 4 = 16-byte elements, 2 = 4-byte elements
};
struct PeerBarrier {
    unsigned * epoch;                                  // this rank's epoch counter (device memory)
    unsigned * local_flags;                            // [MAX_PEERS], slot r written by rank r
    unsigned * peer_flags[MAX_PEERS];                  // the flag arrays of the other ranks (mapped)
    int rank, n_ranks; int * status;
    int spin_limit;                                    // polls before the wait gives up (0: the default, a few seconds)
};
cudaError_t launch_peer_push(const PeerPush & p, const LaunchCtx & c);
cudaError_t launch_peer_barrier(const PeerBarrier & b, const LaunchCtx & c);

// ---- quantized mat-vec (mmvq.cu) ----
struct MmvqArgs {
    int type;
    const void * W;  int64_t w_nb1, w_nb2, w_nb3;
    const void * Xq;                                   // blk_act128 columns ordered [i13][i12][n]
    float * dst;     int64_t dst_nb1, dst_nb2, dst_nb3;
    int M, K, N, ne12, ne13, r2, r3;                   // N = columns of this launch (1..8)
    int x_col0, x_ncols, xq_ne12;                      // first column, columns per batch in Xq, dim-2 extent of Xq (0 = ne12)
    const int32_t * ids; int64_t ids_s12, ids_s13;     // MUL_MAT_ID expert indices (or null)
    int * status; int sm_count, device, use_pdl;
    // up to two more weight matrices of the same type, K and row stride that share Xq (direct Q4_K/Q5_K kernel only)
    int n_extra; const void * extra_W[2]; float * extra_dst[2]; int64_t extra_dst_nb1[2]; int extra_M[2];
    // row-split: every result is also stored at dst + peer_delta[i] (the same place in each peer's mapped arena)
    int n_peer; int64_t peer_delta[MAX_PEERS - 1];
};
bool        mmvq_type_supported(int type);
size_t      act128_bytes(int64_t K, int64_t ncols);
// columns ordered [i13][i12][i11]; s11..s13 are element strides of x
cudaError_t launch_quantize_act128(const float * x, int64_t ne11, int64_t ne12, int64_t ne13,
                                   int64_t s11, int64_t s12, int64_t s13, void * y, int K, cudaStream_t stream, int use_pdl = 0);
cudaError_t launch_mmvq(const MmvqArgs & a, cudaStream_t stream);
// true when the kernel launch_mmvq picks writes the peer copies itself (n_peer, peer_delta); otherwise
// the caller pushes the slab with launch_peer_push
bool        mmvq_stores_to_peers(const MmvqArgs & a);
// direct 128-bit-coalesced variant for Q4_K / Q5_K (mmvq_k.cu); launch_mmvq routes to it when applicable
bool        mmvq_k_applicable(const MmvqArgs & a);
cudaError_t launch_mmvq_k(const MmvqArgs & a, cudaStream_t stream);
// warp-staged variant for Q4_0 / Q8_0 (mmvq_q32.cu)
bool        mmvq_q32_applicable(const MmvqArgs & a);
cudaError_t launch_mmvq_q32(const MmvqArgs & a, cudaStream_t stream);
// warp-staged variant for Q6_K (mmvq_q6k.cu)
bool        mmvq_q6k_applicable(const MmvqArgs & a);
cudaError_t launch_mmvq_q6k(const MmvqArgs & a, cudaStream_t stream);
// 3 .. 8 columns of Q4_K (GGML_B200_MMQ_S8: 0 = off, 1 = also 2 columns and Q8_0, 9..16 = the largest column count) on the
// integer tensor-core instruction (mmq_s8.cu): all n_cols columns from a.x_col0 on, the grouped matrices (n_extra) one launch each.
// shape_ok: what can be told from the node alone.
bool        mmq_s8_shape_ok(int type, int64_t n_cols, int64_t K);
bool        mmq_s8_applicable(const MmvqArgs & a, int64_t n_cols);
cudaError_t launch_mmq_s8(const MmvqArgs & a, int64_t n_cols, cudaStream_t stream);

// ---- float mat-mul for F32/F16/BF16 weights (matmul_f.cu) ----
// dst[i3][i2][n][m] = sum_k W[..][m][k] * X[i3][i2][n][k]; W broadcast over dims 2,3
cudaError_t launch_matmul_f(const TensorD & W, const TensorD & X, const TensorD & dst, const LaunchCtx & c);

// ---- prefill quantized GEMM on tcgen05 (mmq_tc.cu) ----
bool        mmq_tc_supported(int type, int64_t M, int64_t N, int64_t K);
size_t      mmq_tc_workspace_bytes(int64_t N, int64_t K);
bool        mmq_tc_ptr_ok(int type, const void * W, int64_t w_nb1, const void * X, int64_t x_nb1_bytes);
cudaError_t launch_mmq_tc(int type, const void * W, int64_t w_nb1, const float * X, int64_t x_nb1,
                          float * dst, int64_t dst_nb1, int64_t M, int64_t N, int64_t K,
                          void * workspace, const LaunchCtx & c, bool preconverted = false,    // preconverted: workspace already holds X as F16
                          void * partials = nullptr);   // mmq_tc_partial_bytes() of scratch enables split-K when the output has few tiles
size_t      mmq_tc_partial_bytes(int64_t M, int64_t N, int64_t K, int sm_count);
// up to three weight matrices of one type, row length and row stride on the same activations (wq/wk/wv, gate/up) as ONE launch
cudaError_t launch_mmq_tc_group(int type, int n_mats, const void * const * W, int64_t w_nb1, const int64_t * M, float * const * dst,
                                const int64_t * dst_nb1, const float * X, int64_t x_nb1, int64_t N, int64_t K, void * workspace,
                                const LaunchCtx & c, bool preconverted = false, void * partials = nullptr);
size_t      mmq_tc_group_partial_bytes(int n_mats, const int64_t * M, int64_t N, int64_t K, int sm_count);
// MUL_MAT_ID over many (slot, token) pairs on the same GEMM: pairs sorted by expert on the device, one launch for all experts
bool        mmq_tc_moe_supported(int type, int64_t M, int64_t K, int64_t n_expert, int64_t n_pairs);
size_t      mmq_tc_moe_workspace_bytes(int64_t n_pairs, int64_t K, int64_t n_expert);
cudaError_t launch_mmq_tc_moe(int type, const void * W, int64_t w_nb1, int64_t w_nb2, int64_t n_expert, int64_t M, int64_t K,
                              const float * X, int64_t x_nb1, int64_t x_nb2, int64_t ne11,
                              const int32_t * ids, int64_t ids_nb1, int64_t n_used, int64_t n_tok,
                              float * dst, int64_t dst_nb1, int64_t dst_nb2, void * workspace, const LaunchCtx & c);

// ---- F16 / BF16 weight matrices on the fast paths (matmul_f_tc.cu): tcgen05 GEMM for more than 8 columns, warp-per-row mat-vec below ----
bool        mm16_tc_applicable(const TensorD & W, const TensorD & X, const TensorD & dst);
size_t      mm16_tc_workspace_bytes(int64_t N, int64_t K);
cudaError_t launch_mm16_tc(const TensorD & W, const TensorD & X, const TensorD & dst, void * workspace, const LaunchCtx & c);
bool        mv16_applicable(const TensorD & W, const TensorD & X, const TensorD & dst);
cudaError_t launch_mv16(const TensorD & W, const TensorD & X, const TensorD & dst, const LaunchCtx & c);

// ---- measurement of the int8 design alternative of the prefill GEMM (tc_i8_probe.cu); not on a product path ----
cudaError_t launch_tc_i8_probe(int kblocks, int reps, float * us_per_kblock, float * check, float * expected, const LaunchCtx & c);

// ---- glue ops (glue.cu) ----
enum BinOp { BIN_ADD = 0, BIN_SUB = 1, BIN_MUL = 2, BIN_DIV = 3 };
enum UnOp  { UN_SILU = 0, UN_GELU, UN_GELU_QUICK, UN_RELU, UN_TANH, UN_SIGMOID, UN_NEG, UN_EXP, UN_ABS, UN_SGN,
             UN_STEP, UN_ELU, UN_HARDSIGMOID, UN_HARDSWISH, UN_SQR, UN_SQRT, UN_SIN, UN_COS, UN_LOG };

cudaError_t launch_rms_norm(const TensorD & src, const TensorD & dst, float eps, const LaunchCtx & c);
// y = rms_norm(x) * w   (w broadcast like ggml MUL's src1); optionally also emits blk_act128 of y
// norm_out (optional): contiguous rows receiving the plain rms_norm(x).  addend/sum_out (optional, contiguous
// rows): the input becomes src + addend, which is also written to sum_out (fused residual add)
// f16_out (optional): dense [rows][ne0] F16 copy of dst, the operand format of the tensor-core mat-mul
cudaError_t launch_rms_norm_mul(const TensorD & src, const TensorD & w, const TensorD & dst, float eps,
                                void * act128_out, float * norm_out, const float * addend, float * sum_out, const LaunchCtx & c,
                                void * f16_out = nullptr);
cudaError_t launch_norm(const TensorD & src, const TensorD & dst, float eps, const LaunchCtx & c);
cudaError_t launch_bin_bcast(int op, const TensorD & a, const TensorD & b, const TensorD & dst, const LaunchCtx & c);
cudaError_t launch_unary(int op, const TensorD & src, const TensorD & dst, const LaunchCtx & c);
// dst = silu(gate) * up, optionally also emitting blk_act128 of dst
cudaError_t launch_silu_mul(const TensorD & gate, const TensorD & up, const TensorD & dst, void * act128_out, float * silu_out, const LaunchCtx & c,
                            void * f16_out = nullptr);
cudaError_t launch_scale(const TensorD & src, const TensorD & dst, float scale, const LaunchCtx & c);
cudaError_t launch_clamp(const TensorD & src, const TensorD & dst, float lo, float hi, const LaunchCtx & c);

struct RopeParams {
    int n_dims, mode, n_ctx_orig;
    float freq_base, freq_scale, ext_factor, attn_factor, beta_fast, beta_slow;
};
cudaError_t launch_rope(const TensorD & src, const int32_t * pos, const float * freq_factors, const TensorD & dst,
                        const RopeParams & rp, const LaunchCtx & c);

// ROPE(Q) + ROPE(K) + KV-cache store (K rotated, V as is; F32 -> F16) in one launch
struct RopeKvLaunch {
    const float * q_src; float * q_dst; const float * k_src; float * k_dst; const float * v_src;
    int64_t hd, n_head, n_head_kv, n_tok, v_elems;
    void * k_cache; void * v_cache; int64_t k_off, v_off;        // view bases and byte offsets
    const int64_t * k_off_dev; const int64_t * v_off_dev;        // if set, offsets are read from device memory instead
    const int32_t * pos; const float * ff;
    const char * pf_k; const char * pf_v; int64_t pf_bytes;   // optional: this layer's K / V rows, to be brought into L2 ahead of the attention phase
};
cudaError_t launch_rope_kv(const RopeKvLaunch & l, const RopeParams & rp, const LaunchCtx & c);

bool        cpy_supported(int src_type, int dst_type);
// dyn_off (optional, device pointer): byte offset added to dst.data, read by the kernel at run time
cudaError_t launch_cpy(const TensorD & src, const TensorD & dst, const LaunchCtx & c, const int64_t * dyn_off = nullptr);

bool        get_rows_supported(int src_type);
cudaError_t launch_get_rows(const TensorD & src, const TensorD & idx, const TensorD & dst, const LaunchCtx & c);

cudaError_t launch_soft_max(const TensorD & src, const TensorD * mask, const TensorD & dst, float scale, float max_bias,
                            const LaunchCtx & c);

// ---- persistent decode step (decode_step.cu) ----
// One cooperative launch runs a whole sequence of Llama layers for a single token: every phase is either
// a group of mat-vecs that share their input (with the producer of that input fused in front and the
// consumer of the results fused behind) or the attention over the KV cache; phases are separated by
// grid-wide barriers, and every warp keeps streaming the weights of the phases ahead into its own
// shared-memory ring while it waits.
enum { DS_OP_MATVEC = 1, DS_OP_ATTN = 2 };
enum { DS_IN_PLAIN = 0, DS_IN_NORM = 1, DS_IN_ATTN = 2 };       // mat-vec input: x, rms_norm(x) * w, or attention partials to merge
enum { DS_EP_STORE = 0, DS_EP_ROPE_KV = 1, DS_EP_SILU_MUL = 2 }; // what happens to the mat-vec results
struct alignas(16) DsOp {
    int kind;
    // ---- DS_OP_MATVEC ----
    int in_kind, K, nmat, epilogue;
    const float * in0; const float * in1;        // x = in0 (+ in1 when set)
    const float * norm_w; float eps;             // DS_IN_NORM
    float * sum_out;                             // receives x when in1 is set
    int in_slices, in_gqa;                       // DS_IN_ATTN: in0 = partials of the attention phase [n_head_kv][in_slices][in_gqa][DS partial stride]
    float * y_out;                               // optional: receives the (normalised) mat-vec input
    const void * W[3]; int type[3]; int M[3]; int64_t w_nb1[3];
    float * dst[3];                              // DS_EP_STORE: results; other epilogues: optional raw results
    // DS_EP_ROPE_KV: matrices wq, wk, wv; rows are rotated in adjacent pairs (ggml's normal rope mode)
    float * q_rope; float * k_rope;              // rotated Q (required), rotated K as F32 (optional)
    void * k_cache; void * v_cache;              // viewed cache tensors; rows go to base + offset as F16
    int64_t k_off, v_off; const int64_t * k_off_dev; const int64_t * v_off_dev;   // byte offsets: immediate, or read from device memory
    const int32_t * pos; const float * ff;
    const char * pf_k; const char * pf_v; int64_t pf_bytes;   // optional: this layer's K / V rows, to be brought into L2 ahead of the attention phase
    int head_dim, n_dims; float freq_scale, ext_factor, attn_factor, theta_scale, corr0, corr1;
    // DS_EP_SILU_MUL: matrices gate, up
    float * act_out; float * silu_out;           // silu(gate) * up (required), silu(gate) (optional)
    // ---- DS_OP_ATTN (one query token, head size 128, F16 K/V) ----
    const float * q;                             // [n_head][128]
    const char * k; const char * v; int64_t k_nb1, k_nb2, v_nb1, v_nb2;
    const void * mask;                           // F16 [n_kv] or null
    int n_kv, n_head, n_head_kv; float scale;
    float * partials; unsigned * tickets;        // split-KV partial results and per-KV-head counters (zero between uses)
    float * out;                                 // [n_head][128]
    int n_slices, kv_per_slice;
    int consumer_merge;                          // the slices are merged by the input stage of the next phase (DS_IN_ATTN), not here
    // both kinds: the V cache is kept transposed (graphs without FLASH_ATTN_EXT): v_nbd bytes between its head-size rows; F32 mask
    int v_t, mask_f32; int64_t v_nbd;
};
static constexpr int DS_MAX_MERGE_SLICES = 16;   // most KV slices the input stage of the next phase merges (consumer_merge)
static constexpr int DS_PARTIAL_STRIDE = 132;    // floats per (KV head, slice, query row) partial: O[128], max, sum, padding
bool        decode_step_type_ok(int type, int64_t K, int64_t w_nb1, const void * W);
// How many mat-vec ops one launch can hold (their descriptors live in shared memory), given the largest K
int         decode_step_max_matvecs(int device);
int64_t     decode_step_max_k();
// `ops` (host copy) describes the same ops as `ops_dev`; `work` is device memory of decode_step_work_bytes(n_ops)
// that this call fills (asynchronously, on `copy_stream`) with the mat-vec descriptors; sync: 4 zero words
size_t      decode_step_work_bytes(int n_ops);
cudaError_t decode_step_prepare(const DsOp * ops, int n_ops, int sm_count, void * work, cudaStream_t copy_stream);
cudaError_t launch_decode_step(const DsOp * ops_dev, const DsOp * ops, int n_ops, const void * work, unsigned * sync, const LaunchCtx & c,
                               unsigned long long * timing = nullptr);   // optional: 4 time stamps per phase written by CTA 0

// ---- flash attention (fattn.cu) ----
struct FattnParams { float scale, max_bias, logit_softcap; };
bool        fattn_supported(int64_t head_dim, int k_type, int v_type);
size_t      fattn_workspace_bytes(const TensorD & q, const TensorD & k, int sm_count);
// tensor-core kernel for batches of queries (fattn_mma.cu); launch_fattn routes to it when applicable
bool        fattn_mma_applicable(const TensorD & q, const TensorD & k, const TensorD & v, const TensorD * mask);
size_t      fattn_mma_workspace_bytes(const TensorD & q, const TensorD & k);
cudaError_t launch_fattn_mma(const TensorD & q, const TensorD & k, const TensorD & v, const TensorD * mask, const TensorD & dst,
                             const FattnParams & fp, void * workspace, const LaunchCtx & c);
// classifies the 64 x 64 tiles of an F16 mask: 0 mixed, 1 all -inf, 2 all zero (fattn_mma.cu)
cudaError_t launch_fattn_mask_flags(const char * mask, int64_t m_nb1, int n_q, int n_kv, uint8_t * flags, int flags_stride, const LaunchCtx & c);
// tcgen05 kernel for batches of queries at head size 128 (fattn_tc.cu): S and O in tensor memory, K/V by tiled tensor copies;
// workspace: fattn_mma_workspace_bytes()
bool        fattn_tc_applicable(const TensorD & q, const TensorD & k, const TensorD & v, const TensorD * mask, const FattnParams & fp);
cudaError_t launch_fattn_tc(const TensorD & q, const TensorD & k, const TensorD & v, const TensorD * mask, const TensorD & dst,
                            const FattnParams & fp, void * workspace, const LaunchCtx & c);
// n_kernels (optional) receives the number of kernels launched
// GQA-shared split-KV kernel for decode (fattn_dec.cu); needs LaunchCtx::fa_tickets
bool        fattn_dec_applicable(const TensorD & q, const TensorD & k, const TensorD & v, const TensorD * mask);
size_t      fattn_dec_workspace_bytes(const TensorD & q, const TensorD & k, int sm_count);
cudaError_t launch_fattn_dec(const TensorD & q, const TensorD & k, const TensorD & v, const TensorD * mask, const TensorD & dst,
                             const FattnParams & fp, void * tickets, void * partials, const LaunchCtx & c, void * act128_out = nullptr);
cudaError_t launch_fattn(const TensorD & q, const TensorD & k, const TensorD & v, const TensorD * mask, const TensorD & dst,
                         const FattnParams & fp, void * workspace, const LaunchCtx & c, int * n_kernels = nullptr,
                         void * act128_out = nullptr);   // honoured only when fattn_dec_applicable() (blk_act128 of dst, D = 128)

}  // namespace b200
