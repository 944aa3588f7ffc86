/*
 * Flat C-ABI over the B200 (sm_100a) kernels of libggml-b200.so: plain pointers,
 * sizes and ggml_type numbers, no ggml or torch types.  This is the layer a
 * foreign-function binding (ctypes, cgo, JNI ...) would call; the ggml backend
 * plugin declared in ggml-b200.h sits on the same kernels.
 *
 * Conventions
 *  - `type` arguments are ggml_type values (ggml/include/ggml.h:351-392):
 *    0 F32, 1 F16, 2 Q4_0, 3 Q4_1, 6 Q5_0, 7 Q5_1, 8 Q8_0, 10 Q2_K, 11 Q3_K, 12 Q4_K, 13 Q5_K, 14 Q6_K,
 *    20 IQ4_NL, 23 IQ4_XS.
 *  - Matrices use ggml's layout: a weight matrix W[K, M] is M rows of K values,
 *    each row a run of quantized blocks (ggml/src/ggml-common.h:161-328);
 *    activations X[K, N] are N contiguous F32 columns; dst[M, N] is N columns of M.
 *  - Functions ending in `_host` take HOST pointers; they allocate device
 *    memory, copy in, run the kernels on the current device and copy the result
 *    back before returning.  All others take DEVICE pointers and are
 *    asynchronous on `stream` (a cudaStream_t passed as void *).
 *  - Return value: 0 on success, otherwise a cudaError_t value or a negative
 *    B200_E_* code; b200_last_error() returns a message for the calling thread.
 *  - Nothing here falls back to the CPU: without a B200 the calls fail.
 */
#ifndef B200_KERNELS_H
#define B200_KERNELS_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_E_UNSUPPORTED  (-1)   /* type / shape not handled by the kernels */
#define B200_E_BAD_ARG      (-2)
#define B200_E_NO_DEVICE    (-3)   /* no sm_100 device visible */
#define B200_E_SCRATCH      (-4)   /* scratch buffer too small */
#define B200_E_DEVICE_WAIT  (-5)   /* a kernel gave up a bounded wait (status word set) */

int          b200_device_count(void);      /* number of visible sm_100 devices (0 without a GPU) */
const char * b200_last_error(void);
size_t       b200_row_size(int type, int64_t k);   /* bytes of one row of k values; ggml_row_size, ggml/src/ggml.c:1204 */

/* ---- MUL_MAT with quantized weights -------------------------------------
 * dst[n][m] = sum_k W[m][k] * X[n][k], as GGML_OP_MUL_MAT computes it
 * (ggml_mul_mat, ggml/src/ggml.c:2694-2709; CUDA path ggml_cuda_mul_mat,
 * ggml/src/ggml-cuda/ggml-cuda.cu:1839-1900).  Activations are quantized to int8
 * per 32 values on the device (the scratch buffer holds them), N <= 8 takes the
 * bandwidth-bound mat-vec kernel, larger N the tensor-core kernel.            */
size_t b200_mul_mat_q_scratch_bytes(int type, int64_t M, int64_t K, int64_t N);
int    b200_mul_mat_q(int type, const void * W, int64_t w_row_stride_bytes, int64_t M, int64_t K,
                      const float * X, int64_t x_col_stride_elems, int64_t N,
                      float * dst, int64_t dst_col_stride_elems,
                      void * scratch, size_t scratch_bytes, void * stream);
/* The two halves of the N <= 8 path on their own: the activation quantizer (what the reference does in
 * quantize_q8_1, ggml/src/ggml-cuda/quantize.cu:4-38) writing b200_act_bytes(K, N) bytes, and the mat-vec
 * kernel on activations quantized earlier (mul_mat_vec_q, ggml/src/ggml-cuda/mmvq.cu:50-130).          */
size_t b200_act_bytes(int64_t K, int64_t N);
/* Programmatic dependent launch for the device-pointer entry points (off by default; the ggml backend
 * has it on by default): the mat-vec kernels request their first weight rows before waiting for the kernel
 * launched just before them on the stream (griddepcontrol), so consecutive launches overlap head and tail.
 * Only turn it on when no weight operand is written by the kernel launched immediately before it on the
 * same stream.  No reference counterpart. */
void   b200_set_dependent_launch(int on);
int    b200_quantize_act(const float * X, int64_t x_col_stride_elems, int64_t K, int64_t N, void * xq, void * stream);
int    b200_mul_mat_vec_q(int type, const void * W, int64_t w_row_stride_bytes, int64_t M, int64_t K,
                          const void * xq, int64_t N, float * dst, int64_t dst_col_stride_elems, void * stream);
int    b200_mul_mat_q_host(int type, const void * W, int64_t M, int64_t K, const float * X, int64_t N, float * dst);

/* ---- MUL_MAT without any allocation --------------------------------------
 * No counterpart in the reference: an addition of this library.
 *
 * Some callers cannot allocate device memory at the point where they need the product: a
 * real-time serving loop with a frozen memory budget, a plugin host that forbids cudaMalloc after
 * start-up, or a process whose device allocator is owned by another framework.  b200_mul_mat_q needs a caller-provided scratch buffer for the int8 activation
 * blocks; this variant keeps that scratch inside the library instead, in a fixed device array of
 * B200_NOALLOC_SCRATCH_BYTES that every GPU loading the library holds until the process exits.
 * The caller passes only inputs and outputs (device pointers).  The call makes no cudaMalloc,
 * cudaFree or allocating library call.
 *
 *  - Limits: N <= 8 columns and b200_act_bytes(K, N) <= B200_NOALLOC_SCRATCH_BYTES (e.g. K up to
 *    104857 at N = 8); anything larger is rejected with B200_E_SCRATCH / B200_E_UNSUPPORTED and a
 *    message from b200_noalloc_last_error().
 *  - The first call on each device looks up the array's device address (with that device
 *    current) and clears a status word; make that first call before any stream capture begins.
 *    With CUDA's lazy module loading the driver also materialises the array and each kernel
 *    variant (weight type, N) the first time it is used, so "allocates nothing" holds from the
 *    second call of a given (device, type, N) on: warm each combination up once at start-up.
 *    The first call is serialised per device, so several host threads may race to make it.
 *  - All calls on a device share the one array, which keeps whatever the last call wrote.  The
 *    kernels overwrite the part they use before reading it, so no clearing is needed between
 *    calls; but two calls that overlap on the GPU (different streams, no ordering) race on it.
 *  - Asynchronous on `stream`; same arithmetic and results as b200_mul_mat_q for N <= 8.
 *  - Arguments the kernels could fault on (null or misaligned pointers, strides shorter than
 *    a row) are rejected with B200_E_BAD_ARG before anything is launched.
 *  - A kernel that gives up a bounded wait leaves garbage in dst and records it in a status
 *    word; the launching call has long returned 0 by then.  b200_noalloc_status(stream)
 *    synchronises the stream, returns B200_E_DEVICE_WAIT if that happened since the last
 *    check (0 otherwise) and clears the word.  It allocates nothing either.                  */
#define B200_NOALLOC_SCRATCH_BYTES (1u << 20)
int          b200_mul_mat_q_noalloc(int type, const void * W, int64_t w_row_stride_bytes, int64_t M, int64_t K,
                                    const float * X, int64_t x_col_stride_elems, int64_t N,
                                    float * dst, int64_t dst_col_stride_elems, void * stream);
int          b200_noalloc_status(void * stream);
const char * b200_noalloc_last_error(void);

/* ---- single phases of the persistent decode-step kernel -------------------
 * The ggml backend runs a whole run of Llama layers for one token as ONE cooperative launch
 * (csrc/kernels/decode_step.cu) instead of one launch per graph node (the reference's walk,
 * ggml/src/ggml-cuda/ggml-cuda.cu:2691-2765).  These host-buffer entry points run one phase of that
 * kernel at a time so that each can be checked against the oracle of the op sequence it replaces:
 *  - mul_mat:   dst[M] = W . y with y = x (+ x_add), or rms_norm(x (+ x_add), eps) * norm_w when norm_w is set
 *               (ADD, RMS_NORM, MUL, MUL_MAT of src/llama.cpp:1476-1640); sum_out (optional) receives x + x_add
 *  - gate_up:   dst[M] = silu(Wg . x) * (Wu . x)            (MUL_MAT x2, UNARY(SILU), MUL)
 *  - qkv:       q_out = rope(Wq . y), k_row = f16(rope(Wk . y)), v_row = f16(Wv . y) for one token at
 *               position pos; head size 128, adjacent-pair rotation (MUL_MAT x3, ROPE x2, CPY x2)
 *  - attention: FLASH_ATTN_EXT for one query token over contiguous F16 K/V [n_head_kv][n_kv][128], split into
 *               n_slices KV slices, merged in slice order either by the attention phase itself or
 *               (merge_in_next_phase, 2..8 slices) by the input stage of the mat-vec phase that follows
 * Weight types: Q4_K, Q5_K, Q6_K (K a multiple of 256; of 2048 for Q6_K).                                   */
int          b200_decode_step_mul_mat_host(int type, const void * W, int64_t M, int64_t K, const float * x, const float * x_add,
                                           const float * norm_w, float eps, float * dst, float * sum_out);
int          b200_decode_step_gate_up_host(int type, const void * Wg, const void * Wu, int64_t M, int64_t K, const float * x, float * dst);
int          b200_decode_step_qkv_host(int type_qk, int type_v, const void * Wq, const void * Wk, const void * Wv, int64_t n_head,
                                       int64_t n_head_kv, int64_t K, const float * x, const float * norm_w, float eps, int32_t pos,
                                       int n_dims, float freq_base, const float * freq_factors, float * q_out, void * k_row_f16,
                                       void * v_row_f16);
int          b200_decode_step_attention_host(const float * q, const void * k_f16, const void * v_f16, const void * mask_f16,
                                             int64_t n_kv, int64_t n_head, int64_t n_head_kv, float scale, int n_slices,
                                             int merge_in_next_phase, float * dst);
const char * b200_decode_step_last_error(void);

/* ---- the bounded wait of the row-split barrier, observable on one GPU ------
 * No counterpart in the reference (its multi-GPU path synchronises with events inside one process).  The
 * barrier between the ranks of a row-split run (include/ggml-b200.h) spins on flags the peers write; the spin
 * is bounded.  This probe runs that kernel as rank 0 of 2 with both flag arrays in local memory: with
 * peer_arrives = 0 nothing ever writes the flag, the wait runs out after spin_limit polls, *status_out
 * becomes 3 (ERR_PEER_TIMEOUT) and the kernel returns normally; with peer_arrives = 1 it passes (0).   */
int b200_peer_barrier_probe_host(int spin_limit, int peer_arrives, int * status_out);

/* ---- the int8 form of the prefill GEMM, measured ---------------------------
 * No counterpart in the reference.  The reference's prefill mat-mul runs int8 MMAs of 32-deep steps and applies the
 * block scales to each step's int32 result in FP32 (ggml/src/ggml-cuda/mmq.cuh:649-727).  This probe runs that
 * structure on tcgen05 with nothing else around it (fixed operands in shared memory): per step one 128 x 256 x 32
 * `kind::i8` MMA into tensor memory, read back by eight warps and folded into FP32 sums with a row and a column scale.
 * *us_per_kblock = time of one step of one CTA (every SM runs a CTA), *check = one element of the result, *expected =
 * what it must be.  Used by `microbench.py i8_probe` to put a number on the alternative the product does not take.   */
int b200_tc_i8_probe_host(int kblocks, int reps, float * us_per_kblock, float * check, float * expected);

/* ---- FLASH_ATTN_EXT -------------------------------------------------------
 * GGML_OP_FLASH_ATTN_EXT (ggml_flash_attn_ext, ggml/src/ggml.c:4306-4345; CPU
 * semantics ggml/src/ggml-cpu/ggml-cpu.c:10916-11129).  q F32 [D, n_q, n_head],
 * k/v F16 [D, n_kv, n_head_kv] with byte strides (token, head), mask F16
 * [n_kv, >= n_q] contiguous or NULL, dst F32 [D, n_head, n_q].               */
size_t b200_flash_attn_scratch_bytes(int64_t D, int64_t n_q, int64_t n_head, int64_t n_kv);
int    b200_flash_attn(const float * q, int64_t q_nb1, int64_t q_nb2,
                       const void * k, int64_t k_nb1, int64_t k_nb2,
                       const void * v, int64_t v_nb1, int64_t v_nb2,
                       const void * mask, int64_t mask_nb1, float * dst,
                       int64_t D, int64_t n_q, int64_t n_head, int64_t n_kv, int64_t n_head_kv,
                       float scale, float max_bias, float logit_softcap,
                       void * scratch, size_t scratch_bytes, void * stream);
int    b200_flash_attn_host(const float * q, const void * k, const void * v, const void * mask, float * dst,
                            int64_t D, int64_t n_q, int64_t n_head, int64_t n_kv, int64_t n_head_kv,
                            float scale, float max_bias, float logit_softcap);

/* ---- bit-exact format conversions ----------------------------------------
 * dequantize: what GET_ROWS / dequantize_row_* produce (ggml/src/ggml-quants.c:
 * 255-363, 1280-1302, 1482-1507, 1690-1719).  quantize: what CPY F32 -> Q does,
 * i.e. quantize_row_{q8_0,q4_0,q4_1,q5_0,q5_1}_ref (:31-217).  f32_to_f16: the
 * KV-cache store (CPY F32 -> F16, round to nearest even).                     */
int b200_dequantize_rows_host(int type, const void * src, int64_t n_rows, int64_t k, float * dst);
int b200_get_rows_host(int type, const void * src, int64_t n_src_rows, int64_t k, const int32_t * idx, int64_t n_idx, float * dst);
int b200_quantize_rows_host(int type, const float * src, int64_t n_rows, int64_t k, void * dst);
int b200_f32_to_f16_host(const float * src, int64_t n, void * dst);

/* ---- glue ops (host-buffer forms, used by the parity tests) --------------- */
int b200_rms_norm_host(const float * x, int64_t n_rows, int64_t k, float eps, const float * weight /* [k] or NULL */, float * dst);
int b200_rope_host(const float * x, int64_t head_dim, int64_t n_head, int64_t n_tok, const int32_t * pos,
                   const float * freq_factors /* [n_dims/2] or NULL */, int n_dims, int mode, int n_ctx_orig,
                   float freq_base, float freq_scale, float ext_factor, float attn_factor, float beta_fast, float beta_slow,
                   float * dst);
int b200_silu_mul_host(const float * gate, const float * up, int64_t n, float * dst);
int b200_soft_max_host(const float * x, int64_t n_rows, int64_t k, const void * mask_f16 /* [k, n_rows] or NULL */, float scale, float * dst);

#ifdef __cplusplus
}
#endif
#endif /* B200_KERNELS_H */
