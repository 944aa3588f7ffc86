/*
 * Llama-architecture graph driver over the ggml backend C-ABI.
 *
 * It plays the part that libllama + llama-bench play for the reference
 * (llama_decode, src/llama.cpp:8586; graph llm_build_context::build_llama,
 * src/llama.cpp:1476-1640; timing loop examples/llama-bench/llama-bench.cpp:1430-1468):
 * it builds the per-ubatch cgraph of a Llama model (struct ggml_tensor /
 * struct ggml_cgraph laid out by hand, exactly as ggml's constructors would) and
 * runs it through a backend's function tables -- buffer type alloc_buffer,
 * buffer set_tensor/get_tensor, backend graph_compute and synchronize
 * (ggml/src/ggml-backend-impl.h).  Any backend that implements that ABI can be
 * driven: the B200 plugin in this library, or the reference CPU backend loaded
 * from its own shared object (used as the timed CPU baseline).
 *
 * All data crossing this interface are host buffers: quantized weight bytes in,
 * token ids in, logits out.
 */
#ifndef B200_LLAMA_H
#define B200_LLAMA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct b200_llama b200_llama;

typedef struct b200_llama_config {
    int32_t n_layer, n_embd, n_head, n_head_kv, n_ff, n_vocab;
    int32_t n_ctx;          /* KV cache length (tokens) */
    int32_t n_ubatch;       /* largest number of tokens per graph */
    float   rope_theta, rms_eps;
    int32_t n_threads;      /* forwarded to the backend's "ggml_backend_set_n_threads" when it has one */
    int32_t n_ranks, rank;  /* row-split over n_ranks processes, one GPU each (0 or 1: not split); B200 backend only */
} b200_llama_config;

/* reg: a ggml_backend_reg_t (as returned by a backend library's ggml_backend_init), or NULL for
 * this library's own B200 registry.  Weight tensor types follow the reference's Q4_K_M mixture
 * (src/llama-quant.cpp:129-131, 235-243, 291-298): Q4_K, with Q6_K for output.weight and for
 * attn_v / ffn_down on the "more bits" layers; an 80-layer (70B-class) model keeps the other attn_v
 * tensors at Q5_K.  Returns NULL on failure (b200_llama_error()). */
b200_llama * b200_llama_create(void * reg, int32_t device_index, const b200_llama_config * cfg);
void         b200_llama_free(b200_llama * m);
const char * b200_llama_error(void);

/* ---- model files ------------------------------------------------------------------------------
 * b200_llama_load_gguf: the step before the hot path.  Reads a GGUF file of a Llama-architecture model (the
 * reference's on-disk format, ggml/include/gguf.h:1-68; its loader: src/llama-model-loader.cpp, ggml/src/gguf.cpp),
 * takes the hyper-parameters from its `llama.*` keys and the type of every weight from its tensor infos, and
 * copies the tensor data from the read-only file mapping into the backend's weight buffer -- on the B200
 * backend in 16 MB chunks that a few worker threads stage through pinned buffers into asynchronous
 * host-to-device copies, each rank only its own rows when n_ranks > 1.  A file without output.weight uses the token embeddings for the
 * output projection; rope_freqs.weight (Llama-3.1 files), when present, becomes the frequency-factor operand of
 * every ROPE.  Rejected with an error: other architectures, expert tensors, a rope.scaling.type other than
 * none, partial rotary dimensions, tensor types this backend has no kernel for.
 * b200_gguf_*: the reader by itself (metadata and tensor directory of any GGUF file, version 2 or 3). */
typedef struct b200_gguf b200_gguf;
b200_llama * b200_llama_load_gguf(void * reg, int32_t device_index, const char * path, int32_t n_ctx, int32_t n_ubatch,
                                  int32_t n_threads, int32_t n_ranks, int32_t rank);
void         b200_llama_get_config(const b200_llama * m, b200_llama_config * cfg);
b200_gguf *  b200_gguf_open(const char * path);            /* NULL on failure: b200_gguf_error() */
void         b200_gguf_close(b200_gguf * g);
const char * b200_gguf_error(void);
uint32_t     b200_gguf_version(const b200_gguf * g);
uint32_t     b200_gguf_alignment(const b200_gguf * g);
uint64_t     b200_gguf_data_offset(const b200_gguf * g);   /* file offset of the tensor data section */
int64_t      b200_gguf_n_kv(const b200_gguf * g);
int64_t      b200_gguf_n_tensors(const b200_gguf * g);
/* key i in file order with its gguf_type; for arrays (type 9) also the element type and count */
int32_t      b200_gguf_key(const b200_gguf * g, int64_t i, char * key, size_t key_cap, uint32_t * type, uint32_t * elem_type, uint64_t * count);
int32_t      b200_gguf_get_u32(const b200_gguf * g, const char * key, uint32_t * value);     /* 0 if present and integral */
int32_t      b200_gguf_get_f32(const b200_gguf * g, const char * key, float * value);
int32_t      b200_gguf_get_str(const b200_gguf * g, const char * key, char * value, size_t value_cap);
int32_t      b200_gguf_tensor_info(const b200_gguf * g, int64_t i, char * name, size_t name_cap, int32_t * type, int32_t * n_dims,
                                   int64_t * ne /* [4] */, uint64_t * offset, size_t * nbytes);
int64_t      b200_gguf_find_tensor(const b200_gguf * g, const char * name);                  /* index or -1 */
const void * b200_gguf_tensor_data(const b200_gguf * g, int64_t i);                          /* inside the mapping */

/* weight tensors, in a fixed order; names follow the GGUF convention ("blk.0.attn_q.weight") */
int32_t      b200_llama_n_tensors(const b200_llama * m);
int32_t      b200_llama_tensor_info(const b200_llama * m, int32_t i, char * name, size_t name_cap,
                                    int32_t * type, int64_t * ne0, int64_t * ne1, size_t * nbytes);
int32_t      b200_llama_set_tensor(b200_llama * m, int32_t i, const void * host_data, size_t nbytes);
/* address of tensor i inside the backend's weight buffer (a device pointer on the B200 backend) */
void *       b200_llama_tensor_data(const b200_llama * m, int32_t i);

/* ---- row-split (the reference's split-mode row, one process per GPU) -----------------------
 * With n_ranks > 1 every rank holds rows [row_low, row_high) of each 2-D projection matrix and of
 * output.weight (norms, embeddings and the KV cache are replicated), computes that slice of every
 * MUL_MAT and stores it into all peers' activation arenas over NVLink; a barrier kernel then makes
 * the full result readable everywhere (include/ggml-b200.h).  All ranks must call b200_llama_decode
 * with the same tokens.
 *
 * b200_row_split_range: equal shares with boundaries rounded down to a multiple of 128 rows, the last
 *   rank taking the remainder (get_row_split, ggml/src/ggml-cuda/ggml-cuda.cu:725-742).
 * b200_llama_tensor_rows: first row and full row count of tensor i (b200_llama_tensor_info reports
 *   this rank's share: ne1 = row_high - row_low).
 * b200_llama_ipc_handle / b200_llama_attach_peers: set-up.  Each rank exports the CUDA IPC handle of its
 *   arena (B200_LLAMA_IPC_HANDLE_BYTES bytes), the caller gathers the handles of all ranks in rank order
 *   (n_ranks x B200_LLAMA_IPC_HANDLE_BYTES bytes, e.g. with torch.distributed.all_gather_object) and hands
 *   them to attach_peers.  These have no reference counterpart: the reference's ranks share one process. */
#define B200_LLAMA_IPC_HANDLE_BYTES 64
void         b200_row_split_range(int64_t n_rows, int32_t rank, int32_t n_ranks, int64_t * row_low, int64_t * row_high);
int32_t      b200_llama_tensor_rows(const b200_llama * m, int32_t i, int64_t * row_low, int64_t * full_rows);
int32_t      b200_llama_ipc_handle(b200_llama * m, void * handle_out);
int32_t      b200_llama_attach_peers(b200_llama * m, const void * handles);

/* Evaluates n_tokens tokens at KV positions [pos0, pos0 + n_tokens) (one ubatch, n_tokens <= n_ubatch):
 * token ids are copied host->device, the graph is computed, and the logits of the LAST token
 * (n_vocab floats) are copied device->host into logits_host (may be NULL to skip the read).
 * Returns 0 on success. */
int32_t      b200_llama_decode(b200_llama * m, const int32_t * tokens, int32_t n_tokens, int32_t pos0, float * logits_host);

/* statistics of the most recent decode */
int32_t      b200_llama_last_n_nodes(const b200_llama * m);      /* nodes handed to graph_compute */
double       b200_llama_last_compute_ms(const b200_llama * m);   /* device time of graph_compute (CUDA events) on the
                                                                    B200 backend; host wall time on other backends */
uint64_t     b200_llama_launch_count(const b200_llama * m);      /* kernels launched so far (B200 backend only) */
size_t       b200_llama_weight_bytes(const b200_llama * m);      /* bytes of all weight tensors read per token */

#ifdef __cplusplus
}
#endif
#endif /* B200_LLAMA_H */
