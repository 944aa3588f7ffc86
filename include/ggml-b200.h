/*
 * ggml backend plugin entry points of libggml-b200.so.
 *
 * The library is a drop-in ggml device: the reference's registry dlopens it
 * (ggml_backend_load, ggml/src/ggml-backend-reg.cpp:133-256; the environment
 * variable GGML_BACKEND_PATH names an out-of-tree backend, :577-581) and binds
 * exactly the two symbols below.  Everything else is reached through the
 * function tables of ggml/src/ggml-backend-impl.h that the returned registry
 * object carries: reg (:191-207) -> device (:137-179) -> buffer type (:17-35) ->
 * buffer (:41-66) and backend/stream (:87-124, with graph_compute at :110).
 *
 * The types are the reference's own (this header needs ggml-backend.h on the
 * include path); the library does not link any ggml library.
 */
#ifndef GGML_B200_H
#define GGML_B200_H

#include "ggml-backend.h"

#ifdef __cplusplus
extern "C" {
#endif

/* replaces ggml_backend_cuda_reg() as bound by GGML_BACKEND_DL_IMPL
 * (ggml/src/ggml-backend-impl.h:215, :220-232; ggml/src/ggml-cuda/ggml-cuda.cu:3457).
 * Registry name "B200"; one device "B200_<i>" per visible sm_100 GPU. */
ggml_backend_reg_t ggml_backend_init(void);

/* ggml_backend_score_t (ggml/src/ggml-backend-impl.h:218): 0 when no sm_100
 * device is visible, so the loader skips the library. */
int ggml_backend_score(void);

/*
 * Names answered by reg->iface.get_proc_address:
 *   "ggml_backend_split_buffer_type"  ggml_backend_buffer_type_t (*)(int main_device, const float * tensor_split)
 *                                     (ggml/include/ggml-backend.h:188; libllama asks for it in row-split mode,
 *                                      src/llama-model.cpp:308-326).  Returns a buffer type that divides the rows of a
 *                                     matrix over the B200 devices of this process (boundaries rounded down to 128
 *                                     rows, all-zero tensor_split = equal shares; what ggml_backend_cuda_split_buffer_type
 *                                     is to the reference, ggml/src/ggml-cuda/ggml-cuda.cu:714-1040); tensors in it are
 *                                     accepted only as the weight operand of a 2-D MUL_MAT.  NULL for a main_device
 *                                     outside the registry.
 *   "ggml_backend_get_features"       ggml_backend_feature * (*)(ggml_backend_reg_t)   (ggml-backend.h:196-200)
 *   "ggml_backend_b200_get_stream"       void *   (*)(ggml_backend_t)   the backend's cudaStream_t, for event timing
 *   "ggml_backend_b200_get_launch_count" uint64_t (*)(ggml_backend_t)   kernels launched by graph_compute so far
 *   "ggml_backend_b200_get_status"       int      (*)(ggml_backend_t)   device status word (0 = no kernel gave up a wait)
 *   "ggml_backend_b200_set_peers"        int      (*)(ggml_backend_t, const ggml_b200_peers *)   row-split set-up, below
 * Unknown names return NULL.
 */

/*
 * Row-split across the GPUs of one node, one process per GPU.
 *
 * The reference splits the rows of a weight matrix over the devices of ONE process through its split
 * buffer type and gathers the dst slices with peer copies (ggml/src/ggml-cuda/ggml-cuda.cu:714-1040,
 * :1520-1660); the buffer type above does the same.  This second form keeps the exchange inside the kernels
 * and the CUDA graph: every rank is its own process with its own backend; each rank's graph holds only
 * its rows of each split matrix, and a MUL_MAT node says where its slice belongs in the full result:
 *
 *   node->op == GGML_OP_MUL_MAT, node->src[0] = this rank's rows [row_low, row_low + node->ne[0]) of the matrix,
 *   node->data = full_data + 4 * row_low, node->nb[1] = the full result's column stride,
 *   node->extra -> ggml_b200_row_slice {GGML_B200_ROW_SLICE_MAGIC, full_data, full_rows, row_low}
 *
 * After computing such a node the backend stores the slice into the same place of every peer's arena and,
 * before the next node that is not another sliced MUL_MAT, runs a barrier over all ranks; from then on the
 * full result [full_rows x n_cols] at full_data is valid on every rank.  All ranks must run the same graph.
 * ggml_backend_b200_set_peers tells the backend where the peers' arenas are mapped in this process
 * (cudaIpcOpenMemHandle of the peers' compute buffers; they must have the same size and layout).  The
 * first GGML_B200_PEER_FLAG_BYTES of the arena are reserved for the barrier's flags and must be zero.
 */
#define GGML_B200_ROW_SLICE_MAGIC 0x42323030524f5753ull
#define GGML_B200_MAX_PEERS       8
#define GGML_B200_PEER_FLAG_BYTES 256
typedef struct ggml_b200_row_slice {
    uint64_t magic;
    void *   full_data;      /* start of the full [full_rows x n_cols] F32 result in this rank's arena */
    int64_t  full_rows;
    int64_t  row_low;
} ggml_b200_row_slice;
typedef struct ggml_b200_peers {
    int32_t rank, n_ranks;
    void *  arena[GGML_B200_MAX_PEERS];   /* arena[r]: where rank r's arena is mapped here; arena[rank] = this rank's own */
    size_t  arena_bytes;
} ggml_b200_peers;

#ifdef __cplusplus
}
#endif
#endif /* GGML_B200_H */
