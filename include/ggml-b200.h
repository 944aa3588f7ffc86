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
 *                                      src/llama-model.cpp:308-326)
 *   "ggml_backend_get_features"       ggml_backend_feature * (*)(ggml_backend_reg_t)   (ggml-backend.h:196-200)
 *   "ggml_backend_b200_get_stream"       void *   (*)(ggml_backend_t)   the backend's cudaStream_t, for event timing
 *   "ggml_backend_b200_get_launch_count" uint64_t (*)(ggml_backend_t)   kernels launched by graph_compute so far
 *   "ggml_backend_b200_get_status"       int      (*)(ggml_backend_t)   device status word (0 = no kernel gave up a wait)
 * Unknown names return NULL.
 */

#ifdef __cplusplus
}
#endif
#endif /* GGML_B200_H */
