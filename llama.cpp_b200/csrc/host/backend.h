// Internal declarations shared by the files of the B200 ggml backend host layer.
#pragma once

#include "ggml_compat.h"

#include <cstring>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

namespace b200 {

struct DeviceCtx {
    int         device = 0;          // CUDA ordinal
    int         index  = 0;          // index within this backend's registry
    int         sm_count = 0;
    size_t      l2_bytes = 0;
    std::string name, description;
    ggml_backend_buffer_type buft      = {};
    ggml_backend_buffer_type host_buft = {};
    ggml_backend_device      dev       = {};
};

struct BufferCtx {
    int    device;
    void * base;
    size_t size;
};

// per-backend (stream) state
struct BackendCtx {
    DeviceCtx *  dev = nullptr;
    cudaStream_t stream = nullptr;
    int *        status_dev = nullptr;     // device status word written by kernels that give up a wait
    int *        status_host = nullptr;    // pinned mirror
    void *       scratch = nullptr;        // transient per-node workspace (activation blocks, attention partials)
    size_t       scratch_size = 0;
    cudaEvent_t  copy_event = nullptr;
    int          use_pdl = 0;
    int          trace = 0;
    uint64_t     n_launches = 0;           // kernels launched by graph_compute since creation
    std::string  name;

    LaunchCtx launch_ctx() const { return LaunchCtx{stream, dev->device, dev->sm_count, status_dev, use_pdl}; }
    void *    get_scratch(size_t bytes);   // grows (after a stream sync) when needed
};

// registry
std::vector<DeviceCtx *> & devices();
bool buffer_is_ours(ggml_backend_buffer_t buf);
bool buft_is_ours(ggml_backend_buffer_type_t buft);
bool buft_is_split(ggml_backend_buffer_type_t buft);
ggml_backend_buffer_type_t split_buffer_type(int main_device, const float * tensor_split);

// dispatch.cpp
bool             device_supports_op(DeviceCtx * dev, const ggml_tensor * op);
enum ggml_status graph_compute(BackendCtx * ctx, ggml_cgraph * cgraph);

}  // namespace b200
