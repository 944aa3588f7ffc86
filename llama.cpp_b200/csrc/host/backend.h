// Internal declarations shared by the files of the B200 ggml backend host layer.
#pragma once

#include "ggml_compat.h"
#include "ggml-b200.h"

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

// row-split buffer type (split.cpp): what hangs off tensor->extra of a matrix stored in it
static constexpr int SPLIT_MAX_DEVICES = 16;
static constexpr uint32_t SPLIT_EXTRA_MAGIC = 0xb2005917u;
struct SplitExtra {
    uint32_t magic;
    void *   data[SPLIT_MAX_DEVICES];                   // the device's slice (registry index), null where it has no rows
    int64_t  row_low[SPLIT_MAX_DEVICES], row_high[SPLIT_MAX_DEVICES];
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
    int          use_fusion = 1;            // multi-node fusions (GGML_B200_FUSE=0 runs one node per launch group)
    int          use_tc = 1;                // tensor-core GEMM for N > 8 (GGML_B200_TC=0 falls back to the mat-vec kernel)
    int          trace = 0;
    uint64_t     n_launches = 0;           // kernels launched by graph_compute since creation
    std::string  name;

    // int8 activation blocks of recent MUL_MAT inputs, so that mat-muls sharing an input (wq/wk/wv,
    // gate/up) quantize it once and producers (rms_norm*w, silu*up) can emit it directly; valid only
    // within one graph_compute call
    struct ActEntry { const void * src_data = nullptr; int64_t K = 0, ncols = 0; void * q = nullptr; size_t cap = 0; size_t src_bytes = 0; };
    ActEntry     act_cache[2];
    int          act_next = 0;
    // F16 copy of the activations of the most recent tensor-core MUL_MAT (q/k/v and gate/up convert once)
    void *       tc_xh = nullptr; size_t tc_xh_cap = 0; const void * tc_x_data = nullptr; int64_t tc_x_k = 0, tc_x_n = 0; size_t tc_x_bytes = 0;
    void         act_cache_clear() { act_cache[0].src_data = act_cache[1].src_data = nullptr; tc_x_data = nullptr; }
    // a node that writes the bytes [data, data + bytes) makes conversions of anything overlapping them stale: an entry
    // is keyed by the start of its source, but a write into a view of that source (or a larger tensor the allocator
    // placed over it) starts elsewhere
    void         act_cache_invalidate(const void * data, size_t bytes) {
        const char * w0 = (const char *) data, * w1 = w0 + (bytes ? bytes : 1);
        for (ActEntry & e : act_cache) if (e.src_data && w0 < (const char *) e.src_data + e.src_bytes && (const char *) e.src_data < w1) e.src_data = nullptr;
        if (tc_x_data && w0 < (const char *) tc_x_data + tc_x_bytes && (const char *) tc_x_data < w1) tc_x_data = nullptr;
    }
    ActEntry *   act_cache_find(const void * src_data, int64_t K, int64_t ncols);
    ActEntry *   act_cache_take(const void * src_data, int64_t K, int64_t ncols);   // may allocate (never while capturing)

    // CUDA-graph replay of small-batch graphs.  Values that change every token without changing the
    // graph's shape (the byte offset of KV-cache stores) live in device memory (`dyn`), so a captured
    // graph stays valid from token to token.
    int          use_graphs = 1;
    bool         capturing = false, capture_failed = false;
    uint64_t     graph_key = 0, pending_key = 0;
    cudaGraphExec_t graph_exec = nullptr;
    uint64_t     graph_launches = 0;       // kernels inside the instantiated graph
    uint64_t     n_replay = 0, n_capture = 0, n_direct = 0;   // graph_compute calls by how they were executed
    int64_t *    dyn_host = nullptr, * dyn_dev = nullptr;
    int          dyn_used = 0;
    static constexpr int DYN_CAP = 1024;
    uint64_t     scratch_generation = 0;

    unsigned *   fa_tickets = nullptr;     // zero-initialised counters of the decode attention kernel
    // F16 copy of an F32 attention mask (graphs built without FLASH_ATTN_EXT carry it in F32), made once per graph_compute
    void *       mask16 = nullptr; size_t mask16_cap = 0; const void * mask16_src = nullptr;

    // persistent decode step (decode_plan.cpp): scratch, phase lists and barrier words of the single-launch path
    int          use_mega = 1;             // GGML_B200_MEGA=0 keeps one launch per node (group)
    int          mega_max_blocks = 1 << 30;   // GGML_B200_MEGA_MAX_BLOCKS: cut the persistent launch after this many blocks (debugging aid)
    int          mega_ops_used = 0;        // per graph_compute call: phases already placed in the arena's parameter region
    int          mega_timing = 0, mega_last_ops = 0;
    int          mega_keys_per_slice = 128; // GGML_B200_MEGA_KEYS: keys of the KV cache per attention work item
    int          mega_consumer_merge = 16;  // GGML_B200_MEGA_CMERGE: up to this many KV slices are merged by the next phase's input stage
    bool         mega_tried = false;       // per graph_compute call: a failed match is not retried at every node
    void *       mega_arena = nullptr;
    cudaStream_t mega_copy_stream = nullptr;
    uint64_t     n_mega = 0, graph_megas = 0;   // persistent launches so far; of them inside the instantiated CUDA graph

    // row-split over several processes: where the peers' arenas are mapped, and whether slices have been
    // stored to the peers since the last barrier
    ggml_b200_peers peers = {};
    bool         peer_pending = false;
    int          peer_spin_limit = 0;          // GGML_B200_PEER_SPIN_LIMIT: polls before the cross-GPU barrier gives up (0: default)
    std::vector<const void *> pending_full;   // full results whose slices are in flight to the peers
    std::vector<uint8_t> node_done;            // per graph node: already executed ahead of its position (hoisted into a grouped launch)
    const ggml_b200_row_slice * row_slice_of(const ggml_tensor * node) const {
        if (peers.n_ranks < 2 || node->op != GGML_OP_MUL_MAT || !node->extra) return nullptr;
        const ggml_b200_row_slice * rs = (const ggml_b200_row_slice *) node->extra;
        return rs->magic == GGML_B200_ROW_SLICE_MAGIC ? rs : nullptr;
    }

    // MUL_MAT on a matrix of the row-split buffer type: one helper instance (stream, scratch, status word) per other
    // device, the activations' copy and the result slice on that device, and the events that order the exchange
    struct SplitPeer { ggml_backend_t helper = nullptr; void * x = nullptr; size_t x_cap = 0; void * d = nullptr; size_t d_cap = 0; cudaEvent_t done = nullptr; };
    SplitPeer    split_peer[SPLIT_MAX_DEVICES];
    cudaEvent_t  split_ready = nullptr;        // recorded on this stream when the activations may be read
    bool         graph_has_split = false;      // per graph_compute call: such a graph is not captured into a CUDA graph

    LaunchCtx launch_ctx() const { return LaunchCtx{stream, dev->device, dev->sm_count, status_dev, use_pdl, fa_tickets}; }
    void *    get_scratch(size_t bytes);   // grows (after a stream sync) when needed
};

// registry
std::vector<DeviceCtx *> & devices();
bool buffer_is_ours(ggml_backend_buffer_t buf);
bool buft_is_ours(ggml_backend_buffer_type_t buft);
bool buft_is_split(ggml_backend_buffer_type_t buft);
ggml_backend_buffer_type_t split_buffer_type(int main_device, const float * tensor_split);
const SplitExtra * split_extra_of(const ggml_tensor * t);      // null unless t lives in a row-split buffer
ggml_backend_t   init_backend_for(DeviceCtx * d);              // a backend instance on device d (what dev_init_backend returns)
void             free_backend(ggml_backend_t backend);

// decode_plan.cpp
int              try_decode_step(BackendCtx * ctx, ggml_cgraph * g, int i);
void             decode_step_print_timing(BackendCtx * ctx);

// dispatch.cpp
bool             device_supports_op(DeviceCtx * dev, const ggml_tensor * op);
enum ggml_status graph_compute(BackendCtx * ctx, ggml_cgraph * cgraph);
bool             run_single_node(BackendCtx * ctx, ggml_cgraph * g, int i);   // executes node i alone (no fusion with its neighbours)

}  // namespace b200
