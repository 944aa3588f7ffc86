// Row-split buffer type: the rows of a weight matrix are divided over the B200 devices of this process, each device
// holding its slice in its own memory.  What ggml_backend_cuda_split_buffer_type is to the reference
// (ggml/src/ggml-cuda/ggml-cuda.cu:714-742 row ranges, :789-835 per-device slices, :837-911 scatter and gather,
// :1000-1040 the buffer type keyed by main device and split); libllama asks for it by name in split-mode row
// (src/llama-model.cpp:304-326).  The MUL_MAT that consumes such a matrix is run_split_mul_mat in dispatch.cpp.
#include "backend.h"

#include <array>
#include <map>

namespace b200 {

// row boundaries are multiples of this (the reference rounds to its mat-mul tile height, 128 on every device newer
// than Pascal; here it is also the row count of one tensor-core tile)
static constexpr int64_t SPLIT_ROW_ROUNDING = 128;
// kernels read whole 16-byte runs around a row segment: every slice keeps this much slack after its last byte
static constexpr size_t SPLIT_TAIL_SLACK = 256;

struct SplitBuftCtx {
    int main_device;                                    // index in this backend's registry
    std::array<float, SPLIT_MAX_DEVICES> split;         // cumulative start fraction per device
    std::string name;
};
struct SplitBufferCtx {
    std::vector<SplitExtra *> extras;
    ~SplitBufferCtx() {
        for (SplitExtra * e : extras) {
            for (int id = 0; id < SPLIT_MAX_DEVICES; ++id) if (e->data[id]) {
                cudaSetDevice(devices()[(size_t) id]->device);
                cudaFree(e->data[id]);
            }
            delete e;
        }
    }
};

static void row_range(const SplitBuftCtx * bc, int64_t nrows, int id, int64_t * lo, int64_t * hi) {
    const int n = (int) devices().size();
    int64_t l = id == 0 ? 0 : (int64_t) ((float) nrows * bc->split[(size_t) id]);
    l -= l % SPLIT_ROW_ROUNDING;
    int64_t h = nrows;
    if (id != n - 1) { h = (int64_t) ((float) nrows * bc->split[(size_t) id + 1]); h -= h % SPLIT_ROW_ROUNDING; }
    *lo = l; *hi = h;
}
static size_t row_bytes(const ggml_tensor * t) { return (size_t) (t->ne[0] / t_blck(t->type)) * t_size(t->type); }

static void split_buffer_free(ggml_backend_buffer_t buffer) { delete (SplitBufferCtx *) buffer->context; }
static void * split_buffer_get_base(ggml_backend_buffer_t) { return (void *) 0x1000; }   // never dereferenced: slices hang off tensor->extra
static void split_buffer_init_tensor(ggml_backend_buffer_t buffer, ggml_tensor * tensor) {
    B200_ASSERT(tensor->view_src == nullptr);           // views of split tensors are not supported (nor by the reference)
    SplitBufferCtx * ctx = (SplitBufferCtx *) buffer->context;
    const SplitBuftCtx * bc = (const SplitBuftCtx *) buffer->buft->context;
    SplitExtra * e = new SplitExtra{};
    e->magic = SPLIT_EXTRA_MAGIC;
    ctx->extras.push_back(e);
    const int n = (int) devices().size();
    for (int id = 0; id < n; ++id) {
        row_range(bc, t_nrows(tensor), id, &e->row_low[id], &e->row_high[id]);
        const int64_t rows = e->row_high[id] - e->row_low[id];
        if (rows <= 0) continue;
        B200_CUDA_CHECK(cudaSetDevice(devices()[(size_t) id]->device));
        const size_t bytes = (size_t) rows * row_bytes(tensor);
        B200_CUDA_CHECK(cudaMalloc(&e->data[id], bytes + SPLIT_TAIL_SLACK));
        B200_CUDA_CHECK(cudaMemset((char *) e->data[id] + bytes, 0, SPLIT_TAIL_SLACK));
    }
    tensor->extra = e;
}
// split tensors are written and read whole (as in the reference)
static void split_buffer_set_tensor(ggml_backend_buffer_t, ggml_tensor * tensor, const void * data, size_t offset, size_t size) {
    B200_ASSERT(offset == 0 && size == t_nbytes(tensor));
    const SplitExtra * e = (const SplitExtra *) tensor->extra;
    const int n = (int) devices().size();
    for (int id = 0; id < n; ++id) {
        if (!e->data[id]) continue;
        B200_CUDA_CHECK(cudaSetDevice(devices()[(size_t) id]->device));
        B200_CUDA_CHECK(cudaMemcpyAsync(e->data[id], (const char *) data + (size_t) e->row_low[id] * tensor->nb[1],
                                        (size_t) (e->row_high[id] - e->row_low[id]) * row_bytes(tensor), cudaMemcpyHostToDevice, cudaStreamPerThread));
    }
    for (int id = 0; id < n; ++id) {
        if (!e->data[id]) continue;
        B200_CUDA_CHECK(cudaSetDevice(devices()[(size_t) id]->device));
        B200_CUDA_CHECK(cudaStreamSynchronize(cudaStreamPerThread));
    }
}
static void split_buffer_get_tensor(ggml_backend_buffer_t, const ggml_tensor * tensor, void * data, size_t offset, size_t size) {
    B200_ASSERT(offset == 0 && size == t_nbytes(tensor));
    const SplitExtra * e = (const SplitExtra *) tensor->extra;
    const int n = (int) devices().size();
    for (int id = 0; id < n; ++id) {
        if (!e->data[id]) continue;
        B200_CUDA_CHECK(cudaSetDevice(devices()[(size_t) id]->device));
        B200_CUDA_CHECK(cudaMemcpyAsync((char *) data + (size_t) e->row_low[id] * tensor->nb[1], e->data[id],
                                        (size_t) (e->row_high[id] - e->row_low[id]) * row_bytes(tensor), cudaMemcpyDeviceToHost, cudaStreamPerThread));
    }
    for (int id = 0; id < n; ++id) {
        if (!e->data[id]) continue;
        B200_CUDA_CHECK(cudaSetDevice(devices()[(size_t) id]->device));
        B200_CUDA_CHECK(cudaStreamSynchronize(cudaStreamPerThread));
    }
}
static void split_buffer_clear(ggml_backend_buffer_t, uint8_t) {}
static const ggml_backend_buffer_i k_split_buffer_iface = {
    /* free_buffer   */ split_buffer_free,
    /* get_base      */ split_buffer_get_base,
    /* init_tensor   */ split_buffer_init_tensor,
    /* memset_tensor */ nullptr,
    /* set_tensor    */ split_buffer_set_tensor,
    /* get_tensor    */ split_buffer_get_tensor,
    /* cpy_tensor    */ nullptr,
    /* clear         */ split_buffer_clear,
    /* reset         */ nullptr,
};

static const char * split_buft_get_name(ggml_backend_buffer_type_t buft) { return ((const SplitBuftCtx *) buft->context)->name.c_str(); }
bool buft_is_split(ggml_backend_buffer_type_t buft) { return buft && buft->iface.get_name == split_buft_get_name; }
const SplitExtra * split_extra_of(const ggml_tensor * t) {
    if (!t || !t->extra || !t->buffer || !buft_is_split(t->buffer->buft)) return nullptr;
    const SplitExtra * e = (const SplitExtra *) t->extra;
    return e->magic == SPLIT_EXTRA_MAGIC ? e : nullptr;
}
// Device memory is allocated per tensor in init_tensor (the split after rounding is not known before); `size` is the
// cumulative bound get_alloc_size promised, which the graph allocator enforces.
static ggml_backend_buffer_t split_buft_alloc_buffer(ggml_backend_buffer_type_t buft, size_t size) {
    ggml_backend_buffer_t b = new ggml_backend_buffer;          // freed with `delete` by ggml_backend_buffer_free
    b->iface = k_split_buffer_iface; b->buft = buft; b->context = new SplitBufferCtx; b->size = size;
    b->usage = GGML_BACKEND_BUFFER_USAGE_ANY;
    return b;
}
static size_t split_buft_get_alignment(ggml_backend_buffer_type_t) { return 128; }
static size_t split_buft_get_alloc_size(ggml_backend_buffer_type_t buft, const ggml_tensor * tensor) {
    const SplitBuftCtx * bc = (const SplitBuftCtx *) buft->context;
    size_t total = 0;
    for (int id = 0; id < (int) devices().size(); ++id) {
        int64_t lo, hi;
        row_range(bc, t_nrows(tensor), id, &lo, &hi);
        if (hi > lo) total += (size_t) (hi - lo) * row_bytes(tensor) + SPLIT_TAIL_SLACK;
    }
    return total;
}
static bool split_buft_is_host(ggml_backend_buffer_type_t) { return false; }
static const ggml_backend_buffer_type_i k_split_buft_iface = {
    /* get_name       */ split_buft_get_name,
    /* alloc_buffer   */ split_buft_alloc_buffer,
    /* get_alignment  */ split_buft_get_alignment,
    /* get_max_size   */ nullptr,
    /* get_alloc_size */ split_buft_get_alloc_size,
    /* is_host        */ split_buft_is_host,
};

// One buffer type per (main device, split).  `tensor_split` holds one proportion per device (as many entries as the
// registry has devices are read); all zero or null means equal shares.
ggml_backend_buffer_type_t split_buffer_type(int main_device, const float * tensor_split) {
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    static std::map<std::pair<int, std::array<float, SPLIT_MAX_DEVICES>>, ggml_backend_buffer_type> bufts;
    const int n = (int) devices().size();
    if (main_device < 0 || main_device >= n || n > SPLIT_MAX_DEVICES) return nullptr;
    std::array<float, SPLIT_MAX_DEVICES> arr = {};
    bool all_zero = true;
    if (tensor_split) for (int i = 0; i < n; ++i) if (tensor_split[i] != 0.0f) all_zero = false;
    float sum = 0.0f;
    for (int i = 0; i < n; ++i) { arr[(size_t) i] = sum; sum += all_zero ? 1.0f : tensor_split[i]; }
    if (!(sum > 0.0f)) return nullptr;
    for (int i = 0; i < n; ++i) arr[(size_t) i] /= sum;
    auto it = bufts.find({main_device, arr});
    if (it != bufts.end()) return &it->second;
    SplitBuftCtx * bc = new SplitBuftCtx{main_device, arr, devices()[(size_t) main_device]->name + "_Split"};
    ggml_backend_buffer_type buft = {k_split_buft_iface, &devices()[(size_t) main_device]->dev, bc};
    return &bufts.emplace(std::make_pair(main_device, arr), buft).first->second;
}

}  // namespace b200
