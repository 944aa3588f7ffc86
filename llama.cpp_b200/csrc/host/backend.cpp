// ggml backend plugin for NVIDIA B200 (sm_100a): registry, devices, buffer
// types, buffers, streams and events.  This file implements the vtables of
// ggml/src/ggml-backend-impl.h (buffer type :17-35, buffer :41-66, backend
// :87-124, device :137-179, reg :191-207) and exports ggml_backend_init /
// ggml_backend_score (:215-218) so that the reference's registry
// (ggml/src/ggml-backend-reg.cpp:133-256, GGML_BACKEND_PATH at :577-581) loads
// it as an out-of-tree device.  The behaviour mirrors what the reference's CUDA
// host layer does at the same boundary (ggml/src/ggml-cuda/ggml-cuda.cu:506-712
// buffers, :1042-1102 pinned host buffers, :2348-2401 async copies, :2869-3457
// device/reg), written from scratch around one stream per backend object.
#include "backend.h"

namespace b200 {

// ---------------------------------------------------------------------------
// registry state
// ---------------------------------------------------------------------------
std::vector<DeviceCtx *> & devices() {
    static std::vector<DeviceCtx *> devs;
    return devs;
}

static void set_device(int device) { B200_CUDA_CHECK(cudaSetDevice(device)); }

// ---------------------------------------------------------------------------
// device buffers
// ---------------------------------------------------------------------------
static void buffer_free(ggml_backend_buffer_t buffer) {
    BufferCtx * ctx = (BufferCtx *) buffer->context;
    set_device(ctx->device);
    cudaFree(ctx->base);
    delete ctx;
}
static void * buffer_get_base(ggml_backend_buffer_t buffer) { return ((BufferCtx *) buffer->context)->base; }

static void buffer_memset_tensor(ggml_backend_buffer_t buffer, ggml_tensor * tensor, uint8_t value, size_t offset, size_t size) {
    BufferCtx * ctx = (BufferCtx *) buffer->context;
    set_device(ctx->device);
    B200_CUDA_CHECK(cudaMemsetAsync((char *) tensor->data + offset, value, size, cudaStreamPerThread));
    B200_CUDA_CHECK(cudaStreamSynchronize(cudaStreamPerThread));
}
static void buffer_set_tensor(ggml_backend_buffer_t buffer, ggml_tensor * tensor, const void * data, size_t offset, size_t size) {
    BufferCtx * ctx = (BufferCtx *) buffer->context;
    set_device(ctx->device);
    B200_CUDA_CHECK(cudaMemcpyAsync((char *) tensor->data + offset, data, size, cudaMemcpyHostToDevice, cudaStreamPerThread));
    B200_CUDA_CHECK(cudaStreamSynchronize(cudaStreamPerThread));
}
static void buffer_get_tensor(ggml_backend_buffer_t buffer, const ggml_tensor * tensor, void * data, size_t offset, size_t size) {
    BufferCtx * ctx = (BufferCtx *) buffer->context;
    set_device(ctx->device);
    B200_CUDA_CHECK(cudaMemcpyAsync(data, (const char *) tensor->data + offset, size, cudaMemcpyDeviceToHost, cudaStreamPerThread));
    B200_CUDA_CHECK(cudaStreamSynchronize(cudaStreamPerThread));
}
static bool buffer_cpy_tensor(ggml_backend_buffer_t buffer, const ggml_tensor * src, ggml_tensor * dst) {
    ggml_backend_buffer_t sbuf = src->view_src ? src->view_src->buffer : src->buffer;
    if (!buffer_is_ours(sbuf)) return false;
    BufferCtx * sctx = (BufferCtx *) sbuf->context;
    BufferCtx * dctx = (BufferCtx *) buffer->context;
    const size_t n = t_nbytes(src);
    set_device(dctx->device);
    if (sctx->device == dctx->device) {
        B200_CUDA_CHECK(cudaMemcpyAsync(dst->data, src->data, n, cudaMemcpyDeviceToDevice, cudaStreamPerThread));
    } else {
        B200_CUDA_CHECK(cudaMemcpyPeerAsync(dst->data, dctx->device, src->data, sctx->device, n, cudaStreamPerThread));
    }
    B200_CUDA_CHECK(cudaStreamSynchronize(cudaStreamPerThread));
    return true;
}
static void buffer_clear(ggml_backend_buffer_t buffer, uint8_t value) {
    BufferCtx * ctx = (BufferCtx *) buffer->context;
    set_device(ctx->device);
    B200_CUDA_CHECK(cudaDeviceSynchronize());
    B200_CUDA_CHECK(cudaMemset(ctx->base, value, ctx->size));
    B200_CUDA_CHECK(cudaDeviceSynchronize());
}

static const ggml_backend_buffer_i k_buffer_iface = {
    /* free_buffer   */ buffer_free,
    /* get_base      */ buffer_get_base,
    /* init_tensor   */ nullptr,
    /* memset_tensor */ buffer_memset_tensor,
    /* set_tensor    */ buffer_set_tensor,
    /* get_tensor    */ buffer_get_tensor,
    /* cpy_tensor    */ buffer_cpy_tensor,
    /* clear         */ buffer_clear,
    /* reset         */ nullptr,
};

bool buffer_is_ours(ggml_backend_buffer_t buf) { return buf && buf->iface.free_buffer == buffer_free; }

// The host application frees buffers with `delete` (ggml_backend_buffer_free,
// ggml/src/ggml-backend.cpp:99-111), so the object is created with `new` here,
// field for field what ggml_backend_buffer_init does (:84-97).
static ggml_backend_buffer_t make_buffer(ggml_backend_buffer_type_t buft, const ggml_backend_buffer_i & iface, void * ctx, size_t size) {
    ggml_backend_buffer_t b = new ggml_backend_buffer;
    b->iface = iface; b->buft = buft; b->context = ctx; b->size = size;
    b->usage = GGML_BACKEND_BUFFER_USAGE_ANY;
    return b;
}

// ---------------------------------------------------------------------------
// device buffer type
// ---------------------------------------------------------------------------
static const char * buft_get_name(ggml_backend_buffer_type_t buft) { return ((DeviceCtx *) buft->context)->name.c_str(); }

// kernels stream weight rows with 16-byte bulk copies from the aligned superset
// of each row segment, so every buffer keeps this much slack after its last byte
static constexpr size_t BUFFER_TAIL_SLACK = 256;

static ggml_backend_buffer_t buft_alloc_buffer(ggml_backend_buffer_type_t buft, size_t size) {
    DeviceCtx * dev = (DeviceCtx *) buft->context;
    set_device(dev->device);
    void * base = nullptr;
    cudaError_t err = cudaMalloc(&base, (size ? size : 1) + BUFFER_TAIL_SLACK);
    if (err != cudaSuccess) {
        cudaGetLastError();   // clear the sticky-free allocation error; the caller handles NULL
        B200_LOG_ERROR("%s: allocating %.2f MiB on device %d: cudaMalloc failed: %s\n", __func__, size / 1024.0 / 1024.0,
                       dev->device, cudaGetErrorString(err));
        return nullptr;
    }
    return make_buffer(buft, k_buffer_iface, new BufferCtx{dev->device, base, size}, size);
}
static size_t buft_get_alignment(ggml_backend_buffer_type_t) { return 128; }
static size_t buft_get_alloc_size(ggml_backend_buffer_type_t, const ggml_tensor * tensor) { return t_nbytes(tensor); }

static const ggml_backend_buffer_type_i k_buft_iface = {
    /* get_name       */ buft_get_name,
    /* alloc_buffer   */ buft_alloc_buffer,
    /* get_alignment  */ buft_get_alignment,
    /* get_max_size   */ nullptr,
    /* get_alloc_size */ buft_get_alloc_size,
    /* is_host        */ nullptr,
};
bool buft_is_ours(ggml_backend_buffer_type_t buft) { return buft && buft->iface.get_name == buft_get_name; }

// ---------------------------------------------------------------------------
// pinned host buffer type (staging for host<->device copies; CPU ops can use it)
// ---------------------------------------------------------------------------
static const char * host_buft_get_name(ggml_backend_buffer_type_t) { return "B200_Host"; }
static void host_buffer_free(ggml_backend_buffer_t buffer) { cudaFreeHost(buffer->context); }
static void * host_buffer_get_base(ggml_backend_buffer_t buffer) { return buffer->context; }
static void host_buffer_memset_tensor(ggml_backend_buffer_t, ggml_tensor * t, uint8_t v, size_t off, size_t size) { memset((char *) t->data + off, v, size); }
static void host_buffer_set_tensor(ggml_backend_buffer_t, ggml_tensor * t, const void * data, size_t off, size_t size) { memcpy((char *) t->data + off, data, size); }
static void host_buffer_get_tensor(ggml_backend_buffer_t, const ggml_tensor * t, void * data, size_t off, size_t size) { memcpy(data, (const char *) t->data + off, size); }
static bool host_buffer_cpy_tensor(ggml_backend_buffer_t, const ggml_tensor * src, ggml_tensor * dst) {
    ggml_backend_buffer_t sbuf = src->view_src ? src->view_src->buffer : src->buffer;
    if (sbuf && sbuf->buft && sbuf->buft->iface.is_host && sbuf->buft->iface.is_host(sbuf->buft)) {
        memcpy(dst->data, src->data, t_nbytes(src));
        return true;
    }
    return false;
}
static void host_buffer_clear(ggml_backend_buffer_t buffer, uint8_t value) { memset(buffer->context, value, buffer->size); }
static const ggml_backend_buffer_i k_host_buffer_iface = {
    host_buffer_free, host_buffer_get_base, nullptr, host_buffer_memset_tensor, host_buffer_set_tensor,
    host_buffer_get_tensor, host_buffer_cpy_tensor, host_buffer_clear, nullptr,
};
static ggml_backend_buffer_t host_buft_alloc_buffer(ggml_backend_buffer_type_t buft, size_t size) {
    void * ptr = nullptr;
    cudaError_t err = cudaMallocHost(&ptr, size ? size : 1);
    if (err != cudaSuccess) {
        cudaGetLastError();
        B200_LOG_WARN("%s: failed to allocate %.2f MiB of pinned memory: %s\n", __func__, size / 1024.0 / 1024.0, cudaGetErrorString(err));
        return nullptr;
    }
    return make_buffer(buft, k_host_buffer_iface, ptr, size);
}
static size_t host_buft_get_alignment(ggml_backend_buffer_type_t) { return 64; }
static bool   host_buft_is_host(ggml_backend_buffer_type_t) { return true; }
static const ggml_backend_buffer_type_i k_host_buft_iface = {
    host_buft_get_name, host_buft_alloc_buffer, host_buft_get_alignment, nullptr, nullptr, host_buft_is_host,
};

// ---------------------------------------------------------------------------
// backend (stream)
// ---------------------------------------------------------------------------
static uint8_t k_guid[16] = {0xb2, 0x00, 0x5a, 0x10, 0x0a, 0x9e, 0x41, 0x7c, 0x8d, 0x13, 0x67, 0x2f, 0xc4, 0x55, 0x90, 0xee};

BackendCtx::ActEntry * BackendCtx::act_cache_find(const void * src_data, int64_t K, int64_t ncols) {
    for (ActEntry & e : act_cache) if (e.src_data == src_data && e.K == K && e.ncols == ncols) return &e;
    return nullptr;
}
BackendCtx::ActEntry * BackendCtx::act_cache_take(const void * src_data, int64_t K, int64_t ncols) {
    act_cache_invalidate(src_data, (size_t) K * (size_t) ncols * 4);
    ActEntry & e = act_cache[act_next];
    act_next ^= 1;
    const size_t need = act128_bytes(K, ncols);
    if (need > e.cap) {
        if (capturing) { capture_failed = true; return nullptr; }
        B200_CUDA_CHECK(cudaStreamSynchronize(stream));
        if (e.q) B200_CUDA_CHECK(cudaFree(e.q));
        size_t cap = e.cap ? e.cap : (size_t) 1 << 20;
        while (cap < need) cap *= 2;
        B200_CUDA_CHECK(cudaMalloc(&e.q, cap));
        e.cap = cap;
        scratch_generation++;
    }
    e.src_data = src_data; e.K = K; e.ncols = ncols; e.src_bytes = (size_t) K * (size_t) ncols * 4;
    return &e;
}

void * BackendCtx::get_scratch(size_t bytes) {
    if (bytes <= scratch_size) return scratch;
    if (capturing) { capture_failed = true; return scratch; }
    scratch_generation++;
    B200_CUDA_CHECK(cudaStreamSynchronize(stream));
    if (scratch) B200_CUDA_CHECK(cudaFree(scratch));
    size_t cap = scratch_size ? scratch_size : (size_t) 8 << 20;
    while (cap < bytes) cap *= 2;
    B200_CUDA_CHECK(cudaMalloc(&scratch, cap));
    scratch_size = cap;
    return scratch;
}

static const char * backend_get_name(ggml_backend_t backend) { return ((BackendCtx *) backend->context)->name.c_str(); }
static bool backend_is_ours(ggml_backend_t backend) { return backend && backend->iface.get_name == backend_get_name; }

static void backend_free(ggml_backend_t backend) {
    BackendCtx * ctx = (BackendCtx *) backend->context;
    for (BackendCtx::SplitPeer & sp : ctx->split_peer) {            // helper instances on the other devices (row-split mat-muls)
        if (!sp.helper) continue;
        BackendCtx * h = (BackendCtx *) sp.helper->context;
        set_device(h->dev->device);
        cudaStreamSynchronize(h->stream);
        if (sp.x) cudaFree(sp.x);
        if (sp.d) cudaFree(sp.d);
        if (sp.done) cudaEventDestroy(sp.done);
        backend_free(sp.helper);
    }
    set_device(ctx->dev->device);
    cudaStreamSynchronize(ctx->stream);
    if (ctx->split_ready) cudaEventDestroy(ctx->split_ready);
    if (getenv("GGML_B200_VERBOSE"))
        fprintf(stderr, "ggml-b200: %s: graph_compute calls: %llu replayed from a CUDA graph, %llu captured, %llu run directly; %llu kernel launches, %llu of them persistent decode steps\n",
                ctx->name.c_str(), (unsigned long long) ctx->n_replay, (unsigned long long) ctx->n_capture, (unsigned long long) ctx->n_direct,
                (unsigned long long) ctx->n_launches, (unsigned long long) ctx->n_mega);
    decode_step_print_timing(ctx);
    if (ctx->scratch) cudaFree(ctx->scratch);
    if (ctx->tc_xh) cudaFree(ctx->tc_xh);
    for (auto & e : ctx->act_cache) if (e.q) cudaFree(e.q);
    if (ctx->graph_exec) cudaGraphExecDestroy(ctx->graph_exec);
    if (ctx->dyn_dev) cudaFree(ctx->dyn_dev);
    if (ctx->fa_tickets) cudaFree(ctx->fa_tickets);
    if (ctx->mask16) cudaFree(ctx->mask16);
    if (ctx->mega_arena) cudaFree(ctx->mega_arena);
    if (ctx->mega_copy_stream) cudaStreamDestroy(ctx->mega_copy_stream);
    free(ctx->dyn_host);
    if (ctx->status_dev) cudaFree(ctx->status_dev);
    if (ctx->status_host) cudaFreeHost(ctx->status_host);
    if (ctx->copy_event) cudaEventDestroy(ctx->copy_event);
    cudaStreamDestroy(ctx->stream);
    delete ctx;
    delete backend;
}
static void backend_set_tensor_async(ggml_backend_t backend, ggml_tensor * tensor, const void * data, size_t offset, size_t size) {
    BackendCtx * ctx = (BackendCtx *) backend->context;
    set_device(ctx->dev->device);
    B200_CUDA_CHECK(cudaMemcpyAsync((char *) tensor->data + offset, data, size, cudaMemcpyHostToDevice, ctx->stream));
}
static void backend_get_tensor_async(ggml_backend_t backend, const ggml_tensor * tensor, void * data, size_t offset, size_t size) {
    BackendCtx * ctx = (BackendCtx *) backend->context;
    set_device(ctx->dev->device);
    B200_CUDA_CHECK(cudaMemcpyAsync(data, (const char *) tensor->data + offset, size, cudaMemcpyDeviceToHost, ctx->stream));
}
static bool backend_cpy_tensor_async(ggml_backend_t bsrc, ggml_backend_t bdst, const ggml_tensor * src, ggml_tensor * dst) {
    if (!backend_is_ours(bsrc) || !backend_is_ours(bdst)) return false;
    ggml_backend_buffer_t sbuf = src->view_src ? src->view_src->buffer : src->buffer;
    ggml_backend_buffer_t dbuf = dst->view_src ? dst->view_src->buffer : dst->buffer;
    if (!buffer_is_ours(sbuf) || !buffer_is_ours(dbuf)) return false;
    BackendCtx * cs = (BackendCtx *) bsrc->context;
    BackendCtx * cd = (BackendCtx *) bdst->context;
    BufferCtx * bs = (BufferCtx *) sbuf->context;
    BufferCtx * bd = (BufferCtx *) dbuf->context;
    if (cs->dev->device != bs->device || cd->dev->device != bd->device) return false;
    const size_t n = t_nbytes(dst);
    if (bsrc == bdst) {
        set_device(cs->dev->device);
        B200_CUDA_CHECK(cudaMemcpyAsync(dst->data, src->data, n, cudaMemcpyDeviceToDevice, cs->stream));
        return true;
    }
    // copy on the source stream, then make the destination stream wait for it
    set_device(cs->dev->device);
    if (cs->dev->device == cd->dev->device) B200_CUDA_CHECK(cudaMemcpyAsync(dst->data, src->data, n, cudaMemcpyDeviceToDevice, cs->stream));
    else B200_CUDA_CHECK(cudaMemcpyPeerAsync(dst->data, cd->dev->device, src->data, cs->dev->device, n, cs->stream));
    if (!cs->copy_event) B200_CUDA_CHECK(cudaEventCreateWithFlags(&cs->copy_event, cudaEventDisableTiming));
    B200_CUDA_CHECK(cudaEventRecord(cs->copy_event, cs->stream));
    set_device(cd->dev->device);
    B200_CUDA_CHECK(cudaStreamWaitEvent(cd->stream, cs->copy_event, 0));
    return true;
}
static void backend_synchronize(ggml_backend_t backend) {
    BackendCtx * ctx = (BackendCtx *) backend->context;
    set_device(ctx->dev->device);
    B200_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
}
static enum ggml_status backend_graph_compute(ggml_backend_t backend, ggml_cgraph * cgraph) {
    BackendCtx * ctx = (BackendCtx *) backend->context;
    set_device(ctx->dev->device);
    return graph_compute(ctx, cgraph);
}
static void backend_event_record(ggml_backend_t backend, ggml_backend_event_t event) {
    BackendCtx * ctx = (BackendCtx *) backend->context;
    set_device(ctx->dev->device);
    B200_CUDA_CHECK(cudaEventRecord((cudaEvent_t) event->context, ctx->stream));
}
static void backend_event_wait(ggml_backend_t backend, ggml_backend_event_t event) {
    BackendCtx * ctx = (BackendCtx *) backend->context;
    set_device(ctx->dev->device);
    B200_CUDA_CHECK(cudaStreamWaitEvent(ctx->stream, (cudaEvent_t) event->context, 0));
}
static const ggml_backend_i k_backend_iface = {
    /* get_name           */ backend_get_name,
    /* free               */ backend_free,
    /* set_tensor_async   */ backend_set_tensor_async,
    /* get_tensor_async   */ backend_get_tensor_async,
    /* cpy_tensor_async   */ backend_cpy_tensor_async,
    /* synchronize        */ backend_synchronize,
    /* graph_plan_create  */ nullptr,
    /* graph_plan_free    */ nullptr,
    /* graph_plan_update  */ nullptr,
    /* graph_plan_compute */ nullptr,
    /* graph_compute      */ backend_graph_compute,
    /* event_record       */ backend_event_record,
    /* event_wait         */ backend_event_wait,
};

// ---------------------------------------------------------------------------
// device
// ---------------------------------------------------------------------------
static const char * dev_get_name(ggml_backend_dev_t dev) { return ((DeviceCtx *) dev->context)->name.c_str(); }
static const char * dev_get_description(ggml_backend_dev_t dev) { return ((DeviceCtx *) dev->context)->description.c_str(); }
static void dev_get_memory(ggml_backend_dev_t dev, size_t * free, size_t * total) {
    set_device(((DeviceCtx *) dev->context)->device);
    B200_CUDA_CHECK(cudaMemGetInfo(free, total));
}
static enum ggml_backend_dev_type dev_get_type(ggml_backend_dev_t) { return GGML_BACKEND_DEVICE_TYPE_GPU; }
static ggml_backend_buffer_type_t dev_get_buffer_type(ggml_backend_dev_t dev) { return &((DeviceCtx *) dev->context)->buft; }
static ggml_backend_buffer_type_t dev_get_host_buffer_type(ggml_backend_dev_t dev) { return &((DeviceCtx *) dev->context)->host_buft; }
static void dev_get_props(ggml_backend_dev_t dev, ggml_backend_dev_props * props) {
    props->name = dev_get_name(dev);
    props->description = dev_get_description(dev);
    props->type = dev_get_type(dev);
    dev_get_memory(dev, &props->memory_free, &props->memory_total);
    props->caps.async = true;
    props->caps.host_buffer = getenv("GGML_B200_NO_PINNED") == nullptr;
    props->caps.buffer_from_host_ptr = false;
    props->caps.events = true;
}
void free_backend(ggml_backend_t backend) { backend_free(backend); }
ggml_backend_t init_backend_for(DeviceCtx * d) { return d->dev.iface.init_backend(&d->dev, nullptr); }
static ggml_backend_t dev_init_backend(ggml_backend_dev_t dev, const char * /*params*/) {
    DeviceCtx * d = (DeviceCtx *) dev->context;
    set_device(d->device);
    BackendCtx * ctx = new BackendCtx;
    ctx->dev = d;
    ctx->name = d->name;
    if (cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess) { cudaGetLastError(); delete ctx; return nullptr; }
    B200_CUDA_CHECK(cudaMalloc((void **) &ctx->status_dev, sizeof(int)));
    B200_CUDA_CHECK(cudaMemset(ctx->status_dev, 0, sizeof(int)));
    B200_CUDA_CHECK(cudaMallocHost((void **) &ctx->status_host, sizeof(int)));
    *ctx->status_host = 0;
    B200_CUDA_CHECK(cudaMalloc((void **) &ctx->fa_tickets, sizeof(unsigned) * FATTN_DEC_TICKETS));
    B200_CUDA_CHECK(cudaMemset(ctx->fa_tickets, 0, sizeof(unsigned) * FATTN_DEC_TICKETS));
    B200_CUDA_CHECK(cudaMalloc((void **) &ctx->dyn_dev, sizeof(int64_t) * BackendCtx::DYN_CAP));
    // pageable on purpose: cudaMemcpyAsync then snapshots the values at call time, so the next call may overwrite them
    ctx->dyn_host = (int64_t *) malloc(sizeof(int64_t) * BackendCtx::DYN_CAP);
    ctx->use_graphs = getenv("GGML_B200_GRAPHS") ? atoi(getenv("GGML_B200_GRAPHS")) : 1;
    ctx->use_fusion = getenv("GGML_B200_FUSE") ? atoi(getenv("GGML_B200_FUSE")) : 1;
    ctx->use_tc = getenv("GGML_B200_TC") ? atoi(getenv("GGML_B200_TC")) : 1;
    ctx->use_mega = getenv("GGML_B200_MEGA") ? atoi(getenv("GGML_B200_MEGA")) : 1;
    if (getenv("GGML_B200_MEGA_MAX_BLOCKS")) ctx->mega_max_blocks = atoi(getenv("GGML_B200_MEGA_MAX_BLOCKS"));
    if (ctx->mega_max_blocks < 1) ctx->mega_max_blocks = 1;
    if (getenv("GGML_B200_MEGA_KEYS")) ctx->mega_keys_per_slice = atoi(getenv("GGML_B200_MEGA_KEYS"));
    if (ctx->mega_keys_per_slice < 16) ctx->mega_keys_per_slice = 16;
    if (getenv("GGML_B200_MEGA_CMERGE")) ctx->mega_consumer_merge = atoi(getenv("GGML_B200_MEGA_CMERGE"));
    if (getenv("GGML_B200_PEER_SPIN_LIMIT")) ctx->peer_spin_limit = atoi(getenv("GGML_B200_PEER_SPIN_LIMIT"));
    ctx->mega_timing = getenv("GGML_B200_MEGA_TIMING") ? atoi(getenv("GGML_B200_MEGA_TIMING")) : 0;
    const char * pdl = getenv("GGML_B200_PDL");
    ctx->use_pdl = pdl ? atoi(pdl) : 1;
    ctx->trace = getenv("GGML_B200_TRACE") ? atoi(getenv("GGML_B200_TRACE")) : 0;
    ggml_backend_t backend = new ggml_backend;
    backend->guid = &k_guid;
    backend->iface = k_backend_iface;
    backend->device = dev;
    backend->context = ctx;
    return backend;
}
static bool dev_supports_op(ggml_backend_dev_t dev, const ggml_tensor * op) { return device_supports_op((DeviceCtx *) dev->context, op); }
static bool dev_supports_buft(ggml_backend_dev_t dev, ggml_backend_buffer_type_t buft) {
    if (buft_is_split(buft)) return buft->device == dev;        // a split matrix is consumed by the backend of its main device
    return buft_is_ours(buft) && buft->context == dev->context;
}
static bool dev_offload_op(ggml_backend_dev_t, const ggml_tensor * op) {
    // large batches are worth the host->device weight copy (same policy as ggml-cuda.cu:3236-3242)
    const int min_batch = 32;
    return (op->ne[1] >= min_batch && op->op != GGML_OP_GET_ROWS) || (op->ne[2] >= min_batch && op->op == GGML_OP_MUL_MAT_ID);
}
static ggml_backend_event_t dev_event_new(ggml_backend_dev_t dev) {
    set_device(((DeviceCtx *) dev->context)->device);
    cudaEvent_t ev;
    B200_CUDA_CHECK(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    return new ggml_backend_event{dev, ev};
}
static void dev_event_free(ggml_backend_dev_t, ggml_backend_event_t event) {
    cudaEventDestroy((cudaEvent_t) event->context);
    delete event;
}
static void dev_event_synchronize(ggml_backend_dev_t, ggml_backend_event_t event) {
    B200_CUDA_CHECK(cudaEventSynchronize((cudaEvent_t) event->context));
}
static const ggml_backend_device_i k_device_iface = {
    dev_get_name, dev_get_description, dev_get_memory, dev_get_type, dev_get_props, dev_init_backend,
    dev_get_buffer_type, dev_get_host_buffer_type, /* buffer_from_host_ptr */ nullptr,
    dev_supports_op, dev_supports_buft, dev_offload_op, dev_event_new, dev_event_free, dev_event_synchronize,
};

// ---------------------------------------------------------------------------
// registry
// ---------------------------------------------------------------------------
static const char * reg_get_name(ggml_backend_reg_t) { return "B200"; }
static size_t reg_get_device_count(ggml_backend_reg_t) { return devices().size(); }
static ggml_backend_dev_t reg_get_device(ggml_backend_reg_t, size_t index) {
    B200_ASSERT(index < devices().size());
    return &devices()[index]->dev;
}

static ggml_backend_feature * get_features(ggml_backend_reg_t) {
    static ggml_backend_feature features[] = {
        {"ARCH", "sm_100a"}, {"MMVQ", "bulk-copy+dp4a"}, {"MMQ", "tcgen05"}, {"FA", "split-kv"}, {nullptr, nullptr},
    };
    return features;
}
// extra entry points reachable through get_proc_address (documented in include/ggml-b200.h)
static void * b200_get_stream(ggml_backend_t backend) { return backend_is_ours(backend) ? (void *) ((BackendCtx *) backend->context)->stream : nullptr; }
static uint64_t b200_get_launch_count(ggml_backend_t backend) { return backend_is_ours(backend) ? ((BackendCtx *) backend->context)->n_launches : 0; }
static int b200_get_status(ggml_backend_t backend) {
    if (!backend_is_ours(backend)) return -1;
    BackendCtx * ctx = (BackendCtx *) backend->context;
    set_device(ctx->dev->device);
    B200_CUDA_CHECK(cudaMemcpyAsync(ctx->status_host, ctx->status_dev, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
    B200_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
    return *ctx->status_host;
}

static int b200_set_peers(ggml_backend_t backend, const ggml_b200_peers * peers) {
    if (!backend_is_ours(backend) || !peers) return -1;
    BackendCtx * ctx = (BackendCtx *) backend->context;
    if (peers->n_ranks < 1 || peers->n_ranks > GGML_B200_MAX_PEERS || peers->rank < 0 || peers->rank >= peers->n_ranks) return -2;
    for (int r = 0; r < peers->n_ranks; ++r) if (!peers->arena[r] || ((uintptr_t) peers->arena[r] & 255)) return -3;
    if (peers->arena_bytes < GGML_B200_PEER_FLAG_BYTES) return -4;
    ctx->peers = *peers;
    ctx->peer_pending = false;
    if (ctx->graph_exec) { cudaGraphExecDestroy(ctx->graph_exec); ctx->graph_exec = nullptr; ctx->graph_key = 0; }
    ctx->pending_key = 0;
    return 0;
}

static void * reg_get_proc_address(ggml_backend_reg_t, const char * name) {
    if (strcmp(name, "ggml_backend_b200_set_peers") == 0) return (void *) b200_set_peers;
    if (strcmp(name, "ggml_backend_split_buffer_type") == 0) return (void *) split_buffer_type;
    if (strcmp(name, "ggml_backend_get_features") == 0) return (void *) get_features;
    if (strcmp(name, "ggml_backend_b200_get_stream") == 0) return (void *) b200_get_stream;
    if (strcmp(name, "ggml_backend_b200_get_launch_count") == 0) return (void *) b200_get_launch_count;
    if (strcmp(name, "ggml_backend_b200_get_status") == 0) return (void *) b200_get_status;
    return nullptr;
}
static const ggml_backend_reg_i k_reg_iface = {reg_get_name, reg_get_device_count, reg_get_device, reg_get_proc_address};

static int count_b200_devices(std::vector<int> * ordinals) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) { cudaGetLastError(); return 0; }
    int found = 0;
    for (int i = 0; i < n; ++i) {
        int major = 0;
        if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, i) != cudaSuccess) { cudaGetLastError(); continue; }
        if (major == 10) { ++found; if (ordinals) ordinals->push_back(i); }
    }
    return found;
}

static ggml_backend_reg * make_registry() {
    static ggml_backend_reg reg;
    std::vector<int> ordinals;
    count_b200_devices(&ordinals);
    for (size_t i = 0; i < ordinals.size(); ++i) {
        DeviceCtx * d = new DeviceCtx;
        d->device = ordinals[i];
        d->index = (int) i;
        cudaDeviceProp prop;
        B200_CUDA_CHECK(cudaGetDeviceProperties(&prop, d->device));
        d->sm_count = prop.multiProcessorCount;
        d->l2_bytes = (size_t) prop.l2CacheSize;
        d->name = "B200_" + std::to_string(i);
        d->description = prop.name;
        d->dev = ggml_backend_device{k_device_iface, &reg, d};
        d->buft = ggml_backend_buffer_type{k_buft_iface, &d->dev, d};
        d->host_buft = ggml_backend_buffer_type{k_host_buft_iface, &d->dev, d};
        devices().push_back(d);
    }
    reg.api_version = GGML_BACKEND_API_VERSION;
    reg.iface = k_reg_iface;
    reg.context = nullptr;
    return &reg;
}

}  // namespace b200

extern "C" {
__attribute__((visibility("default"))) ggml_backend_reg_t ggml_backend_init(void) {
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    static ggml_backend_reg * reg = b200::make_registry();
    return reg;
}
__attribute__((visibility("default"))) int ggml_backend_score(void) {
    return b200::count_b200_devices(nullptr) > 0 ? 100 : 0;
}
}
