// Llama-architecture graph driver over the ggml backend C-ABI (include/b200_llama.h).
//
// Builds, by hand, the same cgraph that libllama's llm_build_context::build_llama
// emits with flash attention on (src/llama.cpp:1476-1640; KV store :157-199;
// attention :540-662; FFN :349-395), using struct ggml_tensor / ggml_cgraph
// directly: every constructor below sets the fields the corresponding ggml.c
// constructor sets (ggml_mul_mat ggml/src/ggml.c:2694, ggml_rms_norm :2609,
// ggml_rope_ext :3528, ggml_cpy :3159, ggml_flash_attn_ext :4306, ggml_get_rows
// :3340, views/reshape/permute :3050-3330).  No ggml library is linked; the
// graph is executed through the function tables of whatever backend registry is
// passed in.
#include "backend.h"
#include "ggml-impl.h"
#include "b200_llama.h"
#include "gguf_load.h"

#include <chrono>
#include <cmath>
#include <atomic>
#include <map>
#include <memory>
#include <thread>

extern "C" ggml_backend_reg_t ggml_backend_init(void);

namespace {

using namespace b200;

thread_local std::string g_error;

// a weight tensor as this rank stores it: all of it, or (row-split) the rows [row_low, row_low + t.ne[1]) of full_rows
struct Weight { std::string name; ggml_tensor t; size_t offset; int64_t full_rows, row_low; bool split; };

constexpr size_t ALIGN = 128;
inline size_t align_up(size_t x) { return (x + ALIGN - 1) & ~(ALIGN - 1); }

// bump allocator over a region of a backend buffer
struct Region {
    char * base = nullptr; size_t cap = 0, used = 0, peak = 0;
    void * take(size_t n) { used = align_up(used); void * p = base ? base + used : nullptr; used += n; if (used > peak) peak = used; return p; }
    void reset() { used = 0; }
};

}  // namespace

struct b200_llama {
    b200_llama_config cfg;
    int head_dim = 0, n_embd_kv = 0;
    ggml_backend_reg_t reg = nullptr;
    ggml_backend_dev_t dev = nullptr;
    ggml_backend_t backend = nullptr;
    ggml_backend_buffer_type_t buft = nullptr;
    ggml_backend_buffer_t buf_w = nullptr, buf_kv = nullptr, buf_c = nullptr;
    bool is_b200 = false;
    cudaStream_t stream = nullptr;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    uint64_t (*launch_count_fn)(ggml_backend_t) = nullptr;

    int n_ranks = 1, rank = 0;                         // row-split over processes (one per GPU)
    std::vector<ggml_b200_row_slice> slices; size_t slices_used = 0;   // node->extra of sliced MUL_MATs
    void * peer_arena[GGML_B200_MAX_PEERS] = {};       // peers' compute buffers mapped here (CUDA IPC)
    int (*status_fn)(ggml_backend_t) = nullptr;

    std::vector<Weight> weights;                       // fixed order, see add_weights()
    std::vector<ggml_tensor> k_l, v_l;                 // per-layer KV cache tensors (F16, 1-D)

    // graph storage, rebuilt per decode
    std::vector<ggml_tensor> pool; size_t pool_used = 0;
    std::vector<ggml_tensor *> nodes;
    ggml_cgraph graph = {};
    Region rg_global, rg_layer[2];
    Region * cur_region = nullptr;
    bool dry = false;

    // inputs / outputs of the current graph
    ggml_tensor * inp_tokens = nullptr, * inp_pos = nullptr, * inp_mask = nullptr, * inp_out_ids = nullptr, * logits = nullptr;
    // host staging of the per-call inputs and of the logits: page-locked on the B200 backend, so the copies
    // inside b200_llama_decode are true asynchronous DMA transfers
    float * mask_host = nullptr; int32_t * pos_host = nullptr, * tok_host = nullptr; float * logits_stage = nullptr;
    size_t mask_cap = 0;
    bool host_pinned = false;
    void host_free(void * q) { if (!q) return; if (host_pinned) cudaFreeHost(q); else free(q); }

    int last_n_nodes = 0; double last_ms = 0.0; size_t weight_bytes = 0, arena_bytes = 0;

    // ---- tensor constructors ----
    ggml_tensor * raw() {
        B200_ASSERT(pool_used < pool.size());
        ggml_tensor * t = &pool[pool_used++];
        memset(t, 0, sizeof(*t));
        return t;
    }
    static void set_contig(ggml_tensor * t, ggml_type type, int64_t n0, int64_t n1, int64_t n2, int64_t n3) {
        t->type = type; t->ne[0] = n0; t->ne[1] = n1; t->ne[2] = n2; t->ne[3] = n3;
        t->nb[0] = t_size(type); t->nb[1] = t->nb[0] * (size_t) (n0 / t_blck(type));
        t->nb[2] = t->nb[1] * (size_t) n1; t->nb[3] = t->nb[2] * (size_t) n2;
    }
    ggml_tensor * new_tensor(ggml_type type, int64_t n0, int64_t n1 = 1, int64_t n2 = 1, int64_t n3 = 1) {
        ggml_tensor * t = raw();
        set_contig(t, type, n0, n1, n2, n3);
        t->buffer = buf_c;
        t->data = cur_region->take(t_nbytes(t));
        return t;
    }
    ggml_tensor * node(ggml_tensor * t) { nodes.push_back(t); return t; }
    ggml_tensor * view_of(ggml_tensor * a, size_t offset) {
        ggml_tensor * t = raw();
        t->type = a->type; t->buffer = a->buffer;
        t->view_src = a->view_src ? a->view_src : a;
        t->view_offs = offset + a->view_offs;
        t->data = a->data ? (char *) a->data + offset : nullptr;
        t->src[0] = a;
        return t;
    }
    ggml_tensor * view_1d(ggml_tensor * a, int64_t n0, size_t offset) {
        ggml_tensor * t = view_of(a, offset);
        set_contig(t, a->type, n0, 1, 1, 1);
        t->op = GGML_OP_VIEW; memcpy(t->op_params, &offset, sizeof(offset));
        return node(t);
    }
    ggml_tensor * view_3d(ggml_tensor * a, int64_t n0, int64_t n1, int64_t n2, size_t nb1, size_t nb2, size_t offset) {
        ggml_tensor * t = view_of(a, offset);
        t->ne[0] = n0; t->ne[1] = n1; t->ne[2] = n2; t->ne[3] = 1;
        t->nb[0] = t_size(a->type); t->nb[1] = nb1; t->nb[2] = nb2; t->nb[3] = nb2 * (size_t) n2;
        t->op = GGML_OP_VIEW; memcpy(t->op_params, &offset, sizeof(offset));
        return node(t);
    }
    ggml_tensor * reshape(ggml_tensor * a, int64_t n0, int64_t n1 = 1, int64_t n2 = 1) {
        ggml_tensor * t = view_of(a, 0);
        set_contig(t, a->type, n0, n1, n2, 1);
        t->op = GGML_OP_RESHAPE;
        return node(t);
    }
    ggml_tensor * permute(ggml_tensor * a, int ax0, int ax1, int ax2, int ax3) {
        ggml_tensor * t = view_of(a, 0);
        const int ax[4] = {ax0, ax1, ax2, ax3};
        for (int i = 0; i < 4; ++i) { t->ne[ax[i]] = a->ne[i]; t->nb[ax[i]] = a->nb[i]; }
        t->op = GGML_OP_PERMUTE;
        for (int i = 0; i < 4; ++i) t->op_params[i] = ax[i];
        return node(t);
    }
    ggml_tensor * op2(ggml_op op, ggml_tensor * a, ggml_tensor * b, ggml_type type, int64_t n0, int64_t n1, int64_t n2, int64_t n3) {
        ggml_tensor * t = new_tensor(type, n0, n1, n2, n3);
        t->op = op; t->src[0] = a; t->src[1] = b;
        return node(t);
    }
    ggml_tensor * mul_mat(ggml_tensor * w, ggml_tensor * x) { return op2(GGML_OP_MUL_MAT, w, x, GGML_TYPE_F32, w->ne[1], x->ne[1], x->ne[2], x->ne[3]); }
    // MUL_MAT with weight i.  Row-split: this rank computes its rows of the full result in place (a strided
    // view of it) and the backend completes the rest from the peers (include/ggml-b200.h); the full tensor
    // is what the rest of the graph reads.
    ggml_tensor * mul_mat_w(int i, ggml_tensor * x) {
        const Weight & w = weights[(size_t) i];
        if (!w.split) return mul_mat(W(i), x);
        ggml_tensor * full = new_tensor(GGML_TYPE_F32, w.full_rows, x->ne[1]);
        ggml_tensor * t = view_of(full, (size_t) w.row_low * 4);
        t->view_src = nullptr; t->view_offs = 0;                   // an op result in its own right, not a VIEW
        t->ne[0] = w.t.ne[1]; t->ne[1] = x->ne[1]; t->ne[2] = 1; t->ne[3] = 1;
        t->nb[0] = 4; t->nb[1] = full->nb[1]; t->nb[2] = full->nb[2]; t->nb[3] = full->nb[3];
        t->op = GGML_OP_MUL_MAT; t->src[0] = W(i); t->src[1] = x;
        B200_ASSERT(slices_used < slices.size());
        ggml_b200_row_slice * rs = &slices[slices_used++];
        rs->magic = GGML_B200_ROW_SLICE_MAGIC; rs->full_data = full->data; rs->full_rows = w.full_rows; rs->row_low = w.row_low;
        t->extra = rs;
        node(t);
        return full;
    }
    ggml_tensor * add(ggml_tensor * a, ggml_tensor * b) { return op2(GGML_OP_ADD, a, b, a->type, a->ne[0], a->ne[1], a->ne[2], a->ne[3]); }
    ggml_tensor * mul(ggml_tensor * a, ggml_tensor * b) { return op2(GGML_OP_MUL, a, b, a->type, a->ne[0], a->ne[1], a->ne[2], a->ne[3]); }
    ggml_tensor * get_rows(ggml_tensor * a, ggml_tensor * idx) { return op2(GGML_OP_GET_ROWS, a, idx, GGML_TYPE_F32, a->ne[0], idx->ne[0], idx->ne[1], idx->ne[2]); }
    ggml_tensor * rms_norm(ggml_tensor * a, float eps) {
        ggml_tensor * t = op2(GGML_OP_RMS_NORM, a, nullptr, a->type, a->ne[0], a->ne[1], a->ne[2], a->ne[3]);
        memcpy(t->op_params, &eps, sizeof(eps));
        return t;
    }
    ggml_tensor * silu(ggml_tensor * a) {
        ggml_tensor * t = op2(GGML_OP_UNARY, a, nullptr, a->type, a->ne[0], a->ne[1], a->ne[2], a->ne[3]);
        t->op_params[0] = GGML_UNARY_OP_SILU;
        return t;
    }
    ggml_tensor * rope(ggml_tensor * a, ggml_tensor * pos) {
        ggml_tensor * t = op2(GGML_OP_ROPE, a, pos, a->type, a->ne[0], a->ne[1], a->ne[2], a->ne[3]);
        int32_t params[15] = {0};
        params[1] = head_dim; params[2] = 0 /* GGML_ROPE_TYPE_NORMAL */; params[4] = cfg.n_ctx;
        const float f[6] = {cfg.rope_theta, 1.0f, 0.0f, 1.0f, 32.0f, 1.0f};   // base, scale, ext, attn, beta_fast, beta_slow
        memcpy(params + 5, f, sizeof(f));
        memcpy(t->op_params, params, sizeof(params));
        if (w_rope_ff >= 0) t->src[2] = W(w_rope_ff);                // per-frequency divisors (Llama-3.1 files), ggml_rope_ext's `c`
        return t;
    }
    ggml_tensor * cpy(ggml_tensor * a, ggml_tensor * b) {          // result is a view of b
        ggml_tensor * t = view_of(b, 0);
        for (int i = 0; i < 4; ++i) { t->ne[i] = b->ne[i]; t->nb[i] = b->nb[i]; }
        t->op = GGML_OP_CPY; t->src[0] = a; t->src[1] = b;
        return node(t);
    }
    ggml_tensor * cast(ggml_tensor * a, ggml_type type) {
        ggml_tensor * t = new_tensor(type, a->ne[0], a->ne[1], a->ne[2], a->ne[3]);
        t->op = GGML_OP_CPY; t->src[0] = a; t->src[1] = t;
        return node(t);
    }
    ggml_tensor * flash_attn(ggml_tensor * q, ggml_tensor * k, ggml_tensor * v, ggml_tensor * mask, float scale) {
        ggml_tensor * t = new_tensor(GGML_TYPE_F32, q->ne[0], q->ne[2], q->ne[1], q->ne[3]);
        t->op = GGML_OP_FLASH_ATTN_EXT; t->src[0] = q; t->src[1] = k; t->src[2] = v; t->src[3] = mask;
        const float p[3] = {scale, 0.0f, 0.0f};
        memcpy(t->op_params, p, sizeof(p));
        t->op_params[3] = GGML_PREC_F32;                             // libllama forces F32 precision (src/llama.cpp:595)
        return node(t);
    }

    // ---- model ----
    static bool use_more_bits(int il, int n) { return il < n / 8 || il >= 7 * n / 8 || (il - n / 8) % 3 == 2; }
    // tensor types found in a model file replace the synthetic model's Q4_K_M mixture
    const std::map<std::string, int> * type_override = nullptr;
    void add_weight(const std::string & name, ggml_type type, int64_t n0, int64_t n1, bool split = false) {
        if (type_override) { auto it = type_override->find(name); if (it != type_override->end()) type = (ggml_type) it->second; }
        Weight w; w.name = name; memset(&w.t, 0, sizeof(w.t));
        w.full_rows = n1; w.row_low = 0; w.split = split && n_ranks > 1;
        if (w.split) {
            int64_t lo = 0, hi = n1;
            b200_row_split_range(n1, rank, n_ranks, &lo, &hi);
            w.row_low = lo; n1 = hi - lo;
        }
        set_contig(&w.t, type, n0, n1, 1, 1);
        snprintf(w.t.name, sizeof(w.t.name), "%s", name.c_str());
        w.offset = 0;
        weights.push_back(w);
    }
    // per-layer order: attn_norm, attn_q, attn_k, attn_v, attn_output, ffn_norm, ffn_gate, ffn_up, ffn_down
    enum { W_TOK = 0, W_OUT_NORM = 1, W_OUT = 2, W_L0 = 3, W_PER_LAYER = 9 };
    void add_weights() {
        const int E = cfg.n_embd, F = cfg.n_ff, KV = n_embd_kv;
        add_weight("token_embd.weight", GGML_TYPE_Q4_K, E, cfg.n_vocab);
        add_weight("output_norm.weight", GGML_TYPE_F32, E, 1);
        add_weight("output.weight", GGML_TYPE_Q6_K, E, cfg.n_vocab, true);
        for (int il = 0; il < cfg.n_layer; ++il) {
            const std::string p = "blk." + std::to_string(il) + ".";
            const ggml_type more = use_more_bits(il, cfg.n_layer) ? GGML_TYPE_Q6_K : GGML_TYPE_Q4_K;
            // 70B-class models (80 layers, 8 query heads per KV head) keep attn_v at 5 bits or more:
            // src/llama-quant.cpp:238-243
            const ggml_type v_type = (cfg.n_layer == 80 && more == GGML_TYPE_Q4_K) ? GGML_TYPE_Q5_K : more;
            add_weight(p + "attn_norm.weight", GGML_TYPE_F32, E, 1);
            add_weight(p + "attn_q.weight", GGML_TYPE_Q4_K, E, E, true);
            add_weight(p + "attn_k.weight", GGML_TYPE_Q4_K, E, KV, true);
            add_weight(p + "attn_v.weight", v_type, E, KV, true);
            add_weight(p + "attn_output.weight", GGML_TYPE_Q4_K, E, E, true);
            add_weight(p + "ffn_norm.weight", GGML_TYPE_F32, E, 1);
            add_weight(p + "ffn_gate.weight", GGML_TYPE_Q4_K, E, F, true);
            add_weight(p + "ffn_up.weight", GGML_TYPE_Q4_K, E, F, true);
            add_weight(p + "ffn_down.weight", more, F, E, true);
        }
        // optional, last: rope frequency factors of a model file (src/llama-model.cpp: rope_freqs, one tensor shared by the layers)
        if (type_override && type_override->count("rope_freqs.weight")) {
            add_weight("rope_freqs.weight", GGML_TYPE_F32, head_dim / 2, 1);
            w_rope_ff = (int) weights.size() - 1;
        }
    }
    int w_rope_ff = -1;
    ggml_tensor * W(int i) { return &weights[(size_t) i].t; }

    void build_graph(int n_tokens, int pos0) {
        pool_used = 0; nodes.clear(); slices_used = 0;
        rg_global.reset(); rg_layer[0].reset(); rg_layer[1].reset();
        const int n_kv = std::min<int>(cfg.n_ctx, (pos0 + n_tokens + 255) / 256 * 256);
        const int n_pad = (n_tokens + 63) / 64 * 64;
        const float eps = cfg.rms_eps, kq_scale = 1.0f / std::sqrt((float) head_dim);
        const size_t krow = (size_t) n_embd_kv * 2;                // bytes of one token's K (or V) row, all KV heads

        cur_region = &rg_global;
        inp_tokens  = new_tensor(GGML_TYPE_I32, n_tokens);
        inp_pos     = new_tensor(GGML_TYPE_I32, n_tokens);
        inp_mask    = new_tensor(GGML_TYPE_F32, n_kv, n_pad);
        inp_out_ids = new_tensor(GGML_TYPE_I32, 1);
        ggml_tensor * mask16 = cast(inp_mask, GGML_TYPE_F16);
        ggml_tensor * inpL = get_rows(W(W_TOK), inp_tokens);

        for (int il = 0; il < cfg.n_layer; ++il) {
            cur_region = &rg_layer[il & 1];
            cur_region->reset();
            const int wb = W_L0 + il * W_PER_LAYER;
            ggml_tensor * inpSA = inpL;
            ggml_tensor * cur = mul(rms_norm(inpL, eps), W(wb + 0));
            ggml_tensor * Q = mul_mat_w(wb + 1, cur);
            ggml_tensor * K = mul_mat_w(wb + 2, cur);
            ggml_tensor * V = mul_mat_w(wb + 3, cur);
            Q = rope(reshape(Q, head_dim, cfg.n_head, n_tokens), inp_pos);
            K = rope(reshape(K, head_dim, cfg.n_head_kv, n_tokens), inp_pos);
            // KV store: F32 -> F16 into the cache rows [pos0, pos0 + n_tokens)
            cpy(K, view_1d(&k_l[(size_t) il], (int64_t) n_tokens * n_embd_kv, krow * (size_t) pos0));
            cpy(V, view_1d(&v_l[(size_t) il], (int64_t) n_tokens * n_embd_kv, krow * (size_t) pos0));
            ggml_tensor * q = permute(Q, 0, 2, 1, 3);
            ggml_tensor * k = view_3d(&k_l[(size_t) il], head_dim, n_kv, cfg.n_head_kv, krow, (size_t) head_dim * 2, 0);
            ggml_tensor * v = view_3d(&v_l[(size_t) il], head_dim, n_kv, cfg.n_head_kv, krow, (size_t) head_dim * 2, 0);
            cur = flash_attn(q, k, v, mask16, kq_scale);
            cur = reshape(cur, (int64_t) head_dim * cfg.n_head, n_tokens);
            if (il == cfg.n_layer - 1) {                           // only the last token's row is needed from here on
                cur   = get_rows(cur, inp_out_ids);
                inpSA = get_rows(inpSA, inp_out_ids);
            }
            cur = mul_mat_w(wb + 4, cur);
            ggml_tensor * ffn_inp = add(cur, inpSA);
            cur = mul(rms_norm(ffn_inp, eps), W(wb + 5));
            ggml_tensor * up   = mul_mat_w(wb + 7, cur);
            ggml_tensor * gate = mul_mat_w(wb + 6, cur);
            cur = mul(silu(gate), up);
            cur = mul_mat_w(wb + 8, cur);
            inpL = add(cur, ffn_inp);
        }
        cur_region = &rg_global;
        ggml_tensor * cur = mul(rms_norm(inpL, eps), W(W_OUT_NORM));
        logits = mul_mat_w(W_OUT, cur);

        graph = {};
        graph.size = (int) nodes.size(); graph.n_nodes = (int) nodes.size(); graph.nodes = nodes.data();
        graph.order = GGML_CGRAPH_EVAL_ORDER_LEFT_TO_RIGHT;
    }
};

namespace {

ggml_backend_buffer_t alloc_buffer(b200_llama * m, size_t size, const char * what) {
    ggml_backend_buffer_t b = m->buft->iface.alloc_buffer(m->buft, size);
    if (!b) g_error = std::string("alloc_buffer failed for ") + what;
    return b;
}
void free_buffer(ggml_backend_buffer_t b) {
    if (!b) return;
    if (b->iface.free_buffer) b->iface.free_buffer(b);
    delete b;                                            // what ggml_backend_buffer_free does (ggml-backend.cpp:99-111)
}
void upload(b200_llama * m, ggml_tensor * t, const void * data, size_t n) {
    if (m->backend->iface.set_tensor_async) m->backend->iface.set_tensor_async(m->backend, t, data, 0, n);
    else t->buffer->iface.set_tensor(t->buffer, t, data, 0, n);
}

}  // namespace

extern "C" {
#define API __attribute__((visibility("default")))

API const char * b200_llama_error(void) { return g_error.c_str(); }

static b200_llama * create_impl(void * reg_, int32_t device_index, const b200_llama_config * cfg, const std::map<std::string, int> * types);

API b200_llama * b200_llama_create(void * reg_, int32_t device_index, const b200_llama_config * cfg) {
    return create_impl(reg_, device_index, cfg, nullptr);
}

static b200_llama * create_impl(void * reg_, int32_t device_index, const b200_llama_config * cfg, const std::map<std::string, int> * types) {
    std::unique_ptr<b200_llama> m(new b200_llama);
    m->cfg = *cfg;
    m->type_override = types;
    // hyper-parameters may come from a file: nothing below divides by, or sizes a buffer from, an unchecked value
    if (cfg->n_layer <= 0 || cfg->n_layer > 1024 || cfg->n_embd <= 0 || cfg->n_embd > (1 << 20) || cfg->n_head <= 0 || cfg->n_head_kv <= 0 ||
        cfg->n_ff <= 0 || cfg->n_ff > (1 << 24) || cfg->n_vocab <= 0 || cfg->n_ctx <= 0 || cfg->n_ubatch <= 0 || cfg->n_ubatch > cfg->n_ctx) {
        g_error = "model hyper-parameters out of range (layers, widths, heads, vocabulary, context and batch must be positive and sane)";
        return nullptr;
    }
    if (cfg->n_embd % cfg->n_head || cfg->n_head % cfg->n_head_kv || cfg->n_embd % 256 || cfg->n_ff % 256) { g_error = "unsupported model shape"; return nullptr; }
    m->n_ranks = cfg->n_ranks > 1 ? cfg->n_ranks : 1;
    m->rank = m->n_ranks > 1 ? cfg->rank : 0;
    if (m->n_ranks > GGML_B200_MAX_PEERS || m->rank < 0 || m->rank >= m->n_ranks) { g_error = "bad rank / n_ranks"; return nullptr; }
    if (m->n_ranks > 1 && reg_) { g_error = "row-split needs the B200 backend"; return nullptr; }
    m->head_dim = cfg->n_embd / cfg->n_head;
    m->n_embd_kv = m->head_dim * cfg->n_head_kv;
    m->reg = reg_ ? (ggml_backend_reg_t) reg_ : ggml_backend_init();
    m->is_b200 = !reg_;
    if (!m->reg || m->reg->api_version != GGML_BACKEND_API_VERSION) { g_error = "bad backend registry"; return nullptr; }
    if ((size_t) device_index >= m->reg->iface.get_device_count(m->reg)) { g_error = "no such device in the backend registry"; return nullptr; }
    m->dev = m->reg->iface.get_device(m->reg, (size_t) device_index);
    m->backend = m->dev->iface.init_backend(m->dev, nullptr);
    if (!m->backend) { g_error = "init_backend failed"; return nullptr; }
    m->buft = m->dev->iface.get_buffer_type(m->dev);
    if (cfg->n_threads > 0 && m->reg->iface.get_proc_address) {
        auto fn = (void (*)(ggml_backend_t, int)) m->reg->iface.get_proc_address(m->reg, "ggml_backend_set_n_threads");
        if (fn) fn(m->backend, cfg->n_threads);
    }
    if (m->is_b200) {
        auto gs = (void * (*)(ggml_backend_t)) m->reg->iface.get_proc_address(m->reg, "ggml_backend_b200_get_stream");
        m->stream = (cudaStream_t) gs(m->backend);
        m->launch_count_fn = (uint64_t (*)(ggml_backend_t)) m->reg->iface.get_proc_address(m->reg, "ggml_backend_b200_get_launch_count");
        m->status_fn = (int (*)(ggml_backend_t)) m->reg->iface.get_proc_address(m->reg, "ggml_backend_b200_get_status");
        B200_CUDA_CHECK(cudaEventCreate(&m->ev0));
        B200_CUDA_CHECK(cudaEventCreate(&m->ev1));
    }

    // weights: one buffer, tensors at 128-byte aligned offsets
    m->add_weights();
    m->type_override = nullptr;
    size_t off = 0;
    for (Weight & w : m->weights) { off = align_up(off); w.offset = off; off += t_nbytes(&w.t); m->weight_bytes += t_nbytes(&w.t); }
    m->weight_bytes -= t_nbytes(&m->weights[b200_llama::W_TOK].t);   // embeddings: only the gathered rows are read
    m->buf_w = alloc_buffer(m.get(), off, "weights");
    if (!m->buf_w) return nullptr;
    char * wbase = (char *) m->buf_w->iface.get_base(m->buf_w);
    for (Weight & w : m->weights) { w.t.buffer = m->buf_w; w.t.data = wbase + w.offset; }

    // KV cache: per layer K and V, F16, n_ctx rows of n_embd_kv
    const size_t kv_one = align_up((size_t) m->n_embd_kv * 2 * (size_t) cfg->n_ctx);
    m->buf_kv = alloc_buffer(m.get(), kv_one * 2 * (size_t) cfg->n_layer, "kv cache");
    if (!m->buf_kv) { free_buffer(m->buf_w); return nullptr; }
    m->buf_kv->iface.clear(m->buf_kv, 0);
    char * kvbase = (char *) m->buf_kv->iface.get_base(m->buf_kv);
    m->k_l.resize((size_t) cfg->n_layer); m->v_l.resize((size_t) cfg->n_layer);
    for (int il = 0; il < cfg->n_layer; ++il) {
        for (int kv = 0; kv < 2; ++kv) {
            ggml_tensor * t = kv ? &m->v_l[(size_t) il] : &m->k_l[(size_t) il];
            memset(t, 0, sizeof(*t));
            b200_llama::set_contig(t, GGML_TYPE_F16, (int64_t) m->n_embd_kv * cfg->n_ctx, 1, 1, 1);
            t->buffer = m->buf_kv; t->data = kvbase + kv_one * (size_t) (2 * il + kv);
        }
    }

    // compute buffer: size it with a dry run of the largest graph
    m->pool.resize((size_t) cfg->n_layer * 80 + 64);
    m->slices.resize((size_t) cfg->n_layer * 7 + 1);
    m->nodes.reserve(m->pool.size());
    m->build_graph(cfg->n_ubatch, cfg->n_ctx - cfg->n_ubatch);
    // The compute buffer is the arena the peers map in row-split mode: its first bytes hold the barrier
    // flags (zero to begin with), and every rank lays it out identically.
    const size_t sg = align_up(m->rg_global.peak) + ALIGN, sl = align_up(std::max(m->rg_layer[0].peak, m->rg_layer[1].peak)) + ALIGN;
    const size_t fl = GGML_B200_PEER_FLAG_BYTES;
    m->buf_c = alloc_buffer(m.get(), fl + sg + 2 * sl, "compute");
    if (!m->buf_c) { free_buffer(m->buf_w); free_buffer(m->buf_kv); return nullptr; }
    m->buf_c->iface.clear(m->buf_c, 0);
    char * cbase = (char *) m->buf_c->iface.get_base(m->buf_c);
    m->rg_global.base = cbase + fl; m->rg_global.cap = sg;
    m->rg_layer[0].base = cbase + fl + sg; m->rg_layer[0].cap = sl;
    m->rg_layer[1].base = cbase + fl + sg + sl; m->rg_layer[1].cap = sl;
    m->arena_bytes = fl + sg + 2 * sl;
    {
        const size_t n_pad = ((size_t) cfg->n_ubatch + 63) / 64 * 64;
        m->mask_cap = (size_t) cfg->n_ctx * n_pad;
        void * probe = nullptr;
        m->host_pinned = m->is_b200 && cudaMallocHost(&probe, 64) == cudaSuccess;
        if (probe) cudaFreeHost(probe); else cudaGetLastError();
        auto take = [&](size_t n) -> void * { void * q = nullptr; if (m->host_pinned) { if (cudaMallocHost(&q, n) != cudaSuccess) { cudaGetLastError(); q = nullptr; } } else q = malloc(n); return q; };
        m->mask_host = (float *) take(m->mask_cap * 4);
        m->pos_host = (int32_t *) take((size_t) cfg->n_ubatch * 4);
        m->tok_host = (int32_t *) take((size_t) cfg->n_ubatch * 4);
        m->logits_stage = (float *) take((size_t) cfg->n_vocab * 4);
        if (!m->mask_host || !m->pos_host || !m->tok_host || !m->logits_stage) { g_error = "host staging allocation failed"; b200_llama_free(m.release()); return nullptr; }
    }
    return m.release();
}

API void b200_llama_free(b200_llama * m) {
    if (!m) return;
    if (m->backend->iface.synchronize) m->backend->iface.synchronize(m->backend);
    for (int r = 0; r < m->n_ranks; ++r) if (r != m->rank && m->peer_arena[r]) cudaIpcCloseMemHandle(m->peer_arena[r]);
    if (m->ev0) cudaEventDestroy(m->ev0);
    if (m->ev1) cudaEventDestroy(m->ev1);
    m->host_free(m->mask_host); m->host_free(m->pos_host); m->host_free(m->tok_host); m->host_free(m->logits_stage);
    free_buffer(m->buf_c); free_buffer(m->buf_kv); free_buffer(m->buf_w);
    m->backend->iface.free(m->backend);
    delete m;
}

// ---- model files ---------------------------------------------------------------------------
// Host bytes -> weight buffer.  On the B200 backend the tensors are cut into 16 MB jobs that a few worker
// threads pull from a shared counter; each worker copies its job out of the page cache (the file mapping)
// into one of its two pinned staging buffers and queues an asynchronous host-to-device transfer on its own
// stream, so page-cache reads, staging copies and DMA of different jobs overlap.  Other backends take the
// mapping directly through set_tensor.
namespace {
struct Uploader {
    struct Job { char * dst; const uint8_t * src; size_t len; };
    static constexpr size_t CHUNK = (size_t) 16 << 20;
    b200_llama * m;
    std::vector<Job> jobs;
    explicit Uploader(b200_llama * m_) : m(m_) {}
    void put(ggml_tensor * t, const uint8_t * src, size_t n) {
        if (!m->is_b200) { m->buf_w->iface.set_tensor(m->buf_w, t, src, 0, n); return; }
        for (size_t off = 0; off < n; off += CHUNK) jobs.push_back({(char *) t->data + off, src + off, std::min(CHUNK, n - off)});
    }
    static bool worker(int device, const std::vector<Job> * jobs, std::atomic<size_t> * next, std::atomic<bool> * failed) {
        void * stage[2] = {nullptr, nullptr};
        cudaEvent_t done[2] = {nullptr, nullptr};
        cudaStream_t stream = nullptr;
        bool ok = cudaSetDevice(device) == cudaSuccess &&
                  cudaMallocHost(&stage[0], CHUNK) == cudaSuccess && cudaMallocHost(&stage[1], CHUNK) == cudaSuccess &&
                  cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking) == cudaSuccess &&
                  cudaEventCreateWithFlags(&done[0], cudaEventDisableTiming) == cudaSuccess &&
                  cudaEventCreateWithFlags(&done[1], cudaEventDisableTiming) == cudaSuccess;
        int b = 0;
        while (ok && !failed->load()) {
            const size_t i = next->fetch_add(1);
            if (i >= jobs->size()) break;
            const Job & j = (*jobs)[i];
            ok = cudaEventSynchronize(done[b]) == cudaSuccess;                     // this buffer's previous transfer has left it
            if (!ok) break;
            memcpy(stage[b], j.src, j.len);
            ok = cudaMemcpyAsync(j.dst, stage[b], j.len, cudaMemcpyHostToDevice, stream) == cudaSuccess &&
                 cudaEventRecord(done[b], stream) == cudaSuccess;
            b ^= 1;
        }
        if (stream) { ok = cudaStreamSynchronize(stream) == cudaSuccess && ok; cudaStreamDestroy(stream); }
        for (int k = 0; k < 2; ++k) { if (done[k]) cudaEventDestroy(done[k]); if (stage[k]) cudaFreeHost(stage[k]); }
        if (!ok) { cudaGetLastError(); failed->store(true); }
        return ok;
    }
    bool finish() {
        if (jobs.empty()) return true;
        int device = 0;
        if (cudaGetDevice(&device) != cudaSuccess) return false;
        unsigned hw = std::thread::hardware_concurrency();
        const size_t n_threads = std::max<size_t>(1, std::min(std::min<size_t>(8, hw ? hw / 2 : 1), jobs.size()));
        std::atomic<size_t> next{0};
        std::atomic<bool> failed{false};
        std::vector<std::thread> pool;
        for (size_t t = 1; t < n_threads; ++t) pool.emplace_back(worker, device, &jobs, &next, &failed);
        worker(device, &jobs, &next, &failed);
        for (std::thread & t : pool) t.join();
        return !failed.load();
    }
};
}  // namespace

API b200_llama * b200_llama_load_gguf(void * reg_, int32_t device_index, const char * path, int32_t n_ctx, int32_t n_ubatch,
                                      int32_t n_threads, int32_t n_ranks, int32_t rank) {
    GgufFile f;
    if (!f.open(path, g_error)) return nullptr;
    std::string arch;
    if (!f.get_str("general.architecture", arch) || arch != "llama") { g_error = std::string(path) + ": architecture '" + arch + "' is not llama"; return nullptr; }
    auto key = [&](const char * k) { return arch + "." + k; };
    b200_llama_config cfg = {};
    uint32_t n_layer = 0, n_embd = 0, n_head = 0, n_head_kv = 0, n_ff = 0, n_vocab = 0, n_rot = 0, n_expert = 0;
    if (!f.get_u32(key("block_count"), n_layer) || !f.get_u32(key("embedding_length"), n_embd) || !f.get_u32(key("attention.head_count"), n_head) ||
        !f.get_u32(key("feed_forward_length"), n_ff) || n_head == 0) {
        g_error = std::string(path) + ": missing llama hyper-parameters (block_count, embedding_length, feed_forward_length, attention.head_count)";
        return nullptr;
    }
    if (!f.get_u32(key("attention.head_count_kv"), n_head_kv)) n_head_kv = n_head;
    const GgufTensor * tok = f.find("token_embd.weight");
    if (!tok) { g_error = std::string(path) + ": no token_embd.weight"; return nullptr; }
    if (!f.get_u32(key("vocab_size"), n_vocab)) n_vocab = (uint32_t) tok->ne[1];
    if (f.get_u32(key("rope.dimension_count"), n_rot) && n_rot != n_embd / n_head) { g_error = "partial rotary dimensions are not supported by this driver"; return nullptr; }
    if (f.get_u32(key("expert_count"), n_expert) && n_expert > 0) { g_error = "mixture-of-experts files are not supported by this driver"; return nullptr; }
    std::string scaling;
    if (f.get_str(key("rope.scaling.type"), scaling) && scaling != "none") { g_error = "rope scaling '" + scaling + "' is not supported by this driver"; return nullptr; }
    cfg.n_layer = (int32_t) n_layer; cfg.n_embd = (int32_t) n_embd; cfg.n_head = (int32_t) n_head; cfg.n_head_kv = (int32_t) n_head_kv;
    cfg.n_ff = (int32_t) n_ff; cfg.n_vocab = (int32_t) n_vocab;
    cfg.n_ctx = n_ctx; cfg.n_ubatch = n_ubatch; cfg.n_threads = n_threads; cfg.n_ranks = n_ranks; cfg.rank = rank;
    cfg.rope_theta = 10000.0f; cfg.rms_eps = 1e-5f;                     // defaults of the reference's loader (src/llama-model.cpp)
    f.get_f32(key("rope.freq_base"), cfg.rope_theta);
    f.get_f32(key("attention.layer_norm_rms_epsilon"), cfg.rms_eps);

    // tensor types as stored; a file without output.weight ties it to the token embeddings (src/llama-model.cpp: output = tok_embd)
    std::map<std::string, int> types;
    for (const GgufTensor & t : f.tensors) types[t.name] = t.type;
    const bool tied = !f.find("output.weight");
    if (tied) types["output.weight"] = tok->type;
    b200_llama * m = create_impl(reg_, device_index, &cfg, &types);
    if (!m) return nullptr;

    Uploader up(m);
    for (Weight & w : m->weights) {
        const GgufTensor * t = f.find(tied && w.name == "output.weight" ? "token_embd.weight" : w.name);
        std::string why;
        if (!t) why = "is missing";
        else if (t->type != (int32_t) w.t.type) why = "has an unexpected type";
        else if (t->ne[0] != w.t.ne[0] || t->ne[1] != w.full_rows || t->ne[2] != 1 || t->ne[3] != 1) why = "has an unexpected shape";
        else if (w.full_rows == 1 ? t->type != GGML_TYPE_F32
                                  : !(t->type == GGML_TYPE_F32 || t->type == GGML_TYPE_F16 || t->type == GGML_TYPE_BF16 || mmvq_type_supported(t->type)))
            why = "has a type this backend does not compute with";
        if (!why.empty()) { g_error = std::string(path) + ": tensor " + w.name + " " + why; b200_llama_free(m); return nullptr; }
        const size_t row = t_row_size(t->type, t->ne[0]);
        up.put(&w.t, f.data(*t) + (size_t) w.row_low * row, t_nbytes(&w.t));
    }
    if (!up.finish()) { g_error = "weight upload failed"; b200_llama_free(m); return nullptr; }
    return m;
}

API void b200_llama_get_config(const b200_llama * m, b200_llama_config * cfg) { *cfg = m->cfg; }

API int32_t b200_llama_n_tensors(const b200_llama * m) { return (int32_t) m->weights.size(); }

API int32_t b200_llama_tensor_info(const b200_llama * m, int32_t i, char * name, size_t cap, int32_t * type, int64_t * ne0, int64_t * ne1, size_t * nbytes) {
    if (i < 0 || (size_t) i >= m->weights.size()) return -1;
    const Weight & w = m->weights[(size_t) i];
    if (name && cap) snprintf(name, cap, "%s", w.name.c_str());
    if (type) *type = (int32_t) w.t.type;
    if (ne0) *ne0 = w.t.ne[0];
    if (ne1) *ne1 = w.t.ne[1];
    if (nbytes) *nbytes = t_nbytes(&w.t);
    return 0;
}

API int32_t b200_llama_set_tensor(b200_llama * m, int32_t i, const void * data, size_t nbytes) {
    if (i < 0 || (size_t) i >= m->weights.size()) { g_error = "tensor index out of range"; return -1; }
    Weight & w = m->weights[(size_t) i];
    if (nbytes != t_nbytes(&w.t)) { g_error = "size mismatch for " + w.name; return -2; }
    m->buf_w->iface.set_tensor(m->buf_w, &w.t, data, 0, nbytes);
    return 0;
}

API void * b200_llama_tensor_data(const b200_llama * m, int32_t i) {
    return (i < 0 || (size_t) i >= m->weights.size()) ? nullptr : m->weights[(size_t) i].t.data;
}

API int32_t b200_llama_decode(b200_llama * m, const int32_t * tokens, int32_t n_tokens, int32_t pos0, float * logits_host) {
    if (n_tokens < 1 || n_tokens > m->cfg.n_ubatch || pos0 < 0 || pos0 + n_tokens > m->cfg.n_ctx) { g_error = "bad token range"; return -1; }
    m->build_graph(n_tokens, pos0);
    // inputs: positions, causal mask (0 where key <= query position, -inf elsewhere and in pad rows;
    // llama_set_inputs, src/llama-context.cpp:129-203), index of the output row
    const int64_t n_kv = m->inp_mask->ne[0], n_pad = m->inp_mask->ne[1];
    for (int i = 0; i < n_tokens; ++i) { m->pos_host[i] = pos0 + i; m->tok_host[i] = tokens[i]; }
    const size_t mask_n = (size_t) (n_kv * n_pad);
    for (size_t i = 0; i < mask_n; ++i) m->mask_host[i] = -INFINITY;
    for (int i = 0; i < n_tokens; ++i) {
        float * row = m->mask_host + (size_t) i * (size_t) n_kv;
        const int lim = std::min<int64_t>(n_kv, pos0 + i + 1);
        for (int j = 0; j < lim; ++j) row[j] = 0.0f;
    }
    const int32_t out_id = n_tokens - 1;
    upload(m, m->inp_tokens, m->tok_host, (size_t) n_tokens * 4);
    upload(m, m->inp_pos, m->pos_host, (size_t) n_tokens * 4);
    upload(m, m->inp_mask, m->mask_host, mask_n * 4);
    upload(m, m->inp_out_ids, &out_id, 4);

    const auto t0 = std::chrono::steady_clock::now();
    if (m->is_b200) B200_CUDA_CHECK(cudaEventRecord(m->ev0, m->stream));
    const enum ggml_status st = m->backend->iface.graph_compute(m->backend, &m->graph);
    if (m->is_b200) B200_CUDA_CHECK(cudaEventRecord(m->ev1, m->stream));
    if (st != GGML_STATUS_SUCCESS) { g_error = "graph_compute failed"; return -2; }
    if (logits_host) {
        if (m->backend->iface.get_tensor_async) m->backend->iface.get_tensor_async(m->backend, m->logits, m->logits_stage, 0, (size_t) m->cfg.n_vocab * 4);
        else m->logits->buffer->iface.get_tensor(m->logits->buffer, m->logits, m->logits_stage, 0, (size_t) m->cfg.n_vocab * 4);
    }
    if (m->backend->iface.synchronize) m->backend->iface.synchronize(m->backend);
    if (logits_host) memcpy(logits_host, m->logits_stage, (size_t) m->cfg.n_vocab * 4);
    m->last_n_nodes = m->graph.n_nodes;
    if (m->n_ranks > 1 && m->status_fn) {              // a rank that stopped answering shows up as a barrier that gave up
        const int dev_status = m->status_fn(m->backend);
        if (dev_status != 0) { g_error = "device status " + std::to_string(dev_status) + " (3 = a peer did not reach the barrier in time)"; return -3; }
    }
    if (m->is_b200) { float ms = 0; B200_CUDA_CHECK(cudaEventElapsedTime(&ms, m->ev0, m->ev1)); m->last_ms = ms; }
    else m->last_ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
    return 0;
}

API void b200_row_split_range(int64_t n_rows, int32_t rank, int32_t n_ranks, int64_t * row_low, int64_t * row_high) {
    // equal shares, boundaries rounded down to a multiple of 128 rows, the last rank takes the remainder
    // (get_row_split with the MMQ tile height as rounding, ggml/src/ggml-cuda/ggml-cuda.cu:725-742)
    const int64_t R = 128;
    auto bound = [&](int r) -> int64_t {
        if (r <= 0) return 0;
        if (r >= n_ranks) return n_rows;
        const int64_t b = n_rows * r / n_ranks;
        return b - b % R;
    };
    if (n_ranks < 1) n_ranks = 1;
    *row_low = bound(rank); *row_high = bound(rank + 1);
}

API int32_t b200_llama_tensor_rows(const b200_llama * m, int32_t i, int64_t * row_low, int64_t * full_rows) {
    if (i < 0 || (size_t) i >= m->weights.size()) return -1;
    if (row_low) *row_low = m->weights[(size_t) i].row_low;
    if (full_rows) *full_rows = m->weights[(size_t) i].full_rows;
    return 0;
}

API int32_t b200_llama_ipc_handle(b200_llama * m, void * handle_out) {
    if (!m->is_b200) { g_error = "not the B200 backend"; return -1; }
    cudaIpcMemHandle_t h;
    const cudaError_t e = cudaIpcGetMemHandle(&h, m->buf_c->iface.get_base(m->buf_c));
    if (e != cudaSuccess) { cudaGetLastError(); g_error = std::string("cudaIpcGetMemHandle: ") + cudaGetErrorString(e); return -2; }
    static_assert(sizeof(h) == B200_LLAMA_IPC_HANDLE_BYTES, "handle size");
    memcpy(handle_out, &h, sizeof(h));
    return 0;
}

API int32_t b200_llama_attach_peers(b200_llama * m, const void * handles) {
    if (m->n_ranks < 2) return 0;
    ggml_b200_peers pr = {};
    pr.rank = m->rank; pr.n_ranks = m->n_ranks; pr.arena_bytes = m->arena_bytes;
    for (int r = 0; r < m->n_ranks; ++r) {
        if (r == m->rank) { pr.arena[r] = m->buf_c->iface.get_base(m->buf_c); continue; }
        if (!m->peer_arena[r]) {
            cudaIpcMemHandle_t h;
            memcpy(&h, (const char *) handles + (size_t) r * sizeof(h), sizeof(h));
            const cudaError_t e = cudaIpcOpenMemHandle(&m->peer_arena[r], h, cudaIpcMemLazyEnablePeerAccess);
            if (e != cudaSuccess) { cudaGetLastError(); m->peer_arena[r] = nullptr; g_error = std::string("cudaIpcOpenMemHandle: ") + cudaGetErrorString(e); return -2; }
        }
        pr.arena[r] = m->peer_arena[r];
    }
    auto fn = (int (*)(ggml_backend_t, const ggml_b200_peers *)) m->reg->iface.get_proc_address(m->reg, "ggml_backend_b200_set_peers");
    const int rc = fn ? fn(m->backend, &pr) : -100;
    if (rc != 0) { g_error = "ggml_backend_b200_set_peers failed: " + std::to_string(rc); return -3; }
    return 0;
}

API int32_t  b200_llama_last_n_nodes(const b200_llama * m) { return m->last_n_nodes; }
API double   b200_llama_last_compute_ms(const b200_llama * m) { return m->last_ms; }
API uint64_t b200_llama_launch_count(const b200_llama * m) { return m->launch_count_fn ? m->launch_count_fn(m->backend) : 0; }
API size_t   b200_llama_weight_bytes(const b200_llama * m) { return m->weight_bytes; }

}  // extern "C"
