// Recognises runs of Llama layers in a single-token ggml graph and turns them into the phase list of the
// persistent decode-step kernel (csrc/kernels/decode_step.cu).  The graph is the one
// src/llama.cpp:1476-1640 (build_llama) emits: per layer
//     [ADD] RMS_NORM MUL {MUL_MAT q,k,v} ROPE ROPE CPY CPY FLASH_ATTN_EXT MUL_MAT(wo)
//      ADD  RMS_NORM MUL {MUL_MAT gate,up} UNARY(SILU) MUL MUL_MAT(down)
// and finally ADD RMS_NORM MUL MUL_MAT(output).  Matching follows the data flow (who consumes what), not
// the node order, so both libllama's interleaved order and a hand-built graph are recognised.
//
// Inside the covered node range every intermediate value lives in scratch memory owned by the backend, not
// at the address ggml-alloc gave its tensor: the allocator reuses memory according to the ORIGINAL node
// order, and the fused phases compute several nodes at once.  Only tensors that something outside the range
// reads (or that are graph results) are written to their own memory.
#include "backend.h"
#include "ggml-impl.h"

#include <algorithm>
#include <unordered_map>
#include <unordered_set>

namespace b200 {

namespace {

constexpr int    MEGA_MAX_OPS = 1024;
constexpr size_t MEGA_VEC_FLOATS = 32768;
constexpr int    MEGA_N_VEC = 9;
constexpr size_t MEGA_PARTIAL_BYTES = (size_t) 4 << 20;
constexpr size_t MEGA_OFF_SYNC = 0, MEGA_OFF_TICKETS = 256, MEGA_OFF_OPS = 1024;
constexpr size_t MEGA_WORK_PER_OP = 160;                                          // >= decode_step_work_bytes(1)
constexpr size_t MEGA_OPS_REGION = (size_t) MEGA_MAX_OPS * (sizeof(DsOp) + MEGA_WORK_PER_OP);
constexpr size_t MEGA_OFF_VEC = MEGA_OFF_OPS + 2 * MEGA_OPS_REGION;
constexpr size_t MEGA_OFF_PARTIALS = MEGA_OFF_VEC + MEGA_N_VEC * MEGA_VEC_FLOATS * 4;
constexpr size_t MEGA_OFF_TIMING = MEGA_OFF_PARTIALS + MEGA_PARTIAL_BYTES;       // GGML_B200_MEGA_TIMING: 4 time stamps per phase
constexpr size_t MEGA_TIMING_BYTES = (size_t) MEGA_MAX_OPS * 4 * 8;
constexpr size_t MEGA_ARENA_BYTES = MEGA_OFF_TIMING + MEGA_TIMING_BYTES;

bool is_view_op(const ggml_tensor * t) {
    return t->op == GGML_OP_RESHAPE || t->op == GGML_OP_VIEW || t->op == GGML_OP_PERMUTE || t->op == GGML_OP_TRANSPOSE;
}
bool is_vec(const ggml_tensor * t) {      // one F32 row
    return t->type == GGML_TYPE_F32 && t->ne[1] == 1 && t->ne[2] == 1 && t->ne[3] == 1 && t->nb[0] == 4;
}
// GET_ROWS of the only row of a one-row F32 tensor (libllama selects the output rows this way): an identity
bool is_identity_rows(const ggml_tensor * t) {
    if (t->op != GGML_OP_GET_ROWS || !t->src[0] || !t->src[1]) return false;
    const ggml_tensor * a = t->src[0], * ix = t->src[1];
    return a->type == GGML_TYPE_F32 && a->ne[1] == 1 && a->ne[2] == 1 && a->ne[3] == 1 && t_contiguous(a) &&
           ix->type == GGML_TYPE_I32 && t_nelements(ix) == 1 && t->type == GGML_TYPE_F32;
}
const ggml_tensor * root_of(const ggml_tensor * t) {
    while (t && ((is_view_op(t) && t->src[0]) || is_identity_rows(t))) t = t->src[0];
    return t;
}

struct Block {
    int kind = -1;                                         // 0 attention, 1 feed-forward, 2 output head
    const ggml_tensor * add = nullptr, * rn = nullptr, * mu = nullptr;
    const ggml_tensor * mm[3] = {nullptr, nullptr, nullptr};
    const ggml_tensor * rope_q = nullptr, * rope_k = nullptr, * cpy_k = nullptr, * cpy_v = nullptr, * fa = nullptr, * wo = nullptr;
    // the attention itself: FLASH_ATTN_EXT (fa), or the chain MUL_MAT(K, Q) -> SOFT_MAX -> MUL_MAT(V^T, p) -> [PERMUTE] -> CONT that
    // graphs without it hold (chain[]: those four nodes), on a V cache stored transposed (v_t: v_nbd bytes between its rows)
    const ggml_tensor * att_K = nullptr, * att_V = nullptr, * att_mask = nullptr, * att_out = nullptr;
    const ggml_tensor * chain[4] = {nullptr, nullptr, nullptr, nullptr};
    float att_scale = 0.0f; bool v_t = false; int64_t v_nbd = 0;
    int cpy_k_idx = -1, cpy_v_idx = -1;
    const ggml_tensor * silu = nullptr, * mul3 = nullptr, * down = nullptr;
};

struct Matcher {
    BackendCtx * ctx; ggml_cgraph * g; int i0;
    std::unordered_map<const ggml_tensor *, std::vector<int>> users;   // root tensor -> exec nodes reading it
    std::unordered_map<const ggml_tensor *, int> index_of;
    std::vector<uint8_t> taken;                                        // per node: consumed by the plan
    std::vector<Block> blocks;
    int last = -1, n_matvec = 0;
    const char * why = "";                                              // for GGML_B200_TRACE: the check that ended the match
    int why_line = 0;

    bool exec(int i) const {
        const ggml_tensor * n = g->nodes[i];
        return !(t_empty(n) || n->op == GGML_OP_NONE || is_view_op(n));
    }
    void index() {
        taken.assign((size_t) g->n_nodes, 0);
        for (int i = i0; i < g->n_nodes; ++i) {
            const ggml_tensor * n = g->nodes[i];
            index_of[n] = i;
            if (!exec(i) || is_identity_rows(n)) continue;
            for (int s = 0; s < GGML_MAX_SRC; ++s) if (n->src[s]) {
                std::vector<int> & u = users[root_of(n->src[s])];
                if (u.empty() || u.back() != i) u.push_back(i);
            }
        }
    }
    int idx(const ggml_tensor * t) const { auto it = index_of.find(t); return it == index_of.end() ? -1 : it->second; }
    const std::vector<int> & users_of(const ggml_tensor * t) const {
        static const std::vector<int> none;
        auto it = users.find(t);
        return it == users.end() ? none : it->second;
    }
    // the single consumer of t, if it has exactly one and that one is op `op`
    const ggml_tensor * sole_user(const ggml_tensor * t, int op) const {
        const std::vector<int> & u = users_of(t);
        if (u.size() != 1) return nullptr;
        const ggml_tensor * n = g->nodes[u[0]];
        return (int) n->op == op ? n : nullptr;
    }
    bool take(const ggml_tensor * t) {
        const int i = idx(t);
        if (i < 0 || taken[(size_t) i] || ctx->node_done[(size_t) i]) return false;
        taken[(size_t) i] = 1;
        if (i > last) last = i;
        return true;
    }
    static bool weight_ok(const ggml_tensor * mm, int64_t K) {
        const ggml_tensor * W = mm->src[0];
        if (mm->op != GGML_OP_MUL_MAT || !is_vec(mm) || !t_contiguous(mm)) return false;
        if (W->op != GGML_OP_NONE || W->view_src || W->ne[0] != K || W->ne[2] != 1 || W->ne[3] != 1 || W->nb[0] != t_size(W->type)) return false;
        if (buft_is_split(W->buffer ? W->buffer->buft : nullptr)) return false;
        return decode_step_type_ok((int) W->type, K, (int64_t) W->nb[1], W->data);
    }

    bool no(int line) { why_line = line; return false; }

    // [ADD] RMS_NORM MUL {MUL_MAT ...} starting at exec node `at`
    bool match_head(int at, Block & b) {
        const ggml_tensor * n = g->nodes[at];
        if (n->op == GGML_OP_ADD) {
            if (!is_vec(n) || !t_contiguous(n) || !n->src[0] || !n->src[1] || !is_vec(n->src[0]) || !is_vec(n->src[1])) return no(__LINE__);
            if (n->src[0]->ne[0] != n->ne[0] || n->src[1]->ne[0] != n->ne[0] || !t_contiguous(n->src[0]) || !t_contiguous(n->src[1])) return no(__LINE__);
            b.add = n;
            // its consumers: the RMS_NORM, and (later) the next residual ADD
            const ggml_tensor * rn = nullptr;
            for (int u : users_of(n)) if (g->nodes[u]->op == GGML_OP_RMS_NORM) rn = g->nodes[u];
            if (!rn) return no(__LINE__);
            n = rn;
        }
        if (n->op != GGML_OP_RMS_NORM || !is_vec(n) || !t_contiguous(n) || !n->src[0] || !is_vec(n->src[0]) || !t_contiguous(n->src[0])) return no(__LINE__);
        if (b.add && root_of(n->src[0]) != b.add) return no(__LINE__);
        b.rn = n;
        const ggml_tensor * mu = sole_user(n, GGML_OP_MUL);
        if (!mu || !is_vec(mu) || !t_contiguous(mu)) return no(__LINE__);
        const ggml_tensor * w = root_of(mu->src[0]) == n ? mu->src[1] : mu->src[0];
        if ((root_of(mu->src[0]) != n && root_of(mu->src[1]) != n) || !w || w->type != GGML_TYPE_F32 || !t_contiguous(w) || t_nelements(w) != n->ne[0] || w->op != GGML_OP_NONE) return no(__LINE__);
        b.mu = mu;
        const int64_t E = n->ne[0];
        if (E % 128) return no(__LINE__);
        const std::vector<int> & mms = users_of(mu);
        if (mms.empty() || mms.size() > 3) return no(__LINE__);
        int k = 0;
        for (int u : mms) {
            const ggml_tensor * mm = g->nodes[u];
            if (!weight_ok(mm, E) || root_of(mm->src[1]) != mu) return no(__LINE__);
            b.mm[k++] = mm;
        }
        b.kind = k == 3 ? 0 : (k == 2 ? 1 : 2);
        return true;
    }

    bool match_attention(Block & b) {
        const ggml_tensor * q = nullptr, * k = nullptr, * v = nullptr;
        for (int i = 0; i < 3; ++i) {
            const ggml_tensor * mm = b.mm[i];
            if (const ggml_tensor * r = sole_user(mm, GGML_OP_ROPE)) {
                if (root_of(r->src[0]) != mm) return no(__LINE__);
                const ggml_tensor * qk = sole_user(r, GGML_OP_MUL_MAT);              // (the score product of a graph without FLASH_ATTN_EXT)
                if (sole_user(r, GGML_OP_FLASH_ATTN_EXT) || (qk && root_of(qk->src[1]) == r && qk->src[0]->type == GGML_TYPE_F16)) { q = mm; b.rope_q = r; }
                else if (sole_user(r, GGML_OP_CPY))       { k = mm; b.rope_k = r; }
                else return no(__LINE__);
            } else if (sole_user(mm, GGML_OP_CPY)) v = mm;
            else return no(__LINE__);
        }
        if (!q || !k || !v) return no(__LINE__);
        b.mm[0] = q; b.mm[1] = k; b.mm[2] = v;
        const ggml_tensor * rq = b.rope_q, * rk = b.rope_k;
        if (rq->type != GGML_TYPE_F32 || rk->type != GGML_TYPE_F32 || !t_contiguous(rq) || !t_contiguous(rk)) return no(__LINE__);
        if (rq->src[1] != rk->src[1] || rq->src[2] != rk->src[2] || memcmp(rq->op_params, rk->op_params, sizeof(rq->op_params)) != 0) return no(__LINE__);
        if (op_param_i32(rq, 2) != 0) return no(__LINE__);                        // adjacent-pair rotation only
        const int64_t hd = rq->ne[0];
        const int n_dims = op_param_i32(rq, 1);
        if (hd != 128 || rk->ne[0] != hd || n_dims <= 0 || n_dims > hd || (n_dims & 1)) return no(__LINE__);
        if (rq->ne[2] != 1 || rk->ne[2] != 1 || rq->ne[3] != 1 || rk->ne[3] != 1) return no(__LINE__);
        if (!rq->src[1] || rq->src[1]->type != GGML_TYPE_I32) return no(__LINE__);
        if (rq->src[2] && (rq->src[2]->type != GGML_TYPE_F32 || t_nelements(rq->src[2]) < n_dims / 2)) return no(__LINE__);
        if (q->ne[0] != hd * rq->ne[1] || k->ne[0] != hd * rk->ne[1] || v->ne[0] != k->ne[0]) return no(__LINE__);

        b.cpy_k = sole_user(rk, GGML_OP_CPY); b.cpy_v = sole_user(v, GGML_OP_CPY);
        auto store_ok = [&](const ggml_tensor * c, const ggml_tensor * from) {
            if (!c || root_of(c->src[0]) != from || !c->src[1]) return no(__LINE__);
            const ggml_tensor * out = c->src[1];
            return out->type == GGML_TYPE_F16 && t_contiguous(out) && out->view_src && out->view_src->data && out->view_src->op == GGML_OP_NONE &&
                   t_nelements(out) == from->ne[0] * from->ne[1] * from->ne[2] && ((uintptr_t) out->data & 3) == 0;
        };
        // the V row of the token: stored as a row, or (cache kept transposed) as a column of [n_ctx][n_embd_v] with stride nb[1]
        auto store_t_ok = [&](const ggml_tensor * c, const ggml_tensor * from) {
            if (!c || root_of(c->src[0]) != from || !c->src[1]) return false;
            const ggml_tensor * out = c->src[1];
            return out->type == GGML_TYPE_F16 && out->ne[0] == 1 && out->ne[1] == from->ne[0] && out->ne[2] == 1 && out->ne[3] == 1 && out->nb[0] == 2 &&
                   out->nb[1] % 8 == 0 && out->view_src && out->view_src->data && out->view_src->op == GGML_OP_NONE && ((uintptr_t) out->data & 1) == 0;
        };
        if (!store_ok(b.cpy_k, rk)) return no(__LINE__);
        if (store_t_ok(b.cpy_v, v)) { b.v_t = true; b.v_nbd = (int64_t) b.cpy_v->src[1]->nb[1]; }
        else if (!store_ok(b.cpy_v, v)) return no(__LINE__);
        b.cpy_k_idx = idx(b.cpy_k); b.cpy_v_idx = idx(b.cpy_v);

        const ggml_tensor * K = nullptr, * V = nullptr, * mask = nullptr, * out = nullptr;
        if (const ggml_tensor * fa = sole_user(rq, GGML_OP_FLASH_ATTN_EXT)) {
            if (b.v_t || root_of(fa->src[0]) != rq || fa->type != GGML_TYPE_F32 || !t_contiguous(fa)) return no(__LINE__);
            if (fa->src[0]->ne[1] != 1 || fa->src[0]->ne[2] != rq->ne[1] || fa->src[0]->ne[3] != 1) return no(__LINE__);
            if (op_param_f32(fa, 1) != 0.0f || op_param_f32(fa, 2) != 0.0f) return no(__LINE__);   // no ALiBi, no soft-capping
            K = fa->src[1]; V = fa->src[2]; mask = fa->src[3]; out = fa;
            b.fa = fa; b.att_scale = op_param_f32(fa, 0);
            if (!V || V->nb[0] != 2 || V->ne[0] != hd) return no(__LINE__);
        } else {
            const ggml_tensor * kq = sole_user(rq, GGML_OP_MUL_MAT);
            if (!kq || !b.v_t || kq->type != GGML_TYPE_F32 || root_of(kq->src[1]) != rq) return no(__LINE__);
            const ggml_tensor * qv = kq->src[1];                                  // [hd, 1, n_head]: the rotated row, permuted
            if (qv->ne[0] != hd || qv->ne[1] != 1 || qv->ne[2] != rq->ne[1] || qv->ne[3] != 1 || qv->nb[0] != 4 || (int64_t) qv->nb[2] != hd * 4) return no(__LINE__);
            const ggml_tensor * sm = sole_user(kq, GGML_OP_SOFT_MAX);
            if (!sm || sm->src[0] != kq || op_param_f32(sm, 1) != 0.0f) return no(__LINE__);
            const ggml_tensor * kqv = sole_user(sm, GGML_OP_MUL_MAT);
            if (!kqv || kqv->src[1] != sm || kqv->type != GGML_TYPE_F32) return no(__LINE__);
            const ggml_tensor * cont = sole_user(kqv, GGML_OP_CONT);
            if (!cont || root_of(cont->src[0]) != kqv || cont->type != GGML_TYPE_F32 || !t_contiguous(cont) || t_nelements(cont) != hd * rq->ne[1]) return no(__LINE__);
            K = kq->src[0]; V = kqv->src[0]; mask = sm->src[1]; out = cont;
            // V^T [n_kv, hd, n_head_kv] on the transposed cache; the result [hd, 1, n_head] is read through a permutation that
            // leaves a single query's memory order alone
            if (!V || V->type != GGML_TYPE_F16 || V->nb[0] != 2 || V->ne[1] != hd || (int64_t) V->nb[1] != b.v_nbd || (int64_t) V->nb[2] != hd * b.v_nbd) return no(__LINE__);
            if (kqv->ne[0] != hd || kqv->ne[1] != 1 || kqv->ne[2] != rq->ne[1]) return no(__LINE__);
            b.chain[0] = kq; b.chain[1] = sm; b.chain[2] = kqv; b.chain[3] = cont;
            b.att_scale = op_param_f32(sm, 0);
        }
        const int64_t n_kv = K ? K->ne[1] : 0;
        if (!K || K->type != GGML_TYPE_F16 || V->type != GGML_TYPE_F16 || K->nb[0] != 2) return no(__LINE__);
        if (K->ne[0] != hd || (b.v_t ? V->ne[0] : V->ne[1]) != n_kv || K->ne[2] != rk->ne[1] || V->ne[2] != K->ne[2] || K->ne[3] != 1 || V->ne[3] != 1) return no(__LINE__);
        if (root_of(K) != b.cpy_k->src[1]->view_src || root_of(V) != b.cpy_v->src[1]->view_src) return no(__LINE__);
        auto al16 = [](const ggml_tensor * t) { return ((uintptr_t) t->data & 15) == 0 && (t->nb[1] & 15) == 0 && (t->nb[2] & 15) == 0; };
        if (!al16(K) || (!b.v_t && !al16(V)) || (b.v_t && (((uintptr_t) V->data & 7) || (b.v_nbd & 7))) || n_kv < 1 || n_kv > 1 << 20) return no(__LINE__);
        if (rq->ne[1] % rk->ne[1] || rk->ne[1] > 64 || rq->ne[1] / rk->ne[1] > 16) return no(__LINE__);
        if (mask) {
            const bool f16 = mask->type == GGML_TYPE_F16 && mask->nb[0] == 2, f32 = mask->type == GGML_TYPE_F32 && mask->nb[0] == 4;
            if ((!f16 && !f32) || mask->ne[0] < n_kv || root_of(mask) == nullptr) return no(__LINE__);
        }
        b.att_K = K; b.att_V = V; b.att_mask = mask; b.att_out = out;
        const ggml_tensor * fa = out;
        const ggml_tensor * wo = sole_user(fa, GGML_OP_MUL_MAT);
        if (!wo || root_of(wo->src[1]) != fa || !weight_ok(wo, fa->ne[0] * fa->ne[1])) return no(__LINE__);
        b.wo = wo;
        return true;
    }

    bool match_ffn(Block & b) {
        const ggml_tensor * gate = nullptr, * up = nullptr;
        for (int i = 0; i < 2; ++i) {
            const ggml_tensor * mm = b.mm[i];
            if (const ggml_tensor * s = sole_user(mm, GGML_OP_UNARY)) {
                if (op_param_i32(s, 0) != GGML_UNARY_OP_SILU || !is_vec(s) || !t_contiguous(s)) return no(__LINE__);
                gate = mm; b.silu = s;
            } else if (sole_user(mm, GGML_OP_MUL)) up = mm;
            else return no(__LINE__);
        }
        if (!gate || !up || gate->ne[0] != up->ne[0]) return no(__LINE__);
        b.mm[0] = gate; b.mm[1] = up;
        const ggml_tensor * m3 = sole_user(b.silu, GGML_OP_MUL);
        if (!m3 || m3 != sole_user(up, GGML_OP_MUL) || !is_vec(m3) || !t_contiguous(m3)) return no(__LINE__);
        const ggml_tensor * r0 = root_of(m3->src[0]), * r1 = root_of(m3->src[1]);
        if (!((r0 == b.silu && r1 == up) || (r0 == up && r1 == b.silu))) return no(__LINE__);
        b.mul3 = m3;
        const ggml_tensor * down = sole_user(m3, GGML_OP_MUL_MAT);
        if (!down || root_of(down->src[1]) != m3 || !weight_ok(down, m3->ne[0])) return no(__LINE__);
        b.down = down;
        return true;
    }

    // marks the nodes of block b as consumed; false if one of them is not available
    bool claim(const Block & b) {
        const ggml_tensor * all[] = {b.add, b.rn, b.mu, b.mm[0], b.mm[1], b.mm[2], b.rope_q, b.rope_k, b.cpy_k, b.cpy_v, b.fa, b.chain[0], b.chain[1], b.chain[2], b.chain[3],
                                     b.wo, b.silu, b.mul3, b.down};
        for (const ggml_tensor * t : all) if (t && !take(t)) return no(__LINE__);
        return true;
    }

    // the block that continues after tensor `out` (the result of wo / down): its residual ADD
    int next_head(const ggml_tensor * out) const {
        const std::vector<int> & u = users_of(out);
        if (u.size() != 1 || g->nodes[u[0]]->op != GGML_OP_ADD) return -1;
        return u[0];
    }

    void run() {
        index();
        int at = i0;
        for (;;) {
            Block b;
            const std::vector<uint8_t> taken_before = taken;
            const int last_before = last;
            bool ok = match_head(at, b);
            if (ok && b.kind == 0) ok = match_attention(b);
            else if (ok && b.kind == 1) ok = match_ffn(b);
            if (ok && n_matvec + (b.kind == 2 ? 1 : 2) > decode_step_max_matvecs(0)) ok = false;   // the rest goes into the next launch
            if (ok) ok = claim(b);
            if (ok) n_matvec += b.kind == 2 ? 1 : 2;
            if (!ok) { taken = taken_before; last = last_before; break; }
            blocks.push_back(b);
            if (b.kind == 2 || (int) blocks.size() >= ctx->mega_max_blocks) break;
            at = next_head(b.kind == 0 ? b.wo : b.down);
            if (at < 0) break;
        }
        // a feed-forward block reads the residual sum of the attention block before it: the plan is cut after a
        // feed-forward (or output) block only when what follows is missing, never in the middle of the range check
    }

    bool visible(const ggml_tensor * t) const {
        if (t->flags & GGML_TENSOR_FLAG_OUTPUT) return true;
        const std::vector<int> & u = users_of(t);
        if (u.empty()) return true;
        for (int i : u) if (!taken[(size_t) i]) return true;
        return false;
    }
};

void * mega_arena(BackendCtx * ctx) {
    if (ctx->mega_arena) return ctx->mega_arena;
    if (ctx->capturing) return nullptr;
    B200_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
    B200_CUDA_CHECK(cudaMalloc(&ctx->mega_arena, MEGA_ARENA_BYTES));
    B200_CUDA_CHECK(cudaMemset(ctx->mega_arena, 0, MEGA_ARENA_BYTES));
    B200_CUDA_CHECK(cudaStreamCreateWithFlags(&ctx->mega_copy_stream, cudaStreamNonBlocking));
    return ctx->mega_arena;
}

}  // namespace

// Covers the nodes from `i` on with one persistent launch when they are a run of Llama blocks for a single
// token.  Returns the index one past the last covered node, or 0 when nothing was launched.
int try_decode_step(BackendCtx * ctx, ggml_cgraph * g, int i) {
    const ggml_tensor * n0 = g->nodes[i];
    if ((n0->op != GGML_OP_ADD && n0->op != GGML_OP_RMS_NORM) || !is_vec(n0)) return 0;
    Matcher m{ctx, g, i};
    m.run();
    if (ctx->trace > 0) fprintf(stderr, "ggml-b200 trace: decode-step match at node %d (%s): %zu blocks, stopped by the check at decode_plan.cpp:%d\n", i, n0->name, m.blocks.size(), m.why_line);
    // worth a launch from two whole layers on
    if ((int) m.blocks.size() < (ctx->mega_max_blocks < 4 ? ctx->mega_max_blocks : 4)) return 0;
    // Every executable node inside the covered range must belong to the plan.  libllama's node order also puts
    // nodes there that only prepare inputs (the F32 -> F16 cast of the attention mask sits between the first
    // layer's cache stores and its attention): a copy or row gather whose operands are produced outside the range
    // (or by another such node) runs ahead of the persistent launch.  It writes its own tensor, which the
    // allocator keeps apart from everything still live at its original position.
    std::vector<int> hoisted;
    for (int j = i; j <= m.last; ++j) {
        if (!m.exec(j) || m.taken[(size_t) j] || ctx->node_done[(size_t) j]) continue;
        const ggml_tensor * n = g->nodes[j];
        // an identity row selection is skipped when everything that reads it is inside the plan
        if (is_identity_rows(n) && !(n->flags & GGML_TENSOR_FLAG_OUTPUT) && !m.visible(root_of(n))) { m.taken[(size_t) j] = 1; continue; }
        bool ok = n->op == GGML_OP_CPY || n->op == GGML_OP_CONT || n->op == GGML_OP_DUP || n->op == GGML_OP_GET_ROWS;
        if (ok && n->op == GGML_OP_CPY && n->src[1] && n->src[1]->view_src) ok = false;          // stores into views (the KV cache) stay in order
        for (int s_ = 0; s_ < GGML_MAX_SRC && ok; ++s_) {
            if (!n->src[s_] || n->src[s_] == n) continue;                  // (a cast names itself as its destination operand)
            const int ri = m.idx(root_of(n->src[s_]));
            if (ri >= i && std::find(hoisted.begin(), hoisted.end(), ri) == hoisted.end()) ok = false;
        }
        if (!ok) { if (ctx->trace > 0) fprintf(stderr, "ggml-b200 trace: node %d (%s) inside the range is not part of the plan\n", j, n->name); return 0; }
        hoisted.push_back(j);
    }
    char * arena = (char *) mega_arena(ctx);
    if (!arena) return 0;
    const LaunchCtx lc = ctx->launch_ctx();

    float * vec[MEGA_N_VEC];
    for (int v = 0; v < MEGA_N_VEC; ++v) vec[v] = (float *) (arena + MEGA_OFF_VEC) + (size_t) v * MEGA_VEC_FLOATS;
    enum { V_X0 = 0, V_X1, V_X2, V_Q, V_AO, V_WO, V_ACT, V_DN, V_SPARE };
    int x_rot = 0;

    // where the value of a tensor is found by later phases
    std::unordered_map<const ggml_tensor *, float *> where;
    auto loc_of = [&](const ggml_tensor * t) -> const float * {
        const ggml_tensor * r = root_of(t);
        auto it = where.find(r);
        return it != where.end() ? it->second : (const float *) r->data;
    };
    auto place = [&](const ggml_tensor * t, float * scratch) -> float * {
        float * p = m.visible(t) ? (float *) t->data : scratch;
        where[t] = p;
        return p;
    };
    auto opt_out = [&](const ggml_tensor * t) -> float * { return m.visible(t) ? (float *) t->data : nullptr; };

    // byte offsets of the KV-cache stores: immediate, or (while capturing) slots of the per-token table in graph order
    std::vector<int> dyn_ord;
    if (ctx->capturing) {
        dyn_ord.assign((size_t) g->n_nodes + 1, 0);
        int c = 0;
        for (int j = 0; j < g->n_nodes; ++j) {
            dyn_ord[(size_t) j] = c;
            const ggml_tensor * n = g->nodes[j];
            if (t_empty(n) || n->op != GGML_OP_CPY) continue;
            const ggml_tensor * out = n->src[1];
            if (out && out->view_src && out->view_src->data) ++c;
        }
        dyn_ord[(size_t) g->n_nodes] = c;
        if (dyn_ord[(size_t) i] != ctx->dyn_used || dyn_ord[(size_t) m.last + 1] > BackendCtx::DYN_CAP) return 0;
    }

    std::vector<DsOp> ops;
    size_t partial_need = 0;
    for (const Block & b : m.blocks) {
        if (m.visible(b.rn) && b.rn->data != b.mu->data) return 0;       // the plain norm is never materialised
        DsOp o; memset(&o, 0, sizeof(o));
        o.kind = DS_OP_MATVEC; o.in_kind = DS_IN_NORM; o.K = (int) b.rn->ne[0];
        if (b.add) {
            o.in0 = loc_of(b.add->src[0]); o.in1 = loc_of(b.add->src[1]);
            o.sum_out = place(b.add, vec[V_X0 + x_rot]); x_rot = (x_rot + 1) % 3;
        } else {
            o.in0 = loc_of(b.rn->src[0]);
        }
        const ggml_tensor * w = root_of(b.mu->src[0]) == b.rn ? b.mu->src[1] : b.mu->src[0];
        o.norm_w = (const float *) w->data; o.eps = op_param_f32(b.rn, 0);
        o.y_out = opt_out(b.mu);
        o.nmat = b.kind == 0 ? 3 : (b.kind == 1 ? 2 : 1);
        for (int k = 0; k < o.nmat; ++k) {
            const ggml_tensor * W = b.mm[k]->src[0];
            o.W[k] = W->data; o.type[k] = (int) W->type; o.M[k] = (int) W->ne[1]; o.w_nb1[k] = (int64_t) W->nb[1];
        }
        if (b.kind == 0) {
            o.epilogue = DS_EP_ROPE_KV;
            for (int k = 0; k < 3; ++k) o.dst[k] = opt_out(b.mm[k]);
            o.q_rope = place(b.rope_q, vec[V_Q]); o.k_rope = opt_out(b.rope_k);
            const ggml_tensor * ko = b.cpy_k->src[1], * vo = b.cpy_v->src[1];
            o.k_cache = ko->view_src->data; o.v_cache = vo->view_src->data;
            o.k_off = (const char *) ko->data - (const char *) ko->view_src->data;
            o.v_off = (const char *) vo->data - (const char *) vo->view_src->data;
            if (ctx->capturing) {
                const int sk = dyn_ord[(size_t) b.cpy_k_idx], sv = dyn_ord[(size_t) b.cpy_v_idx];
                ctx->dyn_host[sk] = o.k_off; o.k_off_dev = ctx->dyn_dev + sk;
                ctx->dyn_host[sv] = o.v_off; o.v_off_dev = ctx->dyn_dev + sv;
            }
            const ggml_tensor * rq = b.rope_q;
            o.pos = (const int32_t *) rq->src[1]->data; o.ff = rq->src[2] ? (const float *) rq->src[2]->data : nullptr;
            o.head_dim = (int) rq->ne[0]; o.n_dims = op_param_i32(rq, 1);
            const float freq_base = op_param_f32(rq, 5), beta_fast = op_param_f32(rq, 9), beta_slow = op_param_f32(rq, 10);
            const int n_ctx_orig = op_param_i32(rq, 4);
            o.freq_scale = op_param_f32(rq, 6); o.ext_factor = op_param_f32(rq, 7); o.attn_factor = op_param_f32(rq, 8);
            o.theta_scale = powf(freq_base, -2.0f / (float) o.n_dims);
            // correction range of YaRN (ggml_rope_yarn_corr_dims, ggml/src/ggml.c), as launch_rope does
            auto corr_dim = [&](float n_rot) {
                return (float) o.n_dims * logf((float) n_ctx_orig / (n_rot * 2.0f * 3.14159265358979323846f)) / (2.0f * logf(freq_base));
            };
            o.corr0 = fmaxf(0.0f, floorf(corr_dim(beta_fast)));
            o.corr1 = fminf((float) o.n_dims - 1.0f, ceilf(corr_dim(beta_slow)));
            o.v_t = b.v_t ? 1 : 0; o.v_nbd = b.v_nbd;
            if (!b.v_t) {
                const ggml_tensor * K = b.att_K, * V = b.att_V;
                const int64_t kb = (int64_t) K->ne[1] * (int64_t) K->nb[1];
                if ((int64_t) K->nb[2] * K->ne[2] == (int64_t) K->nb[1] && (int64_t) V->nb[2] * V->ne[2] == (int64_t) V->nb[1] && K->nb[1] == V->nb[1] &&
                    kb <= ((int64_t) 8 << 20) && kb % 16 == 0) {
                    o.pf_k = (const char *) K->data; o.pf_v = (const char *) V->data; o.pf_bytes = kb;
                }
            }
            ops.push_back(o);

            DsOp a; memset(&a, 0, sizeof(a));
            const ggml_tensor * K = b.att_K, * V = b.att_V, * mask = b.att_mask;
            a.kind = DS_OP_ATTN;
            a.v_t = b.v_t ? 1 : 0; a.v_nbd = b.v_nbd; a.mask_f32 = mask && mask->type == GGML_TYPE_F32 ? 1 : 0;
            a.q = o.q_rope;
            a.k = (const char *) K->data; a.k_nb1 = (int64_t) K->nb[1]; a.k_nb2 = (int64_t) K->nb[2];
            a.v = (const char *) V->data; a.v_nb1 = (int64_t) V->nb[1]; a.v_nb2 = (int64_t) V->nb[2];
            a.mask = mask ? mask->data : nullptr;
            a.n_kv = (int) K->ne[1]; a.n_head = (int) rq->ne[1]; a.n_head_kv = (int) K->ne[2];
            a.scale = b.att_scale;
            int slices = (a.n_kv + ctx->mega_keys_per_slice - 1) / ctx->mega_keys_per_slice;     // short contexts are latency, not bandwidth: few keys per warp
            const int max_slices = lc.sm_count / a.n_head_kv;
            if (slices > max_slices) slices = max_slices;
            if (slices < 1) slices = 1;
            a.n_slices = slices; a.kv_per_slice = ((a.n_kv + slices - 1) / slices + 3) & ~3;     // (multiples of 4 keys: 8-byte runs of a transposed V row)
            a.partials = (float *) (arena + MEGA_OFF_PARTIALS); a.tickets = (unsigned *) (arena + MEGA_OFF_TICKETS);
            const size_t pn = (size_t) a.n_head_kv * slices * (size_t) (a.n_head / a.n_head_kv) * DS_PARTIAL_STRIDE * 4;
            a.consumer_merge = slices > 1 && slices <= ctx->mega_consumer_merge && slices <= DS_MAX_MERGE_SLICES;                   // few slices: the wo phase merges them while it builds its input
            if (pn > partial_need) partial_need = pn;
            a.out = place(b.att_out, vec[V_AO]);
            ops.push_back(a);

            DsOp c; memset(&c, 0, sizeof(c));
            c.kind = DS_OP_MATVEC; c.in_kind = DS_IN_PLAIN; c.K = (int) b.wo->src[0]->ne[0]; c.nmat = 1; c.epilogue = DS_EP_STORE;
            c.in0 = a.out;
            if (a.consumer_merge) {
                c.in_kind = DS_IN_ATTN; c.in0 = a.partials; c.in_slices = a.n_slices; c.in_gqa = a.n_head / a.n_head_kv;
                c.y_out = m.visible(b.att_out) ? (float *) b.att_out->data : nullptr;
            }
            const ggml_tensor * W = b.wo->src[0];
            c.W[0] = W->data; c.type[0] = (int) W->type; c.M[0] = (int) W->ne[1]; c.w_nb1[0] = (int64_t) W->nb[1];
            c.dst[0] = place(b.wo, vec[V_WO]);
            ops.push_back(c);
        } else if (b.kind == 1) {
            o.epilogue = DS_EP_SILU_MUL;
            o.dst[0] = opt_out(b.mm[0]); o.dst[1] = opt_out(b.mm[1]); o.silu_out = opt_out(b.silu);
            o.act_out = place(b.mul3, vec[V_ACT]);
            ops.push_back(o);
            DsOp c; memset(&c, 0, sizeof(c));
            c.kind = DS_OP_MATVEC; c.in_kind = DS_IN_PLAIN; c.K = (int) b.down->src[0]->ne[0]; c.nmat = 1; c.epilogue = DS_EP_STORE;
            c.in0 = o.act_out;
            const ggml_tensor * W = b.down->src[0];
            c.W[0] = W->data; c.type[0] = (int) W->type; c.M[0] = (int) W->ne[1]; c.w_nb1[0] = (int64_t) W->nb[1];
            c.dst[0] = place(b.down, vec[V_DN]);
            ops.push_back(c);
        } else {
            o.epilogue = DS_EP_STORE;
            o.dst[0] = place(b.mm[0], vec[V_SPARE]);
            if ((size_t) o.M[0] > MEGA_VEC_FLOATS && o.dst[0] == vec[V_SPARE]) return 0;
            ops.push_back(o);
        }
    }
    if ((int) ops.size() > MEGA_MAX_OPS || partial_need > MEGA_PARTIAL_BYTES) return 0;
    int n_mv = 0;
    for (const DsOp & o : ops) {
        if (o.kind != DS_OP_MATVEC) continue;
        ++n_mv;
        if (o.K > (int) MEGA_VEC_FLOATS || o.K > decode_step_max_k()) return 0;
        for (int k = 0; k < o.nmat; ++k) if ((size_t) o.M[k] > MEGA_VEC_FLOATS && o.epilogue != DS_EP_STORE) return 0;
    }
    if (n_mv > decode_step_max_matvecs(lc.device)) return 0;
    // A tensor the first phase writes at its own address must not alias what that phase reads from outside: the
    // CTAs of a phase are not ordered among themselves.  (Later phases read only scratch or tensors written
    // at least one grid barrier earlier.)
    {
        const Block & b0 = m.blocks[0];
        const ggml_tensor * ext[2] = {root_of(b0.add ? b0.add->src[0] : b0.rn->src[0]), b0.add ? root_of(b0.add->src[1]) : nullptr};
        const ggml_tensor * outs[] = {b0.add, b0.mu, b0.mm[0], b0.mm[1], b0.mm[2], b0.rope_q, b0.rope_k, b0.silu, b0.mul3};
        for (const ggml_tensor * t : outs) {
            if (!t || !m.visible(t)) continue;
            for (const ggml_tensor * e : ext) {
                if (!e) continue;
                const char * a0 = (const char *) t->data, * e0 = (const char *) e->data;
                if (a0 < e0 + t_nbytes(e) && e0 < a0 + t_nbytes(t)) return 0;
            }
        }
    }

    for (int j : hoisted) {
        if (!run_single_node(ctx, g, j)) return 0;
        ctx->node_done[(size_t) j] = 1;
    }
    // Phase lists and descriptors live in the arena: region 0 for direct runs, region 1 for the launches recorded
    // in the CUDA graph; every plan of one graph takes its own part of the region (a graph matched in pieces has
    // several), and the part is rewritten only when the graph is run directly / captured again.
    if (ctx->mega_ops_used + (int) ops.size() > MEGA_MAX_OPS) return 0;
    char * region = arena + MEGA_OFF_OPS + (ctx->capturing ? MEGA_OPS_REGION : 0);
    DsOp * ops_dev = (DsOp *) region + ctx->mega_ops_used;
    void * work = region + (size_t) MEGA_MAX_OPS * sizeof(DsOp) + (size_t) ctx->mega_ops_used * MEGA_WORK_PER_OP;
    if (!ctx->capturing && ctx->mega_ops_used == 0) B200_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));   // an earlier direct run may still read region 0
    ctx->mega_ops_used += (int) ops.size();
    if (cudaMemcpyAsync(ops_dev, ops.data(), ops.size() * sizeof(DsOp), cudaMemcpyHostToDevice, ctx->mega_copy_stream) != cudaSuccess ||
        decode_step_prepare(ops.data(), (int) ops.size(), lc.sm_count, work, ctx->mega_copy_stream) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    const cudaError_t e = launch_decode_step(ops_dev, ops.data(), (int) ops.size(), work, (unsigned *) (arena + MEGA_OFF_SYNC), lc,
                                             ctx->mega_timing ? (unsigned long long *) (arena + MEGA_OFF_TIMING) : nullptr);
    if (e != cudaSuccess) {
        cudaGetLastError();
        B200_LOG_WARN("ggml-b200: persistent decode step not launched (%s), using one launch per node\n", cudaGetErrorString(e));
        ctx->use_mega = 0;
        if (ctx->capturing) ctx->capture_failed = true;
        return 0;
    }
    ctx->n_launches++; ctx->n_mega++; ctx->mega_last_ops = (int) ops.size();
    if (ctx->capturing) ctx->dyn_used = dyn_ord[(size_t) m.last + 1];
    for (int j = i; j <= m.last; ++j) if (m.taken[(size_t) j]) ctx->node_done[(size_t) j] = 1;
    ctx->act_cache_clear();
    if (ctx->trace > 0)
        fprintf(stderr, "ggml-b200 trace: nodes %d..%d as one persistent decode step: %zu blocks, %zu phases\n", i, m.last, m.blocks.size(), ops.size());
    return m.last + 1;
}


// GGML_B200_MEGA_TIMING=1: prints, for the most recent persistent launch, what CTA 0 measured per phase
void decode_step_print_timing(BackendCtx * ctx) {
    if (!ctx->mega_timing || !ctx->mega_arena || ctx->mega_last_ops <= 0) return;
    std::vector<unsigned long long> t((size_t) ctx->mega_last_ops * 4);
    if (cudaMemcpy(t.data(), (char *) ctx->mega_arena + MEGA_OFF_TIMING, t.size() * 8, cudaMemcpyDeviceToHost) != cudaSuccess) { cudaGetLastError(); return; }
    fprintf(stderr, "ggml-b200: persistent decode step, per phase (ns, CTA 0): start-of-phase offset | input stage | rows | barrier\n");
    for (int i = 0; i < ctx->mega_last_ops; ++i) {
        const unsigned long long * q = &t[(size_t) i * 4];
        fprintf(stderr, "  phase %3d  +%8llu | %6llu | %6llu | %6llu\n", i, q[0] - t[0], q[1] - q[0], q[2] - q[1], q[3] - q[2]);
    }
}

}  // namespace b200
