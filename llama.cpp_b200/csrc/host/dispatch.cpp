// supports_op and graph_compute of the B200 backend: walks a ggml cgraph
// (struct ggml_cgraph, ggml/src/ggml-impl.h:287-300) node by node on the
// backend's stream and launches the sm_100a kernels.  Replaces the reference's
// ggml_backend_cuda_graph_compute / ggml_cuda_compute_forward
// (ggml/src/ggml-cuda/ggml-cuda.cu:2094-2311, :2691-2765) and its capability
// table (:2936-3215).  View-only ops and empty tensors are skipped as the
// reference does (:2632-2637).  An op is either executed here or rejected by
// supports_op so the scheduler routes it elsewhere; nothing runs on the host.
#include "backend.h"
#include "ggml-impl.h"

namespace b200 {

static int unary_to_unop(int u) {
    switch (u) {
        case GGML_UNARY_OP_SILU:        return UN_SILU;
        case GGML_UNARY_OP_GELU:        return UN_GELU;
        case GGML_UNARY_OP_GELU_QUICK:  return UN_GELU_QUICK;
        case GGML_UNARY_OP_RELU:        return UN_RELU;
        case GGML_UNARY_OP_TANH:        return UN_TANH;
        case GGML_UNARY_OP_SIGMOID:     return UN_SIGMOID;
        case GGML_UNARY_OP_NEG:         return UN_NEG;
        case GGML_UNARY_OP_EXP:         return UN_EXP;
        case GGML_UNARY_OP_ABS:         return UN_ABS;
        case GGML_UNARY_OP_SGN:         return UN_SGN;
        case GGML_UNARY_OP_STEP:        return UN_STEP;
        case GGML_UNARY_OP_ELU:         return UN_ELU;
        case GGML_UNARY_OP_HARDSIGMOID: return UN_HARDSIGMOID;
        case GGML_UNARY_OP_HARDSWISH:   return UN_HARDSWISH;
        default: return -1;
    }
}
static bool is_float_type(int t) { return t == GGML_TYPE_F32 || t == GGML_TYPE_F16 || t == GGML_TYPE_BF16; }

// ---------------------------------------------------------------------------
// capability table
// ---------------------------------------------------------------------------
bool device_supports_op(DeviceCtx * dev, const ggml_tensor * op) {
    (void) dev;
    // tensors in a split buffer can only be the weight operand of MUL_MAT
    for (int i = 0; i < GGML_MAX_SRC; ++i) {
        const ggml_tensor * s = op->src[i];
        if (s && s->buffer && buft_is_split(s->buffer->buft) && !(op->op == GGML_OP_MUL_MAT && i == 0)) return false;
    }
    // ... of a plain 2-D product on contiguous F32 activations (the reference's split path has the same limits:
    // ggml/src/ggml-cuda/ggml-cuda.cu:3028-3040)
    if (op->op == GGML_OP_MUL_MAT && op->src[0] && op->src[0]->buffer && buft_is_split(op->src[0]->buffer->buft)) {
        const ggml_tensor * w = op->src[0], * x = op->src[1];
        if (w->ne[2] != 1 || w->ne[3] != 1 || x->ne[2] != 1 || x->ne[3] != 1 || x->type != GGML_TYPE_F32 || !t_contiguous(x) || !t_contiguous(op)) return false;
    }
    const ggml_tensor * a = op->src[0];
    const ggml_tensor * b = op->src[1];
    switch (op->op) {
        case GGML_OP_NONE: case GGML_OP_RESHAPE: case GGML_OP_VIEW: case GGML_OP_PERMUTE: case GGML_OP_TRANSPOSE:
            return true;
        case GGML_OP_MUL_MAT: {
            if (op->type != GGML_TYPE_F32) return false;
            if (a->ne[0] != b->ne[0]) return false;
            if (is_float_type(a->type)) return b->type == GGML_TYPE_F32 || b->type == GGML_TYPE_F16;
            if (!mmvq_type_supported(a->type)) return false;
            if (b->type != GGML_TYPE_F32 || b->nb[0] != sizeof(float)) return false;
            if (a->nb[0] != t_size(a->type) || a->ne[0] % t_blck(a->type) != 0) return false;
            if (a->nb[1] % 2 || a->nb[2] % 2 || a->nb[3] % 2 || ((uintptr_t) a->data % 2)) return false;
            return true;
        }
        case GGML_OP_MUL_MAT_ID: {
            const ggml_tensor * ids = op->src[2];
            if (op->type != GGML_TYPE_F32 || !mmvq_type_supported(a->type)) return false;
            if (b->type != GGML_TYPE_F32 || b->nb[0] != sizeof(float) || ids->type != GGML_TYPE_I32) return false;
            return a->ne[0] % t_blck(a->type) == 0 && ids->nb[0] == sizeof(int32_t);
        }
        case GGML_OP_FLASH_ATTN_EXT: {
            const ggml_tensor * v = op->src[2];
            const ggml_tensor * mask = op->src[3];
            if (a->type != GGML_TYPE_F32 || op->type != GGML_TYPE_F32) return false;
            if (!fattn_supported(a->ne[0], b->type, v->type) || v->ne[0] != a->ne[0] || b->ne[0] != a->ne[0]) return false;
            if (a->nb[0] != 4 || b->nb[0] != t_size(b->type) || v->nb[0] != t_size(v->type)) return false;
            if (mask && (mask->type != GGML_TYPE_F16 || mask->nb[0] != 2)) return false;
            return true;
        }
        case GGML_OP_RMS_NORM: case GGML_OP_NORM:
            return a->type == GGML_TYPE_F32 && op->type == GGML_TYPE_F32 && a->nb[0] == 4 && t_contiguous(op);
        case GGML_OP_ADD: case GGML_OP_SUB: case GGML_OP_MUL: case GGML_OP_DIV: {
            auto ok = [](int t) { return t == GGML_TYPE_F32 || t == GGML_TYPE_F16; };
            return ok(a->type) && ok(b->type) && ok(op->type) && t_can_repeat(b, a);
        }
        case GGML_OP_UNARY:
            return unary_to_unop(op_param_i32(op, 0)) >= 0 && a->type == GGML_TYPE_F32 && op->type == GGML_TYPE_F32 &&
                   t_contiguous(a) && t_contiguous(op);
        case GGML_OP_SQR: case GGML_OP_SQRT: case GGML_OP_SIN: case GGML_OP_COS: case GGML_OP_LOG:
        case GGML_OP_SCALE: case GGML_OP_CLAMP:
            return a->type == GGML_TYPE_F32 && op->type == GGML_TYPE_F32 && t_contiguous(a) && t_contiguous(op);
        case GGML_OP_ROPE: {
            const int mode = op_param_i32(op, 2);
            if (mode & (GGML_ROPE_TYPE_MROPE | GGML_ROPE_TYPE_VISION) & ~GGML_ROPE_TYPE_NEOX) return false;
            if (a->type != GGML_TYPE_F32 && a->type != GGML_TYPE_F16) return false;
            return a->nb[0] == t_size(a->type) && op->nb[0] == t_size(op->type) && op->type == a->type;
        }
        case GGML_OP_CPY: case GGML_OP_DUP: case GGML_OP_CONT: {
            const int st = a->type, dt = op->op == GGML_OP_CPY ? b->type : op->type;
            if (st == dt && t_contiguous(a) && t_contiguous(op)) return true;   // plain memcpy, any type
            if (!cpy_supported(st, dt)) return false;
            if (t_quantized(dt)) return a->ne[0] % 32 == 0 && op->ne[0] % 32 == 0 && a->nb[0] == 4;
            return true;
        }
        case GGML_OP_GET_ROWS:
            return get_rows_supported(a->type) && b->type == GGML_TYPE_I32 && op->type == GGML_TYPE_F32 &&
                   a->nb[0] == t_size(a->type) && op->nb[0] == 4;
        case GGML_OP_SOFT_MAX: {
            if (a->type != GGML_TYPE_F32 || !t_contiguous(a) || !t_contiguous(op)) return false;
            if (b && b->type != GGML_TYPE_F16 && b->type != GGML_TYPE_F32) return false;
            return a->ne[0] * 4 <= 200 * 1024;
        }
        default:
            return false;
    }
}

// ---------------------------------------------------------------------------
// node execution
// ---------------------------------------------------------------------------
#define RUN(expr)                                                                           \
    do {                                                                                    \
        cudaError_t e_ = (expr);                                                            \
        if (e_ != cudaSuccess) {                                                            \
            B200_LOG_ERROR("ggml-b200: %s failed: %s\n", #expr, cudaGetErrorString(e_));    \
            return false;                                                                   \
        }                                                                                   \
        ctx->n_launches++;                                                                  \
    } while (0)

// the bytes a tensor spans, from its data pointer
static size_t t_extent(const ggml_tensor * t) {
    size_t e = (size_t) (t->ne[0] / t_blck(t->type)) * t->nb[0];
    for (int d = 1; d < 4; ++d) e += (size_t) (t->ne[d] > 0 ? t->ne[d] - 1 : 0) * t->nb[d];
    return e;
}
static void invalidate_written(BackendCtx * ctx, const ggml_tensor * t) { if (t && t->data) ctx->act_cache_invalidate(t->data, t_extent(t)); }

// can the int8 activation blocks of X be produced/kept in the per-graph cache?
static bool act_cacheable(const ggml_tensor * X) {
    return X->type == GGML_TYPE_F32 && t_contiguous(X) && X->ne[1] * X->ne[2] * X->ne[3] <= 8;
}

// ---- row-split over processes (include/ggml-b200.h) ----
// byte distances from this rank's arena to each peer's mapping of its own arena
static int peer_deltas(const BackendCtx * ctx, int64_t * delta) {
    int n = 0;
    const char * mine = (const char *) ctx->peers.arena[ctx->peers.rank];
    for (int r = 0; r < ctx->peers.n_ranks; ++r) if (r != ctx->peers.rank) delta[n++] = (const char *) ctx->peers.arena[r] - mine;
    return n;
}
static bool in_arena(const BackendCtx * ctx, const void * p, size_t bytes) {
    const char * mine = (const char *) ctx->peers.arena[ctx->peers.rank];
    return (const char *) p >= mine + GGML_B200_PEER_FLAG_BYTES && (const char *) p + bytes <= mine + ctx->peers.arena_bytes;
}
// stores the [ne0 x ne1] slice `dst` into the same place of every peer's arena
static bool push_slice(BackendCtx * ctx, const ggml_tensor * dst) {
    PeerPush p = {};
    int64_t delta[MAX_PEERS - 1];
    p.n_peer = peer_deltas(ctx, delta);
    p.src = (const char *) dst->data;
    for (int i = 0; i < p.n_peer; ++i) p.peer_dst[i] = (char *) dst->data + delta[i];
    p.col_bytes = dst->ne[0] * 4; p.col_stride = (int64_t) dst->nb[1]; p.ncols = dst->ne[1];
    p.shift = (p.col_bytes % 16 == 0 && p.col_stride % 16 == 0 && (uintptr_t) dst->data % 16 == 0) ? 4 : 2;
    RUN(launch_peer_push(p, ctx->launch_ctx()));
    return true;
}
static bool peer_barrier(BackendCtx * ctx) {
    PeerBarrier b = {};
    char * mine = (char *) ctx->peers.arena[ctx->peers.rank];
    b.local_flags = (unsigned *) mine; b.epoch = (unsigned *) (mine + 64);
    for (int r = 0; r < ctx->peers.n_ranks; ++r) b.peer_flags[r] = (unsigned *) ctx->peers.arena[r];
    b.rank = ctx->peers.rank; b.n_ranks = ctx->peers.n_ranks; b.status = ctx->status_dev; b.spin_limit = ctx->peer_spin_limit;
    RUN(launch_peer_barrier(b, ctx->launch_ctx()));
    ctx->peer_pending = false;
    return true;
}

// A few activation columns of a plain 2-D Q4_K / Q8_0 MUL_MAT go to the integer tensor-core kernel (mmq_s8.cu), not to the
// tcgen05 GEMM; row-sliced results (several GPUs) keep their path
static bool s8_takes(const BackendCtx * ctx, const ggml_tensor * n) {
    const ggml_tensor * W = n->src[0], * X = n->src[1];
    if (!W || !X || X->ne[2] != 1 || X->ne[3] != 1 || W->ne[2] != 1 || W->ne[3] != 1) return false;
    if (!mmq_s8_shape_ok(W->type, X->ne[1], W->ne[0]) || ((uintptr_t) W->data & 15) || (W->nb[1] & 15) || (n->nb[1] & 3)) return false;
    return ctx->row_slice_of(n) == nullptr;
}

static bool run_mul_mat(BackendCtx * ctx, const ggml_tensor * dst, const ggml_tensor * ids, ggml_tensor * const * extra = nullptr, int n_extra = 0) {
    const ggml_tensor * W = dst->src[0];
    const ggml_tensor * X = dst->src[1];
    const LaunchCtx lc = ctx->launch_ctx();
    const bool sliced = !ids && ctx->row_slice_of(dst) != nullptr;
    if (sliced) {
        const size_t span = (size_t) (dst->ne[1] - 1) * dst->nb[1] + (size_t) dst->ne[0] * 4;
        if (dst->ne[2] != 1 || dst->ne[3] != 1 || !in_arena(ctx, dst->data, span)) {
            B200_LOG_ERROR("ggml-b200: row-sliced MUL_MAT %s lies outside the peer arena or has batch dims\n", dst->name);
            return false;
        }
        ctx->peer_pending = true;
        ctx->pending_full.push_back(ctx->row_slice_of(dst)->full_data);
        ctx->act_cache_invalidate(ctx->row_slice_of(dst)->full_data, (size_t) (dst->ne[1] - 1) * dst->nb[1] + (size_t) ctx->row_slice_of(dst)->full_rows * 4);
        for (int i = 0; i < n_extra; ++i) if (const ggml_b200_row_slice * r2 = ctx->row_slice_of(extra[i])) {
            ctx->pending_full.push_back(r2->full_data);
            ctx->act_cache_invalidate(r2->full_data, (size_t) (extra[i]->ne[1] - 1) * extra[i]->nb[1] + (size_t) r2->full_rows * 4);
        }
    }
    if (!ids && is_float_type(W->type)) {
        // 16-bit weight matrices with plain 2-D operands: warp-per-row mat-vec (at most 8 columns) or the tcgen05 GEMM
        const TensorD wd = to_desc(W), xd = to_desc(X), dd = to_desc(dst);
        if (mv16_applicable(wd, xd, dd)) {
            RUN(launch_mv16(wd, xd, dd, lc));
        } else if (ctx->use_tc && mm16_tc_applicable(wd, xd, dd)) {
            void * ws = ctx->get_scratch(mm16_tc_workspace_bytes(X->ne[1], W->ne[0]));
            if (ctx->capture_failed) return false;
            RUN(launch_mm16_tc(wd, xd, dd, ws, lc));
            ctx->n_launches++;
        } else
        RUN(launch_matmul_f(to_desc(W), to_desc(X), to_desc(dst), lc));
        if (sliced && !push_slice(ctx, dst)) return false;
        return true;
    }
    const int64_t K = W->ne[0], M = W->ne[1];
    const int64_t ne11 = X->ne[1], ne12 = X->ne[2], ne13 = X->ne[3];
    if (!ids && ctx->use_tc && !s8_takes(ctx, dst) && mmq_tc_supported(W->type, M, ne11, K) && mmq_tc_ptr_ok(W->type, W->data, W->nb[1], X->data, X->nb[1]) &&
        W->nb[2] % 16 == 0 && W->nb[3] % 16 == 0 && X->nb[2] % 8 == 0 && X->nb[3] % 8 == 0) {
        // prefill: tensor-core GEMM per 2-D slice (weights broadcast over the batch dims).  The F16 copy of the
        // activations is kept for the next mat-mul that reads the same tensor (wq/wk/wv, gate/up).
        const size_t need = mmq_tc_workspace_bytes(ne11, K);
        const bool single = ne12 * ne13 == 1;
        void * ws = nullptr;
        bool have = false;
        if (single) {
            if (need > ctx->tc_xh_cap) {
                B200_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
                if (ctx->tc_xh) B200_CUDA_CHECK(cudaFree(ctx->tc_xh));
                size_t cap = ctx->tc_xh_cap ? ctx->tc_xh_cap : (size_t) 4 << 20;
                while (cap < need) cap *= 2;
                B200_CUDA_CHECK(cudaMalloc(&ctx->tc_xh, cap));
                ctx->tc_xh_cap = cap; ctx->tc_x_data = nullptr;
            }
            ws = ctx->tc_xh;
            have = ctx->tc_x_data == X->data && ctx->tc_x_k == K && ctx->tc_x_n == ne11;
            ctx->tc_x_data = X->data; ctx->tc_x_k = K; ctx->tc_x_n = ne11; ctx->tc_x_bytes = (size_t) K * (size_t) ne11 * 4;
        } else {
            ws = ctx->get_scratch(need);
        }
        // a grouped launch: the head and up to two more matrices of the same type and row length on the same activations
        const void * gW[3] = {W->data, nullptr, nullptr}; float * gD[3] = {(float *) dst->data, nullptr, nullptr};
        int64_t gM[3] = {M, 0, 0}, gNb[3] = {(int64_t) dst->nb[1], 0, 0};
        const int n_mats = single ? 1 + n_extra : 1;
        for (int i = 0; i < n_extra && single; ++i) {
            gW[1 + i] = extra[i]->src[0]->data; gD[1 + i] = (float *) extra[i]->data;
            gM[1 + i] = extra[i]->src[0]->ne[1]; gNb[1 + i] = (int64_t) extra[i]->nb[1];
        }
        const size_t pbytes = single ? mmq_tc_group_partial_bytes(n_mats, gM, ne11, K, lc.sm_count) : 0;     // partial tiles of the K-divided part
        void * partials = pbytes ? ctx->get_scratch(pbytes) : nullptr;
        if (ctx->capture_failed) return false;
        if (single) {
            RUN(launch_mmq_tc_group(W->type, n_mats, gW, W->nb[1], gM, gD, gNb, (const float *) X->data, X->nb[1], ne11, K, ws, lc, have, partials));
            if (partials) ctx->n_launches++;
            if (!have) ctx->n_launches++;
        } else {
            const int64_t r2 = ne12 / W->ne[2], r3 = ne13 / W->ne[3];
            for (int64_t i13 = 0; i13 < ne13; ++i13) for (int64_t i12 = 0; i12 < ne12; ++i12) {
                const char * w = (const char *) W->data + (i12 / r2) * W->nb[2] + (i13 / r3) * W->nb[3];
                const char * x = (const char *) X->data + i12 * X->nb[2] + i13 * X->nb[3];
                char * d = (char *) dst->data + i12 * dst->nb[2] + i13 * dst->nb[3];
                RUN(launch_mmq_tc(W->type, w, W->nb[1], (const float *) x, X->nb[1], (float *) d, dst->nb[1], M, ne11, K, ws, lc, false, nullptr));
                ctx->n_launches++;
            }
        }
        if (sliced && !push_slice(ctx, dst)) return false;
        return true;
    }
    if (ids && ctx->use_tc) {
        // MUL_MAT_ID over many (slot, token) pairs (a prompt through a mixture-of-experts layer): the pairs are sorted by
        // expert on the device and all experts run as one tensor-core launch; few pairs keep the per-pair mat-vec below
        const int64_t n_used = ids->ne[0], n_tok = ids->ne[1], P = n_used * n_tok, n_expert = W->ne[2];
        if (P >= 32 && W->ne[3] == 1 && X->ne[3] == 1 && mmq_tc_moe_supported(W->type, M, K, n_expert, P) &&
            mmq_tc_ptr_ok(W->type, W->data, W->nb[1], X->data, X->nb[1]) && W->nb[2] % 16 == 0 && X->nb[2] % 8 == 0 &&
            ids->nb[0] == 4 && ids->nb[1] % 4 == 0 && dst->nb[0] == 4 && dst->ne[3] == 1) {
            void * ws = ctx->get_scratch(mmq_tc_moe_workspace_bytes(P, K, n_expert));
            if (ctx->capture_failed) return false;
            RUN(launch_mmq_tc_moe(W->type, W->data, W->nb[1], W->nb[2], n_expert, M, K, (const float *) X->data, X->nb[1], X->nb[2], ne11,
                                  (const int32_t *) ids->data, ids->nb[1], n_used, n_tok, (float *) dst->data, dst->nb[1], dst->nb[2], ws, lc));
            ctx->n_launches += 2;
            return true;
        }
    }
    void * xq = nullptr;
    if (act_cacheable(X)) {
        BackendCtx::ActEntry * e = ctx->act_cache_find(X->data, K, ne11 * ne12 * ne13);
        if (!e) {
            e = ctx->act_cache_take(X->data, K, ne11 * ne12 * ne13);
            if (!e) return false;
            RUN(launch_quantize_act128((const float *) X->data, ne11, ne12, ne13, X->nb[1] / 4, X->nb[2] / 4, X->nb[3] / 4, e->q, (int) K, lc.stream, lc.use_pdl));
        }
        xq = e->q;
    } else {
        xq = ctx->get_scratch(act128_bytes(K, ne11 * ne12 * ne13));
        RUN(launch_quantize_act128((const float *) X->data, ne11, ne12, ne13, X->nb[1] / 4, X->nb[2] / 4, X->nb[3] / 4, xq, (int) K, lc.stream, lc.use_pdl));
    }

    MmvqArgs a = {};
    a.type = W->type; a.W = W->data; a.w_nb1 = W->nb[1]; a.w_nb2 = W->nb[2]; a.w_nb3 = W->nb[3];
    a.Xq = xq; a.M = (int) M; a.K = (int) K;
    a.status = lc.status; a.sm_count = lc.sm_count; a.device = lc.device;
    // the mat-vec kernels fetch weights before they wait for their predecessor: only safe when the weights
    // are not produced inside this graph
    const bool w_is_leaf = W->op == GGML_OP_NONE && (!W->view_src || W->view_src->op == GGML_OP_NONE);
    a.use_pdl = w_is_leaf ? lc.use_pdl : 0;
    for (int i = 0; i < n_extra; ++i) {             // grouped launch: more weight matrices on the same activations
        a.extra_W[i] = extra[i]->src[0]->data; a.extra_dst[i] = (float *) extra[i]->data;
        a.extra_dst_nb1[i] = extra[i]->nb[1]; a.extra_M[i] = (int) extra[i]->src[0]->ne[1];
    }
    a.n_extra = n_extra;
    if (!ids) {
        a.ne12 = (int) ne12; a.ne13 = (int) ne13;
        a.r2 = (int) (ne12 / W->ne[2]); a.r3 = (int) (ne13 / W->ne[3]);
        a.dst_nb1 = dst->nb[1]; a.dst_nb2 = dst->nb[2]; a.dst_nb3 = dst->nb[3];
        a.x_ncols = (int) ne11; a.xq_ne12 = (int) ne12;
        if (!sliced && mmq_s8_applicable(a, ne11)) {        // a few columns at once on the integer tensor-core instruction
            a.x_col0 = 0; a.N = (int) ne11; a.dst = (float *) dst->data;
            RUN(launch_mmq_s8(a, ne11, lc.stream));
            ctx->n_launches += n_extra;
            return true;
        }
        bool pushed = true;
        for (int64_t n0 = 0; n0 < ne11; n0 += 8) {
            a.N = (int) (ne11 - n0 < 8 ? ne11 - n0 : 8);
            a.x_col0 = (int) n0;
            a.dst = (float *) ((char *) dst->data + n0 * dst->nb[1]);
            a.n_peer = 0;
            if (sliced) {
                if (mmvq_stores_to_peers(a)) a.n_peer = peer_deltas(ctx, a.peer_delta);   // the kernel writes the peer copies itself
                else pushed = false;
            }
            RUN(launch_mmvq(a, lc.stream));
        }
        if (sliced && !pushed) {
            if (!push_slice(ctx, dst)) return false;
            for (int i = 0; i < n_extra; ++i) if (!push_slice(ctx, extra[i])) return false;
        }
    } else {
        // MUL_MAT_ID (ggml_mul_mat_id, ggml/src/ggml.c:2735-2759): one mat-vec per (slot e, token t),
        // the expert matrix chosen on the device from ids[e, t]; no host round trip
        const int64_t n_used = ids->ne[0], n_tok = ids->ne[1];
        a.ne12 = (int) n_used; a.ne13 = (int) n_tok; a.r2 = 1; a.r3 = 1;
        a.N = 1; a.x_col0 = 0; a.x_ncols = 1;
        a.xq_ne12 = (int) ne11;                        // src1 is [K, n_used or 1, n_tok]: dim 1 is the slot
        a.ids = (const int32_t *) ids->data; a.ids_s12 = 1; a.ids_s13 = ids->nb[1] / 4;
        a.dst = (float *) dst->data;
        a.dst_nb1 = 0; a.dst_nb2 = dst->nb[1]; a.dst_nb3 = dst->nb[2];
        RUN(launch_mmvq(a, lc.stream));
    }
    return true;
}

// does node `user` consume `t` as the activation operand of a quantized mat-mul?
static bool feeds_quant_mul_mat(const ggml_cgraph * g, int from, const ggml_tensor * t) {
    for (int i = from; i < g->n_nodes && i < from + 8; ++i) {
        const ggml_tensor * n = g->nodes[i];
        if (n->op == GGML_OP_MUL_MAT && n->src[1] == t && mmvq_type_supported(n->src[0]->type)) return true;
    }
    return false;
}

static bool is_noop(const ggml_tensor * node);

// Prefill: when `t` (F32, dense rows, more than 8 of them) is the activation operand of a tensor-core MUL_MAT a few
// nodes on, its producer also writes the F16 copy that GEMM reads; returns where to write it, or null.
static void * tc_f16_out_for(BackendCtx * ctx, const ggml_cgraph * g, int from, const ggml_tensor * t) {
    if (!ctx->use_tc || t->type != GGML_TYPE_F32 || !t_contiguous(t) || t->ne[1] <= 8 || t->ne[2] != 1 || t->ne[3] != 1) return nullptr;
    bool feeds = false;
    for (int i = from; i < g->n_nodes && i < from + 8 && !feeds; ++i) {
        const ggml_tensor * n = g->nodes[i];
        if (n->op != GGML_OP_MUL_MAT || n->src[1] != t) continue;
        const ggml_tensor * W = n->src[0];
        feeds = !is_float_type(W->type) && !s8_takes(ctx, n) && mmq_tc_supported(W->type, W->ne[1], t->ne[1], W->ne[0]) &&
                mmq_tc_ptr_ok(W->type, W->data, W->nb[1], t->data, t->nb[1]) && W->nb[2] % 16 == 0 && W->nb[3] % 16 == 0;
    }
    if (!feeds) return nullptr;
    const size_t need = mmq_tc_workspace_bytes(t->ne[1], t->ne[0]);
    if (need > ctx->tc_xh_cap) {
        if (ctx->capturing) return nullptr;
        B200_CUDA_CHECK(cudaStreamSynchronize(ctx->stream));
        if (ctx->tc_xh) B200_CUDA_CHECK(cudaFree(ctx->tc_xh));
        size_t cap = ctx->tc_xh_cap ? ctx->tc_xh_cap : (size_t) 4 << 20;
        while (cap < need) cap *= 2;
        B200_CUDA_CHECK(cudaMalloc(&ctx->tc_xh, cap));
        ctx->tc_xh_cap = cap;
    }
    ctx->tc_x_data = t->data; ctx->tc_x_k = t->ne[0]; ctx->tc_x_n = t->ne[1]; ctx->tc_x_bytes = (size_t) t->ne[0] * (size_t) t->ne[1] * 4;
    return ctx->tc_xh;
}



// do the byte ranges spanned by two tensors intersect?
static bool t_overlap(const ggml_tensor * a, const ggml_tensor * b) {
    if (!a->data || !b->data) return false;
    auto extent = [](const ggml_tensor * t) {
        size_t e = (size_t) (t->ne[0] / t_blck(t->type)) * t->nb[0];
        for (int d = 1; d < 4; ++d) e += (size_t) (t->ne[d] - 1) * t->nb[d];
        return e;
    };
    const char * a0 = (const char *) a->data, * b0 = (const char *) b->data;
    return a0 < b0 + extent(b) && b0 < a0 + extent(a);
}

// Can MUL_MAT node `n` ride along with `first` in one grouped mat-vec launch?
// MUL_MAT whose weight matrix lives in the row-split buffer type (split.cpp): every device that holds rows computes
// its slice of the result on its own stream, from its own copy of the activations, and copies the slice into the
// result on this (the main) device; this stream then waits for all of them.  The data flow of the reference's
// ggml_cuda_op_mul_mat with split weights (ggml/src/ggml-cuda/ggml-cuda.cu:1520-1660): activations out by peer copy,
// slices back by a strided peer copy, events in between.  The mat-mul itself is the ordinary path of this backend, run
// by a helper instance on each other device.
static bool run_split_mul_mat(BackendCtx * ctx, const ggml_tensor * dst) {
    const ggml_tensor * W = dst->src[0];
    const ggml_tensor * X = dst->src[1];
    const SplitExtra * e = split_extra_of(W);
    const int n_dev = (int) devices().size(), me = ctx->dev->index;
    const int64_t ncols = X->ne[1];
    const size_t xbytes = (size_t) X->ne[0] * (size_t) ncols * 4;
    auto slice_tensors = [&](int id, void * x_data, void * d_data, size_t d_nb1, ggml_tensor & Wf, ggml_tensor & Xf, ggml_tensor & Df) {
        const int64_t rows = e->row_high[id] - e->row_low[id];
        Wf = *W; Wf.data = e->data[id]; Wf.ne[1] = rows; Wf.nb[2] = Wf.nb[3] = (size_t) rows * W->nb[1]; Wf.buffer = nullptr; Wf.extra = nullptr;
        Xf = *X; Xf.data = x_data; Xf.buffer = nullptr; Xf.view_src = nullptr; Xf.extra = nullptr;
        Df = *dst; Df.data = d_data; Df.ne[0] = rows; Df.nb[1] = d_nb1; Df.nb[2] = Df.nb[3] = d_nb1 * (size_t) ncols;
        Df.src[0] = &Wf; Df.src[1] = &Xf; Df.buffer = nullptr; Df.view_src = nullptr; Df.extra = nullptr;
    };
    bool others = false;
    for (int id = 0; id < n_dev; ++id) if (id != me && e->data[id]) others = true;
    if (others) {
        if (!ctx->split_ready) B200_CUDA_CHECK(cudaEventCreateWithFlags(&ctx->split_ready, cudaEventDisableTiming));
        B200_CUDA_CHECK(cudaEventRecord(ctx->split_ready, ctx->stream));
    }
    for (int id = 0; id < n_dev; ++id) {
        if (id == me || !e->data[id]) continue;
        BackendCtx::SplitPeer & sp = ctx->split_peer[id];
        DeviceCtx * d = devices()[(size_t) id];
        B200_CUDA_CHECK(cudaSetDevice(d->device));
        if (!sp.helper) {
            sp.helper = init_backend_for(d);
            if (!sp.helper) { cudaSetDevice(ctx->dev->device); return false; }
            B200_CUDA_CHECK(cudaEventCreateWithFlags(&sp.done, cudaEventDisableTiming));
            // direct copies between the two devices where the machine allows them (the copies work either way)
            if (cudaDeviceEnablePeerAccess(ctx->dev->device, 0) != cudaSuccess) cudaGetLastError();
            cudaSetDevice(ctx->dev->device);
            if (cudaDeviceEnablePeerAccess(d->device, 0) != cudaSuccess) cudaGetLastError();
            B200_CUDA_CHECK(cudaSetDevice(d->device));
        }
        BackendCtx * h = (BackendCtx *) sp.helper->context;
        const int64_t rows = e->row_high[id] - e->row_low[id];
        const size_t dbytes = (size_t) rows * (size_t) ncols * 4;
        auto grow = [&](void *& p, size_t & cap, size_t need) {
            if (need <= cap) return;
            B200_CUDA_CHECK(cudaStreamSynchronize(h->stream));
            if (p) B200_CUDA_CHECK(cudaFree(p));
            cap = need + need / 2;
            B200_CUDA_CHECK(cudaMalloc(&p, cap + 256));
        };
        grow(sp.x, sp.x_cap, xbytes);
        grow(sp.d, sp.d_cap, dbytes);
        B200_CUDA_CHECK(cudaStreamWaitEvent(h->stream, ctx->split_ready, 0));
        B200_CUDA_CHECK(cudaMemcpyPeerAsync(sp.x, d->device, X->data, ctx->dev->device, xbytes, h->stream));
        ggml_tensor Wf, Xf, Df;
        slice_tensors(id, sp.x, sp.d, (size_t) rows * 4, Wf, Xf, Df);
        h->act_cache_clear();                       // the copy lands at the same address every time, with new contents
        const bool ok = run_mul_mat(h, &Df, nullptr);
        ctx->n_launches += 1;
        if (ok) {
            B200_CUDA_CHECK(cudaMemcpy2DAsync((char *) dst->data + (size_t) e->row_low[id] * 4, dst->nb[1], sp.d, (size_t) rows * 4,
                                              (size_t) rows * 4, (size_t) ncols, cudaMemcpyDeviceToDevice, h->stream));
            B200_CUDA_CHECK(cudaEventRecord(sp.done, h->stream));
        }
        if (!ok) { cudaSetDevice(ctx->dev->device); return false; }
    }
    B200_CUDA_CHECK(cudaSetDevice(ctx->dev->device));
    if (e->data[me]) {
        ggml_tensor Wf, Xf, Df;
        slice_tensors(me, X->data, (char *) dst->data + (size_t) e->row_low[me] * 4, dst->nb[1], Wf, Xf, Df);
        if (!run_mul_mat(ctx, &Df, nullptr)) return false;
    }
    for (int id = 0; id < n_dev; ++id) if (id != me && e->data[id]) B200_CUDA_CHECK(cudaStreamWaitEvent(ctx->stream, ctx->split_peer[id].done, 0));
    return true;
}

static bool groupable_mul_mat(const ggml_tensor * first, const ggml_tensor * n) {
    if (n->op != GGML_OP_MUL_MAT || n->src[1] != first->src[1]) return false;
    const ggml_tensor * w0 = first->src[0], * w = n->src[0];
    if (w->type != w0->type || (w->type != GGML_TYPE_Q4_K && w->type != GGML_TYPE_Q5_K)) return false;
    if (w->ne[0] != w0->ne[0] || w->nb[1] != w0->nb[1] || w->ne[2] != 1 || w->ne[3] != 1) return false;
    if (((uintptr_t) w->data & 15) || !t_contiguous(n) || n->type != GGML_TYPE_F32) return false;
    return !buft_is_split(w->buffer ? w->buffer->buft : nullptr);
}
static bool group_head_ok(const ggml_tensor * n) {
    const ggml_tensor * w = n->src[0], * x = n->src[1];
    if (w->type != GGML_TYPE_Q4_K && w->type != GGML_TYPE_Q5_K) return false;
    if (x->ne[1] > 8 || x->ne[2] != 1 || x->ne[3] != 1 || w->ne[2] != 1 || w->ne[3] != 1) return false;
    if ((size_t) x->ne[1] * ((w->ne[0] + 127) / 128) * 160 > 200 * 1024) return false;      // must fit the direct kernel's activation smem
    return ((uintptr_t) w->data & 15) == 0 && (w->nb[1] & 15) == 0 && t_contiguous(n) && x->type == GGML_TYPE_F32 && t_contiguous(x);
}
// the same for the tensor-core GEMM (more than 8 tokens): any type it takes, plain 2-D operands
static bool tc_group_ok(const BackendCtx * ctx, const ggml_tensor * n) {
    const ggml_tensor * w = n->src[0], * x = n->src[1];
    if (!ctx->use_tc || is_float_type(w->type) || x->type != GGML_TYPE_F32 || x->ne[1] <= 8) return false;
    if (x->ne[2] != 1 || x->ne[3] != 1 || w->ne[2] != 1 || w->ne[3] != 1 || n->type != GGML_TYPE_F32 || n->nb[0] != 4) return false;
    if (s8_takes(ctx, n) || !mmq_tc_supported(w->type, w->ne[1], x->ne[1], w->ne[0]) || !mmq_tc_ptr_ok(w->type, w->data, w->nb[1], x->data, x->nb[1])) return false;
    if (w->nb[2] % 16 || w->nb[3] % 16 || x->nb[2] % 8 || x->nb[3] % 8) return false;      // (what run_mul_mat asks of the tensor-core path)
    return !buft_is_split(w->buffer ? w->buffer->buft : nullptr);
}
static bool tc_groupable(const BackendCtx * ctx, const ggml_tensor * first, const ggml_tensor * n) {
    if (n->op != GGML_OP_MUL_MAT || n->src[1] != first->src[1] || !tc_group_ok(ctx, n)) return false;
    const ggml_tensor * w0 = first->src[0], * w = n->src[0];
    return w->type == w0->type && w->ne[0] == w0->ne[0] && w->nb[1] == w0->nb[1];
}
static int next_exec(const BackendCtx * ctx, const ggml_cgraph * g, int i);

// Attention as libllama builds it WITHOUT flash attention (llm_build_kqv, src/llama.cpp:601-650): kq = MUL_MAT(K, Q),
// SOFT_MAX(kq, mask, scale), kqv = MUL_MAT(V^T, p) with V kept transposed in the cache, PERMUTE, CONT.  When those five
// nodes stand in a row and nothing else reads the intermediates, they are computed as ONE flash-attention launch on the
// same operands (the score and probability matrices are never materialised): the result of CONT has exactly the
// [head size, heads, queries] layout FLASH_ATTN_EXT writes.  Returns the number of nodes consumed, 0 for no match.
struct AttnChain { const ggml_tensor * q, * k, * v, * mask; ggml_tensor * out; float scale; int last; };
static bool match_attn_chain(const BackendCtx * ctx, const ggml_cgraph * g, int i, AttnChain & m) {
    const ggml_tensor * kq = g->nodes[i];
    if (kq->op != GGML_OP_MUL_MAT || kq->type != GGML_TYPE_F32) return false;
    const ggml_tensor * k = kq->src[0], * q = kq->src[1];
    if (k->type != GGML_TYPE_F16 || q->type != GGML_TYPE_F32 || k->nb[0] != 2 || q->nb[0] != 4 || q->ne[3] != 1 || k->ne[3] != 1) return false;
    const int64_t D = q->ne[0], n_q = q->ne[1], n_head = q->ne[2], n_kv = k->ne[1], n_head_kv = k->ne[2];
    if (k->ne[0] != D || n_head_kv == 0 || n_head % n_head_kv != 0) return false;
    const int j1 = next_exec(ctx, g, i + 1);
    if (j1 < 0) return false;
    const ggml_tensor * sm = g->nodes[j1];
    if (sm->op != GGML_OP_SOFT_MAX || sm->src[0] != kq || op_param_f32(sm, 1) != 0.0f) return false;          // (ALiBi stays unfused)
    const ggml_tensor * mask = sm->src[1];
    if (mask && (mask->type != GGML_TYPE_F16 && mask->type != GGML_TYPE_F32)) return false;
    if (mask && (mask->ne[0] != n_kv || mask->ne[1] < n_q || mask->ne[2] != 1 || mask->ne[3] != 1 || !t_contiguous(mask))) return false;
    const int j2 = next_exec(ctx, g, j1 + 1);
    if (j2 < 0) return false;
    const ggml_tensor * kqv = g->nodes[j2];
    if (kqv->op != GGML_OP_MUL_MAT || kqv->src[1] != sm || kqv->type != GGML_TYPE_F32) return false;
    const ggml_tensor * v = kqv->src[0];
    if (v->type != GGML_TYPE_F16 || v->nb[0] != 2 || v->ne[0] != n_kv || v->ne[1] != D || v->ne[2] != n_head_kv || v->ne[3] != 1) return false;
    const int j4 = next_exec(ctx, g, j2 + 1);
    if (j4 < 0) return false;
    ggml_tensor * cont = g->nodes[j4];
    const ggml_tensor * perm = cont->src[0];
    if (cont->op != GGML_OP_CONT || !perm || perm->op != GGML_OP_PERMUTE || perm->src[0] != kqv || cont->type != GGML_TYPE_F32 || !t_contiguous(cont)) return false;
    // the permutation swaps queries and heads: [D, n_q, n_head] -> [D, n_head, n_q]
    if (perm->ne[0] != D || perm->ne[1] != n_head || perm->ne[2] != n_q || perm->nb[1] != kqv->nb[2] || perm->nb[2] != kqv->nb[1]) return false;
    if (cont->ne[0] * cont->ne[1] * cont->ne[2] * cont->ne[3] != D * n_head * n_q) return false;
    // nothing else may read the intermediates
    for (int j = i + 1; j < g->n_nodes; ++j) {
        const ggml_tensor * n = g->nodes[j];
        for (int s_ = 0; s_ < GGML_MAX_SRC && n->src[s_]; ++s_) {
            const ggml_tensor * t = n->src[s_];
            const ggml_tensor * root = t->view_src ? t->view_src : t;
            const bool inter = root == kq || root == sm || root == kqv;
            if (!inter) continue;
            const bool expected = (n == sm && t == kq) || (n == kqv && t == sm) || (n == perm && t == kqv) || (n == cont && t == perm);
            if (!expected) return false;
        }
    }
    m.q = q; m.k = k; m.v = v; m.mask = mask; m.out = cont; m.scale = op_param_f32(sm, 0); m.last = j4;
    return true;
}

static RopeParams rope_params_of(const ggml_tensor * dst) {
    RopeParams rp;
    rp.n_dims = op_param_i32(dst, 1); rp.mode = op_param_i32(dst, 2); rp.n_ctx_orig = op_param_i32(dst, 4);
    rp.freq_base = op_param_f32(dst, 5); rp.freq_scale = op_param_f32(dst, 6); rp.ext_factor = op_param_f32(dst, 7);
    rp.attn_factor = op_param_f32(dst, 8); rp.beta_fast = op_param_f32(dst, 9); rp.beta_slow = op_param_f32(dst, 10);
    return rp;
}

// ROPE(Q), ROPE(K), CPY(K -> cache view), CPY(V -> cache view) as emitted per layer (src/llama.cpp:1511-1531,
// :157-199), possibly with view-only nodes in between.  On a match returns the index of the last node.
struct RopeKvMatch { int rk = -1, ck = -1, cv = -1; };    // node indices of ROPE(K), CPY(K), CPY(V); cv < 0: V is stored separately
static bool match_rope_kv(const BackendCtx * ctx, const ggml_cgraph * g, int i, RopeKvMatch * m) {
    const ggml_tensor * rq = g->nodes[i];
    const int j1 = next_exec(ctx, g, i + 1); if (j1 < 0) return false;
    const ggml_tensor * rk = g->nodes[j1];
    if (rk->op != GGML_OP_ROPE || rk->src[1] != rq->src[1] || rk->src[2] != rq->src[2]) return false;
    if (memcmp(rk->op_params, rq->op_params, sizeof(rq->op_params)) != 0) return false;
    auto plain = [](const ggml_tensor * t) { return t->type == GGML_TYPE_F32 && t_contiguous(t) && t_contiguous(t->src[0]) && t->ne[3] == 1; };
    if (!plain(rq) || !plain(rk) || rq->ne[0] != rk->ne[0] || rq->ne[2] != rk->ne[2] || (rq->ne[0] & 1)) return false;
    if (op_param_i32(rq, 2) & ~GGML_ROPE_TYPE_NEOX) return false;
    auto cache_store = [](const ggml_tensor * c, const ggml_tensor * from) {
        if (c->op != GGML_OP_CPY || c->src[0]->type != GGML_TYPE_F32 || !t_contiguous(c->src[0])) return false;
        if (from && c->src[0] != from) return false;
        const ggml_tensor * out = c->src[1];
        return out->type == GGML_TYPE_F16 && t_contiguous(out) && out->view_src && out->view_src->data &&
               t_nelements(out) == t_nelements(c->src[0]) && (t_nelements(out) & 1) == 0 && ((uintptr_t) out->data & 3) == 0;
    };
    // CPY(K): normally next; libllama's order puts MUL_MAT(V) before it (src/llama.cpp:1511-1540, :157-199).  The
    // store may run ahead of a mat-mul it does not depend on: its source stays alive until its own position and
    // its destination is the cache.
    int j2 = next_exec(ctx, g, j1 + 1);
    const ggml_tensor * jumped = nullptr;
    if (j2 >= 0 && g->nodes[j2]->op == GGML_OP_MUL_MAT && g->nodes[j2]->src[0]->op == GGML_OP_NONE) {
        jumped = g->nodes[j2];
        j2 = next_exec(ctx, g, j2 + 1);
    }
    if (j2 < 0) return false;
    const ggml_tensor * ck = g->nodes[j2];
    if (!cache_store(ck, rk)) return false;
    if (jumped && (t_overlap(jumped, ck->src[1]) || t_overlap(jumped->src[1], ck->src[1]))) return false;
    m->rk = j1; m->ck = j2; m->cv = -1;
    const int j3 = next_exec(ctx, g, j2 + 1);
    if (j3 >= 0) {
        const ggml_tensor * cv = g->nodes[j3];
        // V rides along when it has been computed already (not the result of the mat-mul that was jumped over)
        if (cache_store(cv, nullptr) && !((uintptr_t) cv->src[0]->data & 7) && !(jumped && (cv->src[0] == jumped || cv->src[0]->view_src == jumped))) m->cv = j3;
    }
    return true;
}

// Executes node i, fusing it with its successor where the graph allows:
//   RMS_NORM -> MUL(x, w)        one launch; both outputs are written (the MUL result, and the plain
//                                norm in case something else reads it), plus the int8 blocks of the
//                                result when quantized mat-muls consume it
//   UNARY(SILU) -> MUL(silu, up) likewise
// Returns the number of nodes consumed, or 0 on failure.
static int run_node(BackendCtx * ctx, ggml_cgraph * g, int i) {
    ggml_tensor * dst = g->nodes[i];
    const LaunchCtx lc = ctx->launch_ctx();
    const ggml_tensor * a = dst->src[0];
    const ggml_tensor * b = dst->src[1];
    auto fail = [&]() { return 0; };
#define RUN0(expr) do { cudaError_t e_ = (expr); if (e_ != cudaSuccess) { B200_LOG_ERROR("ggml-b200: %s failed: %s\n", #expr, cudaGetErrorString(e_)); return fail(); } ctx->n_launches++; } while (0)
    ggml_tensor * next = i + 1 < g->n_nodes ? g->nodes[i + 1] : nullptr;
    switch (dst->op) {
        case GGML_OP_MUL_MAT: {
            // Mat-vecs on the same activations go out as one grouped launch.  libllama emits them interleaved with
            // their consumers (MUL_MAT q, ROPE q, MUL_MAT k, ROPE k, MUL_MAT v: src/llama.cpp:1511-1540), so the
            // group also takes members from a little further down the graph: such a node depends only on the shared
            // activations and a weight leaf, and it may run early if its output does not alias anything the nodes
            // it jumps over touch (ggml-alloc reuses freed memory).
            if (split_extra_of(dst->src[0])) return run_split_mul_mat(ctx, dst) ? 1 : 0;
            // attention built from MUL_MAT / SOFT_MAX / MUL_MAT (no FLASH_ATTN_EXT in the graph): one flash-attention launch
            if (ctx->use_fusion && ctx->peers.n_ranks < 2 && a->type == GGML_TYPE_F16) {
                AttnChain m;
                if (match_attn_chain(ctx, g, i, m)) {
                    const int64_t D = m.q->ne[0], n_q = m.q->ne[1], n_head = m.q->ne[2], n_kv = m.k->ne[1];
                    const TensorD qd = to_desc(m.q), kd = to_desc(m.k);
                    TensorD vd = to_desc(m.v);                       // described as [D, n_kv, heads] with the head-size dimension strided
                    vd.ne[0] = D; vd.ne[1] = n_kv; vd.nb[0] = m.v->nb[1]; vd.nb[1] = m.v->nb[0];
                    TensorD dd = to_desc(m.out);
                    dd.ne[0] = D; dd.ne[1] = n_head; dd.ne[2] = n_q; dd.ne[3] = 1; dd.nb[0] = 4; dd.nb[1] = D * 4; dd.nb[2] = D * n_head * 4; dd.nb[3] = D * n_head * n_q * 4;
                    TensorD md; bool have_mask = m.mask != nullptr;
                    if (have_mask) md = to_desc(m.mask);
                    const FattnParams fp{m.scale, 0.0f, 0.0f};
                    bool ok = true;
                    if (have_mask && m.mask->type == GGML_TYPE_F32) {
                        const size_t need = (size_t) m.mask->ne[0] * (size_t) m.mask->ne[1] * 2;
                        if (need > ctx->mask16_cap) {
                            if (ctx->capturing) { ctx->capture_failed = true; return fail(); }
                            cudaStreamSynchronize(ctx->stream);
                            if (ctx->mask16) cudaFree(ctx->mask16);
                            ctx->mask16_cap = need + need / 2; ctx->mask16_src = nullptr;
                            if (cudaMalloc(&ctx->mask16, ctx->mask16_cap + 256) != cudaSuccess) { cudaGetLastError(); ctx->mask16 = nullptr; ctx->mask16_cap = 0; ok = false; }
                        }
                        if (ok) {
                            TensorD m16 = md;
                            m16.type = GGML_TYPE_F16; m16.data = ctx->mask16;
                            m16.nb[0] = 2; m16.nb[1] = m16.ne[0] * 2; m16.nb[2] = m16.nb[1] * m16.ne[1]; m16.nb[3] = m16.nb[2];
                            if (ctx->mask16_src != m.mask->data) {
                                RUN0(launch_cpy(md, m16, lc));
                                ctx->mask16_src = m.mask->data;
                            }
                            md = m16;
                        }
                    }
                    const bool dec = lc.fa_tickets && fattn_dec_applicable(qd, kd, vd, have_mask ? &md : nullptr);
                    if (ok && (dec || fattn_tc_applicable(qd, kd, vd, have_mask ? &md : nullptr, fp))) {
                        const size_t ws = fattn_workspace_bytes(qd, kd, lc.sm_count);
                        void * wsp = ws ? ctx->get_scratch(ws) : nullptr;
                        if (ctx->capture_failed) return fail();
                        int nk = 1;
                        RUN0(launch_fattn(qd, kd, vd, have_mask ? &md : nullptr, dd, fp, wsp, lc, &nk, nullptr));
                        ctx->n_launches += (uint64_t) (nk - 1);
                        for (int j = i + 1; j <= m.last; ++j) if (!is_noop(g->nodes[j])) { ctx->node_done[(size_t) j] = 1; invalidate_written(ctx, g->nodes[j]); }
                        return 1;
                    }
                }
            }
            ggml_tensor * extra[2]; int n_extra = 0;
            const bool tc_head = ctx->use_fusion && ctx->peers.n_ranks < 2 && tc_group_ok(ctx, dst);
            if ((ctx->use_fusion && group_head_ok(dst) && !buft_is_split(dst->src[0]->buffer ? dst->src[0]->buffer->buft : nullptr)) || tc_head) {
                const bool sliced = ctx->row_slice_of(dst) != nullptr;
                const ggml_tensor * jumped[16]; int n_jumped = 0;
                for (int j = i + 1; j < g->n_nodes && n_extra < 2 && n_jumped < 16; ++j) {
                    ggml_tensor * n = g->nodes[j];
                    if (is_noop(n) || ctx->node_done[(size_t) j]) continue;
                    if (n->op == GGML_OP_FLASH_ATTN_EXT) break;
                    const bool member = (tc_head ? tc_groupable(ctx, dst, n) : groupable_mul_mat(dst, n)) && n->src[0]->op == GGML_OP_NONE &&
                                        (ctx->row_slice_of(n) != nullptr) == sliced;
                    bool clear = member;
                    for (int q = 0; q < n_jumped && clear; ++q) {
                        if (t_overlap(n, jumped[q])) clear = false;
                        for (int s_ = 0; s_ < GGML_MAX_SRC && jumped[q]->src[s_] && clear; ++s_) if (t_overlap(n, jumped[q]->src[s_])) clear = false;
                    }
                    if (member && clear) {
                        extra[n_extra++] = n; ctx->node_done[(size_t) j] = 1;
                        invalidate_written(ctx, n);
                    } else {
                        if (n->op == GGML_OP_MUL_MAT && n->src[1] != dst->src[1]) break;     // a different stage of the layer
                        if (t_overlap(n, dst->src[1]) || (n->op == GGML_OP_CPY && n->src[1] && t_overlap(n->src[1], dst->src[1]))) break;   // it rewrites the shared input (in place, through a view): later mat-muls must see that
                        jumped[n_jumped++] = n;
                    }
                }
            }
            return run_mul_mat(ctx, dst, nullptr, extra, n_extra) ? 1 : 0;
        }
        case GGML_OP_MUL_MAT_ID: return run_mul_mat(ctx, dst, dst->src[2]) ? 1 : 0;
        case GGML_OP_FLASH_ATTN_EXT: {
            const ggml_tensor * v = dst->src[2];
            const ggml_tensor * mask = dst->src[3];
            FattnParams fp{op_param_f32(dst, 0), op_param_f32(dst, 1), op_param_f32(dst, 2)};
            const TensorD qd = to_desc(a), kd = to_desc(b), vd = to_desc(v), dd = to_desc(dst);
            TensorD md; if (mask) md = to_desc(mask);
            const size_t ws = fattn_workspace_bytes(qd, kd, lc.sm_count);
            void * wsp = ws ? ctx->get_scratch(ws) : nullptr;
            if (ctx->capture_failed) return fail();
            // decode: when the attention output goes straight into a quantized MUL_MAT (wo), the kernel also
            // writes its int8 activation blocks (one head row of 128 values = one block)
            void * act = nullptr;
            if (ctx->use_fusion && lc.fa_tickets && a->ne[0] == 128 && a->ne[3] == 1 && kd.type == GGML_TYPE_F16 && vd.type == GGML_TYPE_F16 &&
                fattn_dec_applicable(qd, kd, vd, mask ? &md : nullptr)) {
                const int j = next_exec(ctx, g, i + 1);
                const ggml_tensor * mm = j >= 0 ? g->nodes[j] : nullptr;
                if (mm && mm->op == GGML_OP_MUL_MAT && mm->src[1]->data == dst->data && mmvq_type_supported(mm->src[0]->type) &&
                    act_cacheable(mm->src[1]) && mm->src[1]->ne[0] == dst->ne[0] * dst->ne[1] && mm->src[1]->ne[1] == dst->ne[2]) {
                    BackendCtx::ActEntry * e = ctx->act_cache_take(dst->data, mm->src[1]->ne[0], mm->src[1]->ne[1]);
                    if (!e) return fail();
                    act = e->q;
                }
            }
            int nk = 1;
            RUN0(launch_fattn(qd, kd, vd, mask ? &md : nullptr, dd, fp, wsp, lc, &nk, act));
            ctx->n_launches += nk - 1;                               // second kernel: split-KV combine or mask-tile flags
            return 1;
        }
        case GGML_OP_RMS_NORM: {
            if (next && next->op == GGML_OP_MUL && next->src[0] == dst && next->type == GGML_TYPE_F32 && next->src[1]->type == GGML_TYPE_F32 &&
                next->src[1]->nb[0] == 4 && t_contiguous(next) && t_can_repeat(next->src[1], dst) && device_supports_op(ctx->dev, next)) {
                void * act = nullptr;
                if (act_cacheable(next) && next->ne[0] % 128 == 0 && feeds_quant_mul_mat(g, i + 2, next)) {
                    BackendCtx::ActEntry * e = ctx->act_cache_take(next->data, next->ne[0], next->ne[1] * next->ne[2] * next->ne[3]);
                    if (!e) return fail();
                    act = e->q;
                }
                void * h16 = tc_f16_out_for(ctx, g, i + 2, next);
                RUN0(launch_rms_norm_mul(to_desc(a), to_desc(next->src[1]), to_desc(next), op_param_f32(dst, 0), act,
                                         dst->data == next->data ? nullptr : (float *) dst->data, nullptr, nullptr, lc, h16));
                return 2;
            }
            RUN0(launch_rms_norm(to_desc(a), to_desc(dst), op_param_f32(dst, 0), lc));
            return 1;
        }
        case GGML_OP_NORM: RUN0(launch_norm(to_desc(a), to_desc(dst), op_param_f32(dst, 0), lc)); return 1;
        case GGML_OP_ADD: {
            // residual add feeding RMS_NORM -> MUL(x, w): one launch writes the sum, the norm, the product and,
            // when quantized mat-muls read the product, its int8 blocks
            ggml_tensor * rn = next;
            ggml_tensor * mu = i + 2 < g->n_nodes ? g->nodes[i + 2] : nullptr;
            if (rn && mu && rn->op == GGML_OP_RMS_NORM && rn->src[0] == dst && mu->op == GGML_OP_MUL && mu->src[0] == rn &&
                dst->type == GGML_TYPE_F32 && a->type == GGML_TYPE_F32 && b->type == GGML_TYPE_F32 && t_same_shape(a, b) &&
                t_contiguous(a) && t_contiguous(b) && t_contiguous(dst) && t_contiguous(rn) && t_contiguous(mu) &&
                mu->type == GGML_TYPE_F32 && mu->src[1]->type == GGML_TYPE_F32 && mu->src[1]->nb[0] == 4 && t_can_repeat(mu->src[1], rn)) {
                void * act = nullptr;
                invalidate_written(ctx, rn);          // (the MUL is often computed in place of the norm's output)
                invalidate_written(ctx, mu);          // written by this launch: cached conversions of its old contents are stale
                if (act_cacheable(mu) && mu->ne[0] % 128 == 0 && feeds_quant_mul_mat(g, i + 3, mu)) {
                    BackendCtx::ActEntry * e = ctx->act_cache_take(mu->data, mu->ne[0], mu->ne[1] * mu->ne[2] * mu->ne[3]);
                    if (!e) return fail();
                    act = e->q;
                }
                void * h16 = tc_f16_out_for(ctx, g, i + 3, mu);
                RUN0(launch_rms_norm_mul(to_desc(a), to_desc(mu->src[1]), to_desc(mu), op_param_f32(rn, 0), act, rn->data == mu->data ? nullptr : (float *) rn->data,
                                         (const float *) b->data, (float *) dst->data, lc, h16));
                return 3;
            }
            RUN0(launch_bin_bcast(BIN_ADD, to_desc(a), to_desc(b), to_desc(dst), lc));
            return 1;
        }
        case GGML_OP_SUB: RUN0(launch_bin_bcast(BIN_SUB, to_desc(a), to_desc(b), to_desc(dst), lc)); return 1;
        case GGML_OP_MUL: RUN0(launch_bin_bcast(BIN_MUL, to_desc(a), to_desc(b), to_desc(dst), lc)); return 1;
        case GGML_OP_DIV: RUN0(launch_bin_bcast(BIN_DIV, to_desc(a), to_desc(b), to_desc(dst), lc)); return 1;
        case GGML_OP_UNARY: {
            const int uop = op_param_i32(dst, 0);
            const int jn = next_exec(ctx, g, i + 1);           // skips a mat-mul that was hoisted into an earlier group
            ggml_tensor * next = jn >= 0 ? g->nodes[jn] : nullptr;
            if (ctx->use_fusion && uop == GGML_UNARY_OP_SILU && next && next->op == GGML_OP_MUL && next->src[0] == dst && next->type == GGML_TYPE_F32 &&
                next->src[1]->type == GGML_TYPE_F32 && t_same_shape(next->src[1], dst) && t_contiguous(next->src[1]) && t_contiguous(next)) {
                void * act = nullptr;
                invalidate_written(ctx, next);
                if (act_cacheable(next) && next->ne[0] % 128 == 0 && feeds_quant_mul_mat(g, jn + 1, next)) {
                    BackendCtx::ActEntry * e = ctx->act_cache_take(next->data, next->ne[0], next->ne[1] * next->ne[2] * next->ne[3]);
                    if (!e) return fail();
                    act = e->q;
                }
                // the intermediate silu(gate) is skipped when the product is computed in place of it
                void * h16 = tc_f16_out_for(ctx, g, jn + 1, next);
                RUN0(launch_silu_mul(to_desc(a), to_desc(next->src[1]), to_desc(next), act, dst->data == next->data ? nullptr : (float *) dst->data, lc, h16));
                ctx->node_done[(size_t) jn] = 1;
                return 1;
            }
            RUN0(launch_unary(unary_to_unop(uop), to_desc(a), to_desc(dst), lc));
            return 1;
        }
        case GGML_OP_SQR:  RUN0(launch_unary(UN_SQR, to_desc(a), to_desc(dst), lc)); return 1;
        case GGML_OP_SQRT: RUN0(launch_unary(UN_SQRT, to_desc(a), to_desc(dst), lc)); return 1;
        case GGML_OP_SIN:  RUN0(launch_unary(UN_SIN, to_desc(a), to_desc(dst), lc)); return 1;
        case GGML_OP_COS:  RUN0(launch_unary(UN_COS, to_desc(a), to_desc(dst), lc)); return 1;
        case GGML_OP_LOG:  RUN0(launch_unary(UN_LOG, to_desc(a), to_desc(dst), lc)); return 1;
        case GGML_OP_SCALE: RUN0(launch_scale(to_desc(a), to_desc(dst), op_param_f32(dst, 0), lc)); return 1;
        case GGML_OP_CLAMP: RUN0(launch_clamp(to_desc(a), to_desc(dst), op_param_f32(dst, 0), op_param_f32(dst, 1), lc)); return 1;
        case GGML_OP_ROPE: {
            const RopeParams rp = rope_params_of(dst);
            const ggml_tensor * ff = dst->src[2];
            RopeKvMatch m;
            if (ctx->use_fusion && match_rope_kv(ctx, g, i, &m) && (!ctx->capturing || ctx->dyn_used + 2 <= BackendCtx::DYN_CAP)) {
                const ggml_tensor * rk = g->nodes[m.rk], * ck = g->nodes[m.ck], * cv = m.cv >= 0 ? g->nodes[m.cv] : nullptr;
                RopeKvLaunch l = {};
                l.q_src = (const float *) a->data; l.q_dst = (float *) dst->data;
                l.k_src = (const float *) rk->src[0]->data; l.k_dst = (float *) rk->data;
                l.hd = dst->ne[0]; l.n_head = dst->ne[1]; l.n_head_kv = rk->ne[1]; l.n_tok = dst->ne[2];
                const ggml_tensor * ko = ck->src[1];
                l.k_cache = ko->view_src->data;
                l.k_off = (const char *) ko->data - (const char *) ko->view_src->data;
                if (cv) {
                    const ggml_tensor * vo = cv->src[1];
                    l.v_src = (const float *) cv->src[0]->data; l.v_elems = t_nelements(cv->src[0]);
                    l.v_cache = vo->view_src->data;
                    l.v_off = (const char *) vo->data - (const char *) vo->view_src->data;
                }
                if (ctx->capturing) {                   // same slot order as the CPY nodes appear in the graph
                    ctx->dyn_host[ctx->dyn_used] = l.k_off; l.k_off_dev = ctx->dyn_dev + ctx->dyn_used++;
                    if (cv) { ctx->dyn_host[ctx->dyn_used] = l.v_off; l.v_off_dev = ctx->dyn_dev + ctx->dyn_used++; }
                }
                l.pos = (const int32_t *) b->data; l.ff = ff ? (const float *) ff->data : nullptr;
                invalidate_written(ctx, rk);
                ctx->node_done[(size_t) m.rk] = 1; ctx->node_done[(size_t) m.ck] = 1;
                if (cv) ctx->node_done[(size_t) m.cv] = 1;
                RUN0(launch_rope_kv(l, rp, lc));
                return 1;
            }
            RUN0(launch_rope(to_desc(a), (const int32_t *) b->data, ff ? (const float *) ff->data : nullptr, to_desc(dst), rp, lc));
            return 1;
        }
        case GGML_OP_CPY: case GGML_OP_DUP: case GGML_OP_CONT: {
            // CPY writes into src1's memory (dst is a view of it); DUP/CONT write dst
            const ggml_tensor * out = dst->op == GGML_OP_CPY ? b : dst;
            if (ctx->capturing && dst->op == GGML_OP_CPY && out->view_src && out->view_src->data && ctx->dyn_used < BackendCtx::DYN_CAP) {
                // a store into a view (the KV-cache rows of this token): the view's byte offset is read by the
                // kernel from device memory, so the captured launch is independent of the token position
                TensorD od = to_desc(out);
                od.data = out->view_src->data;
                ctx->dyn_host[ctx->dyn_used] = (int64_t) ((const char *) out->data - (const char *) out->view_src->data);
                RUN0(launch_cpy(to_desc(a), od, lc, ctx->dyn_dev + ctx->dyn_used));
                ctx->dyn_used++;
                return 1;
            }
            if (a->type == out->type && t_contiguous(a) && t_contiguous(out)) {
                RUN0(cudaMemcpyAsync(out->data, a->data, t_nbytes(a), cudaMemcpyDeviceToDevice, lc.stream));
            } else {
                RUN0(launch_cpy(to_desc(a), to_desc(out), lc));
            }
            return 1;
        }
        case GGML_OP_GET_ROWS: RUN0(launch_get_rows(to_desc(a), to_desc(b), to_desc(dst), lc)); return 1;
        case GGML_OP_SOFT_MAX: {
            TensorD md; if (b) md = to_desc(b);
            RUN0(launch_soft_max(to_desc(a), b ? &md : nullptr, to_desc(dst), op_param_f32(dst, 0), op_param_f32(dst, 1), lc));
            return 1;
        }
        default:
            B200_LOG_ERROR("ggml-b200: op %d reached graph_compute but is not supported\n", (int) dst->op);
            return 0;
    }
#undef RUN0
}

bool run_single_node(BackendCtx * ctx, ggml_cgraph * g, int i) {
    const int fusion = ctx->use_fusion;
    ctx->use_fusion = 0;
    invalidate_written(ctx, g->nodes[i]);
    const int used = run_node(ctx, g, i);
    ctx->use_fusion = fusion;
    return used == 1;
}

static bool is_noop(const ggml_tensor * node) {
    return t_empty(node) || node->op == GGML_OP_NONE || node->op == GGML_OP_RESHAPE || node->op == GGML_OP_VIEW ||
           node->op == GGML_OP_PERMUTE || node->op == GGML_OP_TRANSPOSE;
}

static int next_exec(const BackendCtx * ctx, const ggml_cgraph * g, int i) {
    for (; i < g->n_nodes; ++i) if (!is_noop(g->nodes[i]) && !(i < (int) ctx->node_done.size() && ctx->node_done[(size_t) i])) return i;
    return -1;
}

static bool run_all(BackendCtx * ctx, ggml_cgraph * cgraph) {
    ctx->act_cache_clear();
    std::vector<const void *> & pending_full = ctx->pending_full;
    pending_full.clear();
    ctx->node_done.assign((size_t) cgraph->n_nodes, 0);
    ctx->mega_tried = false; ctx->mega_ops_used = 0;
    ctx->mask16_src = nullptr;
    for (int i = 0; i < cgraph->n_nodes;) {
        ggml_tensor * node = cgraph->nodes[i];
        if (is_noop(node) || ctx->node_done[(size_t) i]) { ++i; continue; }
        // single-token Llama layers: one persistent launch for the whole run of layers (decode_plan.cpp)
        if (ctx->use_mega && ctx->use_fusion && !ctx->mega_tried && ctx->peers.n_ranks < 2 && !ctx->peer_pending &&
            (node->op == GGML_OP_ADD || node->op == GGML_OP_RMS_NORM) && node->ne[1] == 1 && node->ne[2] == 1 && node->ne[3] == 1) {
            const int next = try_decode_step(ctx, cgraph, i);
            if (next > i) { i = next; continue; }
            ctx->mega_tried = true;
        }
        const ggml_b200_row_slice * rs = ctx->row_slice_of(node);
        if (ctx->peer_pending) {
            // slices stored to the peers become readable after a barrier; consecutive sliced MUL_MATs that
            // do not read one of the pending results share one
            bool need = rs == nullptr;
            if (rs) {
                const ggml_tensor * x = node->src[1];
                for (const void * f : pending_full) if (x->data == f || (x->view_src && x->view_src->data == f)) need = true;
            }
            if (need) { if (!peer_barrier(ctx)) return false; pending_full.clear(); }
        }
        invalidate_written(ctx, node);
        if (node->op == GGML_OP_CPY) invalidate_written(ctx, node->src[1]);
        if (i + 1 < cgraph->n_nodes) invalidate_written(ctx, cgraph->nodes[i + 1]);   // it may be fused into this launch
        const uint64_t l0 = ctx->n_launches;
        const int used = run_node(ctx, cgraph, i);
        if (used == 0) return false;
        if (ctx->trace > 0)
            fprintf(stderr, "ggml-b200 trace: node %4d op %2d %-24s ne [%lld %lld %lld] nodes %d launches %llu\n", i, (int) node->op, node->name,
                    (long long) node->ne[0], (long long) node->ne[1], (long long) node->ne[2], used, (unsigned long long) (ctx->n_launches - l0));
        i += used;
    }
    if (ctx->peer_pending && !peer_barrier(ctx)) return false;
    if (ctx->trace > 0) ctx->trace--;                  // GGML_B200_TRACE=n: the first n graphs
    return true;
}

// ---------------------------------------------------------------------------
// CUDA-graph replay for small-batch (decode) graphs
// ---------------------------------------------------------------------------
static inline uint64_t mix(uint64_t h, uint64_t v) { h ^= v + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2); return h * 0xff51afd7ed558ccdull; }

// A CPY whose destination is a view: its position inside the viewed tensor may change from call to
// call (the KV-cache write position) without invalidating a captured graph.
static const ggml_tensor * dyn_cpy_dst(const ggml_tensor * node) {
    if (node->op != GGML_OP_CPY) return nullptr;
    const ggml_tensor * out = node->src[1];
    return (out && out->view_src && out->view_src->data) ? out : nullptr;
}

// key over everything a captured launch sequence depends on; returns 0 when the graph is not a
// candidate (a large batch, or nothing to run)
static uint64_t graph_signature(BackendCtx * ctx, const ggml_cgraph * g, int * n_dyn) {
    uint64_t h = mix(0x1234, ctx->scratch_generation);
    int exec_nodes = 0, dyn = 0;
    for (int i = 0; i < g->n_nodes; ++i) {
        const ggml_tensor * n = g->nodes[i];
        if (is_noop(n)) continue;
        ++exec_nodes;
        // only small batches are worth replaying; dim 1 of the activation operand is the token count (for MUL_MAT_ID
        // dim 2), the attention products of the non-flash path batch over heads in dims 2 and 3
        if (n->op == GGML_OP_MUL_MAT && n->src[1]->ne[1] > 8) return 0;
        if (n->op == GGML_OP_MUL_MAT && split_extra_of(n->src[0])) return 0;     // work on several devices' streams: not captured
        if (n->op == GGML_OP_MUL_MAT_ID && n->src[1]->ne[2] > 8) return 0;
        const ggml_tensor * dd = dyn_cpy_dst(n);
        h = mix(h, (uint64_t) n->op | ((uint64_t) n->type << 32));
        h = mix(h, dd ? (uint64_t) (uintptr_t) dd->view_src->data : (uint64_t) (uintptr_t) n->data);
        if (dd) ++dyn;
        for (int d = 0; d < 4; ++d) { h = mix(h, (uint64_t) n->ne[d]); h = mix(h, (uint64_t) n->nb[d]); }
        const uint64_t * op = (const uint64_t *) n->op_params;
        for (int d = 0; d < 8; ++d) h = mix(h, op[d]);
        for (int s = 0; s < GGML_MAX_SRC && n->src[s]; ++s) {
            const ggml_tensor * t = n->src[s];
            const bool is_dyn_dst = dd && t == dd;
            h = mix(h, is_dyn_dst ? (uint64_t) (uintptr_t) dd->view_src->data : (uint64_t) (uintptr_t) t->data);
            h = mix(h, (uint64_t) t->type);
            for (int d = 0; d < 4; ++d) { h = mix(h, (uint64_t) t->ne[d]); h = mix(h, (uint64_t) t->nb[d]); }
        }
    }
    *n_dyn = dyn;
    if (exec_nodes < 8 || dyn > BackendCtx::DYN_CAP) return 0;
    return h ? h : 1;
}

enum ggml_status graph_compute(BackendCtx * ctx, ggml_cgraph * cgraph) {
    int n_dyn = 0;
    const uint64_t key = ctx->use_graphs ? graph_signature(ctx, cgraph, &n_dyn) : 0;
    if (key == 0) {
        ctx->pending_key = 0; ctx->n_direct++;
        return run_all(ctx, cgraph) ? GGML_STATUS_SUCCESS : GGML_STATUS_FAILED;
    }
    if (key == ctx->graph_key && ctx->graph_exec) {
        ctx->n_replay++;
        // replay: refresh the token-dependent offsets, then one graph launch
        int k = 0;
        for (int i = 0; i < cgraph->n_nodes; ++i) {
            const ggml_tensor * n = cgraph->nodes[i];
            if (is_noop(n)) continue;
            if (const ggml_tensor * dd = dyn_cpy_dst(n)) ctx->dyn_host[k++] = (int64_t) ((const char *) dd->data - (const char *) dd->view_src->data);
        }
        if (k) B200_CUDA_CHECK(cudaMemcpyAsync(ctx->dyn_dev, ctx->dyn_host, sizeof(int64_t) * k, cudaMemcpyHostToDevice, ctx->stream));
        B200_CUDA_CHECK(cudaGraphLaunch(ctx->graph_exec, ctx->stream));
        ctx->n_launches += ctx->graph_launches; ctx->n_mega += ctx->graph_megas;
        return GGML_STATUS_SUCCESS;
    }
    if (key != ctx->pending_key) {
        // first sighting of this graph: run it directly (this also performs any lazy allocation and
        // per-kernel attribute set-up); capture if it comes back
        ctx->pending_key = key; ctx->n_direct++;
        return run_all(ctx, cgraph) ? GGML_STATUS_SUCCESS : GGML_STATUS_FAILED;
    }
    // second sighting: capture
    ctx->n_capture++;
    if (ctx->graph_exec) { cudaGraphExecDestroy(ctx->graph_exec); ctx->graph_exec = nullptr; ctx->graph_key = 0; }
    ctx->capturing = true; ctx->capture_failed = false; ctx->dyn_used = 0;
    const uint64_t launches_before = ctx->n_launches, megas_before = ctx->n_mega;
    B200_CUDA_CHECK(cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeRelaxed));
    const bool ok = run_all(ctx, cgraph);
    cudaGraph_t graph = nullptr;
    const cudaError_t ce = cudaStreamEndCapture(ctx->stream, &graph);
    ctx->capturing = false;
    const uint64_t captured = ctx->n_launches - launches_before;
    ctx->n_launches = launches_before;
    if (!ok || ctx->capture_failed || ce != cudaSuccess || !graph) {
        cudaGetLastError();
        if (graph) cudaGraphDestroy(graph);
        ctx->pending_key = 0;
        B200_LOG_WARN("ggml-b200: CUDA graph capture abandoned, running the graph directly\n");
        return run_all(ctx, cgraph) ? GGML_STATUS_SUCCESS : GGML_STATUS_FAILED;
    }
    cudaGraphExec_t exec = nullptr;
    if (cudaGraphInstantiate(&exec, graph, 0) != cudaSuccess) {
        cudaGetLastError();
        cudaGraphDestroy(graph);
        ctx->pending_key = 0;
        return run_all(ctx, cgraph) ? GGML_STATUS_SUCCESS : GGML_STATUS_FAILED;
    }
    cudaGraphDestroy(graph);
    ctx->graph_exec = exec; ctx->graph_key = key; ctx->graph_launches = captured; ctx->graph_megas = ctx->n_mega - megas_before;
    if (ctx->dyn_used) B200_CUDA_CHECK(cudaMemcpyAsync(ctx->dyn_dev, ctx->dyn_host, sizeof(int64_t) * ctx->dyn_used, cudaMemcpyHostToDevice, ctx->stream));
    B200_CUDA_CHECK(cudaGraphLaunch(ctx->graph_exec, ctx->stream));
    ctx->n_launches += captured;
    return GGML_STATUS_SUCCESS;
}

}  // namespace b200
