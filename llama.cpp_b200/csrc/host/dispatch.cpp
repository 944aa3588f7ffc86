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
            if (a->nb[0] != 4 || b->nb[0] != 2 || v->nb[0] != 2) return false;
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

static bool run_mul_mat(BackendCtx * ctx, const ggml_tensor * dst, const ggml_tensor * ids) {
    const ggml_tensor * W = dst->src[0];
    const ggml_tensor * X = dst->src[1];
    const LaunchCtx lc = ctx->launch_ctx();
    if (!ids && is_float_type(W->type)) {
        RUN(launch_matmul_f(to_desc(W), to_desc(X), to_desc(dst), lc));
        return true;
    }
    const int64_t K = W->ne[0], M = W->ne[1];
    const int64_t ne11 = X->ne[1], ne12 = X->ne[2], ne13 = X->ne[3];
    void * xq = ctx->get_scratch(act128_bytes(K, ne11 * ne12 * ne13));
    RUN(launch_quantize_act128((const float *) X->data, ne11, ne12, ne13, X->nb[1] / 4, X->nb[2] / 4, X->nb[3] / 4, xq, (int) K, lc.stream));

    MmvqArgs a = {};
    a.type = W->type; a.W = W->data; a.w_nb1 = W->nb[1]; a.w_nb2 = W->nb[2]; a.w_nb3 = W->nb[3];
    a.Xq = xq; a.M = (int) M; a.K = (int) K;
    a.status = lc.status; a.sm_count = lc.sm_count; a.device = lc.device; a.use_pdl = lc.use_pdl;
    if (!ids) {
        a.ne12 = (int) ne12; a.ne13 = (int) ne13;
        a.r2 = (int) (ne12 / W->ne[2]); a.r3 = (int) (ne13 / W->ne[3]);
        a.dst_nb1 = dst->nb[1]; a.dst_nb2 = dst->nb[2]; a.dst_nb3 = dst->nb[3];
        a.x_ncols = (int) ne11; a.xq_ne12 = (int) ne12;
        for (int64_t n0 = 0; n0 < ne11; n0 += 8) {
            a.N = (int) (ne11 - n0 < 8 ? ne11 - n0 : 8);
            a.x_col0 = (int) n0;
            a.dst = (float *) ((char *) dst->data + n0 * dst->nb[1]);
            RUN(launch_mmvq(a, lc.stream));
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

static bool run_node(BackendCtx * ctx, ggml_tensor * dst) {
    const LaunchCtx lc = ctx->launch_ctx();
    const ggml_tensor * a = dst->src[0];
    const ggml_tensor * b = dst->src[1];
    switch (dst->op) {
        case GGML_OP_MUL_MAT:    return run_mul_mat(ctx, dst, nullptr);
        case GGML_OP_MUL_MAT_ID: return run_mul_mat(ctx, dst, dst->src[2]);
        case GGML_OP_FLASH_ATTN_EXT: {
            const ggml_tensor * v = dst->src[2];
            const ggml_tensor * mask = dst->src[3];
            FattnParams fp{op_param_f32(dst, 0), op_param_f32(dst, 1), op_param_f32(dst, 2)};
            const TensorD qd = to_desc(a), kd = to_desc(b), vd = to_desc(v), dd = to_desc(dst);
            TensorD md; if (mask) md = to_desc(mask);
            const size_t ws = fattn_workspace_bytes(qd, kd, lc.sm_count);
            void * wsp = ws ? ctx->get_scratch(ws) : nullptr;
            RUN(launch_fattn(qd, kd, vd, mask ? &md : nullptr, dd, fp, wsp, lc));
            if (ws) ctx->n_launches++;
            return true;
        }
        case GGML_OP_RMS_NORM: RUN(launch_rms_norm(to_desc(a), to_desc(dst), op_param_f32(dst, 0), lc)); return true;
        case GGML_OP_NORM:     RUN(launch_norm(to_desc(a), to_desc(dst), op_param_f32(dst, 0), lc)); return true;
        case GGML_OP_ADD: RUN(launch_bin_bcast(BIN_ADD, to_desc(a), to_desc(b), to_desc(dst), lc)); return true;
        case GGML_OP_SUB: RUN(launch_bin_bcast(BIN_SUB, to_desc(a), to_desc(b), to_desc(dst), lc)); return true;
        case GGML_OP_MUL: RUN(launch_bin_bcast(BIN_MUL, to_desc(a), to_desc(b), to_desc(dst), lc)); return true;
        case GGML_OP_DIV: RUN(launch_bin_bcast(BIN_DIV, to_desc(a), to_desc(b), to_desc(dst), lc)); return true;
        case GGML_OP_UNARY: RUN(launch_unary(unary_to_unop(op_param_i32(dst, 0)), to_desc(a), to_desc(dst), lc)); return true;
        case GGML_OP_SQR:  RUN(launch_unary(UN_SQR, to_desc(a), to_desc(dst), lc)); return true;
        case GGML_OP_SQRT: RUN(launch_unary(UN_SQRT, to_desc(a), to_desc(dst), lc)); return true;
        case GGML_OP_SIN:  RUN(launch_unary(UN_SIN, to_desc(a), to_desc(dst), lc)); return true;
        case GGML_OP_COS:  RUN(launch_unary(UN_COS, to_desc(a), to_desc(dst), lc)); return true;
        case GGML_OP_LOG:  RUN(launch_unary(UN_LOG, to_desc(a), to_desc(dst), lc)); return true;
        case GGML_OP_SCALE: RUN(launch_scale(to_desc(a), to_desc(dst), op_param_f32(dst, 0), lc)); return true;
        case GGML_OP_CLAMP: RUN(launch_clamp(to_desc(a), to_desc(dst), op_param_f32(dst, 0), op_param_f32(dst, 1), lc)); return true;
        case GGML_OP_ROPE: {
            RopeParams rp;
            rp.n_dims = op_param_i32(dst, 1); rp.mode = op_param_i32(dst, 2); rp.n_ctx_orig = op_param_i32(dst, 4);
            rp.freq_base = op_param_f32(dst, 5); rp.freq_scale = op_param_f32(dst, 6); rp.ext_factor = op_param_f32(dst, 7);
            rp.attn_factor = op_param_f32(dst, 8); rp.beta_fast = op_param_f32(dst, 9); rp.beta_slow = op_param_f32(dst, 10);
            const ggml_tensor * ff = dst->src[2];
            RUN(launch_rope(to_desc(a), (const int32_t *) b->data, ff ? (const float *) ff->data : nullptr, to_desc(dst), rp, lc));
            return true;
        }
        case GGML_OP_CPY: case GGML_OP_DUP: case GGML_OP_CONT: {
            // CPY writes into src1's memory (dst is a view of it); DUP/CONT write dst
            const ggml_tensor * out = dst->op == GGML_OP_CPY ? b : dst;
            if (a->type == out->type && t_contiguous(a) && t_contiguous(out)) {
                RUN(cudaMemcpyAsync(out->data, a->data, t_nbytes(a), cudaMemcpyDeviceToDevice, lc.stream));
            } else {
                RUN(launch_cpy(to_desc(a), to_desc(out), lc));
            }
            return true;
        }
        case GGML_OP_GET_ROWS: RUN(launch_get_rows(to_desc(a), to_desc(b), to_desc(dst), lc)); return true;
        case GGML_OP_SOFT_MAX: {
            TensorD md; if (b) md = to_desc(b);
            RUN(launch_soft_max(to_desc(a), b ? &md : nullptr, to_desc(dst), op_param_f32(dst, 0), op_param_f32(dst, 1), lc));
            return true;
        }
        default:
            B200_LOG_ERROR("ggml-b200: op %d reached graph_compute but is not supported\n", (int) dst->op);
            return false;
    }
}

enum ggml_status graph_compute(BackendCtx * ctx, ggml_cgraph * cgraph) {
    for (int i = 0; i < cgraph->n_nodes; ++i) {
        ggml_tensor * node = cgraph->nodes[i];
        if (t_empty(node) || node->op == GGML_OP_NONE || node->op == GGML_OP_RESHAPE || node->op == GGML_OP_VIEW ||
            node->op == GGML_OP_PERMUTE || node->op == GGML_OP_TRANSPOSE) {
            continue;
        }
        if (!run_node(ctx, node)) return GGML_STATUS_FAILED;
    }
    return GGML_STATUS_SUCCESS;
}

// ---- row-split buffer type: provided by split.cpp once built; until then absent ----
bool buft_is_split(ggml_backend_buffer_type_t) { return false; }
ggml_backend_buffer_type_t split_buffer_type(int, const float *) { return nullptr; }

}  // namespace b200
