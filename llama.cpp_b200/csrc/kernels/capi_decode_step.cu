// Flat C-ABI over single phases of the persistent decode-step kernel (decode_step.cu), declared in
// include/b200_kernels.h: host buffers in, host buffers out, device memory owned for the duration of the
// call.  They exist so that the parity tests can drive each phase of that kernel on its own -- a mat-vec with
// its fused input stage, the gate/up pair with silu * up, the q/k/v projections with rotation and cache
// store, the attention -- against the same oracle as the one-kernel-per-op entry points.
#include "common.cuh"
#include "kernels.h"
#include "b200_kernels.h"

#include <cstring>
#include <string>
#include <vector>

using namespace b200;

#define API extern "C" __attribute__((visibility("default")))

namespace {
thread_local std::string g_ds_err;
int ds_fail(int code, const std::string & msg) { g_ds_err = msg; return code; }

struct Dev {
    void * p = nullptr;
    ~Dev() { if (p) cudaFree(p); }
    bool alloc(size_t n) { return cudaMalloc(&p, n + 256) == cudaSuccess && cudaMemset(p, 0, n + 256) == cudaSuccess; }
    bool put(const void * src, size_t n) { return alloc(n) && (n == 0 || cudaMemcpy(p, src, n, cudaMemcpyHostToDevice) == cudaSuccess); }
    bool get(void * dst, size_t n) const { return cudaMemcpy(dst, p, n, cudaMemcpyDeviceToHost) == cudaSuccess; }
};

// runs the phases on the current device and waits for them
int run_phases(const std::vector<DsOp> & ops) {
    int dev = 0, major = 0, sm = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess || major != 10) {
        cudaGetLastError();
        return ds_fail(B200_E_NO_DEVICE, "no sm_100 device");
    }
    cudaDeviceGetAttribute(&sm, cudaDevAttrMultiProcessorCount, dev);
    Dev d_ops, d_work, d_sync, d_status;
    if (!d_ops.put(ops.data(), ops.size() * sizeof(DsOp)) || !d_work.alloc(decode_step_work_bytes((int) ops.size())) || !d_sync.alloc(256) || !d_status.alloc(16)) {
        cudaGetLastError();
        return ds_fail(B200_E_SCRATCH, "device allocation failed");
    }
    cudaError_t e = decode_step_prepare(ops.data(), (int) ops.size(), sm, d_work.p, nullptr);
    if (e != cudaSuccess) { cudaGetLastError(); return ds_fail(B200_E_UNSUPPORTED, "shape or type not handled by the decode-step kernel"); }
    LaunchCtx lc = {};
    lc.stream = nullptr; lc.device = dev; lc.sm_count = sm; lc.status = (int *) d_status.p;
    e = launch_decode_step((const DsOp *) d_ops.p, ops.data(), (int) ops.size(), d_work.p, (unsigned *) d_sync.p, lc);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) { cudaGetLastError(); return ds_fail((int) e, std::string("decode-step launch: ") + cudaGetErrorString(e)); }
    int st = 0;
    if (!d_status.get(&st, sizeof(st))) { cudaGetLastError(); return ds_fail(B200_E_DEVICE_WAIT, "status word unreadable"); }
    if (st != 0) return ds_fail(B200_E_DEVICE_WAIT, "the kernel gave up a bounded wait");
    return 0;
}
size_t row_bytes(int type, int64_t K) { return (size_t) (K / type_block_elems(type)) * type_block_bytes(type); }
}  // namespace

API const char * b200_decode_step_last_error(void) { return g_ds_err.c_str(); }

API int b200_decode_step_mul_mat_host(int type, const void * W, int64_t M, int64_t K, const float * x, const float * x_add,
                                      const float * norm_w, float eps, float * dst, float * sum_out) {
    if (!type_block_elems(type) || K <= 0 || M <= 0 || K % 256) return ds_fail(B200_E_BAD_ARG, "bad shape");
    const size_t rb = row_bytes(type, K);
    Dev dw, dx, da, dn, dd, dsum;
    if (!dw.put(W, rb * M) || !dx.put(x, K * 4) || !dd.alloc(M * 4) || !dsum.alloc(K * 4) || (x_add && !da.put(x_add, K * 4)) || (norm_w && !dn.put(norm_w, K * 4))) {
        cudaGetLastError();
        return ds_fail(B200_E_SCRATCH, "device allocation failed");
    }
    DsOp o; memset(&o, 0, sizeof(o));
    o.kind = DS_OP_MATVEC; o.in_kind = norm_w ? DS_IN_NORM : DS_IN_PLAIN; o.K = (int) K; o.nmat = 1; o.epilogue = DS_EP_STORE;
    o.in0 = (const float *) dx.p; o.in1 = x_add ? (const float *) da.p : nullptr; o.norm_w = (const float *) dn.p; o.eps = eps;
    o.sum_out = x_add ? (float *) dsum.p : nullptr;
    o.W[0] = dw.p; o.type[0] = type; o.M[0] = (int) M; o.w_nb1[0] = (int64_t) rb; o.dst[0] = (float *) dd.p;
    if (int rc = run_phases({o})) return rc;
    if (!dd.get(dst, M * 4) || (sum_out && x_add && !dsum.get(sum_out, K * 4))) { cudaGetLastError(); return ds_fail(B200_E_BAD_ARG, "copy back failed"); }
    return 0;
}

API int b200_decode_step_gate_up_host(int type, const void * Wg, const void * Wu, int64_t M, int64_t K, const float * x, float * dst) {
    if (!type_block_elems(type) || K <= 0 || M <= 0 || K % 256) return ds_fail(B200_E_BAD_ARG, "bad shape");
    const size_t rb = row_bytes(type, K);
    Dev dg, du, dx, dd;
    if (!dg.put(Wg, rb * M) || !du.put(Wu, rb * M) || !dx.put(x, K * 4) || !dd.alloc(M * 4)) { cudaGetLastError(); return ds_fail(B200_E_SCRATCH, "device allocation failed"); }
    DsOp o; memset(&o, 0, sizeof(o));
    o.kind = DS_OP_MATVEC; o.in_kind = DS_IN_PLAIN; o.K = (int) K; o.nmat = 2; o.epilogue = DS_EP_SILU_MUL;
    o.in0 = (const float *) dx.p;
    o.W[0] = dg.p; o.W[1] = du.p;
    for (int i = 0; i < 2; ++i) { o.type[i] = type; o.M[i] = (int) M; o.w_nb1[i] = (int64_t) rb; }
    o.act_out = (float *) dd.p;
    if (int rc = run_phases({o})) return rc;
    if (!dd.get(dst, M * 4)) { cudaGetLastError(); return ds_fail(B200_E_BAD_ARG, "copy back failed"); }
    return 0;
}

API int b200_decode_step_qkv_host(int type_qk, int type_v, const void * Wq, const void * Wk, const void * Wv, int64_t n_head, int64_t n_head_kv,
                                  int64_t K, const float * x, const float * norm_w, float eps, int32_t pos, int n_dims, float freq_base,
                                  const float * freq_factors, float * q_out, void * k_row_f16, void * v_row_f16) {
    const int64_t D = 128, Mq = n_head * D, Mkv = n_head_kv * D;
    if (K <= 0 || K % 256 || n_head <= 0 || n_head_kv <= 0 || !norm_w || n_dims <= 0 || n_dims > D || (n_dims & 1)) return ds_fail(B200_E_BAD_ARG, "bad shape");
    const size_t rbq = row_bytes(type_qk, K), rbv = row_bytes(type_v, K);
    Dev dq, dk, dv, dx, dn, dpos, dff, oq, ok, ov;
    if (!dq.put(Wq, rbq * Mq) || !dk.put(Wk, rbq * Mkv) || !dv.put(Wv, rbv * Mkv) || !dx.put(x, K * 4) || !dn.put(norm_w, K * 4) ||
        !dpos.put(&pos, 4) || (freq_factors && !dff.put(freq_factors, n_dims / 2 * 4)) || !oq.alloc(Mq * 4) || !ok.alloc(Mkv * 2) || !ov.alloc(Mkv * 2)) {
        cudaGetLastError();
        return ds_fail(B200_E_SCRATCH, "device allocation failed");
    }
    DsOp o; memset(&o, 0, sizeof(o));
    o.kind = DS_OP_MATVEC; o.in_kind = DS_IN_NORM; o.K = (int) K; o.nmat = 3; o.epilogue = DS_EP_ROPE_KV;
    o.in0 = (const float *) dx.p; o.norm_w = (const float *) dn.p; o.eps = eps;
    o.W[0] = dq.p; o.W[1] = dk.p; o.W[2] = dv.p;
    o.type[0] = o.type[1] = type_qk; o.type[2] = type_v;
    o.M[0] = (int) Mq; o.M[1] = o.M[2] = (int) Mkv;
    o.w_nb1[0] = o.w_nb1[1] = (int64_t) rbq; o.w_nb1[2] = (int64_t) rbv;
    o.q_rope = (float *) oq.p; o.k_cache = ok.p; o.v_cache = ov.p;
    o.pos = (const int32_t *) dpos.p; o.ff = freq_factors ? (const float *) dff.p : nullptr;
    o.head_dim = (int) D; o.n_dims = n_dims; o.freq_scale = 1.0f; o.ext_factor = 0.0f; o.attn_factor = 1.0f;
    o.theta_scale = powf(freq_base, -2.0f / (float) n_dims);
    if (int rc = run_phases({o})) return rc;
    if (!oq.get(q_out, Mq * 4) || !ok.get(k_row_f16, Mkv * 2) || !ov.get(v_row_f16, Mkv * 2)) { cudaGetLastError(); return ds_fail(B200_E_BAD_ARG, "copy back failed"); }
    return 0;
}

API int b200_decode_step_attention_host(const float * q, const void * k_f16, const void * v_f16, const void * mask_f16, int64_t n_kv,
                                        int64_t n_head, int64_t n_head_kv, float scale, int n_slices, int merge_in_next_phase, float * dst) {
    const int64_t D = 128;
    if (n_kv <= 0 || n_head <= 0 || n_head_kv <= 0 || n_head % n_head_kv || n_head_kv > 64 || n_slices < 1 || n_slices > 128) return ds_fail(B200_E_BAD_ARG, "bad shape");
    const int64_t gqa = n_head / n_head_kv;
    Dev dq, dk, dv, dm, dd, dp, dt;
    if (!dq.put(q, n_head * D * 4) || !dk.put(k_f16, n_head_kv * n_kv * D * 2) || !dv.put(v_f16, n_head_kv * n_kv * D * 2) ||
        (mask_f16 && !dm.put(mask_f16, n_kv * 2)) || !dd.alloc(n_head * D * 4) || !dp.alloc((size_t) n_head_kv * n_slices * gqa * DS_PARTIAL_STRIDE * 4) || !dt.alloc(256)) {
        cudaGetLastError();
        return ds_fail(B200_E_SCRATCH, "device allocation failed");
    }
    DsOp a; memset(&a, 0, sizeof(a));
    a.kind = DS_OP_ATTN;
    a.q = (const float *) dq.p;
    a.k = (const char *) dk.p; a.k_nb1 = D * 2; a.k_nb2 = n_kv * D * 2;
    a.v = (const char *) dv.p; a.v_nb1 = D * 2; a.v_nb2 = n_kv * D * 2;
    a.mask = mask_f16 ? dm.p : nullptr;
    a.n_kv = (int) n_kv; a.n_head = (int) n_head; a.n_head_kv = (int) n_head_kv; a.scale = scale;
    a.n_slices = n_slices; a.kv_per_slice = (int) ((n_kv + n_slices - 1) / n_slices);
    a.partials = (float *) dp.p; a.tickets = (unsigned *) dt.p; a.out = (float *) dd.p;
    if (n_slices > 1 && n_slices <= DS_MAX_MERGE_SLICES && merge_in_next_phase) {
        // the slices are merged by the input stage of a following mat-vec phase; an identity-free way to observe the
        // merged vector is that phase's optional copy of its input (y_out); the mat-vec itself multiplies a tiny
        // all-zero Q4_K matrix
        a.consumer_merge = 1;
        Dev dw, dz;
        const int64_t K = n_head * D;
        if (!dw.alloc((size_t) 2 * (K / 256) * 144) || !dz.alloc(16)) { cudaGetLastError(); return ds_fail(B200_E_SCRATCH, "device allocation failed"); }
        DsOp c; memset(&c, 0, sizeof(c));
        c.kind = DS_OP_MATVEC; c.in_kind = DS_IN_ATTN; c.K = (int) K; c.nmat = 1; c.epilogue = DS_EP_STORE;
        c.in0 = a.partials; c.in_slices = n_slices; c.in_gqa = (int) gqa; c.y_out = (float *) dd.p;
        c.W[0] = dw.p; c.type[0] = T_Q4_K; c.M[0] = 2; c.w_nb1[0] = (K / 256) * 144; c.dst[0] = (float *) dz.p;
        if (int rc = run_phases({a, c})) return rc;
    } else if (int rc = run_phases({a})) return rc;
    if (!dd.get(dst, n_head * D * 4)) { cudaGetLastError(); return ds_fail(B200_E_BAD_ARG, "copy back failed"); }
    return 0;
}
