// Flat C-ABI declared in include/b200_kernels.h: thin argument marshalling over
// the kernel launchers.  The `_host` forms own their device memory for the
// duration of the call; the device forms allocate nothing per call (their first
// call on a device creates a status word and the attention kernel's counters).
#include "common.cuh"
#include "kernels.h"
#include "b200_kernels.h"

#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

using namespace b200;

#define API extern "C" __attribute__((visibility("default")))

static thread_local std::string g_err;
static int fail(int code, const char * msg) { g_err = msg; return code; }
static int fail_cuda(cudaError_t e, const char * what) {
    g_err = std::string(what) + ": " + cudaGetErrorString(e);
    cudaGetLastError();
    return (int) e;
}
#define CK(expr) do { cudaError_t e_ = (expr); if (e_ != cudaSuccess) return fail_cuda(e_, #expr); } while (0)

API const char * b200_last_error(void) { return g_err.c_str(); }

API int b200_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) { cudaGetLastError(); return 0; }
    int found = 0;
    for (int i = 0; i < n; ++i) {
        int major = 0;
        if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, i) == cudaSuccess && major == 10) ++found;
    }
    return found;
}

API size_t b200_row_size(int type, int64_t k) {
    const int be = type_block_elems(type);
    return be ? (size_t) (k / be) * type_block_bytes(type) : 0;
}

// per-device launch context for the flat API: SM count and a status word
struct ApiDev { int sm_count = 0; int * status = nullptr; unsigned * tickets = nullptr; bool ready = false; };
static ApiDev g_dev[64];

static int g_flat_pdl = 0;      // programmatic dependent launch for the device-pointer entry points (b200_set_dependent_launch)
static int get_ctx(void * stream, LaunchCtx & lc) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); return fail(B200_E_NO_DEVICE, "no CUDA device"); }
    ApiDev & d = g_dev[dev & 63];
    if (!d.ready) {
        int major = 0;
        CK(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
        if (major != 10) return fail(B200_E_NO_DEVICE, "current device is not sm_100");
        CK(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev));
        CK(cudaMalloc((void **) &d.status, sizeof(int)));
        CK(cudaMemset(d.status, 0, sizeof(int)));
        CK(cudaMalloc((void **) &d.tickets, sizeof(unsigned) * FATTN_DEC_TICKETS));
        CK(cudaMemset(d.tickets, 0, sizeof(unsigned) * FATTN_DEC_TICKETS));
        d.ready = true;
    }
    lc.stream = (cudaStream_t) stream; lc.device = dev; lc.sm_count = d.sm_count; lc.status = d.status; lc.use_pdl = g_flat_pdl; lc.fa_tickets = d.tickets;
    return 0;
}
API void b200_set_dependent_launch(int on) { g_flat_pdl = on ? 1 : 0; }

static int check_status(const LaunchCtx & lc) {
    int st = 0;
    CK(cudaMemcpy(&st, lc.status, sizeof(int), cudaMemcpyDeviceToHost));
    if (st != 0) { cudaMemset(lc.status, 0, sizeof(int)); return fail(B200_E_DEVICE_WAIT, "a kernel gave up a bounded wait"); }
    return 0;
}

// RAII device allocation for the _host entry points
struct DevBuf {
    void * p = nullptr;
    cudaError_t alloc(size_t n) { return cudaMalloc(&p, n ? n + 256 : 256); }
    ~DevBuf() { if (p) cudaFree(p); }
};

static TensorD desc(void * data, int type, int64_t ne0, int64_t ne1, int64_t ne2, int64_t nb1, int64_t nb2) {
    TensorD d;
    d.data = data; d.type = type;
    d.ne[0] = ne0; d.ne[1] = ne1; d.ne[2] = ne2; d.ne[3] = 1;
    d.nb[0] = type_block_bytes(type); d.nb[1] = nb1; d.nb[2] = nb2; d.nb[3] = nb2 * ne2;
    return d;
}

// ---------------------------------------------------------------------------
// MUL_MAT
// ---------------------------------------------------------------------------
// The kernels issue 16-byte bulk copies / vector loads from the activation blocks and 4-byte accesses to X and dst:
// a misaligned caller pointer would raise a sticky device error, so it is refused here, before any launch.
static bool aligned_to(const void * p, size_t a) { return p && ((uintptr_t) p & (a - 1)) == 0; }
static constexpr int64_t I32_MAX = 0x7fffffff;
static constexpr int FLAT_SPLITK_SMS = 148;       // what b200_mul_mat_q_scratch_bytes sizes the split-K partial tiles for

API size_t b200_mul_mat_q_scratch_bytes(int type, int64_t M, int64_t K, int64_t N) {
    (void) M;
    size_t s = act128_bytes(K, N);
    if (mmq_tc_supported(type, M, N, K)) { const size_t t = mmq_tc_workspace_bytes(N, K) + mmq_tc_partial_bytes(M, N, K, FLAT_SPLITK_SMS); if (t > s) s = t; }
    return s;
}

API int b200_mul_mat_q(int type, const void * W, int64_t w_nb1, int64_t M, int64_t K, const float * X, int64_t x_stride, int64_t N,
                       float * dst, int64_t dst_stride, void * scratch, size_t scratch_bytes, void * stream) {
    if (!mmvq_type_supported(type)) return fail(B200_E_UNSUPPORTED, "weight type not supported");
    if (K <= 0 || M <= 0 || N <= 0 || K % type_block_elems(type) != 0) return fail(B200_E_BAD_ARG, "bad shape");
    if (scratch_bytes < b200_mul_mat_q_scratch_bytes(type, M, K, N)) return fail(B200_E_SCRATCH, "scratch buffer too small");
    if (M > I32_MAX || K > I32_MAX || x_stride < K || dst_stride < M || w_nb1 < (int64_t) b200_row_size(type, K))
        return fail(B200_E_BAD_ARG, "strides shorter than a row / column, or a dimension beyond 2^31-1");
    if (!aligned_to(W, 2) || (w_nb1 & 1) || !aligned_to(X, 4) || !aligned_to(dst, 4) || !aligned_to(scratch, 16))
        return fail(B200_E_BAD_ARG, "null or misaligned pointer (weights 2, X and dst 4, scratch 16 bytes)");
    LaunchCtx lc; int rc = get_ctx(stream, lc); if (rc) return rc;
    const bool s8 = mmq_s8_shape_ok(type, N, K) && aligned_to(W, 16) && (w_nb1 & 15) == 0;      // a few columns: the integer tensor-core kernel
    if (!s8 && mmq_tc_supported(type, M, N, K) && mmq_tc_ptr_ok(type, W, w_nb1, X, x_stride * 4)) {
        // split-K partial tiles: never more than the scratch size function allowed for, whatever this device's SM count
        LaunchCtx tc = lc;
        if (tc.sm_count > FLAT_SPLITK_SMS) tc.sm_count = FLAT_SPLITK_SMS;
        const size_t pb = mmq_tc_partial_bytes(M, N, K, tc.sm_count);
        // (a device with fewer SMs may want more partial tiles than the scratch holds: then K is not divided)
        void * partials = pb && mmq_tc_workspace_bytes(N, K) + pb <= scratch_bytes ? (char *) scratch + mmq_tc_workspace_bytes(N, K) : nullptr;
        CK(launch_mmq_tc(type, W, w_nb1, X, x_stride * 4, dst, dst_stride * 4, M, N, K, scratch, tc, false, partials));
        return 0;
    }
    CK(launch_quantize_act128(X, N, 1, 1, x_stride, 0, 0, scratch, (int) K, lc.stream));
    MmvqArgs a = {};
    a.type = type; a.W = W; a.w_nb1 = w_nb1; a.Xq = scratch; a.M = (int) M; a.K = (int) K;
    a.ne12 = 1; a.ne13 = 1; a.r2 = 1; a.r3 = 1; a.x_ncols = (int) N; a.xq_ne12 = 1;
    a.dst_nb1 = dst_stride * 4;
    a.status = lc.status; a.sm_count = lc.sm_count; a.device = lc.device; a.use_pdl = lc.use_pdl;
    a.dst = dst;
    if (s8 && mmq_s8_applicable(a, N)) {
        CK(launch_mmq_s8(a, N, lc.stream));
        return 0;
    }
    for (int64_t n0 = 0; n0 < N; n0 += 8) {
        a.N = (int) (N - n0 < 8 ? N - n0 : 8);
        a.x_col0 = (int) n0;
        a.dst = dst + n0 * dst_stride;
        CK(launch_mmvq(a, lc.stream));
    }
    return 0;
}

API size_t b200_act_bytes(int64_t K, int64_t N) { return act128_bytes(K, N); }

API int b200_quantize_act(const float * X, int64_t x_stride, int64_t K, int64_t N, void * xq, void * stream) {
    if (K <= 0 || N <= 0 || K > I32_MAX || x_stride < K) return fail(B200_E_BAD_ARG, "bad shape");
    if (!aligned_to(X, 4) || !aligned_to(xq, 16)) return fail(B200_E_BAD_ARG, "null or misaligned pointer (X 4, xq 16 bytes)");
    LaunchCtx lc; int rc = get_ctx(stream, lc); if (rc) return rc;
    CK(launch_quantize_act128(X, N, 1, 1, x_stride, 0, 0, xq, (int) K, lc.stream));
    return 0;
}

API int b200_mul_mat_vec_q(int type, const void * W, int64_t w_nb1, int64_t M, int64_t K, const void * xq, int64_t N,
                           float * dst, int64_t dst_stride, void * stream) {
    if (!mmvq_type_supported(type)) return fail(B200_E_UNSUPPORTED, "weight type not supported");
    if (K <= 0 || M <= 0 || N <= 0 || N > 8 || K % type_block_elems(type) != 0) return fail(B200_E_BAD_ARG, "bad shape");
    if (M > I32_MAX || K > I32_MAX || dst_stride < M || w_nb1 < (int64_t) b200_row_size(type, K)) return fail(B200_E_BAD_ARG, "strides shorter than a row / column, or a dimension beyond 2^31-1");
    if (!aligned_to(W, 2) || (w_nb1 & 1) || !aligned_to(xq, 16) || !aligned_to(dst, 4)) return fail(B200_E_BAD_ARG, "null or misaligned pointer (weights 2, xq 16, dst 4 bytes)");
    LaunchCtx lc; int rc = get_ctx(stream, lc); if (rc) return rc;
    MmvqArgs a = {};
    a.type = type; a.W = W; a.w_nb1 = w_nb1; a.Xq = xq; a.M = (int) M; a.K = (int) K; a.N = (int) N;
    a.ne12 = 1; a.ne13 = 1; a.r2 = 1; a.r3 = 1; a.x_ncols = (int) N; a.xq_ne12 = 1; a.x_col0 = 0;
    a.dst = dst; a.dst_nb1 = dst_stride * 4;
    a.status = lc.status; a.sm_count = lc.sm_count; a.device = lc.device; a.use_pdl = lc.use_pdl;
    CK(launch_mmvq(a, lc.stream));
    return 0;
}

API int b200_mul_mat_q_host(int type, const void * W, int64_t M, int64_t K, const float * X, int64_t N, float * dst) {
    if (!mmvq_type_supported(type)) return fail(B200_E_UNSUPPORTED, "weight type not supported");
    if (K <= 0 || M <= 0 || N <= 0 || K % type_block_elems(type) != 0) return fail(B200_E_BAD_ARG, "bad shape");
    LaunchCtx lc; int rc = get_ctx(nullptr, lc); if (rc) return rc;
    const size_t rb = b200_row_size(type, K), sb = b200_mul_mat_q_scratch_bytes(type, M, K, N);
    DevBuf dw, dx, dd, ds;
    CK(dw.alloc(rb * M)); CK(dx.alloc((size_t) K * N * 4)); CK(dd.alloc((size_t) M * N * 4)); CK(ds.alloc(sb));
    CK(cudaMemcpy(dw.p, W, rb * M, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(dx.p, X, (size_t) K * N * 4, cudaMemcpyHostToDevice));
    rc = b200_mul_mat_q(type, dw.p, (int64_t) rb, M, K, (const float *) dx.p, K, N, (float *) dd.p, M, ds.p, sb, nullptr);
    if (rc) return rc;
    CK(cudaDeviceSynchronize());
    CK(cudaMemcpy(dst, dd.p, (size_t) M * N * 4, cudaMemcpyDeviceToHost));
    return check_status(lc);
}

// ---------------------------------------------------------------------------
// FLASH_ATTN_EXT
// ---------------------------------------------------------------------------
static void fa_descs(const float * q, int64_t q_nb1, int64_t q_nb2, const void * k, int64_t k_nb1, int64_t k_nb2,
                     const void * v, int64_t v_nb1, int64_t v_nb2, const void * mask, int64_t m_nb1, float * dst,
                     int64_t D, int64_t n_q, int64_t n_head, int64_t n_kv, int64_t n_head_kv,
                     TensorD & qd, TensorD & kd, TensorD & vd, TensorD & md, TensorD & dd) {
    qd = desc((void *) q, T_F32, D, n_q, n_head, q_nb1, q_nb2);
    kd = desc((void *) k, T_F16, D, n_kv, n_head_kv, k_nb1, k_nb2);
    vd = desc((void *) v, T_F16, D, n_kv, n_head_kv, v_nb1, v_nb2);
    md = desc((void *) mask, T_F16, n_kv, n_q, 1, m_nb1, m_nb1 * n_q);
    dd = desc((void *) dst, T_F32, D, n_head, n_q, D * 4, D * 4 * n_head);
}

API size_t b200_flash_attn_scratch_bytes(int64_t D, int64_t n_q, int64_t n_head, int64_t n_kv) {
    int dev = 0, sm = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sm, cudaDevAttrMultiProcessorCount, dev); else cudaGetLastError();
    // the number of KV heads is not an argument: take the largest need over every grouping of the query heads
    size_t need = 0;
    for (int64_t hkv = 1; hkv <= n_head; ++hkv) {
        if (n_head % hkv) continue;
        TensorD qd = desc(nullptr, T_F32, D, n_q, n_head, 0, 0), kd = desc(nullptr, T_F16, D, n_kv, hkv, 0, 0);
        const size_t b = fattn_workspace_bytes(qd, kd, sm);
        if (b > need) need = b;
    }
    return need;
}

API int b200_flash_attn(const float * q, int64_t q_nb1, int64_t q_nb2, const void * k, int64_t k_nb1, int64_t k_nb2,
                        const void * v, int64_t v_nb1, int64_t v_nb2, const void * mask, int64_t mask_nb1, float * dst,
                        int64_t D, int64_t n_q, int64_t n_head, int64_t n_kv, int64_t n_head_kv,
                        float scale, float max_bias, float softcap, void * scratch, size_t scratch_bytes, void * stream) {
    if (!fattn_supported(D, T_F16, T_F16)) return fail(B200_E_UNSUPPORTED, "head size not supported");
    if (n_head_kv <= 0 || n_head % n_head_kv != 0 || n_q <= 0 || n_kv <= 0) return fail(B200_E_BAD_ARG, "bad shape");
    LaunchCtx lc; int rc = get_ctx(stream, lc); if (rc) return rc;
    TensorD qd, kd, vd, md, dd;
    fa_descs(q, q_nb1, q_nb2, k, k_nb1, k_nb2, v, v_nb1, v_nb2, mask, mask_nb1, dst, D, n_q, n_head, n_kv, n_head_kv, qd, kd, vd, md, dd);
    if (scratch_bytes < fattn_workspace_bytes(qd, kd, lc.sm_count)) return fail(B200_E_SCRATCH, "scratch buffer too small");
    FattnParams fp{scale, max_bias, softcap};
    CK(launch_fattn(qd, kd, vd, mask ? &md : nullptr, dd, fp, scratch, lc));
    return 0;
}

API int b200_flash_attn_host(const float * q, const void * k, const void * v, const void * mask, float * dst,
                             int64_t D, int64_t n_q, int64_t n_head, int64_t n_kv, int64_t n_head_kv,
                             float scale, float max_bias, float softcap) {
    LaunchCtx lc; int rc = get_ctx(nullptr, lc); if (rc) return rc;
    const size_t qb = (size_t) D * n_q * n_head * 4, kb = (size_t) D * n_kv * n_head_kv * 2, mb = (size_t) n_kv * n_q * 2;
    const size_t sb = b200_flash_attn_scratch_bytes(D, n_q, n_head, n_kv);
    DevBuf dq, dk, dv, dm, dd, ds;
    CK(dq.alloc(qb)); CK(dk.alloc(kb)); CK(dv.alloc(kb)); CK(dm.alloc(mb)); CK(dd.alloc(qb)); CK(ds.alloc(sb));
    CK(cudaMemcpy(dq.p, q, qb, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(dk.p, k, kb, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(dv.p, v, kb, cudaMemcpyHostToDevice));
    if (mask) CK(cudaMemcpy(dm.p, mask, mb, cudaMemcpyHostToDevice));
    rc = b200_flash_attn((const float *) dq.p, D * 4, D * 4 * n_q, dk.p, D * 2, D * 2 * n_kv, dv.p, D * 2, D * 2 * n_kv,
                         mask ? dm.p : nullptr, n_kv * 2, (float *) dd.p, D, n_q, n_head, n_kv, n_head_kv,
                         scale, max_bias, softcap, ds.p, sb, nullptr);
    if (rc) return rc;
    CK(cudaDeviceSynchronize());
    CK(cudaMemcpy(dst, dd.p, qb, cudaMemcpyDeviceToHost));
    return 0;
}

// ---------------------------------------------------------------------------
// conversions
// ---------------------------------------------------------------------------
API int b200_get_rows_host(int type, const void * src, int64_t n_src_rows, int64_t k, const int32_t * idx, int64_t n_idx, float * dst) {
    if (!get_rows_supported(type)) return fail(B200_E_UNSUPPORTED, "type not supported");
    if (k <= 0 || k % type_block_elems(type) != 0 || n_idx <= 0) return fail(B200_E_BAD_ARG, "bad shape");
    LaunchCtx lc; int rc = get_ctx(nullptr, lc); if (rc) return rc;
    const size_t rb = b200_row_size(type, k);
    DevBuf ds, di, dd;
    CK(ds.alloc(rb * n_src_rows)); CK(di.alloc(n_idx * 4)); CK(dd.alloc((size_t) k * n_idx * 4));
    CK(cudaMemcpy(ds.p, src, rb * n_src_rows, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(di.p, idx, n_idx * 4, cudaMemcpyHostToDevice));
    TensorD sd = desc(ds.p, type, k, n_src_rows, 1, rb, rb * n_src_rows);
    TensorD id = desc(di.p, T_I32, n_idx, 1, 1, n_idx * 4, n_idx * 4);
    TensorD dd_ = desc(dd.p, T_F32, k, n_idx, 1, k * 4, k * 4 * n_idx);
    CK(launch_get_rows(sd, id, dd_, lc));
    CK(cudaDeviceSynchronize());
    CK(cudaMemcpy(dst, dd.p, (size_t) k * n_idx * 4, cudaMemcpyDeviceToHost));
    return 0;
}

API int b200_dequantize_rows_host(int type, const void * src, int64_t n_rows, int64_t k, float * dst) {
    std::vector<int32_t> idx((size_t) n_rows);
    for (int64_t i = 0; i < n_rows; ++i) idx[(size_t) i] = (int32_t) i;
    return b200_get_rows_host(type, src, n_rows, k, idx.data(), n_rows, dst);
}

API int b200_quantize_rows_host(int type, const float * src, int64_t n_rows, int64_t k, void * dst) {
    if (!cpy_supported(T_F32, type) || type_block_elems(type) != 32) return fail(B200_E_UNSUPPORTED, "type not supported");
    if (k <= 0 || k % 32 != 0 || n_rows <= 0) return fail(B200_E_BAD_ARG, "bad shape");
    LaunchCtx lc; int rc = get_ctx(nullptr, lc); if (rc) return rc;
    const size_t rb = b200_row_size(type, k);
    DevBuf ds, dd;
    CK(ds.alloc((size_t) k * n_rows * 4)); CK(dd.alloc(rb * n_rows));
    CK(cudaMemcpy(ds.p, src, (size_t) k * n_rows * 4, cudaMemcpyHostToDevice));
    TensorD sd = desc(ds.p, T_F32, k, n_rows, 1, k * 4, k * 4 * n_rows);
    TensorD qd = desc(dd.p, type, k, n_rows, 1, rb, rb * n_rows);
    CK(launch_cpy(sd, qd, lc));
    CK(cudaDeviceSynchronize());
    CK(cudaMemcpy(dst, dd.p, rb * n_rows, cudaMemcpyDeviceToHost));
    return 0;
}

API int b200_f32_to_f16_host(const float * src, int64_t n, void * dst) {
    if (n <= 0) return fail(B200_E_BAD_ARG, "bad shape");
    LaunchCtx lc; int rc = get_ctx(nullptr, lc); if (rc) return rc;
    DevBuf ds, dd;
    CK(ds.alloc((size_t) n * 4)); CK(dd.alloc((size_t) n * 2));
    CK(cudaMemcpy(ds.p, src, (size_t) n * 4, cudaMemcpyHostToDevice));
    CK(launch_cpy(desc(ds.p, T_F32, n, 1, 1, n * 4, n * 4), desc(dd.p, T_F16, n, 1, 1, n * 2, n * 2), lc));
    CK(cudaDeviceSynchronize());
    CK(cudaMemcpy(dst, dd.p, (size_t) n * 2, cudaMemcpyDeviceToHost));
    return 0;
}

// ---------------------------------------------------------------------------
// glue ops
// ---------------------------------------------------------------------------
API int b200_rms_norm_host(const float * x, int64_t n_rows, int64_t k, float eps, const float * weight, float * dst) {
    if (n_rows <= 0 || k <= 0) return fail(B200_E_BAD_ARG, "bad shape");
    LaunchCtx lc; int rc = get_ctx(nullptr, lc); if (rc) return rc;
    DevBuf dx, dw, dd;
    CK(dx.alloc((size_t) k * n_rows * 4)); CK(dd.alloc((size_t) k * n_rows * 4)); CK(dw.alloc((size_t) k * 4));
    CK(cudaMemcpy(dx.p, x, (size_t) k * n_rows * 4, cudaMemcpyHostToDevice));
    TensorD xd = desc(dx.p, T_F32, k, n_rows, 1, k * 4, k * 4 * n_rows), dd_ = desc(dd.p, T_F32, k, n_rows, 1, k * 4, k * 4 * n_rows);
    if (weight) {
        CK(cudaMemcpy(dw.p, weight, (size_t) k * 4, cudaMemcpyHostToDevice));
        CK(launch_rms_norm_mul(xd, desc(dw.p, T_F32, k, 1, 1, k * 4, k * 4), dd_, eps, nullptr, nullptr, nullptr, nullptr, lc));
    } else {
        CK(launch_rms_norm(xd, dd_, eps, lc));
    }
    CK(cudaDeviceSynchronize());
    CK(cudaMemcpy(dst, dd.p, (size_t) k * n_rows * 4, cudaMemcpyDeviceToHost));
    return 0;
}

API int b200_rope_host(const float * x, int64_t head_dim, int64_t n_head, int64_t n_tok, const int32_t * pos, const float * ff,
                       int n_dims, int mode, int n_ctx_orig, float freq_base, float freq_scale, float ext_factor,
                       float attn_factor, float beta_fast, float beta_slow, float * dst) {
    if (head_dim <= 0 || head_dim % 2 || n_head <= 0 || n_tok <= 0 || n_dims > head_dim) return fail(B200_E_BAD_ARG, "bad shape");
    LaunchCtx lc; int rc = get_ctx(nullptr, lc); if (rc) return rc;
    const size_t nb = (size_t) head_dim * n_head * n_tok * 4;
    DevBuf dx, dp, df, dd;
    CK(dx.alloc(nb)); CK(dd.alloc(nb)); CK(dp.alloc(n_tok * 4)); CK(df.alloc((size_t) n_dims * 2));
    CK(cudaMemcpy(dx.p, x, nb, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(dp.p, pos, n_tok * 4, cudaMemcpyHostToDevice));
    if (ff) CK(cudaMemcpy(df.p, ff, (size_t) n_dims * 2, cudaMemcpyHostToDevice));
    RopeParams rp{n_dims, mode, n_ctx_orig, freq_base, freq_scale, ext_factor, attn_factor, beta_fast, beta_slow};
    TensorD xd = desc(dx.p, T_F32, head_dim, n_head, n_tok, head_dim * 4, head_dim * 4 * n_head);
    TensorD dd_ = desc(dd.p, T_F32, head_dim, n_head, n_tok, head_dim * 4, head_dim * 4 * n_head);
    CK(launch_rope(xd, (const int32_t *) dp.p, ff ? (const float *) df.p : nullptr, dd_, rp, lc));
    CK(cudaDeviceSynchronize());
    CK(cudaMemcpy(dst, dd.p, nb, cudaMemcpyDeviceToHost));
    return 0;
}

API int b200_silu_mul_host(const float * gate, const float * up, int64_t n, float * dst) {
    if (n <= 0) return fail(B200_E_BAD_ARG, "bad shape");
    LaunchCtx lc; int rc = get_ctx(nullptr, lc); if (rc) return rc;
    DevBuf dg, du, dd;
    CK(dg.alloc((size_t) n * 4)); CK(du.alloc((size_t) n * 4)); CK(dd.alloc((size_t) n * 4));
    CK(cudaMemcpy(dg.p, gate, (size_t) n * 4, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(du.p, up, (size_t) n * 4, cudaMemcpyHostToDevice));
    TensorD g = desc(dg.p, T_F32, n, 1, 1, n * 4, n * 4), u = desc(du.p, T_F32, n, 1, 1, n * 4, n * 4), d = desc(dd.p, T_F32, n, 1, 1, n * 4, n * 4);
    CK(launch_silu_mul(g, u, d, nullptr, nullptr, lc));
    CK(cudaDeviceSynchronize());
    CK(cudaMemcpy(dst, dd.p, (size_t) n * 4, cudaMemcpyDeviceToHost));
    return 0;
}

API int b200_soft_max_host(const float * x, int64_t n_rows, int64_t k, const void * mask, float scale, float * dst) {
    if (n_rows <= 0 || k <= 0) return fail(B200_E_BAD_ARG, "bad shape");
    LaunchCtx lc; int rc = get_ctx(nullptr, lc); if (rc) return rc;
    const size_t nb = (size_t) k * n_rows * 4;
    DevBuf dx, dm, dd;
    CK(dx.alloc(nb)); CK(dd.alloc(nb)); CK(dm.alloc(nb / 2));
    CK(cudaMemcpy(dx.p, x, nb, cudaMemcpyHostToDevice));
    if (mask) CK(cudaMemcpy(dm.p, mask, nb / 2, cudaMemcpyHostToDevice));
    TensorD xd = desc(dx.p, T_F32, k, n_rows, 1, k * 4, nb), dd_ = desc(dd.p, T_F32, k, n_rows, 1, k * 4, nb);
    TensorD md = desc(dm.p, T_F16, k, n_rows, 1, k * 2, nb / 2);
    CK(launch_soft_max(xd, mask ? &md : nullptr, dd_, scale, 0.0f, lc));
    CK(cudaDeviceSynchronize());
    CK(cudaMemcpy(dst, dd.p, nb, cudaMemcpyDeviceToHost));
    return 0;
}

// ---------------------------------------------------------------------------
// the bounded wait of the cross-GPU barrier, on one GPU
// ---------------------------------------------------------------------------
// Runs the row-split barrier kernel (peer.cu) as rank 0 of 2 with both flag arrays in this GPU's memory.  With
// peer_arrives the "peer" has already published the epoch and the barrier passes; without, nothing ever writes the
// flag, the wait runs out after `spin_limit` polls, and the kernel records ERR_PEER_TIMEOUT and returns.
API int b200_tc_i8_probe_host(int kblocks, int reps, float * us_per_kblock, float * check, float * expected) {
    if (kblocks < 1 || kblocks > (1 << 20) || reps < 1 || !us_per_kblock || !check || !expected) return fail(B200_E_BAD_ARG, "bad probe arguments");
    LaunchCtx lc; int rc = get_ctx(nullptr, lc); if (rc) return rc;
    CK(launch_tc_i8_probe(kblocks, reps, us_per_kblock, check, expected, lc));
    return 0;
}

API int b200_peer_barrier_probe_host(int spin_limit, int peer_arrives, int * status_out) {
    LaunchCtx lc; int rc = get_ctx(nullptr, lc); if (rc) return rc;
    DevBuf flags, peer, epoch, status;
    CK(flags.alloc(256)); CK(peer.alloc(256)); CK(epoch.alloc(16)); CK(status.alloc(16));
    CK(cudaMemset(flags.p, 0, 256)); CK(cudaMemset(peer.p, 0, 256)); CK(cudaMemset(epoch.p, 0, 16)); CK(cudaMemset(status.p, 0, 16));
    if (peer_arrives) { const unsigned one = 1; CK(cudaMemcpy((unsigned *) flags.p + 1, &one, 4, cudaMemcpyHostToDevice)); }
    PeerBarrier b = {};
    b.epoch = (unsigned *) epoch.p; b.local_flags = (unsigned *) flags.p;
    b.peer_flags[0] = (unsigned *) flags.p; b.peer_flags[1] = (unsigned *) peer.p;
    b.rank = 0; b.n_ranks = 2; b.status = (int *) status.p; b.spin_limit = spin_limit;
    CK(launch_peer_barrier(b, lc));
    CK(cudaDeviceSynchronize());
    int st = 0;
    CK(cudaMemcpy(&st, status.p, sizeof(int), cudaMemcpyDeviceToHost));
    if (status_out) *status_out = st;
    return 0;
}
