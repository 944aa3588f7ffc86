// Test tool: hand-built ggml graphs with seeded data, computed on the reference's CPU backend (all host threads)
// and on a named device of whatever backends the registry loads, compared element by element.  It is the checker
// behind the full-size parity sweeps (every element of every output, not a sample of rows) and behind the
// graph-level cases that single-op tests cannot express (memory reused inside a graph).  Public ggml API only;
// built by oracle/ref.mk against the reference headers; test infrastructure.
//   graph_cases DEVICE SUITE [N_THREADS]
//   suites: mul_mat (the projection shapes x types x batch sizes), mul_mat_f16 (F16 / BF16 weights), mul_mat_id (experts), flash_attn, alias, attn_chain (attention as the model
//   graphs build it without FLASH_ATTN_EXT: MUL_MAT, SOFT_MAX, MUL_MAT on a transposed V cache, PERMUTE, CONT), split (weights in the device's
//   row-split buffer type, ggml_backend_split_buffer_type by name: a scatter / gather round trip and MUL_MAT)
// One line per case: "CASE <name> nmse=<x> max_abs=<y> n=<elements>"; with GRAPH_CASES_TIME set, a "TIME" line before it
#include "ggml.h"
#include "ggml-backend.h"

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <random>
#include <string>
#include <vector>

struct Input { ggml_tensor * t; std::vector<uint8_t> bytes; };
struct Built { std::vector<Input> inputs; std::vector<ggml_tensor *> outputs; ggml_cgraph * graph; size_t manual_bytes = 0;
               std::vector<std::pair<ggml_tensor *, size_t>> placement;      // manual placement: tensor -> offset (alias cases)
               std::vector<ggml_tensor *> split; };                           // tensors that go into the row-split buffer type on the device
using Builder = std::function<Built(ggml_context *)>;

static std::vector<float> normal(size_t n, float sigma, unsigned seed) {
    std::mt19937 rng(seed);
    std::normal_distribution<float> d(0.0f, sigma);
    std::vector<float> v(n);
    for (auto & x : v) x = d(rng);
    return v;
}
static std::vector<uint8_t> as_bytes(const std::vector<float> & v) {
    std::vector<uint8_t> b(v.size() * 4);
    memcpy(b.data(), v.data(), b.size());
    return b;
}
// `rows` rows of K weights ~ N(0, 0.02): 4096 distinct rows quantized with the reference's quantizer, repeated
static std::vector<uint8_t> quantized(ggml_type type, int64_t K, int64_t rows, unsigned seed) {
    const int64_t distinct = rows < 4096 ? rows : 4096;
    const size_t rb = ggml_row_size(type, K);
    std::vector<float> w = normal((size_t) distinct * K, 0.02f, seed);
    std::vector<uint8_t> q(rb * (size_t) distinct), out(rb * (size_t) rows);
    ggml_quantize_chunk(type, w.data(), q.data(), 0, distinct, K, nullptr);
    for (int64_t r = 0; r < rows; r += distinct) memcpy(out.data() + (size_t) r * rb, q.data(), rb * (size_t) std::min(distinct, rows - r));
    return out;
}

static ggml_backend_buffer_type_t g_split_buft = nullptr;      // set by the split suite; used for Built::split on the device only
static ggml_backend_t g_cpu, g_dev;
static int g_fail = 0;

static std::vector<std::vector<float>> run_on(ggml_backend_t backend, const Builder & build) {
    ggml_init_params ip = {ggml_tensor_overhead() * 64 + ggml_graph_overhead(), nullptr, true};
    ggml_context * ctx = ggml_init(ip);
    Built b = build(ctx);
    ggml_backend_buffer_t buf = nullptr;
    std::vector<ggml_backend_buffer_t> split_bufs;
    if (backend == g_dev && g_split_buft) for (ggml_tensor * w : b.split) {
        ggml_backend_buffer_t sb = ggml_backend_buft_alloc_buffer(g_split_buft, ggml_backend_buft_get_alloc_size(g_split_buft, w));
        if (!sb) { fprintf(stderr, "split buffer allocation failed\n"); exit(1); }
        ggml_backend_tensor_alloc(sb, w, ggml_backend_buffer_get_base(sb));
        split_bufs.push_back(sb);
    }
    if (b.manual_bytes) {
        buf = ggml_backend_alloc_buffer(backend, b.manual_bytes);
        char * base = (char *) ggml_backend_buffer_get_base(buf);
        for (auto & pl : b.placement) {
            if (pl.first->view_src) ggml_backend_view_init(pl.first);
            else ggml_backend_tensor_alloc(buf, pl.first, base + pl.second);
        }
    } else {
        buf = ggml_backend_alloc_ctx_tensors(ctx, backend);
    }
    if (!buf) { fprintf(stderr, "buffer allocation failed\n"); exit(1); }
    for (auto & in : b.inputs) ggml_backend_tensor_set(in.t, in.bytes.data(), 0, in.bytes.size());
    if (ggml_backend_graph_compute(backend, b.graph) != GGML_STATUS_SUCCESS) { fprintf(stderr, "graph_compute failed\n"); exit(1); }
    if (backend == g_dev && getenv("GRAPH_CASES_TIME")) {
        // host clock around repeated runs of the whole graph on the device (informational: "TIME <us per run>")
        ggml_backend_synchronize(backend);
        const int reps = 10;
        const int64_t t0 = ggml_time_us();
        for (int i = 0; i < reps; ++i) ggml_backend_graph_compute(backend, b.graph);
        ggml_backend_synchronize(backend);
        printf("TIME %.1f us per graph\n", (double) (ggml_time_us() - t0) / reps);
    }
    std::vector<std::vector<float>> outs;
    for (ggml_tensor * t : b.outputs) {
        std::vector<float> v((size_t) ggml_nelements(t));
        ggml_backend_tensor_get(t, v.data(), 0, v.size() * 4);
        outs.push_back(std::move(v));
    }
    if (backend == g_dev && g_split_buft) for (auto & in : b.inputs) {
        // what was scattered over the devices reads back as the same bytes
        bool is_split = false;
        for (ggml_tensor * w : b.split) if (w == in.t) is_split = true;
        if (!is_split) continue;
        std::vector<uint8_t> back(in.bytes.size());
        ggml_backend_tensor_get(in.t, back.data(), 0, back.size());
        const bool same = memcmp(back.data(), in.bytes.data(), back.size()) == 0;
        printf("ROUNDTRIP %s %s bytes=%zu\n", in.t->name, same ? "identical" : "DIFFERENT", back.size());
        if (!same) g_fail = 1;
    }
    ggml_backend_buffer_free(buf);
    for (ggml_backend_buffer_t sb : split_bufs) ggml_backend_buffer_free(sb);
    ggml_free(ctx);
    return outs;
}
static void run_case(const std::string & name, const Builder & build) {
    auto want = run_on(g_cpu, build), got = run_on(g_dev, build);
    double num = 0, den = 0, mx = 0; size_t n = 0; bool finite = true;
    for (size_t o = 0; o < want.size(); ++o)
        for (size_t i = 0; i < want[o].size(); ++i) {
            const double a = want[o][i], c = got[o][i];
            if (!std::isfinite(c)) finite = false;
            num += (a - c) * (a - c); den += a * a; mx = std::max(mx, std::fabs(a - c)); ++n;
        }
    printf("CASE %s nmse=%.3e max_abs=%.3e n=%zu%s\n", name.c_str(), den > 0 ? num / den : num, mx, n, finite ? "" : " NONFINITE");
    fflush(stdout);
    if (!finite) g_fail = 1;
}

// ---- suites ----
static void suite_mul_mat() {
    const ggml_type types[] = {GGML_TYPE_Q4_K, GGML_TYPE_Q6_K, GGML_TYPE_Q8_0, GGML_TYPE_Q4_0};
    const int64_t shapes[][2] = {{4096, 4096}, {4096, 14336}, {14336, 4096}, {4096, 128256}};     // K, M
    const int64_t batches[] = {1, 8, 32, 128, 512};
    for (ggml_type type : types) for (auto & sh : shapes) for (int64_t N : batches) {
        if (type == GGML_TYPE_Q4_0 && !(sh[0] == 4096 && sh[1] == 4096 && (N == 1 || N == 512))) continue;      // the single-op configuration
        const int64_t K = sh[0], M = sh[1];
        run_case(std::string("mul_mat.") + ggml_type_name(type) + ".k" + std::to_string(K) + ".m" + std::to_string(M) + ".n" + std::to_string(N), [=](ggml_context * ctx) {
            Built b;
            ggml_tensor * w = ggml_new_tensor_2d(ctx, type, K, M), * x = ggml_new_tensor_2d(ctx, GGML_TYPE_F32, K, N);
            ggml_tensor * y = ggml_mul_mat(ctx, w, x);
            b.graph = ggml_new_graph(ctx);
            ggml_build_forward_expand(b.graph, y);
            b.inputs.push_back({w, quantized(type, K, M, 7)});
            b.inputs.push_back({x, as_bytes(normal((size_t) K * N, 1.0f, 11 + (unsigned) N))});
            b.outputs = {y};
            return b;
        });
    }
}

// 16-bit weight matrices: the warp-per-row mat-vec (at most 8 columns) and the tcgen05 GEMM, row counts off the tile size
static void suite_mul_mat_f16() {
    for (ggml_type type : {GGML_TYPE_F16, GGML_TYPE_BF16}) for (int64_t N : {1, 3, 8, 9, 64, 200, 512}) {
        const int64_t K = 4096, M = 4096 + 200;
        run_case(std::string("mul_mat_f16.") + ggml_type_name(type) + ".n" + std::to_string(N), [=](ggml_context * ctx) {
            Built b;
            ggml_tensor * w = ggml_new_tensor_2d(ctx, type, K, M), * x = ggml_new_tensor_2d(ctx, GGML_TYPE_F32, K, N);
            ggml_tensor * y = ggml_mul_mat(ctx, w, x);
            b.graph = ggml_new_graph(ctx);
            ggml_build_forward_expand(b.graph, y);
            std::vector<float> wf = normal((size_t) K * M, 0.02f, 5);
            std::vector<uint8_t> wb((size_t) K * M * 2);
            if (type == GGML_TYPE_F16) ggml_fp32_to_fp16_row(wf.data(), (ggml_fp16_t *) wb.data(), K * M);
            else ggml_fp32_to_bf16_row(wf.data(), (ggml_bf16_t *) wb.data(), K * M);
            b.inputs.push_back({w, wb});
            b.inputs.push_back({x, as_bytes(normal((size_t) K * N, 1.0f, 11 + (unsigned) N))});
            b.outputs = {y};
            return b;
        });
    }
}

// MUL_MAT_ID: a mixture-of-experts projection for one token, a few, and a prompt (many pairs take the batched path), with
// src1 broadcast over the slots (ne11 = 1, the gate/up form) and per-slot (ne11 = n_used, the down form); one expert unused
static void suite_mul_mat_id() {
    const int64_t n_expert = 8, n_used = 2, K = 2048, M = 1024 + 64;
    for (ggml_type type : {GGML_TYPE_Q4_K, GGML_TYPE_Q6_K, GGML_TYPE_Q8_0}) for (int64_t n_tok : {1, 7, 64, 512}) for (int per_slot = 0; per_slot < 2; ++per_slot) {
        run_case(std::string("mul_mat_id.") + ggml_type_name(type) + ".tok" + std::to_string(n_tok) + (per_slot ? ".per_slot" : ".broadcast"), [=](ggml_context * ctx) {
            Built b;
            ggml_tensor * as = ggml_new_tensor_3d(ctx, type, K, M, n_expert);
            ggml_tensor * x = ggml_new_tensor_3d(ctx, GGML_TYPE_F32, K, per_slot ? n_used : 1, n_tok);
            ggml_tensor * ids = ggml_new_tensor_2d(ctx, GGML_TYPE_I32, n_used, n_tok);
            ggml_tensor * y = ggml_mul_mat_id(ctx, as, x, ids);
            b.graph = ggml_new_graph(ctx);
            ggml_build_forward_expand(b.graph, y);
            b.inputs.push_back({as, quantized(type, K, M * n_expert, 7)});
            b.inputs.push_back({x, as_bytes(normal((size_t) K * (per_slot ? n_used : 1) * n_tok, 1.0f, 11 + (unsigned) n_tok))});
            std::vector<int32_t> idv((size_t) n_used * n_tok);
            std::mt19937 rng(5 + (unsigned) n_tok);
            for (int64_t t = 0; t < n_tok; ++t) {                       // two different experts per token, expert 7 never
                const int a = (int) (rng() % 7), c = (a + 1 + (int) (rng() % 6)) % 7;
                idv[(size_t) t * n_used] = a; idv[(size_t) t * n_used + 1] = c;
            }
            std::vector<uint8_t> ib(idv.size() * 4);
            memcpy(ib.data(), idv.data(), ib.size());
            b.inputs.push_back({ids, ib});
            b.outputs = {y};
            return b;
        });
    }
}

static void suite_flash_attn() {
    const int64_t D = 128, n_head = 32, n_head_kv = 8;
    for (int64_t n_kv : {512, 4096, 32768}) for (int64_t n_q : {1, 512}) {
        run_case("flash_attn.kv" + std::to_string(n_kv) + ".q" + std::to_string(n_q), [=](ggml_context * ctx) {
            Built b;
            const int64_t n_pad = (n_q + 63) / 64 * 64;
            ggml_tensor * q = ggml_new_tensor_3d(ctx, GGML_TYPE_F32, D, n_q, n_head);
            ggml_tensor * k = ggml_new_tensor_3d(ctx, GGML_TYPE_F16, D, n_kv, n_head_kv), * v = ggml_new_tensor_3d(ctx, GGML_TYPE_F16, D, n_kv, n_head_kv);
            ggml_tensor * mask = ggml_new_tensor_2d(ctx, GGML_TYPE_F16, n_kv, n_pad);
            ggml_tensor * y = ggml_flash_attn_ext(ctx, q, k, v, mask, 1.0f / std::sqrt((float) D), 0.0f, 0.0f);
            ggml_flash_attn_ext_set_prec(y, GGML_PREC_F32);
            b.graph = ggml_new_graph(ctx);
            ggml_build_forward_expand(b.graph, y);
            auto half = [](const std::vector<float> & f) { std::vector<uint8_t> h(f.size() * 2); ggml_fp32_to_fp16_row(f.data(), (ggml_fp16_t *) h.data(), (int64_t) f.size()); return h; };
            b.inputs.push_back({q, as_bytes(normal((size_t) (D * n_q * n_head), 1.0f, 21))});
            b.inputs.push_back({k, half(normal((size_t) (D * n_kv * n_head_kv), 1.0f, 22))});
            b.inputs.push_back({v, half(normal((size_t) (D * n_kv * n_head_kv), 1.0f, 23))});
            std::vector<float> m((size_t) (n_kv * n_pad), -INFINITY);                 // causal: query i sees keys 0 .. n_kv - n_q + i
            for (int64_t i = 0; i < n_q; ++i) for (int64_t j = 0; j <= n_kv - n_q + i; ++j) m[(size_t) (i * n_kv + j)] = 0.0f;
            b.inputs.push_back({mask, half(m)});
            b.outputs = {y};
            return b;
        });
    }
}

// graphs whose memory is reused while they run
static void suite_alias() {
    const int64_t K = 4096, M = 512;
    // a mat-mul input is changed in place through a view at a non-zero offset between two mat-muls that read it:
    // conversions of the input cached by its start address would be stale
    run_case("alias.inplace_view_between_mul_mats", [=](ggml_context * ctx) {
        Built b;
        ggml_tensor * w = ggml_new_tensor_2d(ctx, GGML_TYPE_Q4_K, K, M), * x = ggml_new_tensor_2d(ctx, GGML_TYPE_F32, K, 1);
        ggml_tensor * c = ggml_new_tensor_1d(ctx, GGML_TYPE_F32, K / 2);
        ggml_tensor * y1 = ggml_mul_mat(ctx, w, x);
        ggml_tensor * xv = ggml_view_1d(ctx, x, K / 2, (size_t) (K / 2) * 4);
        ggml_tensor * upd = ggml_add_inplace(ctx, xv, c);
        ggml_tensor * y2 = ggml_mul_mat(ctx, w, x);
        b.graph = ggml_new_graph(ctx);
        ggml_build_forward_expand(b.graph, y1);
        ggml_build_forward_expand(b.graph, upd);
        ggml_build_forward_expand(b.graph, y2);
        b.inputs.push_back({w, quantized(GGML_TYPE_Q4_K, K, M, 3)});
        b.inputs.push_back({x, as_bytes(normal((size_t) K, 1.0f, 4))});
        b.inputs.push_back({c, as_bytes(normal((size_t) K / 2, 1.0f, 5))});
        b.outputs = {y1, y2};
        return b;
    });
    // q = Wq x ; r = scale(q) ; k = Wk x placed in q's memory (free once r has read it) ; out = r + k.  A backend
    // that groups the two mat-muls on x into one launch must not let k overwrite q before r has read it.
    run_case("alias.grouped_mul_mat_into_freed_memory", [=](ggml_context * ctx) {
        Built b;
        ggml_tensor * wq = ggml_new_tensor_2d(ctx, GGML_TYPE_Q4_K, K, M), * wk = ggml_new_tensor_2d(ctx, GGML_TYPE_Q4_K, K, M);
        ggml_tensor * x = ggml_new_tensor_2d(ctx, GGML_TYPE_F32, K, 1);
        ggml_tensor * q = ggml_mul_mat(ctx, wq, x);
        ggml_tensor * r = ggml_scale(ctx, q, 0.5f);
        ggml_tensor * k = ggml_mul_mat(ctx, wk, x);
        ggml_tensor * out = ggml_add(ctx, r, k);
        b.graph = ggml_new_graph(ctx);
        ggml_build_forward_expand(b.graph, q);
        ggml_build_forward_expand(b.graph, r);
        ggml_build_forward_expand(b.graph, k);
        ggml_build_forward_expand(b.graph, out);
        const size_t wb = ggml_nbytes(wq);
        size_t off = 0;
        auto put = [&](ggml_tensor * t, size_t at) { b.placement.push_back({t, at}); };
        put(wq, off); off += (wb + 255) / 256 * 256;
        put(wk, off); off += (wb + 255) / 256 * 256;
        put(x, off); off += (size_t) K * 4;
        const size_t q_at = off; off += (size_t) M * 4 + 256;
        put(q, q_at); put(k, q_at);                                            // the same bytes
        put(r, off); off += (size_t) M * 4 + 256;
        put(out, off); off += (size_t) M * 4 + 256;
        b.manual_bytes = off + 4096;
        b.inputs.push_back({wq, quantized(GGML_TYPE_Q4_K, K, M, 6)});
        b.inputs.push_back({wk, quantized(GGML_TYPE_Q4_K, K, M, 7)});
        b.inputs.push_back({x, as_bytes(normal((size_t) K, 1.0f, 8))});
        b.outputs = {out};
        return b;
    });
}

// Attention without FLASH_ATTN_EXT, shaped like libllama's (src/llama.cpp:601-650): K and the transposed V are views of a
// larger cache, the mask is F32 and padded, Q is a permuted view.  `extra_user` adds a second reader of the probabilities
// (the chain must then not be replaced by one fused launch, and the result must still be right).
static void attn_chain_case(const std::string & name, int64_t D, int64_t n_head, int64_t n_head_kv, int64_t n_q, int64_t n_kv, int64_t n_ctx, bool extra_user) {
    run_case(name, [=](ggml_context * ctx) {
        Built b;
        ggml_tensor * kc = ggml_new_tensor_1d(ctx, GGML_TYPE_F16, D * n_head_kv * n_ctx);      // rows of D * n_head_kv per token
        ggml_tensor * vc = ggml_new_tensor_1d(ctx, GGML_TYPE_F16, D * n_head_kv * n_ctx);      // transposed: n_ctx values per (head, d) row
        ggml_tensor * qin = ggml_new_tensor_3d(ctx, GGML_TYPE_F32, D, n_head, n_q);
        const int64_t n_pad = (n_q + 31) / 32 * 32;
        ggml_tensor * mask = ggml_new_tensor_2d(ctx, GGML_TYPE_F32, n_kv, n_pad);
        ggml_tensor * q = ggml_permute(ctx, qin, 0, 2, 1, 3);                                   // [D, n_q, n_head]
        ggml_tensor * k = ggml_view_3d(ctx, kc, D, n_kv, n_head_kv, (size_t) D * n_head_kv * 2, (size_t) D * 2, 0);
        ggml_tensor * kq = ggml_mul_mat(ctx, k, q);                                             // [n_kv, n_q, n_head]
        ggml_tensor * p = ggml_soft_max_ext(ctx, kq, mask, 1.0f / sqrtf((float) D), 0.0f);
        ggml_tensor * v = ggml_view_3d(ctx, vc, n_kv, D, n_head_kv, (size_t) n_ctx * 2, (size_t) n_ctx * D * 2, 0);
        ggml_tensor * kqv = ggml_mul_mat(ctx, v, p);                                            // [D, n_q, n_head]
        ggml_tensor * merged = ggml_permute(ctx, kqv, 0, 2, 1, 3);
        ggml_tensor * out = ggml_cont_2d(ctx, merged, D * n_head, n_q);
        b.graph = ggml_new_graph(ctx);
        ggml_build_forward_expand(b.graph, out);
        b.outputs = {out};
        if (extra_user) {
            ggml_tensor * s2 = ggml_scale(ctx, p, 2.0f);
            ggml_build_forward_expand(b.graph, s2);
            b.outputs.push_back(s2);
        }
        std::vector<float> kf = normal((size_t) D * n_head_kv * n_ctx, 1.0f, 3), vf = normal((size_t) D * n_head_kv * n_ctx, 1.0f, 4);
        std::vector<uint8_t> kb(kf.size() * 2), vb(vf.size() * 2);
        ggml_fp32_to_fp16_row(kf.data(), (ggml_fp16_t *) kb.data(), (int64_t) kf.size());
        ggml_fp32_to_fp16_row(vf.data(), (ggml_fp16_t *) vb.data(), (int64_t) vf.size());
        std::vector<float> mf((size_t) n_kv * n_pad, -INFINITY);
        for (int64_t iq = 0; iq < n_q; ++iq) for (int64_t ik = 0; ik <= n_kv - n_q + iq && ik < n_kv; ++ik) mf[(size_t) iq * n_kv + ik] = 0.0f;
        b.inputs.push_back({kc, kb});
        b.inputs.push_back({vc, vb});
        b.inputs.push_back({qin, as_bytes(normal((size_t) D * n_head * n_q, 1.0f, 5))});
        b.inputs.push_back({mask, as_bytes(mf)});
        return b;
    });
}
static void suite_attn_chain() {
    attn_chain_case("attn_chain.d128.q1.kv512", 128, 32, 8, 1, 512, 1024, false);
    attn_chain_case("attn_chain.d128.q4.kv320", 128, 32, 8, 4, 320, 512, false);
    attn_chain_case("attn_chain.d64.q1.kv256", 64, 8, 2, 1, 256, 256, false);
    attn_chain_case("attn_chain.d128.q37.kv64", 128, 16, 4, 37, 64, 256, false);
    attn_chain_case("attn_chain.d128.q200.kv1024", 128, 8, 2, 200, 1024, 2048, false);
    attn_chain_case("attn_chain.d128.q512.kv512", 128, 32, 8, 512, 512, 512, false);
    attn_chain_case("attn_chain.d128.q512.kv4096", 128, 32, 8, 512, 4096, 4096, false);
    attn_chain_case("attn_chain.d128.q64.kv128.second_reader", 128, 8, 2, 64, 128, 256, true);
}

// MUL_MAT with the weights in the row-split buffer type.  Row counts that are not multiples of the 128-row rounding, an
// uneven split, batch sizes of both the mat-vec and the tensor-core path.
static void suite_split(ggml_backend_dev_t dev) {
    typedef ggml_backend_buffer_type_t (*split_fn_t)(int, const float *);
    ggml_backend_reg_t reg = ggml_backend_dev_backend_reg(dev);
    split_fn_t fn = (split_fn_t) ggml_backend_reg_get_proc_address(reg, "ggml_backend_split_buffer_type");
    if (!fn) { printf("SPLIT unavailable: the registry has no ggml_backend_split_buffer_type\n"); g_fail = 1; return; }
    int main_index = -1;
    const int n_dev = (int) ggml_backend_reg_dev_count(reg);
    for (int i = 0; i < n_dev; ++i) if (ggml_backend_reg_dev_get(reg, (size_t) i) == dev) main_index = i;
    printf("SPLIT devices=%d main=%d\n", n_dev, main_index);
    float uneven[16] = {0};
    for (int i = 0; i < n_dev && i < 16; ++i) uneven[i] = i == 0 ? 3.0f : 1.0f;
    const float * splits[2] = {nullptr, uneven};
    const ggml_type types[] = {GGML_TYPE_Q4_K, GGML_TYPE_Q6_K, GGML_TYPE_Q8_0, GGML_TYPE_F16};
    for (int si = 0; si < 2; ++si) {
        g_split_buft = fn(main_index, splits[si]);
        if (!g_split_buft) { printf("SPLIT unavailable: the entry point returned NULL\n"); g_fail = 1; return; }
        printf("SPLIT buffer type %s\n", ggml_backend_buft_name(g_split_buft));
        for (ggml_type type : types) for (int64_t N : {1, 8, 64, 512}) {
            const int64_t K = 4096, M = si == 0 ? 4096 : 4096 + 200;
            run_case(std::string("split.") + (si ? "uneven." : "equal.") + ggml_type_name(type) + ".m" + std::to_string(M) + ".n" + std::to_string(N), [=](ggml_context * ctx) {
                Built b;
                ggml_tensor * w = ggml_new_tensor_2d(ctx, type, K, M), * x = ggml_new_tensor_2d(ctx, GGML_TYPE_F32, K, N);
                ggml_set_name(w, "w");
                ggml_tensor * y = ggml_mul_mat(ctx, w, x);
                b.graph = ggml_new_graph(ctx);
                ggml_build_forward_expand(b.graph, y);
                if (type == GGML_TYPE_F16) {
                    std::vector<float> wf = normal((size_t) K * M, 0.02f, 5);
                    std::vector<uint8_t> wb((size_t) K * M * 2);
                    ggml_fp32_to_fp16_row(wf.data(), (ggml_fp16_t *) wb.data(), K * M);
                    b.inputs.push_back({w, wb});
                } else {
                    b.inputs.push_back({w, quantized(type, K, M, 7)});
                }
                b.inputs.push_back({x, as_bytes(normal((size_t) K * N, 1.0f, 11 + (unsigned) N))});
                b.outputs = {y};
                b.split = {w};
                return b;
            });
        }
    }
    g_split_buft = nullptr;
}

int main(int argc, char ** argv) {
    ggml_time_init();
    if (argc < 3) { fprintf(stderr, "usage: %s DEVICE SUITE [N_THREADS]\n", argv[0]); return 2; }
    ggml_backend_load_all();
    ggml_backend_dev_t cpu_dev = ggml_backend_dev_by_type(GGML_BACKEND_DEVICE_TYPE_CPU), dev = ggml_backend_dev_by_name(argv[1]);
    if (!cpu_dev || !dev) { fprintf(stderr, "device %s (or the CPU device) not found\n", argv[1]); return 3; }
    g_cpu = ggml_backend_dev_init(cpu_dev, nullptr); g_dev = ggml_backend_dev_init(dev, nullptr);
    if (!g_cpu || !g_dev) { fprintf(stderr, "backend init failed\n"); return 3; }
    if (argc > 3) {
        auto set_threads = (ggml_backend_set_n_threads_t) ggml_backend_reg_get_proc_address(ggml_backend_dev_backend_reg(cpu_dev), "ggml_backend_set_n_threads");
        if (set_threads) set_threads(g_cpu, atoi(argv[3]));
    }
    const std::string suite = argv[2];
    if (suite == "mul_mat") suite_mul_mat();
    else if (suite == "flash_attn") suite_flash_attn();
    else if (suite == "alias") suite_alias();
    else if (suite == "split") suite_split(dev);
    else if (suite == "attn_chain") suite_attn_chain();
    else if (suite == "mul_mat_f16") suite_mul_mat_f16();
    else if (suite == "mul_mat_id") suite_mul_mat_id();
    else { fprintf(stderr, "unknown suite %s\n", argv[2]); return 2; }
    ggml_backend_free(g_dev); ggml_backend_free(g_cpu);
    return g_fail;
}
