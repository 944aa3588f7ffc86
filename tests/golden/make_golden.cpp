// Generates tests/golden/golden.bin by running the UNMODIFIED reference (the
// libraries that oracle/ref.mk builds into oracle/_ref) on small seeded inputs:
// reference quantizers / dequantizers and the reference ggml CPU backend for
// MUL_MAT, FLASH_ATTN_EXT and the glue ops.  The fixtures pin the C restatement
// in oracle/ and are what the CUDA path is compared with on a machine that has no
// reference tree.  Build and run:  make -C tests/golden   (needs oracle/_ref)
//
// Container format: "GOLD" u32 count, then per record: u32 name_len, name bytes,
// u32 dtype (0 f32, 1 u8, 2 i32, 3 f16 bits as u16), u32 ndim, u64 dims[ndim], raw data.
#include "ggml.h"
#include "ggml-alloc.h"
#include "ggml-backend.h"
#include "ggml-cpu.h"

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

struct Rec { std::string name; uint32_t dtype; std::vector<uint64_t> dims; std::vector<uint8_t> data; };
static std::vector<Rec> g_recs;

static void add(const std::string & name, uint32_t dtype, std::vector<uint64_t> dims, const void * p, size_t nbytes) {
    Rec r; r.name = name; r.dtype = dtype; r.dims = dims; r.data.assign((const uint8_t *) p, (const uint8_t *) p + nbytes);
    g_recs.push_back(r);
}
static void add_f32(const std::string & n, const std::vector<float> & v, std::vector<uint64_t> dims) { add(n, 0, dims, v.data(), v.size() * 4); }

// small deterministic generator (splitmix64 + Box-Muller); inputs are stored in the file anyway
struct Rng {
    uint64_t s;
    explicit Rng(uint64_t seed) : s(seed) {}
    uint64_t next() { uint64_t z = (s += 0x9e3779b97f4a7c15ull); z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull; z = (z ^ (z >> 27)) * 0x94d049bb133111ebull; return z ^ (z >> 31); }
    double uni() { return ((next() >> 11) + 0.5) / 9007199254740992.0; }
    float normal(float sigma) { const double u1 = uni(), u2 = uni(); return (float) (sigma * std::sqrt(-2.0 * std::log(u1)) * std::cos(6.283185307179586 * u2)); }
};

static const ggml_type k_types[] = {GGML_TYPE_Q4_0, GGML_TYPE_Q4_1, GGML_TYPE_Q5_0, GGML_TYPE_Q5_1, GGML_TYPE_Q8_0,
                                    GGML_TYPE_Q4_K, GGML_TYPE_Q5_K, GGML_TYPE_Q6_K,
                                    GGML_TYPE_Q2_K, GGML_TYPE_Q3_K, GGML_TYPE_IQ4_NL, GGML_TYPE_IQ4_XS};

static ggml_backend_t g_cpu;

// runs a one-node graph on the reference CPU backend; inputs are set by `fill`
template <typename Build, typename Fill>
static std::vector<float> run_cpu(Build build, Fill fill) {
    ggml_init_params ip = {ggml_tensor_overhead() * 64 + ggml_graph_overhead(), nullptr, true};
    ggml_context * ctx = ggml_init(ip);
    ggml_tensor * out = build(ctx);
    ggml_cgraph * gf = ggml_new_graph(ctx);
    ggml_build_forward_expand(gf, out);
    ggml_backend_buffer_t buf = ggml_backend_alloc_ctx_tensors(ctx, g_cpu);
    fill(ctx);
    ggml_backend_graph_compute(g_cpu, gf);
    std::vector<float> res(ggml_nelements(out));
    ggml_backend_tensor_get(out, res.data(), 0, ggml_nbytes(out));
    ggml_backend_buffer_free(buf);
    ggml_free(ctx);
    return res;
}

int main(int argc, char ** argv) {
    const char * out_path = argc > 1 ? argv[1] : "golden.bin";
    ggml_backend_load_all();
    g_cpu = ggml_backend_init_by_type(GGML_BACKEND_DEVICE_TYPE_CPU, nullptr);
    if (!g_cpu) { fprintf(stderr, "no CPU backend\n"); return 1; }
    auto set_threads = (ggml_backend_set_n_threads_t) ggml_backend_reg_get_proc_address(
        ggml_backend_dev_backend_reg(ggml_backend_get_device(g_cpu)), "ggml_backend_set_n_threads");
    if (set_threads) set_threads(g_cpu, 1);

    // ---- 1. quantize / dequantize on the reference's own synthetic vector (tests/test-quantize-fns.cpp:28-35)
    const int NQ = 1024;
    std::vector<float> cosv(NQ);
    for (int i = 0; i < NQ; ++i) cosv[i] = 0.1f + 2.0f * std::cos((float) i + 0.0f);
    add_f32("quant.input", cosv, {(uint64_t) NQ});
    for (ggml_type t : k_types) {
        std::vector<uint8_t> q(ggml_row_size(t, NQ));
        ggml_quantize_chunk(t, cosv.data(), q.data(), 0, 1, NQ, nullptr);
        std::vector<float> dq(NQ);
        ggml_get_type_traits(t)->to_float(q.data(), dq.data(), NQ);
        add(std::string("quant.q.") + ggml_type_name(t), 1, {q.size()}, q.data(), q.size());
        add_f32(std::string("quant.dq.") + ggml_type_name(t), dq, {(uint64_t) NQ});
    }
    {   // F32 -> F16 (KV-cache store)
        std::vector<float> x(512); Rng r(7);
        for (auto & v : x) v = r.normal(1.0f);
        x[0] = 65504.0f; x[1] = 1e-8f; x[2] = -0.0f; x[3] = 1.00048828125f;   // edge roundings
        std::vector<ggml_fp16_t> h(x.size());
        ggml_fp32_to_fp16_row(x.data(), h.data(), (int64_t) x.size());
        add_f32("f16.input", x, {x.size()});
        add("f16.output", 3, {h.size()}, h.data(), h.size() * 2);
    }

    // ---- 2. MUL_MAT on the reference CPU backend, per weight type
    const int K = 512, M = 32, N = 5;
    {
        Rng r(0);
        std::vector<float> w((size_t) K * M), x((size_t) K * N);
        for (auto & v : w) v = r.normal(0.02f);
        for (auto & v : x) v = r.normal(1.0f);
        add_f32("mul_mat.w_f32", w, {(uint64_t) M, (uint64_t) K});
        add_f32("mul_mat.x", x, {(uint64_t) N, (uint64_t) K});
        for (ggml_type t : k_types) {
            std::vector<uint8_t> q(ggml_row_size(t, K) * M);
            ggml_quantize_chunk(t, w.data(), q.data(), 0, M, K, nullptr);
            ggml_tensor *tw = nullptr, *tx = nullptr;
            std::vector<float> y = run_cpu(
                [&](ggml_context * c) { tw = ggml_new_tensor_2d(c, t, K, M); tx = ggml_new_tensor_2d(c, GGML_TYPE_F32, K, N); return ggml_mul_mat(c, tw, tx); },
                [&](ggml_context *) { ggml_backend_tensor_set(tw, q.data(), 0, q.size()); ggml_backend_tensor_set(tx, x.data(), 0, x.size() * 4); });
            add(std::string("mul_mat.w.") + ggml_type_name(t), 1, {(uint64_t) M, q.size() / M}, q.data(), q.size());
            add_f32(std::string("mul_mat.y.") + ggml_type_name(t), y, {(uint64_t) N, (uint64_t) M});
        }
    }

    // ---- 3. FLASH_ATTN_EXT: GQA 8/2 heads, D=128, causal -inf mask, F16 K/V
    {
        const int D = 128, NH = 8, NHKV = 2, NQ_ = 5, NKV = 128, NQP = 64;   // mask rows padded to GGML_KQ_MASK_PAD
        Rng r(3);
        std::vector<float> q((size_t) D * NQ_ * NH), kf((size_t) D * NKV * NHKV), vf(kf.size());
        for (auto & v : q) v = r.normal(1.0f);
        for (auto & v : kf) v = r.normal(1.0f);
        for (auto & v : vf) v = r.normal(1.0f);
        std::vector<ggml_fp16_t> k(kf.size()), v(vf.size()), mask((size_t) NKV * NQP);
        ggml_fp32_to_fp16_row(kf.data(), k.data(), (int64_t) kf.size());
        ggml_fp32_to_fp16_row(vf.data(), v.data(), (int64_t) vf.size());
        std::vector<float> mf(mask.size());
        for (int iq = 0; iq < NQP; ++iq) for (int ik = 0; ik < NKV; ++ik)
            mf[(size_t) iq * NKV + ik] = (iq < NQ_ && ik <= NKV - NQ_ + iq) ? 0.0f : -INFINITY;
        ggml_fp32_to_fp16_row(mf.data(), mask.data(), (int64_t) mf.size());
        ggml_tensor *tq, *tk, *tv, *tm;
        std::vector<float> y = run_cpu(
            [&](ggml_context * c) {
                tq = ggml_new_tensor_3d(c, GGML_TYPE_F32, D, NQ_, NH);
                tk = ggml_new_tensor_3d(c, GGML_TYPE_F16, D, NKV, NHKV);
                tv = ggml_new_tensor_3d(c, GGML_TYPE_F16, D, NKV, NHKV);
                tm = ggml_new_tensor_2d(c, GGML_TYPE_F16, NKV, NQP);
                ggml_tensor * o = ggml_flash_attn_ext(c, tq, tk, tv, tm, 1.0f / std::sqrt((float) D), 0.0f, 0.0f);
                ggml_flash_attn_ext_set_prec(o, GGML_PREC_F32);
                return o;
            },
            [&](ggml_context *) {
                ggml_backend_tensor_set(tq, q.data(), 0, q.size() * 4);
                ggml_backend_tensor_set(tk, k.data(), 0, k.size() * 2);
                ggml_backend_tensor_set(tv, v.data(), 0, v.size() * 2);
                ggml_backend_tensor_set(tm, mask.data(), 0, mask.size() * 2);
            });
        add_f32("fattn.q", q, {(uint64_t) NH, (uint64_t) NQ_, (uint64_t) D});
        add("fattn.k", 3, {(uint64_t) NHKV, (uint64_t) NKV, (uint64_t) D}, k.data(), k.size() * 2);
        add("fattn.v", 3, {(uint64_t) NHKV, (uint64_t) NKV, (uint64_t) D}, v.data(), v.size() * 2);
        add("fattn.mask", 3, {(uint64_t) NQP, (uint64_t) NKV}, mask.data(), mask.size() * 2);
        add_f32("fattn.y", y, {(uint64_t) NQ_, (uint64_t) NH, (uint64_t) D});
    }

    // ---- 4. glue ops
    {
        const int D = 256, R = 6;
        Rng r(11);
        std::vector<float> x((size_t) D * R), w(D), g((size_t) D * R);
        for (auto & v : x) v = r.normal(3.0f);
        for (auto & v : w) v = 1.0f + r.normal(0.1f);
        for (auto & v : g) v = r.normal(2.0f);
        ggml_tensor *tx, *tw, *tg;
        auto fill_x = [&](ggml_context *) { ggml_backend_tensor_set(tx, x.data(), 0, x.size() * 4); };
        std::vector<float> y = run_cpu([&](ggml_context * c) { tx = ggml_new_tensor_2d(c, GGML_TYPE_F32, D, R); return ggml_rms_norm(c, tx, 1e-5f); }, fill_x);
        add_f32("glue.x", x, {(uint64_t) R, (uint64_t) D});
        add_f32("glue.w", w, {(uint64_t) D});
        add_f32("glue.g", g, {(uint64_t) R, (uint64_t) D});
        add_f32("glue.rms_norm", y, {(uint64_t) R, (uint64_t) D});
        y = run_cpu([&](ggml_context * c) { tx = ggml_new_tensor_2d(c, GGML_TYPE_F32, D, R); tw = ggml_new_tensor_1d(c, GGML_TYPE_F32, D);
                                             return ggml_mul(c, ggml_rms_norm(c, tx, 1e-5f), tw); },
                    [&](ggml_context * c) { fill_x(c); ggml_backend_tensor_set(tw, w.data(), 0, w.size() * 4); });
        add_f32("glue.rms_norm_mul", y, {(uint64_t) R, (uint64_t) D});
        y = run_cpu([&](ggml_context * c) { tx = ggml_new_tensor_2d(c, GGML_TYPE_F32, D, R); tg = ggml_new_tensor_2d(c, GGML_TYPE_F32, D, R);
                                             return ggml_mul(c, ggml_silu(c, tg), tx); },
                    [&](ggml_context * c) { fill_x(c); ggml_backend_tensor_set(tg, g.data(), 0, g.size() * 4); });
        add_f32("glue.silu_mul", y, {(uint64_t) R, (uint64_t) D});
        y = run_cpu([&](ggml_context * c) { tx = ggml_new_tensor_2d(c, GGML_TYPE_F32, D, R); return ggml_soft_max_ext(c, tx, nullptr, 0.125f, 0.0f); }, fill_x);
        add_f32("glue.soft_max", y, {(uint64_t) R, (uint64_t) D});

        // ROPE as Llama-3 uses it: mode 0, theta 5e5, frequency factors, 4 heads x 3 tokens of 128
        const int HD = 128, NHD = 4, NT = 3;
        std::vector<float> rx((size_t) HD * NHD * NT), ff(HD / 2);
        for (auto & v : rx) v = r.normal(1.0f);
        for (int i = 0; i < HD / 2; ++i) ff[i] = i < 40 ? 1.0f : (i < 52 ? 1.0f + (i - 40) * 0.5f : 8.0f);
        std::vector<int32_t> pos = {0, 17, 4099};
        ggml_tensor *tp, *tf;
        for (int mode : {0, 2}) {
            y = run_cpu([&](ggml_context * c) { tx = ggml_new_tensor_3d(c, GGML_TYPE_F32, HD, NHD, NT); tp = ggml_new_tensor_1d(c, GGML_TYPE_I32, NT);
                                                 tf = ggml_new_tensor_1d(c, GGML_TYPE_F32, HD / 2);
                                                 return ggml_rope_ext(c, tx, tp, tf, HD, mode, 8192, 500000.0f, 1.0f, 0.0f, 1.0f, 32.0f, 1.0f); },
                        [&](ggml_context *) { ggml_backend_tensor_set(tx, rx.data(), 0, rx.size() * 4); ggml_backend_tensor_set(tp, pos.data(), 0, pos.size() * 4);
                                              ggml_backend_tensor_set(tf, ff.data(), 0, ff.size() * 4); });
            add_f32(std::string("rope.y.mode") + std::to_string(mode), y, {(uint64_t) NT, (uint64_t) NHD, (uint64_t) HD});
        }
        add_f32("rope.x", rx, {(uint64_t) NT, (uint64_t) NHD, (uint64_t) HD});
        add_f32("rope.ff", ff, {(uint64_t) HD / 2});
        add("rope.pos", 2, {(uint64_t) NT}, pos.data(), pos.size() * 4);
    }

    FILE * f = fopen(out_path, "wb");
    if (!f) { perror(out_path); return 1; }
    const uint32_t n = (uint32_t) g_recs.size();
    fwrite("GOLD", 1, 4, f); fwrite(&n, 4, 1, f);
    for (const Rec & r : g_recs) {
        const uint32_t nl = (uint32_t) r.name.size(), nd = (uint32_t) r.dims.size();
        fwrite(&nl, 4, 1, f); fwrite(r.name.data(), 1, nl, f); fwrite(&r.dtype, 4, 1, f); fwrite(&nd, 4, 1, f);
        fwrite(r.dims.data(), 8, nd, f); fwrite(r.data.data(), 1, r.data.size(), f);
    }
    fclose(f);
    printf("wrote %s: %u records\n", out_path, n);
    ggml_backend_free(g_cpu);
    return 0;
}
