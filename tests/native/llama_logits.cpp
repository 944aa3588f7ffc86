// Test tool: evaluates a fixed token sequence with the reference's libllama (public API, include/llama.h) on
// whatever backends the reference's registry loads, and writes the logits of the last prompt token and of each
// generated position to a binary file (float32, n_vocab per row).  Run once with -ngl 0 (reference CPU backend)
// and once with GGML_BACKEND_PATH pointing at libggml-b200.so and -ngl 99: same loader, same graph builder, same
// scheduler; only the device differs.  Built by oracle/ref.mk against the reference headers; test infrastructure.
//   llama_logits MODEL.gguf OUT.bin N_GPU_LAYERS N_PROMPT N_GEN SEED [FLASH_ATTN=1] [SPLIT_MODE=layer|row|none]
#include "llama.h"
#include "ggml-backend.h"

#include <cstdio>
#include <cstdlib>
#include <random>
#include <string>
#include <vector>

int main(int argc, char ** argv) {
    if (argc < 7) { fprintf(stderr, "usage: %s model out ngl n_prompt n_gen seed\n", argv[0]); return 2; }
    const int ngl = atoi(argv[3]), n_prompt = atoi(argv[4]), n_gen = atoi(argv[5]), seed = atoi(argv[6]);
    const bool fa = argc > 7 ? atoi(argv[7]) != 0 : true;
    ggml_backend_load_all();
    llama_backend_init();
    llama_model_params mp = llama_model_default_params();
    mp.n_gpu_layers = ngl;
    if (argc > 8) {
        const std::string sm = argv[8];
        mp.split_mode = sm == "row" ? LLAMA_SPLIT_MODE_ROW : (sm == "none" ? LLAMA_SPLIT_MODE_NONE : LLAMA_SPLIT_MODE_LAYER);
    }
    llama_model * model = llama_model_load_from_file(argv[1], mp);
    if (!model) { fprintf(stderr, "load failed\n"); return 1; }
    llama_context_params cp = llama_context_default_params();
    cp.n_ctx = 1024; cp.n_batch = 512; cp.n_ubatch = 512; cp.flash_attn = fa; cp.n_threads = 8; cp.n_threads_batch = 8;
    llama_context * ctx = llama_init_from_model(model, cp);
    if (!ctx) { fprintf(stderr, "context failed\n"); return 1; }
    const int n_vocab = llama_vocab_n_tokens(llama_model_get_vocab(model));
    std::mt19937 rng((unsigned) seed);
    std::vector<llama_token> toks((size_t) (n_prompt + n_gen));
    for (auto & t : toks) t = (llama_token) (rng() % (unsigned) n_vocab);
    FILE * f = fopen(argv[2], "wb");
    if (!f) return 1;
    if (llama_decode(ctx, llama_batch_get_one(toks.data(), n_prompt)) != 0) { fprintf(stderr, "decode failed\n"); return 1; }
    fwrite(llama_get_logits_ith(ctx, -1), sizeof(float), (size_t) n_vocab, f);
    for (int i = 0; i < n_gen; ++i) {
        if (llama_decode(ctx, llama_batch_get_one(&toks[(size_t) (n_prompt + i)], 1)) != 0) { fprintf(stderr, "decode failed\n"); return 1; }
        fwrite(llama_get_logits_ith(ctx, -1), sizeof(float), (size_t) n_vocab, f);
    }
    fclose(f);
    llama_free(ctx);
    llama_model_free(model);
    return 0;
}
