// ref_decode.cpp -- drives the REFERENCE's own llama.cpp through llama.h (TEST INFRASTRUCTURE ONLY).
//
// Compiled by oracle/Makefile against the reference's unmodified llama.cpp + ggml twice:
//   oracle/_ref/ref_decode       CPU-only build, which is the --vram-budget 0 path (nothing offloaded, every layer's
//                                gpu_idx all zero): the parity oracle;
//   oracle/_ref/ref_decode_b200  the same sources with -DGGML_USE_CUBLAS, linked against libggml_cuda_b200.so instead
//                                of the reference's ggml-cuda.cu: the reference's own llama_decode -> llm_build_ffn_sparse
//                                -> ggml_graph_compute running over this repository's back end.  REF_VRAM_GB sets
//                                llama_model_params::vram_budget_gb (default 0 = nothing offloaded); at exit it prints,
//                                per ggml op, how many nodes the back end served and how many it handed back to the CPU.  It loads a PowerInfer ("PWRI") GGUF, feeds explicit token ids, and dumps
// the raw logits of every step plus the greedy (argmax of raw logits) continuation, which is what
// llama_sample_token_greedy does; examples/main is not used because its sampler applies a repeat
// penalty even at temperature 0.
//
//   ref_decode MODEL TOKENS.i32 N_PROMPT N_STEPS N_THREADS OUT.f32 [batch|single] [forced]
//
// TOKENS.i32 : int32 ids; the first N_PROMPT are the prompt.  With `forced`, ids N_PROMPT.. are fed as
//              the continuation (teacher forcing) instead of the greedy choice.
// OUT.f32    : N_STEPS records of n_vocab floats: the logits after the last prompt token, then after
//              each fed continuation token.  The chosen greedy ids go to stdout, one per line.
// batch      : prompt in one llama_decode call (default); single: one token per call.
#include "llama.h"

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#ifdef GGML_USE_CUBLAS
#include "ggml.h"
extern "C" void ggml_cuda_b200_counts(int op, long long * served, long long * declined);
extern "C" int  ggml_cuda_b200_op_count(void);
static void print_backend_counts() {
    for (int op = 0; op < ggml_cuda_b200_op_count(); op++) {
        long long s = 0, d = 0;
        ggml_cuda_b200_counts(op, &s, &d);
        if (s || d) fprintf(stderr, "b200_nodes op=%s served=%lld declined=%lld\n", ggml_op_name((enum ggml_op)op), s, d);
    }
}
#endif

static int argmax(const float * x, int n) {
    int b = 0;
    for (int i = 1; i < n; i++) if (x[i] > x[b]) b = i;
    return b;
}

int main(int argc, char ** argv) {
    if (argc < 7) {
        fprintf(stderr, "usage: %s MODEL TOKENS.i32 N_PROMPT N_STEPS N_THREADS OUT.f32 [batch|single] [forced]\n", argv[0]);
        return 2;
    }
    const char * model_path = argv[1];
    const int n_prompt = atoi(argv[3]), n_steps = atoi(argv[4]), n_threads = atoi(argv[5]);
    const bool single = argc > 7 && strcmp(argv[7], "single") == 0;
    const bool forced = argc > 8 && strcmp(argv[8], "forced") == 0;

    std::vector<int32_t> toks;
    {
        FILE * f = fopen(argv[2], "rb");
        if (!f) { perror(argv[2]); return 1; }
        int32_t t;
        while (fread(&t, sizeof t, 1, f) == 1) toks.push_back(t);
        fclose(f);
    }
    if ((int)toks.size() < n_prompt || (forced && (int)toks.size() < n_prompt + n_steps - 1)) {
        fprintf(stderr, "token file too short\n");
        return 1;
    }

    llama_backend_init(false);
    llama_model_params mp = llama_model_default_params();
    mp.n_gpu_layers = 0;
    mp.vram_budget_gb = getenv("REF_VRAM_GB") ? (float)atof(getenv("REF_VRAM_GB")) : 0.0f;
    mp.use_mmap = true;
    llama_context_params cp = llama_context_default_params();
    cp.seed = 0;
    cp.n_ctx = n_prompt + n_steps + 8;
    cp.n_batch = 512;
    cp.n_threads = n_threads;
    cp.n_threads_batch = n_threads;
    // the loader is told the context it will serve, as the reference's own programs do (common/common.cpp:966): with a VRAM
    // budget it then reserves room for the KV cache and offloads the attention nodes as well (llama.cpp:3392-3421)
    llama_model * model = llama_load_model_from_file_with_context(model_path, mp, &cp);
    if (!model) { fprintf(stderr, "load failed\n"); return 1; }

    llama_context * ctx = llama_new_context_with_model(model, cp);
    if (!ctx) { fprintf(stderr, "context failed\n"); return 1; }
    const int n_vocab = llama_n_vocab(model);

    FILE * out = fopen(argv[6], "wb");
    if (!out) { perror(argv[6]); return 1; }

    int n_past = 0;
    if (single) {
        for (int i = 0; i < n_prompt; i++) {
            if (llama_decode(ctx, llama_batch_get_one(&toks[i], 1, n_past, 0))) { fprintf(stderr, "decode failed\n"); return 1; }
            n_past++;
        }
    } else {
        for (int i = 0; i < n_prompt; i += (int)cp.n_batch) {
            const int n = std::min((int)cp.n_batch, n_prompt - i);
            if (llama_decode(ctx, llama_batch_get_one(&toks[i], n, n_past, 0))) { fprintf(stderr, "decode failed\n"); return 1; }
            n_past += n;
        }
    }
    const int64_t t0 = llama_time_us();
    for (int s = 0; s < n_steps; s++) {
        const float * logits = llama_get_logits(ctx);
        fwrite(logits, sizeof(float), n_vocab, out);
        const int g = argmax(logits, n_vocab);
        printf("%d\n", g);
        if (s + 1 == n_steps) break;
        int32_t next = forced ? toks[n_prompt + s] : g;
        if (llama_decode(ctx, llama_batch_get_one(&next, 1, n_past, 0))) { fprintf(stderr, "decode failed\n"); return 1; }
        n_past++;
    }
    const int64_t t1 = llama_time_us();
    fprintf(stderr, "ref_decode: %d decode steps in %.3f ms (%d threads)\n", n_steps - 1, (t1 - t0)/1000.0, n_threads);
    fclose(out);
#ifdef GGML_USE_CUBLAS
    print_backend_counts();
#endif
    llama_free(ctx);
    llama_free_model(model);
    llama_backend_free();
    return 0;
}
