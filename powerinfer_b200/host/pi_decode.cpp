// pi_decode: greedy decoding of token ids from a PowerInfer model file through the C ABI alone (no Python, no ggml).
//
//   pi_decode MODEL.powerinfer.gguf N_PREDICT TOKEN_ID [TOKEN_ID ...]
//
// The host-side sequence a C or C++ program follows, and what the reference's examples/main does around llama_decode
// for a fully offloaded sparse model (llama.cpp:3159-3390 tensor loading, 6764-7006 decode, 8617 greedy sampling):
// open the file (pi_model_file_*), upload every tensor the decode path needs (2-D weights as stored for F16, through
// pi_q4_0_repack for Q4_0; q / k / v rows concatenated per layer), create the engine on caller-owned memory, feed the
// prompt one position per step, then feed back the device-side argmax.  Prints the generated ids on one line.
// Build: nvcc -std=c++17 -I include pi_decode.cpp -L powerinfer_b200 -lpowerinfer_b200 -o pi_decode
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "powerinfer_b200.h"

namespace {

[[noreturn]] void die(const char * what, const char * detail) {
    fprintf(stderr, "pi_decode: %s: %s\n", what, detail);
    exit(1);
}
void pi_ok(int rc, const char * what) { if (rc != PI_OK) die(what, pi_last_error()); }
void cu_ok(cudaError_t e, const char * what) { if (e != cudaSuccess) die(what, cudaGetErrorString(e)); }

struct Loader {
    pi_model_file * f;
    cudaStream_t st;
    int wtype;
    std::vector<void *> owned;

    void * dev_alloc(size_t bytes) {
        void * p = nullptr;
        cu_ok(cudaMalloc(&p, bytes ? bytes : 16), "cudaMalloc");
        owned.push_back(p);
        return p;
    }
    bool has(const std::string & name) const { int t; int64_t ne[4]; return pi_model_file_tensor(f, name.c_str(), &t, ne, nullptr, nullptr) == PI_OK; }

    // a tensor copied as stored (norm vectors F32, predictor and embeddings F16); nullptr when absent and optional
    void * plain(const std::string & name, int want_type, bool required) {
        int type; int64_t ne[4]; const void * data; size_t n;
        if (pi_model_file_tensor(f, name.c_str(), &type, ne, &data, &n) != PI_OK) {
            if (required) die("missing tensor", name.c_str());
            return nullptr;
        }
        if (type != want_type || !data) die("tensor has a type the decode path does not take", name.c_str());
        void * d = dev_alloc(n);
        cu_ok(cudaMemcpyAsync(d, data, n, cudaMemcpyHostToDevice, st), "cudaMemcpyAsync");
        return d;
    }

    // 2-D weights of the model's weight type, several tensors stacked row-wise into one device matrix
    void * weights(const std::vector<std::string> & names, bool required) {
        struct Part { const void * data; size_t bytes; int64_t rows, cols; };
        std::vector<Part> parts;
        size_t total = 0;
        for (const std::string & name : names) {
            int type; int64_t ne[4]; const void * data; size_t n;
            if (pi_model_file_tensor(f, name.c_str(), &type, ne, &data, &n) != PI_OK) {
                if (required) die("missing tensor", name.c_str());
                return nullptr;
            }
            if (type != (wtype == PI_TYPE_Q4_0 ? 2 : 1) || !data) die("weight matrix is not in the model's weight type", name.c_str());
            parts.push_back({data, n, ne[1], ne[0]});
            total += n;
        }
        char * dst = (char *)dev_alloc(total);
        size_t off = 0;
        for (const Part & p : parts) {
            if (wtype == PI_TYPE_Q4_0) {                              // ggml blocks -> planar rows, through a staging copy
                void * staging = nullptr;
                cu_ok(cudaMalloc(&staging, p.bytes), "cudaMalloc");
                cu_ok(cudaMemcpyAsync(staging, p.data, p.bytes, cudaMemcpyHostToDevice, st), "cudaMemcpyAsync");
                pi_ok(pi_q4_0_repack(staging, dst + off, p.rows, p.cols, st), "pi_q4_0_repack");
                cu_ok(cudaStreamSynchronize(st), "cudaStreamSynchronize");
                cu_ok(cudaFree(staging), "cudaFree");
            } else {
                cu_ok(cudaMemcpyAsync(dst + off, p.data, p.bytes, cudaMemcpyHostToDevice, st), "cudaMemcpyAsync");
            }
            off += p.bytes;
        }
        return dst;
    }

    // bias vectors of q / k / v stacked like their matrices (opt)
    float * stacked_f32(const std::vector<std::string> & names) {
        size_t total = 0;
        for (const std::string & n : names) { int t; int64_t ne[4]; const void * d; size_t b; if (pi_model_file_tensor(f, n.c_str(), &t, ne, &d, &b) != PI_OK) return nullptr; if (t != 0) die("bias is not F32", n.c_str()); total += b; }
        char * dst = (char *)dev_alloc(total);
        size_t off = 0;
        for (const std::string & n : names) { int t; int64_t ne[4]; const void * d; size_t b; pi_model_file_tensor(f, n.c_str(), &t, ne, &d, &b); cu_ok(cudaMemcpyAsync(dst + off, d, b, cudaMemcpyHostToDevice, st), "cudaMemcpyAsync"); off += b; }
        return (float *)dst;
    }
};

}  // namespace

int main(int argc, char ** argv) {
    if (argc < 4) { fprintf(stderr, "usage: %s MODEL.powerinfer.gguf N_PREDICT TOKEN_ID [TOKEN_ID ...]\n", argv[0]); return 2; }
    const int n_predict = atoi(argv[2]);
    std::vector<int32_t> prompt;
    for (int i = 3; i < argc; i++) prompt.push_back((int32_t)atoi(argv[i]));

    pi_model_file * f = nullptr;
    pi_ok(pi_model_file_open(argv[1], &f), "open");
    pi_engine_config cfg;
    pi_ok(pi_model_file_engine_config(f, &cfg), "config");
    const char * arch; size_t arch_len;
    pi_ok(pi_model_file_get_str(f, "general.architecture", &arch, &arch_len), "architecture");
    printf("model: arch=%.*s weights=%s layers=%d d=%d ff=%d heads=%d/%d rank=%d vocab=%d ctx=%d threshold=%g\n", (int)arch_len, arch,
           cfg.wtype == PI_TYPE_Q4_0 ? "q4_0" : "f16", cfg.n_layer, cfg.d, cfg.n_ff, cfg.n_head, cfg.n_head_kv, cfg.rank, cfg.n_vocab, cfg.n_ctx,
           (double)cfg.threshold);
    fflush(stdout);
    if ((int)prompt.size() + n_predict > cfg.n_ctx) die("arguments", "prompt + N_PREDICT exceeds the model's context length");
    for (int32_t t : prompt) if (t < 0 || t >= cfg.n_vocab) die("arguments", "token id outside the vocabulary");
    const size_t ws_bytes = pi_engine_workspace_bytes(&cfg), kv_bytes = pi_engine_kv_bytes(&cfg);
    if (!ws_bytes) die("config", pi_last_error());

    Loader L{f, nullptr, cfg.wtype, {}};
    cu_ok(cudaStreamCreate(&L.st), "cudaStreamCreate");
    const bool falcon = cfg.arch == PI_ARCH_FALCON;
    std::vector<pi_layer_weights> layers((size_t)cfg.n_layer);
    for (int il = 0; il < cfg.n_layer; il++) {
        const std::string p = "blk." + std::to_string(il) + ".";
        pi_layer_weights & w = layers[(size_t)il];
        memset(&w, 0, sizeof w);
        w.attn_norm_w  = (const float *)L.plain(p + "attn_norm.weight", 0, true);
        w.attn_norm_b  = (const float *)L.plain(p + "attn_norm.bias", 0, false);
        w.attn_norm2_w = (const float *)L.plain(p + "attn_norm_2.weight", 0, false);
        w.attn_norm2_b = (const float *)L.plain(p + "attn_norm_2.bias", 0, false);
        w.ffn_norm_w   = (const float *)L.plain(p + "ffn_norm.weight", 0, false);
        w.ffn_norm_b   = (const float *)L.plain(p + "ffn_norm.bias", 0, false);
        if (falcon) w.wqkv = L.weights({p + "attn_qkv.weight"}, true);                     // stored fused: q rows, k rows, v rows
        else        w.wqkv = L.weights({p + "attn_q.weight", p + "attn_k.weight", p + "attn_v.weight"}, true);
        w.bqkv = L.stacked_f32({p + "attn_q.bias", p + "attn_k.bias", p + "attn_v.bias"});
        w.wo   = L.weights({p + "attn_output.weight"}, true);
        w.bo   = (const float *)L.plain(p + "attn_output.bias", 0, false);
        w.fc1  = L.plain(p + "fc1.weight", 1, true);
        w.fc2  = L.plain(p + "fc2.weight", 1, true);
        w.gate = L.weights({p + "ffn_gate.weight"}, false);
        w.up   = L.weights({p + "ffn_up.weight"}, true);
        w.down_t = L.weights({p + "ffn_down_t.weight"}, true);
        w.up_b   = (const float *)L.plain(p + "ffn_up.bias", 0, false);
        w.down_b = (const float *)L.plain(p + "ffn_down_t.bias", 0, false);
    }
    pi_model_weights g;
    memset(&g, 0, sizeof g);
    g.tok_embd   = L.plain("token_embd.weight", 1, true);
    g.pos_embd   = L.plain("position_embd.weight", 1, false);
    g.out_norm_w = (const float *)L.plain("output_norm.weight", 0, true);
    g.out_norm_b = (const float *)L.plain("output_norm.bias", 0, false);
    g.output     = L.weights({"output.weight"}, false);                                    // absent: tied to the embeddings (opt)

    void * ws = L.dev_alloc(ws_bytes), * kc = L.dev_alloc(kv_bytes), * vc = L.dev_alloc(kv_bytes);
    cu_ok(cudaMemsetAsync(kc, 0, kv_bytes, L.st), "cudaMemsetAsync");
    cu_ok(cudaMemsetAsync(vc, 0, kv_bytes, L.st), "cudaMemsetAsync");
    cu_ok(cudaStreamSynchronize(L.st), "upload");
    pi_engine * e = nullptr;
    pi_ok(pi_engine_create(&cfg, &g, layers.data(), ws, ws_bytes, kc, vc, L.st, &e), "engine_create");

    int32_t pos = 0, next = 0;
    for (int32_t t : prompt) { pi_ok(pi_engine_decode_host(e, &t, &pos, 1, nullptr, &next, L.st), "decode (prompt)"); pos++; }
    printf("ids:");
    for (int i = 0; i < n_predict; i++) {
        printf(" %d", (int)next);
        if (i + 1 == n_predict) break;
        const int32_t t = next;
        pi_ok(pi_engine_decode_host(e, &t, &pos, 1, nullptr, &next, L.st), "decode");
        pos++;
    }
    printf("\n");
    pi_ok(pi_engine_status(e, L.st), "engine status");
    pi_engine_destroy(e);
    for (void * p : L.owned) cudaFree(p);
    cudaStreamDestroy(L.st);
    pi_model_file_close(f);
    return 0;
}
