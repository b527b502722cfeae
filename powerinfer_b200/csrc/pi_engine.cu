// The decode token loop: what llama_decode -> llm_build_{llama,falcon,opt} -> ggml_graph_compute does for one step
// of n_tokens sequences (llama.cpp:6764-7006, 4949-5468), as one fixed launch sequence over device-resident
// weights, replayed as a CUDA graph.  The residual stream never leaves the device; every mat-vec gets its input
// already in the FP16 / Q8_0 form the reference's CPU path would convert it to.
//
// Sharding (n_ranks > 1): each rank holds a contiguous slice of the FFN neurons (rows of fc2 / up / gate / down_t)
// and of the attention heads (rows of wq/wk/wv, columns of wo, its heads' KV cache).  fc1, norms and embeddings are
// replicated.  The two partial d_model vectors per layer (attention out-projection, FFN down-projection) are
// exchanged by pi_exchange.cu; a rank never reads another rank's memory.
#include "pi_common.cuh"

#include <cmath>
#include <cstdlib>
#include <cstring>
#include <new>
#include <vector>

namespace pi {

// ------------------------------------------------------------------------------------------------ small kernels

// ggml_get_rows on the F16 embedding (+ OPT's learned positions at pos + 2: llama.cpp:5105-5108, 6486-6488)
__global__ void k_embed(const __half * __restrict__ tok_embd, const __half * __restrict__ pos_embd,
                        const int32_t * __restrict__ tokens, const int32_t * __restrict__ pos, int n_vocab, int n_pos,
                        int64_t d, float * __restrict__ x, unsigned int * __restrict__ step_no) {
    const int t = blockIdx.y;
    if (step_no && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) *step_no += 1u;   // numbers the exchanges of this step
    int tok = tokens[t];
    tok = tok < 0 ? 0 : (tok >= n_vocab ? n_vocab - 1 : tok);
    for (int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; c < d; c += (int64_t)gridDim.x * blockDim.x) {
        float v = __half2float(tok_embd[(size_t)tok * d + c]);
        if (pos_embd) {
            int p = pos[t] + 2;
            p = p < 0 ? 0 : (p >= n_pos ? n_pos - 1 : p);
            v = v + __half2float(pos_embd[(size_t)p * d + c]);
        }
        x[(size_t)t * d + c] = v;
    }
}

// llama_sample_token_greedy (llama.cpp:8617): first index of the maximum of the raw logits
__global__ void __launch_bounds__(1024) k_argmax(const float * __restrict__ logits, int n, int32_t * __restrict__ out) {
    __shared__ float s_v[32];
    __shared__ int s_i[32];
    const float * row = logits + (size_t)blockIdx.x * n;
    float bv = -INFINITY; int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = row[i];
        if (v > bv) { bv = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int   oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { s_v[threadIdx.x >> 5] = bv; s_i[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); w++)
            if (s_v[w] > bv || (s_v[w] == bv && s_i[w] < bi)) { bv = s_v[w]; bi = s_i[w]; }
        out[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
    }
}

// Keeps the stream busy for a fixed time (profiling only): while it sleeps the host queues the whole step behind it, so
// the kernels then run back to back and the events around them measure kernels, not the host's launch rate.
__global__ void k_hold(unsigned long long ns) {
    unsigned long long t0, t1;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
    do {
        __nanosleep(2000);
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t1));
    } while (t1 - t0 < ns);
}

// free-running greedy decode without a host round trip: the chosen ids become the next step's input tokens
__global__ void k_advance(int32_t * __restrict__ tokens, int32_t * __restrict__ pos, const int32_t * __restrict__ argmax,
                          int T, int n_ctx) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t < T) { tokens[t] = argmax[t]; pos[t] = min(pos[t] + 1, n_ctx - 1); }
}

}  // namespace pi

using namespace pi;

#ifdef PI_TIMELINE
__device__ unsigned long long pi::g_tl[65536 * 16];
__device__ unsigned int pi::g_tl_n;
extern "C" __attribute__((visibility("default"))) int pi_timeline_read(unsigned long long * host, unsigned int * n, int reset) {
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(n, pi::g_tl_n, 4);
    cudaMemcpyFromSymbol(host, pi::g_tl, sizeof(unsigned long long) * 65536 * 16);
    if (reset) { unsigned int z = 0; cudaMemcpyToSymbol(pi::g_tl_n, &z, 4); }
    return 0;
}
#endif

// ------------------------------------------------------------------------------------------------ engine state

struct pi_engine {
    pi_engine_config c;
    std::vector<pi_layer_weights> layers;
    pi_model_weights g;
    int hd, dq, dkv, F, T_max;
    int G;                                   // axpy row groups
    // device buffers carved from the caller's workspace
    int32_t * tokens, * pos, * seq_ids, * seq_pf, * argmax;   // seq_pf: the sequence of every token of a prompt chunk
    float * x, * x2, * attn_out, * ffn_vec, * qkv, * pred, * h, * partial, * logits, * cs;
    int32_t * list, * count; unsigned int * ticket; uint32_t * masks;
    int8_t * cq; float * cd;
    __half * hidden16;
    ActBuf act_a, act_q, act_p, act_o;       // FFN input, QKV input, predictor input (FP16), out-proj input
    __half * k_cache, * v_cache;             // [n_layer, max_batch, n_ctx, dkv]
    unsigned int * status;                   // device word: bit 0 = an exchange wait ran out
    unsigned long long * active_total;       // device counter: sum of active-list lengths over layers and steps
    pi_exchange xch;
    cudaGraphExec_t graphs[3][PI_MAX_BATCH + 1];   // [0] decode, [1] prompt chunk, [2] prompt chunk without the lm head
    bool warmed[3][PI_MAX_BATCH + 1];
    int graph_nodes[3][PI_MAX_BATCH + 1];          // kernel nodes of each captured graph
    int launches;                            // kernels enqueued by the last enqueue_step
    float * pred_trace;                      // optional [n_layer, max_batch, F]: keeps every layer's predictor logits
    bool pdl;                                // programmatic dependent launch between the kernels of a step
    bool gate_sym;                           // bamboo: relu on the gated product as well
    int qkv_pre;                             // ring stages the QKV mat-vec requests before its dependency wait after a norm that collects vectors (-1: all)
    bool fc2_masks;                          // ... with the activity masks written by the predictor's second mat-vec itself (no mask kernel)
    bool rows1;                              // one token: masks-only compaction + register-streaming sparse kernels (shape eligible)
    long long wait_cycles;                   // bound of the exchange waits (0: about a second)
    unsigned skip_mask;                      // set only inside pi_engine_time_stage: the stages left out of the captured sequence
};

static constexpr int NORM_MAX_GROUPS = 48;      // partial vectors the norm adds itself; more go through k_reduce_partials first

static size_t up256(size_t v) { return (v + 255) & ~size_t(255); }

struct Carver {
    char * p; char * end; bool ok = true;
    template <typename T> T * take(size_t count) {
        const size_t bytes = up256(count * sizeof(T));
        if (p + bytes > end) { ok = false; return nullptr; }
        T * r = (T *)p; p += bytes; return r;
    }
    ActBuf act(int wtype, int64_t n, int T) {
        const size_t bytes = act_bytes(wtype, n, T);
        if (p + bytes > end) { ok = false; return ActBuf(); }
        char * q = p;
        ActBuf a = act_carve(wtype, n, T, &q);
        p += bytes;
        return a;
    }
};

static void carve(pi_engine * e, void * ws, size_t ws_bytes, bool dry, size_t * need) {
    const pi_engine_config & c = e->c;
    Carver cv{(char *)ws, dry ? (char *)ws + (size_t(1) << 60) : (char *)ws + ws_bytes};
    const int T = e->T_max;
    const size_t d = c.d, F = e->F;
    e->tokens = cv.take<int32_t>(T); e->pos = cv.take<int32_t>(T); e->seq_ids = cv.take<int32_t>(T); e->seq_pf = cv.take<int32_t>(T); e->argmax = cv.take<int32_t>(T);
    e->status = cv.take<unsigned int>(1); e->active_total = cv.take<unsigned long long>(1);
    e->x = cv.take<float>(T * d); e->x2 = cv.take<float>(T * d); e->attn_out = cv.take<float>(T * d); e->ffn_vec = cv.take<float>(T * d);
    e->qkv = cv.take<float>((size_t)T * (e->dq + 2 * e->dkv));
    e->pred = cv.take<float>(T * F); e->h = cv.take<float>(T * F);
    e->partial = cv.take<float>((size_t)e->G * T * d);
    e->logits = cv.take<float>((size_t)T * c.n_vocab);
    e->cs = cv.take<float>((size_t)c.n_ctx * e->hd);
    e->list = cv.take<int32_t>(F); e->count = cv.take<int32_t>(1); e->ticket = cv.take<unsigned int>(1);
    e->masks = cv.take<uint32_t>((F + 63) / 64 * 2);
    e->cq = cv.take<int8_t>(T * F); e->cd = cv.take<float>(T * (F / 32 + 1));
    e->hidden16 = cv.take<__half>((size_t)T * c.rank);
    e->act_a = cv.act(c.wtype, c.d, T);
    e->act_q = cv.act(c.wtype, c.d, T);
    e->act_p = cv.act(PI_TYPE_F16, c.d, T);
    e->act_o = cv.act(c.wtype, e->dq, T);
    *need = (size_t)(cv.p - (char *)ws);
    if (!cv.ok && !dry) *need = (size_t)-1;
}

static int validate(const pi_engine_config & c) {
    PI_REQUIRE(c.arch >= 0 && c.arch <= PI_ARCH_BAMBOO, "engine: unknown arch %d", c.arch);
    PI_REQUIRE(c.wtype == PI_TYPE_F16 || c.wtype == PI_TYPE_Q4_0, "engine: unknown weight type %d", c.wtype);
    PI_REQUIRE(c.n_layer > 0 && c.d > 0 && c.n_ff > 0 && c.n_head > 0 && c.n_head_kv > 0 && c.rank > 0 && c.n_vocab > 0 && c.n_ctx > 0,
               "engine: non-positive dimension");
    PI_REQUIRE(c.d % c.n_head == 0 && c.n_head % c.n_head_kv == 0, "engine: d %% n_head or n_head %% n_head_kv != 0");
    PI_REQUIRE(c.max_batch >= 1 && c.max_batch <= PI_MAX_BATCH, "engine: max_batch must be 1..%d", PI_MAX_BATCH);
    PI_REQUIRE(c.n_ranks >= 1 && c.n_ranks <= PI_MAX_RANKS && c.rank_id >= 0 && c.rank_id < c.n_ranks, "engine: bad rank %d of %d", c.rank_id, c.n_ranks);
    PI_REQUIRE(c.n_ff % (32 * c.n_ranks) == 0, "engine: n_ff must be a multiple of 32 x n_ranks (whole 32-neuron blocks per rank)");
    PI_REQUIRE(c.n_head_kv % c.n_ranks == 0, "engine: n_head_kv must be a multiple of n_ranks");
    const int hd = c.d / c.n_head;
    PI_REQUIRE(hd % 32 == 0 && hd <= 256, "engine: head_dim must be a multiple of 32 and <= 256");
    const int align = c.wtype == PI_TYPE_Q4_0 ? 256 : 8;
    PI_REQUIRE(c.d % align == 0 && (c.d / c.n_ranks) % align == 0, "engine: d and d / n_ranks must be multiples of %d for this weight type", align);
    PI_REQUIRE(c.rank % 8 == 0, "engine: predictor rank must be a multiple of 8");
    return PI_OK;
}

extern "C" {
#pragma GCC visibility push(default)

size_t pi_engine_workspace_bytes(const pi_engine_config * cfg) {
    if (!cfg || validate(*cfg) != PI_OK) return 0;
    pi_engine e{};
    e.c = *cfg;
    e.hd = cfg->d / cfg->n_head; e.dq = cfg->d / cfg->n_ranks; e.dkv = e.hd * cfg->n_head_kv / cfg->n_ranks;
    e.F = cfg->n_ff / cfg->n_ranks; e.T_max = cfg->max_batch;
    e.G = axpy_groups(cfg->wtype, cfg->d, cfg->max_batch);
    size_t need = 0;
    carve(&e, nullptr, 0, true, &need);
    return need + 256;
}

size_t pi_engine_kv_bytes(const pi_engine_config * cfg) {
    if (!cfg || validate(*cfg) != PI_OK) return 0;
    const size_t dkv = (size_t)(cfg->d / cfg->n_head) * cfg->n_head_kv / cfg->n_ranks;
    return (size_t)cfg->n_layer * cfg->max_batch * cfg->n_ctx * dkv * sizeof(__half);
}

int pi_engine_create(const pi_engine_config * cfg, const pi_model_weights * gw, const pi_layer_weights * lw,
                     void * workspace, size_t workspace_bytes, void * k_cache, void * v_cache, void * stream,
                     pi_engine ** out) {
    PI_REQUIRE(cfg && gw && lw && workspace && k_cache && v_cache && out, "engine_create: null argument");
    int rc = validate(*cfg);
    if (rc) return rc;
    PI_REQUIRE(((uintptr_t)workspace & 255) == 0, "engine_create: workspace must be 256-byte aligned");
    pi_engine * e = new (std::nothrow) pi_engine();
    PI_REQUIRE(e, "engine_create: out of host memory");
    e->c = *cfg; e->g = *gw;
    // bamboo is the llama graph; relu(gate) * relu(up) == relu(relu(gate) * up) exactly (the first factor is >= 0), so the
    // gated mat-vec's own relu-on-output switch gives the symmetric gate
    e->gate_sym = cfg->arch == PI_ARCH_BAMBOO;
    if (e->gate_sym) e->c.arch = PI_ARCH_LLAMA;
    e->layers.assign(lw, lw + cfg->n_layer);
    e->hd = cfg->d / cfg->n_head; e->dq = cfg->d / cfg->n_ranks; e->dkv = e->hd * cfg->n_head_kv / cfg->n_ranks;
    e->F = cfg->n_ff / cfg->n_ranks; e->T_max = cfg->max_batch;
    e->G = axpy_groups(cfg->wtype, cfg->d, cfg->max_batch);
    size_t need = 0;
    carve(e, workspace, workspace_bytes, false, &need);
    if (need == (size_t)-1) { delete e; set_error("engine_create: workspace of %zu bytes is too small", workspace_bytes); return PI_ERR_WORKSPACE; }
    e->k_cache = (__half *)k_cache; e->v_cache = (__half *)v_cache;
    memset(e->graphs, 0, sizeof e->graphs);
    memset(e->warmed, 0, sizeof e->warmed);
    memset(e->graph_nodes, 0, sizeof e->graph_nodes);
    memset(&e->xch, 0, sizeof e->xch);
    e->pred_trace = nullptr; e->launches = 0;
    { const char * v = getenv("PI_PDL"); e->pdl = !(v && v[0] == '0'); }
    e->skip_mask = 0u; e->wait_cycles = 0;
    e->rows1 = rows_eligible(cfg->wtype, e->F, cfg->d) && axpy_rows_groups(e->F, cfg->d) <= e->G;
    { const char * v = getenv("PI_QKV_PRE"); e->qkv_pre = v ? atoi(v) : 0; }
    { const char * v = getenv("PI_FC2_MASKS"); e->fc2_masks = !(v && v[0] == '0'); }     // 0: the separate mask kernel (diagnostic)
    cudaStream_t st = (cudaStream_t)stream;
    // one-time device state: sequence ids 0..T-1, zeroed ticket / status, RoPE angle table
    std::vector<int32_t> ids(e->T_max);
    for (int i = 0; i < e->T_max; i++) ids[i] = i;
    std::vector<float> cs((size_t)cfg->n_ctx * e->hd);
    pi_rope_table_host(cs.data(), cfg->n_ctx, e->hd, cfg->rope_base);
    cudaError_t ce = cudaMemcpyAsync(e->seq_ids, ids.data(), ids.size() * 4, cudaMemcpyHostToDevice, st);
    if (ce == cudaSuccess) ce = cudaMemcpyAsync(e->cs, cs.data(), cs.size() * 4, cudaMemcpyHostToDevice, st);
    if (ce == cudaSuccess) ce = cudaMemsetAsync(e->ticket, 0, 4, st);
    if (ce == cudaSuccess) ce = cudaMemsetAsync(e->count, 0, 4, st);
    if (ce == cudaSuccess) ce = cudaMemsetAsync(e->status, 0, 4, st);
    if (ce == cudaSuccess) ce = cudaMemsetAsync(e->active_total, 0, 8, st);
    if (ce == cudaSuccess) ce = cudaStreamSynchronize(st);            // the host vectors above die at return
    if (ce != cudaSuccess) { delete e; return cuda_fail(ce, "engine_create"); }
    *out = e;
    return PI_OK;
}

void pi_engine_destroy(pi_engine * e) {
    if (!e) return;
    for (auto & gm : e->graphs) for (auto & g : gm) if (g) cudaGraphExecDestroy(g);
    delete e;
}

int pi_engine_io(pi_engine * e, int32_t ** tokens, int32_t ** pos, float ** logits, int32_t ** argmax) {
    PI_REQUIRE(e, "engine_io: null engine");
    if (tokens) *tokens = e->tokens;
    if (pos) *pos = e->pos;
    if (logits) *logits = e->logits;
    if (argmax) *argmax = e->argmax;
    return PI_OK;
}

int pi_engine_set_exchange(pi_engine * e, const pi_exchange * x) {
    PI_REQUIRE(e && x, "engine_set_exchange: null argument");
    PI_REQUIRE(x->n_ranks == e->c.n_ranks && x->rank_id == e->c.rank_id, "engine_set_exchange: rank layout differs from the engine's");
    PI_REQUIRE(x->slot_floats >= (int64_t)e->T_max * e->c.d && x->mailbox_local && x->epoch,
               "engine_set_exchange: need a mailbox, a step counter and slot_floats >= %lld", (long long)e->T_max * e->c.d);
    e->xch = *x;
    for (auto & gm : e->graphs) for (auto & g : gm) if (g) { cudaGraphExecDestroy(g); g = nullptr; }
    return PI_OK;
}

#pragma GCC visibility pop
}  // extern "C"

// ------------------------------------------------------------------------------------------------ the step

namespace {

// Optional per-stage CUDA-event timing (profile mode only).  Events are queued around every stage and read after the
// whole step has drained, so the GPU never idles between a start event and its kernel.
struct StageTimer {
    bool on = false; cudaStream_t st = nullptr;
    std::vector<cudaEvent_t> pool; std::vector<int> stage_of; size_t used = 0;
    cudaEvent_t next() {
        if (used == pool.size()) { cudaEvent_t ev = nullptr; if (cudaEventCreate(&ev) != cudaSuccess) return nullptr; pool.push_back(ev); }
        return pool[used++];
    }
    int begin() {
        if (!on) return PI_OK;
        cudaEvent_t a = next();
        if (!a) return PI_ERR_CUDA;
        PI_CUDA(cudaEventRecord(a, st));
        return PI_OK;
    }
    int end(int stage) {
        if (!on) return PI_OK;
        cudaEvent_t b = next();
        if (!b) return PI_ERR_CUDA;
        PI_CUDA(cudaEventRecord(b, st));
        stage_of.push_back(stage);
        return PI_OK;
    }
    int collect(float * acc) {
        PI_CUDA(cudaStreamSynchronize(st));
        for (size_t i = 0; i < stage_of.size(); i++) {
            float ms = 0.f;
            PI_CUDA(cudaEventElapsedTime(&ms, pool[2 * i], pool[2 * i + 1]));
            acc[stage_of[i]] += ms;
        }
        return PI_OK;
    }
    ~StageTimer() { for (auto ev : pool) cudaEventDestroy(ev); }
};

#define STAGE(stage, n_kernels, call)                    \
    do {                                                 \
        int rc_;                                         \
        if (e->skip_mask & (1u << (stage))) break;       \
        if ((rc_ = tm.begin())) return rc_;              \
        if ((rc_ = (call))) return rc_;                  \
        if ((rc_ = tm.end(stage))) return rc_;           \
        e->launches += (n_kernels);                      \
    } while (0)

// what the previous layer left to be folded into the next norm: a vector (or mailbox slots) + bias + extra residual
struct Pending {
    const float * vec = nullptr;          // single vector [T, d]
    const float * partial = nullptr; int n_groups = 0;   // or: partial vectors [n_groups, T, d] to be added in group order
    bool exchange = false;                // sharded run: the above is this rank's share, to be exchanged by the norm
    const float * bias = nullptr;
    const float * res = nullptr;          // added before the residual stream (falcon's attention branch)
    bool any() const { return vec || partial; }
};

// what the norm reads: its own share (a vector or partial vectors), exchanged first when the run is sharded
void norm_inputs(pi_engine * e, const Pending & pd, NormArgs & n, int * xch_index, int xch_per_step) {
    if (pd.partial) { n.partial = pd.partial; n.n_groups = pd.n_groups; }
    else            { n.x = pd.vec; }
    n.in_bias = pd.bias;
    if (pd.exchange) {
        n.xch = &e->xch; n.xch_index = (*xch_index)++; n.xch_per_step = xch_per_step; n.xch_extra = pd.res;
        n.wait_cycles = e->wait_cycles; n.status = e->status;
        n.residual = e->x;
    } else if (pd.res) { n.residual = pd.res; n.residual2 = e->x; }
    else               { n.residual = e->x; }
    n.x_out = e->x;
}

// mode 0: T sequences, one new token each; 1: T consecutive tokens of one sequence (a prompt chunk); 2: the same without
// the final norm / lm head (chunks whose logits nobody reads)
int enqueue_step(pi_engine * e, int T, cudaStream_t st, StageTimer & tm, int mode = 0) {
    const pi_engine_config & c = e->c;
    const int64_t d = c.d, F = e->F;
    const int wt = c.wtype;
    const bool multi = c.n_ranks > 1;
    const bool rms = c.arch == PI_ARCH_LLAMA;
    const bool falcon = c.arch == PI_ARCH_FALCON;
    const int qkv_rows = e->dq + 2 * e->dkv;
    const bool pdl = e->pdl && !tm.on;       // profiling wants each kernel alone between its events
    e->launches = 0;
    const int xch_per_step = falcon ? c.n_layer : 2 * c.n_layer;      // exchanges of one step (falcon sums its branches locally first)
    int xch_index = 0;

    if (!(e->skip_mask & (1u << PI_STAGE_OTHER))) {
        const dim3 grid((unsigned)((d + 255) / 256), T);
        if (tm.begin()) return PI_ERR_CUDA;
        k_embed<<<grid, 256, 0, st>>>((const __half *)e->g.tok_embd, (const __half *)e->g.pos_embd, e->tokens, e->pos,
                                      c.n_vocab, c.n_pos, d, e->x, multi ? e->xch.epoch : nullptr);
        PI_LAUNCH_CHECK("k_embed");
        if (tm.end(PI_STAGE_OTHER)) return PI_ERR_CUDA;
        e->launches++;
    }

    Pending pend;
    for (int il = 0; il <= c.n_layer; il++) {
        const bool last = il == c.n_layer;
        const pi_layer_weights * L = last ? nullptr : &e->layers[il];

        // ---- the norm that opens the layer (or the output norm) folds in the previous layer's FFN result
        NormArgs n1;
        n1.pdl = pdl;
        n1.T = T; n1.n = d; n1.rms = rms; n1.eps = c.norm_eps;
        n1.w = last ? e->g.out_norm_w : L->attn_norm_w;
        n1.b = last ? e->g.out_norm_b : L->attn_norm_b;
        const bool n1_collects = pend.partial != nullptr || pend.exchange;     // partial vectors (or the ranks' shares) to read first
        if (pend.any()) norm_inputs(e, pend, n1, &xch_index, xch_per_step); else n1.x = e->x;
        if (last && mode == 2) break;
        if (last) {
            const int out_t = e->g.output ? wt : PI_TYPE_F16;            // opt: tied F16 embedding
            n1.act_type = out_t; n1.act = out_t == wt ? e->act_a : e->act_p;
            STAGE(PI_STAGE_NORM, 1, launch_norm(n1, st));
            GemvArgs g;
            g.status = e->status; g.pdl = pdl;
            g.wtype = out_t; g.W = e->g.output ? e->g.output : e->g.tok_embd; g.nrows = c.n_vocab; g.ncols = d;
            g.x = n1.act.view(); g.T = T; g.dst = e->logits; g.dst_stride = c.n_vocab;
            STAGE(PI_STAGE_LM_HEAD, (T + 7) / 8, launch_gemv(g, st));
            if (!(e->skip_mask & (1u << PI_STAGE_OTHER))) {
                if (tm.begin()) return PI_ERR_CUDA;
                k_argmax<<<T, 1024, 0, st>>>(e->logits, c.n_vocab, e->argmax);
                PI_LAUNCH_CHECK("k_argmax");
                if (tm.end(PI_STAGE_OTHER)) return PI_ERR_CUDA;
                e->launches++;
            }
            break;
        }
        ActBuf qkv_in = e->act_q;
        if (falcon) {
            // attn_norm feeds the FFN; the predictor reads the layer input itself (llama.cpp:5422-5428)
            n1.act_type = wt; n1.act = e->act_a;
            n1.act2_type = PI_TYPE_F16; n1.act2 = e->act_p; n1.act2_src = 0;
            STAGE(PI_STAGE_NORM, 1, launch_norm(n1, st));
            if (L->attn_norm2_w) {
                NormArgs n2;
                n2.pdl = pdl;
                n2.x = e->x; n2.T = T; n2.n = d; n2.rms = 0; n2.eps = c.norm_eps; n2.w = L->attn_norm2_w; n2.b = L->attn_norm2_b;
                n2.act_type = wt; n2.act = e->act_q;
                STAGE(PI_STAGE_NORM, 1, launch_norm(n2, st));
            } else {
                qkv_in = e->act_a;
            }
        } else {
            n1.act_type = wt; n1.act = e->act_q;
            STAGE(PI_STAGE_NORM, 1, launch_norm(n1, st));
        }

        // ---- attention: QKV mat-vec (rows: this rank's Q heads, K heads, V heads), RoPE + KV store + KQV, out-proj
        {
            GemvArgs g;
            g.status = e->status; g.pdl = pdl;
            g.wtype = wt; g.W = L->wqkv; g.nrows = qkv_rows; g.ncols = d; g.x = qkv_in.view(); g.T = T;
            g.bias = L->bqkv; g.dst = e->qkv; g.dst_stride = qkv_rows;
            // A ring kernel requests its first stages of weights (tens of MB over all SMs) the moment it becomes resident, i.e.
            // while the norm before it is still reading the partial vectors; those reads then queue behind the burst
            // (measured: 5 us for 0.5 MB).  After such a norm the QKV mat-vec starts its ring only when its wait is over.
            g.pre_stages = n1_collects ? e->qkv_pre : -1;
            STAGE(PI_STAGE_QKV, (T + 7) / 8, launch_gemv(g, st));
        }
        {
            AttnArgs a;
            a.pdl = pdl;
            a.q = e->qkv; a.k = e->qkv + e->dq; a.v = e->qkv + e->dq + e->dkv;
            a.q_stride = qkv_rows; a.kv_stride = qkv_rows;
            const size_t layer_off = (size_t)il * c.max_batch * c.n_ctx * e->dkv;
            a.k_cache = e->k_cache + layer_off; a.v_cache = e->v_cache + layer_off;
            a.seq = mode ? e->seq_pf : e->seq_ids; a.pos = e->pos; a.T = T;
            a.n_head = c.n_head / c.n_ranks; a.n_head_kv = c.n_head_kv / c.n_ranks; a.head_dim = e->hd; a.n_ctx = c.n_ctx;
            if (c.arch != PI_ARCH_OPT) { a.cs = e->cs; a.neox = falcon; }
            a.out_act_type = wt; a.out_act = e->act_o;
            if (mode) {                                                   // prompt chunk: every token's K / V first, then attention
                a.store_mode = 1;
                STAGE(PI_STAGE_ATTN, 1, launch_attention(a, st));
                a.store_mode = 2;
            }
            STAGE(PI_STAGE_ATTN, 1, launch_attention(a, st));
        }
        {
            GemvArgs g;
            g.status = e->status; g.pdl = pdl;
            g.wtype = wt; g.W = L->wo; g.nrows = d; g.ncols = e->dq; g.x = e->act_o.view(); g.T = T;
            g.bias = c.rank_id == 0 ? L->bo : nullptr;                    // the bias enters the sum over ranks once
            g.dst = e->attn_out; g.dst_stride = d;
            STAGE(PI_STAGE_WO, (T + 7) / 8, launch_gemv(g, st));
        }

        // ---- FFN input.  llama / opt: ffn_inp = attn_out + x, then the FFN norm; the complete attention output is needed,
        //      so sharded runs exchange here.  falcon: n1 already produced both inputs.
        if (!falcon) {
            Pending pa;
            pa.vec = e->attn_out; pa.exchange = multi;
            NormArgs n2;
            n2.pdl = pdl;
            n2.T = T; n2.n = d; n2.rms = rms; n2.eps = c.norm_eps; n2.w = L->ffn_norm_w; n2.b = L->ffn_norm_b;
            norm_inputs(e, pa, n2, &xch_index, xch_per_step);
            n2.act_type = wt; n2.act = e->act_a;
            n2.act2_type = PI_TYPE_F16; n2.act2 = e->act_p; n2.act2_src = 0;      // the predictor reads ffn_inp itself
            STAGE(PI_STAGE_NORM, 1, launch_norm(n2, st));
        }

        // ---- predictor: idx = fc2 . relu(fc1 . p)   (llama.cpp:4688-4695)
        float * pred = e->pred_trace ? e->pred_trace + (size_t)il * c.max_batch * F : e->pred;
        // One token: the sparse kernels rank the active rows themselves from bit masks, which the predictor's second mat-vec
        // writes in its epilogue (then no mask kernel runs at all).  Q4_0 rows with an up bias keep the mask kernel: it also
        // writes relu(bias) into the hidden vector where a row is inactive, which the axpy's per-block quantisation must see.
        const bool rows1 = T == 1 && e->rows1;
        const bool masks1 = rows1 && e->fc2_masks && !(wt == PI_TYPE_Q4_0 && L->up_b);
        {
            GemvArgs g1;
            g1.status = e->status; g1.pdl = pdl;
            g1.W = L->fc1; g1.nrows = c.rank; g1.ncols = d; g1.x = e->act_p.view(); g1.T = T; g1.relu = 1;
            g1.dst16 = e->hidden16; g1.dst_stride = c.rank;
            STAGE(PI_STAGE_PRED, (T + 7) / 8, launch_gemv(g1, st));
            Act hx; hx.h16 = e->hidden16;
            GemvArgs g2;
            g2.status = e->status; g2.pdl = pdl;
            g2.W = L->fc2; g2.nrows = F; g2.ncols = c.rank; g2.x = hx; g2.T = T; g2.dst = pred; g2.dst_stride = F;
            if (masks1) { g2.masks_out = e->masks; g2.masks_threshold = c.threshold; }
            STAGE(PI_STAGE_PRED, (T + 7) / 8, launch_gemv(g2, st));
        }
        // ---- mask -> activity bit masks, and for batches the sorted list of rows active for at least one token.
        //      Where a row is inactive for a token the dense hidden vector holds 0 (or relu(bias)): the Q4_0 axpy quantises
        //      that vector per 32 neurons, and a union list leaves per-token holes.
        if (!masks1) {
            CompactArgs ca;
            ca.pdl = pdl;
            ca.idx = pred; ca.idx_stride = F; ca.T = T; ca.threshold = c.threshold; ca.n_local = F;
            if (!rows1) { ca.list = e->list; ca.count = e->count; }
            ca.masks = e->masks; ca.ticket = e->ticket; ca.total = e->active_total;
            if (wt == PI_TYPE_Q4_0) { ca.zero_dst = e->h; ca.zero_stride = F; ca.fill_bias = L->up_b; ca.fill_relu = 1; }
            STAGE(PI_STAGE_COMPACT, 1, launch_compact(ca, st));
        }
        int used = e->G;
        // ---- one token with masks from the predictor: the whole sparse FFN in one launch where the shape allows it
        FfnRowsArgs f;
        f.pdl = pdl;
        f.wtype = wt; f.up = L->up; f.gate = L->gate; f.down_t = L->down_t; f.nrows = F; f.ncols = d;
        f.x = e->act_a.view(); f.masks = e->masks; f.bias = L->up_b; f.relu = L->gate ? (e->gate_sym ? 1 : 0) : 1;
        f.h = e->h; f.partial = e->partial; f.n_groups = e->G < NORM_MAX_GROUPS ? e->G : NORM_MAX_GROUPS; f.rows_total = e->active_total;
        if (masks1 && ffn_rows_eligible(f)) {                          // (the plan is cached: a table look-up after the first call)
            STAGE(PI_STAGE_FFN, 1, launch_ffn_rows(f, st, &used));
        } else {
            // ---- up (and gate) over the active rows: h = relu(gate.x) * (up.x) | relu(up.x + b)
            {
                GemvArgs g;
                g.status = e->status; g.pdl = pdl;
                g.wtype = wt; g.W = L->up; g.W2 = L->gate; g.nrows = F; g.ncols = d; g.x = e->act_a.view(); g.T = T;
                if (rows1) { g.masks = e->masks; if (masks1) g.rows_total = e->active_total; } else { g.list = e->list; g.count = e->count; }
                g.idx = pred; g.idx_stride = F; g.threshold = c.threshold;
                g.bias = L->up_b; g.relu = L->gate ? (e->gate_sym ? 1 : 0) : 1;
                g.dst = e->h; g.dst_stride = F;
                STAGE(PI_STAGE_UPGATE, (T + 7) / 8, launch_gemv(g, st));
            }
            // ---- down: axpy over the same rows; the sum over row groups (and, sharded, over ranks) is left to the next norm
            if (wt == PI_TYPE_Q4_0 && T > 1) STAGE(PI_STAGE_DOWN, 1, launch_neuron_q8(e->h, F, F, T, e->cq, e->cd, st));
            {
                AxpyArgs a;
                a.pdl = pdl;
                a.wtype = wt; a.Wt = L->down_t; a.nrows = F; a.ncols = d; a.h = e->h; a.h_stride = F; a.T = T;
                if (rows1) { a.masks = e->masks; a.h_uncleared = masks1; } else { a.list = e->list; a.count = e->count; }
                a.idx = pred; a.idx_stride = F; a.threshold = c.threshold;
                a.cq = e->cq; a.cd = e->cd; a.c_stride = F; a.partial = e->partial; a.n_groups = e->G; a.status = e->status;
                STAGE(PI_STAGE_DOWN, T == 1 ? 1 : (wt == PI_TYPE_Q4_0 ? (T + 1) / 2 : (T + 3) / 4), launch_axpy(a, st, &used));
            }
        }
        pend = Pending();
        pend.bias = L->down_b;
        pend.exchange = multi;
        pend.res = falcon ? e->attn_out : nullptr;        // falcon sums its two branches locally first: one exchange per layer (llama.cpp:5443-5447)
        if (used <= NORM_MAX_GROUPS) {
            pend.partial = e->partial; pend.n_groups = used;
        } else {
            STAGE(PI_STAGE_DOWN, 1, launch_reduce_partials(e->partial, used, T, d, nullptr, nullptr, e->ffn_vec, st, pdl));
            pend.vec = e->ffn_vec;
        }
    }
    return PI_OK;
}

int check_T(pi_engine * e, int T) {
    PI_REQUIRE(e, "engine: null");
    PI_REQUIRE(T >= 1 && T <= e->T_max, "engine: T=%d outside 1..%d", T, e->T_max);
    PI_REQUIRE(e->c.n_ranks == 1 || e->xch.mailbox_local, "engine: sharded engine has no exchange configured");
    PI_REQUIRE(e->c.n_ranks == 1 || (e->c.d % 256 == 0), "engine: sharded runs need d_model to be a multiple of 256");
    return PI_OK;
}

// kernel nodes of a captured step: the exact number of kernel launches one replay makes (the per-call estimates added
// up in `launches` do not know which kernel a launcher picked for a batch)
int count_kernel_nodes(cudaGraph_t graph) {
    size_t n = 0;
    if (cudaGraphGetNodes(graph, nullptr, &n) != cudaSuccess || n == 0) return 0;
    std::vector<cudaGraphNode_t> nodes(n);
    if (cudaGraphGetNodes(graph, nodes.data(), &n) != cudaSuccess) return 0;
    int k = 0;
    for (size_t i = 0; i < n; i++) {
        cudaGraphNodeType ty;
        if (cudaGraphNodeGetType(nodes[i], &ty) == cudaSuccess && ty == cudaGraphNodeTypeKernel) k++;
    }
    return k;
}

// first call for a batch size: one plain run (fills every per-kernel attribute cache), then capture
int run_step(pi_engine * e, int T, cudaStream_t st, int mode = 0) {
    StageTimer tm;
    if (e->graphs[mode][T]) { PI_CUDA(cudaGraphLaunch(e->graphs[mode][T], st)); e->launches = e->graph_nodes[mode][T]; return PI_OK; }
    if (!e->warmed[mode][T]) {
        e->warmed[mode][T] = true;
        return enqueue_step(e, T, st, tm, mode);
    }
    cudaGraph_t graph = nullptr;
    PI_CUDA(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
    const int rc = enqueue_step(e, T, st, tm, mode);
    const cudaError_t ce = cudaStreamEndCapture(st, &graph);
    if (rc) { if (graph) cudaGraphDestroy(graph); return rc; }
    if (ce != cudaSuccess) return cuda_fail(ce, "cudaStreamEndCapture");
    { const int k = count_kernel_nodes(graph); if (k > 0) e->launches = k; }
    cudaGraphExec_t exec = nullptr;
    const cudaError_t ci = cudaGraphInstantiate(&exec, graph, 0);
    cudaGraphDestroy(graph);
    if (ci != cudaSuccess) return cuda_fail(ci, "cudaGraphInstantiate");
    e->graphs[mode][T] = exec; e->graph_nodes[mode][T] = e->launches;
    PI_CUDA(cudaGraphLaunch(exec, st));
    return PI_OK;
}

}  // namespace

extern "C" {
#pragma GCC visibility push(default)

int pi_engine_decode(pi_engine * e, int T, void * stream) {
    int rc = check_T(e, T);
    if (rc) return rc;
    return run_step(e, T, (cudaStream_t)stream);
}

int pi_engine_advance(pi_engine * e, int T, void * stream) {
    int rc = check_T(e, T);
    if (rc) return rc;
    k_advance<<<1, 32, 0, (cudaStream_t)stream>>>(e->tokens, e->pos, e->argmax, T, e->c.n_ctx);
    PI_LAUNCH_CHECK("k_advance");
    return PI_OK;
}

int pi_engine_decode_host(pi_engine * e, const int32_t * host_tokens, const int32_t * host_pos, int T,
                          float * host_logits, int32_t * host_argmax, void * stream) {
    int rc = check_T(e, T);
    if (rc) return rc;
    PI_REQUIRE(host_tokens && host_pos, "engine_decode_host: null input");
    cudaStream_t st = (cudaStream_t)stream;
    for (int t = 0; t < T; t++) PI_REQUIRE(host_pos[t] >= 0 && host_pos[t] < e->c.n_ctx, "engine_decode_host: position %d outside the context of %d", host_pos[t], e->c.n_ctx);
    PI_CUDA(cudaMemcpyAsync(e->tokens, host_tokens, (size_t)T * 4, cudaMemcpyHostToDevice, st));
    PI_CUDA(cudaMemcpyAsync(e->pos, host_pos, (size_t)T * 4, cudaMemcpyHostToDevice, st));
    if ((rc = run_step(e, T, st))) return rc;
    if (host_logits) PI_CUDA(cudaMemcpyAsync(host_logits, e->logits, (size_t)T * e->c.n_vocab * 4, cudaMemcpyDeviceToHost, st));
    if (host_argmax) PI_CUDA(cudaMemcpyAsync(host_argmax, e->argmax, (size_t)T * 4, cudaMemcpyDeviceToHost, st));
    PI_CUDA(cudaStreamSynchronize(st));
    return PI_OK;
}

int pi_engine_prefill_host(pi_engine * e, const int32_t * host_tokens, int n_tokens, int seq, int pos0,
                           float * host_logits_last, int32_t * host_argmax_last, void * stream) {
    PI_REQUIRE(e && host_tokens && n_tokens >= 1, "engine_prefill_host: bad arguments");
    PI_REQUIRE(seq >= 0 && seq < e->T_max, "engine_prefill_host: sequence %d outside 0..%d", seq, e->T_max - 1);
    PI_REQUIRE(pos0 >= 0 && (int64_t)pos0 + n_tokens <= e->c.n_ctx, "engine_prefill_host: positions %d..%d outside the context of %d", pos0, pos0 + n_tokens - 1, e->c.n_ctx);
    int rc = check_T(e, 1);
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    std::vector<int32_t> ids(e->T_max, seq), pos(e->T_max);
    PI_CUDA(cudaMemcpyAsync(e->seq_pf, ids.data(), (size_t)e->T_max * 4, cudaMemcpyHostToDevice, st));
    int last_T = 0;
    for (int t0 = 0; t0 < n_tokens; t0 += e->T_max) {
        const int T = n_tokens - t0 < e->T_max ? n_tokens - t0 : e->T_max;
        const bool final_chunk = t0 + T == n_tokens;
        for (int t = 0; t < T; t++) pos[t] = pos0 + t0 + t;
        PI_CUDA(cudaMemcpyAsync(e->tokens, host_tokens + t0, (size_t)T * 4, cudaMemcpyHostToDevice, st));
        PI_CUDA(cudaMemcpyAsync(e->pos, pos.data(), (size_t)T * 4, cudaMemcpyHostToDevice, st));
        PI_CUDA(cudaStreamSynchronize(st));                               // `pos` is rewritten for the next chunk
        const bool head = final_chunk && (host_logits_last || host_argmax_last);
        if ((rc = run_step(e, T, st, head ? 1 : 2))) return rc;
        last_T = T;
    }
    if (host_logits_last) PI_CUDA(cudaMemcpyAsync(host_logits_last, e->logits + (size_t)(last_T - 1) * e->c.n_vocab, (size_t)e->c.n_vocab * 4, cudaMemcpyDeviceToHost, st));
    if (host_argmax_last) PI_CUDA(cudaMemcpyAsync(host_argmax_last, e->argmax + (last_T - 1), 4, cudaMemcpyDeviceToHost, st));
    PI_CUDA(cudaStreamSynchronize(st));
    return PI_OK;
}

int pi_engine_profile_step(pi_engine * e, int T, float * host_ms, int * host_launches, void * stream) {
    int rc = check_T(e, T);
    if (rc) return rc;
    PI_REQUIRE(host_ms, "engine_profile_step: null output");
    cudaStream_t st = (cudaStream_t)stream;
    StageTimer tm;
    tm.on = true; tm.st = st;
    tm.pool.reserve(4096);
    for (int i = 0; i < 2 * (e->launches > 0 ? e->launches + 8 : 2048); i++) tm.next();   // create the events before the clock starts
    tm.used = 0;
    const unsigned long long hold_ns = (unsigned long long)(e->launches > 0 ? e->launches : 1000) * 12000ull;
    k_hold<<<1, 1, 0, st>>>(hold_ns < 30000000ull ? hold_ns : 30000000ull);
    PI_LAUNCH_CHECK("k_hold");
    rc = enqueue_step(e, T, st, tm);
    if (rc) { cudaStreamSynchronize(st); return rc; }
    if (host_launches) *host_launches = e->launches;
    return tm.collect(host_ms);
}

int pi_engine_time_stage(pi_engine * e, int T, int stage, int reps, float * host_ms_per_rep, int * host_launches, void * stream) {
    int rc = check_T(e, T);
    if (rc) return rc;
    PI_REQUIRE(host_ms_per_rep && stage >= 0 && stage < PI_N_STAGES && reps > 0, "engine_time_stage: bad arguments");
    cudaStream_t st = (cudaStream_t)stream;
    const unsigned saved = e->skip_mask;
    const int saved_launches = e->launches;                          // stays the count of the whole step
    e->skip_mask = ~(1u << stage) & ((1u << PI_N_STAGES) - 1u);
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    StageTimer tm;
    cudaError_t ce = cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal);
    if (ce == cudaSuccess) {
        rc = enqueue_step(e, T, st, tm);
        ce = cudaStreamEndCapture(st, &graph);
    }
    e->skip_mask = saved;
    if (host_launches) { const int k = graph ? count_kernel_nodes(graph) : 0; *host_launches = k > 0 ? k : e->launches; }
    e->launches = saved_launches;
    if (rc == PI_OK && ce == cudaSuccess) ce = cudaGraphInstantiate(&exec, graph, 0);
    if (rc == PI_OK && ce == cudaSuccess) ce = cudaEventCreate(&ev0);
    if (rc == PI_OK && ce == cudaSuccess) ce = cudaEventCreate(&ev1);
    if (rc == PI_OK && ce == cudaSuccess) ce = cudaGraphLaunch(exec, st);                    // warm
    if (rc == PI_OK && ce == cudaSuccess) ce = cudaEventRecord(ev0, st);
    for (int i = 0; i < reps && rc == PI_OK && ce == cudaSuccess; i++) ce = cudaGraphLaunch(exec, st);
    if (rc == PI_OK && ce == cudaSuccess) ce = cudaEventRecord(ev1, st);
    if (rc == PI_OK && ce == cudaSuccess) ce = cudaStreamSynchronize(st);
    float ms = 0.f;
    if (rc == PI_OK && ce == cudaSuccess) ce = cudaEventElapsedTime(&ms, ev0, ev1);
    *host_ms_per_rep = ms / (float)reps;
    if (ev0) cudaEventDestroy(ev0);
    if (ev1) cudaEventDestroy(ev1);
    if (exec) cudaGraphExecDestroy(exec);
    if (graph) cudaGraphDestroy(graph);
    if (rc) return rc;
    return ce == cudaSuccess ? PI_OK : cuda_fail(ce, "engine_time_stage");
}

int pi_engine_status(pi_engine * e, void * stream) {
    PI_REQUIRE(e, "engine_status: null");
    unsigned int s = 0;
    PI_CUDA(cudaMemcpyAsync(&s, e->status, 4, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    if (s) PI_CUDA(cudaMemsetAsync(e->status, 0, 4, (cudaStream_t)stream));      // reported once
    PI_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    if (s & 1u) { set_error("an exchange wait ran out: a peer rank did not deliver its partial vector"); return PI_ERR_TIMEOUT; }
    if (s & 14u) { set_error("a bulk-copy wait ran out in a weight-streaming kernel (status %u)", s); return PI_ERR_TIMEOUT; }
    return PI_OK;
}

int pi_engine_set_wait_cycles(pi_engine * e, long long cycles) {
    PI_REQUIRE(e && cycles >= 0, "engine_set_wait_cycles: bad arguments");
    e->wait_cycles = cycles;
    for (auto & gm : e->graphs) for (auto & g : gm) if (g) { cudaGraphExecDestroy(g); g = nullptr; }     // the bound is a kernel argument
    return PI_OK;
}

int pi_engine_set_trace(pi_engine * e, float * pred_trace) {
    PI_REQUIRE(e, "engine_set_trace: null");
    e->pred_trace = pred_trace;
    for (auto & gm : e->graphs) for (auto & g : gm) if (g) { cudaGraphExecDestroy(g); g = nullptr; }     // captured pointers are stale
    return PI_OK;
}

int pi_engine_debug(pi_engine * e, float ** pred, int32_t ** list, int32_t ** count) {
    PI_REQUIRE(e, "engine_debug: null");
    float * p = e->pred_trace ? e->pred_trace + (size_t)(e->c.n_layer - 1) * e->c.max_batch * e->F : e->pred;
    if (e->rows1 && (list || count)) {
        // one-token steps make bit masks only: build the list of the last layer's logits (first sequence) here, on the
        // default stream, after everything queued so far
        PI_CUDA(cudaDeviceSynchronize());
        CompactArgs ca;
        ca.idx = p; ca.idx_stride = e->F; ca.T = 1; ca.threshold = e->c.threshold; ca.n_local = e->F;
        ca.list = e->list; ca.count = e->count; ca.masks = e->masks; ca.ticket = e->ticket;
        const int rc = launch_compact(ca, nullptr);
        if (rc) return rc;
        PI_CUDA(cudaDeviceSynchronize());
    }
    if (pred) *pred = p;
    if (list) *list = e->list;
    if (count) *count = e->count;
    return PI_OK;
}

int pi_engine_launches(pi_engine * e) { return e ? e->launches : 0; }

int pi_engine_active_total(pi_engine * e, int reset, unsigned long long * host_total, void * stream) {
    PI_REQUIRE(e && host_total, "engine_active_total: null");
    cudaStream_t st = (cudaStream_t)stream;
    PI_CUDA(cudaMemcpyAsync(host_total, e->active_total, 8, cudaMemcpyDeviceToHost, st));
    if (reset) PI_CUDA(cudaMemsetAsync(e->active_total, 0, 8, st));
    PI_CUDA(cudaStreamSynchronize(st));
    return PI_OK;
}

#pragma GCC visibility pop
}  // extern "C"
