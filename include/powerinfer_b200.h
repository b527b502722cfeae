/*
 * powerinfer_b200.h -- C ABI of the B200 (sm_100a) implementation of PowerInfer's decode hot path.
 *
 * The library replaces what the reference's CUDA back end (ggml-cuda.cu behind ggml-cuda.h) does
 * for the decode token loop: the activation predictor, the two neuron-sparse operators
 * ggml_mul_mat_idx / ggml_axpy, the Q4_0 / Q8_0 block formats they read, and the dense decode nodes
 * between them (norms, mat-vecs, RoPE, KV store, attention, lm head).  Each entry point names the
 * reference interface it stands in for (file:line in the reference tree).
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless its name starts with host_;
 *   - `stream` is a cudaStream_t passed as void*; all work is enqueued on it, nothing synchronises
 *     unless the comment says so;
 *   - matrices are row-major [rows, cols] with cols contiguous (ggml: ne[0] = cols), activations are
 *     [T tokens, n] with n contiguous;
 *   - functions return PI_OK or an error code and leave a message in pi_last_error(); they never call
 *     exit() (the reference does: ggml-cuda.cu:193-230);
 *   - nothing here allocates device memory: scratch comes in as (workspace, workspace_bytes), sized by
 *     pi_workspace_bytes().  Scratch must be 256-byte aligned.
 */
#ifndef POWERINFER_B200_H
#define POWERINFER_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PI_OK               0
#define PI_ERR_INVALID      1   /* bad argument (shape, alignment, null pointer) */
#define PI_ERR_CUDA         2   /* a CUDA runtime call failed; message holds cudaGetErrorString */
#define PI_ERR_WORKSPACE    3   /* workspace too small or misaligned */
#define PI_ERR_UNSUPPORTED  4
#define PI_ERR_TIMEOUT      5   /* a bounded device-side wait ran out (multi-GPU exchange) */

/* weight storage types (ggml.h GGML_TYPE_F16 / GGML_TYPE_Q4_0) */
#define PI_TYPE_F16   1         /* IEEE half, row of n halves */
#define PI_TYPE_Q4_0  2         /* ggml block_q4_0 {fp16 d; uint8 qs[16]} (ggml-quants.h:11-15), 18 bytes per 32 weights.
                                 * Device copies are held in the PLANAR form made by pi_q4_0_repack. */

const char * pi_last_error(void);
int          pi_version(void);

/* bytes of one weight row: F16 2n, Q4_0 18n/32 (same for the ggml and the planar layout) */
size_t pi_row_bytes(int wtype, int64_t ncols);

/* upper bound of the scratch any single op below needs for these extents */
size_t pi_workspace_bytes(int64_t ncols, int64_t nrows, int T);

/* ---- block formats (ggml-quants.c) ------------------------------------------------------------ */

/* quantize_row_q4_0_reference (ggml-quants.c:428-463): x F32 [nrows, ncols] -> ggml Q4_0 blocks. ncols % 32 == 0 */
int pi_quantize_q4_0(const float * x, void * q4_ggml, int64_t nrows, int64_t ncols, void * stream);

/* Re-layout done once at upload (the reference uploads through ggml_cuda_transform_tensor, ggml-cuda.cu:8946-9000,
 * and the host never looks at device bytes): ggml blocks -> per row [ncols/32 x 16 B nibbles][ncols/32 x fp16 d],
 * so nibbles load as aligned 128-bit words.  Needs ncols % 256 == 0.  src and dst must not overlap. */
int pi_q4_0_repack(const void * q4_ggml, void * q4_planar, int64_t nrows, int64_t ncols, void * stream);

/* dequantize_row_q4_0 (ggml-quants.c:1074-1092) from the planar layout -> F32 [nrows, ncols] */
int pi_dequantize_q4_0(const void * q4_planar, float * y, int64_t nrows, int64_t ncols, void * stream);

/* The activation quantiser of the CPU path, quantize_row_q8_0 (ggml-quants.c:702-760): per 32 values
 * d = amax/127 (stored as fp16), q = rne(x * 127/amax).  Output is ggml block_q8_0 (34-byte blocks). */
int pi_quantize_q8_0(const float * x, void * q8_ggml, int64_t nrows, int64_t ncols, void * stream);

/* ---- the two sparse operators (ggml.h:1094-1112) ------------------------------------------------ */

/* ggml_mul_mat_idx / ggml_mul_mat_idx_upscale -> GGML_OP_MUL_MAT_SPARSE
 * (CPU ggml.c:14030-14282; CUDA ggml-cuda.cu:4684-4824, 5489-5535, dispatch 8787-8803).
 *   W      [n_w_rows, ncols] F16 or planar Q4_0 : rows of up / gate held on this device
 *   x      F32 [T, ncols]
 *   idx    F32 [T, idx_stride]  predictor logits, indexed by GLOBAL neuron id
 *   bucket NULL, or int32 [n_w_rows] sorted global ids of the local rows (gpu_bucket, llama.cpp:2943-2967)
 *   dst    F32 [T, n_dst_rows]  dst[t, g] = idx[t, g] < threshold ? 0 : W[r,:] . x[t,:] with g = bucket ? bucket[r] : r (the reference's
 *          test, ggml.c:14256: a NaN logit therefore counts as active);
 *          rows no local row maps to are written 0.
 * Activations are rounded as the CPU path does before the dot product: to FP16 for F16 weights, to Q8_0 for Q4_0. */
int pi_mul_mat_idx(int wtype, const void * W, int64_t n_w_rows, int64_t ncols,
                   const float * x, int T, const float * idx, int64_t idx_stride,
                   const int32_t * bucket, float threshold,
                   float * dst, int64_t n_dst_rows,
                   void * workspace, size_t workspace_bytes, void * stream);

/* ggml_axpy -> GGML_OP_AXPY (CPU ggml.c:14314-14618, ggml-quants.c:2426-2509; CUDA ggml-cuda.cu:4478-4682,
 * dispatch 8805-8814).
 *   Wt     [n_w_rows, ncols] : rows of ffn_down_t held on this device (one row per neuron)
 *   h      F32 [T, h_stride]   FFN hidden activations, indexed by global neuron id
 *   dst    F32 [T, ncols]      dst[t,:] = sum over local rows r with !(idx[t,g] < threshold) of coef(h[t,g]) * Wt[r,:]
 * coef() is the CPU path's: h rounded to FP16 (F16 weights), or Q8_0 over blocks of 32 consecutive neurons (Q4_0
 * weights; then h_stride % 32 == 0 and a bucket must hold whole 32-neuron blocks).  The sum runs in a fixed order
 * (no atomics): two calls give identical bits. */
int pi_axpy(int wtype, const void * Wt, int64_t n_w_rows, int64_t ncols,
            const float * h, int T, int64_t h_stride, const float * idx, int64_t idx_stride,
            const int32_t * bucket, float threshold,
            float * dst,
            void * workspace, size_t workspace_bytes, void * stream);

/* The whole sparse FFN of llm_build_ffn_sparse (llama.cpp:4652-4757) for rows held on this device, given the predictor
 * logits: dst = sum over active r of act_r * down_t[r,:], with act_r = relu(gate[r,:].x) * (up[r,:].x) when gate != NULL
 * (llama), else relu(up[r,:].x + up_bias[g]) (falcon: up_bias NULL; opt).  One activation conversion, one compaction of
 * the mask, one gather launch for up and gate together, the axpy and the fixed-order reduction, chained with programmatic
 * dependent launch; numerically identical to pi_mul_mat_idx (x2) + the relu / mul / add nodes + pi_axpy.
 * The dense hidden vector (by global neuron id, idx_stride entries per token) lives in the workspace. */
int pi_sparse_ffn(int wtype, const void * up, const void * gate, const void * down_t, int64_t n_w_rows, int64_t ncols,
                  const float * x, int T, const float * idx, int64_t idx_stride, const int32_t * bucket, float threshold,
                  const float * up_bias, float * dst,
                  void * workspace, size_t workspace_bytes, void * stream);

/* pi_axpy for one token with NO workspace argument and no allocation of any kind.  It has no counterpart in the
 * reference (whose CUDA back end allocates from its own pool, ggml-cuda.cu:6387-6459): it exists for hosts that own all
 * device memory and forbid a plug-in to cudaMalloc, and for call sites where allocating is not permitted.  The scratch is a
 * 24 MiB array inside the library's device image (pi_axpy_static_max_bytes()), held by every GPU that loads the library
 * for the life of the process.  Limits: one token, n_w_rows and h_stride <= 65536, ncols <= 16384; anything larger is
 * rejected with PI_ERR_INVALID and a message naming pi_axpy.  The first call on each device looks the array's address up
 * (cudaGetSymbolAddress, with that device current); make that call before any stream capture begins.  All calls share the
 * one array: the words that must start at zero are cleared on the stream at the start of every call, and two calls that
 * overlap on the GPU (different streams, or different host threads) race on it, so serialise them. */
size_t pi_axpy_static_max_bytes(void);

/* Did the last pi_mul_mat_idx / pi_axpy / pi_sparse_ffn that used `workspace` finish all its bounded device-side waits (the
 * batch kernels stream rows through rings of bulk copies guarded by waits that give up after a limit rather than hang)?
 * PI_OK, or PI_ERR_TIMEOUT with the status bits in pi_last_error(): the call's result is then incomplete.  workspace NULL:
 * the built-in array of pi_axpy_static on the current device.  Synchronises `stream`.  (The engine has pi_engine_status.) */
int pi_op_status(const void * workspace, void * stream);
int pi_axpy_static(int wtype, const void * Wt, int64_t n_w_rows, int64_t ncols,
                   const float * h, int64_t h_stride, const float * idx, int64_t idx_stride,
                   const int32_t * bucket, float threshold, float * dst, void * stream);

/* ---- dense decode nodes ------------------------------------------------------------------------------ */

/* ggml_mul_mat with a weight matrix and T <= 32 activation columns (ggml.c:9598-9807; CUDA ggml-cuda.cu:4310-4414):
 * dst[t, r] = W[r,:] . x[t,:] (+ bias[r]).  Same activation rounding as above. */
int pi_mul_mat(int wtype, const void * W, int64_t nrows, int64_t ncols, const float * x, int T,
               const float * bias, float * dst, void * workspace, size_t workspace_bytes, void * stream);

/* The predictor sub-graph of llm_build_ffn_sparse (llama.cpp:4688-4695): idx = fc2 . relu(fc1 . p), both F16.
 *   fc1 [rank, d], fc2 [F, rank], p F32 [T, d] -> idx F32 [T, F] */
int pi_predictor(const void * fc1, const void * fc2, int64_t d, int64_t rank, int64_t F,
                 const float * p, int T, float * idx, void * workspace, size_t workspace_bytes, void * stream);

/* Predictor mask -> sorted list of the neurons active for at least one token (warp ballot / popc compaction).
 * There is no such list in the reference (every row is tested in place: ggml-cuda.cu:4694-4697); it is what lets the
 * sparse kernels spend no warp on an inactive row.  list int32 [F], count int32 [1]. */
int pi_active_list(const float * idx, int64_t F, int T, int64_t idx_stride, float threshold,
                   int32_t * list, int32_t * count, void * workspace, size_t workspace_bytes, void * stream);

/* ggml_rms_norm / ggml_norm followed by the weight (and bias) of llm_build_norm (llama.cpp:4420-4450;
 * ggml.c:9169-9284).  rms != 0 selects RMSNorm.  w, b may be NULL. */
int pi_norm(const float * x, int T, int64_t n, int rms, float eps, const float * w, const float * b,
            float * y, void * stream);

/* ggml_rope_custom modes 0 (pairs (2i, 2i+1)) and 2 (neox: pairs (i, i+n/2)) for one token per row
 * (ggml.c:11163-11325).  x F32 [T, n_heads*head_dim] in place; pos int32 [T].  The angle table
 * cs F32 [n_pos, head_dim/2, 2] = (cos, sin) is built on the host by pi_rope_table_host with the reference's
 * float recurrence theta *= theta_scale, so device and CPU path use the same angles. */
int pi_rope(float * x, int T, int n_heads, int head_dim, const int32_t * pos, const float * cs, int neox, void * stream);
void pi_rope_table_host(float * host_cs, int n_pos, int head_dim, float freq_base);

/* One decode step of attention for T tokens that each own one sequence position (llm_build_kv_store +
 * llm_build_kqv, llama.cpp:4383-4418, 4764-4850): store K,V of the new token as FP16, then softmax(QK^T/sqrt(hd)) V
 * over positions 0..pos[t] of its sequence.  Numerics follow the CPU path: Q and the probabilities are rounded to FP16,
 * exp goes through FP16 (ggml.c:10757-10759).
 *   q F32 [T, n_head*hd] (RoPE'd), k,v F32 [T, n_head_kv*hd]
 *   k_cache, v_cache FP16 [n_seq, n_ctx, n_head_kv*hd]; seq int32 [T] (NULL: sequence 0), pos int32 [T]
 *   out F32 [T, n_head*hd] */
int pi_attention_decode(const float * q, const float * k, const float * v, void * k_cache, void * v_cache,
                        const int32_t * seq, const int32_t * pos, int T, int n_head, int n_head_kv, int head_dim,
                        int n_ctx, float * out, void * stream);

/* ---- the decode token loop ------------------------------------------------------------------------------ */

/* One step of llama_decode (llama.cpp:6764-7006) over device-resident weights for up to max_batch sequences, one new
 * token each (examples/batched-bench/batched-bench.cpp:205-216), for the sparse architectures the reference builds
 * graphs for: llama and its bamboo variant (llama.cpp:4949-5084), falcon (5326-5468), opt (5086-5204).  The launch sequence of a step
 * is captured once per batch size and replayed as a CUDA graph. */

#define PI_ARCH_LLAMA   0
#define PI_ARCH_FALCON  1
#define PI_ARCH_OPT     2
#define PI_ARCH_BAMBOO  3   /* the llama graph with the symmetric gate h = relu(gate) * relu(up) (LLM_FFN_SYM, llama.cpp:4732-4738, 5028) */
#define PI_MAX_BATCH    32
#define PI_MAX_RANKS    8

typedef struct {
    int arch, wtype;                 /* PI_ARCH_*, PI_TYPE_* of the 2-D weights (predictor and embeddings are F16) */
    int n_layer, d, n_ff, n_head, n_head_kv, rank, n_vocab, n_ctx, n_pos;   /* n_pos: rows of pos_embd (opt) */
    float norm_eps, rope_base, threshold;
    int max_batch;
    int n_ranks, rank_id;            /* neuron / head sharding over GPUs; 1, 0 for a single GPU */
} pi_engine_config;

/* Per-layer device pointers.  With n_ranks > 1 a rank holds the slice [rank_id*n/n_ranks, (rank_id+1)*n/n_ranks) of the
 * FFN neurons and of the query / KV heads:
 *   wqkv  [(dq + 2 dkv), d]   rows: this rank's Q heads, then its K heads, then its V heads (dq = d/n_ranks)
 *   wo    [d, dq]             the columns of attn_output that multiply this rank's heads
 *   fc1   [rank, d] (replicated)   fc2 [n_ff/n_ranks, rank]   gate/up/down_t [n_ff/n_ranks, d]
 * 2-D weights are in `wtype` (Q4_0 in the planar layout), fc1/fc2 F16, vectors F32.  Unused pointers are NULL
 * (gate for falcon/opt, biases for llama, attn_norm2 unless falcon-40B style, ffn_norm for falcon). */
typedef struct {
    const float * attn_norm_w, * attn_norm_b, * attn_norm2_w, * attn_norm2_b;
    const void  * wqkv; const float * bqkv;
    const void  * wo;   const float * bo;
    const float * ffn_norm_w, * ffn_norm_b;
    const void  * fc1, * fc2;
    const void  * gate, * up, * down_t;
    const float * up_b, * down_b;
} pi_layer_weights;

typedef struct {
    const void  * tok_embd;          /* F16 [n_vocab, d] */
    const void  * pos_embd;          /* F16 [n_pos, d], opt only */
    const float * out_norm_w, * out_norm_b;
    const void  * output;            /* [n_vocab, d] in wtype; NULL: tied to tok_embd (opt, llama.cpp:5199) */
} pi_model_weights;

/* Peer mailboxes for the per-layer exchange of partial d_model vectors (n_ranks > 1).  Every rank owns a mailbox of
 * [2, n_ranks, slot_floats] 8-byte pairs {F32 value, u32 number of the exchange} in ITS OWN memory, zero-initialised;
 * peers write into it with plain stores (the mapped addresses of every rank's mailbox, own included, are listed here),
 * nobody reads remote memory.  slot_floats >= max_batch * d, so a mailbox takes 2 * n_ranks * slot_floats * 8 bytes.
 * `epoch` is a zero-initialised u32 word in this rank's memory: the engine counts its steps there (all ranks run the
 * same steps, so all agree on the number of every exchange).  The exchange itself is part of the norm kernel that
 * consumes the sum: it writes this rank's share into every other rank's mailbox, each value beside the number of the
 * exchange, and waits (bounded) until the pairs of its own values in its own mailbox carry that number: one trip over
 * the link, no flag, no fence.  The two halves of a mailbox alternate, so a rank that runs ahead cannot overwrite what
 * a slower one has not yet read. */
typedef struct {
    int n_ranks, rank_id;
    int64_t slot_floats;
    unsigned int * mailbox_local;
    unsigned int * mailbox_peer[PI_MAX_RANKS];
    unsigned int * epoch;
} pi_exchange;

typedef struct pi_engine pi_engine;

size_t pi_engine_workspace_bytes(const pi_engine_config * cfg);    /* 0 when cfg is invalid (see pi_last_error) */
size_t pi_engine_kv_bytes(const pi_engine_config * cfg);           /* bytes of EACH of k_cache and v_cache */

/* Replaces llama_new_context_with_model + the per-call graph build (llama.cpp:6408-6753, 6846-6850).  The engine keeps
 * the pointers it is given: weights, workspace (256-byte aligned) and the FP16 KV caches [n_layer, max_batch, n_ctx,
 * dkv] must stay valid and are owned by the caller.  Synchronises `stream` once. */
int  pi_engine_create(const pi_engine_config * cfg, const pi_model_weights * globals, const pi_layer_weights * layers,
                      void * workspace, size_t workspace_bytes, void * k_cache, void * v_cache, void * stream,
                      pi_engine ** out);
void pi_engine_destroy(pi_engine * e);
int  pi_engine_set_exchange(pi_engine * e, const pi_exchange * x);

/* Device-side I/O of a step: tokens int32 [max_batch], pos int32 [max_batch] (position of each sequence's new token),
 * logits F32 [max_batch, n_vocab], argmax int32 [max_batch] (llama_sample_token_greedy, llama.cpp:8617). */
int  pi_engine_io(pi_engine * e, int32_t ** tokens, int32_t ** pos, float ** logits, int32_t ** argmax);

/* Enqueue one step for T sequences on `stream`; inputs are read from / results left in the pi_engine_io buffers. */
int  pi_engine_decode(pi_engine * e, int T, void * stream);

/* Greedy feedback on the device: tokens[t] = argmax[t], pos[t] += 1 (clamped to the context), for a free-running
 * decode loop that never leaves the GPU. */
int  pi_engine_advance(pi_engine * e, int T, void * stream);

/* llama_decode + llama_get_logits with HOST buffers (llama.cpp:10672, 6960-6978): copies T token ids and positions to the
 * device, runs the step, copies back T*n_vocab logits (host_logits != NULL) and T greedy ids (host_argmax != NULL), and
 * synchronises `stream`. */
int  pi_engine_decode_host(pi_engine * e, const int32_t * host_tokens, const int32_t * host_pos, int T,
                           float * host_logits, int32_t * host_argmax, void * stream);

/* Prompt processing (llama_decode with a batch of n_tokens > 1 tokens of one sequence: llama.cpp:6764-7006; the reference's
 * batched sparse kernels are ggml-cuda.cu:4607-4682, 4758-4824): n_tokens consecutive tokens of sequence `seq`, the first
 * at position pos0, go through the engine in chunks of up to max_batch tokens per step.  A chunk's step stores the K / V of
 * all its tokens first and then attends causally, reads every weight row once for the whole chunk, and applies each
 * token's own predictor mask (union list for reading, per-token predicate for writing: ggml.c:14250-14259).  Only the last
 * token's logits are computed and copied back (host_logits_last F32 [n_vocab], host_argmax_last int32 [1]; both may be
 * NULL: then no lm head runs at all).  Synchronises `stream`. */
int  pi_engine_prefill_host(pi_engine * e, const int32_t * host_tokens, int n_tokens, int seq, int pos0,
                            float * host_logits_last, int32_t * host_argmax_last, void * stream);

/* Same step launched kernel by kernel with CUDA events around each stage; adds the milliseconds of each stage to
 * host_ms[PI_N_STAGES] and the number of kernel launches to *host_launches.  Synchronises. */
#define PI_STAGE_NORM      0
#define PI_STAGE_QKV       1
#define PI_STAGE_ATTN      2
#define PI_STAGE_WO        3
#define PI_STAGE_PRED      4
#define PI_STAGE_COMPACT   5
#define PI_STAGE_UPGATE    6
#define PI_STAGE_DOWN      7
#define PI_STAGE_LM_HEAD   8
#define PI_STAGE_EXCHANGE  9
#define PI_STAGE_OTHER    10
#define PI_STAGE_FFN      11     /* up/gate, activation and down in one launch (one token, where the shape allows it) */
#define PI_N_STAGES       12
int  pi_engine_profile_step(pi_engine * e, int T, float * host_ms, int * host_launches, void * stream);
/* Measurement helper: the kernels of ONE stage for every layer, back to back in a CUDA graph exactly as they are launched
 * inside a step (programmatic dependent launch included), `reps` replays between two events.  host_ms_per_rep = time of
 * one replay, host_launches = kernels in it.  The stage's outputs are overwritten with values computed from stale
 * inputs: run a real step afterwards before using results.  Synchronises `stream`. */
int  pi_engine_time_stage(pi_engine * e, int T, int stage, int reps, float * host_ms_per_rep, int * host_launches, void * stream);

/* Device status word: PI_OK, or PI_ERR_TIMEOUT after a bounded device-side wait ran out (an exchange whose peer never
 * delivered, a bulk copy that never landed); the step that hit it still ran to its end.  The word is cleared once it has
 * been reported, and the engine stays usable.  Synchronises `stream`. */
int  pi_engine_status(pi_engine * e, void * stream);
/* Bound of the exchange waits in SM clock cycles (0: the default, about a second). */
int  pi_engine_set_wait_cycles(pi_engine * e, long long cycles);

/* For tests: device pointers of the predictor logits F32 [T, n_ff/n_ranks] that the LAST layer of the last step left
 * behind, and the sorted active list and count of its first sequence (built here when the step itself only made bit
 * masks).  Synchronises the device. */
int  pi_engine_debug(pi_engine * e, float ** pred, int32_t ** list, int32_t ** count);
/* For tests: keep every layer's predictor logits.  pred_trace F32 [n_layer, max_batch, n_ff/n_ranks] (NULL: off). */
int  pi_engine_set_trace(pi_engine * e, float * pred_trace);
/* Sum of the active-list lengths (this rank's neurons) over all layers and steps since the last reset.  Synchronises. */
int  pi_engine_active_total(pi_engine * e, int reset, unsigned long long * host_total, void * stream);
int  pi_engine_launches(pi_engine * e);                            /* kernels enqueued by one step of the last batch size run */

/* ---- model and placement files (host only: no device is touched) -------------------------------------- */

/* Reader for the reference's files: PowerInfer model files (GGUF v2 / v3 container with the magic PWRI, ggml.c:19481-19495;
 * tensors and keys as llm_load_hparams / llm_load_sparse_model_tensors read them, llama.cpp:2330-2400, 3159-3390) and
 * `.generated.gpuidx` placement files (architecture generic.gpu_index, blk.i.gpu_idx / blk.i.gpu_bucket int32 tensors,
 * split.vram_capacity; llama.cpp:2781-2871).  The file is mapped read-only; tensor data pointers point into the mapping
 * and stay valid until pi_model_file_close.  Uploading is the caller's business (F16 as stored; Q4_0 through
 * pi_q4_0_repack).  Malformed or truncated files give PI_ERR_INVALID, never a crash. */
typedef struct pi_model_file pi_model_file;
int     pi_model_file_open(const char * path, pi_model_file ** out);
void    pi_model_file_close(pi_model_file * f);
int     pi_model_file_is_powerinfer(const pi_model_file * f);       /* 1: magic PWRI, 0: plain GGUF */
/* Key lookups.  PI_ERR_INVALID when the key is absent or holds another kind of value.  Any integer or bool type
 * answers get_u64 (negative values are refused); F32 / F64 answer get_f32; the string is NOT NUL-terminated. */
int     pi_model_file_get_u64(const pi_model_file * f, const char * key, uint64_t * value);
int     pi_model_file_get_f32(const pi_model_file * f, const char * key, float * value);
int     pi_model_file_get_str(const pi_model_file * f, const char * key, const char ** str, size_t * len);
/* Tensors: ggml_type as in enum ggml_type (ggml.h:307-333: 0 F32, 1 F16, 2 Q4_0, 18 I32), ne[4] with ne[0] the fastest
 * dimension (unused dimensions 1), nbytes 0 and data NULL for types whose size this reader does not know. */
int64_t pi_model_file_n_tensors(const pi_model_file * f);
int     pi_model_file_tensor_at(const pi_model_file * f, int64_t i, const char ** name, int * ggml_type, int64_t ne[4],
                                const void ** data, size_t * nbytes);
int     pi_model_file_tensor(const pi_model_file * f, const char * name, int * ggml_type, int64_t ne[4],
                             const void ** data, size_t * nbytes);
/* The hyper-parameters of a sparse model file as an engine configuration for one GPU and one sequence (max_batch 1,
 * n_ranks 1): architecture (llama / bamboo / falcon / opt), weight type of blk.0.ffn_up, dimensions, norm epsilon key of
 * the architecture, rope base, powerinfer.sparse_threshold, predictor rank = rows of blk.0.fc1, vocabulary = rows of
 * token_embd.  PI_ERR_INVALID when the file is not a sparse model (no fc1 / fc2 / ffn_down_t tensors). */
int     pi_model_file_engine_config(const pi_model_file * f, pi_engine_config * cfg);

/* ---- plumbing for multi-GPU mailboxes (these DO allocate; nothing else does) ----------------------------- */
int  pi_device_malloc(void ** ptr, size_t bytes);                  /* cudaMalloc + zero fill */
int  pi_device_free(void * ptr);
int  pi_ipc_export(void * ptr, void * host_handle64);              /* cudaIpcGetMemHandle -> 64 bytes */
int  pi_ipc_import(const void * host_handle64, void ** ptr);       /* cudaIpcOpenMemHandle */
int  pi_ipc_close(void * ptr);

#ifdef __cplusplus
}
#endif
#endif
