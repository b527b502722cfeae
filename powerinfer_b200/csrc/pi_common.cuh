// Shared device helpers and the internal launcher interface of the sm_100a kernels.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stddef.h>

#include "../../include/powerinfer_b200.h"

namespace pi {

// ---------------------------------------------------------------------------------------------- errors
void set_error(const char * fmt, ...);
int  cuda_fail(cudaError_t e, const char * what);

#define PI_CUDA(call)                                                         \
    do {                                                                      \
        cudaError_t e_ = (call);                                              \
        if (e_ != cudaSuccess) return ::pi::cuda_fail(e_, #call);             \
    } while (0)

#define PI_REQUIRE(cond, ...)                                                 \
    do {                                                                      \
        if (!(cond)) { ::pi::set_error(__VA_ARGS__); return PI_ERR_INVALID; } \
    } while (0)

#define PI_LAUNCH_CHECK(name)                                                 \
    do {                                                                      \
        cudaError_t e_ = cudaGetLastError();                                  \
        if (e_ != cudaSuccess) return ::pi::cuda_fail(e_, name);              \
    } while (0)

static inline int64_t imin64(int64_t a, int64_t b) { return a < b ? a : b; }
int sm_count();                                   // multiprocessors of the current device (cached per device)

// ---------------------------------------------------------------------------------------- activations
// An activation vector in the form a mat-vec consumes it (the reference's vec_dot_type, ggml.c:430-440):
//   F16 weights  -> h16 [T, n] halves (FP32 rounded to nearest even)
//   Q4_0 weights -> Q8_0 split into planes so that every plane loads as aligned 128-bit words:
//                   lo/hi [T, n/32] uint4 = int8 values 0..15 / 16..31 of each block,
//                   d [T, n/32] float (the FP16-rounded scale), s [T, n/32] int (sum of the block's 32 int8)
struct Act {
    const __half * h16 = nullptr;
    const uint4 *  lo  = nullptr;
    const uint4 *  hi  = nullptr;
    const float *  d   = nullptr;
    const int *    s   = nullptr;
};

struct ActBuf {            // writable view of the same planes
    __half * h16 = nullptr;
    uint4 *  lo  = nullptr;
    uint4 *  hi  = nullptr;
    float *  d   = nullptr;
    int *    s   = nullptr;
    Act view() const { Act a; a.h16 = h16; a.lo = lo; a.hi = hi; a.d = d; a.s = s; return a; }
};

// bytes of an ActBuf for T tokens of n values in the form `wtype` weights consume, rounded up to 256
size_t act_bytes(int wtype, int64_t n, int T);
// carve an ActBuf out of scratch memory; advances *p
ActBuf act_carve(int wtype, int64_t n, int T, char ** p);

// simple bump allocator over caller-provided scratch
struct Scratch {
    char * base; char * cur; char * end;
    Scratch(void * p, size_t n) : base((char *)p), cur((char *)p), end((char *)p + n) {}
    void * take(size_t bytes) {
        bytes = (bytes + 255) & ~size_t(255);
        if (cur + bytes > end) return nullptr;
        void * r = cur; cur += bytes; return r;
    }
};

// ------------------------------------------------------------------------------------------- launchers
// All launchers enqueue on `st` and return PI_OK / error.  Shapes are validated by the callers in pi_capi.cu.

int launch_quantize_q4_0(const float * x, void * q4, int64_t nrows, int64_t ncols, cudaStream_t st);
int launch_q4_0_repack(const void * src, void * dst, int64_t nrows, int64_t ncols, cudaStream_t st);
int launch_dequantize_q4_0(const void * q4p, float * y, int64_t nrows, int64_t ncols, cudaStream_t st);
int launch_quantize_q8_0_ggml(const float * x, void * q8, int64_t nrows, int64_t ncols, cudaStream_t st);

// x F32 [T, n] (row stride x_stride) -> activation planes for `wtype` weights
int launch_convert_act(int wtype, const float * x, int64_t x_stride, int64_t n, int T, ActBuf out, cudaStream_t st);


struct GemvArgs {
    int wtype = PI_TYPE_F16;
    const void * W = nullptr;          // [nrows, ncols]
    int64_t nrows = 0, ncols = 0;
    Act x;                             // T tokens
    int T = 1;
    // row selection: dense when list == nullptr
    const int32_t * list = nullptr;    // compacted LOCAL row numbers (sorted)
    const int32_t * count = nullptr;   // number of entries of list (device)
    const int32_t * bucket = nullptr;  // local row -> global neuron id (nullptr: identity)
    const float * idx = nullptr;       // predictor logits [T, idx_stride] by global id: per-token predicate
    int64_t idx_stride = 0;
    float threshold = 0.f;
    // epilogue
    const float * bias = nullptr;      // by destination row
    int relu = 0;
    float * dst = nullptr;             // F32 [T, dst_stride]; destination row = global id (sparse) or row (dense)
    int64_t dst_stride = 0;
    __half * dst16 = nullptr;          // optional FP16 copy of the result [T, dst_stride] (feeds an F16 mat-vec)
    // second matrix sharing the row selection (gate with up): dst = relu(W2 row . x) * (W row . x)
    const void * W2 = nullptr;
    // one token: activity bit masks (one word per 32 LOCAL rows) instead of a list; selects the register-streaming kernel
    const uint32_t * masks = nullptr;
    unsigned long long * rows_total = nullptr;   // with masks (optional): incremented by the number of active rows (statistics)
    // dense, one token: also write the activity bit masks of the result, bit (row % 32) of word (row / 32) = !(result <
    // masks_threshold): the predictor's mask, made where the logit is.  Room for (nrows + 63) / 64 * 2 words.
    uint32_t * masks_out = nullptr; float masks_threshold = 0.f;
    int pre_stages = -1;               // ring kernels: stages of weights requested before the dependency wait (-1: the whole ring)
    unsigned int * status = nullptr;   // device status word; when given, T == 1 shapes use the bulk-copy ring kernel
    bool pdl = false;                  // launch with programmatic dependent launch (the kernel waits for its producer itself)
};
int launch_gemv(const GemvArgs & a, cudaStream_t st);
// PI_ERR_UNSUPPORTED: not eligible; *wrote_masks: the kernel that ran honoured masks_out itself
int launch_gemv_ring(const GemvArgs & a, unsigned int * status, bool pdl, cudaStream_t st, bool * wrote_masks = nullptr);
int launch_gemv_mma(const GemvArgs & a, cudaStream_t st);                                     // FP16 rows, T <= 32; PI_ERR_UNSUPPORTED: not eligible
int launch_gemv_mma_q4(const GemvArgs & a, cudaStream_t st);                                  // Q4_0 rows, T >= 2; PI_ERR_UNSUPPORTED: not eligible

// predictor logits -> compacted list of LOCAL rows active for >= 1 token; also writes zeros (or relu(bias)) into
// h_init [T, h_stride] for rows that are inactive for a token when h_init != nullptr
struct CompactArgs {
    const float * idx = nullptr; int64_t idx_stride = 0; int T = 1; float threshold = 0.f;
    int64_t n_local = 0; const int32_t * bucket = nullptr;
    int32_t * list = nullptr; int32_t * count = nullptr;   // list == nullptr: only the bit masks are made (no list, no count, no ticket)
    float * zero_dst = nullptr; int64_t zero_stride = 0;   // dense [T, zero_stride] vector: entries of rows inactive for a token are
    const float * fill_bias = nullptr; int fill_relu = 0;  // set to 0, or to (relu of) fill_bias[g] (what the graph's bias add leaves there)
    uint32_t * masks = nullptr;        // scratch: one word per 32 local rows
    unsigned int * ticket = nullptr;   // scratch: one word, must be 0 on entry, is 0 again on exit
    unsigned long long * total = nullptr;   // optional running sum of the counts (statistics)
    bool pdl = false;
};
int launch_compact(const CompactArgs & a, cudaStream_t st);

// pulls the byte ranges into L2 (a hint; nothing may depend on it)

struct AxpyArgs {
    int wtype = PI_TYPE_F16;
    const void * Wt = nullptr; int64_t nrows = 0, ncols = 0;
    const float * h = nullptr; int64_t h_stride = 0; int T = 1;       // by global id
    const int32_t * list = nullptr; const int32_t * count = nullptr; const int32_t * bucket = nullptr;
    const uint32_t * masks = nullptr;                                 // one token: activity bit masks instead of the list
    // with masks: entries of h at inactive rows are taken as 0 whatever h holds there (nobody has cleared them); needs
    // bucket == nullptr.  Only the Q4_0 coefficients look at such entries (the scale of a block of 32 neurons).
    bool h_uncleared = false;
    const float * idx = nullptr; int64_t idx_stride = 0; float threshold = 0.f;
    // Q4_0: coefficient planes made by launch_neuron_q8 (int8 by global id, float scale per 32-neuron block)
    const int8_t * cq = nullptr; const float * cd = nullptr; int64_t c_stride = 0;
    float * partial = nullptr; int n_groups = 0;                      // [n_groups, T, ncols]: room for n_groups partial vectors
    unsigned int * status = nullptr;                                  // device status word (bit 1: a copy wait ran out); enables the
                                                                      // bulk-copy pipelined kernel for T == 1
    bool pdl = false;
};
int axpy_groups(int wtype, int64_t ncols, int T);                     // row groups the launcher will use
int launch_axpy(const AxpyArgs & a, cudaStream_t st, int * groups_used = nullptr);   // groups_used: partial vectors written
int launch_axpy_mma(const AxpyArgs & a, cudaStream_t st, int * groups_used);         // FP16, 2..32 tokens; PI_ERR_UNSUPPORTED: not eligible
// one token, rows named by bit masks, weights streamed into registers (pi_rows.cu); PI_ERR_UNSUPPORTED: not eligible
bool rows_eligible(int wtype, int64_t nrows, int64_t ncols);
int launch_gather_rows(const GemvArgs & a, cudaStream_t st);
int launch_axpy_rows(const AxpyArgs & a, cudaStream_t st, int * groups_used);
int axpy_rows_groups(int64_t nrows, int64_t ncols);                                  // partial vectors launch_axpy_rows writes
// one token, the whole sparse FFN in one launch (pi_ffn_rows.cu): h = act(up/gate rows . x) over the rows the masks name,
// partial[c] = sum of the rows of down_t times their coefficients, one partial vector per cluster (groups_used of them, at
// most n_groups).  h (optional) receives the activations by row.  PI_ERR_UNSUPPORTED: not eligible (use the two kernels).
struct FfnRowsArgs {
    int wtype = PI_TYPE_F16;
    const void * up = nullptr; const void * gate = nullptr; const void * down_t = nullptr;   // [nrows, ncols] each
    int64_t nrows = 0, ncols = 0;
    Act x; const uint32_t * masks = nullptr;
    const float * bias = nullptr; int relu = 0;
    float * h = nullptr; float * partial = nullptr; int n_groups = 0;
    unsigned long long * rows_total = nullptr;
    bool pdl = false;
};
int launch_ffn_rows(const FfnRowsArgs & a, cudaStream_t st, int * groups_used);
bool ffn_rows_eligible(const FfnRowsArgs & a);      // up / gate / down_t (null or not), shape and n_groups as they will be passed
// h F32 [T, stride] -> Q8_0 over 32-neuron blocks: cq int8 [T, stride], cd float [T, stride/32]
int launch_neuron_q8(const float * h, int64_t stride, int64_t n, int T, int8_t * cq, float * cd, cudaStream_t st);

// sum partial [n_groups, T, n] in group order (+ residual + bias) -> dst [T, n]
int static_scratch_address(void ** out);      // device address of pi_axpy_static's built-in scratch array on the current device
int launch_reduce_partials(const float * partial, int n_groups, int T, int64_t n, const float * residual,
                           const float * bias, float * dst, cudaStream_t st, bool pdl = false,
                           const float * residual2 = nullptr, double * stats_out = nullptr);

struct NormArgs {
    const float * x = nullptr; int T = 1; int64_t n = 0; int rms = 1; float eps = 0.f;
    const float * w = nullptr; const float * b = nullptr;
    // optional prologue: the vector to normalise is ((sum_j partial[j, t, :] | x) + in_bias + residual[t, :]) + residual2[t, :]
    // and is written to x_out (the new residual stream; may alias residual or residual2)
    const float * partial = nullptr; int n_groups = 0; const float * residual = nullptr; const float * residual2 = nullptr;
    const float * in_bias = nullptr;
    int64_t partial_stride = 0;        // floats between consecutive partials (0: T * n)
    // Sharded runs (xch != nullptr): the vector built so far (sum of the partials | x, + xch_extra) is this rank's share.
    // The norm writes it into slot rank_id of every other rank's mailbox, every value beside the number of the exchange
    // (plain 16-byte stores of two such pairs), polls the pairs of the same values in ITS OWN mailbox until they carry that
    // number (bounded by wait_cycles; on expiry bit 0 of *status is raised and the kernel carries on), and adds the shares
    // in rank order, so all ranks hold identical sums.
    // xch_index is the number of this exchange within the step (0 .. xch_per_step - 1).
    const pi_exchange * xch = nullptr; int xch_index = 0, xch_per_step = 1; const float * xch_extra = nullptr;
    long long wait_cycles = 0; unsigned int * status = nullptr;
    float * x_out = nullptr;
    float * y = nullptr;               // optional F32 output
    int act_type = 0; ActBuf act;      // optional activation planes of the normalised vector (0: none, else PI_TYPE_*)
    int act2_type = 0; ActBuf act2; int act2_src = 1;   // second set of planes, of the input (src 0) or the output (src 1)
    bool pdl = false;
};
int launch_norm(const NormArgs & a, cudaStream_t st);

int launch_rope(float * x, int T, int n_heads, int head_dim, const int32_t * pos, const float * cs, int neox, cudaStream_t st);

struct AttnArgs {
    const float * q = nullptr; const float * k = nullptr; const float * v = nullptr;
    __half * k_cache = nullptr; __half * v_cache = nullptr;
    const int32_t * seq = nullptr; const int32_t * pos = nullptr;
    int T = 1, n_head = 0, n_head_kv = 0, head_dim = 0, n_ctx = 0;
    int64_t q_stride = 0, kv_stride = 0;               // floats between tokens of q and of k / v (0: dense)
    const float * cs = nullptr; int neox = 0;          // fused RoPE of q and k from the angle table (nullptr: already rotated)
    float * out = nullptr;                             // optional F32 [T, n_head*head_dim]
    int out_act_type = 0; ActBuf out_act;              // optional activation planes of the output
    // 0: store the new K / V and attend in one launch (tokens of DIFFERENT sequences); 1: store only; 2: attend only.
    // Several tokens of one sequence in a step (prompt chunks) take a store pass, then an attend pass: a token must see
    // the rows of the tokens before it, which other CTAs write.
    int store_mode = 0;
    bool pdl = false;
};
int launch_attention(const AttnArgs & a, cudaStream_t st);

// ------------------------------------------------------------------------------------ device primitives
#ifdef __CUDACC__

// Programmatic dependent launch.  A kernel launched with launch_k(..., pdl = true) may start while its predecessor in the
// stream is still running; it must call pdl_wait() before it reads anything the predecessor wrote and before it writes
// anything the predecessor may still read (weights are immutable, so prefetching them before the wait is safe).
// pdl_launch() lets the NEXT kernel be scheduled early.  Both are no-ops for a normally launched kernel.
#ifndef PI_TIMELINE
__device__ __forceinline__ void pdl_wait()   { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#define PI_TL_MARK(i) do { } while (0)
#else
// Timeline builds (-DPI_TIMELINE -rdc=true, never the shipped library): thread 0 of CTA 0 of every kernel stamps the
// global timer when the kernel starts, when its dependency wait begins and when it returns (= its producer is complete).
extern __device__ unsigned long long g_tl[65536 * 16];
extern __device__ unsigned int g_tl_n;
static __shared__ unsigned int s_tl_slot;
__device__ __forceinline__ unsigned long long tl_time() { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }
__device__ __forceinline__ bool tl_me() { return blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0; }
__device__ __forceinline__ void pdl_launch() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (tl_me()) {
        const unsigned int s = atomicAdd(&g_tl_n, 1u) & 65535u;
        s_tl_slot = s;
        unsigned int smid; asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        g_tl[s * 16 + 0] = tl_time(); g_tl[s * 16 + 1] = (unsigned long long)clock64();
        g_tl[s * 16 + 2] = ((unsigned long long)gridDim.x << 32) | blockDim.x; g_tl[s * 16 + 3] = smid;
        for (int k = 8; k < 16; k++) g_tl[s * 16 + k] = 0;
    }
}
__device__ __forceinline__ void pdl_wait() {
    if (tl_me()) { g_tl[s_tl_slot * 16 + 4] = tl_time(); }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (tl_me()) { g_tl[s_tl_slot * 16 + 5] = tl_time(); g_tl[s_tl_slot * 16 + 6] = (unsigned long long)clock64(); }
}
#define PI_TL_MARK(i) do { if (tl_me()) g_tl[s_tl_slot * 16 + 8 + (i)] = tl_time(); } while (0)
#endif

// ---- shared-memory transaction barriers and bulk copies (plain cp.async.bulk: non-tensor, one destination CTA) used by
// every ring kernel.  A wait is always a bounded loop around mbar_try_wait in the caller.
__device__ __forceinline__ uint32_t smem_u32(const void * p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t * bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t * bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t * bar, unsigned parity) {
    unsigned ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Weights are read once per step and a step streams far more of them than L2 holds: they are marked evict-first, so what
// IS re-used between kernels (kernel code, activations, partial vectors, masks) is not pushed out of L2 by them.
#ifndef PI_L2_EVICT_FIRST
#define PI_L2_EVICT_FIRST 1
#endif
__device__ __forceinline__ uint64_t l2_stream_policy() {
    uint64_t pol;
    asm("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));   // not volatile: one per kernel after hoisting
    return pol;
}
__device__ __forceinline__ void bulk_g2s(void * dst, const void * src, unsigned bytes, uint64_t * bar) {
#if PI_L2_EVICT_FIRST
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
                 :: "r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(l2_stream_policy()) : "memory");
#else
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :: "r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
#endif
}
__device__ __forceinline__ void mbar_arrive(uint64_t * bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(smem_u32(bar)) : "memory");
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_k(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool pdl, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

__device__ __forceinline__ uint4 ldg_stream(const void * p) {     // read-once weights: bypass L1 allocation, evict-first in L2
    uint4 v;
#if PI_L2_EVICT_FIRST
    asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.u32 {%0,%1,%2,%3}, [%4], %5;"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p), "l"(l2_stream_policy()));
#else
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
#endif
    return v;
}
__device__ __forceinline__ uint2 ldg_stream8(const void * p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ double warp_sum_d(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ int warp_sum_i(int v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float2 h2f(uint32_t u) {               // two packed halves -> floats
    __half2 h = *reinterpret_cast<__half2 *>(&u);
    return __half22float2(h);
}
__device__ __forceinline__ float round_f16(float x) { return __half2float(__float2half_rn(x)); }

#endif  // __CUDACC__

}  // namespace pi
