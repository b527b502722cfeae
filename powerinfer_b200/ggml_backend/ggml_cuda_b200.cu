// A drop-in for the reference's CUDA back end: this file defines the C symbols the reference's host code binds through
// ggml-cuda.h:14-64 (ggml.c:2217, 14778, 14792, 16692; llama.cpp under GGML_USE_CUBLAS), so that the UNMODIFIED ggml.c and
// llama.cpp, compiled with -DGGML_USE_CUBLAS, link against libggml_cuda_b200.so instead of ggml-cuda.cu.
//
// It is built against the reference's own ggml.h (struct ggml_tensor, the op enums) and calls nothing but the C ABI of
// libpowerinfer_b200.so (include/powerinfer_b200.h) plus a few small kernels of its own for the glue nodes.
//
// Contract kept (ggml-cuda.cu:9218-9346): ggml_cuda_compute_forward returns true when the node is done, false when the
// caller must compute it on the CPU; it returns true without work for every thread but 0 and for the INIT / FINALIZE
// phases.  tensor->extra is this back end's own struct (the host only stores the pointer, or walks the device pointer
// through ggml_cuda_get_data_pp).  Weights arrive through ggml_cuda_transform_tensor; Q4_0 matrices are re-laid out into
// the planar rows the kernels read (pi_q4_0_repack).  Graph nodes live in one scratch buffer at the offsets the host's
// allocator computed (ggml_cuda_assign_scratch_offset), views share their parent's memory.
// Unlike the reference, errors never call exit() from inside a CUDA call chain silently: a failed pi_* / CUDA call prints
// its message and aborts, which is the reference's GGML_ASSERT convention at this ABI.
//
// Every node is served by its own launch here.  Node -> kernel:
//   MUL_MAT (weight x activations)  pi_mul_mat        MUL_MAT_SPARSE  pi_mul_mat_idx       AXPY      pi_axpy
//   RMS_NORM / NORM                 pi_norm           ROPE            pi_rope              the rest  small kernels below
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <vector>

#include "ggml.h"
#include "ggml-cuda.h"
#include "powerinfer_b200.h"

#define B2_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

// Every copy, fill and kernel of this file goes through ONE stream (g_stream, non-blocking).  A synchronous cudaMemcpy
// from pageable host memory may return before its DMA has landed, and a non-blocking stream is not ordered behind the
// default stream: a kernel on g_stream could then read the destination too early.  So: async calls on g_stream only.
// ------------------------------------------------------------------------------------------------ state
struct TensorDev {                 // what tensor->extra points to
    void * data;                   // device address (first member: ggml_cuda_get_data_pp hands out its address)
    int    planar_q4;              // Q4_0 rows are in the planar upload layout
    int    owned;                  // data came from cudaMalloc here and is freed by ggml_cuda_free_data
    size_t bytes;
};

bool         g_loaded = false;
int          g_device = 0, g_device_count = 0;
cudaStream_t g_stream = nullptr;
float        g_threshold = 0.0f;
char *       g_scratch = nullptr;
size_t       g_scratch_size = 0, g_scratch_bump = 0;
void *       g_ws = nullptr;       // workspace of the pi_* operators
size_t       g_ws_bytes = 0;
char *       g_tmp = nullptr;      // staging for CPU-resident operands / results of one node
size_t       g_tmp_bytes = 0, g_tmp_used = 0;
std::vector<TensorDev> g_node_extras(1 << 15);    // per-graph extras, reused round-robin (a graph has a few thousand nodes)
size_t       g_node_extra_next = 0;
std::map<std::pair<int, uint32_t>, float *> g_rope_tables;   // (head_dim, freq_base bits) -> device table
constexpr int ROPE_TABLE_POS = 16384;
long long    g_served[GGML_OP_COUNT], g_declined[GGML_OP_COUNT];

[[noreturn]] void die(const char * what, const char * detail) {
    fprintf(stderr, "ggml_cuda_b200: %s: %s\n", what, detail ? detail : "");
    abort();
}
#define CU(call) do { cudaError_t e_ = (call); if (e_ != cudaSuccess) die(#call, cudaGetErrorString(e_)); } while (0)
#define PI(call) do { int rc_ = (call); if (rc_ != PI_OK) die(#call, pi_last_error()); } while (0)

TensorDev * node_extra() {
    TensorDev * e = &g_node_extras[g_node_extra_next];
    g_node_extra_next = (g_node_extra_next + 1) % g_node_extras.size();
    memset(e, 0, sizeof *e);
    return e;
}

TensorDev * dev_of(const ggml_tensor * t) { return (TensorDev *) t->extra; }

// The few facts about tensors this file needs, computed from the struct itself so that the library does not depend on
// symbols of the host program (the meaning is that of ggml_type_size / ggml_blck_size / ggml_nbytes / ggml_is_contiguous).
size_t t_type_size(ggml_type t) {
    switch (t) {
        case GGML_TYPE_F32: case GGML_TYPE_I32: return 4;
        case GGML_TYPE_F16: case GGML_TYPE_I16: return 2;
        case GGML_TYPE_I8:   return 1;
        case GGML_TYPE_Q4_0: return 18;
        case GGML_TYPE_Q8_0: return 34;
        default: die("tensor type not supported by this back end", "");
    }
}
int64_t t_blck(ggml_type t) { return t == GGML_TYPE_Q4_0 || t == GGML_TYPE_Q8_0 ? 32 : 1; }
int64_t t_nelements(const ggml_tensor * t) { return t->ne[0] * t->ne[1] * t->ne[2] * t->ne[3]; }
int64_t t_nrows(const ggml_tensor * t) { return t->ne[1] * t->ne[2] * t->ne[3]; }
size_t t_nbytes(const ggml_tensor * t) {
    size_t n = (size_t)(t->ne[0] / t_blck(t->type)) * t->nb[0];
    if (t_blck(t->type) == 1) n = t_type_size(t->type) + (size_t)(t->ne[0] - 1) * t->nb[0];
    for (int i = 1; i < 4; i++) n += (size_t)(t->ne[i] - 1) * t->nb[i];
    return n;
}
bool t_contiguous(const ggml_tensor * t) {
    return t->nb[0] == t_type_size(t->type) && t->nb[1] == t->nb[0] * (size_t)(t->ne[0] / t_blck(t->type)) &&
           t->nb[2] == t->nb[1] * (size_t)t->ne[1] && t->nb[3] == t->nb[2] * (size_t)t->ne[2];
}
bool on_gpu(const ggml_tensor * t) { return t && (t->backend == GGML_BACKEND_GPU || t->backend == GGML_BACKEND_GPU_SPLIT); }

void * tmp_take(size_t bytes) {
    bytes = (bytes + 255) & ~size_t(255);
    if (g_tmp_used + bytes > g_tmp_bytes) {
        // grow: everything queued so far may still read the old buffer
        CU(cudaStreamSynchronize(g_stream));
        const size_t want = (g_tmp_used + bytes) * 2 + (size_t(1) << 20);
        char * n = nullptr;
        CU(cudaMalloc(&n, want));
        if (g_tmp) { CU(cudaMemcpyAsync(n, g_tmp, g_tmp_used, cudaMemcpyDeviceToDevice, g_stream)); CU(cudaStreamSynchronize(g_stream)); CU(cudaFree(g_tmp)); }
        g_tmp = n; g_tmp_bytes = want;
    }
    void * p = g_tmp + g_tmp_used;
    g_tmp_used += bytes;
    return p;
}

void * workspace(size_t need) {
    if (need > g_ws_bytes) {
        CU(cudaStreamSynchronize(g_stream));
        if (g_ws) CU(cudaFree(g_ws));
        CU(cudaMalloc(&g_ws, need + 256));
        g_ws_bytes = need + 256;
    }
    return g_ws;
}

// device address of an operand: resident tensors as they are; CPU-resident ones are staged for this node
const void * operand(const ggml_tensor * t) {
    if (on_gpu(t)) {
        if (!t->extra || !dev_of(t)->data) die("operand without device memory", t->name);
        return dev_of(t)->data;
    }
    if (!t_contiguous(t)) die("CPU-resident operand is not contiguous", t->name);
    void * p = tmp_take(t_nbytes(t));
    CU(cudaMemcpyAsync(p, t->data, t_nbytes(t), cudaMemcpyHostToDevice, g_stream));
    return p;
}

struct Result { void * dev; ggml_tensor * t; bool staged; };
Result result_of(ggml_tensor * t) {
    Result r; r.t = t;
    if (on_gpu(t)) { if (!t->extra || !dev_of(t)->data) die("result without device memory", t->name); r.dev = dev_of(t)->data; r.staged = false; }
    else {
        if (!t_contiguous(t)) die("CPU-resident result is not contiguous", t->name);
        r.dev = tmp_take(t_nbytes(t)); r.staged = true;
    }
    return r;
}
void finish(const Result & r) {           // a CPU-resident result goes home, and the host may read it when we return
    if (!r.staged) return;
    CU(cudaMemcpyAsync(r.t->data, r.dev, t_nbytes(r.t), cudaMemcpyDeviceToHost, g_stream));
    CU(cudaStreamSynchronize(g_stream));
}

// ------------------------------------------------------------------------------------------------ glue kernels
struct Shape { int64_t ne[4]; int64_t nb[4]; };           // extents, strides in BYTES
Shape shape_of(const ggml_tensor * t) { Shape s; for (int i = 0; i < 4; i++) { s.ne[i] = t->ne[i]; s.nb[i] = (int64_t)t->nb[i]; } return s; }

// dst = a (op) b with b repeated over the dimensions where it is shorter (ggml_add / ggml_mul, ggml.c:7077, 7752); F32
template <int OP>
__global__ void k_binary(const char * a, Shape sa, const char * b, Shape sb, char * d, Shape sd, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t r = i;
        const int64_t i0 = r % sd.ne[0]; r /= sd.ne[0];
        const int64_t i1 = r % sd.ne[1]; r /= sd.ne[1];
        const int64_t i2 = r % sd.ne[2]; const int64_t i3 = r / sd.ne[2];
        const float x = *(const float *)(a + i0 * sa.nb[0] + i1 * sa.nb[1] + i2 * sa.nb[2] + i3 * sa.nb[3]);
        const float y = *(const float *)(b + (i0 % sb.ne[0]) * sb.nb[0] + (i1 % sb.ne[1]) * sb.nb[1] + (i2 % sb.ne[2]) * sb.nb[2] + (i3 % sb.ne[3]) * sb.nb[3]);
        *(float *)(d + i0 * sd.nb[0] + i1 * sd.nb[1] + i2 * sd.nb[2] + i3 * sd.nb[3]) = OP == 0 ? x + y : x * y;
    }
}

// OP 0: relu, 1: scale by *s
template <int OP>
__global__ void k_unary(const float * a, const float * s, float * d, int64_t n) {
    const float f = OP == 1 ? *s : 0.f;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        d[i] = OP == 0 ? fmaxf(a[i], 0.f) : a[i] * f;
}

// ggml_cpy / ggml_cont / ggml_dup: element k of the source (in its logical order) goes to element k of the destination
// (in ITS logical order); F32 or F16 on either side
template <typename TS, typename TD>
__global__ void k_copy(const char * a, Shape sa, char * d, Shape sd, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t r = i;
        const int64_t a0 = r % sa.ne[0]; r /= sa.ne[0];
        const int64_t a1 = r % sa.ne[1]; r /= sa.ne[1];
        const int64_t a2 = r % sa.ne[2]; const int64_t a3 = r / sa.ne[2];
        r = i;
        const int64_t d0 = r % sd.ne[0]; r /= sd.ne[0];
        const int64_t d1 = r % sd.ne[1]; r /= sd.ne[1];
        const int64_t d2 = r % sd.ne[2]; const int64_t d3 = r / sd.ne[2];
        const float v = (float)*(const TS *)(a + a0 * sa.nb[0] + a1 * sa.nb[1] + a2 * sa.nb[2] + a3 * sa.nb[3]);
        *(TD *)(d + d0 * sd.nb[0] + d1 * sd.nb[1] + d2 * sd.nb[2] + d3 * sd.nb[3]) = (TD)v;
    }
}

// ggml_soft_max over rows of n values with the CPU path's numerics (ggml.c:10708-10777): exp through FP16 on an
// FP16-rounded argument, -inf entries give 0, the sum in double.  One warp per row.
__global__ void k_soft_max(const float * x, float * y, int64_t n, int64_t rows) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const float * xr = x + row * n; float * yr = y + row * n;
    float mx = -INFINITY;
    for (int64_t i = lane; i < n; i += 32) mx = fmaxf(mx, xr[i]);
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    double sum = 0.0;
    for (int64_t i = lane; i < n; i += 32) {
        float v = 0.f;
        if (xr[i] != -INFINITY) {
            const float a = __half2float(__float2half_rn(xr[i] - mx));
            v = __half2float(__float2half_rn(expf(a)));
        }
        yr[i] = v; sum += (double)v;
    }
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float inv = (float)(1.0 / sum);
    for (int64_t i = lane; i < n; i += 32) yr[i] = yr[i] * inv;
}

// ggml_mul_mat for operands that are not uploaded weights (the K and V cache views against q / the probabilities,
// llama.cpp:4792-4830): dst[i0, i1, i2, i3] = sum_k a[k, i0, i2 / r2, i3 / r3] * b[k, i1, i2, i3].  a is F16 or F32 with
// contiguous k; b is F32 and, when a is F16, rounded to FP16 first as the CPU path does (ggml.c:9703-9716).  Warp per output.
template <typename TA>
__global__ void k_mul_mat_views(const char * a, Shape sa, const char * b, Shape sb, float * d, Shape sd, int64_t n_out) {
    const int lane = threadIdx.x & 31;
    const int64_t o = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (o >= n_out) return;
    int64_t r = o;
    const int64_t i0 = r % sd.ne[0]; r /= sd.ne[0];
    const int64_t i1 = r % sd.ne[1]; r /= sd.ne[1];
    const int64_t i2 = r % sd.ne[2]; const int64_t i3 = r / sd.ne[2];
    const int64_t r2 = sb.ne[2] / sa.ne[2], r3 = sb.ne[3] / sa.ne[3];
    const char * ap = a + i0 * sa.nb[1] + (i2 / r2) * sa.nb[2] + (i3 / r3) * sa.nb[3];
    const char * bp = b + i1 * sb.nb[1] + i2 * sb.nb[2] + i3 * sb.nb[3];
    float acc = 0.f;
    for (int64_t k = lane; k < sa.ne[0]; k += 32) {
        const float av = (float)*(const TA *)(ap + k * sa.nb[0]);
        float bv = *(const float *)(bp + k * sb.nb[0]);
        if (sizeof(TA) == 2) bv = __half2float(__float2half_rn(bv));
        acc = fmaf(av, bv, acc);
    }
    for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
    if (lane == 0) *(float *)((char *)d + i0 * sd.nb[0] + i1 * sd.nb[1] + i2 * sd.nb[2] + i3 * sd.nb[3]) = acc;
}

int grid_for(int64_t n, int per_block) { int64_t g = (n + per_block - 1) / per_block; return (int)(g < 1 ? 1 : (g > 65535 * 8 ? 65535 * 8 : g)); }

// ------------------------------------------------------------------------------------------------ node handlers
int pi_type(ggml_type t) { return t == GGML_TYPE_Q4_0 ? PI_TYPE_Q4_0 : PI_TYPE_F16; }

bool is_uploaded_matrix(const ggml_tensor * t) {
    if (!on_gpu(t) || !t->extra || t->op != GGML_OP_NONE || t->ne[2] != 1 || t->ne[3] != 1) return false;
    if (t->type == GGML_TYPE_F16) return t->ne[0] % 8 == 0 && t_contiguous(t);
    return t->type == GGML_TYPE_Q4_0 && dev_of(t)->planar_q4;
}

void op_binary(ggml_tensor * dst, int op) {
    const ggml_tensor * a = dst->src[0], * b = dst->src[1];
    if (a->type != GGML_TYPE_F32 || b->type != GGML_TYPE_F32 || dst->type != GGML_TYPE_F32) die("add / mul: F32 only", dst->name);
    const void * pa = operand(a), * pb = operand(b);
    Result r = result_of(dst);
    const int64_t n = t_nelements(dst);
    Shape sa = shape_of(a), sb = shape_of(b), sd = shape_of(dst);
    if (op == 0) k_binary<0><<<grid_for(n, 256), 256, 0, g_stream>>>((const char *)pa, sa, (const char *)pb, sb, (char *)r.dev, sd, n);
    else         k_binary<1><<<grid_for(n, 256), 256, 0, g_stream>>>((const char *)pa, sa, (const char *)pb, sb, (char *)r.dev, sd, n);
    CU(cudaGetLastError());
    finish(r);
}

void op_unary(ggml_tensor * dst, int op) {
    const ggml_tensor * a = dst->src[0];
    if (a->type != GGML_TYPE_F32 || !t_contiguous(a) || !t_contiguous(dst)) die("relu / scale: contiguous F32 only", dst->name);
    const void * pa = operand(a);
    const void * ps = op == 1 ? operand(dst->src[1]) : nullptr;
    Result r = result_of(dst);
    const int64_t n = t_nelements(dst);
    if (op == 0) k_unary<0><<<grid_for(n, 256), 256, 0, g_stream>>>((const float *)pa, nullptr, (float *)r.dev, n);
    else         k_unary<1><<<grid_for(n, 256), 256, 0, g_stream>>>((const float *)pa, (const float *)ps, (float *)r.dev, n);
    CU(cudaGetLastError());
    finish(r);
}

void op_copy(const ggml_tensor * src, ggml_tensor * dst) {
    const void * pa = operand(src);
    Result r = result_of(dst);
    const int64_t n = t_nelements(src);
    if (n != t_nelements(dst)) die("cpy: element counts differ", dst->name);
    Shape sa = shape_of(src), sd = shape_of(dst);
    const int g = grid_for(n, 256);
    if      (src->type == GGML_TYPE_F32 && dst->type == GGML_TYPE_F32) k_copy<float, float><<<g, 256, 0, g_stream>>>((const char *)pa, sa, (char *)r.dev, sd, n);
    else if (src->type == GGML_TYPE_F32 && dst->type == GGML_TYPE_F16) k_copy<float, __half><<<g, 256, 0, g_stream>>>((const char *)pa, sa, (char *)r.dev, sd, n);
    else if (src->type == GGML_TYPE_F16 && dst->type == GGML_TYPE_F16) k_copy<__half, __half><<<g, 256, 0, g_stream>>>((const char *)pa, sa, (char *)r.dev, sd, n);
    else if (src->type == GGML_TYPE_F16 && dst->type == GGML_TYPE_F32) k_copy<__half, float><<<g, 256, 0, g_stream>>>((const char *)pa, sa, (char *)r.dev, sd, n);
    else die("cpy: unsupported type pair", dst->name);
    CU(cudaGetLastError());
    finish(r);
}

void op_norm(ggml_tensor * dst, int rms) {
    const ggml_tensor * a = dst->src[0];
    if (a->type != GGML_TYPE_F32 || !t_contiguous(a)) die("norm: contiguous F32 only", dst->name);
    float eps; memcpy(&eps, dst->op_params, sizeof eps);
    const void * pa = operand(a);
    Result r = result_of(dst);
    PI(pi_norm((const float *)pa, (int)t_nrows(a), a->ne[0], rms, eps, nullptr, nullptr, (float *)r.dev, g_stream));
    finish(r);
}

void op_rope(ggml_tensor * dst) {
    const ggml_tensor * a = dst->src[0], * pos = dst->src[1];
    const int n_dims = dst->op_params[1], mode = dst->op_params[2];
    float freq_base, freq_scale, ext_factor;
    memcpy(&freq_base, dst->op_params + 5, 4); memcpy(&freq_scale, dst->op_params + 6, 4); memcpy(&ext_factor, dst->op_params + 7, 4);
    if (a->type != GGML_TYPE_F32 || !t_contiguous(a) || n_dims != a->ne[0] || (mode & ~2) != 0 || freq_scale != 1.0f || ext_factor != 0.0f || a->ne[3] != 1)
        die("rope: only modes 0 and 2 over whole heads, no scaling", dst->name);
    uint32_t fb; memcpy(&fb, &freq_base, 4);
    float *& table = g_rope_tables[std::make_pair(n_dims, fb)];
    if (!table) {                                          // the reference's float recurrence theta *= theta_scale, made once
        std::vector<float> host((size_t)ROPE_TABLE_POS * n_dims);
        pi_rope_table_host(host.data(), ROPE_TABLE_POS, n_dims, freq_base);
        CU(cudaMalloc(&table, host.size() * 4));
        CU(cudaMemcpyAsync(table, host.data(), host.size() * 4, cudaMemcpyHostToDevice, g_stream));
        CU(cudaStreamSynchronize(g_stream));                  // `host` dies at the end of this block
    }
    const void * pa = operand(a);
    const void * pp = operand(pos);
    Result r = result_of(dst);
    if (r.dev != pa) CU(cudaMemcpyAsync(r.dev, pa, t_nbytes(a), cudaMemcpyDeviceToDevice, g_stream));
    PI(pi_rope((float *)r.dev, (int)a->ne[2], (int)a->ne[1], n_dims, (const int32_t *)pp, table, (mode & 2) ? 1 : 0, g_stream));
    finish(r);
}

void op_soft_max(ggml_tensor * dst) {
    const ggml_tensor * a = dst->src[0];
    if (a->type != GGML_TYPE_F32 || !t_contiguous(a)) die("soft_max: contiguous F32 only", dst->name);
    const void * pa = operand(a);
    Result r = result_of(dst);
    const int64_t rows = t_nrows(a);
    k_soft_max<<<grid_for(rows, 8), 256, 0, g_stream>>>((const float *)pa, (float *)r.dev, a->ne[0], rows);
    CU(cudaGetLastError());
    finish(r);
}

constexpr int TOKENS_PER_CALL = 32;    // the pi_* operators take up to 32 activation columns; prompts go through in pieces

void op_mul_mat(ggml_tensor * dst) {
    const ggml_tensor * a = dst->src[0], * b = dst->src[1];
    if (b->type != GGML_TYPE_F32) die("mul_mat: F32 activations only", dst->name);
    if (is_uploaded_matrix(a) && t_contiguous(b) && b->ne[2] == 1 && b->ne[3] == 1) {
        const void * pb = operand(b);
        Result r = result_of(dst);
        const int64_t nrows = a->ne[1], ncols = a->ne[0], T = b->ne[1];
        for (int64_t t0 = 0; t0 < T; t0 += TOKENS_PER_CALL) {
            const int tt = (int)(T - t0 < TOKENS_PER_CALL ? T - t0 : TOKENS_PER_CALL);
            void * ws = workspace(pi_workspace_bytes(ncols, nrows, tt));
            PI(pi_mul_mat(pi_type(a->type), dev_of(a)->data, nrows, ncols, (const float *)pb + t0 * ncols, tt, nullptr,
                          (float *)r.dev + t0 * nrows, ws, g_ws_bytes, g_stream));
        }
        finish(r);
        return;
    }
    if ((a->type != GGML_TYPE_F16 && a->type != GGML_TYPE_F32) || a->nb[0] != t_type_size(a->type) || b->nb[0] != 4)
        die("mul_mat: operand layout not supported", dst->name);
    const void * pa = operand(a), * pb = operand(b);
    Result r = result_of(dst);
    const int64_t n = t_nelements(dst);
    Shape sa = shape_of(a), sb = shape_of(b), sd = shape_of(dst);
    if (a->type == GGML_TYPE_F16) k_mul_mat_views<__half><<<grid_for(n, 8), 256, 0, g_stream>>>((const char *)pa, sa, (const char *)pb, sb, (float *)r.dev, sd, n);
    else                          k_mul_mat_views<float><<<grid_for(n, 8), 256, 0, g_stream>>>((const char *)pa, sa, (const char *)pb, sb, (float *)r.dev, sd, n);
    CU(cudaGetLastError());
    finish(r);
}

// ggml_mul_mat_idx / _upscale and ggml_axpy: src[0] rows on this device, src[1] activations, src[2] predictor logits,
// src[3] NULL (all rows here) or gpu_bucket (ggml.c:4100-4190)
void op_sparse(ggml_tensor * dst, bool axpy) {
    const ggml_tensor * w = dst->src[0], * x = dst->src[1], * idx = dst->src[2], * bucket = dst->src[3];
    if (!is_uploaded_matrix(w)) die("sparse op: weight is not an uploaded F16 / Q4_0 matrix", w->name);
    if (x->type != GGML_TYPE_F32 || idx->type != GGML_TYPE_F32 || !t_contiguous(x)) die("sparse op: F32 operands only", dst->name);
    const void * px = operand(x), * pidx = operand(idx);
    const int32_t * pbucket = bucket ? (const int32_t *)operand(bucket) : nullptr;
    Result r = result_of(dst);
    const int64_t n_w_rows = w->ne[1], ncols = w->ne[0], T = x->ne[1];
    const int64_t idx_stride = (int64_t)(idx->nb[1] / 4);
    for (int64_t t0 = 0; t0 < T; t0 += TOKENS_PER_CALL) {
        const int tt = (int)(T - t0 < TOKENS_PER_CALL ? T - t0 : TOKENS_PER_CALL);
        if (!axpy) {
            const int64_t n_dst = dst->ne[0];
            void * ws = workspace(pi_workspace_bytes(ncols, n_dst > n_w_rows ? n_dst : n_w_rows, tt));
            PI(pi_mul_mat_idx(pi_type(w->type), dev_of(w)->data, n_w_rows, ncols, (const float *)px + t0 * ncols, tt,
                              (const float *)pidx + t0 * idx_stride, idx_stride, pbucket, g_threshold,
                              (float *)r.dev + t0 * n_dst, n_dst, ws, g_ws_bytes, g_stream));
        } else {
            const int64_t h_stride = x->ne[0];
            void * ws = workspace(pi_workspace_bytes(ncols, h_stride > n_w_rows ? h_stride : n_w_rows, tt));
            PI(pi_axpy(pi_type(w->type), dev_of(w)->data, n_w_rows, ncols, (const float *)px + t0 * h_stride, tt, h_stride,
                       (const float *)pidx + t0 * idx_stride, idx_stride, pbucket, g_threshold,
                       (float *)r.dev + t0 * ncols, ws, g_ws_bytes, g_stream));
        }
    }
    finish(r);
}

// ggml_get_rows for a table the host keeps (the reference never offloads the embedding tables, llama.cpp:654-658) when
// the result is device-resident (opt's pos_embd): the rows are gathered on the host and sent over.
void op_get_rows_host_table(ggml_tensor * dst) {
    const ggml_tensor * table = dst->src[0], * ids = dst->src[1];
    if (on_gpu(table) || !ids->data || (table->type != GGML_TYPE_F16 && table->type != GGML_TYPE_F32) || dst->type != GGML_TYPE_F32)
        die("get_rows: only host-resident F16 / F32 tables", dst->name);
    const int64_t n = table->ne[0], rows = t_nelements(ids);
    std::vector<float> host((size_t)n * rows);
    for (int64_t r = 0; r < rows; r++) {
        const int32_t id = ((const int32_t *)ids->data)[r];
        const char * src = (const char *)table->data + (size_t)id * table->nb[1];
        for (int64_t c = 0; c < n; c++)
            host[(size_t)r * n + c] = table->type == GGML_TYPE_F32 ? ((const float *)src)[c] : __half2float(((const __half *)src)[c]);
    }
    Result r = result_of(dst);
    CU(cudaMemcpyAsync(r.dev, host.data(), host.size() * 4, cudaMemcpyHostToDevice, g_stream));
    CU(cudaStreamSynchronize(g_stream));                   // `host` dies at return
    finish(r);
}

// ------------------------------------------------------------------------------------------------ buffers
bool is_view_op(ggml_op op) { return op == GGML_OP_RESHAPE || op == GGML_OP_TRANSPOSE || op == GGML_OP_VIEW || op == GGML_OP_PERMUTE; }

bool shares_parent_memory(const ggml_tensor * t) {
    return (t->src[0] != nullptr && t->src[0]->data == t->data) || t->op == GGML_OP_VIEW;
}

size_t view_offset(const ggml_tensor * t) {
    size_t off = 0;
    if (t->op == GGML_OP_VIEW) memcpy(&off, t->op_params, sizeof off);
    return off;
}

void ensure_scratch() {
    if (!g_scratch && g_scratch_size) CU(cudaMalloc(&g_scratch, g_scratch_size));
}

// marks a node (and the view chain / copy target it hangs on) as device-resident and, unless `defer`, gives it memory:
// the parent's for views and in-place results, the copy target's for CPY, scratch or its own allocation otherwise
void assign(ggml_tensor * t, bool scratch, bool force_inplace, bool defer) {
    if (scratch && g_scratch_size == 0) return;
    t->backend = GGML_BACKEND_GPU;
    if (t->src[0] && t->src[0]->backend == GGML_BACKEND_CPU && is_view_op(t->src[0]->op)) assign(t->src[0], scratch, force_inplace, defer);
    if (t->op == GGML_OP_CPY && t->src[1]->backend == GGML_BACKEND_CPU) assign(t->src[1], scratch, force_inplace, defer);
    if (scratch && defer) return;
    TensorDev * e;
    if ((shares_parent_memory(t) || force_inplace) && on_gpu(t->src[0])) {
        e = node_extra();
        e->data = (char *)dev_of(t->src[0])->data + view_offset(t);
    } else if (t->op == GGML_OP_CPY) {
        e = node_extra();
        e->data = dev_of(t->src[1])->data;
    } else if (scratch) {
        const size_t size = t_nbytes(t);
        if (size > g_scratch_size) die("node larger than the scratch buffer", t->name);
        if (g_scratch_bump + size > g_scratch_size) g_scratch_bump = 0;
        ensure_scratch();
        e = node_extra();
        e->data = g_scratch + g_scratch_bump;
        g_scratch_bump += (size + 255) & ~size_t(255);
    } else {
        e = new TensorDev();
        e->bytes = t_nbytes(t); e->owned = 1;
        CU(cudaMalloc(&e->data, e->bytes));
        CU(cudaMemsetAsync(e->data, 0, e->bytes, g_stream));
    }
    t->extra = e;
}

void upload(const void * host, ggml_tensor * t, bool alloc_only) {
    const size_t bytes = t_nbytes(t);
    TensorDev * e = new TensorDev();
    e->bytes = bytes; e->owned = 1;
    CU(cudaMalloc(&e->data, bytes + 256));
    const bool planar = t->type == GGML_TYPE_Q4_0 && t->ne[0] % 256 == 0 && t->ne[2] == 1 && t->ne[3] == 1;
    e->planar_q4 = planar;
    if (!alloc_only) {
        if (planar) {                                      // ggml blocks -> planar rows, through a staging copy
            void * staging = nullptr;
            CU(cudaMalloc(&staging, bytes));
            CU(cudaMemcpyAsync(staging, host, bytes, cudaMemcpyHostToDevice, g_stream));
            PI(pi_q4_0_repack(staging, e->data, t->ne[1], t->ne[0], g_stream));
            CU(cudaStreamSynchronize(g_stream));
            CU(cudaFree(staging));
        } else {
            CU(cudaMemcpyAsync(e->data, host, bytes, cudaMemcpyHostToDevice, g_stream));
            CU(cudaStreamSynchronize(g_stream));
        }
    }
    t->extra = e;
}

}  // namespace

// ------------------------------------------------------------------------------------------------ the symbol set
B2_EXPORT void ggml_init_cublas(void) {
    static bool done = false;
    if (done) return;
    done = true;
    if (cudaGetDeviceCount(&g_device_count) != cudaSuccess || g_device_count <= 0) { g_device_count = 0; cudaGetLastError(); return; }
    if (cudaSetDevice(0) != cudaSuccess || cudaStreamCreateWithFlags(&g_stream, cudaStreamNonBlocking) != cudaSuccess) { cudaGetLastError(); return; }
    g_loaded = true;
    fprintf(stderr, "ggml_init_cublas: powerinfer_b200 back end (pi_version %d), %d device(s)\n", pi_version(), g_device_count);
}
B2_EXPORT bool ggml_cublas_loaded(void) { return g_loaded; }

B2_EXPORT void * ggml_cuda_host_malloc(size_t size) {
    void * p = nullptr;
    if (!g_loaded || cudaMallocHost(&p, size) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    return p;
}
B2_EXPORT void ggml_cuda_host_free(void * ptr) { if (ptr) cudaFreeHost(ptr); }

// the reference uses this to steal large CPU mat-muls for cuBLAS; this back end serves device-resident nodes only
B2_EXPORT bool ggml_cuda_can_mul_mat(const ggml_tensor *, const ggml_tensor *, ggml_tensor *) { return false; }
B2_EXPORT void ggml_cuda_set_tensor_split(const float *) {}
B2_EXPORT void ggml_cuda_set_mul_mat_q(bool) {}
B2_EXPORT void ggml_cuda_set_main_device(int main_device) {
    if (main_device >= 0 && main_device < g_device_count && main_device != g_device) {
        g_device = main_device;
        CU(cudaSetDevice(g_device));
    }
}
B2_EXPORT void ggml_cuda_set_device_constants(float sparse_pred_threshold) { g_threshold = sparse_pred_threshold; }

B2_EXPORT void ggml_cuda_transform_tensor(void * data, ggml_tensor * tensor) { upload(data, tensor, false); }
B2_EXPORT void ggml_cuda_alloc_tensor(ggml_tensor * tensor) { upload(nullptr, tensor, true); }
B2_EXPORT void ggml_cuda_free_data(ggml_tensor * tensor) {
    if (!tensor || !on_gpu(tensor) || !tensor->extra) return;
    TensorDev * e = dev_of(tensor);
    if (!e->owned) return;
    cudaFree(e->data);
    delete e;
    tensor->extra = nullptr;
}
B2_EXPORT void ** ggml_cuda_get_data_pp(ggml_tensor * tensor) { return &dev_of(tensor)->data; }

// one host row into the device row dst currently points at (the striped upload of hot neurons walks the destination
// pointer row by row: llama.cpp:2921-2934).  Q4_0 rows are re-laid out like whole matrices are.
B2_EXPORT void ggml_cuda_cpy_1d(ggml_tensor * dst, const ggml_tensor * src) {
    const size_t bytes = t_nbytes(src);
    if (src->type == GGML_TYPE_Q4_0 && src->ne[0] % 256 == 0) {
        g_tmp_used = 0;
        void * staging = tmp_take(bytes);
        CU(cudaMemcpyAsync(staging, src->data, bytes, cudaMemcpyHostToDevice, g_stream));
        PI(pi_q4_0_repack(staging, dev_of(dst)->data, 1, src->ne[0], g_stream));
        CU(cudaStreamSynchronize(g_stream));
    } else {
        CU(cudaMemcpyAsync(dev_of(dst)->data, src->data, bytes, cudaMemcpyHostToDevice, g_stream));
        CU(cudaStreamSynchronize(g_stream));
    }
}

B2_EXPORT void ggml_cuda_assign_buffers(ggml_tensor * t)               { if (t) assign(t, true, false, false); }
B2_EXPORT void ggml_cuda_assign_buffers_no_alloc(ggml_tensor * t)      { if (t) assign(t, true, false, true); }
B2_EXPORT void ggml_cuda_assign_buffers_no_scratch(ggml_tensor * t)    { if (t) assign(t, false, false, false); }
B2_EXPORT void ggml_cuda_assign_buffers_force_inplace(ggml_tensor * t) { if (t) assign(t, false, true, false); }

// the host's graph allocator has placed the node at `offset` of its own buffer; the device scratch mirrors that layout
// (llama.cpp:6859-6873)
B2_EXPORT void ggml_cuda_assign_scratch_offset(ggml_tensor * t, size_t offset) {
    if (g_scratch_size == 0) return;
    ensure_scratch();
    TensorDev * e = node_extra();
    if (shares_parent_memory(t) && on_gpu(t->src[0]) && t->src[0]->extra) e->data = (char *)dev_of(t->src[0])->data + view_offset(t);
    else if (t->op == GGML_OP_CPY && on_gpu(t->src[1]) && t->src[1]->extra) e->data = dev_of(t->src[1])->data;   // a copy's result IS its target
    else if (offset <= g_scratch_size && t_nbytes(t) <= g_scratch_size - offset) e->data = g_scratch + offset;
    else e->data = nullptr;      // not a node of the host's graph buffer (e.g. a view of the KV cache): never dereferenced as such
    t->extra = e;
}

B2_EXPORT void ggml_cuda_copy_to_device(ggml_tensor * t) {
    CU(cudaMemcpyAsync(dev_of(t)->data, t->data, t_nbytes(t), cudaMemcpyHostToDevice, g_stream));
    CU(cudaStreamSynchronize(g_stream));
}
B2_EXPORT void ggml_cuda_copy_to_host(ggml_tensor * t) {
    CU(cudaMemcpyAsync(t->data, dev_of(t)->data, t_nbytes(t), cudaMemcpyDeviceToHost, g_stream));
    CU(cudaStreamSynchronize(g_stream));
}

B2_EXPORT void ggml_cuda_set_scratch_size(size_t scratch_size) {
    if (scratch_size > g_scratch_size) {
        ggml_cuda_free_scratch();
        g_scratch_size = scratch_size;
    }
}
B2_EXPORT void ggml_cuda_free_scratch(void) {
    if (!g_scratch) return;
    cudaStreamSynchronize(g_stream);
    cudaFree(g_scratch);
    g_scratch = nullptr;
}

B2_EXPORT int ggml_cuda_get_device_count(void) { int n = 0; if (cudaGetDeviceCount(&n) != cudaSuccess) { cudaGetLastError(); return 0; } return n; }
B2_EXPORT void ggml_cuda_get_device_description(int device, char * description, size_t description_size) {
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) { cudaGetLastError(); snprintf(description, description_size, "unknown"); return; }
    snprintf(description, description_size, "%s", prop.name);
}
B2_EXPORT size_t ggml_cuda_get_free_memory(int device) {
    size_t free_b = 0, total_b = 0;
    int cur = 0;
    if (cudaGetDevice(&cur) != cudaSuccess) { cudaGetLastError(); return 0; }
    cudaSetDevice(device);
    if (cudaMemGetInfo(&free_b, &total_b) != cudaSuccess) { cudaGetLastError(); free_b = 0; }
    cudaSetDevice(cur);
    return free_b;
}
B2_EXPORT ggml_backend_t ggml_backend_cuda_init(void) { return nullptr; }   // the backend-v2 vtable is not used by inference

B2_EXPORT bool ggml_cuda_compute_forward(ggml_compute_params * params, ggml_tensor * tensor) {
    if (!g_loaded) return false;
    const ggml_tensor * s0 = tensor->src[0], * s1 = tensor->src[1];
    const bool src0_on_device = on_gpu(s0);
    const bool any_on_device = tensor->backend == GGML_BACKEND_GPU || src0_on_device || (s1 && s1->backend == GGML_BACKEND_GPU);
    const bool sparse = tensor->op == GGML_OP_MUL_MAT_SPARSE || tensor->op == GGML_OP_AXPY;
    enum { NOP, ADD, MUL, RELU, SCALE, COPY, RMS, NORM, ROPE, SOFT, MM, SPARSE_MM, AXPY, ROWS, DECLINE } what = DECLINE;
    if ((sparse && !src0_on_device) || !any_on_device) what = DECLINE;      // weights on the host: the CPU computes (with sparsity)
    else switch (tensor->op) {
        case GGML_OP_RESHAPE: case GGML_OP_VIEW: case GGML_OP_PERMUTE: case GGML_OP_TRANSPOSE: what = NOP; break;
        case GGML_OP_GET_ROWS:       what = !src0_on_device && tensor->backend == GGML_BACKEND_GPU ? ROWS : DECLINE; break;
        case GGML_OP_ADD:            what = ADD; break;
        case GGML_OP_MUL:            what = MUL; break;
        case GGML_OP_UNARY:          what = (ggml_unary_op)tensor->op_params[0] == GGML_UNARY_OP_RELU ? RELU : DECLINE; break;
        case GGML_OP_SCALE:          what = SCALE; break;
        case GGML_OP_CPY: case GGML_OP_CONT: case GGML_OP_DUP: what = COPY; break;
        case GGML_OP_RMS_NORM:       what = RMS; break;
        case GGML_OP_NORM:           what = NORM; break;
        case GGML_OP_ROPE:           what = ROPE; break;
        case GGML_OP_SOFT_MAX:       what = SOFT; break;
        case GGML_OP_MUL_MAT:        what = s0->ne[3] == s1->ne[3] ? MM : DECLINE; break;
        case GGML_OP_MUL_MAT_SPARSE: what = SPARSE_MM; break;
        case GGML_OP_AXPY:           what = AXPY; break;
        default:                     what = DECLINE; break;
    }
    if (what == DECLINE) {
        if (params->ith == 0 && params->type == GGML_TASK_COMPUTE) g_declined[tensor->op]++;
        if (src0_on_device) die("node with device-resident src[0] cannot be served", tensor->name);   // the CPU could not read it either
        return false;
    }
    if (params->ith != 0 || params->type != GGML_TASK_COMPUTE) return true;
    g_served[tensor->op]++;
    g_tmp_used = 0;
    switch (what) {
        case NOP:       break;
        case ADD:       op_binary(tensor, 0); break;
        case MUL:       op_binary(tensor, 1); break;
        case RELU:      op_unary(tensor, 0); break;
        case SCALE:     op_unary(tensor, 1); break;
        case COPY:      op_copy(tensor->src[0], tensor->op == GGML_OP_CPY ? tensor->src[1] : tensor); break;   // ggml_cpy(a, b): b's memory is the destination
        case RMS:       op_norm(tensor, 1); break;
        case NORM:      op_norm(tensor, 0); break;
        case ROPE:      op_rope(tensor); break;
        case SOFT:      op_soft_max(tensor); break;
        case MM:        op_mul_mat(tensor); break;
        case SPARSE_MM: op_sparse(tensor, false); break;
        case AXPY:      op_sparse(tensor, true); break;
        case ROWS:      op_get_rows_host_table(tensor); break;
        default:        break;
    }
    return true;
}

// ---- not part of ggml-cuda.h: how many COMPUTE-phase nodes of each op this back end served / handed back to the CPU
B2_EXPORT void ggml_cuda_b200_counts(int op, long long * served, long long * declined) {
    if (op < 0 || op >= GGML_OP_COUNT) { if (served) *served = 0; if (declined) *declined = 0; return; }
    if (served) *served = g_served[op];
    if (declined) *declined = g_declined[op];
}
B2_EXPORT int ggml_cuda_b200_op_count(void) { return GGML_OP_COUNT; }
