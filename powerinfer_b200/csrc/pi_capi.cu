// extern "C" surface: argument checks, scratch carving, and the launch sequence of each operator.
#include "pi_common.cuh"

#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>

namespace pi {

static thread_local char g_err[512] = "";

void set_error(const char * fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
}

int cuda_fail(cudaError_t e, const char * what) {
    set_error("CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
    return PI_ERR_CUDA;
}

int sm_count() {
    static int cached[16] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (dev < 16 && cached[dev]) return cached[dev];
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    if (dev < 16) cached[dev] = n;
    return n;
}

static bool aligned(const void * p, size_t a) { return ((uintptr_t)p & (a - 1)) == 0; }

static int check_w(int wtype, int64_t ncols, const void * W) {
    PI_REQUIRE(wtype == PI_TYPE_F16 || wtype == PI_TYPE_Q4_0, "unknown weight type %d", wtype);
    if (wtype == PI_TYPE_Q4_0) PI_REQUIRE(ncols > 0 && ncols % 256 == 0, "Q4_0 rows need ncols %% 256 == 0 (got %lld)", (long long)ncols);
    else                       PI_REQUIRE(ncols > 0 && ncols % 8 == 0, "F16 rows need ncols %% 8 == 0 (got %lld)", (long long)ncols);
    PI_REQUIRE(W != nullptr && aligned(W, 16), "weight pointer must be non-null and 16-byte aligned");
    return PI_OK;
}

struct SparseScratch { int32_t * list; int32_t * count; unsigned int * ticket; unsigned int * status; uint32_t * masks; };

// The control words come FIRST in every sparse operator's workspace (count, ticket, status at bytes 0, 4, 8), so that
// pi_op_status can find the status word of whichever operator used the workspace last.
static bool carve_sparse(Scratch & s, int64_t n_rows, SparseScratch & o) {
    int32_t * ct = (int32_t *)s.take(256);
    o.list = (int32_t *)s.take((size_t)n_rows * 4);
    o.masks = (uint32_t *)s.take((size_t)((n_rows + 31) / 32) * 4);
    if (!o.list || !ct || !o.masks) return false;
    o.count = ct; o.ticket = (unsigned int *)(ct + 1); o.status = (unsigned int *)(ct + 2);
    return true;
}

}  // namespace pi

using namespace pi;

extern "C" {
#pragma GCC visibility push(default)

const char * pi_last_error(void) { return g_err; }
int pi_version(void) { return 1; }

size_t pi_row_bytes(int wtype, int64_t ncols) {
    return wtype == PI_TYPE_Q4_0 ? (size_t)(ncols / 32) * 18 : (size_t)ncols * 2;
}

size_t pi_workspace_bytes(int64_t ncols, int64_t nrows, int T) {
    auto up = [](size_t v) { return (v + 255) & ~size_t(255); };
    if (T < 1) T = 1;
    const int64_t m = ncols > nrows ? ncols : nrows;
    size_t b = 0;
    b += act_bytes(PI_TYPE_Q4_0, (m + 31) / 32 * 32, T) + act_bytes(PI_TYPE_F16, m, T) * 2;   // activation planes, predictor hidden
    b += up((size_t)nrows * 4) + 256 + up((size_t)(nrows + 31) / 32 * 4);                    // list, count/ticket, masks
    b += up((size_t)T * nrows) + up((size_t)T * (nrows / 32 + 1) * 4);                       // Q8 coefficients of h
    b += up((size_t)T * nrows * 4);                                                          // hidden vector of pi_sparse_ffn
    b += up((size_t)256 * T * ncols * 4);                                                    // axpy partials (<= 256 groups)
    return b + 4096;
}

int pi_quantize_q4_0(const float * x, void * q4, int64_t nrows, int64_t ncols, void * stream) {
    PI_REQUIRE(x && q4 && nrows >= 0 && ncols % 32 == 0, "quantize_q4_0: bad arguments");
    return launch_quantize_q4_0(x, q4, nrows, ncols, (cudaStream_t)stream);
}

int pi_q4_0_repack(const void * src, void * dst, int64_t nrows, int64_t ncols, void * stream) {
    PI_REQUIRE(src && dst && src != dst && nrows >= 0, "q4_0_repack: bad pointers");
    PI_REQUIRE(ncols % 256 == 0 && aligned(dst, 16) && aligned(src, 2), "q4_0_repack: ncols %% 256 == 0 and a 16-byte aligned destination required");
    return launch_q4_0_repack(src, dst, nrows, ncols, (cudaStream_t)stream);
}

int pi_dequantize_q4_0(const void * q4p, float * y, int64_t nrows, int64_t ncols, void * stream) {
    PI_REQUIRE(q4p && y && ncols % 256 == 0 && aligned(q4p, 16), "dequantize_q4_0: bad arguments");
    return launch_dequantize_q4_0(q4p, y, nrows, ncols, (cudaStream_t)stream);
}

int pi_quantize_q8_0(const float * x, void * q8, int64_t nrows, int64_t ncols, void * stream) {
    PI_REQUIRE(x && q8 && ncols % 32 == 0 && aligned(q8, 2), "quantize_q8_0: bad arguments");
    return launch_quantize_q8_0_ggml(x, q8, nrows, ncols, (cudaStream_t)stream);
}

int pi_mul_mat(int wtype, const void * W, int64_t nrows, int64_t ncols, const float * x, int T,
               const float * bias, float * dst, void * workspace, size_t workspace_bytes, void * stream) {
    int rc = check_w(wtype, ncols, W);
    if (rc) return rc;
    PI_REQUIRE(x && dst && T >= 0 && nrows >= 0, "mul_mat: bad arguments");
    if (T == 0 || nrows == 0) return PI_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (!aligned(workspace, 256) || workspace_bytes < act_bytes(wtype, ncols, T)) { set_error("mul_mat: workspace too small or misaligned"); return PI_ERR_WORKSPACE; }
    char * p = (char *)workspace;
    ActBuf act = act_carve(wtype, ncols, T, &p);
    if ((rc = launch_convert_act(wtype, x, ncols, ncols, T, act, st))) return rc;
    GemvArgs g;
    g.wtype = wtype; g.W = W; g.nrows = nrows; g.ncols = ncols; g.x = act.view(); g.T = T;
    g.bias = bias; g.dst = dst; g.dst_stride = nrows;
    if (workspace_bytes >= act_bytes(wtype, ncols, T) + 256) {       // room for a status word: the bulk-copy ring kernels are eligible
        g.status = (unsigned int *)p;
        PI_CUDA(cudaMemsetAsync(g.status, 0, 4, st));
    }
    return launch_gemv(g, st);
}

int pi_predictor(const void * fc1, const void * fc2, int64_t d, int64_t rank, int64_t F,
                 const float * p_in, int T, float * idx, void * workspace, size_t workspace_bytes, void * stream) {
    int rc;
    if ((rc = check_w(PI_TYPE_F16, d, fc1)) || (rc = check_w(PI_TYPE_F16, rank, fc2))) return rc;
    PI_REQUIRE(p_in && idx && T >= 0, "predictor: bad arguments");
    if (T == 0) return PI_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (!aligned(workspace, 256) || workspace_bytes < act_bytes(PI_TYPE_F16, d, T) + act_bytes(PI_TYPE_F16, rank, T)) {
        set_error("predictor: workspace too small or misaligned"); return PI_ERR_WORKSPACE;
    }
    char * p = (char *)workspace;
    ActBuf a_in = act_carve(PI_TYPE_F16, d, T, &p);
    ActBuf a_h  = act_carve(PI_TYPE_F16, rank, T, &p);
    if ((rc = launch_convert_act(PI_TYPE_F16, p_in, d, d, T, a_in, st))) return rc;
    GemvArgs g1;                                       // hidden = relu(fc1 . p), kept only in the FP16 form fc2 consumes
    g1.W = fc1; g1.nrows = rank; g1.ncols = d; g1.x = a_in.view(); g1.T = T; g1.relu = 1; g1.dst16 = a_h.h16; g1.dst_stride = rank;
    if ((rc = launch_gemv(g1, st))) return rc;
    GemvArgs g2;
    g2.W = fc2; g2.nrows = F; g2.ncols = rank; g2.x = a_h.view(); g2.T = T; g2.dst = idx; g2.dst_stride = F;
    return launch_gemv(g2, st);
}

int pi_active_list(const float * idx, int64_t F, int T, int64_t idx_stride, float threshold,
                   int32_t * list, int32_t * count, void * workspace, size_t workspace_bytes, void * stream) {
    PI_REQUIRE(idx && list && count && F >= 0 && T >= 1 && idx_stride >= F, "active_list: bad arguments");
    cudaStream_t st = (cudaStream_t)stream;
    Scratch s(workspace, workspace_bytes);
    unsigned int * ticket = (unsigned int *)s.take(256);
    uint32_t * masks = (uint32_t *)s.take((size_t)((F + 31) / 32) * 4);
    if (!aligned(workspace, 256) || !ticket || !masks) { set_error("active_list: workspace too small or misaligned"); return PI_ERR_WORKSPACE; }
    PI_CUDA(cudaMemsetAsync(ticket, 0, 4, st));
    CompactArgs c;
    c.idx = idx; c.idx_stride = idx_stride; c.T = T; c.threshold = threshold; c.n_local = F;
    c.list = list; c.count = count; c.masks = masks; c.ticket = ticket;
    return launch_compact(c, st);
}

int pi_mul_mat_idx(int wtype, const void * W, int64_t n_w_rows, int64_t ncols,
                   const float * x, int T, const float * idx, int64_t idx_stride,
                   const int32_t * bucket, float threshold, float * dst, int64_t n_dst_rows,
                   void * workspace, size_t workspace_bytes, void * stream) {
    int rc = check_w(wtype, ncols, W);
    if (rc) return rc;
    PI_REQUIRE(x && idx && dst && T >= 0 && n_w_rows >= 0 && n_dst_rows >= n_w_rows && idx_stride >= n_dst_rows,
               "mul_mat_idx: bad arguments (need n_w_rows <= n_dst_rows <= idx_stride)");
    PI_REQUIRE(bucket || n_w_rows == n_dst_rows, "mul_mat_idx: without a bucket W must hold every destination row");
    if (T == 0 || n_dst_rows == 0) return PI_OK;
    cudaStream_t st = (cudaStream_t)stream;
    Scratch s(workspace, workspace_bytes);
    SparseScratch ss;
    const bool carved = carve_sparse(s, n_w_rows, ss);
    char * actp = (char *)s.take(act_bytes(wtype, ncols, T));
    if (!aligned(workspace, 256) || !actp || !carved) { set_error("mul_mat_idx: workspace too small or misaligned"); return PI_ERR_WORKSPACE; }
    ActBuf act = act_carve(wtype, ncols, T, &actp);
    if (bucket) PI_CUDA(cudaMemsetAsync(dst, 0, (size_t)T * n_dst_rows * 4, st));      // rows held elsewhere read 0
    PI_CUDA(cudaMemsetAsync(ss.count, 0, 12, st));                                      // count, ticket, status
    if (n_w_rows == 0) return PI_OK;
    if ((rc = launch_convert_act(wtype, x, ncols, ncols, T, act, st))) return rc;
    CompactArgs c;
    c.idx = idx; c.idx_stride = idx_stride; c.T = T; c.threshold = threshold; c.n_local = n_w_rows; c.bucket = bucket;
    c.list = ss.list; c.count = ss.count; c.masks = ss.masks; c.ticket = ss.ticket;
    c.zero_dst = dst; c.zero_stride = n_dst_rows;
    if ((rc = launch_compact(c, st))) return rc;
    GemvArgs g;
    g.wtype = wtype; g.W = W; g.nrows = n_w_rows; g.ncols = ncols; g.x = act.view(); g.T = T;
    g.list = ss.list; g.count = ss.count; g.bucket = bucket; g.idx = idx; g.idx_stride = idx_stride; g.threshold = threshold;
    g.dst = dst; g.dst_stride = n_dst_rows; g.status = ss.status;
    if (T == 1) g.masks = ss.masks;
    return launch_gemv(g, st);
}

int pi_axpy(int wtype, const void * Wt, int64_t n_w_rows, int64_t ncols,
            const float * h, int T, int64_t h_stride, const float * idx, int64_t idx_stride,
            const int32_t * bucket, float threshold, float * dst,
            void * workspace, size_t workspace_bytes, void * stream) {
    int rc = check_w(wtype, ncols, Wt);
    if (rc) return rc;
    PI_REQUIRE(h && idx && dst && T >= 0 && n_w_rows >= 0 && h_stride >= n_w_rows && idx_stride >= n_w_rows, "axpy: bad arguments");
    PI_REQUIRE(wtype != PI_TYPE_Q4_0 || h_stride % 32 == 0, "axpy: Q4_0 needs h_stride %% 32 == 0 (coefficients are quantised per 32 neurons)");
    if (T == 0) return PI_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (n_w_rows == 0) { PI_CUDA(cudaMemsetAsync(dst, 0, (size_t)T * ncols * 4, st)); return PI_OK; }
    Scratch s(workspace, workspace_bytes);
    SparseScratch ss;
    const int G = axpy_groups(wtype, ncols, T);
    bool ok = aligned(workspace, 256) && carve_sparse(s, n_w_rows, ss);
    int8_t * cq = nullptr; float * cd = nullptr;
    if (ok && wtype == PI_TYPE_Q4_0) {
        cq = (int8_t *)s.take((size_t)T * h_stride);
        cd = (float *)s.take((size_t)T * (h_stride / 32) * 4);
        ok = cq && cd;
    }
    float * partial = ok ? (float *)s.take((size_t)G * T * ncols * 4) : nullptr;
    if (!ok || !partial) { set_error("axpy: workspace too small or misaligned"); return PI_ERR_WORKSPACE; }
    PI_CUDA(cudaMemsetAsync(ss.count, 0, 12, st));                                      // count, ticket, status
    CompactArgs c;
    c.idx = idx; c.idx_stride = idx_stride; c.T = T; c.threshold = threshold; c.n_local = n_w_rows; c.bucket = bucket;
    c.list = ss.list; c.count = ss.count; c.masks = ss.masks; c.ticket = ss.ticket;
    if ((rc = launch_compact(c, st))) return rc;
    if (wtype == PI_TYPE_Q4_0 && T > 1 && (rc = launch_neuron_q8(h, h_stride, h_stride, T, cq, cd, st))) return rc;
    AxpyArgs a;
    a.wtype = wtype; a.Wt = Wt; a.nrows = n_w_rows; a.ncols = ncols; a.h = h; a.h_stride = h_stride; a.T = T;
    a.list = ss.list; a.count = ss.count; a.bucket = bucket; a.idx = idx; a.idx_stride = idx_stride; a.threshold = threshold;
    a.cq = cq; a.cd = cd; a.c_stride = h_stride; a.partial = partial; a.n_groups = G; a.status = ss.status;
    if (T == 1) a.masks = ss.masks;
    int used = G;
    if ((rc = launch_axpy(a, st, &used))) return rc;
    return launch_reduce_partials(partial, used, T, ncols, nullptr, nullptr, dst, st);
}

int pi_sparse_ffn(int wtype, const void * up, const void * gate, const void * down_t, int64_t n_w_rows, int64_t ncols,
                  const float * x, int T, const float * idx, int64_t idx_stride, const int32_t * bucket, float threshold,
                  const float * up_bias, float * dst, void * workspace, size_t workspace_bytes, void * stream) {
    int rc = check_w(wtype, ncols, up);
    if (rc) return rc;
    PI_REQUIRE(down_t && x && idx && dst && T >= 0 && n_w_rows >= 0 && idx_stride >= n_w_rows, "sparse_ffn: bad arguments");
    PI_REQUIRE(bucket || idx_stride >= n_w_rows, "sparse_ffn: idx_stride must cover every neuron id");
    PI_REQUIRE(wtype != PI_TYPE_Q4_0 || idx_stride % 32 == 0, "sparse_ffn: Q4_0 needs idx_stride %% 32 == 0 (coefficients are quantised per 32 neurons)");
    if (T == 0) return PI_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (n_w_rows == 0) { PI_CUDA(cudaMemsetAsync(dst, 0, (size_t)T * ncols * 4, st)); return PI_OK; }
    const int64_t F = idx_stride;                                  // the hidden vector is indexed by global neuron id
    Scratch s(workspace, workspace_bytes);
    SparseScratch ss;
    const int G = axpy_groups(wtype, ncols, T);
    const bool carved = carve_sparse(s, n_w_rows, ss);
    char * actp = (char *)s.take(act_bytes(wtype, ncols, T));
    bool ok = aligned(workspace, 256) && actp && carved;
    float * h = ok ? (float *)s.take((size_t)T * F * 4) : nullptr;
    int8_t * cq = nullptr; float * cd = nullptr;
    if (ok && wtype == PI_TYPE_Q4_0) {
        cq = (int8_t *)s.take((size_t)T * F);
        cd = (float *)s.take((size_t)T * (F / 32) * 4);
        ok = cq && cd;
    }
    float * partial = ok && h ? (float *)s.take((size_t)G * T * ncols * 4) : nullptr;
    if (!ok || !h || !partial) { set_error("sparse_ffn: workspace too small or misaligned"); return PI_ERR_WORKSPACE; }
    ActBuf act = act_carve(wtype, ncols, T, &actp);
    PI_CUDA(cudaMemsetAsync(ss.count, 0, 12, st));                                      // count, ticket, status
    if (bucket || T > 1 || wtype == PI_TYPE_Q4_0) PI_CUDA(cudaMemsetAsync(h, 0, (size_t)T * F * 4, st));
    if ((rc = launch_convert_act(wtype, x, ncols, ncols, T, act, st))) return rc;
    // the kernels below are chained with programmatic dependent launch: each may start while its predecessor drains
    {
        // one token, every row on this device, no bias that inactive rows would keep: masks, then the whole FFN in one launch
        FfnRowsArgs f;
        f.pdl = true;
        f.wtype = wtype; f.up = up; f.gate = gate; f.down_t = down_t; f.nrows = n_w_rows; f.ncols = ncols;
        f.x = act.view(); f.masks = ss.masks; f.bias = up_bias; f.relu = gate ? 0 : 1;
        f.h = h; f.partial = partial; f.n_groups = G;
        if (T == 1 && !bucket && !(wtype == PI_TYPE_Q4_0 && up_bias) && ffn_rows_eligible(f)) {
            CompactArgs cm;
            cm.pdl = true;
            cm.idx = idx; cm.idx_stride = idx_stride; cm.T = 1; cm.threshold = threshold; cm.n_local = n_w_rows; cm.masks = ss.masks;
            if ((rc = launch_compact(cm, st))) return rc;
            int used1 = G;
            if ((rc = launch_ffn_rows(f, st, &used1))) return rc;
            return launch_reduce_partials(partial, used1, 1, ncols, nullptr, nullptr, dst, st, true);
        }
    }
    CompactArgs c;
    c.pdl = true;
    c.idx = idx; c.idx_stride = idx_stride; c.T = T; c.threshold = threshold; c.n_local = n_w_rows; c.bucket = bucket;
    c.list = ss.list; c.count = ss.count; c.masks = ss.masks; c.ticket = ss.ticket;
    if (wtype == PI_TYPE_Q4_0) { c.zero_dst = h; c.zero_stride = F; c.fill_bias = up_bias; c.fill_relu = 1; }
    if ((rc = launch_compact(c, st))) return rc;
    GemvArgs g;
    g.pdl = true;
    g.wtype = wtype; g.W = up; g.W2 = gate; g.nrows = n_w_rows; g.ncols = ncols; g.x = act.view(); g.T = T;
    g.list = ss.list; g.count = ss.count; g.bucket = bucket; g.idx = idx; g.idx_stride = idx_stride; g.threshold = threshold;
    g.bias = up_bias; g.relu = gate ? 0 : 1;
    g.dst = h; g.dst_stride = F; g.status = ss.status;
    if (T == 1) g.masks = ss.masks;
    if ((rc = launch_gemv(g, st))) return rc;
    if (wtype == PI_TYPE_Q4_0 && T > 1 && (rc = launch_neuron_q8(h, F, F, T, cq, cd, st))) return rc;
    AxpyArgs a;
    a.pdl = !(wtype == PI_TYPE_Q4_0 && T > 1);
    a.wtype = wtype; a.Wt = down_t; a.nrows = n_w_rows; a.ncols = ncols; a.h = h; a.h_stride = F; a.T = T;
    a.list = ss.list; a.count = ss.count; a.bucket = bucket; a.idx = idx; a.idx_stride = idx_stride; a.threshold = threshold;
    a.cq = cq; a.cd = cd; a.c_stride = F; a.partial = partial; a.n_groups = G; a.status = ss.status;
    if (T == 1) a.masks = ss.masks;
    int used = G;
    if ((rc = launch_axpy(a, st, &used))) return rc;
    return launch_reduce_partials(partial, used, T, ncols, nullptr, nullptr, dst, st, T == 1);
}

int pi_op_status(const void * workspace, void * stream) {
    const void * ws = workspace;
    if (!ws) {                                                       // the built-in array of pi_axpy_static on the current device
        void * p = nullptr;
        const int rc = static_scratch_address(&p);
        if (rc) return rc;
        ws = p;
    }
    PI_REQUIRE(aligned(ws, 256), "op_status: the workspace of the call to be checked (256-byte aligned), or NULL for pi_axpy_static");
    cudaStream_t st = (cudaStream_t)stream;
    unsigned int word = 0;
    PI_CUDA(cudaMemcpyAsync(&word, (const char *)ws + 8, 4, cudaMemcpyDeviceToHost, st));
    PI_CUDA(cudaStreamSynchronize(st));
    if (word) { set_error("a bounded wait inside a kernel of the last sparse operator ran out (status bits 0x%x): its result is incomplete", word); return PI_ERR_TIMEOUT; }
    return PI_OK;
}

int pi_norm(const float * x, int T, int64_t n, int rms, float eps, const float * w, const float * b, float * y, void * stream) {
    PI_REQUIRE(x && y && T >= 0 && aligned(x, 16) && aligned(y, 16), "norm: bad arguments (pointers must be 16-byte aligned)");
    NormArgs a;
    a.x = x; a.T = T; a.n = n; a.rms = rms; a.eps = eps; a.w = w; a.b = b; a.y = y;
    return launch_norm(a, (cudaStream_t)stream);
}

int pi_rope(float * x, int T, int n_heads, int head_dim, const int32_t * pos, const float * cs, int neox, void * stream) {
    PI_REQUIRE(x && pos && cs && T >= 0 && n_heads > 0 && head_dim > 0 && head_dim % 2 == 0 && aligned(cs, 8), "rope: bad arguments");
    return launch_rope(x, T, n_heads, head_dim, pos, cs, neox, (cudaStream_t)stream);
}

void pi_rope_table_host(float * host_cs, int n_pos, int head_dim, float freq_base) {
    // ggml.c:11200 theta_scale = powf(freq_base, -2/n_dims); ggml.c:11219 / 11280 theta *= theta_scale per pair
    const float theta_scale = powf(freq_base, -2.0f / (float)head_dim);
    for (int p = 0; p < n_pos; p++) {
        float theta = (float)p;
        for (int i = 0; i < head_dim / 2; i++) {
            host_cs[((size_t)p * (head_dim / 2) + i) * 2 + 0] = cosf(theta);
            host_cs[((size_t)p * (head_dim / 2) + i) * 2 + 1] = sinf(theta);
            theta *= theta_scale;
        }
    }
}

int pi_attention_decode(const float * q, const float * k, const float * v, void * k_cache, void * v_cache,
                        const int32_t * seq, const int32_t * pos, int T, int n_head, int n_head_kv, int head_dim,
                        int n_ctx, float * out, void * stream) {
    PI_REQUIRE(q && k && v && k_cache && v_cache && pos && out && T >= 0 && n_head > 0 && n_head_kv > 0 && n_ctx > 0,
               "attention_decode: bad arguments");
    AttnArgs a;
    a.q = q; a.k = k; a.v = v; a.k_cache = (__half *)k_cache; a.v_cache = (__half *)v_cache; a.seq = seq; a.pos = pos;
    a.T = T; a.n_head = n_head; a.n_head_kv = n_head_kv; a.head_dim = head_dim; a.n_ctx = n_ctx; a.out = out;
    return launch_attention(a, (cudaStream_t)stream);
}

#pragma GCC visibility pop
}  // extern "C"
