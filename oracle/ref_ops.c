/*
 * ref_ops.c -- thin driver over the REFERENCE's own ggml (TEST INFRASTRUCTURE ONLY).
 *
 * Compiled by oracle/Makefile together with the reference's unmodified ggml.c /
 * ggml-quants.c / ggml-alloc.c / ggml-backend.c (read where they lie; nothing of the
 * reference is copied) into oracle/_ref/libpi_ref.so.  Every entry point builds a
 * one-node ggml graph through the public ggml.h API and computes it on the CPU with
 * the requested number of threads, so the numbers that come out are the reference
 * CPU path's, not a restatement.  Used to pin oracle/pi_oracle.c, to generate the
 * fixtures under tests/golden/, and as the timed CPU baseline.
 *
 * Note: the reference's CPU axpy is only correct at one thread (its per-thread partial
 * vectors are merged into dst without a lock, ggml.c:14433-14458), so parity uses
 * n_threads = 1 and only timing uses more.
 */
#include "ggml.h"

#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

static enum ggml_type map_type(int t) { return t == 2 ? GGML_TYPE_Q4_0 : (t == 1 ? GGML_TYPE_F16 : GGML_TYPE_F32); }

static struct ggml_context * new_ctx(size_t work_bytes) {
    struct ggml_init_params ip = { 16u*1024*1024 + work_bytes, NULL, true };
    return ggml_init(ip);
}

static struct ggml_tensor * wrap2(struct ggml_context * ctx, enum ggml_type t, int64_t ne0, int64_t ne1, const void * data) {
    struct ggml_tensor * x = ggml_new_tensor_2d(ctx, t, ne0, ne1);
    x->data = (void *)data;
    return x;
}

/* ggml fills its FP16 lookup tables on the first ggml_init (ggml.c:2155-2195); the row converters
 * and quantisers below read them, so make sure one context has existed. */
static void ensure_init(void) {
    static int done = 0;
    if (!done) { ggml_free(new_ctx(0)); done = 1; }
}

static double now_s(void) {
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return ts.tv_sec + 1e-9*ts.tv_nsec;
}

/* compute `out` reps times; returns the best wall time of one graph compute in seconds */
static double run(struct ggml_context * ctx, struct ggml_tensor * out, int n_threads, int reps) {
    struct ggml_cgraph * gf = ggml_new_graph(ctx);
    ggml_build_forward_expand(gf, out);
    struct ggml_cplan plan = ggml_graph_plan(gf, n_threads);
    void * work = plan.work_size ? malloc(plan.work_size) : NULL;
    plan.work_data = work;
    double best = 1e30;
    for (int i = 0; i < (reps > 0 ? reps : 1); i++) {
        const double t0 = now_s();
        ggml_graph_compute(gf, &plan);
        const double dt = now_s() - t0;
        if (dt < best) best = dt;
    }
    free(work);
    return best;
}

void ref_fp32_to_fp16_row(const float * x, uint16_t * y, int64_t n) { ensure_init(); ggml_fp32_to_fp16_row(x, y, (int)n); }
void ref_fp16_to_fp32_row(const uint16_t * x, float * y, int64_t n) { ensure_init(); ggml_fp16_to_fp32_row(x, y, (int)n); }

/* the quantiser the reference uses to create model files, and the one its CPU path applies to activations */
void ref_quantize_q4_0(const float * x, void * y, int64_t k) {
    ensure_init();
    ggml_type_traits_t tt = ggml_internal_get_type_traits(GGML_TYPE_Q4_0);
    tt.from_float_reference(x, y, (int)k);
}
void ref_quantize_q8_0(const float * x, void * y, int64_t k) {
    ensure_init();
    ggml_type_traits_t tt = ggml_internal_get_type_traits(GGML_TYPE_Q8_0);
    tt.from_float(x, y, (int)k);
}
void ref_dequantize_q4_0(const void * x, float * y, int64_t k) {
    ensure_init();
    ggml_type_traits_t tt = ggml_internal_get_type_traits(GGML_TYPE_Q4_0);
    tt.to_float(x, y, (int)k);
}

double ref_mul_mat(int type, const void * W, int64_t nrows, int64_t ncols, const float * x, int64_t T,
                   float * dst, int n_threads, int reps) {
    struct ggml_context * ctx = new_ctx(0);
    struct ggml_tensor * a = wrap2(ctx, map_type(type), ncols, nrows, W);
    struct ggml_tensor * b = wrap2(ctx, GGML_TYPE_F32, ncols, T, x);
    struct ggml_tensor * o = ggml_mul_mat(ctx, a, b);
    o->data = dst;
    const double t = run(ctx, o, n_threads, reps);
    ggml_free(ctx);
    return t;
}

double ref_mul_mat_idx(int type, const void * W, int64_t nrows, int64_t ncols, const float * x, int64_t T,
                       const float * idx, const int32_t * gpu_idx, float threshold, float * dst,
                       int n_threads, int reps) {
    struct ggml_context * ctx = new_ctx(0);
    sparse_pred_threshold = threshold;
    struct ggml_tensor * a = wrap2(ctx, map_type(type), ncols, nrows, W);
    struct ggml_tensor * b = wrap2(ctx, GGML_TYPE_F32, ncols, T, x);
    struct ggml_tensor * p = wrap2(ctx, GGML_TYPE_F32, nrows, T, idx);
    struct ggml_tensor * g = ggml_new_tensor_1d(ctx, GGML_TYPE_I32, nrows);
    g->data = (void *)gpu_idx;
    struct ggml_tensor * o = ggml_mul_mat_idx(ctx, a, b, p, g);
    o->data = dst;
    const double t = run(ctx, o, n_threads, reps);
    ggml_free(ctx);
    return t;
}

double ref_axpy(int type, const void * Wt, int64_t nrows, int64_t ncols, const float * h, int64_t T,
                const float * idx, const int32_t * gpu_idx, float threshold, float * dst,
                int n_threads, int reps) {
    struct ggml_context * ctx = new_ctx(0);
    sparse_pred_threshold = threshold;
    struct ggml_tensor * a = wrap2(ctx, map_type(type), ncols, nrows, Wt);
    struct ggml_tensor * b = wrap2(ctx, GGML_TYPE_F32, nrows, T, h);
    struct ggml_tensor * p = wrap2(ctx, GGML_TYPE_F32, nrows, T, idx);
    struct ggml_tensor * g = ggml_new_tensor_1d(ctx, GGML_TYPE_I32, nrows);
    g->data = (void *)gpu_idx;
    struct ggml_tensor * o = ggml_axpy(ctx, a, b, p, g);
    o->data = dst;
    const double t = run(ctx, o, n_threads, reps);
    ggml_free(ctx);
    return t;
}

void ref_rms_norm(const float * x, int64_t n, int64_t rows, float eps, float * y) {
    struct ggml_context * ctx = new_ctx(0);
    struct ggml_tensor * a = wrap2(ctx, GGML_TYPE_F32, n, rows, x);
    struct ggml_tensor * o = ggml_rms_norm(ctx, a, eps);
    o->data = y;
    run(ctx, o, 1, 1);
    ggml_free(ctx);
}

void ref_norm(const float * x, int64_t n, int64_t rows, float eps, float * y) {
    struct ggml_context * ctx = new_ctx(0);
    struct ggml_tensor * a = wrap2(ctx, GGML_TYPE_F32, n, rows, x);
    struct ggml_tensor * o = ggml_norm(ctx, a, eps);
    o->data = y;
    run(ctx, o, 1, 1);
    ggml_free(ctx);
}

void ref_soft_max(const float * x, int64_t n, int64_t rows, float * y) {
    struct ggml_context * ctx = new_ctx(0);
    struct ggml_tensor * a = wrap2(ctx, GGML_TYPE_F32, n, rows, x);
    struct ggml_tensor * o = ggml_soft_max(ctx, a);
    o->data = y;
    run(ctx, o, 1, 1);
    ggml_free(ctx);
}

/* x: [n_heads][head_dim] of one token at position pos; mode 0 (llama) or 2 (neox) */
void ref_rope(const float * x, int64_t head_dim, int64_t n_heads, int32_t pos, float freq_base, int mode, float * y) {
    struct ggml_context * ctx = new_ctx(0);
    struct ggml_tensor * a = ggml_new_tensor_3d(ctx, GGML_TYPE_F32, head_dim, n_heads, 1);
    a->data = (void *)x;
    struct ggml_tensor * p = ggml_new_tensor_1d(ctx, GGML_TYPE_I32, 1);
    p->data = &pos;
    struct ggml_tensor * o = ggml_rope_custom(ctx, a, p, (int)head_dim, mode, 0, 0, freq_base, 1.0f, 0.0f, 1.0f, 32.0f, 1.0f);
    o->data = y;
    run(ctx, o, 1, 1);
    ggml_free(ctx);
}
