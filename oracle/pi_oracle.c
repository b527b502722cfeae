/*
 * pi_oracle.c -- CPU restatement of PowerInfer's decode hot path.
 * TEST INFRASTRUCTURE ONLY: the checker for the CUDA path, never part of it.
 * See pi_oracle.h for the parity status.  Citations are file:line in the
 * reference tree.  Build with -O2 -mfma -mf16c-free plain C: all rounding is
 * explicit (fmaf / separate mul+add) so the result does not depend on the
 * compiler's contraction choices; compile with -ffp-contract=off.
 */
#include "pi_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------ fp16 */

float pio_fp16_to_fp32(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    const uint32_t exp  = (h >> 10) & 0x1Fu;
    const uint32_t man  = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {                                   /* subnormal: normalise */
            int e = -1;
            uint32_t m = man;
            do { m <<= 1; e++; } while ((m & 0x400u) == 0);
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((m & 0x3FFu) << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, sizeof f);
    return f;
}

/* round-to-nearest-even, as _cvtss_sh(x, 0) does (ggml.c GGML_COMPUTE_FP32_TO_FP16 with F16C) */
uint16_t pio_fp32_to_fp16(float f) {
    uint32_t x;
    memcpy(&x, &f, sizeof x);
    const uint32_t sign = (x >> 16) & 0x8000u;
    const uint32_t absx = x & 0x7FFFFFFFu;
    if (absx >= 0x7F800000u) {                     /* inf / nan */
        return (uint16_t)(sign | 0x7C00u | (absx > 0x7F800000u ? 0x200u | ((absx >> 13) & 0x3FFu) : 0));
    }
    if (absx >= 0x477FF000u) {                     /* >= 65520 rounds to inf */
        return (uint16_t)(sign | 0x7C00u);
    }
    if (absx < 0x33000001u) {                      /* <= 2^-25 rounds to zero */
        return (uint16_t)sign;
    }
    int32_t e = (int32_t)(absx >> 23) - 127;
    uint32_t m = (absx & 0x7FFFFFu) | 0x800000u;   /* 24-bit significand */
    uint32_t shift, half;
    uint32_t out;
    if (e < -14) {                                 /* subnormal half */
        shift = (uint32_t)(13 + (-14 - e));
        out = m >> shift;
        const uint32_t rem = m & ((1u << shift) - 1u);
        half = 1u << (shift - 1);
        if (rem > half || (rem == half && (out & 1u))) out++;
        return (uint16_t)(sign | out);
    }
    out = ((uint32_t)(e + 15) << 10) | ((m >> 13) & 0x3FFu);
    const uint32_t rem = m & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (out & 1u))) out++;   /* carry may bump the exponent: correct */
    return (uint16_t)(sign | out);
}

void pio_fp32_to_fp16_row(const float * x, uint16_t * y, int64_t n) {
    for (int64_t i = 0; i < n; i++) y[i] = pio_fp32_to_fp16(x[i]);
}
void pio_fp16_to_fp32_row(const uint16_t * x, float * y, int64_t n) {
    for (int64_t i = 0; i < n; i++) y[i] = pio_fp16_to_fp32(x[i]);
}

/* --------------------------------------------------------- block formats */

size_t pio_row_bytes(int type, int64_t n) {
    return type == PIO_Q4_0 ? (size_t)(n / PIO_QK) * sizeof(pio_block_q4_0) : (size_t)n * 2;
}

/* ggml-quants.c:428-463: d = (signed value of largest magnitude) / -8, q = min(15, (int8)(x/d + 8.5)) */
void pio_quantize_row_q4_0(const float * x, pio_block_q4_0 * y, int64_t k) {
    const int64_t nb = k / PIO_QK;
    for (int64_t i = 0; i < nb; i++) {
        float amax = 0.0f, max = 0.0f;
        for (int j = 0; j < PIO_QK; j++) {
            const float v = x[i*PIO_QK + j];
            if (amax < fabsf(v)) { amax = fabsf(v); max = v; }
        }
        const float d  = max / -8;
        const float id = d ? 1.0f/d : 0.0f;
        y[i].d = pio_fp32_to_fp16(d);
        for (int j = 0; j < PIO_QK/2; j++) {
            const float x0 = x[i*PIO_QK + j]*id;
            const float x1 = x[i*PIO_QK + PIO_QK/2 + j]*id;
            int q0 = (int8_t)(x0 + 8.5f); if (q0 > 15) q0 = 15;
            int q1 = (int8_t)(x1 + 8.5f); if (q1 > 15) q1 = 15;
            y[i].qs[j] = (uint8_t)((uint8_t)q0 | ((uint8_t)q1 << 4));
        }
    }
}

/* ggml-quants.c:1074-1092 */
void pio_dequantize_row_q4_0(const pio_block_q4_0 * x, float * y, int64_t k) {
    const int64_t nb = k / PIO_QK;
    for (int64_t i = 0; i < nb; i++) {
        const float d = pio_fp16_to_fp32(x[i].d);
        for (int j = 0; j < PIO_QK/2; j++) {
            y[i*PIO_QK + j]            = (float)((x[i].qs[j] & 0x0F) - 8) * d;
            y[i*PIO_QK + j + PIO_QK/2] = (float)((x[i].qs[j] >> 4)   - 8) * d;
        }
    }
}

/* The activation quantiser the CPU path really runs on x86 is the AVX2 branch of
 * quantize_row_q8_0 (ggml-quants.c:702-760), not the _reference one: d = amax/127,
 * id = 127/amax (NOT 1/d), round-to-nearest-EVEN. */
void pio_quantize_row_q8_0(const float * x, pio_block_q8_0 * y, int64_t k) {
    const int64_t nb = k / PIO_QK;
    for (int64_t i = 0; i < nb; i++) {
        float amax = 0.0f;
        for (int j = 0; j < PIO_QK; j++) {
            const float a = fabsf(x[i*PIO_QK + j]);
            if (a > amax) amax = a;
        }
        const float d  = amax / 127.f;
        const float id = (amax != 0.0f) ? 127.f / amax : 0.0f;
        y[i].d = pio_fp32_to_fp16(d);
        for (int j = 0; j < PIO_QK; j++) {
            y[i].qs[j] = (int8_t)nearbyintf(x[i*PIO_QK + j] * id);   /* default rounding mode = nearest even */
        }
    }
}

/* ------------------------------------------------------------ dot kernels */

/* ggml.c:1188-1221 with the AVX macros of ggml.c:745-841: four 8-lane FMA accumulators
 * over 32-element steps, reduced (0+2),(1+3),(0+1), then lanes (l + l+4), hadd, hadd. */
float pio_vec_dot_f16(int64_t n, const uint16_t * x, const uint16_t * y) {
    float sum[4][8];
    memset(sum, 0, sizeof sum);
    const int64_t np = n & ~(int64_t)31;
    for (int64_t i = 0; i < np; i += 32) {
        for (int j = 0; j < 4; j++) {
            for (int l = 0; l < 8; l++) {
                const int64_t k = i + j*8 + l;
                sum[j][l] = fmaf(pio_fp16_to_fp32(x[k]), pio_fp16_to_fp32(y[k]), sum[j][l]);
            }
        }
    }
    float t0[4];
    for (int l = 0; l < 8; l++) { sum[0][l] = sum[0][l] + sum[2][l]; sum[1][l] = sum[1][l] + sum[3][l]; }
    for (int l = 0; l < 8; l++) { sum[0][l] = sum[0][l] + sum[1][l]; }
    for (int l = 0; l < 4; l++) t0[l] = sum[0][l] + sum[0][l+4];
    const float res = (t0[0] + t0[1]) + (t0[2] + t0[3]);
    double sumf = res;
    for (int64_t i = np; i < n; i++) {
        sumf += (double)(pio_fp16_to_fp32(x[i]) * pio_fp16_to_fp32(y[i]));
    }
    return (float)sumf;
}

/* ggml-quants.c:2586-2610 (AVX2): lane l of an 8-lane accumulator takes the integer sum of
 * products 4l..4l+3 of each block, acc = fma(d4*d8, q, acc); hsum_float_8 (ggml-quants.c:66-72). */
float pio_vec_dot_q4_0_q8_0(int64_t n, const pio_block_q4_0 * x, const pio_block_q8_0 * y) {
    float acc[8] = {0};
    const int64_t nb = n / PIO_QK;
    for (int64_t i = 0; i < nb; i++) {
        const float d = pio_fp16_to_fp32(x[i].d) * pio_fp16_to_fp32(y[i].d);
        for (int l = 0; l < 8; l++) {
            int s = 0;
            for (int k = 0; k < 4; k++) {
                const int j = 4*l + k;
                const int v = j < 16 ? (x[i].qs[j] & 0x0F) - 8 : (x[i].qs[j-16] >> 4) - 8;
                s += v * (int)y[i].qs[j];
            }
            acc[l] = fmaf(d, (float)s, acc[l]);
        }
    }
    float r[4];
    for (int l = 0; l < 4; l++) r[l] = acc[l+4] + acc[l];
    const float a = r[0] + r[2];
    const float b = r[1] + r[3];
    return a + b;
}

/* --------------------------------------------------------------- mat-vec */

static void * xmalloc(size_t n) {
    void * p = malloc(n ? n : 1);
    if (!p) abort();
    return p;
}

/* Convert one activation row to the weight type's vec_dot_type (ggml.c:9703-9716): F16 or Q8_0. */
static void * to_vec_dot_type(int type, const float * x, int64_t n) {
    if (type == PIO_Q4_0) {
        pio_block_q8_0 * q = xmalloc((size_t)(n / PIO_QK) * sizeof *q);
        pio_quantize_row_q8_0(x, q, n);
        return q;
    }
    uint16_t * h = xmalloc((size_t)n * 2);
    pio_fp32_to_fp16_row(x, h, n);
    return h;
}

static float row_dot(int type, const void * W, int64_t r, int64_t ncols, const void * xv) {
    const char * row = (const char *)W + (size_t)r * pio_row_bytes(type, ncols);
    return type == PIO_Q4_0 ? pio_vec_dot_q4_0_q8_0(ncols, (const pio_block_q4_0 *)row, xv)
                            : pio_vec_dot_f16(ncols, (const uint16_t *)row, xv);
}

void pio_mul_mat(int type, const void * W, int64_t nrows, int64_t ncols,
                 const float * x, int64_t T, float * dst) {
    for (int64_t t = 0; t < T; t++) {
        void * xv = to_vec_dot_type(type, x + t*ncols, ncols);
        for (int64_t r = 0; r < nrows; r++) dst[t*nrows + r] = row_dot(type, W, r, ncols, xv);
        free(xv);
    }
}

/* ggml.c:14030-14282; predicate at ggml.c:14256 */
void pio_mul_mat_idx(int type, const void * W, int64_t nrows, int64_t ncols,
                     const float * x, int64_t T, const float * idx, int64_t idx_stride,
                     const int32_t * gpu_idx, float threshold, float * dst) {
    for (int64_t t = 0; t < T; t++) {
        void * xv = to_vec_dot_type(type, x + t*ncols, ncols);
        const float * pred = idx + t*idx_stride;
        for (int64_t r = 0; r < nrows; r++) {
            if ((gpu_idx && gpu_idx[r] == 1) || pred[r] < threshold) { dst[t*nrows + r] = 0.0f; continue; }
            dst[t*nrows + r] = row_dot(type, W, r, ncols, xv);
        }
        free(xv);
    }
}

/* F16: ggml.c:14314-14463 with ggml_axpy_avx_f16 (ggml.c:14292-14312): h rounded to FP16, rows whose
 * FP16 coefficient has bit pattern 0 skipped, acc = fma(w, alpha, acc) per element, rows in order.
 * Q4_0: ggml.c:14465-14618 with ggml_axpy_q4_0_q8_0 (ggml-quants.c:2426-2509): h quantised to Q8_0
 * over 32-NEURON blocks, rows with int8 coefficient 0 skipped, acc += (float)((q-8)*b) * (d4*d8). */
void pio_axpy(int type, const void * Wt, int64_t nrows, int64_t ncols,
              const float * h, int64_t T, const float * idx, int64_t idx_stride,
              const int32_t * gpu_idx, float threshold, float * dst) {
    const size_t rb = pio_row_bytes(type, ncols);
    float * acc = xmalloc((size_t)ncols * sizeof *acc);
    for (int64_t t = 0; t < T; t++) {
        const float * pred = idx + t*idx_stride;
        memset(acc, 0, (size_t)ncols * sizeof *acc);
        void * hv = to_vec_dot_type(type, h + t*nrows, nrows);
        for (int64_t r = 0; r < nrows; r++) {
            const char * row = (const char *)Wt + (size_t)r * rb;
            if (type == PIO_F16) {
                const uint16_t a16 = ((const uint16_t *)hv)[r];
                if (a16 == 0) continue;
                if (gpu_idx && gpu_idx[r] == 1) continue;
                if (pred[r] < threshold) continue;
                const float alpha = pio_fp16_to_fp32(a16);
                const uint16_t * w = (const uint16_t *)row;
                for (int64_t c = 0; c < ncols; c++) acc[c] = fmaf(pio_fp16_to_fp32(w[c]), alpha, acc[c]);
            } else {
                if (gpu_idx && gpu_idx[r] == 1) continue;
                if (pred[r] < threshold) continue;
                const pio_block_q8_0 * hq = (const pio_block_q8_0 *)hv;
                const int b = hq[r / PIO_QK].qs[r % PIO_QK];
                if (b == 0) continue;
                const float d8 = pio_fp16_to_fp32(hq[r / PIO_QK].d);
                const pio_block_q4_0 * w = (const pio_block_q4_0 *)row;
                for (int64_t i = 0; i < ncols / PIO_QK; i++) {
                    const float sc = pio_fp16_to_fp32(w[i].d) * d8;
                    for (int j = 0; j < 16; j++) {
                        const int v0 = (w[i].qs[j] & 0x0F) - 8;
                        const int v1 = (w[i].qs[j] >> 4)   - 8;
                        const float p0 = (float)(v0 * b) * sc;
                        const float p1 = (float)(v1 * b) * sc;
                        acc[i*PIO_QK + j]      = acc[i*PIO_QK + j]      + p0;
                        acc[i*PIO_QK + j + 16] = acc[i*PIO_QK + j + 16] + p1;
                    }
                }
            }
        }
        free(hv);
        /* dst was zeroed in INIT, then the thread's private vector is added (ggml.c:14433-14458) */
        for (int64_t c = 0; c < ncols; c++) dst[t*ncols + c] = 0.0f + acc[c];
    }
    free(acc);
}

/* ------------------------------------------------------------ small nodes */

/* ggml.c:9238-9284: double accumulation of float squares, scale = 1/sqrtf(mean + eps) */
void pio_rms_norm(const float * x, int64_t n, float eps, float * y) {
    double sum = 0.0;
    for (int64_t i = 0; i < n; i++) sum += (double)(x[i] * x[i]);
    const float mean  = (float)(sum / (double)n);
    const float scale = 1.0f / sqrtf(mean + eps);
    for (int64_t i = 0; i < n; i++) y[i] = x[i] * scale;
}

/* ggml.c:9169-9218 */
void pio_norm(const float * x, int64_t n, float eps, float * y) {
    double sum = 0.0;
    for (int64_t i = 0; i < n; i++) sum += (double)x[i];
    const float mean = (float)(sum / (double)n);
    double sum2 = 0.0;
    for (int64_t i = 0; i < n; i++) {
        const float v = x[i] - mean;
        y[i] = v;
        sum2 += (double)(v * v);
    }
    const float variance = (float)(sum2 / (double)n);
    const float scale = 1.0f / sqrtf(variance + eps);
    for (int64_t i = 0; i < n; i++) y[i] = y[i] * scale;
}

/* ggml.c:11163-11325 with n_dims == head_dim, freq_scale 1, ext_factor 0, attn_factor 1, no xPos.
 * theta advances by repeated multiplication (ggml.c:11219 / 11280).  The reference is built with
 * FMA contraction enabled, so a*b - c*d compiles to fma(a, b, -(c*d)); stated explicitly here. */
void pio_rope(float * x, int64_t head_dim, int64_t n_heads, int32_t pos, float freq_base, int neox) {
    const float theta_scale = powf(freq_base, -2.0f / (float)head_dim);
    for (int64_t h = 0; h < n_heads; h++) {
        float * v = x + h*head_dim;
        float theta = (float)pos;
        for (int64_t i0 = 0; i0 < head_dim; i0 += 2) {
            const float c = cosf(theta), s = sinf(theta);
            theta *= theta_scale;
            float * p0, * p1;
            if (neox) { p0 = v + i0/2; p1 = v + i0/2 + head_dim/2; }
            else      { p0 = v + i0;   p1 = v + i0 + 1; }
            const float x0 = *p0, x1 = *p1;
            *p0 = x0*c - x1*s;
            *p1 = x0*s + x1*c;
        }
    }
}

/* ggml.c:10708-10777: exp through an FP16 table on an FP16-rounded argument, double sum */
void pio_soft_max(const float * x, int64_t n, float * y) {
    float max = -INFINITY;
    for (int64_t i = 0; i < n; i++) if (x[i] > max) max = x[i];
    double sum = 0.0;
    for (int64_t i = 0; i < n; i++) {
        if (x[i] == -INFINITY) { y[i] = 0.0f; continue; }
        const uint16_t s = pio_fp32_to_fp16(x[i] - max);
        const float val = pio_fp16_to_fp32(pio_fp32_to_fp16(expf(pio_fp16_to_fp32(s))));  /* ggml.c:2160-2166 table entry */
        sum += (double)val;
        y[i] = val;
    }
    const float inv = (float)(1.0 / sum);
    for (int64_t i = 0; i < n; i++) y[i] = y[i] * inv;
}

/* ------------------------------------------------------------ decode graph */

struct pio_ctx {
    const pio_model * m;
    uint16_t * k_cache;   /* [n_layer][n_ctx][d_kv]      RoPE'd K, FP16 (llama.cpp:4411-4413) */
    uint16_t * v_cache;   /* [n_layer][d_kv][n_ctx]      V transposed, FP16 */
    float * x, * cur, * attn_norm, * q, * k, * v, * att, * kq, * attn_out, * ffn_inp, * pred_h, * pred,
          * up, * gate, * hbuf, * ffn_out, * tmp;
};

static int64_t d_kv(const pio_model * m) { return (int64_t)m->d / m->n_head * m->n_head_kv; }

pio_ctx * pio_ctx_new(const pio_model * m) {
    pio_ctx * c = xmalloc(sizeof *c);
    memset(c, 0, sizeof *c);
    c->m = m;
    const int64_t dkv = d_kv(m);
    const size_t kvn = (size_t)m->n_layer * m->n_ctx * dkv;
    c->k_cache = calloc(kvn, 2);
    c->v_cache = calloc(kvn, 2);
    const size_t d = (size_t)m->d, F = (size_t)m->n_ff;
    c->x = xmalloc(d*4); c->cur = xmalloc(d*4); c->attn_norm = xmalloc(d*4);
    c->q = xmalloc((d + 2*dkv)*4); c->k = xmalloc(dkv*4); c->v = xmalloc(dkv*4);
    c->att = xmalloc(d*4); c->kq = xmalloc((size_t)m->n_ctx*4); c->attn_out = xmalloc(d*4);
    c->ffn_inp = xmalloc(d*4); c->pred_h = xmalloc((size_t)m->rank*4); c->pred = xmalloc(F*4);
    c->up = xmalloc(F*4); c->gate = xmalloc(F*4); c->hbuf = xmalloc(F*4); c->ffn_out = xmalloc(d*4);
    c->tmp = xmalloc(d*4);
    return c;
}

void pio_ctx_free(pio_ctx * c) {
    if (!c) return;
    free(c->k_cache); free(c->v_cache);
    free(c->x); free(c->cur); free(c->attn_norm); free(c->q); free(c->k); free(c->v); free(c->att); free(c->kq);
    free(c->attn_out); free(c->ffn_inp); free(c->pred_h); free(c->pred); free(c->up); free(c->gate);
    free(c->hbuf); free(c->ffn_out); free(c->tmp);
    free(c);
}

/* llm_build_norm (llama.cpp:4420-4450): norm, then * weight, then + bias */
static void build_norm(const pio_model * m, const float * x, const float * w, const float * b, float * y) {
    if (m->arch == PIO_ARCH_LLAMA) pio_rms_norm(x, m->d, m->norm_eps, y);
    else                           pio_norm(x, m->d, m->norm_eps, y);
    if (w) for (int i = 0; i < m->d; i++) y[i] = y[i] * w[i];
    if (b) for (int i = 0; i < m->d; i++) y[i] = y[i] + b[i];
}

/* llm_build_kv_store + llm_build_kqv (llama.cpp:4383-4418, 4764-4850) for one token */
static void attention(pio_ctx * c, int il, int32_t pos, const float * q, const float * k, const float * v, float * out) {
    const pio_model * m = c->m;
    const int64_t hd = m->d / m->n_head, dkv = d_kv(m), n_ctx = m->n_ctx;
    const int64_t group = m->n_head / m->n_head_kv;
    uint16_t * kc = c->k_cache + (size_t)il * n_ctx * dkv;
    uint16_t * vc = c->v_cache + (size_t)il * n_ctx * dkv;
    for (int64_t e = 0; e < dkv; e++) {
        kc[(size_t)pos*dkv + e]   = pio_fp32_to_fp16(k[e]);
        vc[(size_t)e*n_ctx + pos] = pio_fp32_to_fp16(v[e]);
    }
    const int64_t n_kv = pos + 1 > 32 ? pos + 1 : 32;               /* llama.cpp:6842 */
    const float scale = 1.0f / sqrtf((float)hd);                     /* llama.cpp:6500 */
    uint16_t * q16 = xmalloc((size_t)hd * 2);
    uint16_t * p16 = xmalloc((size_t)n_kv * 2);
    float * p = xmalloc((size_t)n_kv * 4);
    for (int64_t h = 0; h < m->n_head; h++) {
        const int64_t hk = h / group;
        pio_fp32_to_fp16_row(q + h*hd, q16, hd);
        for (int64_t j = 0; j < n_kv; j++) {
            float s = pio_vec_dot_f16(hd, kc + (size_t)j*dkv + hk*hd, q16);
            s = s * scale;
            c->kq[j] = j <= pos ? s + 0.0f : s + -INFINITY;
        }
        pio_soft_max(c->kq, n_kv, p);
        pio_fp32_to_fp16_row(p, p16, n_kv);
        for (int64_t e = 0; e < hd; e++) {
            out[h*hd + e] = pio_vec_dot_f16(n_kv, vc + (size_t)(hk*hd + e)*n_ctx, p16);
        }
    }
    free(q16); free(p16); free(p);
}

static void add_bias(float * y, const float * b, int64_t n) {
    if (b) for (int64_t i = 0; i < n; i++) y[i] = y[i] + b[i];
}

/* llm_build_ffn_sparse (llama.cpp:4652-4757) with gpu_idx all zero (the --vram-budget 0 path).
 * idx_imposed (tests only, not something the reference does): when not NULL, the sparse operators take THESE predictor
 * logits instead of the ones computed here; c->pred still receives the logits computed here.  It lets a test compare two
 * implementations under identical active sets, without the cascade one borderline neuron starts in the layers after it. */
static void ffn_sparse(pio_ctx * c, const pio_layer * L, const float * ffn_input, const float * pred_input, float * out,
                       const float * idx_imposed) {
    const pio_model * m = c->m;
    const int64_t F = m->n_ff, d = m->d;
    pio_mul_mat(PIO_F16, L->fc1, m->rank, d, pred_input, 1, c->pred_h);
    for (int i = 0; i < m->rank; i++) c->pred_h[i] = c->pred_h[i] > 0.0f ? c->pred_h[i] : 0.0f;
    pio_mul_mat(PIO_F16, L->fc2, F, m->rank, c->pred_h, 1, c->pred);
    const float * idx = idx_imposed ? idx_imposed : c->pred;
    pio_mul_mat_idx(m->wtype, L->up, F, d, ffn_input, 1, idx, F, NULL, m->threshold, c->up);
    add_bias(c->up, L->up_b, F);
    if (L->gate) {
        pio_mul_mat_idx(m->wtype, L->gate, F, d, ffn_input, 1, idx, F, NULL, m->threshold, c->gate);
        for (int64_t i = 0; i < F; i++) {                                     /* llama.cpp:4725-4738: LLM_FFN_PAR | LLM_FFN_SYM */
            const float u = m->gate_sym ? (c->up[i] > 0.0f ? c->up[i] : 0.0f) : c->up[i];
            c->hbuf[i] = (c->gate[i] > 0.0f ? c->gate[i] : 0.0f) * u;
        }
    } else {
        for (int64_t i = 0; i < F; i++) c->hbuf[i] = c->up[i] > 0.0f ? c->up[i] : 0.0f;
    }
    static const int32_t * zeros = NULL; (void)zeros;
    /* the CPU F16 axpy skips every row when src[3] is NULL (ggml.c:14424); the graph always passes the
     * all-zero gpu_idx, which selects "row lives on the CPU" for every neuron */
    int32_t * gi = calloc((size_t)F, sizeof *gi);
    pio_axpy(m->wtype, L->down_t, F, d, c->hbuf, 1, idx, F, gi, m->threshold, out);
    free(gi);
    add_bias(out, L->down_b, d);
}

void pio_decode(pio_ctx * c, int32_t token, int32_t pos, float * logits, float * pred_out) {
    pio_decode_imposed(c, token, pos, logits, pred_out, NULL);
}

/* pio_decode with the predictor logits of every layer imposed from outside (float [n_layer, n_ff]); see ffn_sparse */
void pio_decode_imposed(pio_ctx * c, int32_t token, int32_t pos, float * logits, float * pred_out, const float * idx_imposed) {
    const pio_model * m = c->m;
    const int64_t d = m->d, dkv = d_kv(m), hd = d / m->n_head;
    pio_fp16_to_fp32_row(m->tok_embd + (size_t)token * d, c->x, d);          /* ggml_get_rows */
    if (m->arch == PIO_ARCH_OPT) {                                           /* llama.cpp:5105-5108, 6486-6488 */
        pio_fp16_to_fp32_row(m->pos_embd + (size_t)(pos + 2) * d, c->tmp, d);
        for (int64_t i = 0; i < d; i++) c->x[i] = c->x[i] + c->tmp[i];
    }
    for (int il = 0; il < m->n_layer; il++) {
        const pio_layer * L = &m->layers[il];
        float * inpL = c->x;
        build_norm(m, inpL, L->attn_norm_w, L->attn_norm_b, c->attn_norm);
        const float * qkv_in = c->attn_norm;
        if (m->arch == PIO_ARCH_FALCON && L->attn_norm2_w) {
            build_norm(m, inpL, L->attn_norm2_w, L->attn_norm2_b, c->cur);
            qkv_in = c->cur;
        }
        float * q = c->q, * k = c->k, * v = c->v;
        if (m->arch == PIO_ARCH_FALCON) {
            pio_mul_mat(m->wtype, L->wq, d + 2*dkv, d, qkv_in, 1, c->q);     /* fused wqkv: Q heads, K heads, V heads */
            k = c->q + d; v = c->q + d + dkv;
        } else {
            pio_mul_mat(m->wtype, L->wq, d,   d, qkv_in, 1, q); add_bias(q, L->bq, d);
            pio_mul_mat(m->wtype, L->wk, dkv, d, qkv_in, 1, k); add_bias(k, L->bk, dkv);
            pio_mul_mat(m->wtype, L->wv, dkv, d, qkv_in, 1, v); add_bias(v, L->bv, dkv);
        }
        if (m->arch != PIO_ARCH_OPT) {
            pio_rope(q, hd, m->n_head,    pos, m->rope_base, m->arch == PIO_ARCH_FALCON);
            pio_rope(k, hd, m->n_head_kv, pos, m->rope_base, m->arch == PIO_ARCH_FALCON);
        }
        attention(c, il, pos, q, k, v, c->att);
        pio_mul_mat(m->wtype, L->wo, d, d, c->att, 1, c->attn_out);
        add_bias(c->attn_out, L->bo, d);

        float * pred_dst = pred_out ? pred_out + (size_t)il * m->n_ff : NULL;
        if (m->arch == PIO_ARCH_FALCON) {
            /* parallel block: FFN reads attn_norm, predictor reads the layer input (llama.cpp:5422-5428) */
            ffn_sparse(c, L, c->attn_norm, inpL, c->ffn_out, idx_imposed ? idx_imposed + (size_t)il * m->n_ff : NULL);
            for (int64_t i = 0; i < d; i++) c->x[i] = (c->ffn_out[i] + c->attn_out[i]) + inpL[i];
        } else {
            for (int64_t i = 0; i < d; i++) c->ffn_inp[i] = c->attn_out[i] + inpL[i];
            build_norm(m, c->ffn_inp, L->ffn_norm_w, L->ffn_norm_b, c->cur);
            ffn_sparse(c, L, c->cur, c->ffn_inp, c->ffn_out, idx_imposed ? idx_imposed + (size_t)il * m->n_ff : NULL);
            for (int64_t i = 0; i < d; i++) c->x[i] = c->ffn_out[i] + c->ffn_inp[i];
        }
        if (pred_dst) memcpy(pred_dst, c->pred, (size_t)m->n_ff * 4);
    }
    build_norm(m, c->x, m->out_norm_w, m->out_norm_b, c->cur);
    if (m->output) pio_mul_mat(m->wtype, m->output, m->n_vocab, d, c->cur, 1, logits);
    else           pio_mul_mat(PIO_F16, m->tok_embd, m->n_vocab, d, c->cur, 1, logits);
}
