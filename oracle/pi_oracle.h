/*
 * pi_oracle.h -- CPU restatement of PowerInfer's decode hot path (TEST INFRASTRUCTURE ONLY).
 *
 * This is the checker, never the product: only tests, the smoke check and the
 * CPU-baseline leg of the benchmark may load it.  Every function restates, in
 * plain C, what the reference CPU path computes for one ggml node (or for the
 * whole decode graph) at one thread, including the activation rounding the
 * reference applies before a mat-vec (FP16 for F16 weights, Q8_0 for Q4_0
 * weights) and the lane order of its AVX2 reductions, so that results can be
 * compared with the reference bit for bit on an AVX2+FMA+F16C build.
 *
 * Parity status: pinned against the reference itself.  oracle/Makefile builds
 * the reference's own ggml.c / ggml-quants.c / llama.cpp (unmodified, from
 * where they lie) into oracle/_ref/, tests/golden/make_golden.py runs both on
 * the same seeded inputs and commits the reference's outputs as fixtures, and
 * tests/test_oracle_golden.py checks this file against those fixtures.  The
 * reference's own test-suite has no vectors for the sparse ops.
 */
#ifndef PI_ORACLE_H
#define PI_ORACLE_H

#include <stdint.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

enum pio_type { PIO_F16 = 1, PIO_Q4_0 = 2 };     /* weight storage types on the hot path */
enum pio_arch { PIO_ARCH_LLAMA = 0, PIO_ARCH_FALCON = 1, PIO_ARCH_OPT = 2 };

#define PIO_QK 32
typedef struct { uint16_t d; uint8_t qs[16]; } pio_block_q4_0;   /* ggml-quants.h:11-15 */
typedef struct { uint16_t d; int8_t  qs[32]; } pio_block_q8_0;   /* ggml-quants.h:43-47 */

/* scalar conversions (IEEE binary16, round-to-nearest-even: what F16C does) */
uint16_t pio_fp32_to_fp16(float f);
float    pio_fp16_to_fp32(uint16_t h);
void     pio_fp32_to_fp16_row(const float * x, uint16_t * y, int64_t n);
void     pio_fp16_to_fp32_row(const uint16_t * x, float * y, int64_t n);

/* block formats */
size_t pio_row_bytes(int type, int64_t n);
void   pio_quantize_row_q4_0(const float * x, pio_block_q4_0 * y, int64_t k);   /* ggml-quants.c:428-463 */
void   pio_dequantize_row_q4_0(const pio_block_q4_0 * x, float * y, int64_t k); /* ggml-quants.c:1074-1092 */
void   pio_quantize_row_q8_0(const float * x, pio_block_q8_0 * y, int64_t k);   /* ggml-quants.c:702-760 (AVX2 branch) */

/* dot products with the reference's AVX2 lane order */
float pio_vec_dot_f16(int64_t n, const uint16_t * x, const uint16_t * y);                        /* ggml.c:1188-1221 */
float pio_vec_dot_q4_0_q8_0(int64_t n, const pio_block_q4_0 * x, const pio_block_q8_0 * y);      /* ggml-quants.c:2586-2610 */

/* dense mat-vec / mat-mat: dst[t*nrows + r] = W[r,:] . x[t,:]   (ggml.c:9598-9807) */
void pio_mul_mat(int type, const void * W, int64_t nrows, int64_t ncols,
                 const float * x, int64_t T, float * dst);

/* ggml_mul_mat_idx (GGML_OP_MUL_MAT_SPARSE), CPU semantics (ggml.c:14030-14282):
 * dst[t*nrows + r] = (gpu_idx && gpu_idx[r]==1) || idx[t*idx_stride + r] < threshold ? 0 : W[r,:].x[t,:] */
void pio_mul_mat_idx(int type, const void * W, int64_t nrows, int64_t ncols,
                     const float * x, int64_t T, const float * idx, int64_t idx_stride,
                     const int32_t * gpu_idx, float threshold, float * dst);

/* ggml_axpy (GGML_OP_AXPY), CPU semantics (ggml.c:14314-14463 F16, 14465-14618 Q4_0):
 * dst[t*ncols + c] = sum over active rows r, in row order, of coef(h[t,r]) * Wt[r,c] */
void pio_axpy(int type, const void * Wt, int64_t nrows, int64_t ncols,
              const float * h, int64_t T, const float * idx, int64_t idx_stride,
              const int32_t * gpu_idx, float threshold, float * dst);

/* elementwise / normalisation nodes */
void pio_rms_norm(const float * x, int64_t n, float eps, float * y);          /* ggml.c:9238-9284 */
void pio_norm(const float * x, int64_t n, float eps, float * y);              /* ggml.c:9169-9218 */
void pio_rope(float * x, int64_t head_dim, int64_t n_heads, int32_t pos,
              float freq_base, int neox);                                     /* ggml.c:11163-11325, modes 0 and 2 */
void pio_soft_max(const float * x, int64_t n, float * y);                     /* ggml.c:10708-10777 */

/* ----- whole decode graph (llama.cpp:4949-5084 llama, 5326-5468 falcon, 5086-5204 opt) ----- */

typedef struct {
    const float * attn_norm_w, * attn_norm_b;      /* F32[d]; bias NULL for llama */
    const float * attn_norm2_w, * attn_norm2_b;    /* falcon-40B second layernorm, else NULL */
    const void  * wq, * wk, * wv, * wo;            /* [d,d] [d_kv,d] [d_kv,d] [d,d]; falcon: wq holds the fused wqkv, wk=wv=NULL */
    const float * bq, * bk, * bv, * bo;            /* OPT biases, else NULL */
    const float * ffn_norm_w, * ffn_norm_b;        /* llama / opt */
    const void  * fc1, * fc2;                      /* predictor, always F16: [R,d], [F,R] */
    const void  * gate, * up, * down_t;            /* [F,d] each; gate NULL for falcon / opt */
    const float * up_b, * down_b;                  /* OPT */
} pio_layer;

typedef struct {
    int arch, wtype;                               /* pio_arch, pio_type of the 2-D weights (predictor stays F16) */
    int n_layer, d, n_ff, n_head, n_head_kv, rank, n_vocab, n_ctx;
    float norm_eps, rope_base, threshold;
    const uint16_t * tok_embd;                     /* F16 [n_vocab, d] */
    const uint16_t * pos_embd;                     /* OPT: F16 [n_ctx+2, d] */
    const float * out_norm_w, * out_norm_b;
    const void  * output;                          /* lm head [n_vocab, d] in wtype (OPT: NULL -> tied to tok_embd, F16) */
    const pio_layer * layers;
    int gate_sym;                                  /* llama graph of the "bamboo" architecture: h = relu(gate) * relu(up)
                                                    * (LLM_FFN_SYM, llama.cpp:4732-4738, 5028) instead of relu(gate) * up */
} pio_model;

typedef struct pio_ctx pio_ctx;
pio_ctx * pio_ctx_new(const pio_model * m);
void      pio_ctx_free(pio_ctx * c);
/* One token at position pos; logits[n_vocab] out.  If mask_out != NULL it receives, per layer,
 * the predictor logits (n_layer * n_ff floats). */
void pio_decode(pio_ctx * c, int32_t token, int32_t pos, float * logits, float * pred_out);
void pio_decode_imposed(pio_ctx * c, int32_t token, int32_t pos, float * logits, float * pred_out, const float * idx_imposed);

#ifdef __cplusplus
}
#endif
#endif
