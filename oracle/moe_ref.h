/*
 * moe_ref.h — CPU oracle for the mixture-of-experts FFN forward path.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the shipped library links, loads or
 * calls this code; it exists so tests and the benchmark's CPU-baseline leg can
 * check the CUDA path against a plain-C restatement of the arithmetic.
 *
 * PARITY: the reference engine (dromara/Omega-AI) has no mixture-of-experts
 * layer, router, top-k or permutation code and ships no golden vectors, so
 * this oracle is assembled from the reference's dense primitives (cited per
 * function in moe_ref.c) plus routing/permutation/combine rules fixed by this
 * project.
 *   - Pinned to the reference itself: softmax, SiLU, the element-wise product,
 *     RMSNorm, the X*W^T product and the dense SwiGLU sequence.  The reference's
 *     own CUDA kernels for these are compiled from its source files into
 *     oracle/_ref (Makefile target ref_kernels) and run beside cuBLAS SGEMM by
 *     refk_driver.cu; tests/test_reference_kernels_gpu.py holds this oracle
 *     (and the product) against their outputs.  Also pinned: the SiLU demo
 *     inputs and the all-ones GEMM check found in the reference's sources.
 *   - PARITY UNPINNED for what the reference does not have: the router's
 *     reduction order, top-k and tie rule, gate renormalisation, permutation
 *     and combine are defined here and have nothing to be pinned to.
 */
#ifndef OMOE_ORACLE_MOE_REF_H
#define OMOE_ORACLE_MOE_REF_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* rows padded to this many per expert in the library's internal dispatch
 * buffer; the oracle reports UNPADDED positions, the constant is exported so
 * tests can convert. */
#define REF_ROW_ALIGN 128

typedef struct ref_moe_shape {
    int32_t T;        /* tokens */
    int32_t d;        /* d_model */
    int32_t dff;      /* expert hidden size */
    int32_t E;        /* experts */
    int32_t k;        /* picks per token */
    int32_t renorm;   /* 1: gate weights renormalised over the k picks */
    int32_t bf16;     /* 1: bf16 rounding points (weights, x, h, yp) */
    int32_t out_bf16; /* 1: y rounded to bf16 */
    int32_t pretransposed; /* 1: w_gate,w_up given as [E,d,dff] and w_down as [E,dff,d]
                              ([in,out]); skips the per-call transposition */
} ref_moe_shape;

/* round-to-nearest-even to bf16 precision, result kept in a float */
float ref_bf16_round(float v);
void ref_bf16_round_array(float *v, int64_t n);

/* silu(x) = x / (1 + expf(-x)) */
void ref_silu(const float *x, float *out, int64_t n);

/* Y[m,n] = X[m,k] * W[n,k]^T, W row-major [out,in]; per-output accumulation
 * sequential in k with separate multiply and add. */
void ref_linear_nt(const float *X, const float *W, float *Y, int64_t m, int64_t n, int64_t k);

/* rows normalised as the block's RMSNorm does: (x / sqrtf(mean(x^2) + eps)) * gamma, fixed reduction tree */
void ref_rmsnorm_rows(const float *x, const float *gamma, float eps, int64_t T, int64_t d, int bf16_out, float *out);

/* row softmax, three passes */
void ref_softmax_rows(const float *in, float *out, int64_t rows, int64_t n);

/* router logits with the fixed 32-lane reduction tree; bias may be NULL */
void ref_router_logits(const float *x, const float *w_r, const float *bias,
                       int64_t T, int64_t d, int64_t E, float *logits);

/* top-k on logits (descending, ties -> lower expert), gate weights from the
 * softmax over all E logits, optionally renormalised over the picks. */
void ref_topk_gate(const float *logits, int64_t T, int64_t E, int64_t k, int renorm,
                   int32_t *topk_idx, float *topk_w);

/* per-expert counts, exclusive offsets[E+1], expert-major stable permutation:
 * perm[offsets[e]+r] = t*k+j, pos[t*k+j] = offsets[e]+r. */
void ref_histogram_permute(const int32_t *topk_idx, int64_t T, int64_t E, int64_t k,
                           int32_t *counts, int32_t *offsets, int32_t *perm, int32_t *pos);

/* Whole layer.  x [T,d]; w_r [E,d]; bias [E] or NULL; w_gate,w_up [E,dff,d];
 * w_down [E,d,dff] (all row-major [out,in]).  Outputs for ALL tokens: logits
 * (nullable), topk_idx, topk_w, counts, offsets, perm (nullable).  y is
 * computed only for the n_sel tokens listed in sel (sel==NULL: all tokens, in
 * order) and written as y[i,:] for the i-th selected token.  Weights must
 * already hold bf16-representable values when shape.bf16 is set (call
 * ref_bf16_round_array first); x is rounded internally for the expert path.
 * nthreads <= 0: all cores. */
void ref_moe_forward(const ref_moe_shape *shape,
                     const float *x, const float *w_r, const float *bias,
                     const float *w_gate, const float *w_up, const float *w_down,
                     float *logits, int32_t *topk_idx, float *topk_w,
                     int32_t *counts, int32_t *offsets, int32_t *perm,
                     const int32_t *sel, int64_t n_sel, float *y, int nthreads);

/* RMSNorm backward (rmsnorm_backward_kernel2, RMSKernel.cu:225-275); dweight [d] is overwritten. */
void ref_rmsnorm_backward_rows(const float *x, const float *gamma, float eps, const float *dout, int64_t T, int64_t d,
                               float *dinp, float *dweight);

/* SiLU and softmax backward, element by element / row by row as the reference's kernels
 * silu_backward (activeFunction.cu:182-190) and softmax_back (SoftmaxKernel.cu:100-112) compute them. */
void ref_silu_backward(const float *x, const float *delta, float *diff, int64_t n);
void ref_softmax_back_rows(const float *out, const float *delta, float *diff, int64_t rows, int64_t n);

/* Backward of the whole layer for a given dy [T,d]: dx [T,d], d_w_r [E,d], d_bias [E] (nullable),
 * d_w_gate/d_w_up [E,dff,d], d_w_down [E,d,dff], all overwritten (the reference's FullyLayer.diff()
 * overwrites diffW).  Routing is recomputed from x; shape.pretransposed must be 0.  The rules and the
 * bf16 rounding points are stated at the definition. */
void ref_moe_backward(const ref_moe_shape *shape, const float *x, const float *w_r, const float *bias,
                      const float *w_gate, const float *w_up, const float *w_down, const float *dy, float aux_coef,
                      float *dx, float *d_w_r, float *d_bias, float *d_w_gate, float *d_w_up, float *d_w_down,
                      int nthreads);

/* Auxiliary load-balancing loss L = E * sum_e (counts[e]/(T*k)) * mean_t p[t,e]; ref_moe_backward's aux_coef
 * adds aux_coef * L to the objective whose gradient it returns. */
float ref_aux_loss(const float *logits, const int32_t *counts, int64_t T, int64_t E, int64_t k);

int ref_num_threads(void);

#ifdef __cplusplus
}
#endif
#endif
