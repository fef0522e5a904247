/*
 * moe_ref.c — CPU oracle for the mixture-of-experts FFN forward path.
 *
 * TEST INFRASTRUCTURE ONLY (see moe_ref.h).  The reference has no MoE layer and
 * no golden vectors for this path; each function below cites the reference
 * primitive whose arithmetic it restates.  Those restatements are pinned to the
 * reference's own kernels, compiled into oracle/_ref and run on a GPU by
 * tests/test_reference_kernels_gpu.py.  The routing rules that have no reference
 * counterpart are stated where they are implemented: PARITY UNPINNED for them.
 *
 * Build with -ffp-contract=off: the reference's host code is Java, which never
 * fuses a multiply and an add, so every `a*b + c` here must stay two roundings.
 * The one place a fused multiply-add is wanted (router logits) calls fmaf().
 */
#include "moe_ref.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

int ref_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ---- bf16 rounding ------------------------------------------------------ */

float ref_bf16_round(float v) {
    uint32_t u;
    memcpy(&u, &v, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) { /* NaN: keep quiet NaN */
        u = (u | 0x00400000u) & 0xffff0000u;
    } else {
        uint32_t lsb = (u >> 16) & 1u;
        u += 0x7fffu + lsb; /* round to nearest, ties to even */
        u &= 0xffff0000u;
    }
    memcpy(&v, &u, 4);
    return v;
}

void ref_bf16_round_array(float *v, int64_t n) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; i++) v[i] = ref_bf16_round(v[i]);
}

/* ---- dense primitives --------------------------------------------------- */

/* src/main/resources/cu/activeFunction.cu:172-180 (silu_forward):
 * output[i] = x[i] / (1.0f + expf(-x[i])). */
static inline float silu1(float x) { return x / (1.0f + expf(-x)); }

void ref_silu(const float *x, float *out, int64_t n) {
    for (int64_t i = 0; i < n; i++) out[i] = silu1(x[i]);
}

/* Y = X * W^T with W stored [out,in] row-major:
 * src/main/java/com/omega/engine/nn/layer/FullyLayer.java:181 (weight shape),
 * :235 (CUBLAS_OP_N, CUBLAS_OP_T call).  Accumulation order follows the
 * engine's host SGEMM, src/main/java/com/omega/engine/cpu/
 * SimplePerfCpuBlasBatchSgemmJdk8.java:106-131: the reduction index p is an
 * outer loop and each output does `C += a*b` once per p, i.e. one sequential
 * chain per output with a separately rounded product.  This small version is
 * the literal form; the blocked one below keeps the same per-output order. */
void ref_linear_nt(const float *X, const float *W, float *Y, int64_t m, int64_t n, int64_t k) {
    for (int64_t i = 0; i < m; i++)
        for (int64_t j = 0; j < n; j++) {
            float acc = 0.0f;
            for (int64_t p = 0; p < k; p++) {
                float prod = X[i * k + p] * W[j * k + p];
                acc = acc + prod;
            }
            Y[i * n + j] = acc;
        }
}

/* src/main/resources/cu/SoftmaxKernel.cu:5-24 (softmax) and its host twin
 * src/main/java/com/omega/engine/gpu/SoftmaxKernel.java:69-87
 * (safeSoftmax_3pass): max with `<=`, e = expf(x - max) summed in index
 * order, then divide. */
void ref_softmax_rows(const float *in, float *out, int64_t rows, int64_t n) {
    for (int64_t r = 0; r < rows; r++) {
        const float *x = in + r * n;
        float *o = out + r * n;
        float mx = -3.402823466e+38F;
        float sum = 0.0f;
        for (int64_t i = 0; i < n; i++)
            if (mx <= x[i]) mx = x[i];
        for (int64_t i = 0; i < n; i++) {
            float e = expf(x[i] - mx);
            sum += e;
            o[i] = e;
        }
        for (int64_t i = 0; i < n; i++) o[i] /= sum;
    }
}

/* RMSNorm in front of the layer: src/main/resources/cu/RMSKernel.cu:185-224
 * (rmsnorm_forward_kernel2, the kernel RMSLayer.output() launches):
 * rms = sqrtf(sum(x*x) / C + eps), out = (x / rms) * weight.  The reference
 * leaves the order of its warp reduction open; it is fixed here like the router
 * tree (lane (i/8)%32 owns element i, one fmaf chain per lane in ascending i,
 * xor butterfly 16..1) so that the rows entering the router are reproducible
 * bit for bit. */
void ref_rmsnorm_rows(const float *x, const float *gamma, float eps, int64_t T, int64_t d, int bf16_out, float *out) {
#pragma omp parallel for schedule(static)
    for (int64_t t = 0; t < T; t++) {
        const float *xr = x + t * d;
        float lane[32];
        for (int l = 0; l < 32; l++) lane[l] = 0.0f;
        for (int64_t i = 0; i < d; i++) {
            int l = (int)((i >> 3) & 31);
            lane[l] = fmaf(xr[i], xr[i], lane[l]);
        }
        for (int m = 16; m >= 1; m >>= 1) {
            float nxt[32];
            for (int l = 0; l < 32; l++) nxt[l] = lane[l] + lane[l ^ m];
            for (int l = 0; l < 32; l++) lane[l] = nxt[l];
        }
        float mean = lane[0] / (float)d;
        float rms = sqrtf(mean + eps);
        for (int64_t i = 0; i < d; i++) {
            float n = xr[i] / rms;
            float v = n * gamma[i];
            out[t * d + i] = bf16_out ? ref_bf16_round(v) : v;
        }
    }
}

/* RMSNorm backward, row by row, as rmsnorm_backward_kernel2 computes it
 * (src/main/resources/cu/RMSKernel.cu:225-275): rms = sqrtf(sum(x^2)/C + eps) (same tree as the forward here),
 * drms = sum_i(x_i * dout_i * w_i) * (-1 / (rms^3 * C)) in index order,
 * dinp_i = dout_i * w_i / rms + drms * x_i,  dweight_i = sum over rows (in row order) of (x_i / rms) * dout_i.
 * dweight is overwritten. */
void ref_rmsnorm_backward_rows(const float *x, const float *gamma, float eps, const float *dout, int64_t T, int64_t d,
                               float *dinp, float *dweight) {
    for (int64_t i = 0; i < d; i++) dweight[i] = 0.0f;
    for (int64_t t = 0; t < T; t++) {
        const float *xr = x + t * d, *gr = dout + t * d;
        float lane[32];
        for (int l = 0; l < 32; l++) lane[l] = 0.0f;
        for (int64_t i = 0; i < d; i++) {
            int l = (int)((i >> 3) & 31);
            lane[l] = fmaf(xr[i], xr[i], lane[l]);
        }
        for (int m = 16; m >= 1; m >>= 1) {
            float nxt[32];
            for (int l = 0; l < 32; l++) nxt[l] = lane[l] + lane[l ^ m];
            for (int l = 0; l < 32; l++) lane[l] = nxt[l];
        }
        float rms = sqrtf(lane[0] / (float)d + eps);
        float drms = 0.0f;
        for (int64_t i = 0; i < d; i++) drms += xr[i] * gr[i] * gamma[i];
        drms = drms * (-1.0f / (rms * rms * rms * (float)d));
        for (int64_t i = 0; i < d; i++) {
            dinp[t * d + i] = gr[i] * gamma[i] / rms + drms * xr[i];
            dweight[i] += (xr[i] / rms) * gr[i];
        }
    }
}

/* ---- routing (no reference counterpart; rules fixed here) ---------------- */

/* Router logits = x * W_r^T (+ bias), FullyLayer semantics as above, but with a
 * FIXED reduction tree so that a 32-lane GPU warp can reproduce every bit:
 *   lane l in [0,32) owns the elements i with (i / 8) % 32 == l and folds them
 *   with TWO fmaf chains, one over its even-numbered elements and one over its
 *   odd-numbered ones, each in ascending i starting at +0 (the pair maps onto
 *   one packed two-wide fp32 multiply-add on the GPU); the lane's partial is
 *   even + odd;
 *   the 32 partials are then combined by an xor butterfly over lane distances
 *   16, 8, 4, 2, 1, every lane computing a[l] = a[l] + a[l ^ m] at once (IEEE
 *   addition commutes, so all lanes agree); lane 0 is the result.
 *   The bias, when present, is added last. */
void ref_router_logits(const float *x, const float *w_r, const float *bias,
                       int64_t T, int64_t d, int64_t E, float *logits) {
#pragma omp parallel for schedule(static)
    for (int64_t t = 0; t < T; t++) {
        const float *xr = x + t * d;
        for (int64_t e = 0; e < E; e++) {
            const float *w = w_r + e * d;
            float even[32], odd[32], lane[32];
            for (int l = 0; l < 32; l++) { even[l] = 0.0f; odd[l] = 0.0f; }
            for (int64_t i = 0; i < d; i++) {
                int l = (int)((i >> 3) & 31);
                if (i & 1) odd[l] = fmaf(xr[i], w[i], odd[l]);
                else even[l] = fmaf(xr[i], w[i], even[l]);
            }
            for (int l = 0; l < 32; l++) lane[l] = even[l] + odd[l];
            for (int m = 16; m >= 1; m >>= 1) {
                float nxt[32];
                for (int l = 0; l < 32; l++) nxt[l] = lane[l] + lane[l ^ m];
                for (int l = 0; l < 32; l++) lane[l] = nxt[l];
            }
            float v = lane[0];
            if (bias) v = v + bias[e];
            logits[t * E + e] = v;
        }
    }
}

/* Top-k and gate weights.  The k picks are taken on the LOGITS: pick j is the
 * largest logit not picked before, a tie going to the lower expert index (the
 * reference's only arg-max, MatrixOperation.maxIndex at
 * src/main/java/com/omega/common/utils/MatrixOperation.java:2008-2020, lets
 * the last maximum win; with no reference top-k to match, the lower index was
 * chosen here and is what the CUDA path implements).  Gate weights are the
 * three-pass softmax over all E logits (ref_softmax_rows arithmetic) read at
 * the picks, and with renorm divided by their sum taken in pick order. */
void ref_topk_gate(const float *logits, int64_t T, int64_t E, int64_t k, int renorm,
                   int32_t *topk_idx, float *topk_w) {
#pragma omp parallel
    {
        float *p = (float *)malloc(sizeof(float) * (size_t)E);
        unsigned char *used = (unsigned char *)malloc((size_t)E);
#pragma omp for schedule(static)
        for (int64_t t = 0; t < T; t++) {
            const float *x = logits + t * E;
            ref_softmax_rows(x, p, 1, E);
            memset(used, 0, (size_t)E);
            float wsum = 0.0f;
            for (int64_t j = 0; j < k; j++) {
                int64_t best = -1;
                for (int64_t e = 0; e < E; e++) {
                    if (used[e]) continue;
                    if (best < 0 || x[e] > x[best]) best = e;
                }
                used[best] = 1;
                topk_idx[t * k + j] = (int32_t)best;
                topk_w[t * k + j] = p[best];
                wsum += p[best];
            }
            if (renorm)
                for (int64_t j = 0; j < k; j++) topk_w[t * k + j] = topk_w[t * k + j] / wsum;
        }
        free(p);
        free(used);
    }
}

/* Histogram, exclusive scan and the dispatch permutation.  Rows are grouped
 * expert-major; inside one expert they keep the order of the flat pick index
 * f = t*k + j (a stable counting sort). */
void ref_histogram_permute(const int32_t *topk_idx, int64_t T, int64_t E, int64_t k,
                           int32_t *counts, int32_t *offsets, int32_t *perm, int32_t *pos) {
    for (int64_t e = 0; e < E; e++) counts[e] = 0;
    for (int64_t f = 0; f < T * k; f++) counts[topk_idx[f]]++;
    offsets[0] = 0;
    for (int64_t e = 0; e < E; e++) offsets[e + 1] = offsets[e] + counts[e];
    if (!perm && !pos) return;
    int32_t *cur = (int32_t *)malloc(sizeof(int32_t) * (size_t)E);
    for (int64_t e = 0; e < E; e++) cur[e] = offsets[e];
    for (int64_t f = 0; f < T * k; f++) {
        int32_t e = topk_idx[f];
        int32_t r = cur[e]++;
        if (perm) perm[r] = (int32_t)f;
        if (pos) pos[f] = r;
    }
    free(cur);
}

/* ---- expert products ---------------------------------------------------- */

/* Y[m,n] (+)= X[m,kk] * Wt[kk,n] where Wt is W transposed to [in,out].  For
 * every output the products are added in ascending reduction index, each
 * product rounded on its own — the same per-output chain as ref_linear_nt and
 * as the engine's tiledSgemm (p outer, `C += a*b`).  Blocking over rows and
 * output columns only changes which outputs are worked on together. */
static void linear_t_block(const float *X, int64_t ldx, const float *Wt, int64_t n,
                           float *Yb, int64_t ldy, int64_t ycol0, int64_t m, int64_t kk,
                           int64_t c0, int64_t c1) {
    /* output column c is stored at Yb[r*ldy + c - ycol0] */
    float *Y = Yb - ycol0;
    for (int64_t r = 0; r < m; r++)
        for (int64_t c = c0; c < c1; c++) Y[r * ldy + c] = 0.0f;
    int64_t r = 0;
    for (; r + 4 <= m; r += 4) {
        float *y0 = Y + (r + 0) * ldy, *y1 = Y + (r + 1) * ldy;
        float *y2 = Y + (r + 2) * ldy, *y3 = Y + (r + 3) * ldy;
        for (int64_t p = 0; p < kk; p++) {
            const float *w = Wt + p * n;
            float a0 = X[(r + 0) * ldx + p], a1 = X[(r + 1) * ldx + p];
            float a2 = X[(r + 2) * ldx + p], a3 = X[(r + 3) * ldx + p];
            for (int64_t c = c0; c < c1; c++) {
                float wv = w[c];
                y0[c] += a0 * wv;
                y1[c] += a1 * wv;
                y2[c] += a2 * wv;
                y3[c] += a3 * wv;
            }
        }
    }
    for (; r < m; r++) {
        float *y0 = Y + r * ldy;
        for (int64_t p = 0; p < kk; p++) {
            const float *w = Wt + p * n;
            float a0 = X[r * ldx + p];
            for (int64_t c = c0; c < c1; c++) y0[c] += a0 * w[c];
        }
    }
}

static void transpose(const float *W, float *Wt, int64_t rows, int64_t cols) {
    /* W [rows, cols] -> Wt [cols, rows] */
    const int64_t B = 32;
#pragma omp parallel for schedule(static) collapse(2)
    for (int64_t r0 = 0; r0 < rows; r0 += B)
        for (int64_t c0 = 0; c0 < cols; c0 += B) {
            int64_t r1 = r0 + B < rows ? r0 + B : rows;
            int64_t c1 = c0 + B < cols ? c0 + B : cols;
            for (int64_t r = r0; r < r1; r++)
                for (int64_t c = c0; c < c1; c++) Wt[c * rows + r] = W[r * cols + c];
        }
}

/* One expert's SwiGLU FFN over m gathered rows.  Order of operations follows
 * src/main/java/com/omega/engine/nn/layer/llama/LlamaMLPLayer.java:117-123:
 * linear1 (gate) -> SiLU -> linear3 (up) -> element-wise multiply
 * (src/main/resources/cu/OPKernel.cu:1040, R = X*Y) -> linear2 (down).
 * bf16 mode inserts the roundings the tensor-core path has: h and yp. */
static void expert_ffn(const float *Xe, int64_t m, int64_t d, int64_t dff,
                       const float *WgT, const float *WuT, const float *WdT,
                       int bf16, float *H, float *Yp) {
    const int64_t CB = 512, RB = 16;
    int64_t nrb = (m + RB - 1) / RB;
    int64_t ncb1 = (dff + CB - 1) / CB, ncb2 = (d + CB - 1) / CB;
#pragma omp parallel
    {
        float *tmp = (float *)malloc(sizeof(float) * (size_t)(RB * CB * 2));
#pragma omp for schedule(dynamic) collapse(2)
        for (int64_t rb = 0; rb < nrb; rb++)
            for (int64_t cb = 0; cb < ncb1; cb++) {
                int64_t r0 = rb * RB, r1 = r0 + RB < m ? r0 + RB : m;
                int64_t c0 = cb * CB, c1 = c0 + CB < dff ? c0 + CB : dff;
                int64_t mm = r1 - r0, w = c1 - c0;
                float *g = tmp, *u = tmp + RB * CB;
                linear_t_block(Xe + r0 * d, d, WgT, dff, g, CB, c0, mm, d, c0, c1);
                linear_t_block(Xe + r0 * d, d, WuT, dff, u, CB, c0, mm, d, c0, c1);
                for (int64_t r = 0; r < mm; r++)
                    for (int64_t c = 0; c < w; c++) {
                        float hv = silu1(g[r * CB + c]) * u[r * CB + c];
                        H[(r0 + r) * dff + c0 + c] = bf16 ? ref_bf16_round(hv) : hv;
                    }
            }
#pragma omp for schedule(dynamic) collapse(2)
        for (int64_t rb = 0; rb < nrb; rb++)
            for (int64_t cb = 0; cb < ncb2; cb++) {
                int64_t r0 = rb * RB, r1 = r0 + RB < m ? r0 + RB : m;
                int64_t c0 = cb * CB, c1 = c0 + CB < d ? c0 + CB : d;
                linear_t_block(H + r0 * dff, dff, WdT, d, Yp + r0 * d, d, 0, r1 - r0, dff, c0, c1);
                if (bf16)
                    for (int64_t r = r0; r < r1; r++)
                        for (int64_t c = c0; c < c1; c++) Yp[r * d + c] = ref_bf16_round(Yp[r * d + c]);
            }
        free(tmp);
    }
}

/* ---- whole layer -------------------------------------------------------- */

void ref_moe_forward(const ref_moe_shape *s,
                     const float *x, const float *w_r, const float *bias,
                     const float *w_gate, const float *w_up, const float *w_down,
                     float *logits, int32_t *topk_idx, float *topk_w,
                     int32_t *counts, int32_t *offsets, int32_t *perm,
                     const int32_t *sel, int64_t n_sel, float *y, int nthreads) {
    const int64_t T = s->T, d = s->d, dff = s->dff, E = s->E, k = s->k;
#ifdef _OPENMP
    int saved = omp_get_max_threads();
    if (nthreads > 0) omp_set_num_threads(nthreads);
#else
    (void)nthreads;
#endif
    float *lg = logits ? logits : (float *)malloc(sizeof(float) * (size_t)(T * E));
    ref_router_logits(x, w_r, bias, T, d, E, lg);
    ref_topk_gate(lg, T, E, k, s->renorm, topk_idx, topk_w);
    ref_histogram_permute(topk_idx, T, E, k, counts, offsets, perm, NULL);
    if (!logits) free(lg);

    if (y && (sel ? n_sel : T) > 0) {
        int64_t ns = sel ? n_sel : T;
        /* dispatch of the selected tokens only: expert-major, stable */
        int64_t R = ns * k;
        int32_t *scount = (int32_t *)calloc((size_t)E + 1, sizeof(int32_t));
        int32_t *soff = (int32_t *)calloc((size_t)E + 1, sizeof(int32_t));
        int32_t *spos = (int32_t *)malloc(sizeof(int32_t) * (size_t)R);
        for (int64_t i = 0; i < ns; i++) {
            int64_t t = sel ? sel[i] : i;
            for (int64_t j = 0; j < k; j++) scount[topk_idx[t * k + j]]++;
        }
        for (int64_t e = 0; e < E; e++) soff[e + 1] = soff[e] + scount[e];
        int32_t *cur = (int32_t *)malloc(sizeof(int32_t) * (size_t)E);
        for (int64_t e = 0; e < E; e++) cur[e] = soff[e];
        float *Xp = (float *)malloc(sizeof(float) * (size_t)(R * d));
        for (int64_t i = 0; i < ns; i++) {
            int64_t t = sel ? sel[i] : i;
            for (int64_t j = 0; j < k; j++) {
                int32_t e = topk_idx[t * k + j];
                int32_t r = cur[e]++;
                spos[i * k + j] = r;
                for (int64_t c = 0; c < d; c++) {
                    float v = x[t * d + c];
                    Xp[(int64_t)r * d + c] = s->bf16 ? ref_bf16_round(v) : v;
                }
            }
        }
        int64_t mmax = 0;
        for (int64_t e = 0; e < E; e++)
            if (scount[e] > mmax) mmax = scount[e];
        float *H = (float *)malloc(sizeof(float) * (size_t)(mmax * dff + 1));
        float *Yp = (float *)malloc(sizeof(float) * (size_t)(R * d + 1));
        float *WgT = NULL, *WuT = NULL, *WdT = NULL;
        if (!s->pretransposed) {
            WgT = (float *)malloc(sizeof(float) * (size_t)(d * dff));
            WuT = (float *)malloc(sizeof(float) * (size_t)(d * dff));
            WdT = (float *)malloc(sizeof(float) * (size_t)(d * dff));
        }
        for (int64_t e = 0; e < E; e++) {
            int64_t m = scount[e];
            if (m == 0) continue;
            const float *g = w_gate + e * dff * d, *u = w_up + e * dff * d, *dn = w_down + e * d * dff;
            if (!s->pretransposed) {
                transpose(g, WgT, dff, d); /* [dff,d] -> [d,dff] */
                transpose(u, WuT, dff, d);
                transpose(dn, WdT, d, dff); /* [d,dff] -> [dff,d] */
                g = WgT; u = WuT; dn = WdT;
            }
            expert_ffn(Xp + (int64_t)soff[e] * d, m, d, dff, g, u, dn, s->bf16, H,
                       Yp + (int64_t)soff[e] * d);
        }
        /* Combine: y[t,:] = ((w0*yp0) + w1*yp1) + ... in pick order, fp32,
         * each product rounded before it is added. */
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < ns; i++) {
            int64_t t = sel ? sel[i] : i;
            for (int64_t c = 0; c < d; c++) {
                float acc = 0.0f;
                for (int64_t j = 0; j < k; j++) {
                    float prod = topk_w[t * k + j] * Yp[(int64_t)spos[i * k + j] * d + c];
                    acc = (j == 0) ? prod : acc + prod;
                }
                y[i * d + c] = s->out_bf16 ? ref_bf16_round(acc) : acc;
            }
        }
        free(WgT); free(WuT); free(WdT);
        free(H); free(Yp); free(Xp);
        free(cur); free(spos); free(soff); free(scount);
    }
#ifdef _OPENMP
    omp_set_num_threads(saved);
#endif
}

/* ---- backward of the whole layer ---------------------------------------- */

/* C[M,N] = sum_p A(m,p) * B(p,n); element (i,j) of A is A[i*sa0 + j*sa1], of B
 * B[i*sb0 + j*sb1].  One chain per output, p ascending, every product rounded
 * on its own: the order of the engine's host SGEMM
 * (src/main/java/com/omega/engine/cpu/SimplePerfCpuBlasBatchSgemmJdk8.java:106-131). */
static void gemm_strided(const float *A, int64_t sa0, int64_t sa1, const float *B, int64_t sb0, int64_t sb1,
                         float *C, int64_t M, int64_t N, int64_t K) {
#pragma omp parallel for schedule(static)
    for (int64_t m = 0; m < M; m++)
        for (int64_t n = 0; n < N; n++) {
            float acc = 0.0f;
            for (int64_t p = 0; p < K; p++) acc += A[m * sa0 + p * sa1] * B[p * sb0 + n * sb1];
            C[m * N + n] = acc;
        }
}

static void round_if(float *v, int64_t n, int bf16) {
    if (bf16) ref_bf16_round_array(v, n);
}

/* d SiLU / dx as the reference's silu_backward computes it
 * (src/main/resources/cu/activeFunction.cu:182-190): s = 1/(1+exp(-x)), s*(1 + x*(1-s)). */
static inline float silu_grad1(float x) {
    float sg = 1.0f / (1.0f + expf(-x));
    return sg * (1.0f + x * (1.0f - sg));
}

void ref_silu_backward(const float *x, const float *delta, float *diff, int64_t n) {
    for (int64_t i = 0; i < n; i++) diff[i] = delta[i] * silu_grad1(x[i]);
}

/* Softmax backward, row by row, as the reference's softmax_back
 * (src/main/resources/cu/SoftmaxKernel.cu:100-112): sum = sum_i out_i*delta_i in
 * index order, diff_i = (delta_i - sum) * out_i. */
void ref_softmax_back_rows(const float *out, const float *delta, float *diff, int64_t rows, int64_t n) {
    for (int64_t r = 0; r < rows; r++) {
        float sum = 0.0f;
        for (int64_t i = 0; i < n; i++) sum += out[r * n + i] * delta[r * n + i];
        for (int64_t i = 0; i < n; i++) diff[r * n + i] = (delta[r * n + i] - sum) * out[r * n + i];
    }
}

/* Gradients of y = MoE(x) for a given dy.  The chain follows the reference's dense layers:
 *   LlamaMLPLayer.diff() (src/main/java/com/omega/engine/nn/layer/llama/LlamaMLPLayer.java:139-158):
 *     linear2.back(delta); d_up = d_h * silu(g); d_gate = silu_backward(g, d_h * u);
 *     diff = linear1.diff + linear3.diff
 *   FullyLayer.diff() (src/main/java/com/omega/engine/nn/layer/FullyLayer.java:292-334):
 *     diffW = delta^T * input (overwritten, not accumulated), diff = delta * W, diffB = column sums of delta
 *   softmax_back (SoftmaxKernel.cu:100-112) for the router probabilities.
 * Rules with no reference counterpart: the picks are constants (no gradient through the selection);
 * with renormalised gates w_j = p_j / s, s = sum of the picked p, d p_j = (d w_j - sum_i d w_i w_i) / s;
 * d w_j = <dy[t], yp_j>; dx[t] = ((dxp_0 + dxp_1) + ...) in pick order, then the router's term
 * (sum over experts in index order, one chain) added last.  aux_coef != 0 adds aux_coef * L_aux
 * (ref_aux_loss) to the objective: its gradient enters at the router's probabilities.
 * bf16 mode rounds where the tensor-core path stores bf16: xp, g, u, h, yp, dyp, dh, dg, du, dxp
 * (weight gradients and everything on the router's side stay fp32); dx is rounded when out_bf16. */
/* Auxiliary load-balancing loss of a step (no reference counterpart; the usual switch-routing form):
 *   L = E * sum_e f_e * P_e,  f_e = counts[e] / (T*k) (share of the picks that went to e, a constant),
 *   P_e = (1/T) * sum_t p[t,e] (mean router probability).  Sums in index order.  T == 0: 0. */
float ref_aux_loss(const float *logits, const int32_t *counts, int64_t T, int64_t E, int64_t k) {
    if (T == 0) return 0.0f;
    float *p = (float *)malloc(sizeof(float) * (size_t)(T * E));
    ref_softmax_rows(logits, p, T, E);
    float loss = 0.0f;
    for (int64_t e = 0; e < E; e++) {
        float ps = 0.0f;
        for (int64_t t = 0; t < T; t++) ps += p[t * E + e];
        loss += ((float)counts[e] / (float)(T * k)) * (ps / (float)T);
    }
    free(p);
    return (float)E * loss;
}

void ref_moe_backward(const ref_moe_shape *s, const float *x, const float *w_r, const float *bias,
                      const float *w_gate, const float *w_up, const float *w_down, const float *dy, float aux_coef,
                      float *dx, float *d_w_r, float *d_bias, float *d_w_gate, float *d_w_up, float *d_w_down,
                      int nthreads) {
    const int64_t T = s->T, d = s->d, dff = s->dff, E = s->E, k = s->k;
    const int bf = s->bf16;
#ifdef _OPENMP
    int saved = omp_get_max_threads();
    if (nthreads > 0) omp_set_num_threads(nthreads);
#else
    (void)nthreads;
#endif
    float *logits = (float *)malloc(sizeof(float) * (size_t)(T * E));
    float *probs = (float *)malloc(sizeof(float) * (size_t)(T * E));
    int32_t *idx = (int32_t *)malloc(sizeof(int32_t) * (size_t)(T * k));
    float *gw = (float *)malloc(sizeof(float) * (size_t)(T * k));
    int32_t *counts = (int32_t *)malloc(sizeof(int32_t) * (size_t)E);
    int32_t *offsets = (int32_t *)malloc(sizeof(int32_t) * (size_t)(E + 1));
    int32_t *perm = (int32_t *)malloc(sizeof(int32_t) * (size_t)(T * k));
    int32_t *pos = (int32_t *)malloc(sizeof(int32_t) * (size_t)(T * k));
    ref_router_logits(x, w_r, bias, T, d, E, logits);
    ref_topk_gate(logits, T, E, k, s->renorm, idx, gw);
    ref_histogram_permute(idx, T, E, k, counts, offsets, perm, pos);
    ref_softmax_rows(logits, probs, T, E);

    float *dgw = (float *)malloc(sizeof(float) * (size_t)(T * k));       /* d w[t,j] */
    float *dxp = (float *)malloc(sizeof(float) * (size_t)(T * k * d + 1));
    for (int64_t e = 0; e < E; e++) {
        const int64_t m = counts[e], r0 = offsets[e];
        float *dWg = d_w_gate + e * dff * d, *dWu = d_w_up + e * dff * d, *dWd = d_w_down + e * d * dff;
        if (m == 0) { /* diffW = delta^T * input over no rows */
            memset(dWg, 0, sizeof(float) * (size_t)(dff * d));
            memset(dWu, 0, sizeof(float) * (size_t)(dff * d));
            memset(dWd, 0, sizeof(float) * (size_t)(dff * d));
            continue;
        }
        const float *Wg = w_gate + e * dff * d, *Wu = w_up + e * dff * d, *Wd = w_down + e * d * dff;
        float *Xe = (float *)malloc(sizeof(float) * (size_t)(m * d));
        float *dYp = (float *)malloc(sizeof(float) * (size_t)(m * d));
        float *Yp = (float *)malloc(sizeof(float) * (size_t)(m * d));
        float *G = (float *)malloc(sizeof(float) * (size_t)(m * dff));
        float *U = (float *)malloc(sizeof(float) * (size_t)(m * dff));
        float *H = (float *)malloc(sizeof(float) * (size_t)(m * dff));
        float *dH = (float *)malloc(sizeof(float) * (size_t)(m * dff));
        float *dG = (float *)malloc(sizeof(float) * (size_t)(m * dff));
        float *dU = (float *)malloc(sizeof(float) * (size_t)(m * dff));
        float *t1 = (float *)malloc(sizeof(float) * (size_t)(m * d));
        for (int64_t r = 0; r < m; r++) {
            const int64_t f = perm[r0 + r], t = f / k;
            for (int64_t c = 0; c < d; c++) {
                Xe[r * d + c] = bf ? ref_bf16_round(x[t * d + c]) : x[t * d + c];
                dYp[r * d + c] = gw[f] * dy[t * d + c];
            }
        }
        round_if(dYp, m * d, bf);
        /* forward again, keeping what the backward needs */
        gemm_strided(Xe, d, 1, Wg, 1, d, G, m, dff, d);
        gemm_strided(Xe, d, 1, Wu, 1, d, U, m, dff, d);
        round_if(G, m * dff, bf);
        round_if(U, m * dff, bf);
        for (int64_t i = 0; i < m * dff; i++) H[i] = silu1(G[i]) * U[i];
        round_if(H, m * dff, bf);
        gemm_strided(H, dff, 1, Wd, 1, dff, Yp, m, d, dff);
        round_if(Yp, m * d, bf);
        for (int64_t r = 0; r < m; r++) { /* d w = <dy[t], yp> */
            const int64_t f = perm[r0 + r], t = f / k;
            float acc = 0.0f;
            for (int64_t c = 0; c < d; c++) acc += dy[t * d + c] * Yp[r * d + c];
            dgw[f] = acc;
        }
        /* linear2.back: diffW = delta^T * input, diff = delta * W */
        gemm_strided(dYp, 1, d, H, dff, 1, dWd, d, dff, m);
        gemm_strided(dYp, d, 1, Wd, dff, 1, dH, m, dff, d);
        round_if(dH, m * dff, bf);
        for (int64_t i = 0; i < m * dff; i++) {
            dU[i] = dH[i] * silu1(G[i]);
            dG[i] = (dH[i] * U[i]) * silu_grad1(G[i]);
        }
        round_if(dU, m * dff, bf);
        round_if(dG, m * dff, bf);
        gemm_strided(dG, 1, dff, Xe, d, 1, dWg, dff, d, m);
        gemm_strided(dU, 1, dff, Xe, d, 1, dWu, dff, d, m);
        /* diff = linear1.diff + linear3.diff */
        gemm_strided(dG, dff, 1, Wg, d, 1, t1, m, d, dff);
        gemm_strided(dU, dff, 1, Wu, d, 1, dxp + r0 * d, m, d, dff);
        for (int64_t i = 0; i < m * d; i++) dxp[r0 * d + i] = t1[i] + dxp[r0 * d + i];
        round_if(dxp + r0 * d, m * d, bf);
        free(Xe); free(dYp); free(Yp); free(G); free(U); free(H); free(dH); free(dG); free(dU); free(t1);
    }

    /* router: d w -> d p (picks only) -> d logits (softmax_back) */
    float *dp = (float *)calloc((size_t)(T * E), sizeof(float));
    float *dl = (float *)malloc(sizeof(float) * (size_t)(T * E));
    for (int64_t t = 0; t < T; t++) {
        if (s->renorm) {
            float ssum = 0.0f, dot = 0.0f;
            for (int64_t j = 0; j < k; j++) ssum += probs[t * E + idx[t * k + j]];
            for (int64_t j = 0; j < k; j++) dot += dgw[t * k + j] * gw[t * k + j];
            for (int64_t j = 0; j < k; j++) dp[t * E + idx[t * k + j]] = (dgw[t * k + j] - dot) / ssum;
        } else {
            for (int64_t j = 0; j < k; j++) dp[t * E + idx[t * k + j]] = dgw[t * k + j];
        }
        /* aux_coef * dL/dp[t,e] = aux_coef * E * f_e / T, added to every expert's entry */
        if (aux_coef != 0.0f)
            for (int64_t e = 0; e < E; e++)
                dp[t * E + e] += (aux_coef * (float)E / (float)T) * ((float)counts[e] / (float)(T * k));
    }
    ref_softmax_back_rows(probs, dp, dl, T, E);
    /* router's FullyLayer.diff(): diffW = dl^T * x, diffB = column sums, diff = dl * W_r */
    gemm_strided(dl, 1, E, x, d, 1, d_w_r, E, d, T);
    if (d_bias)
        for (int64_t e = 0; e < E; e++) {
            float acc = 0.0f;
            for (int64_t t = 0; t < T; t++) acc += dl[t * E + e];
            d_bias[e] = acc;
        }
#pragma omp parallel for schedule(static)
    for (int64_t t = 0; t < T; t++)
        for (int64_t c = 0; c < d; c++) {
            float acc = 0.0f;
            for (int64_t j = 0; j < k; j++) {
                float v = dxp[(int64_t)pos[t * k + j] * d + c];
                acc = (j == 0) ? v : acc + v;
            }
            float r = 0.0f;
            for (int64_t e = 0; e < E; e++) r += dl[t * E + e] * w_r[e * d + c];
            acc += r;
            dx[t * d + c] = s->out_bf16 ? ref_bf16_round(acc) : acc;
        }
    free(dp); free(dl); free(dxp); free(dgw);
    free(logits); free(probs); free(idx); free(gw); free(counts); free(offsets); free(perm); free(pos);
#ifdef _OPENMP
    omp_set_num_threads(saved);
#endif
}
