// Backward of the MoE layer: gradients with respect to the input rows and to every weight, for a
// given gradient of the output.
//
// The chain is the reference's, applied per expert to the rows that expert received:
//   LlamaMLPLayer.diff() (src/main/java/com/omega/engine/nn/layer/llama/LlamaMLPLayer.java:139-158):
//     linear2.back(delta); d_up = d_h * silu(g); d_gate = silu_backward(g, d_h * u); diff = linear1.diff + linear3.diff
//   FullyLayer.diff() (src/main/java/com/omega/engine/nn/layer/FullyLayer.java:292-334):
//     diffW = delta^T * input (overwritten each call), diff = delta * W, diffB = column sums of delta
//   silu_backward (src/main/resources/cu/activeFunction.cu:182-190), softmax_back
//   (src/main/resources/cu/SoftmaxKernel.cu:100-112) for the router's probabilities.
// What the reference does not have is fixed here: the picks are constants; with renormalised gates
// w_j = p_j / s the probabilities get d p_j = (d w_j - sum_i d w_i w_i) / s; d w_j = <dy[t], yp_j>;
// dx[t] = sum of the picks' dxp rows in pick order plus the router's term, added last.
//
// A forward in training mode keeps what this needs: the pre-activation rows g and u (one buffer
// [rows, 2*d_ff], g in the left half), h, yp and the routing.  The fused SiLU epilogue of the inference
// forward cannot keep g and u, so the training forward runs the up/gate products as two plain products
// plus one element-wise pass.
//
// bf16 layers: every product runs on the tcgen05 kernels.  The two input-gradient products are the
// forward's persistent kernel on transposed copies of the weights (W_down^T, and [W_gate^T | W_up^T] so
// that dxp = [dg | du] * [W_gate ; W_up] is ONE product over K = 2*d_ff); the weight-gradient products
// (experts_sm100_wgrad.cu) reduce over an expert's rows, so their operands are the transposed
// activations, written by a pass that also zero-fills each expert's padding rows.
// fp32 layers: a plain tiled FMA kernel with strided operands (sized for parity runs, not for speed).
#include <stdlib.h>
#include <string.h>

#include <new>
#include <type_traits>

#include "backward.cuh"
#include "common.cuh"
#include "ep.cuh"

namespace omoe {

struct BwState {
    bool training;
    bool fwd_valid;   // the last forward ran in training mode and its saved rows are intact
    bool wt_valid;    // transposed weight copies match the current weights
    int fwd_T;
    float aux_coef;   // weight of the auxiliary load-balancing loss in the objective (0: none)
    float *aux_ps;    // [E] column sums of the router probabilities (omoe_get_aux_loss)
    void *dxn;        // [t_max, d] gradient of the normalised rows (block form), io dtype
    float *inv_rms;   // [t_max] 1/rms of every row (block form)
    void *gu;         // [rows_cap, 2*dff] g | u (compute dtype)
    void *dyp;        // [rows_cap, d]
    void *dh;         // [rows_cap, dff]
    void *dgu;        // [rows_cap, 2*dff] dg | du
    void *dxp;        // [rows_cap, d]
    float *dgw;       // [t_max*k] gradient of the gate weights
    void **dyp_table, **dxp_table;  // device [world]: every rank's dyp / dxp buffer (entry `rank` is this GPU's)
    bool own_grad_rows;  // dyp, dxp and the tables were allocated here (one GPU); else they belong to the transport
    float *dl;        // [t_max, E] gradient of the logits
    float *dwr_part;  // [slices][E][d] partial sums of d W_router
    int dwr_slices;
    // bf16 layers only
    void *wdT;        // [El, dff, d]     W_down^T
    void *wguT;       // [El, d, 2*dff]   [W_gate^T | W_up^T]
    void *xpT, *hT, *dypT, *dguT;  // [cols, rows_cap] transposed activations
    // gradients (fp32)
    float *d_router, *d_bias, *d_gate, *d_up, *d_down;
    // tensor maps of the bf16 products
    CUtensorMap m_g_out, m_u_out;          // halves of gu as store targets
    CUtensorMap m_dyp_a, m_wdT_b, m_dh_c;  // dh = dyp * W_down
    CUtensorMap m_dgu_a, m_wguT_b, m_dxp_c;  // dxp = [dg|du] * [Wg;Wu]
    CUtensorMap m_dypT, m_hT, m_dguT, m_xpT;  // weight-gradient operands, transposed copies (older path)
    CUtensorMap m_dyp_r, m_h_r, m_dgu_r, m_xp_r;  // weight-gradient operands read in place (64-row boxes)
    bool wgrad_transposed;  // OMOE_WGRAD_TRANSPOSED=1: use the transposed copies
};

namespace {

// ---- element access for fp32 and bf16 rows --------------------------------------------------------
__device__ __forceinline__ float ldf(const float *p) { return *p; }
__device__ __forceinline__ float ldf(const __nv_bfloat16 *p) { return __bfloat162float(*p); }


__device__ __forceinline__ float silu_f32(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float silu_grad_f32(float x) {
    const float sg = 1.0f / (1.0f + expf(-x));
    return sg * (1.0f + x * (1.0f - sg));
}

// ---- element-wise passes over the rows in use -----------------------------------------------------
// h = silu(g) * u for rows [0, *rows_in_use); gu is [rows, 2*dff] with g in the left half.
template <typename T>
__global__ void __launch_bounds__(256)
swiglu_fwd_kernel(const T *__restrict__ gu, T *__restrict__ h, const int32_t *__restrict__ rows_in_use, int dff) {
    const int64_t vec = dff / 8, total = (int64_t)*rows_in_use * vec;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / vec, c = (i % vec) * 8;
        float g[8], u[8], o[8];
        load8(gu + r * 2 * dff + c, g);
        load8(gu + r * 2 * dff + dff + c, u);
#pragma unroll
        for (int j = 0; j < 8; j++) o[j] = silu_f32(g[j]) * u[j];
        store8(h + r * dff + c, o);
    }
}

// dg = (dh * u) * silu'(g), du = dh * silu(g); dgu is [rows, 2*dff] with dg in the left half.
template <typename T>
__global__ void __launch_bounds__(256)
swiglu_bwd_kernel(const T *__restrict__ dh, const T *__restrict__ gu, T *__restrict__ dgu,
                  const int32_t *__restrict__ rows_in_use, int dff) {
    const int64_t vec = dff / 8, total = (int64_t)*rows_in_use * vec;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / vec, c = (i % vec) * 8;
        float g[8], u[8], dv[8], dg[8], du[8];
        load8(gu + r * 2 * dff + c, g);
        load8(gu + r * 2 * dff + dff + c, u);
        load8(dh + r * dff + c, dv);
#pragma unroll
        for (int j = 0; j < 8; j++) {
            du[j] = dv[j] * silu_f32(g[j]);
            dg[j] = (dv[j] * u[j]) * silu_grad_f32(g[j]);
        }
        store8(dgu + r * 2 * dff + c, dg);
        store8(dgu + r * 2 * dff + dff + c, du);
    }
}

// ---- combine backward + router backward: one warp per token ---------------------------------------
// dyp[pos_j] = w_j * dy[t];  d w_j = <dy[t], yp[pos_j]>;  then lane 0 turns the k values d w into the
// E values d logits (gate renormalisation, softmax_back), serially and in index order like softmax_back itself.
// With expert parallelism the yp row is read from, and the dyp row written to, the buffers of the rank that
// owns the pick's expert (peer loads and stores); the last block to finish raises "rows have landed" on
// every rank, as the forward's dispatch does.
template <typename YT, typename OT>
__global__ void __launch_bounds__(256)
combine_bwd_kernel(const OT *__restrict__ dy, void *const *__restrict__ yp_table, void *const *__restrict__ dyp_table,
                   int e_local, EpSignal sig, int32_t *ticket, const int32_t *__restrict__ pos, const int32_t *__restrict__ topk_idx,
                   const float *__restrict__ topk_w, const float *__restrict__ logits, float *__restrict__ dgw,
                   float *__restrict__ dl, int T, int d, int k, int E, int renorm, float aux_c,
                   const int32_t *__restrict__ counts) {
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t < T) {
    float dw[kMaxTopK];
    for (int j = 0; j < k; j++) {
        const int r = pos[(size_t)t * k + j];
        const int q = topk_idx[(size_t)t * k + j] / e_local;  // rank that owns the pick's expert
        const YT *yp = static_cast<const YT *>(yp_table[q]);
        YT *dyp = static_cast<YT *>(dyp_table[q]);
        const float w = topk_w[(size_t)t * k + j];
        float acc = 0.f;
        // r < 0: the pick has no row (a refused expert-parallel step); nothing is read or written for it
        for (int c = lane * 8; r >= 0 && c < d; c += 256) {
            float a[8], y[8], o[8];
            load8(dy + (size_t)t * d + c, a);
            load8(yp + (size_t)r * d + c, y);
#pragma unroll
            for (int i = 0; i < 8; i++) {
                acc = fmaf(a[i], y[i], acc);
                o[i] = w * a[i];
            }
            store8(dyp + (size_t)r * d + c, o);
        }
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        dw[j] = acc;
    }
    if (lane == 0) {
        const float *lg = logits + (size_t)t * E;
        float *out = dl + (size_t)t * E;
        // softmax of the row, three passes (SoftmaxKernel.cu:5-24)
        float mx = lg[0];
        for (int e = 1; e < E; e++) mx = fmaxf(mx, lg[e]);
        float sum = 0.f;
        for (int e = 0; e < E; e++) sum += expf(lg[e] - mx);
        float ssum = 0.f, dot = 0.f;
        for (int j = 0; j < k; j++) {
            dgw[(size_t)t * k + j] = dw[j];
            ssum += expf(lg[topk_idx[(size_t)t * k + j]] - mx) / sum;
            dot += dw[j] * topk_w[(size_t)t * k + j];
        }
        // d p: the picks' terms, plus aux_c * f_e on every expert when the auxiliary loss is on (f_e = share
        // of the step's picks that went to e; aux_c = coef * E / T).  softmax_back: sum_i p_i dp_i, then
        // (dp_i - sum) * p_i.
        const float inv_picks = 1.0f / ((float)T * (float)k);
        float pd = 0.f;
        if (aux_c != 0.f)
            for (int e = 0; e < E; e++) pd += (expf(lg[e] - mx) / sum) * (aux_c * ((float)counts[e] * inv_picks));
        for (int j = 0; j < k; j++) {
            const float p = expf(lg[topk_idx[(size_t)t * k + j]] - mx) / sum;
            const float dp = renorm ? (dw[j] - dot) / ssum : dw[j];
            pd += p * dp;
        }
        for (int e = 0; e < E; e++) {
            const float a = aux_c != 0.f ? aux_c * ((float)counts[e] * inv_picks) : 0.f;
            out[e] = (a - pd) * (expf(lg[e] - mx) / sum);
        }
        for (int j = 0; j < k; j++) {
            const int e = topk_idx[(size_t)t * k + j];
            const float p = expf(lg[e] - mx) / sum;
            const float a = aux_c != 0.f ? aux_c * ((float)counts[e] * inv_picks) : 0.f;
            const float dp = (renorm ? (dw[j] - dot) / ssum : dw[j]) + a;
            out[e] = (dp - pd) * p;
        }
    }
    }  // t < T
    if (sig.flags != nullptr) {
        // make this block's rows visible system-wide, take a ticket, and let the last block tell every rank
        __threadfence_system();
        __syncthreads();
        __shared__ int s_last;
        if (threadIdx.x == 0) s_last = (atomicAdd(ticket, 1) == (int)gridDim.x - 1);
        __syncthreads();
        if (s_last && (int)threadIdx.x < sig.world) {
            __threadfence_system();
            uint32_t *f = sig.flags[threadIdx.x] + sig.rank;
            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(*sig.seq) : "memory");
        }
        if (s_last && threadIdx.x == 0) *ticket = 0;  // every block has arrived: zero for the next user
    }
}

// ps[e] = sum_t softmax(logits[t, :])[e]: one block per expert, threads stride the tokens, fixed tree at the end.
__global__ void __launch_bounds__(256)
prob_colsum_kernel(const float *__restrict__ logits, float *__restrict__ ps, int T, int E) {
    __shared__ float s[256];
    const int e = blockIdx.x;
    float acc = 0.f;
    for (int t = threadIdx.x; t < T; t += 256) {
        const float *lg = logits + (size_t)t * E;
        float mx = lg[0];
        for (int i = 1; i < E; i++) mx = fmaxf(mx, lg[i]);
        float sum = 0.f;
        for (int i = 0; i < E; i++) sum += expf(lg[i] - mx);
        acc += expf(lg[e] - mx) / sum;
    }
    s[threadIdx.x] = acc;
    __syncthreads();
    for (int o = 128; o >= 1; o >>= 1) {
        if ((int)threadIdx.x < o) s[threadIdx.x] += s[threadIdx.x + o];
        __syncthreads();
    }
    if (threadIdx.x == 0) ps[e] = s[0];
}

// dx[t] = ((dxp[pos_0] + dxp[pos_1]) + ...) + sum_e dl[t,e] * W_r[e,:]   (one warp per token)
// With expert parallelism the dxp rows are read from their owners' buffers once every owner has raised
// "outputs ready" for this step (bounded wait).
template <typename YT, typename OT>
__global__ void __launch_bounds__(256)
dx_kernel(void *const *__restrict__ dxp_table, int e_local, const int32_t *__restrict__ topk_idx, EpWait wait,
          int32_t *dev_err, const int32_t *__restrict__ pos, const float *__restrict__ dl,
          const float *__restrict__ w_r, OT *__restrict__ dx, int T, int d, int k, int E) {
    extern __shared__ float s_dl[];  // [warps][E]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.x * (blockDim.x >> 5) + warp;
    if (wait.flags != nullptr) {
        if ((int)threadIdx.x < wait.world) ep_wait_flag(wait.flags + threadIdx.x, *wait.seq, wait.timeout_ns, dev_err);
        __syncthreads();
    }
    if (t >= T) return;
    float *my = s_dl + warp * E;
    for (int e = lane; e < E; e += 32) my[e] = dl[(size_t)t * E + e];
    __syncwarp();
    for (int c = lane * 8; c < d; c += 256) {
        float acc[8];
        for (int j = 0; j < k; j++) {
            float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            const YT *dxp = static_cast<const YT *>(dxp_table[topk_idx[(size_t)t * k + j] / e_local]);
            const int r = pos[(size_t)t * k + j];
            if (r >= 0) load8(dxp + (size_t)r * d + c, v);  // r < 0: no row (a refused expert-parallel step)
#pragma unroll
            for (int i = 0; i < 8; i++) acc[i] = (j == 0) ? v[i] : acc[i] + v[i];
        }
        float r[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int e = 0; e < E; e++) {
            float w[8];
            load8(w_r + (size_t)e * d + c, w);
            const float g = my[e];
#pragma unroll
            for (int i = 0; i < 8; i++) r[i] = fmaf(g, w[i], r[i]);
        }
#pragma unroll
        for (int i = 0; i < 8; i++) acc[i] += r[i];
        store8(dx + (size_t)t * d + c, acc);
    }
}

// d W_router[e, c] = sum_t dl[t, e] * x[t, c].  A block owns 32 columns and one slice of the tokens; lane =
// column, warp w keeps the experts e = w, w+8, ...  Partials go to part[slice][E][d]; a second kernel adds
// the slices in order, so the sum has one fixed order.
template <typename XT, int EPW>
__global__ void __launch_bounds__(256)
dwr_partial_kernel(const XT *__restrict__ x, const float *__restrict__ dl, float *__restrict__ part, int T, int d,
                   int E, int slices) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int c = blockIdx.x * 32 + lane;
    const int per = (T + slices - 1) / slices;
    const int t0 = blockIdx.y * per, t1 = min(T, t0 + per);
    float acc[EPW];
#pragma unroll
    for (int i = 0; i < EPW; i++) acc[i] = 0.f;
    if (c < d) {
        for (int t = t0; t < t1; t++) {
            const float xv = ldf(x + (size_t)t * d + c);
#pragma unroll
            for (int i = 0; i < EPW; i++) {
                const int e = warp + 8 * i;
                if (e < E) acc[i] = fmaf(__ldg(dl + (size_t)t * E + e), xv, acc[i]);
            }
        }
#pragma unroll
        for (int i = 0; i < EPW; i++) {
            const int e = warp + 8 * i;
            if (e < E) part[((size_t)blockIdx.y * E + e) * d + c] = acc[i];
        }
    }
}

__global__ void __launch_bounds__(256)
dwr_reduce_kernel(const float *__restrict__ part, float *__restrict__ out, int n, int slices) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float acc = 0.f;
    for (int s = 0; s < slices; s++) acc += part[(size_t)s * n + i];
    out[i] = acc;
}

// d bias[e] = sum_t dl[t, e]: one block per expert, threads stride the tokens, fixed tree at the end.
__global__ void __launch_bounds__(256) dbias_kernel(const float *__restrict__ dl, float *__restrict__ out, int T, int E) {
    __shared__ float s[256];
    const int e = blockIdx.x;
    float acc = 0.f;
    for (int t = threadIdx.x; t < T; t += 256) acc += dl[(size_t)t * E + e];
    s[threadIdx.x] = acc;
    __syncthreads();
    for (int o = 128; o >= 1; o >>= 1) {
        if ((int)threadIdx.x < o) s[threadIdx.x] += s[threadIdx.x + o];
        __syncthreads();
    }
    if (threadIdx.x == 0) out[e] = s[0];
}

// Zero the padding rows of every expert's segment (rows [poffsets[e] + counts[e], poffsets[e+1])) of buf
// [rows, ld] (16-byte vectors; ld*sizeof(T) is a multiple of 16).  blockIdx.x = expert.
template <typename T>
__global__ void __launch_bounds__(256)
zero_pad_rows_kernel(T *__restrict__ buf, int ld, const int32_t *__restrict__ poffsets,
                     const int32_t *__restrict__ counts) {
    const int e = blockIdx.x;
    const int r0 = poffsets[e] + counts[e], r1 = poffsets[e + 1];
    const int vec_per_row = ld * (int)sizeof(T) / 16;
    const int64_t total = (int64_t)(r1 - r0) * vec_per_row;
    uint4 *base = reinterpret_cast<uint4 *>(buf + (size_t)r0 * ld);
    for (int64_t i = (int64_t)blockIdx.y * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.y * blockDim.x)
        base[i] = make_uint4(0u, 0u, 0u, 0u);
}

// ---- transposes (bf16 layers) ---------------------------------------------------------------------
// dst[c, r] = src[r, c] for the rows in use, r < *rows_in_use (a multiple of 128); rows of an expert's
// segment beyond its count are written as zeros, so a reduction over the padded segment adds nothing.
// src [rows, C] with leading dimension ld_src; dst [C, ld_dst].  64 x 64 tiles through shared memory.
__global__ void __launch_bounds__(256)
transpose_rows_kernel(const __nv_bfloat16 *__restrict__ src, int ld_src, __nv_bfloat16 *__restrict__ dst, int ld_dst,
                      int C, const int32_t *__restrict__ rows_in_use, const int32_t *__restrict__ tile_expert,
                      const int32_t *__restrict__ poffsets, const int32_t *__restrict__ counts) {
    __shared__ __nv_bfloat16 tile[64][66];
    const int r0 = blockIdx.x * 64, c0 = blockIdx.y * 64;
    if (r0 >= *rows_in_use) return;
    const int e = tile_expert[r0 / kRowAlign];
    const int valid_end = poffsets[e] + counts[e];  // rows of this segment at or beyond it are padding
    const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;  // 64 x 4
    for (int i = ty; i < 64; i += 4) {
        const int r = r0 + i, c = c0 + tx;
        tile[i][tx] = (r < valid_end && c < C) ? src[(size_t)r * ld_src + c] : __float2bfloat16_rn(0.f);
    }
    __syncthreads();
    for (int i = ty; i < 64; i += 4) {
        const int c = c0 + i, r = r0 + tx;
        if (c < C) dst[(size_t)c * ld_dst + r] = tile[tx][i];
    }
}

// Batched plain transpose: for each batch b, dst_b[c, r] = src_b[r, c]; src_b = src + b*R*C ([R, C]);
// dst_b = dst + b*dst_batch + dst_col0, leading dimension ld_dst.
__global__ void __launch_bounds__(256)
transpose_batched_kernel(const __nv_bfloat16 *__restrict__ src, __nv_bfloat16 *__restrict__ dst, int R, int C,
                         int ld_dst, size_t dst_batch, int dst_col0) {
    __shared__ __nv_bfloat16 tile[64][66];
    const __nv_bfloat16 *s = src + (size_t)blockIdx.z * R * C;
    __nv_bfloat16 *o = dst + (size_t)blockIdx.z * dst_batch + dst_col0;
    const int r0 = blockIdx.x * 64, c0 = blockIdx.y * 64;
    const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;
    for (int i = ty; i < 64; i += 4) {
        const int r = r0 + i, c = c0 + tx;
        if (r < R && c < C) tile[i][tx] = s[(size_t)r * C + c];
    }
    __syncthreads();
    for (int i = ty; i < 64; i += 4) {
        const int c = c0 + i, r = r0 + tx;
        if (c < C && r < R) o[(size_t)c * ld_dst + r] = tile[tx][i];
    }
}

// ---- fp32 products (parity-sized) -----------------------------------------------------------------
// Rows grouped by expert: C[r, n] (+)= sum_k A[r, k] * B_e(k, n) for the rows in use, where the expert of
// a row comes from its 128-row tile and B_e(k, n) = B[e*sbe + k*sbk + n*sbn].  64 x 64 tiles, 4 x 4 per thread.
__global__ void __launch_bounds__(256)
sgemm_rows_kernel(const float *__restrict__ A, int lda, const float *__restrict__ B, size_t sbe, int sbk, int sbn,
                  float *__restrict__ Cm, int ldc, int N, int K, const int32_t *__restrict__ rows_in_use,
                  const int32_t *__restrict__ tile_expert, int accumulate) {
    __shared__ float sa[16][65], sb[16][65];
    const int r0 = blockIdx.x * 64, n0 = blockIdx.y * 64;
    if (r0 >= *rows_in_use) return;
    const int e = tile_expert[r0 / kRowAlign];
    const float *Be = B + (size_t)e * sbe;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += 16) {
        for (int i = threadIdx.x; i < 64 * 16; i += 256) {
            const int kk = i & 15, m = i >> 4;
            sa[kk][m] = (k0 + kk < K) ? A[(size_t)(r0 + m) * lda + k0 + kk] : 0.f;
            const int n = n0 + m;
            sb[kk][m] = (k0 + kk < K && n < N) ? Be[(size_t)(k0 + kk) * sbk + (size_t)n * sbn] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 16; kk++) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; i++) { a[i] = sa[kk][ty * 4 + i]; b[i] = sb[kk][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
    for (int i = 0; i < 4; i++)
        for (int j = 0; j < 4; j++) {
            const int r = r0 + ty * 4 + i, n = n0 + tx * 4 + j;
            if (n < N) {
                float *p = Cm + (size_t)r * ldc + n;
                *p = accumulate ? *p + acc[i][j] : acc[i][j];
            }
        }
}

// Weight gradient of one expert (blockIdx.z): C_e[m, n] = sum over the expert's rows r of A[r, m] * B[r, n].
__global__ void __launch_bounds__(256)
sgemm_wgrad_kernel(const float *__restrict__ A, int lda, const float *__restrict__ B, int ldb, float *__restrict__ Cm,
                   int M, int N, const int32_t *__restrict__ poffsets, const int32_t *__restrict__ counts) {
    __shared__ float sa[16][65], sb[16][65];
    const int e = blockIdx.z, m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
    const int row0 = poffsets[e], cnt = counts[e];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < cnt; k0 += 16) {
        for (int i = threadIdx.x; i < 64 * 16; i += 256) {
            const int kk = i >> 6, m = i & 63;
            const bool in = k0 + kk < cnt;
            sa[kk][m] = (in && m0 + m < M) ? A[(size_t)(row0 + k0 + kk) * lda + m0 + m] : 0.f;
            sb[kk][m] = (in && n0 + m < N) ? B[(size_t)(row0 + k0 + kk) * ldb + n0 + m] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 16; kk++) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; i++) { a[i] = sa[kk][ty * 4 + i]; b[i] = sb[kk][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
    for (int i = 0; i < 4; i++)
        for (int j = 0; j < 4; j++) {
            const int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
            if (m < M && n < N) Cm[((size_t)e * M + m) * N + n] = acc[i][j];
        }
}

int grid_for(int64_t work_items, int sm_count) {
    int64_t b = (work_items + 255) / 256;
    const int64_t cap = (int64_t)sm_count * 8;
    return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

#define BW_TRY(expr)                                  \
    do {                                              \
        cudaError_t _e = (expr);                      \
        if (_e != cudaSuccess) return _e;             \
    } while (0)

template <typename CT>
cudaError_t forward_experts_t(omoe_handle *h, BwState *b, cudaStream_t s, int *n) {
    const int d = h->cfg.d_model, dff = h->cfg.d_ff, El = h->e_local;
    const int32_t *rows_in_use = h->ex_poffsets + El;
    CT *gu = static_cast<CT *>(b->gu);
    // padding rows hold rows of earlier steps: zero them, so that g, u and h are zero there too and a
    // reduction over a padded segment (the weight gradients) adds nothing
    zero_pad_rows_kernel<CT><<<dim3(El, 8), 256, 0, s>>>(static_cast<CT *>(h->xp), d, h->ex_poffsets, h->ex_counts);
    BW_TRY(cudaGetLastError());
    (*n)++;
    if constexpr (sizeof(CT) == 2) {
        BW_TRY(launch_grouped_plain(h, s, h->maps.a_x, h->maps.b_gate, b->m_g_out, dff, d));
        BW_TRY(launch_grouped_plain(h, s, h->maps.a_x, h->maps.b_up, b->m_u_out, dff, d));
    } else {
        dim3 grid((unsigned)(h->rows_cap / 64), (unsigned)ceil_div(dff, 64));
        const float *xp = static_cast<const float *>(h->xp);
        // g[r, f] = sum_c xp[r, c] * Wg[e][f][c]
        sgemm_rows_kernel<<<grid, 256, 0, s>>>(xp, d, static_cast<const float *>(h->w_gate), (size_t)dff * d, 1, d,
                                               reinterpret_cast<float *>(gu), 2 * dff, dff, d, rows_in_use,
                                               h->ex_tile_expert, 0);
        sgemm_rows_kernel<<<grid, 256, 0, s>>>(xp, d, static_cast<const float *>(h->w_up), (size_t)dff * d, 1, d,
                                               reinterpret_cast<float *>(gu) + dff, 2 * dff, dff, d, rows_in_use,
                                               h->ex_tile_expert, 0);
        BW_TRY(cudaGetLastError());
    }
    *n += 2;
    swiglu_fwd_kernel<CT><<<grid_for(h->rows_cap * (int64_t)dff / 8, h->sm_count), 256, 0, s>>>(
        gu, static_cast<CT *>(h->hbuf), rows_in_use, dff);
    BW_TRY(cudaGetLastError());
    (*n)++;
    if constexpr (sizeof(CT) == 2) {
        BW_TRY(launch_grouped_plain(h, s, h->maps.a_h, h->maps.b_down, h->maps.c_y, d, dff));
    } else {
        dim3 grid((unsigned)(h->rows_cap / 64), (unsigned)ceil_div(d, 64));
        // yp[r, c] = sum_f h[r, f] * Wd[e][c][f]
        sgemm_rows_kernel<<<grid, 256, 0, s>>>(static_cast<const float *>(h->hbuf), dff,
                                               static_cast<const float *>(h->w_down), (size_t)dff * d, 1, dff,
                                               static_cast<float *>(h->yp), d, d, dff, rows_in_use, h->ex_tile_expert,
                                               0);
        BW_TRY(cudaGetLastError());
    }
    (*n)++;
    return cudaSuccess;
}

cudaError_t transpose_weights(omoe_handle *h, BwState *b, cudaStream_t s, int *n) {
    const int d = h->cfg.d_model, dff = h->cfg.d_ff, El = h->e_local;
    auto *wg = static_cast<const __nv_bfloat16 *>(h->w_gate), *wu = static_cast<const __nv_bfloat16 *>(h->w_up);
    auto *wd = static_cast<const __nv_bfloat16 *>(h->w_down);
    // W_down [El][d][dff] -> wdT [El][dff][d]
    transpose_batched_kernel<<<dim3(ceil_div(d, 64), ceil_div(dff, 64), El), 256, 0, s>>>(
        wd, static_cast<__nv_bfloat16 *>(b->wdT), d, dff, d, (size_t)dff * d, 0);
    // W_gate, W_up [El][dff][d] -> wguT [El][d][2*dff] (gate in columns [0, dff), up in [dff, 2*dff))
    transpose_batched_kernel<<<dim3(ceil_div(dff, 64), ceil_div(d, 64), El), 256, 0, s>>>(
        wg, static_cast<__nv_bfloat16 *>(b->wguT), dff, d, 2 * dff, (size_t)d * 2 * dff, 0);
    transpose_batched_kernel<<<dim3(ceil_div(dff, 64), ceil_div(d, 64), El), 256, 0, s>>>(
        wu, static_cast<__nv_bfloat16 *>(b->wguT), dff, d, 2 * dff, (size_t)d * 2 * dff, dff);
    BW_TRY(cudaGetLastError());
    *n += 3;
    b->wt_valid = true;
    return cudaSuccess;
}

template <typename CT, typename OT>
cudaError_t backward_t(omoe_handle *h, BwState *b, const void *x, bool x_is_compute, const void *dy, void *dx, int T,
                       cudaStream_t s, int *n) {
    const int d = h->cfg.d_model, dff = h->cfg.d_ff, El = h->e_local, E = h->cfg.n_experts, k = h->cfg.top_k;
    const int32_t *rows_in_use = h->ex_poffsets + El;
    const int warps = 8, tblocks = ceil_div(T, warps);
    const bool ep = h->cfg.world > 1;
    EpSignal sig{nullptr, 1, 0, nullptr};
    if (ep) {
        BW_TRY(ep_bw_advance(h, s));  // the backward is a step of its own for the flags
        (*n)++;
        sig = ep_rows_signal(h);
    }
    if (T > 0) {
        combine_bwd_kernel<CT, OT><<<tblocks, 256, 0, s>>>(
            static_cast<const OT *>(dy), h->d_out_table, b->dyp_table, El, sig, h->ticket, h->pos, h->topk_idx,
            h->topk_w, h->logits, b->dgw, b->dl, T, d, k, E, h->cfg.renormalize,
            b->aux_coef != 0.f ? b->aux_coef * (float)E / (float)T : 0.f, h->counts);
        BW_TRY(cudaGetLastError());
    } else {
        BW_TRY(ep_signal_rows(h, s));  // no tokens here: nothing to send, but the owners wait for every rank
    }
    (*n)++;
    if (ep) {
        BW_TRY(ep_wait_rows(h, s));  // every rank's gradient rows for my experts have landed
        (*n)++;
    }
    zero_pad_rows_kernel<CT><<<dim3(El, 8), 256, 0, s>>>(static_cast<CT *>(b->dyp), d, h->ex_poffsets, h->ex_counts);
    BW_TRY(cudaGetLastError());
    (*n)++;
    const int ew_grid = grid_for(h->rows_cap * (int64_t)dff / 8, h->sm_count);
    if constexpr (sizeof(CT) == 2) {
        if (!b->wt_valid) BW_TRY(transpose_weights(h, b, s, n));
        // dh = dyp * W_down      (rows x d) * (d x dff): the forward's kernel on W_down^T
        BW_TRY(launch_grouped_plain(h, s, b->m_dyp_a, b->m_wdT_b, b->m_dh_c, dff, d));
        (*n)++;
        swiglu_bwd_kernel<CT><<<ew_grid, 256, 0, s>>>(static_cast<const CT *>(b->dh), static_cast<const CT *>(b->gu),
                                                      static_cast<CT *>(b->dgu), rows_in_use, dff);
        BW_TRY(cudaGetLastError());
        (*n)++;
        // dxp = [dg | du] * [W_gate ; W_up]: one product over K = 2*dff
        BW_TRY(launch_grouped_plain(h, s, b->m_dgu_a, b->m_wguT_b, b->m_dxp_c, d, 2 * dff));
        (*n)++;
        if (ep) {
            // the input-gradient rows are complete: the token ranks may fetch them while the weight gradients run
            BW_TRY(ep_signal_out(h, s));
            (*n)++;
        }
        // d W_down[e] [d, dff] = dyp_e^T * h_e;  [d W_gate ; d W_up][e] [2*dff, d] = [dg | du]_e^T * xp_e
        if (!b->wgrad_transposed) {
            // operands read in place as MN-major tiles; dyp's padding rows are zero, hence dh's and [dg|du]'s
            BW_TRY(launch_wgrad_bf16_rows(h, s, b->m_dyp_r, b->m_h_r, d, dff, d, b->d_down, b->d_down));
            BW_TRY(launch_wgrad_bf16_rows(h, s, b->m_dgu_r, b->m_xp_r, 2 * dff, d, dff, b->d_gate, b->d_up));
        } else {
            // transposed copies with each expert's padding rows zero-filled, then K-major operands
            auto tr = [&](const void *src, int ld, void *dst, int C) {
                transpose_rows_kernel<<<dim3((unsigned)(h->rows_cap / 64), (unsigned)ceil_div(C, 64)), 256, 0, s>>>(
                    static_cast<const __nv_bfloat16 *>(src), ld, static_cast<__nv_bfloat16 *>(dst), (int)h->rows_cap, C,
                    rows_in_use, h->ex_tile_expert, h->ex_poffsets, h->ex_counts);
                (*n)++;
            };
            tr(b->dyp, d, b->dypT, d);
            tr(h->hbuf, dff, b->hT, dff);
            tr(b->dgu, 2 * dff, b->dguT, 2 * dff);
            tr(h->xp, d, b->xpT, d);
            BW_TRY(cudaGetLastError());
            BW_TRY(launch_wgrad_bf16(h, s, b->m_dypT, b->m_hT, d, dff, d, b->d_down, b->d_down));
            BW_TRY(launch_wgrad_bf16(h, s, b->m_dguT, b->m_xpT, 2 * dff, d, dff, b->d_gate, b->d_up));
        }
        *n += 2;
    } else {
        const float *dyp = static_cast<const float *>(b->dyp);
        float *dgu = static_cast<float *>(b->dgu);
        dim3 g1((unsigned)(h->rows_cap / 64), (unsigned)ceil_div(dff, 64));
        // dh[r, f] = sum_c dyp[r, c] * Wd[e][c][f]
        sgemm_rows_kernel<<<g1, 256, 0, s>>>(dyp, d, static_cast<const float *>(h->w_down), (size_t)dff * d, dff, 1,
                                             static_cast<float *>(b->dh), dff, dff, d, rows_in_use, h->ex_tile_expert,
                                             0);
        swiglu_bwd_kernel<CT><<<ew_grid, 256, 0, s>>>(static_cast<const CT *>(b->dh), static_cast<const CT *>(b->gu),
                                                      static_cast<CT *>(b->dgu), rows_in_use, dff);
        dim3 g2((unsigned)(h->rows_cap / 64), (unsigned)ceil_div(d, 64));
        // dxp[r, c] = sum_f dg[r, f] * Wg[e][f][c] + sum_f du[r, f] * Wu[e][f][c]
        sgemm_rows_kernel<<<g2, 256, 0, s>>>(dgu, 2 * dff, static_cast<const float *>(h->w_gate), (size_t)dff * d, d, 1,
                                             static_cast<float *>(b->dxp), d, d, dff, rows_in_use, h->ex_tile_expert, 0);
        sgemm_rows_kernel<<<g2, 256, 0, s>>>(dgu + dff, 2 * dff, static_cast<const float *>(h->w_up), (size_t)dff * d,
                                             d, 1, static_cast<float *>(b->dxp), d, d, dff, rows_in_use,
                                             h->ex_tile_expert, 1);
        if (ep) {
            BW_TRY(ep_signal_out(h, s));
            (*n)++;
        }
        // d W_down[e][c][f] = sum_r dyp[r, c] * h[r, f];  d W_gate[e][f][c] = sum_r dg[r, f] * xp[r, c]
        sgemm_wgrad_kernel<<<dim3(ceil_div(dff, 64), ceil_div(d, 64), El), 256, 0, s>>>(
            dyp, d, static_cast<const float *>(h->hbuf), dff, b->d_down, d, dff, h->ex_poffsets, h->ex_counts);
        sgemm_wgrad_kernel<<<dim3(ceil_div(d, 64), ceil_div(dff, 64), El), 256, 0, s>>>(
            dgu, 2 * dff, static_cast<const float *>(h->xp), d, b->d_gate, dff, d, h->ex_poffsets, h->ex_counts);
        sgemm_wgrad_kernel<<<dim3(ceil_div(d, 64), ceil_div(dff, 64), El), 256, 0, s>>>(
            dgu + dff, 2 * dff, static_cast<const float *>(h->xp), d, b->d_up, dff, d, h->ex_poffsets, h->ex_counts);
        BW_TRY(cudaGetLastError());
        *n += 7;
    }
    // router: d W_router = dl^T * x, d bias = column sums of dl
    {
        const int slices = b->dwr_slices;
        dim3 grid((unsigned)ceil_div(d, 32), (unsigned)slices);
        auto run = [&](auto *xr) {
            using XT = typename std::remove_cv<typename std::remove_pointer<decltype(xr)>::type>::type;
            if (E <= 8) dwr_partial_kernel<XT, 1><<<grid, 256, 0, s>>>(xr, b->dl, b->dwr_part, T, d, E, slices);
            else if (E <= 16) dwr_partial_kernel<XT, 2><<<grid, 256, 0, s>>>(xr, b->dl, b->dwr_part, T, d, E, slices);
            else if (E <= 32) dwr_partial_kernel<XT, 4><<<grid, 256, 0, s>>>(xr, b->dl, b->dwr_part, T, d, E, slices);
            else if (E <= 64) dwr_partial_kernel<XT, 8><<<grid, 256, 0, s>>>(xr, b->dl, b->dwr_part, T, d, E, slices);
            else dwr_partial_kernel<XT, 16><<<grid, 256, 0, s>>>(xr, b->dl, b->dwr_part, T, d, E, slices);
        };
        // x: the rows the router saw (the caller's rows, or the normalised rows of the block form)
        if (x_is_compute) run(static_cast<const CT *>(x));
        else run(static_cast<const OT *>(x));
        dwr_reduce_kernel<<<ceil_div(E * d, 256), 256, 0, s>>>(b->dwr_part, b->d_router, E * d, slices);
        dbias_kernel<<<E, 256, 0, s>>>(b->dl, b->d_bias, T, E);
        BW_TRY(cudaGetLastError());
        *n += 3;
    }
    if (T > 0) {
        const EpWait wt = ep ? ep_out_wait(h) : EpWait{nullptr, 1, nullptr, 0};
        dx_kernel<CT, OT><<<tblocks, 256, warps * E * sizeof(float), s>>>(
            b->dxp_table, El, h->topk_idx, wt, h->dev_err, h->pos, b->dl, h->w_router, static_cast<OT *>(dx), T, d, k, E);
        BW_TRY(cudaGetLastError());
        (*n)++;
    }
    return cudaSuccess;
}

void free_state(BwState *b) {
    if (!b->own_grad_rows) b->dyp = b->dxp = nullptr, b->dyp_table = b->dxp_table = nullptr;
    void *ptrs[] = {b->dyp_table, b->dxp_table, b->gu, b->dyp, b->dh, b->dgu, b->dxp, b->dgw, b->dl, b->dwr_part, b->wdT, b->wguT, b->xpT, b->hT,
                    b->dypT, b->dguT, b->d_router, b->d_bias, b->d_gate, b->d_up, b->d_down, b->aux_ps, b->dxn, b->inv_rms};
    for (void *p : ptrs)
        if (p) cudaFree(p);
    delete b;
}

}  // namespace

int bw_set_training(omoe_handle *h, int on) {
    BwState *b = static_cast<BwState *>(h->bw);
    if (!on) {
        if (b) { b->training = false; b->fwd_valid = false; }
        return OMOE_OK;
    }
    if (b) { b->training = true; return OMOE_OK; }
    b = new (std::nothrow) BwState();
    if (!b) return OMOE_ERR_NOMEM;
    memset(b, 0, sizeof(*b));
    const size_t cs = h->cfg.compute_dtype == OMOE_BF16 ? 2 : 4;
    const size_t rows = (size_t)h->rows_cap, d = h->cfg.d_model, dff = h->cfg.d_ff, El = h->e_local;
    const size_t E = h->cfg.n_experts, tm = h->cfg.t_max, k = h->cfg.top_k;
    b->dwr_slices = (int)(tm >= 4096 ? 64 : (tm >= 256 ? 8 : 1));
    struct { void **p; size_t bytes; } bufs[] = {
        {&b->gu, rows * 2 * dff * cs}, {&b->dh, rows * dff * cs},
        {&b->dgu, rows * 2 * dff * cs}, {(void **)&b->dgw, tm * k * 4},
        {(void **)&b->dl, tm * E * 4}, {(void **)&b->dwr_part, (size_t)b->dwr_slices * E * d * 4},
        {(void **)&b->d_router, E * d * 4}, {(void **)&b->d_bias, E * 4}, {(void **)&b->aux_ps, E * 4}, {(void **)&b->d_gate, El * dff * d * 4},
        {(void **)&b->d_up, El * dff * d * 4}, {(void **)&b->d_down, El * dff * d * 4}};
    bool ok = true;
    for (auto &x : bufs) ok = ok && cudaMalloc(x.p, x.bytes ? x.bytes : 1) == cudaSuccess;
    if (h->cfg.world > 1) {
        // gradient rows cross GPUs: the buffers the peers can reach belong to the transport
        ep_grad_buffers(h, &b->dyp, &b->dxp, &b->dyp_table, &b->dxp_table);
        b->own_grad_rows = false;
    } else {
        b->own_grad_rows = true;
        ok = ok && cudaMalloc(&b->dyp, rows * d * cs) == cudaSuccess && cudaMalloc(&b->dxp, rows * d * cs) == cudaSuccess &&
             cudaMalloc(&b->dyp_table, sizeof(void *)) == cudaSuccess &&
             cudaMalloc(&b->dxp_table, sizeof(void *)) == cudaSuccess;
        if (ok) {
            cudaMemcpy(b->dyp_table, &b->dyp, sizeof(void *), cudaMemcpyHostToDevice);
            cudaMemcpy(b->dxp_table, &b->dxp, sizeof(void *), cudaMemcpyHostToDevice);
        }
    }
    const char *wt = getenv("OMOE_WGRAD_TRANSPOSED");
    b->wgrad_transposed = wt && atoi(wt) != 0;
    if (ok && cs == 2) {
        struct { void **p; size_t bytes; } tb[] = {{&b->wdT, El * dff * d * 2}, {&b->wguT, El * d * 2 * dff * 2}};
        for (auto &x : tb) ok = ok && cudaMalloc(x.p, x.bytes) == cudaSuccess;
    }
    if (ok && cs == 2 && b->wgrad_transposed) {
        struct { void **p; size_t bytes; } tb[] = {{&b->xpT, d * rows * 2}, {&b->hT, dff * rows * 2},
                                                   {&b->dypT, d * rows * 2}, {&b->dguT, 2 * dff * rows * 2}};
        for (auto &x : tb) ok = ok && cudaMalloc(x.p, x.bytes) == cudaSuccess;
    }
    if (!ok) {
        cudaGetLastError();
        free_state(b);
        snprintf(h->err, sizeof(h->err), "omoe_set_training: device allocation of the backward buffers failed");
        return OMOE_ERR_NOMEM;
    }
    // padding rows are read by the row-wise products (their results are never used): keep them finite
    cudaMemset(b->gu, 0, rows * 2 * dff * cs);
    if (b->own_grad_rows) cudaMemset(b->dyp, 0, rows * d * cs);
    cudaMemset(b->dgu, 0, rows * 2 * dff * cs);
    if (cs == 2) {
        // columns of the transposed buffers beyond the rows in use are never read
        bool m = encode_map_bf16(&b->m_g_out, b->gu, rows, dff, 2 * dff, 128) &&
                 encode_map_bf16(&b->m_u_out, static_cast<__nv_bfloat16 *>(b->gu) + dff, rows, dff, 2 * dff, 128) &&
                 encode_map_bf16(&b->m_dyp_a, b->dyp, rows, d, d, 128) &&
                 encode_map_bf16(&b->m_wdT_b, b->wdT, El * dff, d, d, 128) &&
                 encode_map_bf16(&b->m_dh_c, b->dh, rows, dff, dff, 128) &&
                 encode_map_bf16(&b->m_dgu_a, b->dgu, rows, 2 * dff, 2 * dff, 128) &&
                 encode_map_bf16(&b->m_wguT_b, b->wguT, El * d, 2 * dff, 2 * dff, 128) &&
                 encode_map_bf16(&b->m_dxp_c, b->dxp, rows, d, d, 128) &&
                 encode_map_bf16(&b->m_dyp_r, b->dyp, rows, d, d, 64) &&
                 encode_map_bf16(&b->m_h_r, h->hbuf, rows, dff, dff, 64) &&
                 encode_map_bf16(&b->m_dgu_r, b->dgu, rows, 2 * dff, 2 * dff, 64) &&
                 encode_map_bf16(&b->m_xp_r, h->xp, rows, d, d, 64);
        if (m && b->wgrad_transposed)
            m = encode_map_bf16(&b->m_dypT, b->dypT, d, rows, rows, 128) &&
                encode_map_bf16(&b->m_hT, b->hT, dff, rows, rows, 128) &&
                encode_map_bf16(&b->m_dguT, b->dguT, 2 * dff, rows, rows, 128) &&
                encode_map_bf16(&b->m_xpT, b->xpT, d, rows, rows, 128);
        if (!m) {
            free_state(b);
            snprintf(h->err, sizeof(h->err), "omoe_set_training: cuTensorMapEncodeTiled failed");
            return OMOE_ERR_CUDA;
        }
    }
    if (cudaDeviceSynchronize() != cudaSuccess) {
        free_state(b);
        return OMOE_ERR_CUDA;
    }
    b->training = true;
    h->bw = b;
    return OMOE_OK;
}

bool bw_training(const omoe_handle *h) { return h->bw && static_cast<BwState *>(h->bw)->training; }

void bw_weights_changed(omoe_handle *h) {
    if (h->bw) static_cast<BwState *>(h->bw)->wt_valid = false;
}

void bw_forward_invalidate(omoe_handle *h) {
    if (h->bw) static_cast<BwState *>(h->bw)->fwd_valid = false;
}

void bw_forward_empty(omoe_handle *h) {
    BwState *b = static_cast<BwState *>(h->bw);
    if (b && b->training) {
        b->fwd_valid = true;
        b->fwd_T = 0;
    }
}

cudaError_t bw_forward_experts(omoe_handle *h, int T, cudaStream_t s, int *n) {
    BwState *b = static_cast<BwState *>(h->bw);
    cudaError_t e = h->cfg.compute_dtype == OMOE_BF16 ? forward_experts_t<__nv_bfloat16>(h, b, s, n)
                                                      : forward_experts_t<float>(h, b, s, n);
    b->fwd_valid = e == cudaSuccess;
    b->fwd_T = T;
    return e;
}

int bw_backward(omoe_handle *h, const void *x, bool x_is_compute, const void *dy, void *dx, int T, int io_dtype,
                cudaStream_t s, int *launches) {
    BwState *b = static_cast<BwState *>(h->bw);
    if (!b || !b->training) {
        snprintf(h->err, sizeof(h->err), "omoe_backward: call omoe_set_training(h, 1) and a forward first");
        return OMOE_ERR_STATE;
    }
    if (h->cfg.world > 1 && !ep_ready(h)) {
        snprintf(h->err, sizeof(h->err), "omoe_backward: call omoe_ep_export / omoe_ep_import on every rank first");
        return OMOE_ERR_STATE;
    }
    if (!b->fwd_valid || b->fwd_T != T) {
        snprintf(h->err, sizeof(h->err), "omoe_backward: no training-mode forward of T=%d rows precedes this call", T);
        return OMOE_ERR_STATE;
    }
    if (T == 0 && h->cfg.world == 1) {  // no rows: every gradient is zero
        const size_t E = h->cfg.n_experts, d = h->cfg.d_model, dff = h->cfg.d_ff, El = h->e_local;
        cudaMemsetAsync(b->d_router, 0, E * d * 4, s);
        cudaMemsetAsync(b->d_bias, 0, E * 4, s);
        cudaMemsetAsync(b->d_gate, 0, El * dff * d * 4, s);
        cudaMemsetAsync(b->d_up, 0, El * dff * d * 4, s);
        cudaMemsetAsync(b->d_down, 0, El * dff * d * 4, s);
        return OMOE_OK;
    }
    cudaError_t e;
    if (h->cfg.compute_dtype == OMOE_BF16)
        e = io_dtype == OMOE_BF16 ? backward_t<__nv_bfloat16, __nv_bfloat16>(h, b, x, x_is_compute, dy, dx, T, s, launches)
                                  : backward_t<__nv_bfloat16, float>(h, b, x, x_is_compute, dy, dx, T, s, launches);
    else
        e = backward_t<float, float>(h, b, x, x_is_compute, dy, dx, T, s, launches);
    if (e != cudaSuccess) {
        snprintf(h->err, sizeof(h->err), "omoe_backward: %s", cudaGetErrorString(e));
        return OMOE_ERR_CUDA;
    }
    // Expert parallel: one backward per forward.  The owners raise "outputs ready" before their weight-gradient
    // kernels, which still read the gradient rows; only the next forward's count exchange orders the peers
    // behind those kernels, so a second backward could overwrite rows that are still being read.
    if (h->cfg.world > 1) b->fwd_valid = false;
    return OMOE_OK;
}

int bw_get_grads(omoe_handle *h, float *d_router, float *d_bias, float *d_gate, float *d_up, float *d_down,
                 cudaStream_t s) {
    BwState *b = static_cast<BwState *>(h->bw);
    if (!b) {
        snprintf(h->err, sizeof(h->err), "omoe_get_weight_grads: no backward has run");
        return OMOE_ERR_STATE;
    }
    const size_t E = h->cfg.n_experts, d = h->cfg.d_model, dff = h->cfg.d_ff, El = h->e_local;
    struct { float *dst; const float *src; size_t n; } cp[] = {
        {d_router, b->d_router, E * d}, {d_bias, b->d_bias, E}, {d_gate, b->d_gate, El * dff * d},
        {d_up, b->d_up, El * dff * d}, {d_down, b->d_down, El * dff * d}};
    for (auto &c : cp)
        if (c.dst && cudaMemcpyAsync(c.dst, c.src, c.n * 4, cudaMemcpyDefault, s) != cudaSuccess) {
            snprintf(h->err, sizeof(h->err), "omoe_get_weight_grads: copy failed");
            return OMOE_ERR_CUDA;
        }
    if (cudaStreamSynchronize(s) != cudaSuccess) return OMOE_ERR_CUDA;
    return OMOE_OK;
}

namespace {

// RMSNorm backward of one row per warp, after rmsnorm_backward_kernel2 (src/main/resources/cu/RMSKernel.cu:225-275):
//   rms = sqrtf(sum(x^2)/C + eps);  drms = sum(x * dout * w) * (-1 / (rms^3 * C));
//   dinp = dout * w / rms + drms * x.
// Here dx = dy + dinp (the residual branch of the block adds dy itself) and 1/rms is kept per row for the
// weight gradient, which the reference accumulates with atomics and this build sums in a fixed order.
template <typename OT>
__global__ void __launch_bounds__(256)
rmsnorm_bwd_kernel(const OT *__restrict__ x, const float *__restrict__ gamma, const OT *__restrict__ dxn,
                   const OT *__restrict__ dy, OT *__restrict__ dx, float *__restrict__ inv_rms, float eps, int T,
                   int d) {
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= T) return;
    const OT *xr = x + (size_t)t * d, *gr = dxn + (size_t)t * d;
    float ss = 0.f, dot = 0.f;
    for (int c = lane * 8; c < d; c += 256) {
        float xv[8], gv[8], wv[8];
        load8(xr + c, xv);
        load8(gr + c, gv);
        load8(gamma + c, wv);
#pragma unroll
        for (int i = 0; i < 8; i++) {
            ss = fmaf(xv[i], xv[i], ss);
            dot = fmaf(xv[i] * gv[i], wv[i], dot);
        }
    }
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) {
        ss += __shfl_xor_sync(0xffffffffu, ss, o);
        dot += __shfl_xor_sync(0xffffffffu, dot, o);
    }
    const float rms = sqrtf(ss / (float)d + eps);
    const float drms = dot * (-1.0f / (rms * rms * rms * (float)d));
    if (lane == 0) inv_rms[t] = 1.0f / rms;
    for (int c = lane * 8; c < d; c += 256) {
        float xv[8], gv[8], wv[8], dv[8], o[8];
        load8(xr + c, xv);
        load8(gr + c, gv);
        load8(gamma + c, wv);
        load8(dy + (size_t)t * d + c, dv);
#pragma unroll
        for (int i = 0; i < 8; i++) o[i] = dv[i] + (gv[i] * wv[i] / rms + drms * xv[i]);
        store8(dx + (size_t)t * d + c, o);
    }
}

// d gamma[c] = sum_t (x[t,c] / rms_t) * dxn[t,c]: thread = column, blockIdx.y = slice of the tokens;
// partials [slices][d] are added in order by dwr_reduce_kernel.
template <typename OT>
__global__ void __launch_bounds__(256)
dgamma_partial_kernel(const OT *__restrict__ x, const OT *__restrict__ dxn, const float *__restrict__ inv_rms,
                      float *__restrict__ part, int T, int d, int slices) {
    const int c = blockIdx.x * 256 + threadIdx.x;
    if (c >= d) return;
    const int per = (T + slices - 1) / slices;
    const int t0 = blockIdx.y * per, t1 = min(T, t0 + per);
    float acc = 0.f;
    for (int t = t0; t < t1; t++) acc = fmaf(ldf(x + (size_t)t * d + c) * inv_rms[t], ldf(dxn + (size_t)t * d + c), acc);
    part[(size_t)blockIdx.y * d + c] = acc;
}

template <typename OT>
cudaError_t block_tail_t(omoe_handle *h, BwState *b, const void *x, const float *gamma, float eps, const void *dy,
                         void *dx, float *dgamma, int T, cudaStream_t s, int *n) {
    const int d = h->cfg.d_model, slices = b->dwr_slices;
    if (T > 0)
        rmsnorm_bwd_kernel<OT><<<ceil_div(T, 8), 256, 0, s>>>(static_cast<const OT *>(x), gamma,
                                                             static_cast<const OT *>(b->dxn),
                                                             static_cast<const OT *>(dy), static_cast<OT *>(dx),
                                                             b->inv_rms, eps, T, d);
    // the partial buffer of the router's weight gradient is free again by now ([slices][E][d] >= [slices][d])
    dgamma_partial_kernel<OT><<<dim3(ceil_div(d, 256), slices), 256, 0, s>>>(
        static_cast<const OT *>(x), static_cast<const OT *>(b->dxn), b->inv_rms, b->dwr_part, T, d, slices);
    dwr_reduce_kernel<<<ceil_div(d, 256), 256, 0, s>>>(b->dwr_part, dgamma, d, slices);
    BW_TRY(cudaGetLastError());
    *n += 3;
    return cudaSuccess;
}

}  // namespace

// Backward of y = x + MoE(rmsnorm(x) * gamma): the layer's backward on the normalised rows the forward kept,
// then the RMSNorm backward, with the residual branch's dy added in the same pass.
int bw_backward_block(omoe_handle *h, const void *x, const float *gamma, float eps, const void *dy, void *dx,
                      float *dgamma, int T, int io_dtype, cudaStream_t s, int *launches) {
    BwState *b = static_cast<BwState *>(h->bw);
    if (!b || !b->training) {
        snprintf(h->err, sizeof(h->err), "omoe_backward_block: call omoe_set_training(h, 1) and a forward first");
        return OMOE_ERR_STATE;
    }
    if (!b->dxn) {
        const size_t bytes = (size_t)h->cfg.t_max * h->cfg.d_model * 4;
        if (cudaMalloc(&b->dxn, bytes) != cudaSuccess || cudaMalloc(&b->inv_rms, (size_t)h->cfg.t_max * 4) != cudaSuccess) {
            cudaGetLastError();
            snprintf(h->err, sizeof(h->err), "omoe_backward_block: device allocation failed");
            return OMOE_ERR_NOMEM;
        }
    }
    int rc = bw_backward(h, h->xn, true, dy, b->dxn, T, io_dtype, s, launches);
    if (rc != OMOE_OK) return rc;
    cudaError_t e = io_dtype == OMOE_BF16
                        ? block_tail_t<__nv_bfloat16>(h, b, x, gamma, eps, dy, dx, dgamma, T, s, launches)
                        : block_tail_t<float>(h, b, x, gamma, eps, dy, dx, dgamma, T, s, launches);
    if (e != cudaSuccess) {
        snprintf(h->err, sizeof(h->err), "omoe_backward_block: %s", cudaGetErrorString(e));
        return OMOE_ERR_CUDA;
    }
    return OMOE_OK;
}

int bw_set_aux(omoe_handle *h, float coef) {
    BwState *b = static_cast<BwState *>(h->bw);
    if (!b) {
        snprintf(h->err, sizeof(h->err), "omoe_set_aux_loss: switch training mode on first");
        return OMOE_ERR_STATE;
    }
    b->aux_coef = coef;
    return OMOE_OK;
}

int bw_aux_loss(omoe_handle *h, float *loss_host, cudaStream_t s) {
    BwState *b = static_cast<BwState *>(h->bw);
    if (!b) {
        snprintf(h->err, sizeof(h->err), "omoe_get_aux_loss: switch training mode on first");
        return OMOE_ERR_STATE;
    }
    const int T = h->last_T, E = h->cfg.n_experts, k = h->cfg.top_k;
    *loss_host = 0.f;
    if (T == 0) return OMOE_OK;
    prob_colsum_kernel<<<E, 256, 0, s>>>(h->logits, b->aux_ps, T, E);
    float ps[kMaxExperts];
    int32_t cnt[kMaxExperts];
    if (cudaGetLastError() != cudaSuccess ||
        cudaMemcpyAsync(ps, b->aux_ps, sizeof(float) * E, cudaMemcpyDeviceToHost, s) != cudaSuccess ||
        cudaMemcpyAsync(cnt, h->counts, sizeof(int32_t) * E, cudaMemcpyDeviceToHost, s) != cudaSuccess ||
        cudaStreamSynchronize(s) != cudaSuccess) {
        snprintf(h->err, sizeof(h->err), "omoe_get_aux_loss: CUDA error");
        return OMOE_ERR_CUDA;
    }
    float loss = 0.f;
    for (int e = 0; e < E; e++) loss += ((float)cnt[e] / ((float)T * (float)k)) * (ps[e] / (float)T);
    *loss_host = (float)E * loss;
    return OMOE_OK;
}

void bw_destroy(omoe_handle *h) {
    if (h->bw) free_state(static_cast<BwState *>(h->bw));
    h->bw = nullptr;
}

}  // namespace omoe
