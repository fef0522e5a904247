// Self-checking build (-DOMOE_BOUNDS_CHECK, libomoe_check.so): what a memory checker would look for, done by the
// library itself.  Before every one-GPU forward the dispatch, hidden and expert-output buffers are filled with
// the all-ones byte pattern (a NaN in bf16 and fp32), so a read of a row that the step never wrote shows up as
// NaN in the output; after the dispatch a kernel validates every routing index against its bounds (experts,
// row positions inside their expert's segment, counts and offsets consistent, 128-row alignment, the tile
// table) and checks that the padding rows of the dispatch buffer still hold the fill pattern (nothing wrote
// outside the rows in use).  Failures raise the bounds bit of the device error word, which the next
// synchronising call reports as OMOE_ERR_DEVICE.  The product build compiles none of this.
#ifdef OMOE_BOUNDS_CHECK
#include "common.cuh"

namespace omoe {

namespace {

__global__ void __launch_bounds__(256)
check_routing_kernel(const int32_t *__restrict__ topk_idx, const float *__restrict__ topk_w,
                     const int32_t *__restrict__ pos, const int32_t *__restrict__ counts,
                     const int32_t *__restrict__ offsets, const int32_t *__restrict__ poffsets,
                     const int32_t *__restrict__ tile_expert, int T, int k, int E, int rows_cap, int renorm,
                     int32_t *dev_err) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    bool ok = true;
    if (t < T) {
        float wsum = 0.f;
        for (int j = 0; j < k; j++) {
            const int e = topk_idx[(size_t)t * k + j];
            const float w = topk_w[(size_t)t * k + j];
            const int p = pos[(size_t)t * k + j];
            ok = ok && e >= 0 && e < E;
            ok = ok && w >= 0.f && w <= 1.0001f;   // also false for NaN
            if (e >= 0 && e < E) ok = ok && p >= poffsets[e] && p < poffsets[e] + counts[e] && p < rows_cap;
            for (int i = 0; i < j; i++) ok = ok && topk_idx[(size_t)t * k + i] != e;   // an expert is picked once
            wsum += w;
        }
        if (renorm) ok = ok && fabsf(wsum - 1.0f) < 1e-4f;
    }
    if (t == 0) {
        int off = 0, poff = 0;
        for (int e = 0; e < E; e++) {
            ok = ok && counts[e] >= 0 && offsets[e] == off && poffsets[e] == poff && poff % kRowAlign == 0;
            off += counts[e];
            poff += (counts[e] + kRowAlign - 1) / kRowAlign * kRowAlign;
        }
        ok = ok && off == T * k && offsets[E] == off && poffsets[E] == poff && poff <= rows_cap;
        for (int i = 0; i < rows_cap / kRowAlign; i++) {
            const int ex = tile_expert[i];
            if (i * kRowAlign < poff) ok = ok && ex >= 0 && ex < E && poffsets[ex] <= i * kRowAlign && i * kRowAlign < poffsets[ex + 1];
            else ok = ok && ex == -1;
        }
    }
    if (!ok) atomicOr(dev_err, kDevErrBounds);
}

// One warp per row of the dispatch buffer: rows in use hold no fill pattern, every other row holds nothing else.
__global__ void __launch_bounds__(256)
check_rows_kernel(const uint32_t *__restrict__ xp, int row_words, const int32_t *__restrict__ counts,
                  const int32_t *__restrict__ poffsets, int E, int rows_cap, int32_t *dev_err) {
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= rows_cap) return;
    bool used = false;
    for (int e = 0; e < E; e++) used = used || (row >= poffsets[e] && row < poffsets[e] + counts[e]);
    bool ok = true;
    for (int w = lane; w < row_words; w += 32) {
        const uint32_t v = xp[(size_t)row * row_words + w];
        ok = ok && (used ? v != 0xffffffffu : v == 0xffffffffu);
    }
    if (!ok) atomicOr(dev_err, kDevErrBounds);
}

}  // namespace

cudaError_t check_fill(omoe_handle *h, cudaStream_t s) {
    const size_t cs = h->cfg.compute_dtype == OMOE_BF16 ? 2 : 4;
    cudaError_t e = cudaMemsetAsync(h->xp, 0xff, (size_t)h->rows_cap * h->cfg.d_model * cs, s);
    if (e == cudaSuccess) e = cudaMemsetAsync(h->hbuf, 0xff, (size_t)h->rows_cap * h->cfg.d_ff * cs, s);
    if (e == cudaSuccess) e = cudaMemsetAsync(h->yp, 0xff, (size_t)h->rows_cap * h->cfg.d_model * cs, s);
    return e;
}

cudaError_t check_after_dispatch(omoe_handle *h, int T, cudaStream_t s) {
    const size_t cs = h->cfg.compute_dtype == OMOE_BF16 ? 2 : 4;
    check_routing_kernel<<<ceil_div(T, 256), 256, 0, s>>>(h->topk_idx, h->topk_w, h->pos, h->counts, h->offsets,
                                                          h->poffsets, h->tile_expert, T, h->cfg.top_k,
                                                          h->cfg.n_experts, (int)h->rows_cap, h->cfg.renormalize,
                                                          h->dev_err);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    check_rows_kernel<<<ceil_div((int)h->rows_cap, 8), 256, 0, s>>>(static_cast<const uint32_t *>(h->xp),
                                                                   (int)(h->cfg.d_model * cs / 4), h->counts,
                                                                   h->poffsets, h->cfg.n_experts, (int)h->rows_cap,
                                                                   h->dev_err);
    return cudaGetLastError();
}

}  // namespace omoe

// Rows [first, first + n) of the dispatch buffer (which = 0), the hidden rows (1) or the expert outputs (2) of
// the last forward, in the layer's compute dtype, to a host buffer.  Exists in the self-checking build only, so
// a test can compare every intermediate with a CPU restatement.
extern "C" __attribute__((visibility("default"))) int omoe_check_read_rows(omoe_handle *h, int which, void *dst_host,
                                                                           long first, long n) {
    if (!h || !dst_host || which < 0 || which > 2 || first < 0 || n < 0 || first + n > h->rows_cap) return OMOE_ERR_INVALID;
    const size_t cs = h->cfg.compute_dtype == OMOE_BF16 ? 2 : 4;
    const size_t width = which == 1 ? h->cfg.d_ff : h->cfg.d_model;
    const char *src = static_cast<const char *>(which == 0 ? h->xp : (which == 1 ? h->hbuf : h->yp));
    if (cudaStreamSynchronize(h->last_stream) != cudaSuccess) return OMOE_ERR_CUDA;
    return cudaMemcpy(dst_host, src + (size_t)first * width * cs, (size_t)n * width * cs, cudaMemcpyDeviceToHost) ==
                   cudaSuccess
               ? OMOE_OK
               : OMOE_ERR_CUDA;
}
#endif  // OMOE_BOUNDS_CHECK
