// Gate-weighted combine: y[t,:] = ((w0*yp[p0,:]) + w1*yp[p1,:]) + ... in pick
// order with fp32 accumulation, reading every expert output row exactly once
// and holding the k gate weights and row positions in registers.
//
// No reference kernel exists for this stage; the nearest idiom is the
// accumulate kernel axpy_kernel (src/main/java/com/omega/engine/gpu/BaseKernel.java:306-329)
// and the residual add at LlamaTransformerBlock.java:136.
#include "common.cuh"

namespace omoe {

namespace {

// y = residual + combined rows: the residual add of the transformer block
// (LlamaTransformerBlock.java:136) folded into this pass; fp32 add, one rounding.
__device__ __forceinline__ void add_residual(const float *r, float (&acc)[8]) {
    float4 a = __ldg(reinterpret_cast<const float4 *>(r)), b = __ldg(reinterpret_cast<const float4 *>(r) + 1);
    acc[0] = a.x + acc[0]; acc[1] = a.y + acc[1]; acc[2] = a.z + acc[2]; acc[3] = a.w + acc[3];
    acc[4] = b.x + acc[4]; acc[5] = b.y + acc[5]; acc[6] = b.z + acc[6]; acc[7] = b.w + acc[7];
}
__device__ __forceinline__ void add_residual(const __nv_bfloat16 *r, float (&acc)[8]) {
    float v[8];
    unpack8(__ldg(reinterpret_cast<const uint4 *>(r)), v);
#pragma unroll
    for (int i = 0; i < 8; i++) acc[i] = v[i] + acc[i];
}

// One warp per token, 8 columns per lane per step (16 bytes of bf16 / 32 bytes of fp32).
template <typename YT, typename OT, int K>
__global__ void __launch_bounds__(256)
combine_kernel(void *const *__restrict__ out_table, OT *__restrict__ y, const OT *__restrict__ resid,
               const int32_t *__restrict__ pos, const int32_t *__restrict__ topk_idx,
               const float *__restrict__ topk_w, int T, int d, int k_rt, int e_local, EpWait wait, int32_t *dev_err) {
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    pdl_trigger();
    pdl_wait();
    if (wait.flags != nullptr) {
        // expert-parallel return: rows are read from the owners' output buffers
        // over NVLink once every rank has published them
        if ((int)threadIdx.x < wait.world) ep_wait_flag(wait.flags + threadIdx.x, *wait.seq, wait.timeout_ns, dev_err);
        __syncthreads();
    }
    if (t >= T) return;
    const int k = (K > 0) ? K : k_rt;
    constexpr int KR = (K > 0) ? K : kMaxTopK;
    const YT *src[KR];
    float w[KR];
    {
        int r = 0, q = 0;
        float g = 0.f;
        if (lane < k) {
            r = pos[(size_t)t * k + lane];
            q = topk_idx[(size_t)t * k + lane] / e_local;
            g = topk_w[(size_t)t * k + lane];
        }
#pragma unroll
        for (int j = 0; j < KR; j++) {
            int rj = __shfl_sync(0xffffffffu, r, j);
            int qj = __shfl_sync(0xffffffffu, q, j);
            w[j] = __shfl_sync(0xffffffffu, g, j);
            // rj < 0: the pick has no row (an expert-parallel step that was refused); it contributes zeros
            src[j] = (j < k && rj >= 0) ? static_cast<const YT *>(out_table[qj]) + (size_t)rj * d : nullptr;
        }
    }
    const int cw = ((d / (int)gridDim.y + 7) / 8) * 8;  // blockIdx.y walks one slice of the row
    const int c_lo = blockIdx.y * cw, c_hi = min(d, c_lo + cw);
    // bf16 rows with few picks: the loads of two column chunks are requested before the first is used (the loads,
    // over NVLink for remote rows, are the latency here); the arithmetic and its order are the same either way
    constexpr int U = (K > 0 && K <= 4 && sizeof(YT) == 2) ? 2 : 1;
    for (int c0 = c_lo + lane * 8; c0 < c_hi; c0 += 256 * U) {
        uint4 raw[U][KR];
        if constexpr (U == 2) {
#pragma unroll
            for (int u = 0; u < U; u++)
#pragma unroll
                for (int j = 0; j < KR; j++)
                    if (j < k && src[j] != nullptr && c0 + u * 256 < c_hi)
                        raw[u][j] = __ldcs(reinterpret_cast<const uint4 *>(src[j] + c0 + u * 256));
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
        const int c = c0 + u * 256;
        if (c >= c_hi) break;
        float acc[8];
#pragma unroll
        for (int j = 0; j < KR; j++) {
            if (j < k) {
                float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                if (src[j] == nullptr) {
                } else if constexpr (U == 2) {
                    unpack8(raw[u][j], v);
                } else if constexpr (sizeof(YT) == 2) {
                    uint4 r = __ldcs(reinterpret_cast<const uint4 *>(src[j] + c));
                    unpack8(r, v);
                } else {
                    float4 a = __ldcs(reinterpret_cast<const float4 *>(src[j] + c));
                    float4 b = __ldcs(reinterpret_cast<const float4 *>(src[j] + c) + 1);
                    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
                    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
                }
#pragma unroll
                for (int i = 0; i < 8; i++) acc[i] = (j == 0) ? w[0] * v[i] : fmaf(w[j], v[i], acc[i]);
            }
        }
        if (resid != nullptr) add_residual(resid + (size_t)t * d + c, acc);
        if constexpr (sizeof(OT) == 2) {
            uint4 o;
            o.x = pack_bf16(acc[0], acc[1]);
            o.y = pack_bf16(acc[2], acc[3]);
            o.z = pack_bf16(acc[4], acc[5]);
            o.w = pack_bf16(acc[6], acc[7]);
            *reinterpret_cast<uint4 *>(y + (size_t)t * d + c) = o;
        } else {
            float4 *o = reinterpret_cast<float4 *>(y + (size_t)t * d + c);
            o[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
            o[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
        }
        }  // u
    }
}

// A few tokens: one thread per 8 output columns, so every load of the step is
// in flight at once instead of one warp walking a row (same arithmetic order).
template <typename YT, typename OT>
__global__ void __launch_bounds__(256)
combine_small_kernel(void *const *__restrict__ out_table, OT *__restrict__ y, const OT *__restrict__ resid,
                     const int32_t *__restrict__ pos, const int32_t *__restrict__ topk_idx,
                     const float *__restrict__ topk_w, int T, int d, int k, int e_local) {
    const int vec = d / 8;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    pdl_trigger();
    pdl_wait();
    if (idx >= T * vec) return;
    const int t = idx / vec, c = (idx % vec) * 8;
    float acc[8];
    for (int j = 0; j < k; j++) {
        const int r = __ldg(pos + (size_t)t * k + j);
        const int q = __ldg(topk_idx + (size_t)t * k + j) / e_local;
        const float w = __ldg(topk_w + (size_t)t * k + j);
        const YT *src = static_cast<const YT *>(out_table[q]) + (size_t)r * d + c;
        float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (r < 0) {
        } else if constexpr (sizeof(YT) == 2) {
            unpack8(__ldcs(reinterpret_cast<const uint4 *>(src)), v);
        } else {
            float4 a = __ldcs(reinterpret_cast<const float4 *>(src));
            float4 b = __ldcs(reinterpret_cast<const float4 *>(src) + 1);
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
            v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        }
#pragma unroll
        for (int i = 0; i < 8; i++) acc[i] = (j == 0) ? w * v[i] : fmaf(w, v[i], acc[i]);
    }
    if (resid != nullptr) add_residual(resid + (size_t)t * d + c, acc);
    if constexpr (sizeof(OT) == 2) {
        uint4 o;
        o.x = pack_bf16(acc[0], acc[1]);
        o.y = pack_bf16(acc[2], acc[3]);
        o.z = pack_bf16(acc[4], acc[5]);
        o.w = pack_bf16(acc[6], acc[7]);
        *reinterpret_cast<uint4 *>(y + (size_t)t * d + c) = o;
    } else {
        float4 *o = reinterpret_cast<float4 *>(y + (size_t)t * d + c);
        o[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
        o[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
    }
}

template <typename YT, typename OT>
cudaError_t launch_k(omoe_handle *h, void *y, const void *resid_v, int T, cudaStream_t s, const EpWait *wait) {
    const int d = h->cfg.d_model, k = h->cfg.top_k, El = h->e_local;
    int split = 1;
    while (split < 8 && (long long)T * split < 32LL * h->sm_count && d / (split * 2) >= 512) split *= 2;
    dim3 grid(ceil_div(T, 8), split), block(256);
    OT *out = static_cast<OT *>(y);
    const OT *resid = static_cast<const OT *>(resid_v);
    if (wait == nullptr && (long long)T * (d / 8) <= 65536) {
        const int threads = T * (d / 8);
        return launch_ex(combine_small_kernel<YT, OT>, dim3(ceil_div(threads, 256)), dim3(256), 0, s, h->pdl,
                         h->d_out_table, out, resid, h->pos, h->topk_idx, h->topk_w, T, d, k, El);
    }
    EpWait wt = wait ? *wait : EpWait{nullptr, 1, 0, 0};
    cudaError_t e;
#define OMOE_COMBINE(KK)                                                                                         \
    e = launch_ex(combine_kernel<YT, OT, KK>, grid, block, 0, s, h->pdl, h->d_out_table, out, resid, h->pos,      \
                  h->topk_idx, h->topk_w, T, d, k, El, wt, h->dev_err)
    switch (k) {
        case 1: OMOE_COMBINE(1); break;
        case 2: OMOE_COMBINE(2); break;
        case 4: OMOE_COMBINE(4); break;
        case 6: OMOE_COMBINE(6); break;
        case 8: OMOE_COMBINE(8); break;
        default: OMOE_COMBINE(0); break;
    }
#undef OMOE_COMBINE
    return e;
}

}  // namespace

cudaError_t launch_combine(omoe_handle *h, void *y, int io_dtype, int T, cudaStream_t s, int *n, const EpWait *wait,
                           const void *resid) {
    const bool cbf = h->cfg.compute_dtype == OMOE_BF16;
    cudaError_t e;
    if (cbf && io_dtype == OMOE_BF16)
        e = launch_k<__nv_bfloat16, __nv_bfloat16>(h, y, resid, T, s, wait);
    else if (cbf && io_dtype == OMOE_F32)
        e = launch_k<__nv_bfloat16, float>(h, y, resid, T, s, wait);
    else if (!cbf && io_dtype == OMOE_F32)
        e = launch_k<float, float>(h, y, resid, T, s, wait);
    else
        return cudaErrorInvalidValue;
    if (e == cudaSuccess) (*n)++;
    return e;
}

}  // namespace omoe
