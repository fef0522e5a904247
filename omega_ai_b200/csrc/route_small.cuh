// Device pieces shared by the one-launch routing kernels for decode steps (route_small.cu on one GPU,
// the expert-parallel form in ep.cu): the logits and picks of one token by one block, and the ranking of all
// picks of a step by one block.
#pragma once

#include "common.cuh"
#include "router_common.cuh"

namespace omoe {
namespace small {

constexpr int kSmallMaxTokens = 8;
constexpr int kSmallMaxPicks = kSmallMaxTokens * kMaxTopK;  // 128

// Logits of token t (eight warps split the experts; reduction tree as in router.cu), then softmax statistics,
// top-k and gate weights by warp 0.  sl: kMaxExperts floats of shared memory.  All 256 threads call this.
template <int PL, typename XT>
__device__ __forceinline__ void token_logits_topk(const XT *__restrict__ x, const float *__restrict__ w_r,
                                                  const float *__restrict__ bias, int t, int d, int E, int k, int renorm,
                                                  float *__restrict__ logits, int32_t *__restrict__ topk_idx,
                                                  float *__restrict__ topk_w, float *sl) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const XT *xr = x + (size_t)t * d;
    for (int e = warp; e < E; e += 8) {
        const float *wr = w_r + (size_t)e * d;
        float acc_even = 0.f, acc_odd = 0.f;  // the two chains of the reduction rule
        for (int i0 = lane * 8; i0 < d; i0 += 4 * 256) {
            float xv[4][8], wv[4][8];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int i = i0 + u * 256;
                if (i < d) {
                    ldg8(xr + i, xv[u]);
                    ldg8(wr + i, wv[u]);
                }
            }
#pragma unroll
            for (int u = 0; u < 4; u++) {
                if (i0 + u * 256 < d) {
#pragma unroll
                    for (int j = 0; j < 8; j += 2) {
                        acc_even = fmaf(xv[u][j], wv[u][j], acc_even);
                        acc_odd = fmaf(xv[u][j + 1], wv[u][j + 1], acc_odd);
                    }
                }
            }
        }
        float acc = acc_even + acc_odd;
#pragma unroll
        for (int m = 16; m >= 1; m >>= 1) acc = acc + __shfl_xor_sync(0xffffffffu, acc, m);
        if (lane == 0) {
            float v = acc;
            if (bias != nullptr) v = v + __ldg(bias + e);
            sl[e] = v;
            logits[(size_t)t * E + e] = v;
        }
    }
    __syncthreads();
    if (warp == 0) {
        int my_e;
        float my_w;
        warp_softmax_topk<PL>(sl, E, k, renorm, lane, my_e, my_w);
        if (lane < k) {
            topk_idx[(size_t)t * k + lane] = my_e;
            topk_w[(size_t)t * k + lane] = my_w;
        }
    }
}

// s_idx[0..n) holds the step's picks in flat order t*k+j.  s_rank[f] becomes the rank of pick f among the picks
// of its expert (stable), s_cnt[e] the number of picks of expert e.  All 256 threads call this; the caller
// synchronises afterwards.
__device__ __forceinline__ void rank_picks(int n, int E, const int32_t *s_idx, int32_t *s_rank, int32_t *s_cnt) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int e = warp; e < E; e += 8) {
        int base = 0;
        for (int c = 0; c < n; c += 32) {
            const int f = c + lane;
            const int v = (f < n) ? s_idx[f] : -1;
            const uint32_t m = __ballot_sync(0xffffffffu, v == e);
            if (v == e) s_rank[f] = base + __popc(m & ((1u << lane) - 1u));
            base += __popc(m);
        }
        if (lane == 0) s_cnt[e] = base;
    }
}

}  // namespace small
}  // namespace omoe
