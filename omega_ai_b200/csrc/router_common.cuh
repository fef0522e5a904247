// Pieces shared by the router kernels: softmax statistics and top-k of one token by one warp.
#pragma once

#include "common.cuh"

namespace omoe {

// lv[0..E) holds the token's logits in shared memory and is overwritten with
// expf(logit - max).  Arithmetic of src/main/resources/cu/SoftmaxKernel.cu:5-24:
// max, exponentials, their sum in index order, divide.  The k picks are taken on
// the logits, largest first, a tie going to the lower expert.  Lane j < k
// returns pick j and its gate weight (renormalised over the picks in pick order
// when renorm is set).  PL = logits per lane (ceil(E_padded / 32)).
// GW = lanes that share one token (8, 16 or 32; a power of two): lane gl of the group holds
// logits gl, gl + GW, ...; groups of one warp work on different tokens at the same time.  Every
// lane of the warp must call this (the shuffles are warp-wide, with xor distances below GW).
template <int PL, int GW>
__device__ __forceinline__ void group_softmax_topk(float *lv, int E, int k, int renorm, int lane, int &my_e, float &my_w) {
    float v[PL];
    float mx = -3.402823466e+38F;
#pragma unroll
    for (int m = 0; m < PL; m++) {
        const int e = lane + GW * m;
        v[m] = (e < E) ? lv[e] : -INFINITY;
        mx = fmaxf(mx, v[m]);
    }
#pragma unroll
    for (int o = GW / 2; o >= 1; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    __syncwarp();
#pragma unroll
    for (int m = 0; m < PL; m++) {
        const int e = lane + GW * m;
        if (e < E) lv[e] = expf(v[m] - mx);  // the row now holds the exponentials
    }
    __syncwarp();
    float sum = 0.f;
    for (int e = 0; e < E; e++) sum += lv[e];  // index order, every lane redundantly (broadcast reads)
    float w = 0.f, wsum = 0.f;
    int pick = 0;
#pragma unroll 1
    for (int j = 0; j < k; j++) {
        float bv = -INFINITY;
        int be = 0x7fffffff;
#pragma unroll
        for (int m = 0; m < PL; m++) {
            const int e = lane + GW * m;
            if (v[m] > bv || (v[m] == bv && e < be)) { bv = v[m]; be = e; }  // NaN never wins
        }
#pragma unroll
        for (int o = GW / 2; o >= 1; o >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            int oe = __shfl_xor_sync(0xffffffffu, be, o);
            if (ov > bv || (ov == bv && oe < be)) { bv = ov; be = oe; }
        }
#pragma unroll
        for (int m = 0; m < PL; m++)
            if (lane + GW * m == be) v[m] = -INFINITY;  // taken
        const float p = lv[be] / sum;
        wsum += p;
        if (lane == j) { w = p; pick = be; }
    }
    my_e = pick;
    my_w = renorm ? w / wsum : w;
}

}  // namespace omoe

namespace omoe {
// The whole warp on one token.
template <int PL>
__device__ __forceinline__ void warp_softmax_topk(float *lv, int E, int k, int renorm, int lane, int &my_e, float &my_w) {
    group_softmax_topk<PL, 32>(lv, E, k, renorm, lane, my_e, my_w);
}
}  // namespace omoe
