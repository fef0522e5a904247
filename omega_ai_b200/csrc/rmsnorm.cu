// Pre-FFN RMSNorm of the transformer block, feeding the MoE layer.
//
// Arithmetic of the reference kernel rmsnorm_forward_kernel2
// (src/main/resources/cu/RMSKernel.cu:185-224, the kernel RMSLayer.output()
// launches: RMSLayer.java:222-230): rms = sqrtf(sum(x^2) / C + eps),
// out = (x / rms) * weight.  The reference reduces the squares with an
// unspecified warp reduction; here the order is fixed so that the normalised
// rows — and with them the router's bit-exact logits — are reproducible: lane l
// owns the elements i with (i/8)%32 == l and folds x*x into one fmaf chain in
// ascending i, then an xor butterfly over 16,8,4,2,1.  Square root and
// divisions are IEEE-rounded.  One warp per row; the row is read twice (the
// second time from cache) and written once in the layer's compute dtype.
#include "common.cuh"

namespace omoe {

namespace {


template <typename XT, typename OT>
__global__ void __launch_bounds__(256)
rmsnorm_kernel(const XT *__restrict__ x, const float *__restrict__ gamma, OT *__restrict__ out, int T, int d, float eps) {
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= T) return;
    const XT *row = x + (size_t)t * d;
    float ss = 0.f;
    for (int c = lane * 8; c < d; c += 256) {
        float v[8];
        ldg8(row + c, v);
#pragma unroll
        for (int j = 0; j < 8; j++) ss = fmaf(v[j], v[j], ss);
    }
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1) ss = ss + __shfl_xor_sync(0xffffffffu, ss, m);
    const float rms = sqrtf(ss / (float)d + eps);
    OT *o = out + (size_t)t * d;
    for (int c = lane * 8; c < d; c += 256) {
        float v[8], g[8];
        ldg8(row + c, v);
        ldg8(gamma + c, g);
#pragma unroll
        for (int j = 0; j < 8; j++) v[j] = (v[j] / rms) * g[j];
        store8(o + c, v);
    }
}

}  // namespace

cudaError_t launch_rmsnorm(omoe_handle *h, const void *x, int x_dtype, const float *gamma, float eps, int T,
                           cudaStream_t s, int *n) {
    const int d = h->cfg.d_model;
    dim3 grid(ceil_div(T, 8)), block(256);
    const bool cbf = h->cfg.compute_dtype == OMOE_BF16;
    if (x_dtype == OMOE_F32 && cbf)
        rmsnorm_kernel<float, __nv_bfloat16><<<grid, block, 0, s>>>(static_cast<const float *>(x), gamma,
                                                                   static_cast<__nv_bfloat16 *>(h->xn), T, d, eps);
    else if (x_dtype == OMOE_BF16 && cbf)
        rmsnorm_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, block, 0, s>>>(
            static_cast<const __nv_bfloat16 *>(x), gamma, static_cast<__nv_bfloat16 *>(h->xn), T, d, eps);
    else if (x_dtype == OMOE_F32 && !cbf)
        rmsnorm_kernel<float, float><<<grid, block, 0, s>>>(static_cast<const float *>(x), gamma,
                                                           static_cast<float *>(h->xn), T, d, eps);
    else
        return cudaErrorInvalidValue;
    (*n)++;
    return cudaGetLastError();
}

}  // namespace omoe
