// Eight consecutive row elements at a time: 16-byte loads and stores of bf16 rows (32 bytes of fp32 rows) to and
// from fp32 registers.  Shared by every kernel that walks rows (dispatch, combine, RMSNorm, the decode-step
// kernels, the backward pass).  bf16 <-> fp32 is exact one way (a shift) and round-to-nearest-even the other.
#pragma once

#include <cuda_bf16.h>
#include <stdint.h>

namespace omoe {

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&v);
}

__device__ __forceinline__ void unpack8(const uint4 &r, float (&v)[8]) {
    uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

__device__ __forceinline__ uint4 pack8(const float (&v)[8]) {
    uint4 o;
    o.x = pack_bf16(v[0], v[1]);
    o.y = pack_bf16(v[2], v[3]);
    o.z = pack_bf16(v[4], v[5]);
    o.w = pack_bf16(v[6], v[7]);
    return o;
}

// plain loads (data another kernel of the same step may have written through a peer mapping)
__device__ __forceinline__ void load8(const float *p, float (&v)[8]) {
    float4 a = *reinterpret_cast<const float4 *>(p), b = *(reinterpret_cast<const float4 *>(p) + 1);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16 *p, float (&v)[8]) {
    unpack8(*reinterpret_cast<const uint4 *>(p), v);
}

// read-only path (inputs and weights that no kernel of the step writes)
__device__ __forceinline__ void ldg8(const float *p, float (&v)[8]) {
    float4 a = __ldg(reinterpret_cast<const float4 *>(p)), b = __ldg(reinterpret_cast<const float4 *>(p) + 1);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void ldg8(const __nv_bfloat16 *p, float (&v)[8]) {
    unpack8(__ldg(reinterpret_cast<const uint4 *>(p)), v);
}

__device__ __forceinline__ void store8(float *p, const float (&v)[8]) {
    float4 *o = reinterpret_cast<float4 *>(p);
    o[0] = make_float4(v[0], v[1], v[2], v[3]);
    o[1] = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void store8(__nv_bfloat16 *p, const float (&v)[8]) {
    *reinterpret_cast<uint4 *>(p) = pack8(v);
}

}  // namespace omoe
