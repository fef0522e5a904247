// Expert products for a handful of tokens (decode steps): a weight-streaming
// path on CUDA cores.  With one or two rows per expert the tensor-core tiles of
// experts_sm100.cu would be 99 % padding and, worse, there are too few tiles to
// keep every SM's share of HBM busy.  Here the work item is one output column
// (one weight row, or a gate/up pair of rows): a pair of warps streams it once
// with 16-byte loads and folds it against the expert's token rows held in shared
// memory, so the items spread evenly over all SMs and the kernel runs at HBM
// speed.  Same arithmetic points as the tensor-core path (bf16 operands, fp32
// accumulate, h and yp rounded to bf16); it replaces the same reference calls
// (LlamaMLPLayer.java:117-123).
#include <stdlib.h>

#include "common.cuh"

namespace omoe {

namespace {

constexpr int kDecThreads = 256;
constexpr int kPairs = kDecThreads / 64;

// 64-thread barrier of one warp pair; the id is a literal so the kernel reserves only the barriers it uses
__device__ __forceinline__ void pair_sync(int pair) {
    switch (pair) {
        case 0: asm volatile("bar.sync 1, 64;" ::: "memory"); break;
        case 1: asm volatile("bar.sync 2, 64;" ::: "memory"); break;
        case 2: asm volatile("bar.sync 3, 64;" ::: "memory"); break;
        default: asm volatile("bar.sync 4, 64;" ::: "memory"); break;
    }
}

__device__ __forceinline__ uint4 ld_stream(const void *p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}

// out[row, n] = f( A[row, :] . W0[e][n, :],  A[row, :] . W1[e][n, :] )  for the rows of every expert e that has any.
// SWIGLU: f(g, u) = silu(g) * u;  else f(g, -) = g and W1 is unused.
// Items (expert, n) are numbered expert-major over the experts that have rows and dealt out in equal contiguous
// runs to the blocks; inside a block the four warp pairs take them round-robin, each warp half of K.
// RP: token rows of one expert folded per pass over its weights (1, 2 or 4).
template <bool SWIGLU, int RP>
__global__ void __launch_bounds__(kDecThreads, 2)
decode_gemv_kernel(const __nv_bfloat16 *__restrict__ A, const __nv_bfloat16 *__restrict__ W0,
                   const __nv_bfloat16 *__restrict__ W1, __nv_bfloat16 *__restrict__ out, int K, int N,
                   const int32_t *__restrict__ counts, const int32_t *__restrict__ poffsets, int El) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16 *rows = reinterpret_cast<__nv_bfloat16 *>(smem_raw);  // [RP][K]
    __shared__ int s_active[kMaxExperts];
    __shared__ int s_n_active;
    __shared__ float s_part[kPairs][2][RP];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int pair = warp >> 1, half = warp & 1;
    pdl_trigger();
    pdl_wait();
    if (tid == 0) {
        int n = 0;
        for (int e = 0; e < El; e++)
            if (counts[e] > 0) s_active[n++] = e;
        s_n_active = n;
    }
    __syncthreads();
    const long long total = (long long)s_n_active * N;
    const long long per = (total + gridDim.x - 1) / gridDim.x;
    const long long g0 = (long long)blockIdx.x * per;
    const long long g1 = g0 + per < total ? g0 + per : total;
    const int kh = (K / 2 + 7) / 8 * 8;           // first warp of a pair takes [0, kh), the second [kh, K)
    const int k_lo = half ? kh : 0, k_hi = half ? K : kh;

    long long g = g0;
    while (g < g1) {
        const int ai = (int)(g / N);
        const int e = s_active[ai];
        const long long g_end_e = (long long)(ai + 1) * N < g1 ? (long long)(ai + 1) * N : g1;
        const int m = counts[e];
        const int row0 = poffsets[e];
        for (int r0 = 0; r0 < m; r0 += RP) {
            const int mr = m - r0 < RP ? m - r0 : RP;
            __syncthreads();
            for (int i = tid; i < mr * (K / 8); i += kDecThreads) {
                int r = i / (K / 8), c = i % (K / 8);
                reinterpret_cast<uint4 *>(rows + (size_t)r * K)[c] =
                    reinterpret_cast<const uint4 *>(A + (size_t)(row0 + r0 + r) * K)[c];
            }
            __syncthreads();
            for (long long it = g + pair; it < g_end_e; it += kPairs) {
                const int n = (int)(it - (long long)ai * N);
                const __nv_bfloat16 *w0 = W0 + ((size_t)e * N + n) * K;
                const __nv_bfloat16 *w1 = SWIGLU ? W1 + ((size_t)e * N + n) * K : nullptr;
                float acc0[RP], acc1[RP];
#pragma unroll
                for (int r = 0; r < RP; r++) { acc0[r] = 0.f; acc1[r] = 0.f; }
                constexpr int U = SWIGLU ? 4 : 8;  // 16-byte loads per operand in flight per lane
                for (int k0 = k_lo + lane * 8; k0 < k_hi; k0 += 32 * 8 * U) {
                    uint4 q0[U], q1[SWIGLU ? U : 1];
#pragma unroll
                    for (int u = 0; u < U; u++) {
                        const int kk = k0 + u * 256;
                        if (kk < k_hi) {
                            q0[u] = ld_stream(w0 + kk);
                            if (SWIGLU) q1[u] = ld_stream(w1 + kk);
                        }
                    }
#pragma unroll
                    for (int u = 0; u < U; u++) {
                        const int kk = k0 + u * 256;
                        if (kk < k_hi) {
                            float wv0[8], wv1[8];
                            unpack8(q0[u], wv0);
                            if (SWIGLU) unpack8(q1[u], wv1);
#pragma unroll
                            for (int r = 0; r < RP; r++) {
                                if (r < mr) {
                                    float av[8];
                                    unpack8(*reinterpret_cast<const uint4 *>(rows + (size_t)r * K + kk), av);
#pragma unroll
                                    for (int j = 0; j < 8; j++) {
                                        acc0[r] = fmaf(av[j], wv0[j], acc0[r]);
                                        if (SWIGLU) acc1[r] = fmaf(av[j], wv1[j], acc1[r]);
                                    }
                                }
                            }
                        }
                    }
                }
#pragma unroll
                for (int r = 0; r < RP; r++) {
#pragma unroll
                    for (int o = 16; o >= 1; o >>= 1) {
                        acc0[r] += __shfl_xor_sync(0xffffffffu, acc0[r], o);
                        if (SWIGLU) acc1[r] += __shfl_xor_sync(0xffffffffu, acc1[r], o);
                    }
                }
                // second warp of the pair hands its half over; the first finishes the column
                if (half == 1 && lane == 0) {
#pragma unroll
                    for (int r = 0; r < RP; r++) { s_part[pair][0][r] = acc0[r]; s_part[pair][1][r] = acc1[r]; }
                }
                pair_sync(pair);
                if (half == 0 && lane == 0) {
#pragma unroll
                    for (int r = 0; r < RP; r++) {
                        if (r < mr) {
                            float g_ = acc0[r] + s_part[pair][0][r];
                            float v = g_;
                            if (SWIGLU) {
                                float u_ = acc1[r] + s_part[pair][1][r];
                                v = __fdividef(g_, 1.0f + __expf(-g_)) * u_;
                            }
                            out[(size_t)(row0 + r0 + r) * N + n] = __float2bfloat16_rn(v);
                        }
                    }
                }
                pair_sync(pair);
            }
        }
        g = g_end_e;
    }
}

}  // namespace

// Largest token count of one forward for which the streaming path is used.  A
// token picks an expert at most once, so no expert then holds more rows than this.
// Above a couple of tokens the per-row arithmetic on CUDA cores costs more than the padding of tensor-core tiles.
int decode_tokens_threshold() {
    static int v = -1;
    if (v < 0) {
        const char *s = getenv("OMOE_DECODE_MAX_T");  // tuning knob, 0..8
        int t = s ? atoi(s) : 2;
        v = t < 0 ? 0 : (t > 8 ? 8 : t);
    }
    return v;
}

namespace {

template <bool SWIGLU, int RP>
cudaError_t launch_gemv(omoe_handle *h, const void *A, const void *W0, const void *W1, void *out, int K, int N,
                        cudaStream_t s) {
    auto kern = decode_gemv_kernel<SWIGLU, RP>;
    const size_t smem = (size_t)RP * K * 2;
    if (smem > 200 * 1024) return cudaErrorInvalidValue;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    int per_sm = 1;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kDecThreads, smem);
    if (e != cudaSuccess) return e;
    if (per_sm < 1) per_sm = 1;
    if (per_sm > 4) per_sm = 4;
    const int sms = h->sm_count > 0 ? h->sm_count : 148;
    return launch_ex(kern, dim3(sms * per_sm), dim3(kDecThreads), smem, s, h->pdl,
                     static_cast<const __nv_bfloat16 *>(A), static_cast<const __nv_bfloat16 *>(W0),
                     static_cast<const __nv_bfloat16 *>(W1), static_cast<__nv_bfloat16 *>(out), K, N, h->ex_counts,
                     h->ex_poffsets, h->e_local);
}

template <int RP>
cudaError_t launch_both(omoe_handle *h, cudaStream_t s, int *n, cudaEvent_t mid) {
    const int d = h->cfg.d_model, dff = h->cfg.d_ff;
    cudaError_t e = launch_gemv<true, RP>(h, h->xp, h->w_gate, h->w_up, h->hbuf, d, dff, s);
    if (e != cudaSuccess) return e;
    (*n)++;
    if (mid) cudaEventRecord(mid, s);
    e = launch_gemv<false, RP>(h, h->hbuf, h->w_down, nullptr, h->yp, dff, d, s);
    if (e == cudaSuccess) (*n)++;
    return e;
}

}  // namespace

cudaError_t launch_experts_decode(omoe_handle *h, int T, cudaStream_t s, int *n, cudaEvent_t mid) {
    // the streaming kernels keep RP token rows of the longer reduction in shared memory; layers too wide for
    // that take the tensor-core kernels, as steps with more tokens do
    const int rp = T <= 1 ? 1 : (T <= 2 ? 2 : 4);
    const int kmax = h->cfg.d_model > h->cfg.d_ff ? h->cfg.d_model : h->cfg.d_ff;
    if ((size_t)rp * kmax * 2 > 200 * 1024) return launch_experts_bf16(h, s, n, mid, (long)T * h->cfg.top_k);
    if (T <= 1) return launch_both<1>(h, s, n, mid);
    if (T <= 2) return launch_both<2>(h, s, n, mid);
    return launch_both<4>(h, s, n, mid);
}

}  // namespace omoe
