// fp32 expert products on CUDA cores (compute_dtype = OMOE_F32).  This is the
// arithmetic the reference's FullyLayer performs (cublasSgemm, fp32 in and out;
// src/main/java/com/omega/engine/nn/layer/FullyLayer.java:235 ->
// src/main/java/com/omega/engine/gpu/GPUOP.java:405-417) in the order of
// LlamaMLPLayer.output() (LlamaMLPLayer.java:117-123), with SiLU
// (src/main/resources/cu/activeFunction.cu:172-180) and the element-wise
// product (src/main/resources/cu/OPKernel.cu:1040) fused into the first
// product's epilogue instead of being three more passes over [rows, d_ff].
// It serves small fp32 layers sized for a host-side reference run; the
// throughput path is the bf16 tensor-core kernel.
#include "common.cuh"

namespace omoe {

namespace {

constexpr int BM = 64, BN = 64, BK = 16;

// C[rows, N] = A[rows, K] * B_e[N, K]^T per expert; SWIGLU: C = silu(A*Bg^T) * (A*Bu^T).
template <bool SWIGLU>
__global__ void __launch_bounds__(256)
grouped_sgemm_kernel(const float *__restrict__ A, const float *__restrict__ B0, const float *__restrict__ B1,
                     float *__restrict__ C, int N, int K, const int32_t *__restrict__ tile_expert,
                     const int32_t *__restrict__ poffsets, const int32_t *__restrict__ counts, int E) {
    const int row0 = blockIdx.y * BM;
    if (row0 >= poffsets[E]) return;
    const int e = tile_expert[row0 / kRowAlign];
    const int valid = poffsets[e] + counts[e] - row0;  // rows of this tile that carry tokens
    if (valid <= 0) return;
    const int n0 = blockIdx.x * BN;

    __shared__ float As[BK][BM + 4];
    __shared__ float Bs0[BK][BN + 4];
    __shared__ float Bs1[SWIGLU ? BK : 1][BN + 4];

    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;  // 16x16 threads, 4x4 outputs each
    const float *Bg = B0 + (size_t)e * N * K;
    const float *Bu = SWIGLU ? B1 + (size_t)e * N * K : nullptr;

    float acc0[4][4], acc1[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) { acc0[i][j] = 0.f; acc1[i][j] = 0.f; }

    // each thread loads 4 consecutive k of one row: 64 rows x 16 k = 256 float4
    const int lr = tid / 4, lk = (tid % 4) * 4;
    for (int k0 = 0; k0 < K; k0 += BK) {
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b0 = a, b1 = a;
        if (k0 + lk < K) {  // K is a multiple of 4
            if (lr < valid) a = *reinterpret_cast<const float4 *>(A + (size_t)(row0 + lr) * K + k0 + lk);
            if (n0 + lr < N) {
                b0 = __ldg(reinterpret_cast<const float4 *>(Bg + (size_t)(n0 + lr) * K + k0 + lk));
                if (SWIGLU) b1 = __ldg(reinterpret_cast<const float4 *>(Bu + (size_t)(n0 + lr) * K + k0 + lk));
            }
        }
        __syncthreads();
        As[lk + 0][lr] = a.x; As[lk + 1][lr] = a.y; As[lk + 2][lr] = a.z; As[lk + 3][lr] = a.w;
        Bs0[lk + 0][lr] = b0.x; Bs0[lk + 1][lr] = b0.y; Bs0[lk + 2][lr] = b0.z; Bs0[lk + 3][lr] = b0.w;
        if (SWIGLU) {
            Bs1[lk + 0][lr] = b1.x; Bs1[lk + 1][lr] = b1.y; Bs1[lk + 2][lr] = b1.z; Bs1[lk + 3][lr] = b1.w;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; kk++) {
            float av[4], bv0[4], bv1[4];
#pragma unroll
            for (int i = 0; i < 4; i++) av[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                bv0[j] = Bs0[kk][tx * 4 + j];
                bv1[j] = SWIGLU ? Bs1[kk][tx * 4 + j] : 0.f;
            }
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    acc0[i][j] = fmaf(av[i], bv0[j], acc0[i][j]);
                    if (SWIGLU) acc1[i][j] = fmaf(av[i], bv1[j], acc1[i][j]);
                }
        }
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int r = ty * 4 + i;
        if (r >= valid) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            int c = n0 + tx * 4 + j;
            if (c >= N) continue;
            float v = acc0[i][j];
            if (SWIGLU) v = (v / (1.0f + expf(-v))) * acc1[i][j];
            C[(size_t)(row0 + r) * N + c] = v;
        }
    }
}

}  // namespace

cudaError_t launch_experts_f32(omoe_handle *h, cudaStream_t s, int *n) {
    const int d = h->cfg.d_model, dff = h->cfg.d_ff, E = h->e_local;
    const int m_tiles = (int)(h->rows_cap / BM);
    dim3 block(256);
    dim3 g1(ceil_div(dff, BN), m_tiles);
    grouped_sgemm_kernel<true><<<g1, block, 0, s>>>(
        static_cast<const float *>(h->xp), static_cast<const float *>(h->w_gate),
        static_cast<const float *>(h->w_up), static_cast<float *>(h->hbuf), dff, d, h->ex_tile_expert,
        h->ex_poffsets, h->ex_counts, E);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    (*n)++;
    dim3 g2(ceil_div(d, BN), m_tiles);
    grouped_sgemm_kernel<false><<<g2, block, 0, s>>>(
        static_cast<const float *>(h->hbuf), static_cast<const float *>(h->w_down), nullptr,
        static_cast<float *>(h->yp), d, dff, h->ex_tile_expert, h->ex_poffsets, h->ex_counts, E);
    e = cudaGetLastError();
    if (e == cudaSuccess) (*n)++;
    return e;
}

}  // namespace omoe
