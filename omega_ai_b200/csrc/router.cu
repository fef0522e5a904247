// Fused router: logits = x * W_r^T (+bias), softmax, top-k, gate weights,
// per-block expert histogram and the stable in-block rank of every pick.
//
// No reference kernel exists for this stage.  The dense semantics are those of
// FullyLayer (Y = X * W^T, W [out,in];
// src/main/java/com/omega/engine/nn/layer/FullyLayer.java:181,235) and the
// softmax arithmetic is that of src/main/resources/cu/SoftmaxKernel.cu:5-24
// (max, expf(x-max) summed in index order, divide).
//
// Bit-exact routing needs a fixed summation order for the logits.  The order
// is: lane l of a warp owns the elements i with (i/8)%32 == l and folds them in
// ascending i with one fmaf chain; the 32 partial sums are then combined by an
// xor butterfly over distances 16,8,4,2,1; the bias is added last.  One warp
// computes several tokens at once so every router weight read from shared
// memory is used for TPW tokens.
#include <string.h>

#include "common.cuh"

namespace omoe {

namespace {

constexpr int kSub = 256;  // elements one warp covers per step (32 lanes x 8)

__device__ __forceinline__ void load8(const float *p, float (&v)[8]) {
    float4 a = __ldg(reinterpret_cast<const float4 *>(p));
    float4 b = __ldg(reinterpret_cast<const float4 *>(p) + 1);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

__device__ __forceinline__ void load8(const __nv_bfloat16 *p, float (&v)[8]) {
    uint4 r = __ldg(reinterpret_cast<const uint4 *>(p));
    uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

// EMAX: experts held in registers per token (>= E); TPW: tokens per warp;
// DCG: 256-element sub-chunks of W_r staged in shared memory per chunk.
template <int EMAX, int TPW, int DCG, typename XT>
__global__ void __launch_bounds__(kRouterWarps * 32, (EMAX <= 32) ? 2 : 1)
router_kernel(const XT *__restrict__ x, const float *__restrict__ w_r, const float *__restrict__ bias,
              int T, int d, int E, int k, int renorm,
              float *__restrict__ logits, int32_t *__restrict__ topk_idx, float *__restrict__ topk_w,
              int32_t *__restrict__ block_counts, int32_t *__restrict__ local_rank) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float *ws = reinterpret_cast<float *>(smem_raw);                    // [EMAX][DCG][256] (lane-split layout)
    float *sl = ws + EMAX * DCG * kSub;                                  // [warps][TPW][EMAX] logits
    int32_t *sidx = reinterpret_cast<int32_t *>(sl + kRouterWarps * TPW * EMAX);  // [warps*TPW][k]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int TB = kRouterWarps * TPW;
    const int t0 = blockIdx.x * TB;
    const int tw = t0 + warp * TPW;  // first token of this warp

    float acc[TPW][EMAX];
#pragma unroll
    for (int i = 0; i < TPW; i++)
#pragma unroll
        for (int e = 0; e < EMAX; e++) acc[i][e] = 0.0f;

    // this lane's 8 elements of one 256-element step, for the warp's TPW tokens
    auto load_x = [&](int i0, float (&dst)[TPW][8]) {
#pragma unroll
        for (int i = 0; i < TPW; i++) {
            if (i0 < d && tw + i < T) {
                load8(x + (size_t)(tw + i) * d + i0, dst[i]);
            } else {
#pragma unroll
                for (int j = 0; j < 8; j++) dst[i][j] = 0.f;
            }
        }
    };

    float xc[TPW][8], xn[TPW][8];
    load_x(lane * 8, xc);
    constexpr int DC = DCG * kSub;
    for (int c0 = 0; c0 < d; c0 += DC) {
        __syncthreads();
        // stage W_r[:, c0:c0+DC) — float4 units, zero beyond d or E
        for (int u = tid; u < EMAX * (DC / 4); u += blockDim.x) {
            int e = u / (DC / 4), q = u % (DC / 4);
            int i = c0 + 4 * q;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (e < E && i < d) v = __ldg(reinterpret_cast<const float4 *>(w_r + (size_t)e * d + i));
            int sub = (4 * q) / kSub, within = (4 * q) % kSub;
            int ln = within >> 3, half = (within & 7) >> 2;
            *reinterpret_cast<float4 *>(ws + (e * DCG + sub) * kSub + half * 128 + ln * 4) = v;
        }
        __syncthreads();
#pragma unroll 1
        for (int sub = 0; sub < DCG; sub++) {
            const int i0 = c0 + sub * kSub + lane * 8;
            if (c0 + sub * kSub >= d) break;
            load_x(i0 + kSub, xn);  // next step's rows are in flight while this step is folded in
            if (i0 < d) {           // d is a multiple of 8: a lane's group is whole or absent
#pragma unroll
                for (int e = 0; e < EMAX; e++) {
                    const float *wp = ws + (e * DCG + sub) * kSub + lane * 4;
                    float4 wa = *reinterpret_cast<const float4 *>(wp);
                    float4 wb = *reinterpret_cast<const float4 *>(wp + 128);
                    float wv[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
#pragma unroll
                    for (int i = 0; i < TPW; i++)
#pragma unroll
                        for (int j = 0; j < 8; j++) acc[i][e] = fmaf(xc[i][j], wv[j], acc[i][e]);
                }
            }
#pragma unroll
            for (int i = 0; i < TPW; i++)
#pragma unroll
                for (int j = 0; j < 8; j++) xc[i][j] = xn[i][j];
        }
    }

    // xor butterfly, then lane (e % 32) publishes logit e
#pragma unroll
    for (int i = 0; i < TPW; i++)
#pragma unroll
        for (int e = 0; e < EMAX; e++) {
            float a = acc[i][e];
#pragma unroll
            for (int m = 16; m >= 1; m >>= 1) a = a + __shfl_xor_sync(0xffffffffu, a, m);
            if (lane == (e & 31) && e < E) {
                float v = a;
                if (bias != nullptr) v = v + __ldg(bias + e);
                sl[(warp * TPW + i) * EMAX + e] = v;
                if (tw + i < T) logits[(size_t)(tw + i) * E + e] = v;
            }
        }
    __syncwarp();

    // one lane per token: softmax statistics, top-k on the logits, gate weights
    if (lane < TPW) {
        const int t = tw + lane;
        const float *lv = sl + (warp * TPW + lane) * EMAX;
        int32_t *my_idx = sidx + (warp * TPW + lane) * k;
        if (t < T) {
            float mx = -3.402823466e+38F;
            for (int e = 0; e < E; e++)
                if (mx <= lv[e]) mx = lv[e];
            float sum = 0.f;
            for (int e = 0; e < E; e++) sum += expf(lv[e] - mx);
            uint32_t used[kMaxExperts / 32];
#pragma unroll
            for (int i = 0; i < kMaxExperts / 32; i++) used[i] = 0u;
            float wk[kMaxTopK];
            float wsum = 0.f;
#pragma unroll 1
            for (int j = 0; j < k; j++) {
                int best = -1;
                float bv = 0.f;
                for (int e = 0; e < E; e++) {
                    if ((used[e >> 5] >> (e & 31)) & 1u) continue;
                    float v = lv[e];
                    if (best < 0 || v > bv) { best = e; bv = v; }
                }
                used[best >> 5] |= 1u << (best & 31);
                float p = expf(bv - mx) / sum;
                wk[j] = p;
                wsum += p;
                my_idx[j] = best;
                topk_idx[(size_t)t * k + j] = best;
            }
#pragma unroll 1
            for (int j = 0; j < k; j++) topk_w[(size_t)t * k + j] = renorm ? wk[j] / wsum : wk[j];
        } else {
            for (int j = 0; j < k; j++) my_idx[j] = -1;
        }
    }
    __syncthreads();

    // Stable rank of every pick among the block's picks of the same expert, in
    // order of the flat index t*k+j; the last running count is the histogram.
    const int n_entries = TB * k;
    for (int e = warp; e < E; e += kRouterWarps) {
        int base = 0;
        for (int c = 0; c < n_entries; c += 32) {
            int f = c + lane;
            int v = (f < n_entries) ? sidx[f] : -1;
            uint32_t m = __ballot_sync(0xffffffffu, v == e);
            if (v == e) local_rank[(size_t)t0 * k + f] = base + __popc(m & ((1u << lane) - 1u));
            base += __popc(m);
        }
        if (lane == 0) block_counts[(size_t)e * gridDim.x + blockIdx.x] = base;  // expert-major
    }
}

template <int EMAX, int TPW, int DCG, typename XT>
cudaError_t launch_one(omoe_handle *h, const XT *x, int T, cudaStream_t s) {
    constexpr int TB = kRouterWarps * TPW;
    const int k = h->cfg.top_k;
    size_t smem = sizeof(float) * (EMAX * DCG * kSub + kRouterWarps * TPW * EMAX) + sizeof(int32_t) * TB * k;
    auto kern = router_kernel<EMAX, TPW, DCG, XT>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    h->tokens_per_block = TB;  // the scan and dispatch kernels walk the histogram with this granularity
    int blocks = ceil_div(T, TB);
    kern<<<blocks, kRouterWarps * 32, smem, s>>>(x, h->w_router, h->router_bias, T, h->cfg.d_model,
                                                  h->cfg.n_experts, k, h->cfg.renormalize, h->logits,
                                                  h->topk_idx, h->topk_w, h->block_counts, h->pos);
    return cudaGetLastError();
}

// More tokens per warp reuse every router weight read from shared memory more
// often; fewer give more blocks.  Take the largest that still fills the GPU twice.
template <int EMAX, int DCG, int TPW_MAX, typename XT>
cudaError_t launch_tpw(omoe_handle *h, const XT *x, int T, cudaStream_t s) {
    const int want_blocks = 2 * (h->sm_count > 0 ? h->sm_count : 148);
    if constexpr (TPW_MAX >= 4)
        if (ceil_div(T, kRouterWarps * 4) >= want_blocks) return launch_one<EMAX, 4, DCG, XT>(h, x, T, s);
    if constexpr (TPW_MAX >= 2)
        if (ceil_div(T, kRouterWarps * 2) >= want_blocks) return launch_one<EMAX, 2, DCG, XT>(h, x, T, s);
    return launch_one<EMAX, 1, DCG, XT>(h, x, T, s);
}

template <typename XT>
cudaError_t launch_typed(omoe_handle *h, const XT *x, int T, cudaStream_t s) {
    const int E = h->cfg.n_experts;
    if (E <= 8) return launch_tpw<8, 8, 4, XT>(h, x, T, s);
    if (E <= 16) return launch_tpw<16, 4, 2, XT>(h, x, T, s);
    if (E <= 32) return launch_tpw<32, 2, 2, XT>(h, x, T, s);
    if (E <= 64) return launch_tpw<64, 1, 2, XT>(h, x, T, s);
    return launch_tpw<128, 1, 1, XT>(h, x, T, s);
}

}  // namespace

// Smallest number of tokens one router block may cover (sizes the per-block histogram array).
int router_tokens_per_block(int) { return kRouterWarps; }

cudaError_t launch_router(omoe_handle *h, const void *x, int io_dtype, int T, cudaStream_t s, int *n) {
    cudaError_t e;
    if (io_dtype == OMOE_F32)
        e = launch_typed<float>(h, static_cast<const float *>(x), T, s);
    else
        e = launch_typed<__nv_bfloat16>(h, static_cast<const __nv_bfloat16 *>(x), T, s);
    if (e == cudaSuccess) (*n)++;
    return e;
}

}  // namespace omoe

// ---------------------------------------------------------------------------
// Routing without any allocation.
//
// Some hosts of this library may not allocate device memory at the moment they
// need a routing decision: a serving loop that has handed all free memory to
// its own pool and forbids cudaMalloc on the request path (it would synchronise
// the device and may fail), or a caller inside a region where allocation calls
// are not permitted.  For them omoe_route_noalloc runs the same fused router
// kernel as omoe_forward, but keeps the kernel's scratch (logits, per-block
// histograms, in-block ranks) in a fixed array that is part of the library
// image instead of a cudaMalloc'd workspace.  Inputs and outputs are still the
// caller's buffers.
//
// The array is a host-side stand-in when named from host code; its device
// address is looked up once per device with cudaGetSymbolAddress, on the first
// call made while that device is current.
// ---------------------------------------------------------------------------

namespace omoe {
namespace {

constexpr int kNaMaxTokens = OMOE_NOALLOC_MAX_TOKENS;
constexpr size_t kNaLogitsBytes = sizeof(float) * (size_t)kNaMaxTokens * kMaxExperts;      // 2 MiB
constexpr size_t kNaBlocksBytes = sizeof(int32_t) * (size_t)(kNaMaxTokens / kRouterWarps) * kMaxExperts;  // 256 KiB
constexpr size_t kNaRankBytes = sizeof(int32_t) * (size_t)kNaMaxTokens * kMaxTopK;         // 256 KiB
constexpr size_t kNaScratchBytes = kNaLogitsBytes + kNaBlocksBytes + kNaRankBytes;

// Scratch shared by every omoe_route_noalloc call on a device (about 2.5 MiB,
// held by each GPU that loads the library until the process exits).
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNaScratchBytes];

constexpr int kNaMaxDevices = 64;
unsigned char *g_na_ptr[kNaMaxDevices] = {};  // device address of the array, per device ordinal

// counts[e] = sum over router blocks of block_counts[b][e]; one warp per expert.
__global__ void noalloc_counts_kernel(const int32_t *__restrict__ block_counts, int n_blocks, int E,
                                      int32_t *__restrict__ counts) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int e = warp; e < E; e += nwarps) {
        int sum = 0;
        for (int b = lane; b < n_blocks; b += 32) sum += block_counts[(size_t)e * n_blocks + b];
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if (lane == 0) counts[e] = sum;
    }
}

thread_local char g_na_err[256] = "";

int na_fail(int code, const char *msg, const char *detail = "") {
    snprintf(g_na_err, sizeof(g_na_err), "omoe_route_noalloc: %s%s", msg, detail);
    return code;
}

}  // namespace
}  // namespace omoe

extern "C" {

const char *omoe_route_noalloc_error(void) { return omoe::g_na_err; }

int omoe_route_noalloc(const void *x_dev, const float *w_router_dev, const float *router_bias_dev, int32_t T,
                       int32_t d_model, int32_t n_experts, int32_t top_k, int32_t renormalize, int32_t io_dtype,
                       int32_t *topk_idx_dev, float *topk_w_dev, int32_t *counts_dev, void *cuda_stream) {
    using namespace omoe;
    if (T < 0 || d_model <= 0 || n_experts <= 0 || top_k <= 0) return na_fail(OMOE_ERR_INVALID, "sizes must be positive");
    if (T > kNaMaxTokens || n_experts > kMaxExperts || top_k > kMaxTopK || top_k > n_experts) {
        char lim[128];
        snprintf(lim, sizeof(lim), " (limits: T <= %d, n_experts <= %d, top_k <= min(n_experts, %d))", kNaMaxTokens,
                 kMaxExperts, kMaxTopK);
        return na_fail(OMOE_ERR_TOO_LARGE, "the fixed scratch array is too small for this call", lim);
    }
    if (d_model % 8) return na_fail(OMOE_ERR_INVALID, "d_model must be a multiple of 8");
    if (io_dtype != OMOE_F32 && io_dtype != OMOE_BF16) return na_fail(OMOE_ERR_INVALID, "bad io_dtype");
    if (!counts_dev || (T > 0 && (!x_dev || !w_router_dev || !topk_idx_dev || !topk_w_dev)))
        return na_fail(OMOE_ERR_INVALID, "null buffer");

    // set-up, once per device, with that device current
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kNaMaxDevices)
        return na_fail(OMOE_ERR_CUDA, "cudaGetDevice failed or device ordinal out of range");
    if (g_na_ptr[dev] == nullptr) {
        void *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess || p == nullptr) return na_fail(OMOE_ERR_CUDA, "cudaGetSymbolAddress failed: ", cudaGetErrorString(e));
        g_na_ptr[dev] = static_cast<unsigned char *>(p);
    }
    unsigned char *scratch = g_na_ptr[dev];
    cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);

    // A stack handle that only carries what the router launcher reads; every
    // workspace pointer lands in the fixed array, every output in caller memory.
    omoe_handle hd;
    memset(&hd, 0, sizeof(hd));
    hd.cfg.d_model = d_model;
    hd.cfg.n_experts = n_experts;
    hd.cfg.top_k = top_k;
    hd.cfg.renormalize = renormalize;
    hd.w_router = const_cast<float *>(w_router_dev);
    hd.router_bias = const_cast<float *>(router_bias_dev);
    hd.logits = reinterpret_cast<float *>(scratch);
    hd.block_counts = reinterpret_cast<int32_t *>(scratch + kNaLogitsBytes);
    hd.pos = reinterpret_cast<int32_t *>(scratch + kNaLogitsBytes + kNaBlocksBytes);
    hd.topk_idx = topk_idx_dev;
    hd.topk_w = topk_w_dev;
    if (T > 0) {
        int n = 0;
        cudaError_t e = launch_router(&hd, x_dev, io_dtype, T, s, &n);
        if (e != cudaSuccess) return na_fail(OMOE_ERR_CUDA, "router launch failed: ", cudaGetErrorString(e));
    }
    const int n_blocks = T > 0 ? ceil_div(T, hd.tokens_per_block) : 0;
    // Nothing in the array has to start at zero: every router block writes all
    // n_experts entries of its histogram row, and only rows [0, n_blocks) are read.
    noalloc_counts_kernel<<<1, 256, 0, s>>>(hd.block_counts, n_blocks, n_experts, counts_dev);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return na_fail(OMOE_ERR_CUDA, "counts launch failed: ", cudaGetErrorString(e));
    g_na_err[0] = 0;
    return OMOE_OK;
}

}  // extern "C"
