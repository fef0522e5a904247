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
// is: lane l of a warp owns the elements i with (i/8)%32 == l and folds them
// with two fmaf chains, one over its even-numbered and one over its
// odd-numbered elements, each in ascending i; the lane's partial is even + odd;
// the 32 partials are then combined by an xor butterfly over distances
// 16,8,4,2,1; the bias is added last.  The two chains are the two halves of
// one packed fma.rn.f32x2, which halves the multiply-add instruction count of
// this issue-bound kernel.
//
// Data movement: a block covers TB tokens and walks d_model in steps of 256
// columns.  Each step's token rows [TB x 256] and router weights [E x 256] are
// brought into a ring of shared-memory stages with 16-byte cp.async copies, so
// several steps of HBM traffic are in flight while one is being folded in.  A
// warp holds TPW tokens x EPW experts of accumulators; with many experts ES
// warps share one token group and split the experts, so every weight read from
// shared memory feeds TPW tokens.
#include <stdlib.h>
#include <string.h>

#include <mutex>

#include "common.cuh"
#include "router_common.cuh"

namespace omoe {

namespace {

constexpr int kSub = 256;  // columns per step (32 lanes x 8)


__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Eight consecutive row elements as four (even, odd) fp32 pairs, each pair packed in 64 bits.
__device__ __forceinline__ void lds_pairs(const float *p, unsigned long long (&v)[4]) {
    const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p));
    asm volatile("ld.shared.v2.b64 {%0, %1}, [%2];" : "=l"(v[0]), "=l"(v[1]) : "r"(a));
    asm volatile("ld.shared.v2.b64 {%0, %1}, [%2];" : "=l"(v[2]), "=l"(v[3]) : "r"(a + 16));
}

__device__ __forceinline__ void lds_pairs(const __nv_bfloat16 *p, unsigned long long (&v)[4]) {
    uint4 r = *reinterpret_cast<const uint4 *>(p);
    uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        // a 32-bit word holds elements 2i (low half) and 2i+1 (high half); bf16 -> fp32 is a 16-bit shift
        asm("mov.b64 %0, {%1, %2};" : "=l"(v[i]) : "r"(w[i] << 16), "r"(w[i] & 0xffff0000u));
    }
}

// (acc.lo, acc.hi) = (x.lo * w.lo + acc.lo, x.hi * w.hi + acc.hi), each half an IEEE fused multiply-add
__device__ __forceinline__ void fma2(unsigned long long &acc, unsigned long long x, unsigned long long w) {
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(x), "l"(w));
}

// WT: element type of the router weights staged in shared memory.  float always works; __nv_bfloat16 is used
// when the weights were handed over as bf16 (every value is then exactly representable, so the logits keep
// every bit) and halves the bytes a block pulls from L2 per step, which is what bounds the kernel when there
// are many experts (a block re-reads all E rows for its 8 tokens).
template <int EMAX, int ES, int TPW, typename XT, typename WT = float>
struct RouterCfg {
    static constexpr int EPW = EMAX / ES;                 // experts per warp
    static constexpr int NG = kRouterWarps / ES;          // token groups per block
    static constexpr int TB = NG * TPW;                   // tokens per block
    // 256-column steps per stage: a stage reads NSUB*256 contiguous columns of every token row
    static constexpr int NSUB = 1;
    static constexpr int CS = NSUB * kSub;                // columns per stage
    static constexpr int XBYTES = TB * CS * (int)sizeof(XT);
    static constexpr int WBYTES = EMAX * CS * (int)sizeof(WT);
    static constexpr int STAGE = XBYTES + WBYTES;
    static constexpr int BUDGET = (EMAX <= 16) ? 100 * 1024 : 212 * 1024;  // two blocks per SM for few experts
    static constexpr int S0 = BUDGET / STAGE;
    static constexpr int S = S0 >= 4 ? 4 : (S0 < 1 ? 1 : S0);             // ring depth
    static constexpr int MINB = (S * STAGE <= 100 * 1024 && EPW * TPW <= 32) ? 2 : 1;
};

// EMAX: experts padded to a power of two (>= E); ES: warps sharing a token
// group; TPW: tokens per warp.
template <int EMAX, int ES, int TPW, typename XT, typename WT = float>
__global__ void __launch_bounds__(kRouterWarps * 32, RouterCfg<EMAX, ES, TPW, XT, WT>::MINB)
router_kernel(const XT *__restrict__ x, const WT *__restrict__ w_r, const float *__restrict__ bias,
              int T, int d, int E, int k, int renorm,
              float *__restrict__ logits, int32_t *__restrict__ topk_idx, float *__restrict__ topk_w,
              int32_t *__restrict__ block_counts, int32_t *__restrict__ local_rank) {
    using C = RouterCfg<EMAX, ES, TPW, XT, WT>;
    constexpr int EPW = C::EPW, TB = C::TB, S = C::S, NSUB = C::NSUB, CS = C::CS;
    constexpr bool WBF = sizeof(WT) == 2;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    // stage layout: x rows [TB][CS] XT, then weights [NSUB][2 halves][EMAX][32 lanes][4] fp32
    float *sl = reinterpret_cast<float *>(smem_raw + S * C::STAGE);  // [TB][EMAX] logits, later exp values
    int32_t *sidx = reinterpret_cast<int32_t *>(sl + TB * EMAX);      // [TB][k]
    const uint32_t smem_base = static_cast<uint32_t>(__cvta_generic_to_shared(smem_raw));
    pdl_trigger();
    pdl_wait();  // the step before may still be reading the routing arrays this kernel overwrites

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int grp = warp / ES, es = warp % ES;
    const int t0 = blockIdx.x * TB;
    // the bias is read once per block here, not once per accumulator behind a dependent global load
    float *sbias = reinterpret_cast<float *>(sidx + TB * kMaxTopK);
    for (int e = tid; e < EMAX; e += kRouterWarps * 32) sbias[e] = (bias != nullptr && e < E) ? __ldg(bias + e) : 0.f;
    const int nsub = (d + CS - 1) / CS;  // stages to walk

    // Copy pattern of a stage.  Thread tid copies 16-byte piece (tid % PPR) of token rows tid/PPR,
    // tid/PPR + 256/PPR, ... and float4 (tid % 64) of router rows tid/64, tid/64 + 4, ...: everything
    // but the stage's column offset is fixed per thread, so the addresses are set up once.
    static_assert(NSUB == 1, "the per-thread copy pattern below assumes one 256-column step per stage");
    constexpr int PPR = kSub * (int)sizeof(XT) / 16;      // 16-byte pieces per token row (32 bf16 / 64 fp32)
    constexpr int XROWS_PER_IT = kRouterWarps * 32 / PPR;  // token rows covered per pass of the block
    constexpr int XIT = (TB + XROWS_PER_IT - 1) / XROWS_PER_IT;
    // fp32 weights: 64 pieces per row, 4 rows per pass; bf16 weights: 32 pieces per row, 8 rows per pass, and a
    // piece is exactly one lane's 8 elements
    constexpr int WIT = WBF ? EMAX / 8 : EMAX / 4;
    const int x_row0 = tid / PPR, x_piece = tid % PPR;
    const int x_col = x_piece * (16 / (int)sizeof(XT));    // column inside the step
    const XT *x_src0 = x + (size_t)(t0 + x_row0) * d + x_col;
    const int w_e0 = WBF ? tid >> 5 : tid >> 6, w_q = WBF ? tid & 31 : tid & 63;
    const int w_col = WBF ? 8 * w_q : 4 * w_q;
    const WT *w_src0 = w_r + (size_t)w_e0 * d + w_col;
    const uint32_t w_dst0 = WBF ? C::XBYTES + (w_e0 * 32 + w_q) * 16  // [expert][lane] 16-byte chunks
                                : C::XBYTES + (((w_q & 1) * EMAX + w_e0) * 32 + (w_q >> 1)) * 16;  // lane-split layout
    constexpr int W_ROWS_PER_IT = WBF ? 8 : 4;
    auto issue_stage = [&](int su) {
        const uint32_t st = smem_base + (su % S) * C::STAGE;
        const int c0 = su * CS;
        const bool xcol_ok = c0 + x_col < d;  // d is a multiple of 8: a piece is whole or absent
#pragma unroll
        for (int it = 0; it < XIT; it++) {
            const int row = x_row0 + it * XROWS_PER_IT;
            if (XIT * XROWS_PER_IT == TB || row < TB) {
                const bool ok = xcol_ok && (t0 + row < T);
                const XT *src = ok ? x_src0 + (size_t)it * XROWS_PER_IT * d + c0 : x;
                cp_async16(st + (uint32_t)(tid + it * kRouterWarps * 32) * 16, src, ok ? 16 : 0);
            }
        }
        const bool wcol_ok = c0 + w_col < d;
#pragma unroll
        for (int it = 0; it < WIT; it++) {
            const bool ok = wcol_ok && (w_e0 + W_ROWS_PER_IT * it < E);
            const WT *src = ok ? w_src0 + (size_t)it * W_ROWS_PER_IT * d + c0 : w_r;
            cp_async16(st + w_dst0 + (uint32_t)it * (W_ROWS_PER_IT * 32 * 16), src, ok ? 16 : 0);
        }
    };

    unsigned long long acc[TPW][EPW];  // (even chain, odd chain) of every token x expert
#pragma unroll
    for (int i = 0; i < TPW; i++)
#pragma unroll
        for (int e = 0; e < EPW; e++) acc[i][e] = 0ull;

#pragma unroll
    for (int su = 0; su < S - 1; su++) {
        if (su < nsub) issue_stage(su);
        cp_async_commit();
    }
#pragma unroll 1
    for (int su = 0; su < nsub; su++) {
        if constexpr (S == 1) {
            issue_stage(su);
            cp_async_commit();
            cp_async_wait<0>();
        } else {
            cp_async_wait<S - 2>();  // this step's stage has landed (for this thread's copies)
        }
        __syncthreads();             // ... and for everyone's; all warps are done with the previous step
        if constexpr (S > 1) {
            if (su + S - 1 < nsub) issue_stage(su + S - 1);  // refill the stage consumed one step ago
            cp_async_commit();
        }
        const unsigned char *st = smem_raw + (su % S) * C::STAGE;
        const XT *xs = reinterpret_cast<const XT *>(st);
        const float *wst = reinterpret_cast<const float *>(st + C::XBYTES);
#pragma unroll 1
        for (int sub = 0; sub < NSUB; sub++) {
            if (su * CS + sub * kSub + lane * 8 >= d) break;  // ascending: later steps are absent too
            const float *ws = wst + sub * 2 * EMAX * 128;
            unsigned long long xv[TPW][4];
#pragma unroll
            for (int i = 0; i < TPW; i++) lds_pairs(xs + (grp * TPW + i) * CS + sub * kSub + lane * 8, xv[i]);
#pragma unroll
            for (int e = 0; e < EPW; e++) {
                const int eg = es * EPW + e;
                unsigned long long wv[4];
                if constexpr (WBF) {
                    lds_pairs(reinterpret_cast<const __nv_bfloat16 *>(wst) + (eg * 32 + lane) * 8, wv);
                } else {
                    const uint32_t wa = static_cast<uint32_t>(__cvta_generic_to_shared(ws + (eg * 32 + lane) * 4));
                    const uint32_t wb =
                        static_cast<uint32_t>(__cvta_generic_to_shared(ws + ((EMAX + eg) * 32 + lane) * 4));
                    asm volatile("ld.shared.v2.b64 {%0, %1}, [%2];" : "=l"(wv[0]), "=l"(wv[1]) : "r"(wa));
                    asm volatile("ld.shared.v2.b64 {%0, %1}, [%2];" : "=l"(wv[2]), "=l"(wv[3]) : "r"(wb));
                }
#pragma unroll
                for (int i = 0; i < TPW; i++)
#pragma unroll
                    for (int j = 0; j < 4; j++) fma2(acc[i][e], xv[i][j], wv[j]);
            }
        }
        if constexpr (S == 1) __syncthreads();
    }

    // xor butterfly over all accumulators first (independent chains overlap), then lane (e % 32) publishes logit e
    float red[TPW][EPW];
#pragma unroll
    for (int i = 0; i < TPW; i++)
#pragma unroll
        for (int e = 0; e < EPW; e++)
            red[i][e] = __uint_as_float((uint32_t)acc[i][e]) + __uint_as_float((uint32_t)(acc[i][e] >> 32));  // even + odd
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1)
#pragma unroll
        for (int i = 0; i < TPW; i++)
#pragma unroll
            for (int e = 0; e < EPW; e++) red[i][e] = red[i][e] + __shfl_xor_sync(0xffffffffu, red[i][e], m);
#pragma unroll
    for (int i = 0; i < TPW; i++)
#pragma unroll
        for (int e = 0; e < EPW; e++) {
            const int eg = es * EPW + e, tt = grp * TPW + i;
            if (lane == (e & 31) && eg < E) {
                float v = red[i][e];
                if (bias != nullptr) v = v + sbias[eg];
                sl[tt * EMAX + eg] = v;
                if (t0 + tt < T) logits[(size_t)(t0 + tt) * E + eg] = v;
            }
        }
    __syncthreads();

    // Softmax statistics, top-k on the logits, gate weights: a group of GW lanes per token
    // (8 lanes for up to 8 experts, so a warp works on 4 tokens at once).
    constexpr int GW = EMAX <= 8 ? 8 : (EMAX <= 16 ? 16 : 32);
    constexpr int PL = (EMAX + GW - 1) / GW;  // logits per lane
    constexpr int TPP = 32 / GW;              // tokens per warp pass
    static_assert(TB % TPP == 0, "a warp pass never straddles the end of the block's tokens");
    for (int tb = warp * TPP; tb < TB; tb += kRouterWarps * TPP) {
        const int tt = tb + lane / GW, gl = lane % GW;
        const int t = t0 + tt;
        const bool live = t < T;
        int my_e;
        float my_w;
        group_softmax_topk<PL, GW>(sl + tt * EMAX, E, k, renorm, gl, my_e, my_w);
        if (gl < k) {
            sidx[tt * k + gl] = live ? my_e : -1;
            if (live) {
                topk_idx[(size_t)t * k + gl] = my_e;
                topk_w[(size_t)t * k + gl] = my_w;
            }
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

template <int EMAX, int ES, int TPW, typename XT, typename WT = float>
cudaError_t launch_one(omoe_handle *h, const XT *x, int T, cudaStream_t s) {
    using C = RouterCfg<EMAX, ES, TPW, XT, WT>;
    const int k = h->cfg.top_k;
    size_t smem = (size_t)C::S * C::STAGE + sizeof(float) * C::TB * EMAX + sizeof(int32_t) * C::TB * kMaxTopK +
                  sizeof(float) * EMAX;
    auto kern = router_kernel<EMAX, ES, TPW, XT, WT>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    h->tokens_per_block = C::TB;  // the scan and dispatch kernels walk the histogram with this granularity
    int blocks = ceil_div(T, C::TB);
    const WT *w;
    if constexpr (sizeof(WT) == 2) w = h->w_router_bf16;
    else w = h->w_router;
    return launch_ex(kern, dim3(blocks), dim3(kRouterWarps * 32), smem, s, h->pdl, x, w, h->router_bias, T,
                     h->cfg.d_model, h->cfg.n_experts, k, h->cfg.renormalize, h->logits, h->topk_idx, h->topk_w,
                     h->block_counts, h->lrank);
}

// More tokens per warp reuse every router weight read from shared memory more
// often; fewer give more blocks.  Take the largest that still gives most SMs a block
// (measured on 2048 to 8192 tokens: fatter blocks beat fuller grids, the per-block
// prologue and epilogue being what they are).
template <int EMAX, int ES, typename XT, typename WT = float>
cudaError_t launch_tpw(omoe_handle *h, const XT *x, int T, cudaStream_t s) {
    // OMOE_ROUTER_FILL: blocks wanted per SM before a smaller tokens-per-warp is taken (tuning knob)
    static const float fill = getenv("OMOE_ROUTER_FILL") ? (float)atof(getenv("OMOE_ROUTER_FILL")) : 0.8f;
    const int want_blocks = (int)(fill * (float)(h->sm_count > 0 ? h->sm_count : 148));
    constexpr int NG = kRouterWarps / ES;
    // accumulators take 2 registers per (token, expert): 4 tokens x 16 experts per warp is the most that fits
    if constexpr (EMAX / ES <= 16)
        if (ceil_div(T, NG * 4) >= want_blocks) return launch_one<EMAX, ES, 4, XT, WT>(h, x, T, s);
    if (ceil_div(T, NG * 2) >= want_blocks) return launch_one<EMAX, ES, 2, XT, WT>(h, x, T, s);
    return launch_one<EMAX, ES, 1, XT, WT>(h, x, T, s);
}

template <typename XT>
cudaError_t launch_typed(omoe_handle *h, const XT *x, int T, cudaStream_t s) {
    const int E = h->cfg.n_experts;
    if (E <= 8) return launch_tpw<8, 1, XT>(h, x, T, s);
    // beyond 16 experts several warps share a token group, 16 experts each
    if (E <= 16) return launch_tpw<16, 1, XT>(h, x, T, s);
    // many experts: the weight rows a block re-reads per step dominate its traffic; stage them as bf16 when exact
    static const bool wbf_off = getenv("OMOE_ROUTER_W32") && atoi(getenv("OMOE_ROUTER_W32")) != 0;
    if (h->w_router_bf16 != nullptr && !wbf_off) {
        if (E <= 32) return launch_tpw<32, 2, XT, __nv_bfloat16>(h, x, T, s);
        if (E <= 64) return launch_tpw<64, 4, XT, __nv_bfloat16>(h, x, T, s);
        return launch_tpw<128, 8, XT, __nv_bfloat16>(h, x, T, s);
    }
    if (E <= 32) return launch_tpw<32, 2, XT>(h, x, T, s);
    if (E <= 64) return launch_tpw<64, 4, XT>(h, x, T, s);
    return launch_tpw<128, 8, XT>(h, x, T, s);
}

}  // namespace


// Smallest number of tokens one router block may cover (sizes the per-block histogram arrays).
int router_tokens_per_block(int E) { return E <= 16 ? kRouterWarps : (E <= 32 ? 4 : (E <= 64 ? 2 : 1)); }

cudaError_t launch_router(omoe_handle *h, const void *x, int io_dtype, int T, cudaStream_t s, int *n) {
    if ((reinterpret_cast<uintptr_t>(x) & 15u) != 0) return cudaErrorMisalignedAddress;  // 16-byte copies
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
// address is looked up with cudaGetSymbolAddress on the first call made in a
// CUDA context (one per device for runtime-API hosts; a host with its own
// driver-API contexts gets one look-up per context), with that context current.
// ---------------------------------------------------------------------------

namespace omoe {
namespace {

constexpr int kNaMaxTokens = OMOE_NOALLOC_MAX_TOKENS;
constexpr size_t kNaLogitsBytes = sizeof(float) * (size_t)kNaMaxTokens * kMaxExperts;      // 2 MiB
// a router block covers at least 1 token (128 experts), 2 (64), 4 (32) or 8 (16 and fewer)
constexpr size_t kNaBlocksBytes = sizeof(int32_t) * (size_t)kNaMaxTokens * kMaxExperts;  // 2 MiB
constexpr size_t kNaRankBytes = sizeof(int32_t) * (size_t)kNaMaxTokens * kMaxTopK;         // 256 KiB
constexpr size_t kNaScratchBytes = kNaLogitsBytes + kNaBlocksBytes + kNaRankBytes;

// Scratch shared by every omoe_route_noalloc call on a device (about 4.3 MiB,
// held by each GPU that loads the library until the process exits).
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNaScratchBytes];

// Device address of the array, per CUDA context.  A __device__ symbol is instantiated once per context that
// loads the module, not once per device ordinal: a host that created its own driver-API context (the
// reference engine does, CUDAUtils.java:124-130) and the primary context of the same device each have their
// own copy, so the cache is keyed by the context that is current at the call.
constexpr int kNaMaxContexts = 64;
struct NaSlot {
    void *ctx;
    unsigned char *ptr;
};
NaSlot g_na_slots[kNaMaxContexts] = {};
int g_na_used = 0;
std::mutex g_na_mutex;

typedef CUresult (*CtxGetCurrentFn)(CUcontext *);
CtxGetCurrentFn na_ctx_fn() {
    static CtxGetCurrentFn fn = nullptr;
    if (fn) return fn;
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuCtxGetCurrent", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
        return nullptr;
    fn = reinterpret_cast<CtxGetCurrentFn>(p);
    return fn;
}

// Address of the scratch array in the current context; looks it up (and, under lazy module loading, makes
// the runtime load this library's module into the context) the first time a context is seen.
cudaError_t na_scratch(unsigned char **out) {
    *out = nullptr;
    CtxGetCurrentFn get = na_ctx_fn();
    CUcontext ctx = nullptr;
    if (get && get(&ctx) == CUDA_SUCCESS && ctx != nullptr) {
        std::lock_guard<std::mutex> lock(g_na_mutex);
        for (int i = 0; i < g_na_used; i++)
            if (g_na_slots[i].ctx == ctx) {
                *out = g_na_slots[i].ptr;
                return cudaSuccess;
            }
    }
    void *p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess) return e;
    if (p == nullptr) return cudaErrorInvalidSymbol;
    // the runtime call above binds the primary context when the thread had none; ask again
    if (ctx == nullptr && get) get(&ctx);
    if (ctx != nullptr) {
        std::lock_guard<std::mutex> lock(g_na_mutex);
        if (g_na_used < kNaMaxContexts) g_na_slots[g_na_used++] = NaSlot{ctx, static_cast<unsigned char *>(p)};
        // table full: later calls from further contexts look the address up every time (still no allocation)
    }
    *out = static_cast<unsigned char *>(p);
    return cudaSuccess;
}

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

    // rows and router weights move as 16-byte vectors; a misaligned address would raise a sticky device fault
    if (T > 0 && (((reinterpret_cast<uintptr_t>(x_dev) | reinterpret_cast<uintptr_t>(w_router_dev)) & 15u) != 0))
        return na_fail(OMOE_ERR_INVALID, "x_dev and w_router_dev must be 16-byte aligned");
    if (((reinterpret_cast<uintptr_t>(topk_idx_dev) | reinterpret_cast<uintptr_t>(topk_w_dev) |
          reinterpret_cast<uintptr_t>(counts_dev) | reinterpret_cast<uintptr_t>(router_bias_dev)) & 3u) != 0)
        return na_fail(OMOE_ERR_INVALID, "output and bias buffers must be 4-byte aligned");

    // set-up, once per context, with that context current
    unsigned char *scratch = nullptr;
    {
        cudaError_t e = na_scratch(&scratch);
        if (e != cudaSuccess) return na_fail(OMOE_ERR_CUDA, "cudaGetSymbolAddress failed: ", cudaGetErrorString(e));
    }
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
    hd.lrank = reinterpret_cast<int32_t *>(scratch + kNaLogitsBytes + kNaBlocksBytes);
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
