// Routing and dispatch of a decode step (a handful of tokens) in ONE launch.
//
// With T <= 8 the separate router, scan and dispatch kernels are pure launch and
// dependent-load latency (about 40 us for work that takes a few).  Here block t
// computes token t's logits (eight warps split the experts), picks its experts,
// and the block that finishes last turns all picks into counts, offsets, row
// positions and the tile table, then copies the token rows into the dispatch
// buffer.  Outputs are the same arrays, with the same contents, as the
// three-kernel path; the logits follow the same fixed reduction tree, so the
// routing stays bit-exact.  Single GPU only (expert-parallel steps need the
// count exchange between the two halves).
#include "route_small.cuh"

namespace omoe {

namespace {

using namespace small;

template <int PL, typename XT>
__global__ void __launch_bounds__(256)
route_small_kernel(const XT *__restrict__ x, const float *__restrict__ w_r, const float *__restrict__ bias, int T, int d,
                   int E, int k, int renorm, float *__restrict__ logits, int32_t *__restrict__ topk_idx,
                   float *__restrict__ topk_w, int32_t *__restrict__ counts, int32_t *__restrict__ offsets,
                   int32_t *__restrict__ poffsets, int32_t *__restrict__ tile_expert, int max_tiles,
                   int32_t *__restrict__ pos, __nv_bfloat16 *__restrict__ xp, int32_t *ticket) {
    __shared__ float sl[kMaxExperts];
    __shared__ int32_t s_idx[kSmallMaxPicks], s_rank[kSmallMaxPicks], s_pos[kSmallMaxPicks];
    __shared__ int32_t s_cnt[kMaxExperts], s_poff[kMaxExperts + 1];
    __shared__ int s_last;
    const int tid = threadIdx.x;
    const int t = blockIdx.x;
    pdl_trigger();
    pdl_wait();  // the step before may still be reading the routing arrays this kernel overwrites

    token_logits_topk<PL, XT>(x, w_r, bias, t, d, E, k, renorm, logits, topk_idx, topk_w, sl);
    // ---- the block that finishes last does the scan and the dispatch ----
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = (atomicAdd(ticket, 1) == (int)gridDim.x - 1);
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const int n = T * k;
    if (tid < n) s_idx[tid] = __ldcg(topk_idx + tid);
    __syncthreads();
    rank_picks(n, E, s_idx, s_rank, s_cnt);
    __syncthreads();
    if (tid == 0) {
        int off = 0, poff = 0;
        for (int e = 0; e < E; e++) {
            const int c = s_cnt[e];
            counts[e] = c;
            offsets[e] = off;
            poffsets[e] = poff;
            s_poff[e] = poff;
            off += c;
            poff += (c + kRowAlign - 1) / kRowAlign * kRowAlign;
        }
        offsets[E] = off;
        poffsets[E] = poff;
        s_poff[E] = poff;
        *ticket = 0;  // ready for the next step
    }
    __syncthreads();
    const int n_tiles = s_poff[E] / kRowAlign;
    for (int i = tid; i < max_tiles; i += blockDim.x) {
        int ex = -1;
        if (i < n_tiles) {
            const int row = i * kRowAlign;
            ex = 0;
            while (ex + 1 < E && s_poff[ex + 1] <= row) ex++;
        }
        tile_expert[i] = ex;
    }
    if (tid < n) {
        const int p = s_poff[s_idx[tid]] + s_rank[tid];
        s_pos[tid] = p;
        pos[tid] = p;
    }
    __syncthreads();
    // copy the token rows to their k places (bf16 rows out; fp32 rows are converted)
    const int vec = d / 8;  // 8 elements per step
    for (int i = tid; i < T * vec; i += blockDim.x) {
        const int tt = i / vec, c = (i % vec) * 8;
        float v[8];
        ldg8(x + (size_t)tt * d + c, v);
        uint4 o;
        o.x = pack_bf16(v[0], v[1]);
        o.y = pack_bf16(v[2], v[3]);
        o.z = pack_bf16(v[4], v[5]);
        o.w = pack_bf16(v[6], v[7]);
        for (int j = 0; j < k; j++)
            *reinterpret_cast<uint4 *>(xp + (size_t)s_pos[tt * k + j] * d + c) = o;
    }
}

template <typename XT>
cudaError_t launch_typed(omoe_handle *h, const XT *x, int T, cudaStream_t s) {
    const int E = h->cfg.n_experts;
    const int max_tiles = (int)(h->rows_cap / kRowAlign);
    cudaError_t e;
#define OMOE_RS(PLV)                                                                                             \
    e = launch_ex(route_small_kernel<PLV, XT>, dim3(T), dim3(256), 0, s, h->pdl, x, h->w_router, h->router_bias, T, \
                  h->cfg.d_model, E, h->cfg.top_k, h->cfg.renormalize, h->logits, h->topk_idx, h->topk_w, h->counts, \
                  h->offsets, h->poffsets, h->tile_expert, max_tiles, h->pos, static_cast<__nv_bfloat16 *>(h->xp),  \
                  h->ticket)
    if (E <= 32) OMOE_RS(1);
    else if (E <= 64) OMOE_RS(2);
    else OMOE_RS(4);
#undef OMOE_RS
    return e;
}

}  // namespace

int route_small_max_tokens() { return kSmallMaxTokens; }

cudaError_t launch_route_small(omoe_handle *h, const void *x, int io_dtype, int T, cudaStream_t s, int *n) {
    if ((reinterpret_cast<uintptr_t>(x) & 15u) != 0) return cudaErrorMisalignedAddress;
    cudaError_t e = io_dtype == OMOE_F32 ? launch_typed<float>(h, static_cast<const float *>(x), T, s)
                                         : launch_typed<__nv_bfloat16>(h, static_cast<const __nv_bfloat16 *>(x), T, s);
    if (e == cudaSuccess) (*n)++;
    return e;
}

}  // namespace omoe
