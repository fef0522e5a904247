// Prefix sums over the per-block expert histograms and the dispatch copy of
// token rows into per-expert contiguous buffers.
//
// No reference kernel exists for this stage; the nearest precedent is the row
// gather EmbeddingFW (src/main/resources/cu/EmbeddingKernel.cu:13-33), which
// carries indices as floats — here every index is int32.
//
// Layout produced: rows of expert e start at poffsets[e], a multiple of 128, so
// a 128-row tensor-core tile belongs to exactly one expert; inside an expert
// rows keep the order of the flat pick index t*k+j (stable), which is what
// makes the permutation reproducible bit for bit.
#include "common.cuh"
#include "scan.cuh"

namespace omoe {

namespace {

__global__ void __launch_bounds__(1024)
scan_kernel(const int32_t *__restrict__ block_counts, int32_t *__restrict__ block_base, int n_blocks, int E,
            int32_t *__restrict__ counts, int32_t *__restrict__ offsets,
            int32_t *__restrict__ poffsets, int32_t *__restrict__ tile_expert, int max_tiles) {
    __shared__ int32_t s_cnt[kMaxExperts];
    __shared__ int32_t s_poff[kMaxExperts + 1];
    pdl_trigger();
    pdl_wait();
    scan_body(block_counts, block_base, n_blocks, E, counts, offsets, poffsets, tile_expert, max_tiles, s_cnt, s_poff);
}

// One warp per token: finalise the k row positions, read the token's row once
// and write it to its k places with 16-byte stores.
// Rows go to the dispatch buffer of the rank that owns the expert: row_table[q]
// is that buffer's base (this GPU's own for q == rank, a peer-mapped NVLink
// address otherwise), dst_base[e] the first row reserved there for this rank's
// picks of expert e.
template <typename XT, typename OT>
__global__ void __launch_bounds__(256)
permute_kernel(const XT *__restrict__ x, void *const *__restrict__ row_table, const int32_t *__restrict__ topk_idx,
               const int32_t *__restrict__ lrank, int32_t *__restrict__ pos, const int32_t *__restrict__ block_base,
               const int32_t *__restrict__ dst_base, int T, int d, int n_blocks, int e_local, int k, int tokens_per_block,
               EpSignal sig, int32_t *ticket, int rows_cap, int32_t *dev_err, int pass) {
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    pdl_trigger();
    pdl_wait();
    int my = 0, owner = 0;
    if (t < T && lane < k) {
        int f = t * k + lane;
        int e = topk_idx[f];
        int b = t / tokens_per_block;
        my = dst_base[e] + block_base[(size_t)e * n_blocks + b] + lrank[f];
        owner = e / e_local;
        // No row outside the owner's buffer is ever touched: a step the count exchange refused gives negative
        // positions (nothing moves, consumers skip the pick); a position beyond the capacity cannot follow
        // from an accepted layout and is reported.
        if (my >= rows_cap) {
            atomicOr(dev_err, kDevErrBounds);
            my = -1;
        } else if (my < 0) {
            my = -1;
        }
        if (blockIdx.y == 0 && pass != 2) pos[f] = my;
    }
    if (t < T) {
    OT *dst[kMaxTopK];
    bool any = false;  // a token none of whose picks belongs to this pass is not read at all
#pragma unroll
    for (int j = 0; j < kMaxTopK; j++) {
        int row = __shfl_sync(0xffffffffu, my, j);
        int q = __shfl_sync(0xffffffffu, owner, j);
        // pass 1 moves only the picks whose expert this rank owns, pass 2 only the others (0: all of them)
        const bool mine = pass == 0 || ((pass == 1) == (q == sig.rank));
        dst[j] = (j < k && row >= 0 && mine) ? static_cast<OT *>(row_table[q]) + (size_t)row * d : nullptr;
        any = any || dst[j] != nullptr;
    }
    if (any) {

    // blockIdx.y walks one slice of the row (more warps in flight when there are few tokens)
    const int cw = ((d / (int)gridDim.y + 7) / 8) * 8;
    const int c_lo = blockIdx.y * cw, c_hi = min(d, c_lo + cw);
    const XT *src = x + (size_t)t * d;
    if constexpr (sizeof(XT) == sizeof(OT)) {
        constexpr int V = 16 / sizeof(XT);
        // four 16-byte loads in flight per lane before the first store (the loads are the latency here)
        for (int c0 = c_lo + lane * V; c0 < c_hi; c0 += 4 * 32 * V) {
            uint4 v[4];
#pragma unroll
            for (int u = 0; u < 4; u++)
                if (c0 + u * 32 * V < c_hi) v[u] = __ldg(reinterpret_cast<const uint4 *>(src + c0 + u * 32 * V));
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int c = c0 + u * 32 * V;
                if (c < c_hi) {
#pragma unroll
                    for (int j = 0; j < kMaxTopK; j++)
                        if (j < k && dst[j] != nullptr) *reinterpret_cast<uint4 *>(dst[j] + c) = v[u];
                }
            }
        }
    } else {
        // fp32 rows in, bf16 rows out: 8 elements per lane per step
        for (int c = c_lo + lane * 8; c < c_hi; c += 32 * 8) {
            float4 a = __ldg(reinterpret_cast<const float4 *>(src + c));
            float4 b = __ldg(reinterpret_cast<const float4 *>(src + c) + 1);
            uint4 v;
            v.x = pack_bf16(a.x, a.y);
            v.y = pack_bf16(a.z, a.w);
            v.z = pack_bf16(b.x, b.y);
            v.w = pack_bf16(b.z, b.w);
#pragma unroll
            for (int j = 0; j < kMaxTopK; j++)
                if (j < k && dst[j] != nullptr) *reinterpret_cast<uint4 *>(dst[j] + c) = v;
        }
    }
    }  // any
    }
    if (sig.flags != nullptr) {
        // Expert parallel: make this block's rows visible system-wide, take a
        // ticket, and let the last block raise "rows have landed" on every rank.
        __threadfence_system();
        __syncthreads();
        __shared__ int s_last;
        if (threadIdx.x == 0) s_last = (atomicAdd(ticket, 1) == (int)(gridDim.x * gridDim.y) - 1);
        __syncthreads();
        // pass 1 has completed this rank's own rows only: it tells this rank alone; pass 2 tells the others
        if (s_last && (int)threadIdx.x < sig.world &&
            (pass == 0 || ((pass == 1) == ((int)threadIdx.x == sig.rank)))) {
            __threadfence_system();
            uint32_t *f = sig.flags[threadIdx.x] + sig.rank;
            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(*sig.seq) : "memory");
        }
        // every block has arrived: leave the counter at zero for whichever kernel uses it next (a decode step's
        // one-launch routing counts its blocks with it and does not pass through the count-exchange kernel)
        if (s_last && threadIdx.x == 0) *ticket = 0;
    }
}

// perm[offsets[e] + (pos[f] - dst_base[e])] = f : the unpadded permutation of this rank's picks.
__global__ void perm_readout_kernel(const int32_t *__restrict__ topk_idx, const int32_t *__restrict__ pos,
                                    const int32_t *__restrict__ offsets, const int32_t *__restrict__ poffsets /* dst_base */,
                                    int32_t *__restrict__ perm, int n) {
    int f = blockIdx.x * blockDim.x + threadIdx.x;
    if (f >= n) return;
    int e = topk_idx[f];
    if (pos[f] < 0) return;  // a refused expert-parallel step placed no row
    perm[offsets[e] + (pos[f] - poffsets[e])] = f;
}

}  // namespace

cudaError_t launch_scan(omoe_handle *h, int T, cudaStream_t s, int *n) {
    int n_blocks = ceil_div(T, h->tokens_per_block);
    int max_tiles = (int)(h->rows_cap / kRowAlign);
    (*n)++;
    return launch_ex(scan_kernel, dim3(1), dim3(1024), 0, s, h->pdl, h->block_counts, h->block_base, n_blocks,
                     h->cfg.n_experts, h->counts, h->offsets, h->poffsets, h->tile_expert, max_tiles);
}

cudaError_t launch_permute(omoe_handle *h, const void *x, int io_dtype, int T, cudaStream_t s, int *n,
                           const EpSignal *sig, int pass) {
    const int d = h->cfg.d_model, k = h->cfg.top_k, El = h->e_local;
    const int nb = ceil_div(T, h->tokens_per_block);
    const int wpb = 8;
    // enough warps to keep every SM's memory pipes busy: split rows when there are few tokens
    int split = 1;
    while (split < 8 && (long long)T * split < 32LL * h->sm_count && d / (split * 2) >= 512) split *= 2;
    dim3 grid(ceil_div(T, wpb), split), block(wpb * 32);
    const bool cbf = h->cfg.compute_dtype == OMOE_BF16;
    EpSignal sg = sig ? *sig : EpSignal{nullptr, 1, 0, 0};
    const bool pdl = h->pdl;
    cudaError_t e;
#define OMOE_PERMUTE(XT, OT)                                                                                        \
    e = launch_ex(permute_kernel<XT, OT>, grid, block, 0, s, pdl, static_cast<const XT *>(x), h->d_row_table,       \
                  h->topk_idx, h->lrank, h->pos, h->block_base, h->dst_base, T, d, nb, El, k, h->tokens_per_block,  \
                  sg, h->ticket, (int)h->rows_cap, h->dev_err, pass)
    if (io_dtype == OMOE_F32 && !cbf) OMOE_PERMUTE(float, float);
    else if (io_dtype == OMOE_F32 && cbf) OMOE_PERMUTE(float, __nv_bfloat16);
    else if (io_dtype == OMOE_BF16 && cbf) OMOE_PERMUTE(__nv_bfloat16, __nv_bfloat16);
    else return cudaErrorInvalidValue;  // bf16 rows into an fp32 layer are rejected by the API
#undef OMOE_PERMUTE
    if (e == cudaSuccess) (*n)++;
    return e;
}

cudaError_t launch_perm_readout(omoe_handle *h, int T, cudaStream_t s) {
    int n = T * h->cfg.top_k;
    if (n == 0) return cudaSuccess;
    perm_readout_kernel<<<ceil_div(n, 256), 256, 0, s>>>(h->topk_idx, h->pos, h->offsets, h->dst_base,
                                                         h->perm_out, n);
    return cudaGetLastError();
}

}  // namespace omoe
