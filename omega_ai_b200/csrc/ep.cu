// Expert-parallel transport over NVLink peer memory.
//
// The reference's only multi-GPU mechanism is cudaMemcpyPeerAsync between Java
// threads, driven from the host (src/main/java/com/omega/engine/parallel/dp/
// NetworkRunnable.java:442-459).  Here each rank is a process on one GPU and
// the kernels themselves move the rows: the dispatch kernel stores every token
// row straight into the dispatch buffer of the rank that owns the expert, and
// the combine kernel loads the expert outputs back from the owners' buffers.
// Buffers are shared between processes with CUDA IPC handles; no host
// synchronisation happens inside a forward, and no collective library is used.
//
// One forward (sequence number seq) on every rank:
//   1. router                                 (local)
//   2. scan + count exchange (one kernel): publish my per-expert counts to
//      every rank, wait for all rows of the count matrix, derive where my picks
//      go on each owner (dst_base) and how the rows I receive are laid out
//      (ex_* arrays, and for every 128-row tile the set of ranks its rows come from)
//   3. dispatch: rows -> owners' buffers, then "rows landed" flag to every rank
//      (a decode step of <= 8 tokens does 1-3 in ONE launch; a large step
//      moves only the rows this rank keeps here and leaves the rest to 4)
//   4. up/gate product: its producer thread waits, tile by tile, only for the
//      ranks whose rows the tile holds, and walks the tiles that hold only local
//      rows first; in a large step two extra warps of every CTA carry this
//      rank's rows for the OTHER ranks across NVLink meanwhile (peer stores
//      in the same kernel as the tensor-core tiles); no separate wait launch
//   5. down product; the CTA that finishes last raises "outputs ready" on
//      every rank; no separate signal launch
//   6. combine: wait for all owners' flags, gather rows over NVLink
// Flags carry the sequence number, so nothing is reset between forwards; the
// count matrix is double-buffered by the parity of seq.  Every wait is bounded
// and reports through the device error word instead of hanging.
#include <stdlib.h>
#include <string.h>

#include "ep.cuh"
#include "backward.cuh"
#include "route_small.cuh"
#include "scan.cuh"

namespace omoe {

namespace {

struct EpState {
    EpCtl *ctl;                 // this rank's control block (device)
    EpCtl **d_ctl_table;        // device [world]
    uint32_t **d_rows_flags;    // device [world]: &peer_ctl[q]->flag_rows[0]
    uint32_t **d_out_flags;     // device [world]: &peer_ctl[q]->flag_out[0]
    int32_t *ex_counts, *ex_poffsets, *ex_tile_expert;  // layout of the rows this rank receives
    uint32_t *ex_tile_mask;     // [m tiles] bit s: the tile holds rows that source rank s sent
    int32_t *ex_tile_order;     // [m tiles] walk order of the tiles: this rank's own rows first
    long overlap_min_bytes;     // smallest dispatch (bytes of rows) whose remote half travels inside the product
    void *peer_ptrs[kMaxWorld][5];  // opened IPC mappings (ctl, xp, yp, dyp, dxp), null for self
    void *dyp, *dxp;            // [rows_cap, d] gradient rows of the backward pass (peers write dyp, read dxp)
    void **d_dyp_table, **d_dxp_table;  // device [world]
    bool imported;
    uint32_t *d_seq;  // device: sequence number of the last step started on this rank
    unsigned long long timeout_ns;
};

struct IpcBlob {
    cudaIpcMemHandle_t ctl, xp, yp, dyp, dxp;
};
static_assert(sizeof(IpcBlob) == OMOE_EP_BLOB_BYTES, "blob size is part of the ABI");

__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Shared memory of the count exchange.
struct ExSmem {
    int32_t cnt[kMaxWorld][kMaxExperts];
    int32_t tot[kMaxExperts];
    int32_t rpoff[kMaxExperts + kMaxWorld];  // padded start of expert e in its owner's buffer
    int32_t mypoff[kMaxExperts + 1];
    int32_t base[kMaxExperts];               // dst_base of this rank
    // tiles that hold nothing but this rank's own rows, per local expert: how many, the first one, and the
    // running sums that place them (and the other tiles) in the walk order
    int32_t nloc[kMaxExperts], afirst[kMaxExperts], loc_pre[kMaxExperts], rem_pre[kMaxExperts];
    int n_loc_total;
    int bad;
    uint32_t seq;
};

// Arguments of the count exchange that do not change from step to step.
struct ExArgs {
    EpCtl *self;
    EpCtl *const *peers;
    int W, r, E, El;
    uint32_t *seq_ptr;
    int rows_cap;
    int32_t *dst_base, *ex_counts, *ex_poffsets, *ex_tile_expert;
    uint32_t *ex_tile_mask;
    int32_t *ex_tile_order;
    int max_tiles;
    int32_t *ticket, *dev_err;
    unsigned long long timeout_ns;
};

// The count exchange, by one block (any number of threads >= world).  A new step begins here: the sequence
// number advances (this is the first piece of a step to need it, the later kernels read it).  Publishes this
// rank's per-expert counts to every rank, waits (bounded) for all rows of the count matrix, and derives: where
// this rank's picks of every expert start in the owner's buffer (dst_base; sm.base keeps a copy), and how the
// rows this rank receives are laid out (ex_counts, ex_poffsets, ex_tile_expert, ex_tile_mask).  A step that
// does not fit some owner's buffer is refused by every rank alike.  counts: this rank's counts [E] (global or
// shared memory, complete and visible to the whole block on entry).
__device__ void exchange_body(ExSmem &sm, const ExArgs &a, const int32_t *counts) {
    const int tid = threadIdx.x, nt = blockDim.x;
    const int W = a.W, r = a.r, E = a.E, El = a.El;
    if (tid == 0) { sm.seq = *a.seq_ptr + 1u; *a.seq_ptr = sm.seq; *a.ticket = 0; sm.bad = 0; }
    __syncthreads();
    const uint32_t seq = sm.seq;
    const int par = seq & 1u;
    // publish my counts to every rank (my own included)
    for (int i = tid; i < W * E; i += nt) {
        int q = i / E, e = i % E;
        a.peers[q]->cnt[par][r][e] = counts[e];
    }
    __threadfence_system();
    __syncthreads();
    if (tid < W) st_release_sys(&a.peers[tid]->flag_cnt[par][r], seq);
    // wait for every source's row
    if (tid < W) {
        if (!ep_wait_flag(&a.self->flag_cnt[par][tid], seq, a.timeout_ns, a.dev_err)) sm.bad = 1;
    }
    __syncthreads();
    __threadfence_system();
    for (int i = tid; i < W * E; i += nt) {
        int s = i / E, e = i % E;
        sm.cnt[s][e] = *(volatile int32_t *)&a.self->cnt[par][s][e];
    }
    __syncthreads();
    for (int e = tid; e < E; e += nt) {
        int t = 0;
        for (int s = 0; s < W; s++) t += sm.cnt[s][e];
        sm.tot[e] = t;
    }
    __syncthreads();
    if (tid < W) {  // thread q lays out owner q's buffer
        int q = tid, off = 0;
        for (int le = 0; le < El; le++) {
            int e = q * El + le;
            sm.rpoff[e] = off;
            off += (sm.tot[e] + kRowAlign - 1) / kRowAlign * kRowAlign;
        }
        if (off > a.rows_cap) sm.bad = 1;  // every rank sees the same matrix, so all of them refuse together
        if (q == r) {
            for (int le = 0; le < El; le++) sm.mypoff[le] = sm.rpoff[q * El + le];
            sm.mypoff[El] = off;
        }
    }
    __syncthreads();
    const bool bad = sm.bad != 0;
    if (bad && tid == 0) atomicOr(a.dev_err, kDevErrBounds);
    for (int e = tid; e < E; e += nt) {
        int before = 0;
        for (int s = 0; s < r; s++) before += sm.cnt[s][e];
        // a refused step moves no row: the base is far below zero, so every position the dispatch derives from
        // it is negative, and the dispatch, combine and backward kernels skip rows with a negative position
        const int b = bad ? kRefusedBase : sm.rpoff[e] + before;
        sm.base[e] = b;
        a.dst_base[e] = b;
    }
    for (int le = tid; le < El; le += nt) {
        a.ex_counts[le] = bad ? 0 : sm.tot[r * El + le];
        a.ex_poffsets[le] = bad ? 0 : sm.mypoff[le];
    }
    if (tid == 0) a.ex_poffsets[El] = bad ? 0 : sm.mypoff[El];
    const int n_tiles = bad ? 0 : sm.mypoff[El] / kRowAlign;
    for (int le = tid; le < El; le += nt) {
        sm.nloc[le] = 0;
        sm.afirst[le] = 0x7fffffff;
    }
    __syncthreads();
    for (int i = tid; i < a.max_tiles; i += nt) {
        int ex = -1;
        uint32_t mask = 0;
        if (i < n_tiles) {
            const int row = i * kRowAlign;
            ex = 0;
            while (ex + 1 < El && sm.mypoff[ex + 1] <= row) ex++;
            // rows [lo, lo + 128) of the expert's segment; source s holds [before_s, before_s + cnt_s) of it
            const int lo = row - sm.mypoff[ex], hi = lo + kRowAlign;
            int before = 0;
            for (int s = 0; s < W; s++) {
                const int c = sm.cnt[s][r * El + ex];
                if (c > 0 && before < hi && before + c > lo) mask |= 1u << s;
                before += c;
            }
        }
        a.ex_tile_expert[i] = ex;
        a.ex_tile_mask[i] = mask;
        if (mask == (1u << r)) {  // only this rank's own rows (a contiguous run of tiles inside the expert)
            atomicAdd(&sm.nloc[ex], 1);
            atomicMin(&sm.afirst[ex], i);
        }
    }
    __syncthreads();
    // Walk order of the tiles: first the tiles that hold only this rank's own rows (they are complete as soon as
    // the local pass of the dispatch is, before anything has crossed NVLink), expert by expert, then the others
    // in buffer order.  Tiles of one expert stay together, so a band of tiles still shares its weight tiles.
    if (tid == 0) {
        int L = 0, R = 0;
        for (int le = 0; le < El; le++) {
            sm.loc_pre[le] = L;
            sm.rem_pre[le] = R;
            L += sm.nloc[le];
            R += (sm.mypoff[le + 1] - sm.mypoff[le]) / kRowAlign - sm.nloc[le];
        }
        sm.n_loc_total = L;
    }
    __syncthreads();
    for (int i = tid; i < n_tiles; i += nt) {
        const int ex = a.ex_tile_expert[i];  // written above by this same thread
        int p;
        if (a.ex_tile_mask[i] == (1u << r)) {
            p = sm.loc_pre[ex] + (i - sm.afirst[ex]);
        } else {
            int j = i - sm.mypoff[ex] / kRowAlign;
            if (sm.nloc[ex] > 0 && i > sm.afirst[ex]) j -= sm.nloc[ex];
            p = sm.n_loc_total + sm.rem_pre[ex] + j;
        }
        a.ex_tile_order[p] = i;
    }
    __syncthreads();
}

// Scan of the router's per-block histograms and the count exchange in one launch (one block of 1024 threads).
__global__ void __launch_bounds__(1024)
ep_scan_exchange_kernel(const int32_t *__restrict__ block_counts, int32_t *__restrict__ block_base, int n_blocks,
                        int32_t *__restrict__ counts, int32_t *__restrict__ offsets, int32_t *__restrict__ poffsets,
                        int32_t *__restrict__ tile_expert, const ExArgs a) {
    __shared__ ExSmem sm;
    __shared__ int32_t s_cnt[kMaxExperts];
    __shared__ int32_t s_poff[kMaxExperts + 1];
    // the local tile table is not used with expert parallelism (the expert kernels read the ex_* arrays)
    scan_body(block_counts, block_base, n_blocks, a.E, counts, offsets, poffsets, tile_expert, 0, s_cnt, s_poff);
    __syncthreads();
    exchange_body(sm, a, s_cnt);
}

// A decode step under expert parallelism in ONE launch: block t computes token t's logits and picks (as the
// one-GPU route_small_kernel does); the block that finishes last ranks the picks, runs the count exchange,
// stores every token row straight into the dispatch buffer of the rank that owns the pick's expert (peer
// stores) and raises "rows have landed" on every rank.  T <= 8 tokens on this rank (0 is allowed: the grid is
// one block that only takes part in the exchange).
template <int PL, typename XT>
__global__ void __launch_bounds__(256)
route_small_ep_kernel(const XT *__restrict__ x, const float *__restrict__ w_r, const float *__restrict__ bias, int T,
                      int d, int k, int renorm, float *__restrict__ logits, int32_t *__restrict__ topk_idx,
                      float *__restrict__ topk_w, int32_t *__restrict__ counts, int32_t *__restrict__ offsets,
                      int32_t *__restrict__ pos, void *const *__restrict__ row_table, uint32_t *const *rows_flags,
                      int32_t *ticket_blocks, const ExArgs a) {
    using namespace small;
    __shared__ ExSmem sm;
    __shared__ float sl[kMaxExperts];
    __shared__ int32_t s_idx[kSmallMaxPicks], s_rank[kSmallMaxPicks], s_pos[kSmallMaxPicks];
    __shared__ int32_t s_cnt[kMaxExperts];
    __shared__ int s_last;
    const int tid = threadIdx.x;
    const int t = blockIdx.x;
    const int E = a.E;
    pdl_trigger();
    pdl_wait();  // the step before may still be reading the routing arrays this kernel overwrites
    if (t < T) token_logits_topk<PL, XT>(x, w_r, bias, t, d, E, k, renorm, logits, topk_idx, topk_w, sl);
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = (atomicAdd(ticket_blocks, 1) == (int)gridDim.x - 1);
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (tid == 0) *ticket_blocks = 0;  // ready for the next step
    const int n = T * k;
    if (tid < n) s_idx[tid] = __ldcg(topk_idx + tid);
    __syncthreads();
    rank_picks(n, E, s_idx, s_rank, s_cnt);
    __syncthreads();
    if (tid == 0) {
        int off = 0;
        for (int e = 0; e < E; e++) {
            counts[e] = s_cnt[e];
            offsets[e] = off;
            off += s_cnt[e];
        }
        offsets[E] = off;
    }
    exchange_body(sm, a, s_cnt);
    if (tid < n) {
        int p = sm.base[s_idx[tid]] + s_rank[tid];
        if (p >= a.rows_cap) {  // cannot follow from an accepted layout; reported, and the row is not moved
            atomicOr(a.dev_err, kDevErrBounds);
            p = -1;
        } else if (p < 0) {
            p = -1;  // refused step
        }
        s_pos[tid] = p;
        pos[tid] = p;
    }
    __syncthreads();
    // copy the token rows to their k places in the owners' buffers (bf16 rows out; fp32 rows are converted)
    const int vec = d / 8;
    for (int i = tid; i < T * vec; i += blockDim.x) {
        const int tt = i / vec, c = (i % vec) * 8;
        float v[8];
        ldg8(x + (size_t)tt * d + c, v);
        uint4 o;
        o.x = pack_bf16(v[0], v[1]);
        o.y = pack_bf16(v[2], v[3]);
        o.z = pack_bf16(v[4], v[5]);
        o.w = pack_bf16(v[6], v[7]);
        for (int j = 0; j < k; j++) {
            const int p = s_pos[tt * k + j];
            if (p < 0) continue;
            __nv_bfloat16 *dst = static_cast<__nv_bfloat16 *>(row_table[s_idx[tt * k + j] / a.El]);
            *reinterpret_cast<uint4 *>(dst + (size_t)p * d + c) = o;
        }
    }
    // the rows are visible system-wide before the flag is
    __threadfence_system();
    __syncthreads();
    if (tid < a.W) {
        __threadfence_system();
        st_release_sys(rows_flags[tid] + a.r, sm.seq);
    }
}

__global__ void ep_wait_kernel(const uint32_t *flags, int W, const uint32_t *seq, int32_t *dev_err,
                               unsigned long long timeout_ns) {
    if ((int)threadIdx.x < W) ep_wait_flag(flags + threadIdx.x, *seq, timeout_ns, dev_err);
}

// flags[q] points at the flag array on rank q; slot `r` there belongs to this rank.
__global__ void ep_signal_kernel(uint32_t *const *flags, int W, int r, const uint32_t *seq) {
    __threadfence_system();
    if ((int)threadIdx.x < W) st_release_sys(flags[threadIdx.x] + r, *seq);
}

int ep_fail(omoe_handle *h, int code, const char *what, cudaError_t e) {
    snprintf(h->err, sizeof(h->err), "%s: %s", what, cudaGetErrorString(e));
    return code;
}

}  // namespace

int ep_create(omoe_handle *h) {
    EpState *st = static_cast<EpState *>(calloc(1, sizeof(EpState)));
    if (!st) return OMOE_ERR_NOMEM;
    h->ep = st;
    const int W = h->cfg.world, El = h->e_local;
    const size_t grad_bytes = (size_t)h->rows_cap * h->cfg.d_model * (h->cfg.compute_dtype == OMOE_BF16 ? 2 : 4);
    cudaError_t e;
    if ((e = cudaMalloc(&st->ctl, sizeof(EpCtl))) != cudaSuccess) return ep_fail(h, OMOE_ERR_NOMEM, "cudaMalloc(ctl)", e);
    cudaMemset(st->ctl, 0, sizeof(EpCtl));
    if ((e = cudaMalloc(&st->d_ctl_table, sizeof(void *) * W)) != cudaSuccess ||
        (e = cudaMalloc(&st->d_rows_flags, sizeof(void *) * W)) != cudaSuccess ||
        (e = cudaMalloc(&st->d_out_flags, sizeof(void *) * W)) != cudaSuccess ||
        (e = cudaMalloc(&st->d_seq, sizeof(uint32_t))) != cudaSuccess ||
        (e = cudaMalloc(&st->d_dyp_table, sizeof(void *) * W)) != cudaSuccess ||
        (e = cudaMalloc(&st->d_dxp_table, sizeof(void *) * W)) != cudaSuccess ||
        (e = cudaMalloc(&st->dyp, grad_bytes)) != cudaSuccess || (e = cudaMalloc(&st->dxp, grad_bytes)) != cudaSuccess ||
        (e = cudaMalloc(&st->ex_counts, sizeof(int32_t) * El)) != cudaSuccess ||
        (e = cudaMalloc(&st->ex_poffsets, sizeof(int32_t) * (El + 1))) != cudaSuccess ||
        (e = cudaMalloc(&st->ex_tile_expert, sizeof(int32_t) * (h->rows_cap / kRowAlign))) != cudaSuccess ||
        (e = cudaMalloc(&st->ex_tile_mask, sizeof(uint32_t) * (h->rows_cap / kRowAlign))) != cudaSuccess ||
        (e = cudaMalloc(&st->ex_tile_order, sizeof(int32_t) * (h->rows_cap / kRowAlign))) != cudaSuccess)
        return ep_fail(h, OMOE_ERR_NOMEM, "cudaMalloc(expert-parallel state)", e);
    cudaMemset(st->d_seq, 0, sizeof(uint32_t));
    cudaMemset(st->dyp, 0, grad_bytes);
    cudaMemset(st->dxp, 0, grad_bytes);
    h->ex_counts = st->ex_counts;
    h->ex_poffsets = st->ex_poffsets;
    h->ex_tile_expert = st->ex_tile_expert;
    // Measured on 8 GPUs (Mixtral-shaped layer): with 268 MB of rows per rank the step gains 1.2 %, with 33 MB it
    // loses 0.9 % (the dispatch warps take issue slots from the product and the tiles of remote rows wait for
    // them); the default sends only steps of at least 160 MB through the product.
    st->overlap_min_bytes = 160l << 20;
    if (const char *v = getenv("OMOE_EP_OVERLAP_MIN_MB")) st->overlap_min_bytes = atol(v) < 0 ? (1l << 60) : (atol(v) << 20);
    st->timeout_ns = 10ull * 1000 * 1000 * 1000;
    if (const char *v = getenv("OMOE_EP_WAIT_MS")) {
        long ms = atol(v);
        if (ms > 0) st->timeout_ns = (unsigned long long)ms * 1000000ull;
    }
    return OMOE_OK;
}

void ep_destroy(omoe_handle *h) {
    EpState *st = static_cast<EpState *>(h->ep);
    if (!st) return;
    for (int q = 0; q < kMaxWorld; q++)
        for (int i = 0; i < 5; i++)
            if (st->peer_ptrs[q][i]) cudaIpcCloseMemHandle(st->peer_ptrs[q][i]);
    void *ptrs[] = {st->ctl, st->d_ctl_table, st->d_rows_flags, st->d_out_flags, st->d_seq, st->d_dyp_table,
                    st->d_dxp_table, st->dyp, st->dxp, st->ex_counts, st->ex_poffsets,
                    st->ex_tile_expert, st->ex_tile_mask, st->ex_tile_order};
    for (void *p : ptrs)
        if (p) cudaFree(p);
    free(st);
    h->ep = nullptr;
}

int ep_export(omoe_handle *h, void *blob) {
    EpState *st = static_cast<EpState *>(h->ep);
    if (!st) {
        snprintf(h->err, sizeof(h->err), "omoe_ep_export: the layer was created with world == 1");
        return OMOE_ERR_STATE;
    }
    IpcBlob b;
    cudaError_t e;
    if ((e = cudaIpcGetMemHandle(&b.ctl, st->ctl)) != cudaSuccess || (e = cudaIpcGetMemHandle(&b.xp, h->xp)) != cudaSuccess ||
        (e = cudaIpcGetMemHandle(&b.yp, h->yp)) != cudaSuccess ||
        (e = cudaIpcGetMemHandle(&b.dyp, st->dyp)) != cudaSuccess ||
        (e = cudaIpcGetMemHandle(&b.dxp, st->dxp)) != cudaSuccess)
        return ep_fail(h, OMOE_ERR_COMM, "cudaIpcGetMemHandle", e);
    memcpy(blob, &b, sizeof(b));
    return OMOE_OK;
}

int ep_import(omoe_handle *h, const void *all_blobs) {
    EpState *st = static_cast<EpState *>(h->ep);
    if (!st) {
        snprintf(h->err, sizeof(h->err), "omoe_ep_import: the layer was created with world == 1");
        return OMOE_ERR_STATE;
    }
    if (st->imported) {
        snprintf(h->err, sizeof(h->err), "omoe_ep_import: already imported");
        return OMOE_ERR_STATE;
    }
    const int W = h->cfg.world, r = h->cfg.rank;
    const IpcBlob *blobs = static_cast<const IpcBlob *>(all_blobs);
    void *ctl[kMaxWorld], *xp[kMaxWorld], *yp[kMaxWorld], *dyp[kMaxWorld], *dxp[kMaxWorld];
    uint32_t *rows_flags[kMaxWorld], *out_flags[kMaxWorld];
    for (int q = 0; q < W; q++) {
        if (q == r) {
            ctl[q] = st->ctl;
            xp[q] = h->xp;
            yp[q] = h->yp;
            dyp[q] = st->dyp;
            dxp[q] = st->dxp;
        } else {
            const cudaIpcMemHandle_t *hs[5] = {&blobs[q].ctl, &blobs[q].xp, &blobs[q].yp, &blobs[q].dyp, &blobs[q].dxp};
            for (int i = 0; i < 5; i++) {
                cudaError_t e = cudaIpcOpenMemHandle(&st->peer_ptrs[q][i], *hs[i], cudaIpcMemLazyEnablePeerAccess);
                if (e != cudaSuccess) return ep_fail(h, OMOE_ERR_COMM, "cudaIpcOpenMemHandle (is peer access available?)", e);
            }
            ctl[q] = st->peer_ptrs[q][0];
            xp[q] = st->peer_ptrs[q][1];
            yp[q] = st->peer_ptrs[q][2];
            dyp[q] = st->peer_ptrs[q][3];
            dxp[q] = st->peer_ptrs[q][4];
        }
        rows_flags[q] = static_cast<EpCtl *>(ctl[q])->flag_rows;  // address arithmetic only
        out_flags[q] = static_cast<EpCtl *>(ctl[q])->flag_out;
    }
    cudaError_t e;
    if ((e = cudaMemcpy(st->d_ctl_table, ctl, sizeof(void *) * W, cudaMemcpyHostToDevice)) != cudaSuccess ||
        (e = cudaMemcpy(st->d_rows_flags, rows_flags, sizeof(void *) * W, cudaMemcpyHostToDevice)) != cudaSuccess ||
        (e = cudaMemcpy(st->d_out_flags, out_flags, sizeof(void *) * W, cudaMemcpyHostToDevice)) != cudaSuccess ||
        (e = cudaMemcpy(h->d_row_table, xp, sizeof(void *) * W, cudaMemcpyHostToDevice)) != cudaSuccess ||
        (e = cudaMemcpy(h->d_out_table, yp, sizeof(void *) * W, cudaMemcpyHostToDevice)) != cudaSuccess ||
        (e = cudaMemcpy(st->d_dyp_table, dyp, sizeof(void *) * W, cudaMemcpyHostToDevice)) != cudaSuccess ||
        (e = cudaMemcpy(st->d_dxp_table, dxp, sizeof(void *) * W, cudaMemcpyHostToDevice)) != cudaSuccess)
        return ep_fail(h, OMOE_ERR_CUDA, "cudaMemcpy(peer tables)", e);
    st->imported = true;
    return OMOE_OK;
}

// One process drives every GPU (the reference's own multi-GPU mode: one thread per device in one JVM,
// src/main/java/com/omega/engine/parallel/dp/DP.java:68-94).  IPC handles cannot be opened in the process that
// made them, and need not be: with peer access enabled the other handles' buffers are addressed directly.
int ep_connect_local(omoe_handle **hs, int world) {
    int saved = 0;
    cudaGetDevice(&saved);
    auto fail_all = [&](omoe_handle *h, int code, const char *what, cudaError_t e) {
        cudaSetDevice(saved);
        return ep_fail(h, code, what, e);
    };
    for (int r = 0; r < world; r++) {
        omoe_handle *h = hs[r];
        EpState *st = static_cast<EpState *>(h->ep);
        if (!st || h->cfg.world != world || h->cfg.rank != r || st->imported) {
            cudaSetDevice(saved);
            snprintf(h->err, sizeof(h->err),
                     "omoe_ep_connect_local: handle %d must be created with world=%d, rank=%d and not be connected yet", r,
                     world, r);
            return OMOE_ERR_STATE;
        }
        for (int q = 0; q < r; q++)
            if (hs[q]->device == h->device) {
                cudaSetDevice(saved);
                snprintf(h->err, sizeof(h->err), "omoe_ep_connect_local: ranks %d and %d are on the same device", q, r);
                return OMOE_ERR_INVALID;
            }
    }
    for (int r = 0; r < world; r++) {
        omoe_handle *h = hs[r];
        EpState *st = static_cast<EpState *>(h->ep);
        cudaError_t e = cudaSetDevice(h->device);
        if (e != cudaSuccess) return fail_all(h, OMOE_ERR_CUDA, "cudaSetDevice", e);
        void *ctl[kMaxWorld], *xp[kMaxWorld], *yp[kMaxWorld], *dyp[kMaxWorld], *dxp[kMaxWorld];
        uint32_t *rows_flags[kMaxWorld], *out_flags[kMaxWorld];
        for (int q = 0; q < world; q++) {
            if (q != r) {
                e = cudaDeviceEnablePeerAccess(hs[q]->device, 0);
                if (e == cudaErrorPeerAccessAlreadyEnabled) {
                    cudaGetLastError();
                } else if (e != cudaSuccess) {
                    return fail_all(h, OMOE_ERR_COMM, "cudaDeviceEnablePeerAccess", e);
                }
            }
            EpState *sq = static_cast<EpState *>(hs[q]->ep);
            ctl[q] = sq->ctl;
            xp[q] = hs[q]->xp;
            yp[q] = hs[q]->yp;
            dyp[q] = sq->dyp;
            dxp[q] = sq->dxp;
            rows_flags[q] = sq->ctl->flag_rows;  // address arithmetic only
            out_flags[q] = sq->ctl->flag_out;
        }
        if ((e = cudaMemcpy(st->d_ctl_table, ctl, sizeof(void *) * world, cudaMemcpyHostToDevice)) != cudaSuccess ||
            (e = cudaMemcpy(st->d_rows_flags, rows_flags, sizeof(void *) * world, cudaMemcpyHostToDevice)) != cudaSuccess ||
            (e = cudaMemcpy(st->d_out_flags, out_flags, sizeof(void *) * world, cudaMemcpyHostToDevice)) != cudaSuccess ||
            (e = cudaMemcpy(h->d_row_table, xp, sizeof(void *) * world, cudaMemcpyHostToDevice)) != cudaSuccess ||
            (e = cudaMemcpy(h->d_out_table, yp, sizeof(void *) * world, cudaMemcpyHostToDevice)) != cudaSuccess ||
            (e = cudaMemcpy(st->d_dyp_table, dyp, sizeof(void *) * world, cudaMemcpyHostToDevice)) != cudaSuccess ||
            (e = cudaMemcpy(st->d_dxp_table, dxp, sizeof(void *) * world, cudaMemcpyHostToDevice)) != cudaSuccess)
            return fail_all(h, OMOE_ERR_CUDA, "cudaMemcpy(peer tables)", e);
        st->imported = true;
    }
    cudaSetDevice(saved);
    return OMOE_OK;
}

namespace {

ExArgs exchange_args(omoe_handle *h, EpState *st) {
    ExArgs a;
    a.self = st->ctl;
    a.peers = st->d_ctl_table;
    a.W = h->cfg.world;
    a.r = h->cfg.rank;
    a.E = h->cfg.n_experts;
    a.El = h->e_local;
    a.seq_ptr = st->d_seq;
    a.rows_cap = (int)h->rows_cap;
    a.dst_base = h->dst_base;
    a.ex_counts = st->ex_counts;
    a.ex_poffsets = st->ex_poffsets;
    a.ex_tile_expert = st->ex_tile_expert;
    a.ex_tile_mask = st->ex_tile_mask;
    a.ex_tile_order = st->ex_tile_order;
    a.max_tiles = (int)(h->rows_cap / kRowAlign);
    a.ticket = h->ticket;
    a.dev_err = h->dev_err;
    a.timeout_ns = st->timeout_ns;
    return a;
}

template <typename XT>
cudaError_t launch_route_small_ep(omoe_handle *h, EpState *st, const XT *x, int T, cudaStream_t s) {
    const ExArgs a = exchange_args(h, st);
    const int E = h->cfg.n_experts;
    const int blocks = T > 0 ? T : 1;
    cudaError_t e;
#define OMOE_RSE(PLV)                                                                                              \
    e = launch_ex(route_small_ep_kernel<PLV, XT>, dim3(blocks), dim3(256), 0, s, h->pdl, x, h->w_router,           \
                  h->router_bias, T, h->cfg.d_model, h->cfg.top_k, h->cfg.renormalize, h->logits, h->topk_idx,     \
                  h->topk_w, h->counts, h->offsets, h->pos, h->d_row_table, st->d_rows_flags, h->ticket, a)
    if (E <= 32) OMOE_RSE(1);
    else if (E <= 64) OMOE_RSE(2);
    else OMOE_RSE(4);
#undef OMOE_RSE
    return e;
}

}  // namespace

// One forward of this rank.  Launches (bf16 layer, inference): router, scan + count exchange, dispatch (raises
// "rows landed"), up/gate product (its producer waits for the rows, tile by tile), down product (its last CTA
// raises "outputs ready"), combine (waits for the owners' flags) -- six; a decode step of at most 8 tokens
// takes one launch for everything before the products -- four.
int ep_forward(omoe_handle *h, const void *x, int x_dtype, void *y, int y_dtype, const void *resid, int T,
               cudaStream_t s) {
    EpState *st = static_cast<EpState *>(h->ep);
    if (!st || !st->imported) {
        snprintf(h->err, sizeof(h->err), "omoe_forward: call omoe_ep_export / omoe_ep_import on every rank first");
        return OMOE_ERR_STATE;
    }
    const int W = h->cfg.world, r = h->cfg.rank;
    uint32_t *const seq = st->d_seq;  // advanced on the device by the count exchange
    int n = 0;
    cudaError_t e = cudaSuccess;
    const bool prof = h->profiling;
    const bool bf16 = h->cfg.compute_dtype == OMOE_BF16;
    bool overlapped = false;
    // OMOE_EP_UNFUSED=1: separate wait / signal launches around the products and no one-launch decode routing
    static const bool unfused = getenv("OMOE_EP_UNFUSED") && atoi(getenv("OMOE_EP_UNFUSED")) != 0;
    // the products take the wait and the signal themselves (no launches of their own around them)
    const bool gated_step = bf16 && !bw_training(h) && !unfused;
#define MARK(i) do { if (prof) cudaEventRecord(h->ev[i], s); } while (0)
#define TRY(expr)                                                                      \
    do {                                                                               \
        e = (expr);                                                                    \
        if (e != cudaSuccess) return ep_fail(h, OMOE_ERR_CUDA, #expr, e);              \
    } while (0)
    // Programmatic dependent launch along the decode chain only (one-launch routing, products, combine).
    const bool small_path = bf16 && !unfused && T <= route_small_max_tokens();
    struct PdlScope {
        omoe_handle *h;
        bool saved;
        ~PdlScope() { h->pdl = saved; }
    } pdl_scope{h, h->pdl};
    h->pdl = h->pdl && small_path && gated_step;
    MARK(0);
    if (small_path) {
        if (T > 0 && (reinterpret_cast<uintptr_t>(x) & 15u) != 0) return ep_fail(h, OMOE_ERR_CUDA, "x", cudaErrorMisalignedAddress);
        if (x_dtype == OMOE_F32) TRY(launch_route_small_ep<float>(h, st, static_cast<const float *>(x), T, s));
        else TRY(launch_route_small_ep<__nv_bfloat16>(h, st, static_cast<const __nv_bfloat16 *>(x), T, s));
        n++;
        MARK(1);
        MARK(2);
    } else {
        if (T > 0) TRY(launch_router(h, x, x_dtype, T, s, &n));
        MARK(1);
        // T == 0: zero router blocks, all counts zero
        ep_scan_exchange_kernel<<<1, 1024, 0, s>>>(h->block_counts, h->block_base, ceil_div(T, h->tokens_per_block),
                                                   h->counts, h->offsets, h->poffsets, h->tile_expert,
                                                   exchange_args(h, st));
        TRY(cudaGetLastError());
        n++;
        MARK(2);
        EpSignal sig{st->d_rows_flags, W, r, seq};
        // Large steps: the rows this rank keeps go first (local pass, tells this rank alone); the rows for the
        // other ranks travel INSIDE the up/gate product (two extra warps per CTA, peer stores) while its other
        // warps already multiply the tiles that hold only local rows -- the producer waits, tile by tile, for
        // exactly the ranks a tile's rows come from, and the tiles are walked local-first.
        const long rows_ub = (long)h->cfg.t_max * W * h->cfg.top_k;
        overlapped = gated_step && T > 0 && experts_up_is_persistent(h, rows_ub) &&
                     (long)T * h->cfg.top_k * h->cfg.d_model * 2 >= st->overlap_min_bytes;
        if (overlapped) {
            TRY(launch_permute(h, x, x_dtype, T, s, &n, &sig, 1));
        } else if (T > 0) {
            TRY(launch_permute(h, x, x_dtype, T, s, &n, &sig));
        } else {
            ep_signal_kernel<<<1, 32, 0, s>>>(st->d_rows_flags, W, r, seq);
            TRY(cudaGetLastError());
            n++;
        }
    }
    MARK(3);
    const bool gated = gated_step;
    if (!gated) {
        ep_wait_kernel<<<1, 32, 0, s>>>(st->ctl->flag_rows, W, seq, h->dev_err, st->timeout_ns);
        TRY(cudaGetLastError());
        n++;
    }
    MARK(4);
    if (bw_training(h)) {
        TRY(bw_forward_experts(h, T, s, &n));  // keeps g and u for the backward pass
        MARK(5);
    } else if (bf16) {
        EpGate gate{};
        gate.wait_flags = st->ctl->flag_rows;
        gate.tile_src_mask = st->ex_tile_mask;
        gate.tile_order = st->ex_tile_order;
        if (overlapped) {
            EpDispatch &dp = gate.disp;
            dp.x = x;
            dp.x_is_f32 = x_dtype == OMOE_F32;
            dp.row_table = h->d_row_table;
            dp.topk_idx = h->topk_idx;
            dp.lrank = h->lrank;
            dp.block_base = h->block_base;
            dp.dst_base = h->dst_base;
            dp.T = T;
            dp.d = h->cfg.d_model;
            dp.n_blocks = ceil_div(T, h->tokens_per_block);
            dp.e_local = h->e_local;
            dp.k = h->cfg.top_k;
            dp.tokens_per_block = h->tokens_per_block;
            dp.rows_cap = (int)h->rows_cap;
            dp.rows_flags = st->d_rows_flags;
            dp.ticket = h->ticket3;
        }
        gate.signal_flags = st->d_out_flags;
        gate.ticket = h->ticket2;
        gate.seq = seq;
        gate.timeout_ns = st->timeout_ns;
        gate.world = W;
        gate.rank = r;
        // rows can come from every rank's tokens; a rank's step holds at most t_max of them
        TRY(launch_experts_bf16(h, s, &n, prof ? h->ev[5] : nullptr, (long)h->cfg.t_max * W * h->cfg.top_k,
                                gated ? &gate : nullptr));
    } else {
        TRY(launch_experts_f32(h, s, &n));
        MARK(5);
    }
    MARK(6);
    if (!gated) {
        ep_signal_kernel<<<1, 32, 0, s>>>(st->d_out_flags, W, r, seq);
        TRY(cudaGetLastError());
        n++;
    }
    MARK(7);
    EpWait wt{st->ctl->flag_out, W, seq, st->timeout_ns};
    if (T > 0) {
        TRY(launch_combine(h, y, y_dtype, T, s, &n, &wt, resid));
    } else {
        // still wait: the owners' outputs of this step must not be overwritten
        // by a later step before every rank has passed this point
        ep_wait_kernel<<<1, 32, 0, s>>>(st->ctl->flag_out, W, seq, h->dev_err, st->timeout_ns);
        TRY(cudaGetLastError());
        n++;
    }
    MARK(8);
#undef MARK
#undef TRY
    h->ev_valid = prof;
    h->last_launches = n;
    return OMOE_OK;
}

// ---- pieces the backward pass (backward.cu) builds its expert-parallel form from -----------------------
namespace {
__global__ void ep_advance_kernel(uint32_t *seq, int32_t *ticket) {
    *seq = *seq + 1u;  // a backward pass is a step of its own: gradient rows out, input gradients back
    *ticket = 0;
}
}  // namespace

bool ep_ready(const omoe_handle *h) { return h->ep && static_cast<EpState *>(h->ep)->imported; }

void ep_grad_buffers(omoe_handle *h, void **dyp, void **dxp, void ***dyp_table, void ***dxp_table) {
    EpState *st = static_cast<EpState *>(h->ep);
    *dyp = st->dyp;
    *dxp = st->dxp;
    *dyp_table = st->d_dyp_table;
    *dxp_table = st->d_dxp_table;
}

cudaError_t ep_bw_advance(omoe_handle *h, cudaStream_t s) {
    EpState *st = static_cast<EpState *>(h->ep);
    ep_advance_kernel<<<1, 1, 0, s>>>(st->d_seq, h->ticket);
    return cudaGetLastError();
}

EpSignal ep_rows_signal(omoe_handle *h) {
    EpState *st = static_cast<EpState *>(h->ep);
    return EpSignal{st->d_rows_flags, h->cfg.world, h->cfg.rank, st->d_seq};
}

EpWait ep_out_wait(omoe_handle *h) {
    EpState *st = static_cast<EpState *>(h->ep);
    return EpWait{st->ctl->flag_out, h->cfg.world, st->d_seq, st->timeout_ns};
}

cudaError_t ep_signal_rows(omoe_handle *h, cudaStream_t s) {
    EpState *st = static_cast<EpState *>(h->ep);
    ep_signal_kernel<<<1, 32, 0, s>>>(st->d_rows_flags, h->cfg.world, h->cfg.rank, st->d_seq);
    return cudaGetLastError();
}

cudaError_t ep_wait_rows(omoe_handle *h, cudaStream_t s) {
    EpState *st = static_cast<EpState *>(h->ep);
    ep_wait_kernel<<<1, 32, 0, s>>>(st->ctl->flag_rows, h->cfg.world, st->d_seq, h->dev_err, st->timeout_ns);
    return cudaGetLastError();
}

cudaError_t ep_signal_out(omoe_handle *h, cudaStream_t s) {
    EpState *st = static_cast<EpState *>(h->ep);
    ep_signal_kernel<<<1, 32, 0, s>>>(st->d_out_flags, h->cfg.world, h->cfg.rank, st->d_seq);
    return cudaGetLastError();
}

}  // namespace omoe
