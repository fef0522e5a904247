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
//   1. router, scan                          (local)
//   2. exchange kernel: publish my per-expert counts to every rank, wait for
//      all rows of the count matrix, derive where my picks go on each owner
//      (dst_base) and how the rows I receive are laid out (ex_* arrays)
//   3. dispatch: rows -> owners' buffers, then "rows landed" flag to every rank
//   4. wait kernel: all ranks' rows have landed here
//   5. grouped expert products                (local)
//   6. signal kernel: "outputs ready" flag to every rank
//   7. combine: wait for all owners' flags, gather rows over NVLink
// Flags carry the sequence number, so nothing is reset between forwards; the
// count matrix is double-buffered by the parity of seq.  Every wait is bounded
// and reports through the device error word instead of hanging.
#include <stdlib.h>
#include <string.h>

#include "ep.cuh"
#include "backward.cuh"

namespace omoe {

namespace {

// Control block of one rank, written by its peers.  Lives in IPC-shared memory.
struct EpCtl {
    int32_t cnt[2][kMaxWorld][kMaxExperts];  // [parity][source rank][expert]
    uint32_t flag_cnt[2][kMaxWorld];         // seq once source's count row is complete
    uint32_t flag_rows[kMaxWorld];           // seq once source's rows have landed in my dispatch buffer
    uint32_t flag_out[kMaxWorld];            // seq once owner's expert outputs are readable
};

struct EpState {
    EpCtl *ctl;                 // this rank's control block (device)
    EpCtl **d_ctl_table;        // device [world]
    uint32_t **d_rows_flags;    // device [world]: &peer_ctl[q]->flag_rows[0]
    uint32_t **d_out_flags;     // device [world]: &peer_ctl[q]->flag_out[0]
    int32_t *ex_counts, *ex_poffsets, *ex_tile_expert;  // layout of the rows this rank receives
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

// One block of 256 threads.
__global__ void __launch_bounds__(256)
ep_exchange_kernel(EpCtl *self, EpCtl *const *__restrict__ peers, const int32_t *__restrict__ counts, int W, int r,
                   int E, int El, uint32_t *seq_ptr, int rows_cap, int32_t *__restrict__ dst_base,
                   int32_t *__restrict__ ex_counts, int32_t *__restrict__ ex_poffsets,
                   int32_t *__restrict__ ex_tile_expert, int max_tiles, int32_t *ticket, int32_t *dev_err,
                   unsigned long long timeout_ns) {
    __shared__ int32_t s_cnt[kMaxWorld][kMaxExperts];
    __shared__ int32_t s_tot[kMaxExperts];
    __shared__ int32_t s_rpoff[kMaxExperts + kMaxWorld];  // padded start of expert e in its owner's buffer
    __shared__ int32_t s_mypoff[kMaxExperts + 1];
    __shared__ int s_bad;
    __shared__ uint32_t s_seq;
    const int tid = threadIdx.x;
    // a new step begins: this kernel is the first of the step to need the number, the later ones read it
    if (tid == 0) { s_seq = *seq_ptr + 1u; *seq_ptr = s_seq; *ticket = 0; s_bad = 0; }
    __syncthreads();
    const uint32_t seq = s_seq;
    const int par = seq & 1u;
    // publish my counts to every rank (my own included)
    for (int i = tid; i < W * E; i += blockDim.x) {
        int q = i / E, e = i % E;
        peers[q]->cnt[par][r][e] = counts[e];
    }
    __threadfence_system();
    __syncthreads();
    if (tid < W) st_release_sys(&peers[tid]->flag_cnt[par][r], seq);
    // wait for every source's row
    if (tid < W) {
        if (!ep_wait_flag(&self->flag_cnt[par][tid], seq, timeout_ns, dev_err)) s_bad = 1;
    }
    __syncthreads();
    __threadfence_system();
    for (int i = tid; i < W * E; i += blockDim.x) {
        int s = i / E, e = i % E;
        s_cnt[s][e] = *(volatile int32_t *)&self->cnt[par][s][e];
    }
    __syncthreads();
    for (int e = tid; e < E; e += blockDim.x) {
        int t = 0;
        for (int s = 0; s < W; s++) t += s_cnt[s][e];
        s_tot[e] = t;
    }
    __syncthreads();
    if (tid < W) {  // thread q lays out owner q's buffer
        int q = tid, off = 0;
        for (int le = 0; le < El; le++) {
            int e = q * El + le;
            s_rpoff[e] = off;
            off += (s_tot[e] + kRowAlign - 1) / kRowAlign * kRowAlign;
        }
        if (off > rows_cap) s_bad = 1;  // every rank sees the same matrix, so all of them refuse together
        if (q == r) {
            for (int le = 0; le < El; le++) s_mypoff[le] = s_rpoff[q * El + le];
            s_mypoff[El] = off;
        }
    }
    __syncthreads();
    const bool bad = s_bad != 0;
    if (bad && tid == 0) atomicOr(dev_err, kDevErrBounds);
    for (int e = tid; e < E; e += blockDim.x) {
        int before = 0;
        for (int s = 0; s < r; s++) before += s_cnt[s][e];
        // a refused step moves no row: the base is far below zero, so every position the dispatch derives from
        // it is negative, and the dispatch, combine and backward kernels skip rows with a negative position
        dst_base[e] = bad ? kRefusedBase : s_rpoff[e] + before;
    }
    for (int le = tid; le < El; le += blockDim.x) {
        ex_counts[le] = bad ? 0 : s_tot[r * El + le];
        ex_poffsets[le] = bad ? 0 : s_mypoff[le];
    }
    if (tid == 0) ex_poffsets[El] = bad ? 0 : s_mypoff[El];
    const int n_tiles = bad ? 0 : s_mypoff[El] / kRowAlign;
    for (int i = tid; i < max_tiles; i += blockDim.x) {
        int ex = -1;
        if (i < n_tiles) {
            int row = i * kRowAlign;
            ex = 0;
            while (ex + 1 < El && s_mypoff[ex + 1] <= row) ex++;
        }
        ex_tile_expert[i] = ex;
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
        (e = cudaMalloc(&st->ex_tile_expert, sizeof(int32_t) * (h->rows_cap / kRowAlign))) != cudaSuccess)
        return ep_fail(h, OMOE_ERR_NOMEM, "cudaMalloc(expert-parallel state)", e);
    cudaMemset(st->d_seq, 0, sizeof(uint32_t));
    cudaMemset(st->dyp, 0, grad_bytes);
    cudaMemset(st->dxp, 0, grad_bytes);
    h->ex_counts = st->ex_counts;
    h->ex_poffsets = st->ex_poffsets;
    h->ex_tile_expert = st->ex_tile_expert;
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
                    st->ex_tile_expert};
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

int ep_forward(omoe_handle *h, const void *x, int x_dtype, void *y, int y_dtype, const void *resid, int T,
               cudaStream_t s) {
    EpState *st = static_cast<EpState *>(h->ep);
    if (!st || !st->imported) {
        snprintf(h->err, sizeof(h->err), "omoe_forward: call omoe_ep_export / omoe_ep_import on every rank first");
        return OMOE_ERR_STATE;
    }
    const int W = h->cfg.world, r = h->cfg.rank, E = h->cfg.n_experts, El = h->e_local;
    uint32_t *const seq = st->d_seq;  // advanced on the device by the count exchange
    int n = 0;
    cudaError_t e = cudaSuccess;
    const bool prof = h->profiling;
#define MARK(i) do { if (prof) cudaEventRecord(h->ev[i], s); } while (0)
#define TRY(expr)                                                                      \
    do {                                                                               \
        e = (expr);                                                                    \
        if (e != cudaSuccess) return ep_fail(h, OMOE_ERR_CUDA, #expr, e);              \
    } while (0)
    MARK(0);
    if (T > 0) {
        TRY(launch_router(h, x, x_dtype, T, s, &n));
    }
    MARK(1);
    TRY(launch_scan(h, T, s, &n));  // T == 0: zero blocks, all counts zero
    MARK(2);
    ep_exchange_kernel<<<1, 256, 0, s>>>(st->ctl, st->d_ctl_table, h->counts, W, r, E, El, seq, (int)h->rows_cap,
                                         h->dst_base, st->ex_counts, st->ex_poffsets, st->ex_tile_expert,
                                         (int)(h->rows_cap / kRowAlign), h->ticket, h->dev_err, st->timeout_ns);
    TRY(cudaGetLastError());
    n++;
    EpSignal sig{st->d_rows_flags, W, r, seq};
    if (T > 0) {
        TRY(launch_permute(h, x, x_dtype, T, s, &n, &sig));
    } else {
        ep_signal_kernel<<<1, 32, 0, s>>>(st->d_rows_flags, W, r, seq);
        TRY(cudaGetLastError());
        n++;
    }
    MARK(3);
    ep_wait_kernel<<<1, 32, 0, s>>>(st->ctl->flag_rows, W, seq, h->dev_err, st->timeout_ns);
    TRY(cudaGetLastError());
    n++;
    MARK(4);
    if (bw_training(h)) {
        TRY(bw_forward_experts(h, T, s, &n));  // keeps g and u for the backward pass
        MARK(5);
    } else if (h->cfg.compute_dtype == OMOE_BF16) {
        // rows can come from every rank's tokens; a rank's step holds at most t_max of them
        TRY(launch_experts_bf16(h, s, &n, prof ? h->ev[5] : nullptr, (long)h->cfg.t_max * W * h->cfg.top_k));
    } else {
        TRY(launch_experts_f32(h, s, &n));
        MARK(5);
    }
    MARK(6);
    ep_signal_kernel<<<1, 32, 0, s>>>(st->d_out_flags, W, r, seq);
    TRY(cudaGetLastError());
    n++;
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
