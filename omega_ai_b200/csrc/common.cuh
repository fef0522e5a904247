// Shared declarations of the MoE forward library: the handle, error helpers
// and the launchers each .cu file exports to api.cu.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/omoe.h"
#include "pdl.cuh"
#include "vec8.cuh"

namespace omoe {

// Rows of one expert in the dispatch buffers start on a multiple of this, so a
// 128-row tensor-core tile never straddles two experts.
constexpr int kRowAlign = 128;
constexpr int kMaxTopK = 16;
constexpr int kMaxExperts = 128;
constexpr int kRouterWarps = 8;  // warps per router block
constexpr int kHostChunksMax = 8;  // pieces a host-buffer forward is cut into to overlap copies and kernels
constexpr int kMaxWorld = 8;     // expert-parallel ranks (GPUs of one NVSwitch node)
constexpr int kProfSlots = 32;   // profiled forwards whose stage events are kept

// Device-side error word bits (set by kernels instead of trapping).
constexpr int kDevErrTimeout = 1;   // a bounded wait ran out
constexpr int kDevErrBounds = 2;    // an index check failed

// dst_base of every expert in a step that the count exchange refused (an owner's buffer would overflow): any
// row position derived from it is negative, and kernels touch no row whose position is outside [0, rows_cap).
constexpr int32_t kRefusedBase = -(1 << 30);

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Function attributes (the opt-in to more than 48 KB of dynamic shared memory) are per device: a launcher keeps
// one "done" flag per device ordinal, so a process that drives several GPUs sets them on each.
constexpr int kMaxDevices = 64;
struct PerDeviceOnce {
    bool done[kMaxDevices] = {};
    // slot of the current device, or nullptr when it cannot be told (the caller then sets the attribute every time)
    bool *slot() {
        int dev = -1;
        if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
        return &done[dev];
    }
};
inline int64_t round_up(int64_t a, int64_t b) { return (a + b - 1) / b * b; }

struct TensorMaps {
    CUtensorMap a_x;     // dispatch rows xp [rows_cap, d]
    CUtensorMap a_h;     // hidden rows h [rows_cap, dff]
    CUtensorMap b_gate;  // [E_local*dff, d]
    CUtensorMap b_up;    // [E_local*dff, d]
    CUtensorMap b_down;  // [E_local*d, dff]
    CUtensorMap c_y;     // expert outputs yp [rows_cap, d] (store target)
    CUtensorMap a_x32, a_h32;  // xp and h with a 32-row box (tiles with few tokens, split-K kernels)
};

}  // namespace omoe

struct omoe_handle {
    omoe_config cfg;
    int e_local;      // experts owned by this rank
    int e_first;      // first owned expert (global index)
    int sm_count;
    int device;       // CUDA device ordinal the handle was created on
    int tokens_per_block;  // router block granularity
    int n_blocks_max;      // router blocks at t_max
    int64_t rows_cap;      // row capacity of xp / h / yp (padded)
    bool weights_set;

    // weights (device)
    float *w_router;      // [E, d] fp32
    float *router_bias;   // [E] fp32 or null
    __nv_bfloat16 *w_router_bf16;  // [E, d] copy, only while the router weights were given as bf16 (exact)
    void *w_gate, *w_up;  // [E_local, dff, d] compute dtype
    void *w_down;         // [E_local, d, dff]

    // routing workspace (device)
    float *logits;        // [t_max, E]
    int32_t *topk_idx;    // [t_max, k]
    float *topk_w;        // [t_max, k]
    int32_t *block_counts;  // [E][n_blocks] per-router-block histograms (expert-major)
    int32_t *block_base;    // [E][n_blocks] exclusive prefix of block_counts over blocks
    int32_t *counts;      // [E]
    int32_t *offsets;     // [E+1] exclusive scan of counts (unpadded)
    int32_t *poffsets;    // [E+1] exclusive scan of counts rounded up to kRowAlign
    int32_t *tile_expert; // [rows_cap/kRowAlign] local expert of each 128-row tile
    // Views the expert kernels read.  On one GPU they alias the arrays above;
    // with expert parallelism they describe the rows received from all ranks.
    int32_t *ex_counts, *ex_poffsets, *ex_tile_expert;
    int32_t *lrank;       // [t_max*k] rank of each pick among its router block's picks of the same expert
    int32_t *pos;         // [t_max*k] row of each pick in its owner's padded dispatch buffer
    // Where this rank's picks of expert e start in the dispatch buffer of the
    // rank that owns e.  On one GPU this is poffsets; with expert parallelism
    // it is computed from the all-ranks count matrix.
    int32_t *dst_base;    // [E]
    // Device tables [world]: base address of every rank's dispatch buffer (xp)
    // and expert-output buffer (yp); entry `rank` is this GPU's own buffer.
    void **d_row_table, **d_out_table;
    int32_t *ticket;      // blocks of the dispatch kernel that have finished (EP)
    int32_t *ticket2;     // CTAs of the down product that have finished (EP: the last one raises "outputs ready")
    int32_t *ticket3;     // dispatch warps of the up/gate product that have finished (EP)
    int32_t *perm_out;    // [t_max*k] scratch for omoe_get_routing
    int32_t *dev_err;     // device error word
    bool pdl;             // launch the forward's kernels with programmatic dependent launch (pdl.cuh)

    // activations (device, compute dtype)
    void *xp, *hbuf, *yp;
    void *xn;  // [t_max, d] normalised rows of omoe_forward_block (compute dtype)
    // staging for the host-buffer entry points: two sets that alternate from call to call
    void *x_stage[2], *y_stage[2];
    int stage_next;
    size_t stage_bytes;
    cudaStream_t copy_in, copy_out;
    // per chunk of a call: rows staged on the device / forward done; per staging set: the last call that used it
    // has consumed the staged rows / has copied its outputs back
    cudaEvent_t ev_in[omoe::kHostChunksMax], ev_out[omoe::kHostChunksMax], ev_set_fwd[2], ev_set_d2h[2];
    int host_chunk_min;     // smallest chunk (tokens) worth its own forward, one GPU
    int host_chunk_min_ep;  // the same with expert parallelism
    bool host_pending;      // an omoe_forward_host_async call has not been waited for yet

    omoe::TensorMaps maps;
    bool maps_ready;

    // bookkeeping of the last forward
    int last_T;
    int last_io_dtype;
    bool last_resid;  // the last forward was the block form (RMSNorm in front, residual added)
    cudaStream_t last_stream;
    int last_launches;
    bool profiling;
    // Stage events: a ring of event sets, one per profiled forward, so a caller can time many forwards back to
    // back and read the stages afterwards without a host synchronisation in between.  `ev` points at the set
    // the running forward records into; set 0 exists from creation, the others once profiling is switched on.
    cudaEvent_t ev_ring[omoe::kProfSlots][OMOE_N_STAGES + 1];
    cudaEvent_t *ev;
    long prof_count;  // profiled forwards so far
    bool ev_valid;

    void *ep;  // expert-parallel state (ep.cu)
    void *bw;  // backward-pass state (backward.cu), null until training mode is first switched on

    char err[512];
};

namespace omoe {

// ---- launchers (defined in the kernel files) ------------------------------
// All return cudaError_t of the launch and add the kernels they launched to *n.

cudaError_t launch_router(omoe_handle *h, const void *x, int io_dtype, int T, cudaStream_t s, int *n);
cudaError_t launch_scan(omoe_handle *h, int T, cudaStream_t s, int *n);
// Router + scan + dispatch in one launch for T <= route_small_max_tokens() (single GPU, bf16 layer).
cudaError_t launch_route_small(omoe_handle *h, const void *x, int io_dtype, int T, cudaStream_t s, int *n);
int route_small_max_tokens();
// sig != nullptr: after the last block has written its rows, raise the
// "rows have landed" flag on every rank (expert-parallel dispatch).
struct EpSignal;
// pass (expert parallel): 0 = all picks; 1 = only the picks whose expert this rank owns (tells this rank alone;
// the others travel inside the up/gate product, see EpDispatch); 2 = only the picks other ranks own (tells them)
cudaError_t launch_permute(omoe_handle *h, const void *x, int io_dtype, int T, cudaStream_t s, int *n,
                           const EpSignal *sig, int pass = 0);
cudaError_t launch_perm_readout(omoe_handle *h, int T, cudaStream_t s);
// wait != nullptr: every block first waits (bounded) until all ranks have
// published their expert outputs (expert-parallel return).
struct EpWait;
// resid != nullptr: rows of y's element type added to the combined output (the block's residual).
cudaError_t launch_combine(omoe_handle *h, void *y, int io_dtype, int T, cudaStream_t s, int *n, const EpWait *wait,
                           const void *resid);
// xn = (x / rms(x)) * gamma per row, in the layer's compute dtype (the block's pre-FFN RMSNorm).
cudaError_t launch_rmsnorm(omoe_handle *h, const void *x, int x_dtype, const float *gamma, float eps, int T,
                           cudaStream_t s, int *n);
cudaError_t launch_experts_f32(omoe_handle *h, cudaStream_t s, int *n);
// rows_ub: upper bound on the rows (token, expert picks) this GPU's experts hold in the step, -1 if unknown; a small
// bound sends a product with few tiles to the split-K kernels
// gate: expert parallel only -- the up/gate product waits for the dispatched rows, the down product raises
// "outputs ready" (see EpGate); null on one GPU
struct EpGate;
cudaError_t launch_experts_bf16(omoe_handle *h, cudaStream_t s, int *n, cudaEvent_t mid, long rows_ub = -1,
                                const EpGate *gate = nullptr);
// split-K over a thread-block cluster of S CTAs (experts_sm100_splitk.cu); splitk_ways_*() pick S, 0 = use the
// persistent kernels of experts_sm100.cu
// m_tiles_ub: bound on the step's 128-row tiles, -1 if unknown
int splitk_ways_up_gate(omoe_handle *h, long m_tiles_ub);
// true when launch_experts_bf16 with this row bound runs the up/gate product on the persistent kernel (the one
// that can carry the remote half of the dispatch)
bool experts_up_is_persistent(omoe_handle *h, long rows_ub);
int splitk_ways_down(omoe_handle *h, long m_tiles_ub);
cudaError_t launch_up_gate_splitk(omoe_handle *h, cudaStream_t s, int S, const EpGate *gate);
cudaError_t launch_down_splitk(omoe_handle *h, cudaStream_t s, int S, const EpGate *gate);
// Weight-streaming expert products for decode steps (T <= decode_tokens_threshold(), bf16).
cudaError_t launch_experts_decode(omoe_handle *h, int T, cudaStream_t s, int *n, cudaEvent_t mid);
int decode_tokens_threshold();
cudaError_t launch_convert_f32_to_bf16(const float *src, __nv_bfloat16 *dst, int64_t n, cudaStream_t s);
cudaError_t launch_convert_bf16_to_f32(const __nv_bfloat16 *src, float *dst, int64_t n, cudaStream_t s);

// Encodes the TMA descriptors of the bf16 path; returns false and fills h->err
// when the driver entry point is missing or an encode fails.
bool build_tensor_maps(omoe_handle *h);

int router_tokens_per_block(int E);

#ifdef OMOE_BOUNDS_CHECK
// Self-checking build (check.cu): fill the row buffers with NaN patterns before a step; validate the routing
// arrays and the padding rows after the dispatch.
cudaError_t check_fill(omoe_handle *h, cudaStream_t s);
cudaError_t check_after_dispatch(omoe_handle *h, int T, cudaStream_t s);
#endif

// Flag words the expert-parallel kernels exchange through peer-mapped memory.
// The step's sequence number lives in device memory (the count-exchange kernel, first of a step, advances
// it): no kernel argument changes from step to step, so a captured forward replays correctly.
struct EpSignal {
    uint32_t *const *flags;  // device table [world]: address of flag_rows[0] on every rank
    int world, rank;
    const uint32_t *seq;     // device: sequence number of the running step
};
struct EpWait {
    const uint32_t *flags;   // this rank's flag_yp[world]
    int world;
    const uint32_t *seq;     // device: sequence number of the running step
    unsigned long long timeout_ns;
};

// What ties an expert product to the expert-parallel exchange without launches of its own.  Wait side (the
// up/gate product): the rows of source rank s have landed once wait_flags[s] >= *seq; tile_src_mask[mt], when
// given, names the sources whose rows 128-row tile mt holds, so a tile starts as soon as ITS sources are in
// (otherwise all sources are awaited before the first tile).  Signal side (the down product): the CTA that
// finishes last stores *seq into slot `rank` of every rank's signal_flags array ("outputs ready").
// The remote half of the dispatch, carried out by two extra warps of every CTA of the up/gate product while its
// other warps multiply the tiles that are already complete: token rows whose expert lives on another rank are
// stored into that rank's dispatch buffer (peer stores), and the warp that finishes last raises "rows landed"
// on those ranks.  Inside the product's kernel the transfer can never wait for a place on the GPU.
struct EpDispatch {
    const void *x;                   // [T, d] token rows; null = nothing to dispatch
    int x_is_f32;                    // rows are fp32 (converted to bf16 on the way) or bf16
    void *const *row_table;          // device table [world]: every rank's dispatch buffer
    const int32_t *topk_idx, *lrank, *block_base, *dst_base;
    int T, d, n_blocks, e_local, k, tokens_per_block, rows_cap;
    uint32_t *const *rows_flags;     // device table [world]: every rank's flag_rows array
    int32_t *ticket;                 // dispatch warps that have finished (left at 0)
};

struct EpGate {
    EpDispatch disp;
    const uint32_t *wait_flags;      // this rank's flag_rows[world]; null = no wait
    const uint32_t *tile_src_mask;   // [m tiles] bit s set = the tile holds rows of source rank s; may be null
    const int32_t *tile_order;       // [m tiles] order in which the 128-row tiles are walked (this rank's own rows
                                     // first: they are here before anything crosses NVLink); null = as they lie
    uint32_t *const *signal_flags;   // device table [world] of the ranks' flag_out arrays; null = no signal
    int32_t *ticket;                 // CTAs of the signalling kernel that have finished (left at 0)
    const uint32_t *seq;             // device: sequence number of the running step
    unsigned long long timeout_ns;
    int world, rank;
};

// Bounded spin until *flag >= seq (acquire, system scope).  Returns false on
// time-out or when the device error word is already set.
__device__ __forceinline__ bool ep_wait_flag(const uint32_t *flag, uint32_t seq, unsigned long long timeout_ns,
                                             int32_t *dev_err) {
    unsigned long long t0 = 0;
    for (uint32_t spin = 0;; spin++) {
        uint32_t v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
        if ((int32_t)(v - seq) >= 0) return true;
        if ((spin & 63u) == 63u) {
            if (*(volatile int32_t *)dev_err != 0) return false;
            unsigned long long now;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
            if (t0 == 0) t0 = now;
            else if (now - t0 > timeout_ns) {
                atomicOr(dev_err, kDevErrTimeout);
                return false;
            }
        }
    }
}

// Producer side of an EpGate: wait (bounded) until every source in `need` that has not been seen yet has
// landed its rows, then order the tensor-memory-accelerator reads that follow behind the peers' stores.
__device__ __forceinline__ bool ep_gate_wait(const EpGate &g, uint32_t need, uint32_t &seen, int32_t *dev_err) {
    need &= ~seen;
    if (need == 0) return true;
    const uint32_t seq = *g.seq;
    while (need) {
        const int s = __ffs(need) - 1;
        if (!ep_wait_flag(g.wait_flags + s, seq, g.timeout_ns, dev_err)) return false;
        seen |= 1u << s;
        need &= need - 1;
    }
    asm volatile("fence.proxy.async;" ::: "memory");
    return true;
}

// Signal side of an EpGate, called by ONE WARP per CTA (all 32 lanes, converged) after that CTA's output stores
// are complete: either lane 0 of the calling warp issued them itself and has waited for them (the TMA stores of
// the persistent kernel), or the call follows a __syncthreads() that follows the storing threads'
// __threadfence_system().  The last CTA's lanes raise the flags on all ranks at once: one release store per
// lane, so the round trips to the other GPUs overlap instead of queueing behind one another.
__device__ __forceinline__ void ep_gate_signal(const EpGate &g, int n_ctas) {
    const int lane = threadIdx.x & 31;
    int last = 0;
    if (lane == 0) {
        asm volatile("fence.proxy.async;" ::: "memory");
        __threadfence_system();
        last = atomicAdd(g.ticket, 1) == n_ctas - 1;
    }
    last = __shfl_sync(0xffffffffu, last, 0);
    if (last) {
        __threadfence_system();
        if (lane == 0) *g.ticket = 0;  // every CTA has arrived; ready for the next step
        const uint32_t seq = *g.seq;
        if (lane < g.world)
            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(g.signal_flags[lane] + g.rank), "r"(seq) : "memory");
    }
}

}  // namespace omoe
