// Shared declarations of the MoE forward library: the handle, error helpers
// and the launchers each .cu file exports to api.cu.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/omoe.h"

namespace omoe {

// Rows of one expert in the dispatch buffers start on a multiple of this, so a
// 128-row tensor-core tile never straddles two experts.
constexpr int kRowAlign = 128;
constexpr int kMaxTopK = 16;
constexpr int kMaxExperts = 128;
constexpr int kRouterWarps = 8;  // warps per router block

// Device-side error word bits (set by kernels instead of trapping).
constexpr int kDevErrTimeout = 1;   // a bounded wait ran out
constexpr int kDevErrBounds = 2;    // an index check failed

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
inline int64_t round_up(int64_t a, int64_t b) { return (a + b - 1) / b * b; }

struct TensorMaps {
    CUtensorMap a_x;     // dispatch rows xp [rows_cap, d]
    CUtensorMap a_h;     // hidden rows h [rows_cap, dff]
    CUtensorMap b_gate;  // [E_local*dff, d]
    CUtensorMap b_up;    // [E_local*dff, d]
    CUtensorMap b_down;  // [E_local*d, dff]
    CUtensorMap c_y;     // expert outputs yp [rows_cap, d] (store target)
};

}  // namespace omoe

struct omoe_handle {
    omoe_config cfg;
    int e_local;      // experts owned by this rank
    int e_first;      // first owned expert (global index)
    int sm_count;
    int tokens_per_block;  // router block granularity
    int n_blocks_max;      // router blocks at t_max
    int64_t rows_cap;      // row capacity of xp / h / yp (padded)
    bool weights_set;

    // weights (device)
    float *w_router;      // [E, d] fp32
    float *router_bias;   // [E] fp32 or null
    void *w_gate, *w_up;  // [E_local, dff, d] compute dtype
    void *w_down;         // [E_local, d, dff]

    // routing workspace (device)
    float *logits;        // [t_max, E]
    int32_t *topk_idx;    // [t_max, k]
    float *topk_w;        // [t_max, k]
    int32_t *block_counts;  // [n_blocks_max, E] counts, overwritten by per-block bases
    int32_t *counts;      // [E]
    int32_t *offsets;     // [E+1] exclusive scan of counts (unpadded)
    int32_t *poffsets;    // [E+1] exclusive scan of counts rounded up to kRowAlign
    int32_t *tile_expert; // [rows_cap/kRowAlign] local expert of each 128-row tile
    // Views the expert kernels read.  On one GPU they alias the arrays above;
    // with expert parallelism they describe the rows received from all ranks.
    int32_t *ex_counts, *ex_poffsets, *ex_tile_expert;
    int32_t *pos;         // [t_max*k] row of each pick in the padded dispatch buffer
    int32_t *perm_out;    // [t_max*k] scratch for omoe_get_routing
    int32_t *dev_err;     // device error word

    // activations (device, compute dtype)
    void *xp, *hbuf, *yp;
    // staging for omoe_forward_host
    void *x_stage, *y_stage;
    size_t stage_bytes;

    omoe::TensorMaps maps;
    bool maps_ready;

    // bookkeeping of the last forward
    int last_T;
    int last_io_dtype;
    cudaStream_t last_stream;
    int last_launches;
    bool profiling;
    cudaEvent_t ev[OMOE_N_STAGES + 1];
    bool ev_valid;

    void *ep;  // expert-parallel state (ep.cu)

    char err[512];
};

namespace omoe {

// ---- launchers (defined in the kernel files) ------------------------------
// All return cudaError_t of the launch and add the kernels they launched to *n.

cudaError_t launch_router(omoe_handle *h, const void *x, int io_dtype, int T, cudaStream_t s, int *n);
cudaError_t launch_scan(omoe_handle *h, int T, cudaStream_t s, int *n);
cudaError_t launch_permute(omoe_handle *h, const void *x, int io_dtype, int T, cudaStream_t s, int *n);
cudaError_t launch_perm_readout(omoe_handle *h, int T, cudaStream_t s);
cudaError_t launch_combine(omoe_handle *h, void *y, int io_dtype, int T, cudaStream_t s, int *n);
cudaError_t launch_experts_f32(omoe_handle *h, cudaStream_t s, int *n);
cudaError_t launch_experts_bf16(omoe_handle *h, cudaStream_t s, int *n, cudaEvent_t mid);
cudaError_t launch_convert_f32_to_bf16(const float *src, __nv_bfloat16 *dst, int64_t n, cudaStream_t s);
cudaError_t launch_convert_bf16_to_f32(const __nv_bfloat16 *src, float *dst, int64_t n, cudaStream_t s);

// Encodes the TMA descriptors of the bf16 path; returns false and fills h->err
// when the driver entry point is missing or an encode fails.
bool build_tensor_maps(omoe_handle *h);

int router_tokens_per_block(int E);

}  // namespace omoe
