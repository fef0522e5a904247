// Expert-parallel transport of the MoE forward (ep.cu).
#pragma once

#include "common.cuh"

namespace omoe {

// Control block of one rank, written by its peers.  Lives in memory the other ranks have mapped.
struct EpCtl {
    int32_t cnt[2][kMaxWorld][kMaxExperts];  // [parity][source rank][expert]
    uint32_t flag_cnt[2][kMaxWorld];         // seq once source's count row is complete
    uint32_t flag_rows[kMaxWorld];           // seq once source's rows have landed in my dispatch buffer
    uint32_t flag_out[kMaxWorld];            // seq once owner's expert outputs are readable
};

int ep_create(omoe_handle *h);   // allocates the control block and receive-side layout arrays
int ep_export(omoe_handle *h, void *blob);
int ep_import(omoe_handle *h, const void *all_blobs);
// All ranks live in this process (one handle per GPU): exchange plain device pointers instead of IPC handles.
int ep_connect_local(omoe_handle **hs, int world);
// x has element type x_dtype, y (and resid, when not null) y_dtype
int ep_forward(omoe_handle *h, const void *x, int x_dtype, void *y, int y_dtype, const void *resid, int T,
               cudaStream_t s);
void ep_destroy(omoe_handle *h);

// Pieces of the expert-parallel backward pass.  A backward is a step of its own (ep_bw_advance): gradient rows
// travel to the experts' owners like the forward's rows (peer stores, "rows landed" flags), input-gradient
// rows are read back from the owners like the forward's outputs (peer loads behind "outputs ready" flags).
bool ep_ready(const omoe_handle *h);
void ep_grad_buffers(omoe_handle *h, void **dyp, void **dxp, void ***dyp_table, void ***dxp_table);
cudaError_t ep_bw_advance(omoe_handle *h, cudaStream_t s);
EpSignal ep_rows_signal(omoe_handle *h);
EpWait ep_out_wait(omoe_handle *h);
cudaError_t ep_signal_rows(omoe_handle *h, cudaStream_t s);
cudaError_t ep_wait_rows(omoe_handle *h, cudaStream_t s);
cudaError_t ep_signal_out(omoe_handle *h, cudaStream_t s);

}  // namespace omoe
