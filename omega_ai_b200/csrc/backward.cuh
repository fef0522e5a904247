// Backward pass of the layer (backward.cu) and the tensor-core products it adds to the forward's.
#pragma once

#include "common.cuh"

namespace omoe {

int bw_set_training(omoe_handle *h, int on);
bool bw_training(const omoe_handle *h);
void bw_weights_changed(omoe_handle *h);
void bw_forward_invalidate(omoe_handle *h);
// A training-mode forward of no rows on one GPU launches nothing and still counts as the forward a backward follows.
void bw_forward_empty(omoe_handle *h);
// Expert stage of a training-mode forward: g and u kept, then h = silu(g) * u, then the down product.
cudaError_t bw_forward_experts(omoe_handle *h, int T, cudaStream_t s, int *n);
// x_is_compute: x has the layer's compute dtype (the normalised rows of the block form) instead of io_dtype
int bw_backward(omoe_handle *h, const void *x, bool x_is_compute, const void *dy, void *dx, int T, int io_dtype,
                cudaStream_t s, int *launches);
int bw_backward_block(omoe_handle *h, const void *x, const float *gamma, float eps, const void *dy, void *dx,
                      float *dgamma, int T, int io_dtype, cudaStream_t s, int *launches);
int bw_get_grads(omoe_handle *h, float *d_router, float *d_bias, float *d_gate, float *d_up, float *d_down,
                 cudaStream_t s);
int bw_set_aux(omoe_handle *h, float coef);
int bw_aux_loss(omoe_handle *h, float *loss_host, cudaStream_t s);
void bw_destroy(omoe_handle *h);

// 2-D bf16 tensor map: [rows, cols] with `ld` elements between rows, box box_rows x 64 columns, 128-byte swizzle.
bool encode_map_bf16(CUtensorMap *m, void *ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows);
// out[r, 0..n_out) = a[r, 0..K) * B_e^T for the rows in use, B_e = rows [e*n_out, (e+1)*n_out) of b ([.., K]):
// the persistent tcgen05 kernel of the forward's down product with other operands (experts_sm100.cu).
cudaError_t launch_grouped_plain(omoe_handle *h, cudaStream_t s, const CUtensorMap &a, const CUtensorMap &b,
                                 const CUtensorMap &c, int n_out, int K);
// Per local expert e: C_e [M, N] (fp32) = AT[:, seg_e] * BT[:, seg_e]^T, seg_e = the expert's (padded, zero-filled)
// rows; at [M, rows_cap], bt [N, rows_cap] bf16.  Row m of C_e goes to out0[e][m][:] when m < split, else to
// out1[e][m - split][:].  (experts_sm100_wgrad.cu)
cudaError_t launch_wgrad_bf16(omoe_handle *h, cudaStream_t s, const CUtensorMap &at, const CUtensorMap &bt, int M,
                              int N, int split, float *out0, float *out1);

// The same product straight from the row-major activations a [rows_cap, M], b [rows_cap, N] (tensor maps with a
// 64-row box): MN-major tensor-core operands, no transposed copies.  Padding rows of a must be zero, of b finite.
cudaError_t launch_wgrad_bf16_rows(omoe_handle *h, cudaStream_t s, const CUtensorMap &a, const CUtensorMap &b, int M,
                                   int N, int split, float *out0, float *out1);

}  // namespace omoe
