// Expert-parallel transport of the MoE forward (ep.cu).
#pragma once

#include "common.cuh"

namespace omoe {

int ep_create(omoe_handle *h);   // allocates the control block and receive-side layout arrays
int ep_export(omoe_handle *h, void *blob);
int ep_import(omoe_handle *h, const void *all_blobs);
// x has element type x_dtype, y (and resid, when not null) y_dtype
int ep_forward(omoe_handle *h, const void *x, int x_dtype, void *y, int y_dtype, const void *resid, int T,
               cudaStream_t s);
void ep_destroy(omoe_handle *h);

}  // namespace omoe
