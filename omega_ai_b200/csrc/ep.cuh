// Expert-parallel transport of the MoE forward (ep.cu).
#pragma once

#include "common.cuh"

namespace omoe {

int ep_unique_id(void *id_out);
int ep_init(omoe_handle *h, const void *id);
int ep_forward(omoe_handle *h, const void *x, void *y, int T, int io_dtype, cudaStream_t s);
void ep_destroy(omoe_handle *h);

}  // namespace omoe
