// Expert-parallel transport (placeholder until the NCCL path lands).
#include "ep.cuh"

namespace omoe {

int ep_unique_id(void *) { return OMOE_ERR_UNSUPPORTED; }
int ep_init(omoe_handle *h, const void *) {
    snprintf(h->err, sizeof(h->err), "expert parallelism is not built yet");
    return OMOE_ERR_UNSUPPORTED;
}
int ep_forward(omoe_handle *h, const void *, void *, int, int, cudaStream_t) {
    snprintf(h->err, sizeof(h->err), "expert parallelism is not built yet");
    return OMOE_ERR_UNSUPPORTED;
}
void ep_destroy(omoe_handle *) {}

}  // namespace omoe
