/*
 * omoe.h — C ABI of libomoe.so: the mixture-of-experts FFN layer for
 * Omega-AI (forward, and the backward pass for training), built for NVIDIA
 * B200 (sm_100a).
 *
 * The library takes the place of the JCuda "load a CUfunction by name and
 * cuLaunchKernel it" plumbing for this one layer.  A Java layer (or any other
 * host) passes raw 64-bit device addresses and sizes; no C++ or torch types
 * cross this boundary.  Every call returns OMOE_OK (0) or a negative
 * OMOE_ERR_* code and never exits the process or throws.
 *
 * Conventions shared by all entry points
 *   - Weights are row-major [out,in], as the engine's FullyLayer stores them
 *     (src/main/java/com/omega/engine/nn/layer/FullyLayer.java:181), experts
 *     contiguous on the leading dimension.
 *   - Work is enqueued on the CUDA stream the caller passes; 0 means the legacy
 *     default stream, which is what every reference kernel launch uses
 *     (src/main/java/com/omega/engine/gpu/BaseKernel.java:66-72), so later
 *     JCuda work is ordered after it without extra synchronisation.
 *   - The library runs in the caller's current CUDA context and on its current
 *     device; it never switches devices and never frees caller buffers.
 *   - A handle is used by one host thread at a time.
 */
#ifndef OMOE_H
#define OMOE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define OMOE_VERSION 1

#if defined(__GNUC__)
#define OMOE_API __attribute__((visibility("default")))
#else
#define OMOE_API
#endif

/* element types for weights and activations */
#define OMOE_F32 0
#define OMOE_BF16 1

/* status codes */
#define OMOE_OK 0
#define OMOE_ERR_INVALID (-1)      /* bad argument (null pointer, bad shape, bad dtype) */
#define OMOE_ERR_CUDA (-2)         /* a CUDA runtime/driver call failed */
#define OMOE_ERR_TOO_LARGE (-3)    /* T exceeds the handle's t_max (no hidden realloc) */
#define OMOE_ERR_STATE (-4)        /* call order (e.g. forward before set_weights) */
#define OMOE_ERR_UNSUPPORTED (-5)  /* shape not supported by the selected arithmetic */
#define OMOE_ERR_DEVICE (-6)       /* a kernel reported a device-side error word */
#define OMOE_ERR_COMM (-7)         /* expert-parallel transport failed */
#define OMOE_ERR_NOMEM (-8)        /* device or host allocation failed */

typedef struct omoe_handle omoe_handle;

/*
 * Layer description.  Mirrors the constructor arguments of the Java layer
 * (embedDim, dff, numExperts, topK, bias, network) that sits where
 * LlamaMLPLayer is built today
 * (src/main/java/com/omega/engine/nn/layer/llama/LlamaTransformerBlock.java:97).
 */
typedef struct omoe_config {
    int32_t t_max;           /* largest token count one forward may carry on this rank */
    int32_t d_model;         /* multiple of 8 */
    int32_t d_ff;            /* multiple of 8 */
    int32_t n_experts;       /* global expert count E */
    int32_t top_k;           /* 1..min(E,16) */
    int32_t compute_dtype;   /* OMOE_F32: fp32 FMA everywhere; OMOE_BF16: bf16 tensor cores, fp32 accumulate */
    int32_t renormalize;     /* 1: gate weights divided by the sum over the k picks */
    int32_t has_router_bias; /* 1: a per-expert bias is added to the router logits */
    int32_t world;           /* expert-parallel ranks (1 = single GPU, at most 8) */
    int32_t rank;            /* this rank; owns experts [rank*E/world, (rank+1)*E/world) */
    int32_t recv_rows_max;   /* EP only: capacity (rows) of the buffer that receives dispatched
                                tokens; 0 = t_max*top_k*world (worst case) */
    int32_t reserved[5];     /* must be zero */
} omoe_config;

/* Replaces: constructing the layer's kernels (BaseKernel.java:38-56 loads the
 * CUfunctions; FullyLayer.initKernel at FullyLayer.java:108-114).  Allocates
 * the workspace (dispatch buffers, maps, bf16 weight copies) once. */
OMOE_API int omoe_create(const omoe_config *cfg, omoe_handle **out);
OMOE_API int omoe_destroy(omoe_handle *h);

/* Message for the last error on this handle (or on the last failed create
 * when h is NULL).  The pointer stays valid until the next call on the handle. */
OMOE_API const char *omoe_last_error(const omoe_handle *h);

/*
 * Copies (and for compute_dtype=BF16 converts) the weights from DEVICE memory.
 *   w_router [E, d]              always kept in fp32 for the router
 *   router_bias [E] or NULL
 *   w_gate, w_up [E_local, d_ff, d]   (linear1 and linear3 of LlamaMLPLayer,
 *   w_down [E_local, d, d_ff]          linear2; LlamaMLPLayer.java:70-87)
 * E_local = E/world experts owned by this rank, in global expert order.
 * src_dtype is the element type of all five buffers.
 * Replaces: the per-layer weight tensors handed to cublasSgemm
 * (FullyLayer.java:235 -> GPUOP.java:405-417).
 */
OMOE_API int omoe_set_weights(omoe_handle *h, const void *w_router, const void *router_bias,
                     const void *w_gate, const void *w_up, const void *w_down,
                     int32_t src_dtype, void *cuda_stream);

/*
 * y[T, d] = MoE(x[T, d]) with x and y in DEVICE memory of element type
 * io_dtype.  Replaces LlamaMLPLayer.output()
 * (LlamaMLPLayer.java:117-130: linear1 -> SiLU -> linear3 -> mul -> linear2)
 * with router -> top-k -> dispatch -> grouped SwiGLU -> combine.  Does not
 * synchronise the host.  With world > 1 this is a collective call: every rank
 * calls it with its own T tokens (T may differ per rank).
 */
OMOE_API int omoe_forward(omoe_handle *h, const void *x_dev, void *y_dev, int32_t T,
                 int32_t io_dtype, void *cuda_stream);

/*
 * The feed-forward half of a transformer block in one call:
 *   y = x + MoE( rmsnorm(x) * gamma )
 * i.e. norm2 -> mlp -> residual add of LlamaTransformerBlock.output()
 * (src/main/java/com/omega/engine/nn/layer/llama/LlamaTransformerBlock.java:134-136),
 * with the RMSNorm arithmetic of rmsnorm_forward_kernel2
 * (src/main/resources/cu/RMSKernel.cu:185-224: rms = sqrtf(sum(x^2)/d + eps),
 * (x / rms) * gamma; the reference fixes eps = 1e-5).  The normalised rows are
 * written once in the layer's compute dtype and the residual add happens inside
 * the combine kernel, so the two extra passes over [T, d] that the reference's
 * RMS and add kernels make disappear.  gamma_dev [d_model] fp32 on the device;
 * x_dev must not alias y_dev.
 */
OMOE_API int omoe_forward_block(omoe_handle *h, const void *x_dev, const float *gamma_dev, float eps,
                                void *y_dev, int32_t T, int32_t io_dtype, void *cuda_stream);

/*
 * Same layer with x and y in HOST memory (pinned memory makes the copies
 * asynchronous).  This is the call behind Layer.forward(Tensor) for a Tensor
 * whose data lives in its float[] (Tensor.hostToDevice / syncHost,
 * src/main/java/com/omega/engine/tensor/Tensor.java:559-579): H2D copy of x,
 * forward, D2H copy of y, then a stream synchronise so y is readable on return.
 * On one GPU a batch of 8192 tokens or more is cut into chunks of at least 4096 whose
 * copies overlap the kernels of their neighbours (tokens are independent, so
 * y is bit-identical); the routing read-outs then describe the last chunk.
 * With world > 1 the call is collective like omoe_forward, and the batch is cut
 * too: into as many chunks (at most 8, of at least 512 tokens) as t_max allows,
 * the same number on every rank, each chunk one collective forward.
 *
 * omoe_forward_host_async is the same call without the final synchronise: it
 * enqueues the copies and the forward(s) and returns; y_host is complete, and
 * a device-side failure is reported, once omoe_wait(h) has returned.  Several
 * calls may be enqueued before one omoe_wait: they run in order, each as one
 * forward (no chunks), and two staging sets alternate between them so that the
 * copy-in of the next call and the copy-out of the previous one run while the
 * kernels of the current one do (the host buffers of a call must stay
 * untouched until the wait).  x_host must hold the rows when the call is made:
 * the copy-in is not ordered behind work queued earlier on cuda_stream.  The reference splits the same
 * work into Tensor.hostToDevice() and Tensor.syncHost()
 * (src/main/java/com/omega/engine/tensor/Tensor.java:559-579), each of which
 * synchronises the whole device.
 */
OMOE_API int omoe_forward_host(omoe_handle *h, const void *x_host, void *y_host, int32_t T,
                      int32_t io_dtype, void *cuda_stream);
OMOE_API int omoe_forward_host_async(omoe_handle *h, const void *x_host, void *y_host, int32_t T,
                      int32_t io_dtype, void *cuda_stream);
OMOE_API int omoe_wait(omoe_handle *h);

/*
 * Training mode and the backward pass.
 *
 * omoe_set_training(h, 1) allocates the buffers of the backward pass (first call only) and makes every
 * following omoe_forward / omoe_forward_block keep what the backward needs: the pre-activation rows of
 * the gate and up products, h, the expert outputs and the routing.  The reference's layers keep the same
 * things as the output tensors of linear1, the SiLU layer and linear3
 * (src/main/java/com/omega/engine/nn/layer/llama/LlamaMLPLayer.java:117-123).  A training-mode forward runs
 * the gate and up products unfused (their outputs must be stored) and rounds g and u to the compute dtype
 * before SiLU; on a bf16 layer its output can differ from the inference forward's in the last bf16 place.
 * omoe_set_training(h, 0) goes back to the inference kernels and keeps the buffers.
 *
 * omoe_backward replaces LlamaMLPLayer.diff() (LlamaMLPLayer.java:139-158) and the FullyLayer.diff() calls
 * under it (src/main/java/com/omega/engine/nn/layer/FullyLayer.java:292-334): given dy_dev [T, d_model]
 * (gradient of the output of the LAST forward, which must have run in training mode with the same T,
 * io_dtype and x_dev contents), it writes dx_dev [T, d_model] of io_dtype and the weight gradients
 * (library-owned, fp32, OVERWRITTEN by every call as FullyLayer.diff() overwrites diffW):
 * d W_gate, d W_up [E/world, d_ff, d_model], d W_down [E/world, d_model, d_ff], d W_router [E, d_model],
 * d router_bias [E].  The expert picks are constants (no gradient flows through the selection); the gate
 * weights' gradient reaches the router through the renormalisation and the reference's softmax_back rule
 * (src/main/resources/cu/SoftmaxKernel.cu:100-112).
 * Does not synchronise the host.
 *
 * omoe_backward_block is the backward of omoe_forward_block (y = x + MoE(rmsnorm(x) * gamma)), i.e. of
 * norm2 -> mlp -> residual add in LlamaTransformerBlock (LlamaTransformerBlock.java:134-136): the layer's
 * backward on the normalised rows the forward kept, then the RMSNorm backward of rmsnorm_backward_kernel2
 * (src/main/resources/cu/RMSKernel.cu:225-275) with the residual branch's dy added in the same pass.
 * x_dev must hold the rows given to that forward; dgamma_dev [d_model] fp32 is overwritten (the reference
 * accumulates it with atomics; here the sum has a fixed order).
 *
 * With world > 1 omoe_backward is a collective call like omoe_forward (every rank calls it, T may differ per
 * rank): the gradient rows travel to the experts' owners and the input-gradient rows back through peer memory,
 * ordered by the same device-side flags.  The expert weight gradients of a rank ([n_experts/world, ...]) are
 * complete; d W_router and d router_bias cover the rank's own tokens and must be summed over the ranks by the
 * caller (the router is replicated); the auxiliary loss term uses the rank's own tokens and counts.
 * With world > 1 a forward takes ONE backward: a second omoe_backward without a new training-mode forward
 * returns OMOE_ERR_STATE (on one GPU a backward may be repeated).
 * All device pointers of the forward and backward entry points must be 16-byte aligned (rows move as
 * 16-byte vectors); a misaligned one is refused with OMOE_ERR_INVALID before anything is launched.
 *
 * omoe_get_weight_grads copies the gradients of the last omoe_backward into the caller's DEVICE (or host)
 * fp32 buffers (any may be NULL) and synchronises the stream.
 */
OMOE_API int omoe_set_training(omoe_handle *h, int32_t on);
OMOE_API int omoe_backward(omoe_handle *h, const void *x_dev, const void *dy_dev, void *dx_dev, int32_t T,
                           int32_t io_dtype, void *cuda_stream);
OMOE_API int omoe_backward_block(omoe_handle *h, const void *x_dev, const float *gamma_dev, float eps,
                                 const void *dy_dev, void *dx_dev, float *dgamma_dev, int32_t T, int32_t io_dtype,
                                 void *cuda_stream);
OMOE_API int omoe_get_weight_grads(omoe_handle *h, float *d_router, float *d_router_bias, float *d_gate,
                                   float *d_up, float *d_down, void *cuda_stream);

/*
 * Auxiliary load-balancing loss (no reference counterpart; the usual switch-routing form):
 *   L = E * sum_e f_e * P_e,  f_e = counts[e] / (T * top_k),  P_e = mean over the step's tokens of the
 *   router probability of expert e.
 * omoe_set_aux_loss(h, coef) (training mode on) makes every following omoe_backward return the gradients of
 * <dy, y> + coef * L: the extra term coef * E * f_e / T enters at the router's probabilities (f_e is a
 * constant) and reaches d W_router, d router_bias and dx.  coef = 0 (the default) switches it off.
 * omoe_get_aux_loss writes L of the last forward to *loss_host; it launches one small kernel on that
 * forward's stream and synchronises it.
 */
OMOE_API int omoe_set_aux_loss(omoe_handle *h, float coef);
OMOE_API int omoe_get_aux_loss(omoe_handle *h, float *loss_host);

/*
 * Routing results of the last forward on this rank, copied to HOST buffers
 * (any may be NULL).  Synchronises the stream of that forward.
 *   topk_idx [T, k] int32, topk_w [T, k] fp32, counts [E] int32,
 *   offsets [E+1] int32 (exclusive scan of counts),
 *   perm [T*k] int32: perm[offsets[e]+r] = t*k+j, expert-major, stable in t*k+j.
 * There is no reference counterpart; this exists so parity tests can compare
 * indices, counts and the permutation bit for bit.
 */
OMOE_API int omoe_get_routing(omoe_handle *h, int32_t *topk_idx, float *topk_w, int32_t *counts,
                     int32_t *offsets, int32_t *perm);

/* Router logits [T, E] fp32 of the last forward, to a HOST buffer (debug/parity). */
OMOE_API int omoe_get_logits(omoe_handle *h, float *logits);

/* Kernels launched by the last forward on this handle (for accounting). */
OMOE_API int omoe_last_launch_count(const omoe_handle *h);

/* Per-stage device times of the last forward in milliseconds, when stage
 * timing was enabled with omoe_set_profiling(h, 1).  Order: router, scan,
 * permute, dispatch, up_gate, down, return, combine.  Synchronises. */
#define OMOE_N_STAGES 8
OMOE_API int omoe_set_profiling(omoe_handle *h, int32_t enabled);
OMOE_API int omoe_get_stage_ms(omoe_handle *h, float *ms /* [OMOE_N_STAGES] */);
/* The same for an earlier forward: back = 0 is the last one, 1 the one before, ... up to the last 32 forwards
 * made since profiling was switched on.  Lets a caller time a run of forwards back to back (no host
 * synchronisation between them) and read every forward's stages afterwards.  No reference counterpart. */
OMOE_API int omoe_get_stage_ms_at(omoe_handle *h, int32_t back, float *ms /* [OMOE_N_STAGES] */);

/*
 * Expert-parallel transport.  The reference's only multi-GPU mechanism is
 * cudaMemcpyPeerAsync between Java threads, driven from the host
 * (src/main/java/com/omega/engine/parallel/dp/NetworkRunnable.java:442-459).
 * Here every rank is one process on one GPU of an NVLink/NVSwitch node, and
 * the kernels move the rows themselves: the dispatch kernel stores each token
 * row into the buffer of the rank that owns the expert, the combine kernel
 * loads expert outputs back from the owners, both over peer-mapped memory.
 *
 * Set-up, once: every rank calls omoe_ep_export, the host gathers the blobs
 * of all ranks in rank order (any transport: a file, sockets,
 * torch.distributed), every rank calls omoe_ep_import with the gathered
 * array, and a host barrier follows before the first forward.  After that
 * omoe_forward is a collective: every rank calls it the same number of
 * times, each with its own T (0 is allowed).  A rank that does not show up
 * makes the others' bounded waits (10 s, or OMOE_EP_WAIT_MS) run out:
 * they return normally and the next synchronising call reports
 * OMOE_ERR_DEVICE.
 */
#define OMOE_EP_BLOB_BYTES 320
OMOE_API int omoe_ep_export(omoe_handle *h, void *blob /* [OMOE_EP_BLOB_BYTES] */);
OMOE_API int omoe_ep_import(omoe_handle *h, const void *all_blobs /* [world][OMOE_EP_BLOB_BYTES] */);

/*
 * The same set-up when ONE process drives every GPU, as the reference's own multi-GPU mode does (one thread
 * per device in one JVM: src/main/java/com/omega/engine/parallel/dp/DP.java:68-94): handles[r] was created
 * with (world, rank = r) while device r' was current, all in this process.  The call enables peer access
 * between the handles' devices and hands every handle the others' buffers (no IPC).  It is the one entry
 * point that switches the current device (and puts the caller's back before it returns).  Afterwards each
 * rank's omoe_forward / omoe_backward is called with its own device current, from one thread per device or
 * from one thread in turn: the calls only enqueue work, so issuing them one after the other cannot deadlock
 * as long as every rank's call has been issued before the host waits for any of them.  Such a process must load
 * its CUDA modules eagerly (CUDA_MODULE_LOADING=EAGER in its environment): with lazy loading the first use of a
 * kernel on one device can wait for the kernel running on another device, which is itself waiting (bounded) for
 * that rank.
 */
OMOE_API int omoe_ep_connect_local(omoe_handle **handles, int32_t world);

/*
 * Routing only, with NO allocation.  This entry point has no counterpart in
 * the reference.  It exists for hosts that may not call cudaMalloc where they
 * need a routing decision (a serving loop whose memory pool owns all free
 * device memory and bans allocation on the request path, or any caller that
 * must avoid the device-wide synchronisation an allocation implies).  It runs
 * the same fused router kernel as omoe_forward; the kernel's scratch lives in
 * a fixed array inside the library image (about 4.3 MiB per GPU that loads
 * the library, held until the process exits) and the call itself makes no
 * cudaMalloc, cudaFree or other allocating call.  One qualification: with
 * CUDA's lazy module loading the driver brings this library's module -- the
 * array included -- onto the device the first time one of its symbols is
 * used in a context, so the FIRST call in a context may make the driver
 * reserve those 4.3 MiB; later calls leave the device's free memory untouched.
 * Make that first call early (at start-up, outside the request path).
 *
 *   x_dev [T, d_model] of io_dtype; w_router_dev [n_experts, d_model] fp32;
 *   router_bias_dev [n_experts] fp32 or NULL.
 *   Outputs (caller's DEVICE buffers): topk_idx_dev [T, top_k] int32,
 *   topk_w_dev [T, top_k] fp32, counts_dev [n_experts] int32.
 *
 * Limits: T <= OMOE_NOALLOC_MAX_TOKENS, n_experts <= 128, top_k <= 16; a call
 * beyond them returns OMOE_ERR_TOO_LARGE and launches nothing.
 * x_dev and w_router_dev must be 16-byte aligned (OMOE_ERR_INVALID otherwise).
 * The first call in each CUDA context (one per device for a runtime-API host; a
 * host that creates its own driver-API contexts has one per context) looks up
 * the array's device address in that context; make that first call before any
 * stream capture begins there.
 * All calls in one context share the array: it keeps the previous call's
 * contents (nothing in it needs clearing between calls), and two calls whose
 * kernels overlap on the GPU (different streams, no ordering) race on it.
 * Error text: omoe_route_noalloc_error().
 */
#define OMOE_NOALLOC_MAX_TOKENS 4096
OMOE_API int omoe_route_noalloc(const void *x_dev, const float *w_router_dev, const float *router_bias_dev,
                                int32_t T, int32_t d_model, int32_t n_experts, int32_t top_k,
                                int32_t renormalize, int32_t io_dtype, int32_t *topk_idx_dev,
                                float *topk_w_dev, int32_t *counts_dev, void *cuda_stream);
OMOE_API const char *omoe_route_noalloc_error(void);

#ifdef __cplusplus
}
#endif
#endif /* OMOE_H */
