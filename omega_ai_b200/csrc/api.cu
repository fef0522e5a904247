// C ABI of libomoe.so (declared in include/omoe.h): handle life cycle, weight
// upload, the forward pass and the read-outs used by parity tests.
#include <stdarg.h>
#include <stdlib.h>
#include <string.h>

#include <new>

#include <nvtx3/nvToolsExt.h>

#include "backward.cuh"
#include "common.cuh"
#include "ep.cuh"

using namespace omoe;

namespace {

thread_local char g_create_err[512] = "";

int fail(omoe_handle *h, int code, const char *fmt, ...) {
    char *dst = h ? h->err : g_create_err;
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(dst, 512, fmt, ap);
    va_end(ap);
    return code;
}

#define CU_TRY(h, expr)                                                                            \
    do {                                                                                           \
        cudaError_t _e = (expr);                                                                   \
        if (_e != cudaSuccess)                                                                     \
            return fail(h, _e == cudaErrorMemoryAllocation ? OMOE_ERR_NOMEM : OMOE_ERR_CUDA,       \
                        "%s failed: %s", #expr, cudaGetErrorString(_e));                           \
    } while (0)

template <typename T>
cudaError_t dev_alloc(T **p, size_t count) {
    *p = nullptr;
    if (count == 0) count = 1;
    return cudaMalloc(reinterpret_cast<void **>(p), count * sizeof(T));
}

size_t elt_size(int dtype) { return dtype == OMOE_BF16 ? 2 : 4; }

// NVTX range over the host side of one entry point (header-only NVTX: a no-op unless a tool is attached), so a
// timeline shows which launches belong to which call of the layer.
struct NvtxRange {
    explicit NvtxRange(const char *name) { nvtxRangePushA(name); }
    ~NvtxRange() { nvtxRangePop(); }
};

bool misaligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) != 0; }

__global__ void f32_to_bf16_kernel(const float *__restrict__ src, __nv_bfloat16 *__restrict__ dst, int64_t n) {
    int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x * 4;
    for (; i + 3 < n; i += stride) {
        float4 v = *reinterpret_cast<const float4 *>(src + i);
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 o;
        o.x = *reinterpret_cast<uint32_t *>(&a);
        o.y = *reinterpret_cast<uint32_t *>(&b);
        *reinterpret_cast<uint2 *>(dst + i) = o;
    }
}

__global__ void bf16_to_f32_kernel(const __nv_bfloat16 *__restrict__ src, float *__restrict__ dst, int64_t n) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) dst[i] = __bfloat162float(src[i]);
}

int check_dev_err(omoe_handle *h) {
    int32_t v = 0;
    CU_TRY(h, cudaMemcpy(&v, h->dev_err, sizeof(v), cudaMemcpyDeviceToHost));
    if (v != 0) {
        cudaMemset(h->dev_err, 0, sizeof(int32_t));
        cudaMemset(h->ticket, 0, sizeof(int32_t));
        cudaMemset(h->ticket2, 0, sizeof(int32_t));
        cudaMemset(h->ticket3, 0, sizeof(int32_t));
        return fail(h, OMOE_ERR_DEVICE, "device error word = %d (%s%s)", v,
                    (v & kDevErrTimeout) ? "a bounded wait ran out " : "",
                    (v & kDevErrBounds) ? "an index check failed" : "");
    }
    return OMOE_OK;
}

}  // namespace

namespace omoe {

cudaError_t launch_convert_f32_to_bf16(const float *src, __nv_bfloat16 *dst, int64_t n, cudaStream_t s) {
    if (n == 0) return cudaSuccess;
    int64_t blocks = (n / 4 + 255) / 256;  // n is a multiple of 8 for every weight tensor
    if (blocks > 148 * 16) blocks = 148 * 16;
    f32_to_bf16_kernel<<<(int)blocks, 256, 0, s>>>(src, dst, n);
    return cudaGetLastError();
}

cudaError_t launch_convert_bf16_to_f32(const __nv_bfloat16 *src, float *dst, int64_t n, cudaStream_t s) {
    if (n == 0) return cudaSuccess;
    int64_t blocks = (n + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    bf16_to_f32_kernel<<<(int)blocks, 256, 0, s>>>(src, dst, n);
    return cudaGetLastError();
}

}  // namespace omoe

extern "C" {

const char *omoe_last_error(const omoe_handle *h) { return h ? h->err : g_create_err; }

int omoe_destroy(omoe_handle *h) {
    if (!h) return OMOE_OK;
    ep_destroy(h);
    bw_destroy(h);
    void *ptrs[] = {h->w_router, h->w_router_bf16, h->router_bias, h->w_gate, h->w_up, h->w_down, h->logits, h->topk_idx,
                    h->topk_w, h->block_counts, h->block_base, h->counts, h->offsets, h->poffsets, h->tile_expert, h->pos, h->lrank,
                    h->perm_out, h->dev_err, h->xp, h->hbuf, h->yp, h->xn, h->x_stage[0], h->y_stage[0], h->x_stage[1], h->y_stage[1], h->d_row_table,
                    h->d_out_table, h->ticket, h->ticket2, h->ticket3, h->dst_base != h->poffsets ? h->dst_base : nullptr};
    for (void *p : ptrs)
        if (p) cudaFree(p);
    for (int r = 0; r < kProfSlots; r++)
        for (int i = 0; i <= OMOE_N_STAGES; i++)
            if (h->ev_ring[r][i]) cudaEventDestroy(h->ev_ring[r][i]);
    for (int i = 0; i < kHostChunksMax; i++) {
        if (h->ev_in[i]) cudaEventDestroy(h->ev_in[i]);
        if (h->ev_out[i]) cudaEventDestroy(h->ev_out[i]);
    }
    for (int i = 0; i < 2; i++) {
        if (h->ev_set_fwd[i]) cudaEventDestroy(h->ev_set_fwd[i]);
        if (h->ev_set_d2h[i]) cudaEventDestroy(h->ev_set_d2h[i]);
    }
    if (h->copy_in) cudaStreamDestroy(h->copy_in);
    if (h->copy_out) cudaStreamDestroy(h->copy_out);
    delete h;
    return OMOE_OK;
}

int omoe_create(const omoe_config *cfg, omoe_handle **out) {
    if (!cfg || !out) return fail(nullptr, OMOE_ERR_INVALID, "omoe_create: null argument");
    *out = nullptr;
    const omoe_config &c = *cfg;
    if (c.t_max <= 0 || c.d_model <= 0 || c.d_ff <= 0 || c.n_experts <= 0 || c.top_k <= 0)
        return fail(nullptr, OMOE_ERR_INVALID, "omoe_create: sizes must be positive");
    if (c.d_model % 8 || c.d_ff % 8)
        return fail(nullptr, OMOE_ERR_INVALID, "omoe_create: d_model and d_ff must be multiples of 8");
    if (c.n_experts > kMaxExperts)
        return fail(nullptr, OMOE_ERR_UNSUPPORTED, "omoe_create: at most %d experts", kMaxExperts);
    if (c.top_k > c.n_experts || c.top_k > kMaxTopK)
        return fail(nullptr, OMOE_ERR_INVALID, "omoe_create: top_k must be <= min(n_experts, %d)", kMaxTopK);
    if (c.compute_dtype != OMOE_F32 && c.compute_dtype != OMOE_BF16)
        return fail(nullptr, OMOE_ERR_INVALID, "omoe_create: compute_dtype must be OMOE_F32 or OMOE_BF16");
    if (c.world < 1 || c.world > kMaxWorld || c.rank < 0 || c.rank >= c.world || c.n_experts % c.world)
        return fail(nullptr, OMOE_ERR_INVALID, "omoe_create: need 0 <= rank < world <= %d and world dividing n_experts",
                    kMaxWorld);
    if (c.compute_dtype == OMOE_BF16 && (c.d_model < 64 || c.d_ff < 64))
        return fail(nullptr, OMOE_ERR_UNSUPPORTED, "omoe_create: the bf16 path needs d_model, d_ff >= 64");
    for (int i = 0; i < 5; i++)
        if (c.reserved[i] != 0) return fail(nullptr, OMOE_ERR_INVALID, "omoe_create: reserved fields must be zero");

    int dev = 0, major = 0, sms = 0;
    CU_TRY(nullptr, cudaGetDevice(&dev));
    CU_TRY(nullptr, cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    CU_TRY(nullptr, cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    if (major != 10)
        return fail(nullptr, OMOE_ERR_UNSUPPORTED,
                    "omoe_create: this library is built for sm_100a only (device has compute capability %d.x)", major);

    omoe_handle *h = new (std::nothrow) omoe_handle();
    if (!h) return fail(nullptr, OMOE_ERR_NOMEM, "omoe_create: host allocation failed");
    memset(h, 0, sizeof(*h));
    h->cfg = c;
    h->e_local = c.n_experts / c.world;
    h->e_first = c.rank * h->e_local;
    h->sm_count = sms;
    h->device = dev;
    h->tokens_per_block = router_tokens_per_block(c.n_experts);
    h->n_blocks_max = ceil_div(c.t_max, h->tokens_per_block);

    const int64_t E = c.n_experts, k = c.top_k, d = c.d_model, dff = c.d_ff, tm = c.t_max;
    // Rows the expert kernels may see on this rank: its own picks on one GPU,
    // or up to recv_rows_max rows arriving from all ranks; every local expert's
    // segment is rounded up to kRowAlign.
    int64_t rows_in = tm * k;
    if (c.world > 1) rows_in = c.recv_rows_max > 0 ? (int64_t)c.recv_rows_max : tm * k * c.world;
    h->rows_cap = ((rows_in + kRowAlign - 1) / kRowAlign + h->e_local) * (int64_t)kRowAlign;
    const size_t cs = elt_size(c.compute_dtype);

#define ALLOC(field, count)                                                          \
    do {                                                                             \
        cudaError_t _e = dev_alloc(&h->field, (size_t)(count));                      \
        if (_e != cudaSuccess) {                                                     \
            int rc = fail(nullptr, OMOE_ERR_NOMEM, "omoe_create: cudaMalloc(%s, %lld) failed: %s", #field, \
                          (long long)(count), cudaGetErrorString(_e));               \
            omoe_destroy(h);                                                         \
            return rc;                                                               \
        }                                                                            \
    } while (0)

    ALLOC(w_router, E * d);
    if (c.has_router_bias) ALLOC(router_bias, E);
    {
        struct { void **p; size_t bytes; } bufs[] = {
            {&h->w_gate, (size_t)h->e_local * dff * d * cs}, {&h->w_up, (size_t)h->e_local * dff * d * cs},
            {&h->w_down, (size_t)h->e_local * dff * d * cs}, {&h->xp, (size_t)h->rows_cap * d * cs},
            {&h->hbuf, (size_t)h->rows_cap * dff * cs},      {&h->yp, (size_t)h->rows_cap * d * cs},
            {&h->x_stage[0], (size_t)tm * d * 4},            {&h->y_stage[0], (size_t)tm * d * 4},
            {&h->x_stage[1], (size_t)tm * d * 4},            {&h->y_stage[1], (size_t)tm * d * 4},
            {&h->xn, (size_t)tm * d * cs}};
        h->stage_bytes = (size_t)tm * d * 4;
        for (auto &b : bufs) {
            cudaError_t e = cudaMalloc(b.p, b.bytes ? b.bytes : 1);
            if (e != cudaSuccess) {
                *b.p = nullptr;
                int rc = fail(nullptr, OMOE_ERR_NOMEM, "omoe_create: cudaMalloc of %zu bytes failed: %s", b.bytes,
                              cudaGetErrorString(e));
                omoe_destroy(h);
                return rc;
            }
        }
    }
    ALLOC(logits, tm * E);
    ALLOC(topk_idx, tm * k);
    ALLOC(topk_w, tm * k);
    ALLOC(block_counts, (int64_t)h->n_blocks_max * E);
    ALLOC(block_base, (int64_t)h->n_blocks_max * E);
    ALLOC(counts, E);
    ALLOC(offsets, E + 1);
    ALLOC(poffsets, E + 1);
    ALLOC(tile_expert, h->rows_cap / kRowAlign);
    ALLOC(pos, tm * k);
    ALLOC(lrank, tm * k);
    ALLOC(perm_out, tm * k);
    ALLOC(dev_err, 1);
    ALLOC(ticket, 1);
    ALLOC(ticket2, 1);
    ALLOC(ticket3, 1);
    ALLOC(d_row_table, c.world);
    ALLOC(d_out_table, c.world);
    if (c.world > 1) ALLOC(dst_base, E);
#undef ALLOC
    h->ex_counts = h->counts;
    h->ex_poffsets = h->poffsets;
    h->ex_tile_expert = h->tile_expert;
    if (c.world == 1) {
        h->dst_base = h->poffsets;
        cudaMemcpy(h->d_row_table, &h->xp, sizeof(void *), cudaMemcpyHostToDevice);
        cudaMemcpy(h->d_out_table, &h->yp, sizeof(void *), cudaMemcpyHostToDevice);
    } else {
        int rc = ep_create(h);
        if (rc != OMOE_OK) {
            fail(nullptr, rc, "omoe_create: %s", h->err);
            omoe_destroy(h);
            return rc;
        }
    }
    cudaMemset(h->dev_err, 0, sizeof(int32_t));
    cudaMemset(h->ticket, 0, sizeof(int32_t));
    cudaMemset(h->ticket2, 0, sizeof(int32_t));
    cudaMemset(h->ticket3, 0, sizeof(int32_t));
    // padding rows of the dispatch buffers are never read back, but start them
    // at zero so no stale NaN pattern ever enters a tensor-core tile
    cudaMemset(h->xp, 0, (size_t)h->rows_cap * d * cs);
    h->ev = h->ev_ring[0];
    for (int i = 0; i <= OMOE_N_STAGES; i++)
        if (cudaEventCreate(&h->ev[i]) != cudaSuccess) {
            int rc = fail(nullptr, OMOE_ERR_CUDA, "omoe_create: cudaEventCreate failed");
            omoe_destroy(h);
            return rc;
        }
    // copy streams of omoe_forward_host: non-blocking, so they can overlap kernels on the legacy default stream
    h->pdl = !(getenv("OMOE_PDL") && atoi(getenv("OMOE_PDL")) == 0);
    h->host_chunk_min = 4096;
    h->host_chunk_min_ep = 512;  // expert parallel: the per-rank batch is small, and so are its chunks
    if (const char *v = getenv("OMOE_HOST_CHUNK_MIN")) {
        h->host_chunk_min = atoi(v) > 0 ? atoi(v) : 1 << 30;
        h->host_chunk_min_ep = h->host_chunk_min;
    }
    bool ok_streams = cudaStreamCreateWithFlags(&h->copy_in, cudaStreamNonBlocking) == cudaSuccess &&
                      cudaStreamCreateWithFlags(&h->copy_out, cudaStreamNonBlocking) == cudaSuccess;
    for (int i = 0; ok_streams && i < kHostChunksMax; i++)
        ok_streams = cudaEventCreateWithFlags(&h->ev_in[i], cudaEventDisableTiming) == cudaSuccess &&
                     cudaEventCreateWithFlags(&h->ev_out[i], cudaEventDisableTiming) == cudaSuccess;
    for (int i = 0; ok_streams && i < 2; i++)
        ok_streams = cudaEventCreateWithFlags(&h->ev_set_fwd[i], cudaEventDisableTiming) == cudaSuccess &&
                     cudaEventCreateWithFlags(&h->ev_set_d2h[i], cudaEventDisableTiming) == cudaSuccess;
    if (!ok_streams) {
        int rc = fail(nullptr, OMOE_ERR_CUDA, "omoe_create: could not create the copy streams");
        omoe_destroy(h);
        return rc;
    }
    if (c.compute_dtype == OMOE_BF16 && !build_tensor_maps(h)) {
        int rc = fail(nullptr, OMOE_ERR_CUDA, "omoe_create: %s", h->err);
        omoe_destroy(h);
        return rc;
    }
    if (cudaDeviceSynchronize() != cudaSuccess) {
        int rc = fail(nullptr, OMOE_ERR_CUDA, "omoe_create: device synchronise failed");
        omoe_destroy(h);
        return rc;
    }
    h->err[0] = 0;
    *out = h;
    return OMOE_OK;
}

int omoe_set_weights(omoe_handle *h, const void *w_router, const void *router_bias, const void *w_gate,
                     const void *w_up, const void *w_down, int32_t src_dtype, void *cuda_stream) {
    if (!h) return OMOE_ERR_INVALID;
    if (!w_router || !w_gate || !w_up || !w_down) return fail(h, OMOE_ERR_INVALID, "omoe_set_weights: null weight pointer");
    if (src_dtype != OMOE_F32 && src_dtype != OMOE_BF16) return fail(h, OMOE_ERR_INVALID, "omoe_set_weights: bad src_dtype");
    if (h->cfg.has_router_bias && !router_bias)
        return fail(h, OMOE_ERR_INVALID, "omoe_set_weights: the layer was created with a router bias but none was given");
    cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
    const int64_t E = h->cfg.n_experts, d = h->cfg.d_model, dff = h->cfg.d_ff, El = h->e_local;
    const int64_t n_exp = El * dff * d;
    // router weights and bias are always held in fp32
    if (src_dtype == OMOE_BF16 && E > 16) {
        // bf16 values are exact in both copies; the router kernel stages the narrow one (half the L2 traffic)
        if (!h->w_router_bf16) CU_TRY(h, cudaMalloc(reinterpret_cast<void **>(&h->w_router_bf16), E * d * 2));
        CU_TRY(h, cudaMemcpyAsync(h->w_router_bf16, w_router, E * d * 2, cudaMemcpyDeviceToDevice, s));
    } else if (h->w_router_bf16) {
        CU_TRY(h, cudaStreamSynchronize(s));  // an earlier forward may still read it
        cudaFree(h->w_router_bf16);
        h->w_router_bf16 = nullptr;
    }
    if (src_dtype == OMOE_F32) {
        CU_TRY(h, cudaMemcpyAsync(h->w_router, w_router, E * d * 4, cudaMemcpyDeviceToDevice, s));
        if (h->cfg.has_router_bias)
            CU_TRY(h, cudaMemcpyAsync(h->router_bias, router_bias, E * 4, cudaMemcpyDeviceToDevice, s));
    } else {
        CU_TRY(h, launch_convert_bf16_to_f32(static_cast<const __nv_bfloat16 *>(w_router), h->w_router, E * d, s));
        if (h->cfg.has_router_bias)
            CU_TRY(h, launch_convert_bf16_to_f32(static_cast<const __nv_bfloat16 *>(router_bias), h->router_bias, E, s));
    }
    const void *src[3] = {w_gate, w_up, w_down};
    void *dst[3] = {h->w_gate, h->w_up, h->w_down};
    for (int i = 0; i < 3; i++) {
        if (h->cfg.compute_dtype == OMOE_BF16) {
            if (src_dtype == OMOE_BF16)
                CU_TRY(h, cudaMemcpyAsync(dst[i], src[i], n_exp * 2, cudaMemcpyDeviceToDevice, s));
            else
                CU_TRY(h, launch_convert_f32_to_bf16(static_cast<const float *>(src[i]),
                                                     static_cast<__nv_bfloat16 *>(dst[i]), n_exp, s));
        } else {
            if (src_dtype == OMOE_F32)
                CU_TRY(h, cudaMemcpyAsync(dst[i], src[i], n_exp * 4, cudaMemcpyDeviceToDevice, s));
            else
                CU_TRY(h, launch_convert_bf16_to_f32(static_cast<const __nv_bfloat16 *>(src[i]),
                                                     static_cast<float *>(dst[i]), n_exp, s));
        }
    }
    h->weights_set = true;
    bw_weights_changed(h);
    return OMOE_OK;
}

// The layer proper.  x (x_dtype) feeds router and dispatch; y and the optional
// residual rows have y_dtype.  pre != 0: kernels already launched for this
// forward (the block entry point's RMSNorm).
static int forward_impl(omoe_handle *h, const void *x_dev, int x_dtype, void *y_dev, int y_dtype, const void *resid,
                        int32_t T, cudaStream_t s, int pre) {
    NvtxRange range("omoe_forward");
    h->last_T = T;
    h->last_io_dtype = y_dtype;
    h->last_stream = s;
    h->last_launches = 0;
    h->ev_valid = false;
    if (h->profiling) h->ev = h->ev_ring[h->prof_count % kProfSlots];
    h->last_resid = resid != nullptr;
    bw_forward_invalidate(h);  // the rows a backward pass would read are about to be overwritten
    if (h->cfg.world > 1) {
        int rc = ep_forward(h, x_dev, x_dtype, y_dev, y_dtype, resid, T, s);
        h->last_launches += pre;
        if (rc == OMOE_OK && h->ev_valid) h->prof_count++;
        return rc;
    }
    if (T == 0) {
        bw_forward_empty(h);
        return OMOE_OK;
    }

    int n = pre;
    const bool prof = h->profiling;
#define MARK(i) do { if (prof) cudaEventRecord(h->ev[i], s); } while (0)
#ifdef OMOE_BOUNDS_CHECK
    CU_TRY(h, check_fill(h, s));  // self-checking build: a row the step never wrote reads as NaN
#endif
    MARK(0);
    if (h->cfg.compute_dtype == OMOE_BF16 && T <= route_small_max_tokens()) {
        CU_TRY(h, launch_route_small(h, x_dev, x_dtype, T, s, &n));
        MARK(1);
        MARK(2);
    } else {
        CU_TRY(h, launch_router(h, x_dev, x_dtype, T, s, &n));
        MARK(1);
        CU_TRY(h, launch_scan(h, T, s, &n));
        MARK(2);
        CU_TRY(h, launch_permute(h, x_dev, x_dtype, T, s, &n, nullptr));
    }
#ifdef OMOE_BOUNDS_CHECK
    CU_TRY(h, check_after_dispatch(h, T, s));  // routing indices in bounds, padding rows untouched
#endif
    MARK(3);
    MARK(4);
    if (bw_training(h)) {
        // training mode: the pre-activation rows are kept for the backward pass
        CU_TRY(h, bw_forward_experts(h, T, s, &n));
        MARK(5);
    } else if (h->cfg.compute_dtype == OMOE_BF16 && T <= decode_tokens_threshold()) {
        CU_TRY(h, launch_experts_decode(h, T, s, &n, prof ? h->ev[5] : nullptr));
    } else if (h->cfg.compute_dtype == OMOE_BF16) {
        CU_TRY(h, launch_experts_bf16(h, s, &n, prof ? h->ev[5] : nullptr, (long)T * h->cfg.top_k));
    } else {
        CU_TRY(h, launch_experts_f32(h, s, &n));
        MARK(5);
    }
    MARK(6);
    MARK(7);
    CU_TRY(h, launch_combine(h, y_dev, y_dtype, T, s, &n, nullptr, resid));
    MARK(8);
#undef MARK
    h->ev_valid = prof;
    if (prof) h->prof_count++;
    h->last_launches = n;
    return OMOE_OK;
}

static int check_forward_args(omoe_handle *h, const void *x_dev, void *y_dev, int32_t T, int32_t io_dtype,
                              const char *who) {
    if (!h->weights_set) return fail(h, OMOE_ERR_STATE, "%s: call omoe_set_weights first", who);
    if (T < 0) return fail(h, OMOE_ERR_INVALID, "%s: negative token count", who);
    if (T > h->cfg.t_max) return fail(h, OMOE_ERR_TOO_LARGE, "%s: T=%d exceeds t_max=%d", who, T, h->cfg.t_max);
    if (io_dtype != OMOE_F32 && io_dtype != OMOE_BF16) return fail(h, OMOE_ERR_INVALID, "%s: bad io_dtype", who);
    if (h->cfg.compute_dtype == OMOE_F32 && io_dtype != OMOE_F32)
        return fail(h, OMOE_ERR_UNSUPPORTED, "%s: an fp32 layer takes fp32 rows", who);
    if (T > 0 && (!x_dev || !y_dev)) return fail(h, OMOE_ERR_INVALID, "%s: null buffer", who);
    // rows move as 16-byte vectors; a misaligned address would raise a sticky device fault
    if (T > 0 && (misaligned16(x_dev) || misaligned16(y_dev)))
        return fail(h, OMOE_ERR_INVALID, "%s: device buffers must be 16-byte aligned", who);
    return OMOE_OK;
}

int omoe_forward(omoe_handle *h, const void *x_dev, void *y_dev, int32_t T, int32_t io_dtype, void *cuda_stream) {
    if (!h) return OMOE_ERR_INVALID;
    int rc = check_forward_args(h, x_dev, y_dev, T, io_dtype, "omoe_forward");
    if (rc != OMOE_OK) return rc;
    return forward_impl(h, x_dev, io_dtype, y_dev, io_dtype, nullptr, T, static_cast<cudaStream_t>(cuda_stream), 0);
}

int omoe_forward_block(omoe_handle *h, const void *x_dev, const float *gamma_dev, float eps, void *y_dev, int32_t T,
                       int32_t io_dtype, void *cuda_stream) {
    if (!h) return OMOE_ERR_INVALID;
    int rc = check_forward_args(h, x_dev, y_dev, T, io_dtype, "omoe_forward_block");
    if (rc != OMOE_OK) return rc;
    if (!gamma_dev) return fail(h, OMOE_ERR_INVALID, "omoe_forward_block: null gamma");
    if (misaligned16(gamma_dev)) return fail(h, OMOE_ERR_INVALID, "omoe_forward_block: gamma must be 16-byte aligned");
    cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
    int pre = 0;
    if (T > 0) CU_TRY(h, launch_rmsnorm(h, x_dev, io_dtype, gamma_dev, eps, T, s, &pre));
    return forward_impl(h, h->xn, h->cfg.compute_dtype, y_dev, io_dtype, x_dev, T, s, pre);
}

int omoe_set_training(omoe_handle *h, int32_t on) {
    if (!h) return OMOE_ERR_INVALID;
    return bw_set_training(h, on);
}

int omoe_backward(omoe_handle *h, const void *x_dev, const void *dy_dev, void *dx_dev, int32_t T, int32_t io_dtype,
                  void *cuda_stream) {
    if (!h) return OMOE_ERR_INVALID;
    int rc = check_forward_args(h, x_dev, dx_dev, T, io_dtype, "omoe_backward");
    if (rc != OMOE_OK) return rc;
    if (T > 0 && !dy_dev) return fail(h, OMOE_ERR_INVALID, "omoe_backward: null buffer");
    if (T > 0 && misaligned16(dy_dev)) return fail(h, OMOE_ERR_INVALID, "omoe_backward: device buffers must be 16-byte aligned");
    if (io_dtype != h->last_io_dtype && T > 0)
        return fail(h, OMOE_ERR_INVALID, "omoe_backward: io_dtype differs from the forward's");
    int n = 0;
    NvtxRange range("omoe_backward");
    if (h->last_resid)
        return fail(h, OMOE_ERR_STATE,
                    "omoe_backward: the last forward was omoe_forward_block; its backward is omoe_backward_block");
    rc = bw_backward(h, x_dev, false, dy_dev, dx_dev, T, io_dtype, static_cast<cudaStream_t>(cuda_stream), &n);
    h->last_launches = n;
    return rc;
}

int omoe_backward_block(omoe_handle *h, const void *x_dev, const float *gamma_dev, float eps, const void *dy_dev,
                        void *dx_dev, float *dgamma_dev, int32_t T, int32_t io_dtype, void *cuda_stream) {
    if (!h) return OMOE_ERR_INVALID;
    int rc = check_forward_args(h, x_dev, dx_dev, T, io_dtype, "omoe_backward_block");
    if (rc != OMOE_OK) return rc;
    if (!gamma_dev || !dgamma_dev || (T > 0 && !dy_dev)) return fail(h, OMOE_ERR_INVALID, "omoe_backward_block: null buffer");
    if (T > 0 && (misaligned16(dy_dev) || misaligned16(gamma_dev) || misaligned16(dgamma_dev)))
        return fail(h, OMOE_ERR_INVALID, "omoe_backward_block: device buffers must be 16-byte aligned");
    if (!h->last_resid)
        return fail(h, OMOE_ERR_STATE, "omoe_backward_block: the last forward was not omoe_forward_block");
    if (io_dtype != h->last_io_dtype && T > 0)
        return fail(h, OMOE_ERR_INVALID, "omoe_backward_block: io_dtype differs from the forward's");
    int n = 0;
    rc = bw_backward_block(h, x_dev, gamma_dev, eps, dy_dev, dx_dev, dgamma_dev, T, io_dtype,
                           static_cast<cudaStream_t>(cuda_stream), &n);
    h->last_launches = n;
    return rc;
}

int omoe_get_weight_grads(omoe_handle *h, float *d_router, float *d_router_bias, float *d_gate, float *d_up,
                          float *d_down, void *cuda_stream) {
    if (!h) return OMOE_ERR_INVALID;
    int rc = bw_get_grads(h, d_router, d_router_bias, d_gate, d_up, d_down, static_cast<cudaStream_t>(cuda_stream));
    if (rc != OMOE_OK) return rc;
    return check_dev_err(h);
}

int omoe_set_aux_loss(omoe_handle *h, float coef) {
    if (!h) return OMOE_ERR_INVALID;
    return bw_set_aux(h, coef);
}

int omoe_get_aux_loss(omoe_handle *h, float *loss_host) {
    if (!h || !loss_host) return OMOE_ERR_INVALID;
    return bw_aux_loss(h, loss_host, h->last_stream);
}

int omoe_ep_connect_local(omoe_handle **handles, int32_t world) {
    if (!handles || world < 2 || world > kMaxWorld) return OMOE_ERR_INVALID;
    for (int r = 0; r < world; r++)
        if (!handles[r]) return OMOE_ERR_INVALID;
    return ep_connect_local(handles, world);
}

// Enqueues one host-buffer forward: H2D copies, the forward(s), D2H copies.  No host synchronisation.
//
// Two staging sets alternate from call to call, so the copy-in of call n+1 and the copy-out of call n-1 run
// while the kernels of call n do: calls enqueued back to back (omoe_forward_host_async) cost the longer of
// their copies and their kernels.  A set is reused by the call two later, which waits (on the device) for the
// earlier call's forward to have consumed the staged rows and for its copy-out to have left the output rows.
//
// `chunked` (the synchronous entry point, where nothing else overlaps the call): tokens are independent, so a
// large batch is cut into chunks that run as separate forwards and the copy-in of chunk i+1 and the copy-out of
// chunk i-1 overlap the kernels of chunk i.  Every output row has the same bits as in one big forward.  With
// expert parallelism every forward is a collective step, so all ranks must cut their batches into the SAME
// number of chunks: the count follows from t_max (identical on every rank), and a rank with fewer tokens makes
// forwards of fewer (or zero) tokens.
static int forward_host_enqueue(omoe_handle *h, const void *x_host, void *y_host, int32_t T, int32_t io_dtype,
                                cudaStream_t s, bool chunked) {
    NvtxRange range("omoe_forward_host");
    const size_t row_bytes = (size_t)h->cfg.d_model * elt_size(io_dtype);
    int chunks = 1;
    if (chunked) {
        const int basis = h->cfg.world == 1 ? T : h->cfg.t_max;
        const int cmin = h->cfg.world == 1 ? h->host_chunk_min : h->host_chunk_min_ep;
        while (chunks < kHostChunksMax && basis / (chunks * 2) >= cmin) chunks *= 2;
    }
    const int per = (T + chunks - 1) / chunks;
    const int set = h->stage_next;
    h->stage_next ^= 1;
    char *xs = static_cast<char *>(h->x_stage[set]), *ys = static_cast<char *>(h->y_stage[set]);
    // The copy-in does NOT wait for work already queued on the caller's stream (that is what lets it run under
    // the previous call's kernels): x_host must hold the rows when the call is made.  The copy-out only ever
    // follows this call's own forward.
    // the call two before this one used the same staging set
    CU_TRY(h, cudaStreamWaitEvent(h->copy_in, h->ev_set_fwd[set], 0));
    CU_TRY(h, cudaStreamWaitEvent(s, h->ev_set_d2h[set], 0));
    for (int i = 0; i < chunks; i++) {
        const int t0 = i * per, n = t0 >= T ? 0 : ((t0 + per <= T) ? per : T - t0);
        const size_t off = (size_t)t0 * row_bytes;
        if (n > 0)
            CU_TRY(h, cudaMemcpyAsync(xs + off, static_cast<const char *>(x_host) + off, (size_t)n * row_bytes,
                                      cudaMemcpyHostToDevice, h->copy_in));
        CU_TRY(h, cudaEventRecord(h->ev_in[i], h->copy_in));
    }
    for (int i = 0; i < chunks; i++) {
        const int t0 = i * per, n = t0 >= T ? 0 : ((t0 + per <= T) ? per : T - t0);
        const size_t off = (size_t)(n > 0 ? t0 : 0) * row_bytes;
        CU_TRY(h, cudaStreamWaitEvent(s, h->ev_in[i], 0));
        if (n > 0 || h->cfg.world > 1) {
            int rc = omoe_forward(h, xs + off, ys + off, n, io_dtype, s);
            if (rc != OMOE_OK) return rc;
        }
        CU_TRY(h, cudaEventRecord(h->ev_out[i], s));
        CU_TRY(h, cudaStreamWaitEvent(h->copy_out, h->ev_out[i], 0));
        if (n > 0)
            CU_TRY(h, cudaMemcpyAsync(static_cast<char *>(y_host) + off, ys + off, (size_t)n * row_bytes,
                                      cudaMemcpyDeviceToHost, h->copy_out));
    }
    CU_TRY(h, cudaEventRecord(h->ev_set_fwd[set], s));
    CU_TRY(h, cudaEventRecord(h->ev_set_d2h[set], h->copy_out));
    h->last_stream = s;
    h->host_pending = true;
    return OMOE_OK;
}

static int check_host_args(omoe_handle *h, const void *x_host, void *y_host, int32_t T, int32_t io_dtype,
                           const char *who) {
    if (T < 0 || T > h->cfg.t_max)
        return fail(h, T < 0 ? OMOE_ERR_INVALID : OMOE_ERR_TOO_LARGE, "%s: T=%d outside [0, %d]", who, T, h->cfg.t_max);
    if (io_dtype != OMOE_F32 && io_dtype != OMOE_BF16) return fail(h, OMOE_ERR_INVALID, "%s: bad io_dtype", who);
    if (T > 0 && (!x_host || !y_host)) return fail(h, OMOE_ERR_INVALID, "%s: null buffer", who);
    if ((size_t)h->cfg.d_model * elt_size(io_dtype) % 16 != 0)
        return fail(h, OMOE_ERR_UNSUPPORTED, "%s: a row must be a multiple of 16 bytes", who);
    return OMOE_OK;
}

int omoe_forward_host_async(omoe_handle *h, const void *x_host, void *y_host, int32_t T, int32_t io_dtype,
                            void *cuda_stream) {
    if (!h) return OMOE_ERR_INVALID;
    int rc = check_host_args(h, x_host, y_host, T, io_dtype, "omoe_forward_host_async");
    if (rc != OMOE_OK) return rc;
    return forward_host_enqueue(h, x_host, y_host, T, io_dtype, static_cast<cudaStream_t>(cuda_stream), false);
}

int omoe_wait(omoe_handle *h) {
    if (!h) return OMOE_ERR_INVALID;
    if (h->host_pending) {
        CU_TRY(h, cudaStreamSynchronize(h->copy_out));
        h->host_pending = false;
    }
    CU_TRY(h, cudaStreamSynchronize(h->last_stream));
    return check_dev_err(h);
}

int omoe_forward_host(omoe_handle *h, const void *x_host, void *y_host, int32_t T, int32_t io_dtype,
                      void *cuda_stream) {
    if (!h) return OMOE_ERR_INVALID;
    int rc = check_host_args(h, x_host, y_host, T, io_dtype, "omoe_forward_host");
    if (rc != OMOE_OK) return rc;
    rc = forward_host_enqueue(h, x_host, y_host, T, io_dtype, static_cast<cudaStream_t>(cuda_stream), true);
    if (rc != OMOE_OK) return rc;
    return omoe_wait(h);
}

int omoe_get_routing(omoe_handle *h, int32_t *topk_idx, float *topk_w, int32_t *counts, int32_t *offsets,
                     int32_t *perm) {
    if (!h) return OMOE_ERR_INVALID;
    const int T = h->last_T, k = h->cfg.top_k, E = h->cfg.n_experts;
    cudaStream_t s = h->last_stream;
    if (perm && T > 0) CU_TRY(h, launch_perm_readout(h, T, s));
    CU_TRY(h, cudaStreamSynchronize(s));
    int rc = check_dev_err(h);
    if (rc != OMOE_OK) return rc;
    const size_t n = (size_t)T * k;
    if (topk_idx && n) CU_TRY(h, cudaMemcpy(topk_idx, h->topk_idx, n * 4, cudaMemcpyDeviceToHost));
    if (topk_w && n) CU_TRY(h, cudaMemcpy(topk_w, h->topk_w, n * 4, cudaMemcpyDeviceToHost));
    if (T == 0) {
        if (counts) memset(counts, 0, sizeof(int32_t) * E);
        if (offsets) memset(offsets, 0, sizeof(int32_t) * (E + 1));
        return OMOE_OK;
    }
    if (counts) CU_TRY(h, cudaMemcpy(counts, h->counts, sizeof(int32_t) * E, cudaMemcpyDeviceToHost));
    if (offsets) CU_TRY(h, cudaMemcpy(offsets, h->offsets, sizeof(int32_t) * (E + 1), cudaMemcpyDeviceToHost));
    if (perm && n) CU_TRY(h, cudaMemcpy(perm, h->perm_out, n * 4, cudaMemcpyDeviceToHost));
    return OMOE_OK;
}

int omoe_get_logits(omoe_handle *h, float *logits) {
    if (!h || !logits) return OMOE_ERR_INVALID;
    CU_TRY(h, cudaStreamSynchronize(h->last_stream));
    const size_t n = (size_t)h->last_T * h->cfg.n_experts;
    if (n) CU_TRY(h, cudaMemcpy(logits, h->logits, n * 4, cudaMemcpyDeviceToHost));
    return OMOE_OK;
}

int omoe_last_launch_count(const omoe_handle *h) { return h ? h->last_launches : 0; }

int omoe_set_profiling(omoe_handle *h, int32_t enabled) {
    if (!h) return OMOE_ERR_INVALID;
    if (enabled) {
        for (int r = 0; r < kProfSlots; r++)
            for (int i = 0; i <= OMOE_N_STAGES; i++)
                if (!h->ev_ring[r][i]) CU_TRY(h, cudaEventCreate(&h->ev_ring[r][i]));
    }
    h->profiling = enabled != 0;
    h->prof_count = 0;
    h->ev = h->ev_ring[0];
    h->ev_valid = false;
    return OMOE_OK;
}

int omoe_get_stage_ms_at(omoe_handle *h, int32_t back, float *ms) {
    if (!h || !ms) return OMOE_ERR_INVALID;
    if (!h->ev_valid) return fail(h, OMOE_ERR_STATE, "omoe_get_stage_ms: profiling was off for the last forward");
    if (back < 0 || back >= kProfSlots || back >= h->prof_count)
        return fail(h, OMOE_ERR_INVALID, "omoe_get_stage_ms_at: only the last %d profiled forwards are kept (%ld so far)",
                    kProfSlots, h->prof_count);
    cudaEvent_t *ev = h->ev_ring[(h->prof_count - 1 - back) % kProfSlots];
    CU_TRY(h, cudaEventSynchronize(h->ev_ring[(h->prof_count - 1) % kProfSlots][OMOE_N_STAGES]));
    for (int i = 0; i < OMOE_N_STAGES; i++) CU_TRY(h, cudaEventElapsedTime(&ms[i], ev[i], ev[i + 1]));
    return back == 0 ? check_dev_err(h) : OMOE_OK;
}

int omoe_get_stage_ms(omoe_handle *h, float *ms) { return omoe_get_stage_ms_at(h, 0, ms); }

int omoe_ep_export(omoe_handle *h, void *blob) {
    if (!h || !blob) return OMOE_ERR_INVALID;
    return ep_export(h, blob);
}

int omoe_ep_import(omoe_handle *h, const void *all_blobs) {
    if (!h || !all_blobs) return OMOE_ERR_INVALID;
    return ep_import(h, all_blobs);
}

}  // extern "C"
