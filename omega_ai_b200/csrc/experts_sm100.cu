// Grouped expert products on Blackwell tensor cores (compute_dtype = OMOE_BF16).
//
// Replaces, per expert, the three cublasSgemm calls plus the silu_forward and
// mul_kernel passes of LlamaMLPLayer.output()
// (src/main/java/com/omega/engine/nn/layer/llama/LlamaMLPLayer.java:117-123;
// FullyLayer.java:235; src/main/resources/cu/activeFunction.cu:172-180;
// src/main/resources/cu/OPKernel.cu:1040) with two persistent kernels:
//   up/gate:  h  = silu(xp * Wg^T) * (xp * Wu^T)      (SiLU and product in the epilogue)
//   down:     yp = h * Wd^T
// Both are the same mainloop: one CTA per SM walks a list of 128 x 256 output
// tiles; a producer thread feeds a 4-stage shared-memory ring with TMA
// (128-byte swizzle), one thread issues tcgen05.mma (M=128, N=256, K=16, bf16
// in, fp32 accumulate in tensor memory), and eight epilogue warps read the
// accumulator with tcgen05.ld while the next tile's mainloop already runs in
// the other half of tensor memory.
//
// Every wait on an mbarrier is bounded: when it runs out the kernel raises a
// flag in the device error word, lets outstanding copies land, frees its tensor
// memory and returns, so the context stays usable.
#include <stdlib.h>

#include "backward.cuh"
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace omoe {

namespace {

using namespace sm100;
constexpr int kStages = 4;
constexpr int kAccStages = 2;
constexpr int kTmemCols = 512;
constexpr int kABytes = BLOCK_M * BLOCK_K * 2;      // 16 KB
constexpr int kBHalfBytes = 128 * BLOCK_K * 2;      // 16 KB (one 128-row TMA box)
constexpr int kStageBytes = kABytes + 2 * kBHalfBytes;  // 48 KB
constexpr int kOutSubBytes = 128 * 64 * 2;          // one [128 x 64] bf16 sub-tile of the output staging
constexpr int kOutBytes = 2 * kOutSubBytes;         // 32 KB: 128 output columns per pass
constexpr int kSmemBytes = kStages * kStageBytes + kOutBytes + 1024 /*align slack*/ + 256 /*barriers*/;
constexpr int kThreads = 384;  // warp 0 producer, warp 1 MMA, warps 2-9 epilogue, warps 10-11 dispatch (expert parallel)
constexpr int kDispatchWarps = 2;


struct TileCoord {
    int mt, nt;
};

// Tiles are walked in bands of `band` m-tiles x all n-tiles, m fastest, so the
// rows of a band stay in L2 while the weight tiles stream past them.
// order (may be null): the m-tiles are walked in this order instead of as they lie in the buffer.
__device__ __forceinline__ TileCoord tile_coord(int tile, int num_m_tiles, int n_tiles, int kband,
                                                const int32_t *__restrict__ order) {
    int per_band = kband * n_tiles;
    int band = tile / per_band, r = tile % per_band;
    int m0 = band * kband;
    int bm = min(kband, num_m_tiles - m0);
    TileCoord c;
    c.mt = m0 + r % bm;
    if (order != nullptr) c.mt = order[c.mt];
    c.nt = r / bm;
    return c;
}

// SWIGLU = true : B0 = W_gate, B1 = W_up, tile nt covers output columns [128 nt, 128 nt + 128)
// SWIGLU = false: B0 = B1 = W_down,     tile nt covers output columns [256 nt, 256 nt + 256)
// n_out: output features per expert (d_ff or d_model); K: reduction length.
template <bool SWIGLU>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b0,
                    const __grid_constant__ CUtensorMap map_b1, const __grid_constant__ CUtensorMap map_out, int n_out,
                    int K, const int32_t *__restrict__ tile_expert, const int32_t *__restrict__ poffsets,
                    int E, int kband, int32_t *dev_err, const EpGate gate) {
    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;  // stages need 1024-byte alignment for the swizzle
    unsigned char *base_ptr = smem_raw + (base - raw);
    uint64_t *bars = reinterpret_cast<uint64_t *>(base_ptr + kStages * kStageBytes + kOutBytes);
    const uint32_t bar0 = base + kStages * kStageBytes + kOutBytes;
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (kStages + s); };
    auto tfull_bar = [&](int s) { return bar0 + 8u * (2 * kStages + s); };
    auto tempty_bar = [&](int s) { return bar0 + 8u * (2 * kStages + kAccStages + s); };
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * kStages + 2 * kAccStages);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    pdl_trigger();
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; s++) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int s = 0; s < kAccStages; s++) {
            mbar_init(tfull_bar(s), 1);
            mbar_init(tempty_bar(s), 8);  // one arrival per epilogue warp
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // barriers and tensor memory are set up; everything from here on reads what earlier kernels wrote
    pdl_wait();
    const int num_m_tiles = poffsets[E] / kRowAlign;
    const int n_tile_w = SWIGLU ? 128 : 256;
    const int n_tiles = (n_out + n_tile_w - 1) / n_tile_w;
    const int total = num_m_tiles * n_tiles;
    const int num_kb = (K + BLOCK_K - 1) / BLOCK_K;

    if (warp == 0) {
        // ---------------- producer: TMA loads into the ring ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            // the expert of the next tile is fetched while the current tile streams
            int e_next = (int)blockIdx.x < total ? tile_expert[tile_coord(blockIdx.x, num_m_tiles, n_tiles, kband, gate.tile_order).mt] : 0;
            uint32_t seen = 0;  // expert parallel: sources whose rows are known to have landed
            for (int tile = blockIdx.x; ok && tile < total; tile += gridDim.x) {
                TileCoord tc = tile_coord(tile, num_m_tiles, n_tiles, kband, gate.tile_order);
                const int e = e_next;
                if (gate.wait_flags != nullptr) {
                    // the rows of this tile come from the ranks named in its mask; wait for those only
                    const uint32_t need = gate.tile_src_mask ? gate.tile_src_mask[tc.mt] : ((1u << gate.world) - 1u);
                    if (!ep_gate_wait(gate, need, seen, dev_err)) { *abort_flag = 1; ok = false; break; }
                }
                if (tile + (int)gridDim.x < total)
                    e_next = tile_expert[tile_coord(tile + gridDim.x, num_m_tiles, n_tiles, kband, gate.tile_order).mt];
                const int row_a = tc.mt * BLOCK_M;
                const int row_b0 = e * n_out + tc.nt * n_tile_w;
                const int row_b1 = SWIGLU ? row_b0 : row_b0 + 128;
                for (int kb = 0; kb < num_kb; kb++) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, dev_err)) { ok = false; break; }
                    const uint32_t sa = base + stage * kStageBytes;
                    mbar_expect_tx(full_bar(stage), kStageBytes);
                    tma_load_2d(sa, &map_a, full_bar(stage), kb * BLOCK_K, row_a);
                    tma_load_2d(sa + kABytes, &map_b0, full_bar(stage), kb * BLOCK_K, row_b0);
                    tma_load_2d(sa + kABytes + kBHalfBytes, &map_b1, full_bar(stage), kb * BLOCK_K, row_b1);
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
            }
            // Expert parallel: the product that follows overwrites the output rows of the previous step, which a
            // rank may still be gathering until it has sent this step's rows -- so this kernel does not end
            // before EVERY rank has raised its flag, also those that sent this GPU nothing.
            if (ok && gate.wait_flags != nullptr) ep_gate_wait(gate, (1u << gate.world) - 1u, seen, dev_err);
            if (!ok) {
                // let copies that were already issued land before the CTA retires
                unsigned long long t0 = globaltimer_ns();
                while (globaltimer_ns() - t0 < 2000000ull) { }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            int stage = 0, as = 0;
            uint32_t phase = 0, aphase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < total; tile += gridDim.x) {
                if (!mbar_wait(tempty_bar(as), aphase ^ 1u, abort_flag, dev_err)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + as * BLOCK_N;
                for (int kb = 0; kb < num_kb; kb++) {
                    if (!mbar_wait(full_bar(stage), phase, abort_flag, dev_err)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = base + stage * kStageBytes;
                    const uint64_t adesc = make_sw128_desc(sa);
                    const uint64_t bdesc = make_sw128_desc(sa + kABytes);
#pragma unroll
                    for (int k = 0; k < BLOCK_K / UMMA_K; k++) {
                        // advance 32 bytes (16 bf16) inside the swizzled row: +2 in 16-byte units
                        tc_mma_bf16(d_tmem, adesc + 2u * k, bdesc + 2u * k, kIdesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    tc_commit(empty_bar(stage));  // frees the stage once these MMAs have read it
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                tc_commit(tfull_bar(as));  // accumulator complete
                if (++as == kAccStages) { as = 0; aphase ^= 1u; }
            }
        }
    } else if (warp >= 10) {
        // ---------------- dispatch warps (expert parallel, up/gate product only) ----------------
        // The rows this rank's tokens send to experts on OTHER ranks cross NVLink here, while the warps above
        // already multiply the tiles whose rows are in place (this rank's own rows went first, in a kernel of
        // their own).  One warp per token; nothing in here waits for anything.
        if constexpr (SWIGLU) {
            const EpDispatch &dp = gate.disp;
            if (dp.x != nullptr) {
                const int n_warps = (int)gridDim.x * kDispatchWarps;
                for (int t = (int)blockIdx.x * kDispatchWarps + (warp - 10); t < dp.T; t += n_warps) {
                    int my = -1, owner = 0;
                    if (lane < dp.k) {
                        const int f = t * dp.k + lane;
                        const int e = dp.topk_idx[f];
                        const int b = t / dp.tokens_per_block;
                        my = dp.dst_base[e] + dp.block_base[(size_t)e * dp.n_blocks + b] + dp.lrank[f];
                        owner = e / dp.e_local;
                        if (my < 0 || my >= dp.rows_cap || owner == gate.rank) my = -1;  // refused step / local pick
                    }
                    __nv_bfloat16 *dst[kMaxTopK];
                    bool any = false;
#pragma unroll
                    for (int j = 0; j < kMaxTopK; j++) {
                        const int row = __shfl_sync(0xffffffffu, my, j);
                        const int q = __shfl_sync(0xffffffffu, owner, j);
                        dst[j] = (j < dp.k && row >= 0)
                                     ? static_cast<__nv_bfloat16 *>(dp.row_table[q]) + (size_t)row * dp.d
                                     : nullptr;
                        any = any || dst[j] != nullptr;
                    }
                    if (!any) continue;
                    // four 16-byte loads in flight per lane before the first store: the warp is alone with the
                    // memory latency here
                    for (int c0 = lane * 8; c0 < dp.d; c0 += 4 * 256) {
                        uint4 v[4];
#pragma unroll
                        for (int u = 0; u < 4; u++) {
                            const int c = c0 + u * 256;
                            if (c >= dp.d) break;
                            if (dp.x_is_f32) {
                                float r[8];
                                ldg8(static_cast<const float *>(dp.x) + (size_t)t * dp.d + c, r);
                                v[u] = pack8(r);
                            } else {
                                v[u] = __ldg(reinterpret_cast<const uint4 *>(static_cast<const __nv_bfloat16 *>(dp.x) +
                                                                             (size_t)t * dp.d + c));
                            }
                        }
#pragma unroll
                        for (int u = 0; u < 4; u++) {
                            const int c = c0 + u * 256;
                            if (c >= dp.d) break;
#pragma unroll
                            for (int j = 0; j < kMaxTopK; j++)
                                if (dst[j] != nullptr) *reinterpret_cast<uint4 *>(dst[j] + c) = v[u];
                        }
                    }
                }
                // rows before flag, system-wide; the warp that finishes last tells the other ranks
                __threadfence_system();
                __syncwarp();
                int last = 0;
                if (lane == 0) last = atomicAdd(dp.ticket, 1) == (int)gridDim.x * kDispatchWarps - 1;
                last = __shfl_sync(0xffffffffu, last, 0);
                if (last) {
                    __threadfence_system();
                    const uint32_t seq = *gate.seq;
                    if (lane < gate.world && lane != gate.rank)
                        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(dp.rows_flags[lane] + gate.rank), "r"(seq)
                                     : "memory");
                    if (lane == 0) *dp.ticket = 0;
                }
            }
        }
    } else {
        // ---------------- epilogue: TMEM -> registers -> shared -> TMA store ----------------
        // Eight warps: warp%4 selects the 32 TMEM lanes (rows) the hardware lets it
        // read, (warp-2)/4 the 64-column half of a 128-column pass.  Each pass is
        // staged in shared memory as two [128 rows x 64 cols] sub-tiles in the
        // 128-byte-swizzled layout the output tensor map expects.
        const int ew = warp - 2;
        const int quarter = warp & 3;
        const int half = ew >> 2;
        const int r = quarter * 32 + lane;
        const uint32_t out_stage = base + kStages * kStageBytes;
        const uint32_t my_row = out_stage + half * kOutSubBytes + r * 128;
        constexpr int kPasses = SWIGLU ? 1 : 2;
        int as = 0;
        uint32_t aphase = 0;
        for (int tile = blockIdx.x; tile < total; tile += gridDim.x) {
            TileCoord tc = tile_coord(tile, num_m_tiles, n_tiles, kband, gate.tile_order);
            bool ok = mbar_wait(tfull_bar(as), aphase, abort_flag, dev_err);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const uint32_t t_acc = tmem_base + as * BLOCK_N + ((uint32_t)(quarter * 32) << 16);
#pragma unroll
            for (int p = 0; p < kPasses; p++) {
#pragma unroll
                for (int c = 0; c < 2; c++) {
                    const int col = p * 128 + half * 64 + c * 32;  // accumulator column of this chunk
                    uint32_t o[16];
                    if constexpr (SWIGLU) {
                        uint32_t g[32], u[32];
                        tc_ld32(t_acc + col, g);
                        tc_ld32(t_acc + 128 + col, u);
                        tc_wait_ld();
                        if (c == 1) {  // all of this warp's accumulator reads are done
                            tc_fence_before();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(tempty_bar(as));
                        }
#pragma unroll
                        for (int i = 0; i < 16; i++) {
                            float g0 = __uint_as_float(g[2 * i]), g1 = __uint_as_float(g[2 * i + 1]);
                            float u0 = __uint_as_float(u[2 * i]), u1 = __uint_as_float(u[2 * i + 1]);
                            o[i] = pack_bf16(silu_f(g0) * u0, silu_f(g1) * u1);
                        }
                    } else {
                        uint32_t a[32];
                        tc_ld32(t_acc + col, a);
                        tc_wait_ld();
                        if (p == kPasses - 1 && c == 1) {
                            tc_fence_before();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(tempty_bar(as));
                        }
#pragma unroll
                        for (int i = 0; i < 16; i++)
                            o[i] = pack_bf16(__uint_as_float(a[2 * i]), __uint_as_float(a[2 * i + 1]));
                    }
                    if (c == 0) {
                        // the previous pass's TMA store must have finished reading the staging tile
                        if (warp == 2 && lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                        asm volatile("bar.sync 1, 256;" ::: "memory");
                    }
#pragma unroll
                    for (int v = 0; v < 4; v++) {
                        const int chunk = (c * 4 + v) ^ (r & 7);  // 128-byte swizzle: 16-byte chunk ^ (row % 8)
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(my_row + chunk * 16),
                                     "r"(o[4 * v]), "r"(o[4 * v + 1]), "r"(o[4 * v + 2]), "r"(o[4 * v + 3])
                                     : "memory");
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                asm volatile("bar.sync 1, 256;" ::: "memory");
                if (warp == 2 && lane == 0) {
                    const int x0 = tc.nt * (SWIGLU ? 128 : 256) + p * 128;
                    const int y0 = tc.mt * BLOCK_M;
                    if (x0 < n_out) tma_store_2d(&map_out, out_stage, x0, y0);
                    if (x0 + 64 < n_out) tma_store_2d(&map_out, out_stage + kOutSubBytes, x0 + 64, y0);
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                }
            }
            if (++as == kAccStages) { as = 0; aphase ^= 1u; }
        }
        if (warp == 2) {
            if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
            __syncwarp();
            // expert parallel: this CTA's output rows are complete; the last CTA tells every rank
            if (gate.signal_flags != nullptr) ep_gate_signal(gate, (int)gridDim.x);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn) return fn;
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
        return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(p);
    return fn;
}

// 2-D bf16 tensor [rows, cols] row-major, box 128 rows x 64 columns, 128-byte swizzle.
bool encode_map(EncodeTiledFn fn, CUtensorMap *m, void *ptr, uint64_t rows, uint64_t cols, uint32_t box_rows = 128) {
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols * 2};
    cuuint32_t box[2] = {BLOCK_K, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, ptr, dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

}  // namespace


bool build_tensor_maps(omoe_handle *h) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) {
        snprintf(h->err, sizeof(h->err), "cuTensorMapEncodeTiled is not available from this driver");
        return false;
    }
    const uint64_t d = h->cfg.d_model, dff = h->cfg.d_ff, El = h->e_local, rows = h->rows_cap;
    bool ok = encode_map(fn, &h->maps.a_x, h->xp, rows, d) && encode_map(fn, &h->maps.a_h, h->hbuf, rows, dff) &&
              encode_map(fn, &h->maps.b_gate, h->w_gate, El * dff, d) &&
              encode_map(fn, &h->maps.b_up, h->w_up, El * dff, d) &&
              encode_map(fn, &h->maps.b_down, h->w_down, El * d, dff) && encode_map(fn, &h->maps.c_y, h->yp, rows, d) &&
              encode_map(fn, &h->maps.a_x32, h->xp, rows, d, 32) && encode_map(fn, &h->maps.a_h32, h->hbuf, rows, dff, 32);
    if (!ok) snprintf(h->err, sizeof(h->err), "cuTensorMapEncodeTiled failed (d=%d, d_ff=%d)", (int)d, (int)dff);
    h->maps_ready = ok;
    return ok;
}

namespace {
cudaError_t set_smem_attrs() {
    static PerDeviceOnce once;
    bool *done = once.slot();
    if (done && *done) return cudaSuccess;
    cudaError_t e = cudaFuncSetAttribute(grouped_gemm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kSmemBytes);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(grouped_gemm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return e;
    if (done) *done = true;
    return cudaSuccess;
}
}  // namespace

bool encode_map_bf16(CUtensorMap *m, void *ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {ld * 2};
    cuuint32_t box[2] = {BLOCK_K, box_rows};
    cuuint32_t estr[2] = {1, 1};
    return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

cudaError_t launch_grouped_plain(omoe_handle *h, cudaStream_t s, const CUtensorMap &a, const CUtensorMap &b,
                                 const CUtensorMap &c, int n_out, int K) {
    cudaError_t e = set_smem_attrs();
    if (e != cudaSuccess) return e;
    static int band = getenv("OMOE_BAND_DOWN") ? atoi(getenv("OMOE_BAND_DOWN")) : 16;
    return launch_ex(grouped_gemm_kernel<false>, dim3(h->sm_count), dim3(kThreads), kSmemBytes, s, false, a, b, b, c,
                     n_out, K, h->ex_tile_expert, h->ex_poffsets, h->e_local, band, h->dev_err, EpGate{});
}

// most 128-row tiles any placement of rows_ub rows on the local experts can give (-1: unknown)
static long m_tiles_bound(omoe_handle *h, long rows_ub) {
    if (rows_ub < 0) return -1;
    const long act = rows_ub < h->e_local ? rows_ub : h->e_local;
    return act + (rows_ub - act) / kRowAlign;
}

bool experts_up_is_persistent(omoe_handle *h, long rows_ub) {
    return splitk_ways_up_gate(h, m_tiles_bound(h, rows_ub)) == 0;
}

cudaError_t launch_experts_bf16(omoe_handle *h, cudaStream_t s, int *n, cudaEvent_t mid, long rows_ub,
                                const EpGate *gate) {
    // the up/gate product takes the wait side of the gate, the down product the signal side
    EpGate g_up{}, g_dn{};
    if (gate != nullptr) {
        g_up = *gate;
        g_up.signal_flags = nullptr;
        g_dn = *gate;
        g_dn.wait_flags = nullptr;
        g_dn.tile_src_mask = nullptr;
        g_dn.tile_order = nullptr;
        g_dn.disp = EpDispatch{};
    }
    {
        cudaError_t e0 = set_smem_attrs();
        if (e0 != cudaSuccess) return e0;
    }
    const int d = h->cfg.d_model, dff = h->cfg.d_ff;
    static int band_up = getenv("OMOE_BAND_UP") ? atoi(getenv("OMOE_BAND_UP")) : 16;
    static int band_dn = getenv("OMOE_BAND_DOWN") ? atoi(getenv("OMOE_BAND_DOWN")) : 16;
    dim3 grid(h->sm_count), block(kThreads);
    // With very few row tiles, whole tiles per CTA would leave most SMs (and their share of the memory
    // system) idle: split K over a cluster instead (experts_sm100_splitk.cu).
    const long m_tiles_ub = m_tiles_bound(h, rows_ub);
    const int s_up = splitk_ways_up_gate(h, m_tiles_ub), s_dn = splitk_ways_down(h, m_tiles_ub);
    cudaError_t e;
    if (s_up > 0) {
        e = launch_up_gate_splitk(h, s, s_up, gate ? &g_up : nullptr);
    } else {
        e = launch_ex(grouped_gemm_kernel<true>, grid, block, kSmemBytes, s, h->pdl, h->maps.a_x, h->maps.b_gate,
                      h->maps.b_up, h->maps.a_h, dff, d, h->ex_tile_expert, h->ex_poffsets, h->e_local, band_up,
                      h->dev_err, g_up);
    }
    if (e != cudaSuccess) return e;
    (*n)++;
    if (mid) cudaEventRecord(mid, s);
    if (s_dn > 0) {
        e = launch_down_splitk(h, s, s_dn, gate ? &g_dn : nullptr);
        if (e == cudaSuccess) (*n)++;
        return e;
    }
    e = launch_ex(grouped_gemm_kernel<false>, grid, block, kSmemBytes, s, h->pdl, h->maps.a_h, h->maps.b_down,
                  h->maps.b_down, h->maps.c_y, d, dff, h->ex_tile_expert, h->ex_poffsets, h->e_local, band_dn,
                  h->dev_err, g_dn);
    if (e == cudaSuccess) (*n)++;
    return e;
}

}  // namespace omoe
