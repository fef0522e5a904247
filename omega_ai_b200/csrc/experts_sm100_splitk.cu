// Grouped expert products for steps with very few row tiles (compute_dtype = OMOE_BF16): the reduction
// length is split over the CTAs of a thread-block cluster.
//
// Same products as experts_sm100.cu (LlamaMLPLayer.java:117-123: linear1/linear3, SiLU, product, linear2)
// and the same tile (128 rows x 256 accumulator columns, tcgen05.mma, fp32 accumulators in tensor memory).
// When a step leaves a GPU one or two row tiles (decode with the experts spread over many GPUs), whole
// tiles per CTA would put 16 or so CTAs to work and the weights, which are all of the traffic, would be
// fetched by a tenth of the machine.  Here a cluster of S CTAs shares one tile: CTA c multiplies the
// c-th slice of K, leaves its fp32 partial tile in its own shared memory (the TMA ring, idle by then),
// and after a cluster barrier reduces the c-th slice of the tile's columns over all S partials, read
// through distributed shared memory in rank order, so the sum has one fixed order.  Only rows that hold
// a token are reduced and written.
//
// Every mbarrier wait is bounded (sm100_ptx.cuh).  The cluster barriers are hardware barriers without a
// bound, so a CTA that gave up keeps walking its tiles, doing nothing, and still arrives at each of them.
#include <stdlib.h>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace omoe {

namespace {

using namespace sm100;
// Two shapes of the ring.  A step in which no expert holds more than 32 tokens (the case this kernel is for)
// fetches 32 rows of A per stage and fits six stages; the copies in flight are what hides the memory latency
// when only a fraction of the SMs pulls on HBM.  Otherwise four stages with all 128 rows, as in experts_sm100.cu.
constexpr int kBHalfBytesK = 128 * BLOCK_K * 2;            // 16 KB (one 128-row TMA box)
constexpr int kABytesBig = BLOCK_M * BLOCK_K * 2;          // 16 KB
constexpr int kABytesSmall = 32 * BLOCK_K * 2;             // 4 KB
constexpr int kStagesBig = 4, kStagesSmall = 6, kStagesMax = 6;
constexpr int kStageBytesBig = kABytesBig + 2 * kBHalfBytesK;      // 48 KB
constexpr int kStageBytesSmall = kABytesSmall + 2 * kBHalfBytesK;  // 36 KB
constexpr int kRingBytes = kStagesSmall * kStageBytesSmall;        // 216 KB
static_assert(kRingBytes >= kStagesBig * kStageBytesBig, "both shapes fit the ring");
constexpr int kPartialBytes = BLOCK_N * BLOCK_M * 4;       // 128 KB, laid over the ring
static_assert(kPartialBytes <= kRingBytes, "the partial tile reuses the ring");
constexpr int kSmemBytesK = kRingBytes + 1024 /*align slack*/ + 256 /*barriers*/;
static_assert(kSmemBytesK <= 227 * 1024, "shared memory of one CTA");
constexpr int kThreadsK = 320;  // warp 0 producer, warp 1 MMA, warps 2-9 epilogue and reduction
constexpr int kTmemColsK = 256;

__device__ __forceinline__ uint32_t sreg_cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t sreg_cluster_nctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t sreg_clusterid() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t sreg_nclusterid() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%nclusterid.x;" : "=r"(r));
    return r;
}
// every thread of every CTA of the cluster, with all lanes of its warp converged
__device__ __forceinline__ void cluster_barrier() {
    __syncwarp();
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float ld_peer_f32(uint32_t local_addr, uint32_t rank) {
    uint32_t a;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(local_addr), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(a) : "memory");
    return v;
}

// SWIGLU = true : B0 = W_gate, B1 = W_up; tile nt gives output columns [128 nt, 128 nt + 128) of h
// SWIGLU = false: B0 = B1 = W_down;      tile nt gives output columns [256 nt, 256 nt + 256) of yp
// out: [rows, n_out] bf16; counts/poffsets: rows and first (128-aligned) row of each local expert.
// map_a32: the same rows as map_a with a 32-row box, for steps in which no expert holds more than 32 tokens:
// the MMA still multiplies 128 rows, but rows 32.. are whatever follows in shared memory (the weight tile),
// and nobody reads their accumulator rows.
template <bool SWIGLU>
__global__ void __launch_bounds__(kThreadsK, 1)
grouped_gemm_splitk_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_a32,
                           const __grid_constant__ CUtensorMap map_b0,
                           const __grid_constant__ CUtensorMap map_b1, __nv_bfloat16 *__restrict__ out, int n_out,
                           int K, const int32_t *__restrict__ tile_expert, const int32_t *__restrict__ poffsets,
                           const int32_t *__restrict__ counts, int E, int32_t *dev_err, const EpGate gate) {
    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;  // stages need 1024-byte alignment for the swizzle
    unsigned char *base_ptr = smem_raw + (base - raw);
    uint64_t *bars = reinterpret_cast<uint64_t *>(base_ptr + kRingBytes);
    const uint32_t bar0 = base + kRingBytes;
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (kStagesMax + s); };
    const uint32_t tfull_bar = bar0 + 8u * (2 * kStagesMax);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * kStagesMax + 1);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    volatile int *small_flag = abort_flag + 1;
    float *partial = reinterpret_cast<float *>(base_ptr);  // [256 accumulator columns][128 rows]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = sreg_cluster_ctarank(), S = sreg_cluster_nctarank();
    const int cid = (int)sreg_clusterid(), ncl = (int)sreg_nclusterid();

    pdl_trigger();
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStagesMax; s++) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        mbar_init(tfull_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 2) {  // does any expert hold more than 32 tokens?
        pdl_wait();   // the counts come from the kernel before this one
        int mx = 0;
        for (int e = lane; e < E; e += 32) mx = max(mx, counts[e]);
        mx = __reduce_max_sync(0xffffffffu, mx);
        if (lane == 0) *small_flag = mx <= 32;
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(kTmemColsK)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // barriers and tensor memory are set up; everything from here on reads what earlier kernels wrote
    pdl_wait();
    const bool small = *small_flag != 0;
    const int n_stages = small ? kStagesSmall : kStagesBig;
    const uint32_t stage_bytes = small ? kStageBytesSmall : kStageBytesBig;
    const uint32_t a_bytes = small ? kABytesSmall : kABytesBig;

    const int num_m_tiles = poffsets[E] / kRowAlign;
    constexpr int n_tile_w = SWIGLU ? 128 : 256;
    const int n_tiles = (n_out + n_tile_w - 1) / n_tile_w;
    const int total = num_m_tiles * n_tiles;
    const int num_kb = (K + BLOCK_K - 1) / BLOCK_K;
    const int kb0 = (int)(((long long)num_kb * rank) / S), kb1 = (int)(((long long)num_kb * (rank + 1)) / S);

    // ring position and accumulator phase live across tiles (each role keeps its own copy)
    int stage = 0;
    uint32_t phase = 0, tphase = 0;
    bool ok = true;
    uint32_t seen = 0;  // expert parallel: sources whose rows are known to have landed (producer thread)

    for (int tile = cid; tile < total; tile += ncl) {
        int mt = tile % num_m_tiles;  // row tiles fastest: a weight tile is fetched once
        const int nt = tile / num_m_tiles;
        if (gate.tile_order != nullptr) mt = gate.tile_order[mt];
        const int e = tile_expert[mt];
        const int m_valid = min(BLOCK_M, counts[e] - (mt * BLOCK_M - poffsets[e]));
        // all lanes are converged here; a role that gave up (or whose CTA did) sits out the remaining tiles
        ok = __all_sync(0xffffffffu, ok && !*abort_flag);

        if (warp == 0) {
            // ---------------- producer: this CTA's slice of K into the ring ----------------
            if (lane == 0 && ok) {
                // the ring held the previous tile's partial sums, written and read with ordinary accesses
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                const int row_a = mt * BLOCK_M;
                const int row_b0 = e * n_out + nt * n_tile_w;
                const int row_b1 = SWIGLU ? row_b0 : row_b0 + 128;
                if (gate.wait_flags != nullptr) {
                    const uint32_t need = gate.tile_src_mask ? gate.tile_src_mask[mt] : ((1u << gate.world) - 1u);
                    if (!ep_gate_wait(gate, need, seen, dev_err)) { *abort_flag = 1; ok = false; }
                }
                for (int kb = kb0; ok && kb < kb1; kb++) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, dev_err)) { ok = false; break; }
                    const uint32_t sa = base + stage * stage_bytes;
                    mbar_expect_tx(full_bar(stage), stage_bytes);
                    if (small) tma_load_2d(sa, &map_a32, full_bar(stage), kb * BLOCK_K, row_a);
                    else tma_load_2d(sa, &map_a, full_bar(stage), kb * BLOCK_K, row_a);
                    tma_load_2d(sa + a_bytes, &map_b0, full_bar(stage), kb * BLOCK_K, row_b0);
                    tma_load_2d(sa + a_bytes + kBHalfBytesK, &map_b1, full_bar(stage), kb * BLOCK_K, row_b1);
                    if (++stage == n_stages) { stage = 0; phase ^= 1u; }
                }
                if (!ok) {
                    // let copies that were already issued land before anything else happens to the ring
                    unsigned long long t0 = globaltimer_ns();
                    while (globaltimer_ns() - t0 < 2000000ull) { }
                }
            }
        } else if (warp == 1) {
            // ---------------- MMA issuer ----------------
            if (lane == 0 && ok) {
                for (int kb = kb0; kb < kb1; kb++) {
                    if (!mbar_wait(full_bar(stage), phase, abort_flag, dev_err)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = base + stage * stage_bytes;
                    const uint64_t adesc = make_sw128_desc(sa);  // small: rows 32.. of the tile alias the B rows
                    const uint64_t bdesc = make_sw128_desc(sa + a_bytes);
#pragma unroll
                    for (int k = 0; k < BLOCK_K / UMMA_K; k++)
                        tc_mma_bf16(tmem_base, adesc + 2u * k, bdesc + 2u * k, kIdesc, (kb > kb0 || k != 0) ? 1u : 0u);
                    tc_commit(empty_bar(stage));
                    if (++stage == n_stages) { stage = 0; phase ^= 1u; }
                }
                if (ok) tc_commit(tfull_bar);  // accumulator complete, and every stage of the ring has been read
            }
        } else {
            // ---------------- partial tile: TMEM -> registers -> own shared memory ----------------
            // warp%4 selects the 32 TMEM lanes (rows) the hardware lets a warp read, (warp-2)/4 a 128-column half
            const int quarter = warp & 3, half = (warp - 2) >> 2;
            if (ok) {  // uniform over the warp
                const bool got = mbar_wait(tfull_bar, tphase, abort_flag, dev_err);
                ok = __all_sync(0xffffffffu, got);
            }
            tphase ^= 1u;
            if (ok && quarter * 32 < m_valid) {
                tc_fence_after();
                const int row = quarter * 32 + lane;
                const uint32_t t_acc = tmem_base + ((uint32_t)(quarter * 32) << 16);
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    const int col = half * 128 + c * 32;
                    uint32_t a[32];
                    if (kb1 > kb0) {
                        tc_ld32(t_acc + col, a);
                        tc_wait_ld();
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j++) a[j] = 0u;  // an empty slice of K adds nothing
                    }
#pragma unroll
                    for (int j = 0; j < 32; j++) partial[(col + j) * BLOCK_M + row] = __uint_as_float(a[j]);
                }
            }
            tc_fence_before();
        }

        cluster_barrier();  // all S partial tiles are in place

        if (warp >= 2 && !*abort_flag) {
            // ---------------- reduction of this CTA's slice of the columns, in rank order ----------------
            constexpr int kOutCols = SWIGLU ? 128 : 256;
            const int w = kOutCols / (int)S;  // output columns per CTA
            const int mv = (m_valid + 31) & ~31;
            const uint32_t p0 = smem_u32(partial);
            for (int i = threadIdx.x - 64; i < w * mv; i += kThreadsK - 64) {
                const int row = i % mv, j = (int)rank * w + i / mv;  // j: output column inside the tile
                const int oc = nt * kOutCols + j;
                if (row >= m_valid || oc >= n_out) continue;
                // all S partials are requested before the first is used (the loads are the latency here); they are
                // then added in rank order, so the sum keeps its one fixed order
                float gv[8], uv[8];
#pragma unroll
                for (uint32_t s = 0; s < 8; s++) {
                    if (s < S) {
                        gv[s] = ld_peer_f32(p0 + 4u * (uint32_t)(j * BLOCK_M + row), s);
                        if (SWIGLU) uv[s] = ld_peer_f32(p0 + 4u * (uint32_t)((128 + j) * BLOCK_M + row), s);
                    }
                }
                float g = 0.f, u = 0.f;
#pragma unroll
                for (uint32_t s = 0; s < 8; s++) {
                    if (s < S) {
                        g += gv[s];
                        if (SWIGLU) u += uv[s];
                    }
                }
                const float v = SWIGLU ? silu_f(g) * u : g;
                out[(size_t)(mt * BLOCK_M + row) * n_out + oc] = __float2bfloat16_rn(v);
            }
        }

        cluster_barrier();  // nobody reads this CTA's partial tile or accumulator any more
    }

    // Expert parallel, wait side: the product that follows overwrites the output rows of the previous step, which
    // a rank may still be gathering until it has sent this step's rows -- so this kernel does not end before
    // EVERY rank has raised its flag, also those that sent this GPU nothing.
    if (gate.wait_flags != nullptr && warp == 0 && lane == 0 && ok)
        ep_gate_wait(gate, (1u << gate.world) - 1u, seen, dev_err);
    // signal side: every thread's output stores are ordered system-wide before the CTA reports in
    if (gate.signal_flags != nullptr) __threadfence_system();
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemColsK)
                     : "memory");
    }
    if (gate.signal_flags != nullptr && warp == 0) ep_gate_signal(gate, (int)gridDim.x);
}

template <bool SWIGLU>
cudaError_t prepare_splitk(omoe_handle *h, int S, cudaLaunchConfig_t *cfg, cudaLaunchAttribute *at, int *clusters) {
    auto kern = grouped_gemm_splitk_kernel<SWIGLU>;
    static PerDeviceOnce once;  // one per instantiation
    bool *done = once.slot();
    if (!done || !*done) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytesK);
        if (e != cudaSuccess) return e;
        if (done) *done = true;
    }
    *cfg = cudaLaunchConfig_t{};
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = S;
    at[0].val.clusterDim.y = 1;
    at[0].val.clusterDim.z = 1;
    at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[1].val.programmaticStreamSerializationAllowed = 1;
    cfg->blockDim = dim3(kThreadsK);
    cfg->dynamicSmemBytes = kSmemBytesK;
    cfg->attrs = at;
    cfg->numAttrs = h->pdl ? 2 : 1;  // [0] cluster shape, [1] programmatic dependent launch
    // as many clusters as can be resident at once (a cluster lives inside one GPC)
    static int max_clusters[9] = {0};
    if (max_clusters[S] == 0) {
        cfg->gridDim = dim3(h->sm_count / S * S);
        int n = 0;
        cudaError_t e = cudaOccupancyMaxActiveClusters(&n, kern, cfg);
        if (e != cudaSuccess) return e;
        if (n < 1) return cudaErrorInvalidConfiguration;
        max_clusters[S] = n < h->sm_count / S ? n : h->sm_count / S;
    }
    *clusters = max_clusters[S];
    cfg->gridDim = dim3(max_clusters[S] * S);
    return cudaSuccess;
}

template <bool SWIGLU>
cudaError_t launch_splitk(omoe_handle *h, cudaStream_t s, int S, const CUtensorMap &a, const CUtensorMap &a32,
                          const CUtensorMap &b0, const CUtensorMap &b1, void *out, int n_out, int K,
                          const EpGate *gate) {
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute at[2];
    int clusters = 0;
    cudaError_t e = prepare_splitk<SWIGLU>(h, S, &cfg, at, &clusters);
    if (e != cudaSuccess) return e;
    cfg.stream = s;
    return cudaLaunchKernelEx(&cfg, grouped_gemm_splitk_kernel<SWIGLU>, a, a32, b0, b1,
                              static_cast<__nv_bfloat16 *>(out), n_out, K, (const int32_t *)h->ex_tile_expert,
                              (const int32_t *)h->ex_poffsets, (const int32_t *)h->ex_counts, h->e_local, h->dev_err,
                              gate ? *gate : EpGate{});
}

// Number of CTAs to share one tile of a product with `tiles_ub` tiles at most and `num_kb` blocks of K:
// the largest of 8 (the portable cluster size), 4, 2, 1 for which all tiles are in flight at once (one tile
// per resident cluster) and every CTA still gets a few blocks.  With 1 the tile is not split, but the step
// still gains the deeper ring.  0: too many tiles for this kernel, use the persistent one.
template <bool SWIGLU>
int splitk_ways(omoe_handle *h, long tiles_ub, int num_kb) {
    static int forced = getenv("OMOE_SPLITK") ? atoi(getenv("OMOE_SPLITK")) : -1;  // tests and tuning: 0, 1, 2, 4, 8
    if (forced >= 0) return forced == 1 || forced == 2 || forced == 4 || forced == 8 ? forced : 0;
    if (tiles_ub < 0 || tiles_ub > h->sm_count) return 0;
    for (int S = 8; S >= 1; S /= 2) {
        if (S > 1 && num_kb < 8 * S) continue;
        cudaLaunchConfig_t cfg;
        cudaLaunchAttribute at[2];
        int clusters = 0;
        if (prepare_splitk<SWIGLU>(h, S, &cfg, at, &clusters) != cudaSuccess) {
            cudaGetLastError();
            continue;
        }
        if (tiles_ub <= clusters) return S;
    }
    return 0;
}

}  // namespace

int splitk_ways_up_gate(omoe_handle *h, long m_tiles_ub) {
    return splitk_ways<true>(h, m_tiles_ub < 0 ? -1 : m_tiles_ub * ((h->cfg.d_ff + 127) / 128),
                             (h->cfg.d_model + BLOCK_K - 1) / BLOCK_K);
}

int splitk_ways_down(omoe_handle *h, long m_tiles_ub) {
    return splitk_ways<false>(h, m_tiles_ub < 0 ? -1 : m_tiles_ub * ((h->cfg.d_model + 255) / 256),
                              (h->cfg.d_ff + BLOCK_K - 1) / BLOCK_K);
}

cudaError_t launch_up_gate_splitk(omoe_handle *h, cudaStream_t s, int S, const EpGate *gate) {
    return launch_splitk<true>(h, s, S, h->maps.a_x, h->maps.a_x32, h->maps.b_gate, h->maps.b_up, h->hbuf,
                               h->cfg.d_ff, h->cfg.d_model, gate);
}

cudaError_t launch_down_splitk(omoe_handle *h, cudaStream_t s, int S, const EpGate *gate) {
    return launch_splitk<false>(h, s, S, h->maps.a_h, h->maps.a_h32, h->maps.b_down, h->maps.b_down, h->yp,
                                h->cfg.d_model, h->cfg.d_ff, gate);
}

}  // namespace omoe
