// Grouped expert products with CTA pairs (tcgen05 cta_group::2).
//
// Same job and same mainloop roles as experts_sm100.cu, but two CTAs on
// neighbouring SMs (a cluster of 2) share one 256 x 256 output tile: each CTA
// holds its own 128 rows of A and HALF of the B tile (128 of the 256 weight
// rows), and one tcgen05.mma.cta_group::2 issued by the pair's leader drives
// both SMs' tensor cores, each reading the other's B half over the pair link.
// Per CTA and k-step that is 32 KB of shared-memory fill instead of 48 KB, so
// the ring is 6 stages deep instead of 4 and the L2 -> SM stream of the weight
// operand is halved.  For the up/gate product the two halves are natural: the
// leader loads the gate rows, its peer the up rows.
//
// Every load is a plain 2-D TMA tile load into the issuing CTA only; completion of both
// CTAs' loads is counted on the leader's barrier; the leader signals "stage
// free" and "accumulator ready" to both CTAs with one tcgen05.commit per
// barrier.  Every wait is bounded as in the single-CTA kernel.
#include <stdlib.h>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace omoe {

namespace {

using namespace sm100;

constexpr int kStages2 = 6;
constexpr int kAccStages2 = 2;
constexpr int kTmemCols2 = 512;
constexpr int kABytes2 = BLOCK_M * BLOCK_K * 2;        // 16 KB: this CTA's 128 rows of A
constexpr int kBBytes2 = 128 * BLOCK_K * 2;            // 16 KB: this CTA's half of the B tile
constexpr int kStageBytes2 = kABytes2 + kBBytes2;      // 32 KB
constexpr int kOutSub2 = 128 * 64 * 2;
constexpr int kOutBytes2 = 2 * kOutSub2;               // 32 KB staging for 128 output columns
constexpr int kTableBytes = 2 * (kMaxExperts + 1) * 2; // two uint16 tables
constexpr int kSmemBytes2 = kStages2 * kStageBytes2 + kOutBytes2 + 1024 + 256 + kTableBytes;
constexpr int kThreads2 = 320;

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// shared::cluster address of the same shared-memory location in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
    return r;
}

__device__ __forceinline__ void mbar_expect_tx_cluster(uint32_t cluster_bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(cluster_bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}

// TMA tile load of a CTA pair: data lands in this CTA, bytes are counted on the barrier at cluster address `bar`
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
        : "memory");
}

__device__ __forceinline__ void tc_commit_pair(uint32_t cluster_bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar) : "memory");
}

__device__ __forceinline__ void tc_mma_bf16_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                 uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// fp32 accumulator, bf16 A and B, both K-major, N = 256, M = 256 across the pair
constexpr uint32_t kIdescPair = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(256 >> 3) << 17) |
                                ((uint32_t)(256 >> 4) << 24);

struct PairTile {
    int mt;      // this CTA's 128-row tile
    int nt;      // 256-wide (128 for up/gate outputs) column tile
    int expert;
    bool store;  // false for the peer half of an expert's last, unpaired m-tile
};

// Work item w -> (pair-tile p, nt) in bands of `kband` pair-tiles x all n-tiles; pair-tile p -> expert and m-tiles.
__device__ __forceinline__ PairTile pair_tile(int w, int n_ptiles, int n_tiles, int kband, const uint16_t *pt_start,
                                              const uint16_t *mt_start, int E, uint32_t rank) {
    const int per_band = kband * n_tiles;
    const int band = w / per_band, r = w % per_band;
    const int p0 = band * kband;
    const int bp = min(kband, n_ptiles - p0);
    const int p = p0 + r % bp;
    PairTile t;
    t.nt = r / bp;
    int lo = 0, hi = E;  // largest e with pt_start[e] <= p
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (pt_start[mid] <= p) lo = mid; else hi = mid;
    }
    t.expert = lo;
    const int local = p - pt_start[lo];
    const int n_mt = mt_start[lo + 1] - mt_start[lo];
    const bool has2 = 2 * local + 1 < n_mt;
    t.mt = mt_start[lo] + 2 * local + ((rank == 1 && has2) ? 1 : 0);
    t.store = rank == 0 || has2;
    return t;
}

template <bool SWIGLU>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads2, 1)
grouped_gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b0,
                         const __grid_constant__ CUtensorMap map_b1, const __grid_constant__ CUtensorMap map_out,
                         int n_out, int K, const int32_t *__restrict__ poffsets, int E, int kband, int32_t *dev_err) {
    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    unsigned char *base_ptr = smem_raw + (base - raw);
    constexpr int kDataBytes = kStages2 * kStageBytes2 + kOutBytes2;
    uint64_t *bars = reinterpret_cast<uint64_t *>(base_ptr + kDataBytes);
    const uint32_t bar0 = base + kDataBytes;
    auto full_bar = [&](int s) { return bar0 + 8u * s; };                       // used in the leader
    auto empty_bar = [&](int s) { return bar0 + 8u * (kStages2 + s); };          // one per CTA
    auto tfull_bar = [&](int s) { return bar0 + 8u * (2 * kStages2 + s); };      // one per CTA
    auto tempty_bar = [&](int s) { return bar0 + 8u * (2 * kStages2 + kAccStages2 + s); };  // used in the leader
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * kStages2 + 2 * kAccStages2);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    uint16_t *pt_start = reinterpret_cast<uint16_t *>(base_ptr + kDataBytes + 256);  // [E+1] first pair-tile of expert e
    uint16_t *mt_start = pt_start + (kMaxExperts + 1);                                // [E+1] first 128-row tile of expert e

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();  // 0 = leader of the pair
    const uint32_t peer = rank ^ 1u;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages2; s++) {
            mbar_init(full_bar(s), 2);   // one arrive.expect_tx from each CTA's producer
            mbar_init(empty_bar(s), 1);  // the leader's commit
        }
        for (int s = 0; s < kAccStages2; s++) {
            mbar_init(tfull_bar(s), 1);    // the leader's commit
            mbar_init(tempty_bar(s), 16);  // eight epilogue warps in each CTA
        }
        *abort_flag = 0;
        int pt = 0;
        for (int e = 0; e < E; e++) {
            pt_start[e] = (uint16_t)pt;
            mt_start[e] = (uint16_t)(poffsets[e] / kRowAlign);
            pt += ((poffsets[e + 1] - poffsets[e]) / kRowAlign + 1) / 2;
        }
        pt_start[E] = (uint16_t)pt;
        mt_start[E] = (uint16_t)(poffsets[E] / kRowAlign);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(kTmemCols2)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // both CTAs' barriers exist before anyone signals across the pair
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int n_ptiles = pt_start[E];
    const int n_tile_w = SWIGLU ? 128 : 256;
    const int n_tiles = (n_out + n_tile_w - 1) / n_tile_w;
    const int total = n_ptiles * n_tiles;
    const int num_kb = (K + BLOCK_K - 1) / BLOCK_K;
    const int pair_id = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;

    if (warp == 0) {
        // ---------------- producer (both CTAs): own A rows and own half of B ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int w = pair_id; ok && w < total; w += n_pairs) {
                const PairTile t = pair_tile(w, n_ptiles, n_tiles, kband, pt_start, mt_start, E, rank);
                const int row_a = t.mt * BLOCK_M;
                // leader: gate rows / first 128 weight rows; peer: up rows / second 128 weight rows
                const CUtensorMap *mb = (SWIGLU && rank == 1) ? &map_b1 : &map_b0;
                const int row_b = t.expert * n_out + t.nt * n_tile_w + ((!SWIGLU && rank == 1) ? 128 : 0);
                for (int kb = 0; kb < num_kb; kb++) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, dev_err)) { ok = false; break; }
                    const uint32_t sa = base + stage * kStageBytes2;
                    const uint32_t lead_full = map_to_rank(full_bar(stage), 0);
                    mbar_expect_tx_cluster(lead_full, kStageBytes2);
                    tma_load_2d_pair(sa, &map_a, lead_full, kb * BLOCK_K, row_a);
                    tma_load_2d_pair(sa + kABytes2, mb, lead_full, kb * BLOCK_K, row_b);
                    if (++stage == kStages2) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok) {
                unsigned long long t0 = globaltimer_ns();
                while (globaltimer_ns() - t0 < 2000000ull) { }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (leader only) ----------------
        if (rank == 0 && lane == 0) {
            int stage = 0, as = 0;
            uint32_t phase = 0, aphase = 0;
            bool ok = true;
            for (int w = pair_id; ok && w < total; w += n_pairs) {
                if (!mbar_wait(tempty_bar(as), aphase ^ 1u, abort_flag, dev_err)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + as * BLOCK_N;
                for (int kb = 0; kb < num_kb; kb++) {
                    if (!mbar_wait(full_bar(stage), phase, abort_flag, dev_err)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = base + stage * kStageBytes2;
                    const uint64_t adesc = make_sw128_desc(sa);
                    const uint64_t bdesc = make_sw128_desc(sa + kABytes2);
#pragma unroll
                    for (int k = 0; k < BLOCK_K / UMMA_K; k++)
                        tc_mma_bf16_pair(d_tmem, adesc + 2u * k, bdesc + 2u * k, kIdescPair, (kb | k) != 0 ? 1u : 0u);
                    // the stage is free in both CTAs once these MMAs have read it
                    tc_commit_pair(empty_bar(stage));
                    tc_commit_pair(map_to_rank(empty_bar(stage), 1));
                    if (++stage == kStages2) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                tc_commit_pair(tfull_bar(as));
                tc_commit_pair(map_to_rank(tfull_bar(as), 1));
                if (++as == kAccStages2) { as = 0; aphase ^= 1u; }
            }
        }
    } else {
        // ---------------- epilogue (both CTAs): own 128 rows of the accumulator ----------------
        const int ew = warp - 2;
        const int quarter = warp & 3;
        const int half = ew >> 2;
        const int r = quarter * 32 + lane;
        const uint32_t out_stage = base + kStages2 * kStageBytes2;
        const uint32_t my_row = out_stage + half * kOutSub2 + r * 128;
        constexpr int kPasses = SWIGLU ? 1 : 2;
        int as = 0;
        uint32_t aphase = 0;
        for (int w = pair_id; w < total; w += n_pairs) {
            const PairTile t = pair_tile(w, n_ptiles, n_tiles, kband, pt_start, mt_start, E, rank);
            bool ok = mbar_wait(tfull_bar(as), aphase, abort_flag, dev_err);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const uint32_t t_acc = tmem_base + as * BLOCK_N + ((uint32_t)(quarter * 32) << 16);
            const uint32_t lead_tempty = map_to_rank(tempty_bar(as), 0);
#pragma unroll
            for (int p = 0; p < kPasses; p++) {
#pragma unroll
                for (int c = 0; c < 2; c++) {
                    const int col = p * 128 + half * 64 + c * 32;
                    uint32_t o[16];
                    if constexpr (SWIGLU) {
                        uint32_t g[32], u[32];
                        tc_ld32(t_acc + col, g);
                        tc_ld32(t_acc + 128 + col, u);
                        tc_wait_ld();
                        if (c == 1) {
                            tc_fence_before();
                            __syncwarp();
                            if (lane == 0) mbar_arrive_cluster(lead_tempty);
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
                            if (lane == 0) mbar_arrive_cluster(lead_tempty);
                        }
#pragma unroll
                        for (int i = 0; i < 16; i++)
                            o[i] = pack_bf16(__uint_as_float(a[2 * i]), __uint_as_float(a[2 * i + 1]));
                    }
                    if (c == 0) {
                        if (warp == 2 && lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                        asm volatile("bar.sync 1, 256;" ::: "memory");
                    }
#pragma unroll
                    for (int v = 0; v < 4; v++) {
                        const int chunk = (c * 4 + v) ^ (r & 7);
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(my_row + chunk * 16),
                                     "r"(o[4 * v]), "r"(o[4 * v + 1]), "r"(o[4 * v + 2]), "r"(o[4 * v + 3])
                                     : "memory");
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                asm volatile("bar.sync 1, 256;" ::: "memory");
                if (warp == 2 && lane == 0 && t.store) {
                    const int x0 = t.nt * (SWIGLU ? 128 : 256) + p * 128;
                    const int y0 = t.mt * BLOCK_M;
                    if (x0 < n_out) tma_store_2d(&map_out, out_stage, x0, y0);
                    if (x0 + 64 < n_out) tma_store_2d(&map_out, out_stage + kOutSub2, x0 + 64, y0);
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                }
            }
            if (++as == kAccStages2) { as = 0; aphase ^= 1u; }
        }
        if (warp == 2 && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }

    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // the peer may still be reading this CTA's shared memory or signalling its barriers
    if (warp == 1) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols2) : "memory");
    }
}

}  // namespace

cudaError_t launch_experts_bf16_pair(omoe_handle *h, cudaStream_t s, int *n, cudaEvent_t mid) {
    static PerDeviceOnce once;
    bool *done = once.slot();
    if (!done || !*done) {
        cudaError_t e = cudaFuncSetAttribute(grouped_gemm_pair_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             kSmemBytes2);
        if (e != cudaSuccess) return e;
        e = cudaFuncSetAttribute(grouped_gemm_pair_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes2);
        if (e != cudaSuccess) return e;
        if (done) *done = true;
    }
    const int d = h->cfg.d_model, dff = h->cfg.d_ff;
    static int band_up = getenv("OMOE_BAND_UP") ? atoi(getenv("OMOE_BAND_UP")) : 16;
    static int band_dn = getenv("OMOE_BAND_DOWN") ? atoi(getenv("OMOE_BAND_DOWN")) : 16;
    dim3 grid(h->sm_count & ~1), block(kThreads2);
    // bands are counted in pair-tiles here (two 128-row tiles each)
    grouped_gemm_pair_kernel<true><<<grid, block, kSmemBytes2, s>>>(h->maps.a_x, h->maps.b_gate, h->maps.b_up, h->maps.a_h,
                                                                   dff, d, h->ex_poffsets, h->e_local,
                                                                   band_up > 1 ? band_up / 2 : 1, h->dev_err);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    (*n)++;
    if (mid) cudaEventRecord(mid, s);
    grouped_gemm_pair_kernel<false><<<grid, block, kSmemBytes2, s>>>(h->maps.a_h, h->maps.b_down, h->maps.b_down,
                                                                    h->maps.c_y, d, dff, h->ex_poffsets, h->e_local,
                                                                    band_dn > 1 ? band_dn / 2 : 1, h->dev_err);
    e = cudaGetLastError();
    if (e == cudaSuccess) (*n)++;
    return e;
}

}  // namespace omoe
