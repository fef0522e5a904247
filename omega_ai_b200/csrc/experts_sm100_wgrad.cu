// Weight gradients of the expert products on Blackwell tensor cores (compute_dtype = OMOE_BF16).
//
// FullyLayer.diff() forms diffW = delta^T * input with one cublasSgemm per layer
// (src/main/java/com/omega/engine/nn/layer/FullyLayer.java:292-301).  Here every expert has its own rows,
// so the product is grouped the other way round from the forward: per expert e
//     C_e [M, N] = sum over the expert's rows r of  A[r, m] * B[r, n]
// with the row index as the reduction.  The activations are stored [rows, features], so in this product the
// reduction index is the SLOW one of both operands: they are "MN-major" tiles for the tensor core.  TMA
// brings 64-feature x 64-row boxes (128-byte swizzle; a 128 x 64 A tile is two boxes, a 256 x 64 B tile
// four), the shared-memory descriptors say: 64 features contiguous, next row of the reduction 128 bytes on,
// next group of 8 rows 1024 bytes on, next 64 features one box (8 KB) on, and the instruction descriptor
// marks both operands MN-major.  Padding rows of an expert's segment must be zero in the A operand and
// finite in the B operand (backward.cu zeroes them).  MN_MAJOR = false is the older form of the same
// kernel on explicitly transposed copies (AT [M, rows], BT [N, rows], K-major as in the forward).
// The mainloop is otherwise the forward's: one CTA per SM walks (expert, n-tile, m-tile) triples; a producer
// thread feeds a 4-stage TMA ring (128-byte swizzle), one thread issues tcgen05.mma (M=128, N=256, K=16)
// into a double-buffered accumulator in tensor memory, eight epilogue warps read it with tcgen05.ld and
// store fp32 rows straight to the gradient (each thread owns one row and writes 128 contiguous bytes at a
// time).  An expert without rows has no K blocks: its tiles are written as zeros.
//
// Every mbarrier wait is bounded (sm100_ptx.cuh): when one runs out the kernel raises the device error
// word, lets outstanding copies land, frees its tensor memory and returns.
#include "backward.cuh"
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace omoe {

namespace {

using namespace sm100;
constexpr int kStagesW = 4;
constexpr int kAccStagesW = 2;
constexpr int kTmemColsW = 512;
constexpr int kABytesW = BLOCK_M * BLOCK_K * 2;            // 16 KB
constexpr int kBHalfBytesW = 128 * BLOCK_K * 2;            // 16 KB (one 128-row TMA box)
constexpr int kStageBytesW = kABytesW + 2 * kBHalfBytesW;  // 48 KB
constexpr int kSmemBytesW = kStagesW * kStageBytesW + 1024 /*align slack*/ + 256 /*barriers*/;
constexpr int kThreadsW = 320;  // warp 0 producer, warp 1 MMA, warps 2-9 epilogue

struct WTile {
    int e, mt, nt;
};
// m-tiles fastest: neighbouring CTAs share the (wider) B tile
__device__ __forceinline__ WTile wtile(int tile, int m_tiles, int n_tiles) {
    WTile t;
    const int per_e = m_tiles * n_tiles;
    t.e = tile / per_e;
    const int r = tile - t.e * per_e;
    t.nt = r / m_tiles;
    t.mt = r - t.nt * m_tiles;
    return t;
}

// 64 (MN) x 64 (K) bf16 box: 8 KB
constexpr int kBoxBytesW = 64 * BLOCK_K * 2;

// MN-major operand, 128-byte swizzle: blocks of 64 MN-elements kBoxBytesW apart (leading byte offset),
// groups of 8 reduction rows 1024 bytes apart (stride byte offset).
__device__ __forceinline__ uint64_t make_mn_sw128_desc(uint32_t smem_addr) {
    uint64_t desc = 0;
    desc |= (uint64_t)((smem_addr & 0x3ffffu) >> 4);
    desc |= (uint64_t)(kBoxBytesW >> 4) << 16;
    desc |= (uint64_t)(1024 >> 4) << 32;
    desc |= (uint64_t)1 << 46;
    desc |= (uint64_t)2 << 61;
    return desc;
}
constexpr uint32_t kIdescMN = kIdesc | (1u << 15) | (1u << 16);  // A and B MN-major

template <bool MN_MAJOR>
__global__ void __launch_bounds__(kThreadsW, 1)
wgrad_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
             float *__restrict__ out0, float *__restrict__ out1, int M, int N, int split,
             const int32_t *__restrict__ poffsets, const int32_t *__restrict__ counts, int E, int32_t *dev_err) {
    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;  // stages need 1024-byte alignment for the swizzle
    unsigned char *base_ptr = smem_raw + (base - raw);
    uint64_t *bars = reinterpret_cast<uint64_t *>(base_ptr + kStagesW * kStageBytesW);
    const uint32_t bar0 = base + kStagesW * kStageBytesW;
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (kStagesW + s); };
    auto tfull_bar = [&](int s) { return bar0 + 8u * (2 * kStagesW + s); };
    auto tempty_bar = [&](int s) { return bar0 + 8u * (2 * kStagesW + kAccStagesW + s); };
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * kStagesW + 2 * kAccStagesW);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStagesW; s++) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int s = 0; s < kAccStagesW; s++) {
            mbar_init(tfull_bar(s), 1);
            mbar_init(tempty_bar(s), 8);  // one arrival per epilogue warp
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(kTmemColsW)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int m_tiles = (M + BLOCK_M - 1) / BLOCK_M, n_tiles = (N + BLOCK_N - 1) / BLOCK_N;
    const int total = E * m_tiles * n_tiles;

    if (warp == 0) {
        // ---------------- producer: TMA loads into the ring ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < total; tile += gridDim.x) {
                const WTile t = wtile(tile, m_tiles, n_tiles);
                const int seg0 = poffsets[t.e];
                const int num_kb = (counts[t.e] + BLOCK_K - 1) / BLOCK_K;
                for (int kb = 0; kb < num_kb; kb++) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, dev_err)) { ok = false; break; }
                    const uint32_t sa = base + stage * kStageBytesW;
                    const int x = seg0 + kb * BLOCK_K;  // a multiple of 64 elements: 128-byte aligned
                    mbar_expect_tx(full_bar(stage), kStageBytesW);
                    if constexpr (MN_MAJOR) {
                        // maps are [rows, features]: the feature index is the inner coordinate
#pragma unroll
                        for (int i = 0; i < 2; i++)
                            tma_load_2d(sa + i * kBoxBytesW, &map_a, full_bar(stage), t.mt * BLOCK_M + 64 * i, x);
#pragma unroll
                        for (int i = 0; i < 4; i++)
                            tma_load_2d(sa + kABytesW + i * kBoxBytesW, &map_b, full_bar(stage),
                                        t.nt * BLOCK_N + 64 * i, x);
                    } else {
                        tma_load_2d(sa, &map_a, full_bar(stage), x, t.mt * BLOCK_M);
                        tma_load_2d(sa + kABytesW, &map_b, full_bar(stage), x, t.nt * BLOCK_N);
                        tma_load_2d(sa + kABytesW + kBHalfBytesW, &map_b, full_bar(stage), x, t.nt * BLOCK_N + 128);
                    }
                    if (++stage == kStagesW) { stage = 0; phase ^= 1u; }
                }
            }
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
                const WTile t = wtile(tile, m_tiles, n_tiles);
                const int num_kb = (counts[t.e] + BLOCK_K - 1) / BLOCK_K;
                if (!mbar_wait(tempty_bar(as), aphase ^ 1u, abort_flag, dev_err)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + as * BLOCK_N;
                for (int kb = 0; kb < num_kb; kb++) {
                    if (!mbar_wait(full_bar(stage), phase, abort_flag, dev_err)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = base + stage * kStageBytesW;
                    if constexpr (MN_MAJOR) {
                        const uint64_t adesc = make_mn_sw128_desc(sa);
                        const uint64_t bdesc = make_mn_sw128_desc(sa + kABytesW);
                        // 16 rows of the reduction are 16 x 128 bytes further on: +128 in 16-byte units
#pragma unroll
                        for (int k = 0; k < BLOCK_K / UMMA_K; k++)
                            tc_mma_bf16(d_tmem, adesc + 128u * k, bdesc + 128u * k, kIdescMN, (kb | k) != 0 ? 1u : 0u);
                    } else {
                        const uint64_t adesc = make_sw128_desc(sa);
                        const uint64_t bdesc = make_sw128_desc(sa + kABytesW);
#pragma unroll
                        for (int k = 0; k < BLOCK_K / UMMA_K; k++)
                            tc_mma_bf16(d_tmem, adesc + 2u * k, bdesc + 2u * k, kIdesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    tc_commit(empty_bar(stage));  // frees the stage once these MMAs have read it
                    if (++stage == kStagesW) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                tc_commit(tfull_bar(as));  // accumulator complete (at once for an expert without rows)
                if (++as == kAccStagesW) { as = 0; aphase ^= 1u; }
            }
        }
    } else {
        // ---------------- epilogue: TMEM -> registers -> global fp32 ----------------
        // warp%4 selects the 32 TMEM lanes (rows) the hardware lets a warp read, (warp-2)/4 a 64-column half
        // of each 128-column pass.
        const int quarter = warp & 3, half = (warp - 2) >> 2;
        const int row = quarter * 32 + lane;
        int as = 0;
        uint32_t aphase = 0;
        for (int tile = blockIdx.x; tile < total; tile += gridDim.x) {
            const WTile t = wtile(tile, m_tiles, n_tiles);
            const bool empty = counts[t.e] == 0;
            bool ok = mbar_wait(tfull_bar(as), aphase, abort_flag, dev_err);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const uint32_t t_acc = tmem_base + as * BLOCK_N + ((uint32_t)(quarter * 32) << 16);
            const int m = t.mt * BLOCK_M + row;
            float *orow = nullptr;
            if (m < M)
                orow = m < split ? out0 + ((size_t)t.e * split + m) * N
                                 : out1 + ((size_t)t.e * (M - split) + (m - split)) * N;
#pragma unroll
            for (int p = 0; p < 2; p++) {
#pragma unroll
                for (int c = 0; c < 2; c++) {
                    const int col = p * 128 + half * 64 + c * 32;
                    uint32_t a[32];
                    if (!empty) {
                        tc_ld32(t_acc + col, a);
                        tc_wait_ld();
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j++) a[j] = 0u;
                    }
                    if (p == 1 && c == 1) {  // all of this warp's accumulator reads are done
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(tempty_bar(as));
                    }
                    const int n0 = t.nt * BLOCK_N + col;
                    if (orow != nullptr) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4)
                            if (n0 + j < N)  // N is a multiple of 8
                                *reinterpret_cast<float4 *>(orow + n0 + j) =
                                    make_float4(__uint_as_float(a[j]), __uint_as_float(a[j + 1]),
                                                __uint_as_float(a[j + 2]), __uint_as_float(a[j + 3]));
                    }
                }
            }
            if (++as == kAccStagesW) { as = 0; aphase ^= 1u; }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemColsW)
                     : "memory");
    }
}

}  // namespace

template <bool MN_MAJOR>
static cudaError_t launch_wgrad_t(omoe_handle *h, cudaStream_t s, const CUtensorMap &a, const CUtensorMap &b, int M,
                                  int N, int split, float *out0, float *out1) {
    static PerDeviceOnce once;  // one per instantiation
    bool *done = once.slot();
    if (!done || !*done) {
        cudaError_t e = cudaFuncSetAttribute(wgrad_kernel<MN_MAJOR>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             kSmemBytesW);
        if (e != cudaSuccess) return e;
        if (done) *done = true;
    }
    wgrad_kernel<MN_MAJOR><<<dim3(h->sm_count), dim3(kThreadsW), kSmemBytesW, s>>>(
        a, b, out0, out1, M, N, split, h->ex_poffsets, h->ex_counts, h->e_local, h->dev_err);
    return cudaGetLastError();
}

cudaError_t launch_wgrad_bf16(omoe_handle *h, cudaStream_t s, const CUtensorMap &at, const CUtensorMap &bt, int M,
                              int N, int split, float *out0, float *out1) {
    return launch_wgrad_t<false>(h, s, at, bt, M, N, split, out0, out1);
}

cudaError_t launch_wgrad_bf16_rows(omoe_handle *h, cudaStream_t s, const CUtensorMap &a, const CUtensorMap &b, int M,
                                   int N, int split, float *out0, float *out1) {
    return launch_wgrad_t<true>(h, s, a, b, M, N, split, out0, out1);
}

}  // namespace omoe
