// Expert products for a handful of tokens (decode steps): weight-streaming
// kernels.  With one or two rows per expert the tensor-core tiles of
// experts_sm100.cu would be 99 % padding and, worse, there are too few tiles to
// keep every SM's share of HBM busy.  Here the work item is one output column
// (one weight row, or a gate/up pair of rows), streamed once in 512-byte
// pieces and folded against the expert's token rows held in shared memory, so
// the items spread evenly over all SMs and the kernels run at HBM speed.  Two
// kernels: one that loads into registers and folds on the CUDA cores (1-4
// token rows per pass) and one that stages the weights through shared-memory
// rings with bulk copies and folds with warp-level MMAs (one or two rows; the
// default where it applies).  Same arithmetic points as the tensor-core path
// (bf16 operands, fp32 accumulate, h and yp rounded to bf16); they replace the
// same reference calls (LlamaMLPLayer.java:117-123).
#include <stdlib.h>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace omoe {

namespace {

constexpr int kDecThreads = 256;
constexpr int kPairs = kDecThreads / 64;

// 64-thread barrier of one warp pair; the id is a literal so the kernel reserves only the barriers it uses
__device__ __forceinline__ void pair_sync(int pair) {
    switch (pair) {
        case 0: asm volatile("bar.sync 1, 64;" ::: "memory"); break;
        case 1: asm volatile("bar.sync 2, 64;" ::: "memory"); break;
        case 2: asm volatile("bar.sync 3, 64;" ::: "memory"); break;
        default: asm volatile("bar.sync 4, 64;" ::: "memory"); break;
    }
}

__device__ __forceinline__ uint4 ld_stream(const void *p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}

// out[row, n] = f( A[row, :] . W0[e][n, :],  A[row, :] . W1[e][n, :] )  for the rows of every expert e that has any.
// SWIGLU: f(g, u) = silu(g) * u;  else f(g, -) = g and W1 is unused.
// Items (expert, n) are numbered expert-major over the experts that have rows and dealt out in equal contiguous
// runs to the blocks; inside a block the four warp pairs take them round-robin, each warp half of K.
// RP: token rows of one expert folded per pass over its weights (1, 2 or 4).
template <bool SWIGLU, int RP>
__global__ void __launch_bounds__(kDecThreads, 2)
decode_gemv_kernel(const __nv_bfloat16 *__restrict__ A, const __nv_bfloat16 *__restrict__ W0,
                   const __nv_bfloat16 *__restrict__ W1, __nv_bfloat16 *__restrict__ out, int K, int N,
                   const int32_t *__restrict__ counts, const int32_t *__restrict__ poffsets, int El) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __nv_bfloat16 *rows = reinterpret_cast<__nv_bfloat16 *>(smem_raw);  // [RP][K]
    __shared__ int s_active[kMaxExperts];
    __shared__ int s_n_active;
    __shared__ float s_part[kPairs][2][RP];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int pair = warp >> 1, half = warp & 1;
    pdl_trigger();
    pdl_wait();
    if (tid == 0) {
        int n = 0;
        for (int e = 0; e < El; e++)
            if (counts[e] > 0) s_active[n++] = e;
        s_n_active = n;
    }
    __syncthreads();
    const long long total = (long long)s_n_active * N;
    const long long per = (total + gridDim.x - 1) / gridDim.x;
    const long long g0 = (long long)blockIdx.x * per;
    const long long g1 = g0 + per < total ? g0 + per : total;
    const int kh = (K / 2 + 7) / 8 * 8;           // first warp of a pair takes [0, kh), the second [kh, K)
    const int k_lo = half ? kh : 0, k_hi = half ? K : kh;

    long long g = g0;
    while (g < g1) {
        const int ai = (int)(g / N);
        const int e = s_active[ai];
        const long long g_end_e = (long long)(ai + 1) * N < g1 ? (long long)(ai + 1) * N : g1;
        const int m = counts[e];
        const int row0 = poffsets[e];
        for (int r0 = 0; r0 < m; r0 += RP) {
            const int mr = m - r0 < RP ? m - r0 : RP;
            __syncthreads();
            for (int i = tid; i < mr * (K / 8); i += kDecThreads) {
                int r = i / (K / 8), c = i % (K / 8);
                reinterpret_cast<uint4 *>(rows + (size_t)r * K)[c] =
                    reinterpret_cast<const uint4 *>(A + (size_t)(row0 + r0 + r) * K)[c];
            }
            __syncthreads();
            for (long long it = g + pair; it < g_end_e; it += kPairs) {
                const int n = (int)(it - (long long)ai * N);
                const __nv_bfloat16 *w0 = W0 + ((size_t)e * N + n) * K;
                const __nv_bfloat16 *w1 = SWIGLU ? W1 + ((size_t)e * N + n) * K : nullptr;
                float acc0[RP], acc1[RP];
#pragma unroll
                for (int r = 0; r < RP; r++) { acc0[r] = 0.f; acc1[r] = 0.f; }
                constexpr int U = SWIGLU ? 4 : 8;  // 16-byte loads per operand in flight per lane
                for (int k0 = k_lo + lane * 8; k0 < k_hi; k0 += 32 * 8 * U) {
                    uint4 q0[U], q1[SWIGLU ? U : 1];
#pragma unroll
                    for (int u = 0; u < U; u++) {
                        const int kk = k0 + u * 256;
                        if (kk < k_hi) {
                            q0[u] = ld_stream(w0 + kk);
                            if (SWIGLU) q1[u] = ld_stream(w1 + kk);
                        }
                    }
#pragma unroll
                    for (int u = 0; u < U; u++) {
                        const int kk = k0 + u * 256;
                        if (kk < k_hi) {
                            float wv0[8], wv1[8];
                            unpack8(q0[u], wv0);
                            if (SWIGLU) unpack8(q1[u], wv1);
#pragma unroll
                            for (int r = 0; r < RP; r++) {
                                if (r < mr) {
                                    float av[8];
                                    unpack8(*reinterpret_cast<const uint4 *>(rows + (size_t)r * K + kk), av);
#pragma unroll
                                    for (int j = 0; j < 8; j++) {
                                        acc0[r] = fmaf(av[j], wv0[j], acc0[r]);
                                        if (SWIGLU) acc1[r] = fmaf(av[j], wv1[j], acc1[r]);
                                    }
                                }
                            }
                        }
                    }
                }
#pragma unroll
                for (int r = 0; r < RP; r++) {
#pragma unroll
                    for (int o = 16; o >= 1; o >>= 1) {
                        acc0[r] += __shfl_xor_sync(0xffffffffu, acc0[r], o);
                        if (SWIGLU) acc1[r] += __shfl_xor_sync(0xffffffffu, acc1[r], o);
                    }
                }
                // second warp of the pair hands its half over; the first finishes the column
                if (half == 1 && lane == 0) {
#pragma unroll
                    for (int r = 0; r < RP; r++) { s_part[pair][0][r] = acc0[r]; s_part[pair][1][r] = acc1[r]; }
                }
                pair_sync(pair);
                if (half == 0 && lane == 0) {
#pragma unroll
                    for (int r = 0; r < RP; r++) {
                        if (r < mr) {
                            float g_ = acc0[r] + s_part[pair][0][r];
                            float v = g_;
                            if (SWIGLU) {
                                float u_ = acc1[r] + s_part[pair][1][r];
                                v = __fdividef(g_, 1.0f + __expf(-g_)) * u_;
                            }
                            out[(size_t)(row0 + r0 + r) * N + n] = __float2bfloat16_rn(v);
                        }
                    }
                }
                pair_sync(pair);
            }
        }
        g = g_end_e;
    }
}

// ---- the same product with the dot products on the tensor cores' warp-level MMA ----
//
// The kernel above spends 26 (one token row) to 43 (two) instructions per 16 bytes of weights, unpacking bf16
// pairs and issuing one FMA per element, which makes it issue-bound from two rows on; and after every output
// column its warps stop requesting memory while they reduce.  This kernel keeps the access pattern (512
// contiguous bytes of ONE weight row at a time) but stages the weights through shared memory with bulk copies
// and hands the arithmetic to `mma.sync.m16n8k16`.
//
// Staging: each of the eight warps owns a ring of three 4 KB stages; lane 0 keeps one `cp.async.bulk` copy
// (completion on the stage's mbarrier, bounded waits) in flight per stage, the warp folds a stage as soon as it
// has landed and re-arms it at once, so the next columns' weights are already requested while a column is
// reduced and stored.  Three stages (96 KB per SM in flight) measured best; deeper rings were slower.
//
// Fold: lane (g, t) (g = lane/4, t = lane%4) reads 16 bytes = 8 consecutive k of the weight row, which the MMA
// takes as the B operand's k slots {2t, 2t+1, 2t+8, 2t+9} of "column" g (two MMAs per 16 bytes); the same lane
// supplies the token's values at the same k as row g (first token) and row g+8 (second token) of the A operand.
// Then D[g][g] is the lane group's share of the first token's dot product and D[g+8][g] of the second: the
// diagonal is what is kept, summed over the lanes at the end of a weight row.  The products off the diagonal
// are wasted work on a pipe that has nothing else to do.
//
// Work split: a block works for ONE expert (the blocks are dealt evenly over the experts that have rows), so the
// expert's token rows stay in shared memory for the whole launch; its warps take the output columns round-robin
// and own them whole, so nothing is handed between warps and nothing synchronises once the rows are staged.
// Any K that is a multiple of 8: a short last piece of a weight row is masked.
constexpr int kRingWarps = 8;
constexpr int kRingThreads = kRingWarps * 32;
constexpr int kRingStageBytes = 4096;
constexpr int kRingStages = 3;
constexpr int kRingHeader = 1024;  // mbarriers: kRingWarps * kRingStages * 8 bytes

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 r;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "r"(addr));
    return r;
}

// d (16x8, fp32) += a (16x16 bf16: rows 0-7 from a_lo/a_hi, rows 8-15 from b_lo/b_hi) * w (16x8 bf16)
__device__ __forceinline__ void mma_diag(float (&d)[4], uint32_t a_lo, uint32_t b_lo, uint32_t a_hi, uint32_t b_hi,
                                         uint32_t w_lo, uint32_t w_hi) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a_lo), "r"(b_lo), "r"(a_hi), "r"(b_hi), "r"(w_lo), "r"(w_hi));
}

__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

// NT: token rows folded (1 or 2); an expert never holds more when the step has at most NT tokens
template <bool SWIGLU, int NT>
__global__ void __launch_bounds__(kRingThreads, 1)
decode_mma_kernel(const __nv_bfloat16 *__restrict__ A, const __nv_bfloat16 *__restrict__ W0,
                   const __nv_bfloat16 *__restrict__ W1, __nv_bfloat16 *__restrict__ out, int K, int N,
                   const int32_t *__restrict__ counts, const int32_t *__restrict__ poffsets, int El, int stages,
                   int32_t *dev_err) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ int s_active[kMaxExperts];
    __shared__ int s_n_active;
    __shared__ int s_abort;
    constexpr int CH = SWIGLU ? 2 : 1;
    constexpr int CE = SWIGLU ? kRingStageBytes / 4 : kRingStageBytes / 2;  // elements of K per stage and operand
    constexpr int UNITS = CE / 256;                                          // 512-byte pieces per stage and operand

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t smem0 = sm100::smem_u32(smem_raw);
    const uint32_t bars = smem0 + warp * kRingStages * 8;
    const uint32_t ring = smem0 + kRingHeader + warp * stages * kRingStageBytes;
    const uint32_t rows = smem0 + kRingHeader + kRingWarps * stages * kRingStageBytes;  // [NT][K] bf16
    __nv_bfloat16 *rows_p = reinterpret_cast<__nv_bfloat16 *>(smem_raw + kRingHeader +
                                                               (size_t)kRingWarps * stages * kRingStageBytes);
    pdl_trigger();
    if (lane == 0)
        for (int s = 0; s < stages; s++) sm100::mbar_init(bars + s * 8, 1);
    if (tid == 0) s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    pdl_wait();
    if (tid == 0) {
        int n = 0;
        for (int e = 0; e < El; e++)
            if (counts[e] > 0) s_active[n++] = e;
        s_n_active = n;
    }
    __syncthreads();
    const int n_active = s_n_active;
    if (n_active == 0) return;
    const int bpe = gridDim.x / n_active;  // blocks per expert (the host keeps n_active <= gridDim.x)
    const int ai = blockIdx.x / bpe;
    if (ai >= n_active) return;
    const int e = s_active[ai];
    const int lb = blockIdx.x - ai * bpe;
    const int per = (N + bpe - 1) / bpe;
    const int n0 = lb * per;
    const int n1 = n0 + per < N ? n0 + per : N;
    if (n1 <= n0) return;
    const int m = counts[e];
    const int mr = m < NT ? m : NT;
    const int row0 = poffsets[e];

    const int nch = (K + CE - 1) / CE;  // stages per column
    const int cnt = n1 - n0 > warp ? (n1 - n0 - warp + kRingWarps - 1) / kRingWarps : 0;  // this warp's columns
    const int total = cnt * nch;
    const __nv_bfloat16 *w0 = W0 + ((size_t)e * N + n0 + warp) * K;
    const __nv_bfloat16 *w1 = SWIGLU ? W1 + ((size_t)e * N + n0 + warp) * K : nullptr;

    // lane 0's issue cursor: chunk i_ch of the column at w0/w1 goes into stage i_stage
    int i_ch = 0, i_stage = 0, issued = 0;
    auto issue_one = [&]() {
        const int k0 = i_ch * CE;
        const uint32_t bytes = (uint32_t)((K - k0 < CE ? K - k0 : CE) * 2);
        const uint32_t bar = bars + i_stage * 8;
        const uint32_t dst = ring + i_stage * kRingStageBytes;
        sm100::mbar_expect_tx(bar, SWIGLU ? 2 * bytes : bytes);
        bulk_load(dst, w0 + k0, bytes, bar);
        if (SWIGLU) bulk_load(dst + kRingStageBytes / 2, w1 + k0, bytes, bar);
        if (++i_ch == nch) {
            i_ch = 0;
            w0 += (size_t)kRingWarps * K;
            if (SWIGLU) w1 += (size_t)kRingWarps * K;
        }
        if (++i_stage == stages) i_stage = 0;
        issued++;
    };
    if (lane == 0)
        while (issued < total && issued < stages) issue_one();
    // the token rows come in while the first weights are on their way
    for (int i = tid; i < NT * (K / 8); i += kRingThreads) {
        int r = i / (K / 8), c = i % (K / 8);
        // a missing second row is read as zeros
        reinterpret_cast<uint4 *>(rows_p + (size_t)r * K)[c] =
            r < mr ? reinterpret_cast<const uint4 *>(A + (size_t)(row0 + r) * K)[c] : make_uint4(0u, 0u, 0u, 0u);
    }
    __syncthreads();

    float acc[CH][2][4];
#pragma unroll
    for (int c = 0; c < CH; c++)
#pragma unroll
        for (int s = 0; s < 2; s++)
#pragma unroll
            for (int j = 0; j < 4; j++) acc[c][s][j] = 0.f;
    const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
    int c_stage = 0, ch = 0, col = 0;
    uint32_t c_parity = 0;
    int c = 0;
    for (; c < total; c++) {
        // one answer for the whole warp: the lanes poll on their own and must not part ways here
        if (!__all_sync(0xffffffffu, sm100::mbar_wait(bars + c_stage * 8, c_parity, &s_abort, dev_err))) break;
        const int k0 = ch * CE;
        const int left8 = (K - k0) / 8 - lane;  // 16-byte pieces of the row from this lane's first one on
        const uint32_t st = ring + c_stage * kRingStageBytes + lane * 16;
        const uint32_t xa = rows + (uint32_t)(k0 + lane * 8) * 2;
#pragma unroll
        for (int u = 0; u < UNITS; u++) {
            const bool in = u * 32 < left8;
            const uint4 q0 = in ? lds128(st + u * 512) : zero4;
            const uint4 x0 = in ? lds128(xa + u * 512) : zero4;
            uint4 x1 = zero4;
            if (NT > 1 && in) x1 = lds128(xa + u * 512 + (uint32_t)K * 2);
            mma_diag(acc[0][0], x0.x, x1.x, x0.y, x1.y, q0.x, q0.y);
            mma_diag(acc[0][1], x0.z, x1.z, x0.w, x1.w, q0.z, q0.w);
            if (SWIGLU) {
                const uint4 q1 = in ? lds128(st + kRingStageBytes / 2 + u * 512) : zero4;
                mma_diag(acc[CH - 1][0], x0.x, x1.x, x0.y, x1.y, q1.x, q1.y);
                mma_diag(acc[CH - 1][1], x0.z, x1.z, x0.w, x1.w, q1.z, q1.w);
            }
        }
        __syncwarp();
        if (lane == 0 && issued < total) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the stage was read; a copy overwrites it
            issue_one();
        }
        if (++c_stage == stages) { c_stage = 0; c_parity ^= 1u; }
        if (++ch == nch) {
            ch = 0;
            // the column is folded: pick the diagonal, sum it over the lanes, finish and store
            float v[CH][NT];
#pragma unroll
            for (int cc = 0; cc < CH; cc++) {
                const bool mine = t == (g >> 1);
                const bool odd = g & 1;
                const float d0 = acc[cc][0][0] + acc[cc][1][0], d1 = acc[cc][0][1] + acc[cc][1][1];
                v[cc][0] = mine ? (odd ? d1 : d0) : 0.f;
                if (NT > 1) {
                    const float d2 = acc[cc][0][2] + acc[cc][1][2], d3 = acc[cc][0][3] + acc[cc][1][3];
                    v[cc][NT - 1] = mine ? (odd ? d3 : d2) : 0.f;
                }
#pragma unroll
                for (int s = 0; s < 2; s++)
#pragma unroll
                    for (int j = 0; j < 4; j++) acc[cc][s][j] = 0.f;
#pragma unroll
                for (int r = 0; r < NT; r++)
#pragma unroll
                    for (int o = 16; o >= 1; o >>= 1) v[cc][r] += __shfl_xor_sync(0xffffffffu, v[cc][r], o);
            }
            if (lane < mr) {
                float a = lane == 0 ? v[0][0] : v[0][NT - 1];
                if (SWIGLU) a = __fdividef(a, 1.0f + __expf(-a)) * (lane == 0 ? v[CH - 1][0] : v[CH - 1][NT - 1]);
                out[(size_t)(row0 + lane) * N + n0 + warp + col * kRingWarps] = __float2bfloat16_rn(a);
            }
            col++;
        }
    }
    if (c < total) {
        // a wait ran out (the error word is set): let this warp's copies in flight land, each wait bounded again,
        // before the block's shared memory can go to another block
        int pending = __shfl_sync(0xffffffffu, issued, 0) - c;
        for (; pending > 0; pending--) {
            const unsigned long long t0 = sm100::globaltimer_ns();
            while (!sm100::mbar_try_wait(bars + c_stage * 8, c_parity) && sm100::globaltimer_ns() - t0 < sm100::kWaitNs) {}
            if (++c_stage == stages) { c_stage = 0; c_parity ^= 1u; }
        }
    }
}

}  // namespace

// Largest token count of one forward for which the streaming path is used.  A
// token picks an expert at most once, so no expert then holds more rows than this.
// Above a couple of tokens the per-row arithmetic on CUDA cores costs more than the padding of tensor-core tiles.
int decode_tokens_threshold() {
    static int v = -1;
    if (v < 0) {
        const char *s = getenv("OMOE_DECODE_MAX_T");  // tuning knob, 0..8
        int t = s ? atoi(s) : 2;
        v = t < 0 ? 0 : (t > 8 ? 8 : t);
    }
    return v;
}

namespace {

template <bool SWIGLU, int RP>
cudaError_t launch_gemv(omoe_handle *h, const void *A, const void *W0, const void *W1, void *out, int K, int N,
                        cudaStream_t s) {
    auto kern = decode_gemv_kernel<SWIGLU, RP>;
    const size_t smem = (size_t)RP * K * 2;
    if (smem > 200 * 1024) return cudaErrorInvalidValue;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    int per_sm = 1;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kDecThreads, smem);
    if (e != cudaSuccess) return e;
    if (per_sm < 1) per_sm = 1;
    if (per_sm > 4) per_sm = 4;
    const int sms = h->sm_count > 0 ? h->sm_count : 148;
    return launch_ex(kern, dim3(sms * per_sm), dim3(kDecThreads), smem, s, h->pdl,
                     static_cast<const __nv_bfloat16 *>(A), static_cast<const __nv_bfloat16 *>(W0),
                     static_cast<const __nv_bfloat16 *>(W1), static_cast<__nv_bfloat16 *>(out), K, N, h->ex_counts,
                     h->ex_poffsets, h->e_local);
}

// Stages per warp of decode_mma_kernel beside `nt` token rows of length K: kRingStages, or 2 when the rows leave
// less room; 0 when not even two fit.
int mma_stages(int nt, int K) {
    const long budget = 224 * 1024 - kRingHeader - (long)nt * K * 2;
    long st = budget / ((long)kRingWarps * kRingStageBytes);
    if (st > kRingStages) st = kRingStages;
    return st < 2 ? 0 : (int)st;
}

template <bool SWIGLU, int NT>
cudaError_t launch_mma(omoe_handle *h, const void *A, const void *W0, const void *W1, void *out, int K, int N,
                       cudaStream_t s) {
    auto kern = decode_mma_kernel<SWIGLU, NT>;
    const int stages = mma_stages(NT, K);
    const size_t smem = kRingHeader + (size_t)kRingWarps * stages * kRingStageBytes + (size_t)NT * K * 2;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    const int sms = h->sm_count > 0 ? h->sm_count : 148;
    return launch_ex(kern, dim3(sms), dim3(kRingThreads), smem, s, h->pdl, static_cast<const __nv_bfloat16 *>(A),
                     static_cast<const __nv_bfloat16 *>(W0), static_cast<const __nv_bfloat16 *>(W1),
                     static_cast<__nv_bfloat16 *>(out), K, N, h->ex_counts, h->ex_poffsets, h->e_local, stages,
                     h->dev_err);
}

// OMOE_DECODE_MMA=0 keeps the CUDA-core kernels (decode_gemv_kernel)
bool mma_enabled() {
    static int v = -1;
    if (v < 0) {
        const char *s = getenv("OMOE_DECODE_MMA");
        v = (s && atoi(s) == 0) ? 0 : 1;
    }
    return v != 0;
}

template <int RP>
cudaError_t launch_both(omoe_handle *h, int T, cudaStream_t s, int *n, cudaEvent_t mid) {
    const int d = h->cfg.d_model, dff = h->cfg.d_ff;
    const int sms = h->sm_count > 0 ? h->sm_count : 148;
    // decode_mma_kernel: one or two token rows, and every expert with rows gets blocks of its own
    constexpr int NT = RP <= 1 ? 1 : 2;
    const bool mma = mma_enabled() && RP <= 2 && (long)T * h->cfg.top_k <= sms && mma_stages(NT, d) && mma_stages(NT, dff);
    cudaError_t e = mma ? launch_mma<true, NT>(h, h->xp, h->w_gate, h->w_up, h->hbuf, d, dff, s)
                        : launch_gemv<true, RP>(h, h->xp, h->w_gate, h->w_up, h->hbuf, d, dff, s);
    if (e != cudaSuccess) return e;
    (*n)++;
    if (mid) cudaEventRecord(mid, s);
    e = mma ? launch_mma<false, NT>(h, h->hbuf, h->w_down, nullptr, h->yp, dff, d, s)
            : launch_gemv<false, RP>(h, h->hbuf, h->w_down, nullptr, h->yp, dff, d, s);
    if (e == cudaSuccess) (*n)++;
    return e;
}

}  // namespace

cudaError_t launch_experts_decode(omoe_handle *h, int T, cudaStream_t s, int *n, cudaEvent_t mid) {
    // the streaming kernels keep RP token rows of the longer reduction in shared memory; layers too wide for
    // that take the tensor-core kernels, as steps with more tokens do
    const int rp = T <= 1 ? 1 : (T <= 2 ? 2 : 4);
    const int kmax = h->cfg.d_model > h->cfg.d_ff ? h->cfg.d_model : h->cfg.d_ff;
    if ((size_t)rp * kmax * 2 > 200 * 1024) return launch_experts_bf16(h, s, n, mid, (long)T * h->cfg.top_k);
    if (T <= 1) return launch_both<1>(h, T, s, n, mid);
    if (T <= 2) return launch_both<2>(h, T, s, n, mid);
    return launch_both<4>(h, T, s, n, mid);
}

}  // namespace omoe
