// Expert products for a handful of tokens (decode steps): weight-streaming
// kernels.  With one or two rows per expert the tensor-core tiles of
// experts_sm100.cu would be 99 % padding and, worse, there are too few tiles to
// keep every SM's share of HBM busy.  Here the work item is one output column
// (one weight row, or a gate/up pair of rows): a pair of warps streams it once
// with 16-byte loads, 512 contiguous bytes per warp and load, and folds it
// against the expert's token rows held in shared memory, so the items spread
// evenly over all SMs and the kernels run at HBM speed.  Two kernels: one that
// folds on the CUDA cores (any K, 1-4 token rows per pass) and one that folds
// with warp-level MMAs and keeps requesting memory while a column is reduced
// (K a multiple of 512, one or two rows; the default where it applies).  Same
// arithmetic points as the tensor-core path (bf16 operands, fp32 accumulate, h
// and yp rounded to bf16); they replace the same reference calls
// (LlamaMLPLayer.java:117-123).
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
// column its warps stop requesting memory while they reduce.  This kernel keeps its access pattern (a warp reads
// 512 contiguous bytes of ONE weight row per load, full 128-byte lines) and hands the arithmetic to
// `mma.sync.m16n8k16`: lane (g, t) (g = lane/4, t = lane%4) holds 8 consecutive k of the row, which the MMA takes
// as the B operand's k slots {2t, 2t+1, 2t+8, 2t+9} of "column" g (two MMAs per 16 bytes); the same lane supplies
// the token's values at the same k as row g (first token) and row g+8 (second token) of the A operand.  Then
// D[g][g] is the lane group's share of the first token's dot product and D[g+8][g] of the second: the diagonal is
// what is kept, summed over g at the end of a weight row.  The products off the diagonal are wasted work on a
// pipe that has nothing else to do.  One load, one or two shared-memory loads and two MMAs per 16 bytes.
//
// Work split: a block works for ONE expert (the blocks are dealt evenly over the experts that have rows), so the
// expert's token rows stay in shared memory for the whole launch.  Its 8 warp pairs take the output columns
// round-robin, each warp of a pair one half of K, and every warp runs a register ring of loads that continues
// across columns: the next columns' weights are already requested while a column is reduced.  The second warp of
// a pair leaves its partial sums in one of four shared-memory slots (full/empty mbarriers, bounded waits); the
// first adds them to its own one column late, applies SiLU·mul and stores.
constexpr int kMmaWarps = 16;
constexpr int kMmaThreads = kMmaWarps * 32;
constexpr int kMmaPairs = kMmaWarps / 2;
constexpr int kMmaSlots = 4;
constexpr int kMmaHeader = 4096;  // mbarriers: [pairs][slots] full, then empty (512 B); partial sums from 1024

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

// NT: token rows folded (1 or 2); an expert never holds more when the step has at most NT tokens
template <bool SWIGLU, int NT>
__global__ void __launch_bounds__(kMmaThreads, 1)
decode_mma_kernel(const __nv_bfloat16 *__restrict__ A, const __nv_bfloat16 *__restrict__ W0,
                  const __nv_bfloat16 *__restrict__ W1, __nv_bfloat16 *__restrict__ out, int K, int N,
                  const int32_t *__restrict__ counts, const int32_t *__restrict__ poffsets, int El,
                  int32_t *dev_err) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ int s_active[kMaxExperts];
    __shared__ int s_n_active;
    __shared__ int s_abort;
    constexpr int CH = SWIGLU ? 2 : 1;
    constexpr int U = SWIGLU ? 6 : 12;  // 512-byte pieces per operand in flight per warp

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int pair = warp >> 1, half = warp & 1;
    const uint32_t smem0 = sm100::smem_u32(smem_raw);
    const uint32_t bar_full = smem0 + pair * kMmaSlots * 8;
    const uint32_t bar_empty = smem0 + 256 + pair * kMmaSlots * 8;
    // partial sums: [pair][slot][half][CH][NT]
    float *part = reinterpret_cast<float *>(smem_raw + 1024) + (size_t)pair * kMmaSlots * 2 * CH * NT;
    __nv_bfloat16 *rows_p = reinterpret_cast<__nv_bfloat16 *>(smem_raw + kMmaHeader);  // [NT][K]
    const uint32_t rows = smem0 + kMmaHeader;

    pdl_trigger();
    if (tid < kMmaPairs * kMmaSlots) {
        sm100::mbar_init(smem0 + tid * 8, 1);
        sm100::mbar_init(smem0 + 256 + tid * 8, 1);
    }
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
    const int nu = K / 512;                                       // 512-byte pieces of half a weight row
    const int cnt = n1 - n0 > pair ? (n1 - n0 - pair + kMmaPairs - 1) / kMmaPairs : 0;  // this pair's columns
    const int total = cnt * nu;
    const size_t first = ((size_t)e * N + n0 + pair) * K + (size_t)half * (K / 2) + lane * 8;
    const uint4 *lp0 = reinterpret_cast<const uint4 *>(W0 + first);
    const uint4 *lp1 = SWIGLU ? reinterpret_cast<const uint4 *>(W1 + first) : nullptr;
    const int row_jump = (kMmaPairs * K * 2 - K) / 16;             // from the end of a half row to the next column's
    uint32_t xaddr = rows + (uint32_t)(half * (K / 2) + lane * 8) * 2;

    float acc[CH][2][4];
#pragma unroll
    for (int c = 0; c < CH; c++)
#pragma unroll
        for (int s = 0; s < 2; s++)
#pragma unroll
            for (int j = 0; j < 4; j++) acc[c][s][j] = 0.f;

    // first warp of the pair: column j of this pair is complete in slot j % kMmaSlots; finish and store it
    auto combine = [&](int j) -> bool {
        const int b = j & (kMmaSlots - 1);
        if (!__all_sync(0xffffffffu, sm100::mbar_wait(bar_full + b * 8, (uint32_t)(j / kMmaSlots) & 1u, &s_abort, dev_err)))
            return false;
        __syncwarp();
        if (lane < mr) {
            const float *p0 = part + (size_t)(b * 2 + 0) * CH * NT, *p1 = part + (size_t)(b * 2 + 1) * CH * NT;
            float v = p0[lane] + p1[lane];
            if (SWIGLU) v = __fdividef(v, 1.0f + __expf(-v)) * (p0[NT + lane] + p1[NT + lane]);
            out[(size_t)(row0 + lane) * N + n0 + pair + j * kMmaPairs] = __float2bfloat16_rn(v);
        }
        __syncwarp();
        if (lane == 0) sm100::mbar_arrive(bar_empty + b * 8);
        return true;
    };
    // this warp's half of column i is folded: pick the diagonal, sum it over the lanes, leave it in the slot
    auto row_end = [&](int i) -> bool {
        const int b = i & (kMmaSlots - 1);
        float v[CH][NT];
#pragma unroll
        for (int c = 0; c < CH; c++) {
            const bool mine = t == (g >> 1);
            const bool odd = g & 1;
            const float d0 = acc[c][0][0] + acc[c][1][0], d1 = acc[c][0][1] + acc[c][1][1];
            v[c][0] = mine ? (odd ? d1 : d0) : 0.f;
            if (NT > 1) {
                const float d2 = acc[c][0][2] + acc[c][1][2], d3 = acc[c][0][3] + acc[c][1][3];
                v[c][NT - 1] = mine ? (odd ? d3 : d2) : 0.f;
            }
#pragma unroll
            for (int s = 0; s < 2; s++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[c][s][j] = 0.f;
#pragma unroll
            for (int r = 0; r < NT; r++)
#pragma unroll
                for (int o = 16; o >= 1; o >>= 1) v[c][r] += __shfl_xor_sync(0xffffffffu, v[c][r], o);
        }
        if (half == 1 && i >= kMmaSlots &&
            !__all_sync(0xffffffffu, sm100::mbar_wait(bar_empty + b * 8, (uint32_t)(i / kMmaSlots - 1) & 1u, &s_abort, dev_err)))
            return false;
        if (lane == 0) {
            float *p = part + (size_t)(b * 2 + half) * CH * NT;
#pragma unroll
            for (int c = 0; c < CH; c++)
#pragma unroll
                for (int r = 0; r < NT; r++) p[c * NT + r] = v[c][r];
            if (half == 1) sm100::mbar_arrive(bar_full + b * 8);
        }
        if (half == 0 && i >= 1) return combine(i - 1);
        return true;
    };

    int l_left = nu, c_left = nu, c_row = 0, loaded = 0, done = 0;
    uint4 q0[U], q1[SWIGLU ? U : 1];
    auto load_unit = [&](uint4 &a, uint4 &b) {
        a = ld_stream(lp0);
        lp0 += 32;
        if (SWIGLU) { b = ld_stream(lp1); lp1 += 32; }
        if (--l_left == 0) {
            l_left = nu;
            lp0 += row_jump;
            if (SWIGLU) lp1 += row_jump;
        }
        loaded++;
    };
    auto fold_unit = [&](const uint4 &a, const uint4 &b) -> bool {
        const uint4 x0 = lds128(xaddr);
        uint4 x1 = make_uint4(0u, 0u, 0u, 0u);
        if (NT > 1) x1 = lds128(xaddr + (uint32_t)K * 2);
        xaddr += 512;
        mma_diag(acc[0][0], x0.x, x1.x, x0.y, x1.y, a.x, a.y);
        mma_diag(acc[0][1], x0.z, x1.z, x0.w, x1.w, a.z, a.w);
        if (SWIGLU) {
            mma_diag(acc[CH - 1][0], x0.x, x1.x, x0.y, x1.y, b.x, b.y);
            mma_diag(acc[CH - 1][1], x0.z, x1.z, x0.w, x1.w, b.z, b.w);
        }
        done++;
        if (--c_left == 0) {
            c_left = nu;
            xaddr -= (uint32_t)nu * 512;
            return row_end(c_row++);
        }
        return true;
    };

#pragma unroll
    for (int u = 0; u < U; u++)
        if (u < total) load_unit(q0[u], q1[SWIGLU ? u : 0]);
    // the token rows come in while the first weights are on their way
    for (int i = tid; i < NT * (K / 8); i += kMmaThreads) {
        int r = i / (K / 8), c = i % (K / 8);
        // a missing second row is read as zeros
        reinterpret_cast<uint4 *>(rows_p + (size_t)r * K)[c] =
            r < mr ? reinterpret_cast<const uint4 *>(A + (size_t)(row0 + r) * K)[c] : make_uint4(0u, 0u, 0u, 0u);
    }
    __syncthreads();
    while (loaded + U <= total) {  // whole rounds of the ring: no bounds to check
#pragma unroll
        for (int u = 0; u < U; u++) {
            if (!fold_unit(q0[u], q1[SWIGLU ? u : 0])) return;
            load_unit(q0[u], q1[SWIGLU ? u : 0]);
        }
    }
#pragma unroll
    for (int u = 0; u < U; u++) {
        if (done < total) {
            if (!fold_unit(q0[u], q1[SWIGLU ? u : 0])) return;
            if (loaded < total) load_unit(q0[u], q1[SWIGLU ? u : 0]);
        }
    }
#pragma unroll
    for (int u = 0; u < U; u++)
        if (done < total && !fold_unit(q0[u], q1[SWIGLU ? u : 0])) return;
    if (half == 0 && cnt > 0) combine(cnt - 1);
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

// Shared memory of decode_mma_kernel for `nt` token rows of length K; 0 when it does not fit.
size_t mma_smem(int nt, int K) {
    const size_t need = kMmaHeader + (size_t)nt * K * 2;
    return need <= 224 * 1024 ? need : 0;
}

template <bool SWIGLU, int NT>
cudaError_t launch_mma(omoe_handle *h, const void *A, const void *W0, const void *W1, void *out, int K, int N,
                       cudaStream_t s) {
    auto kern = decode_mma_kernel<SWIGLU, NT>;
    const size_t smem = mma_smem(NT, K);
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    const int sms = h->sm_count > 0 ? h->sm_count : 148;
    return launch_ex(kern, dim3(sms), dim3(kMmaThreads), smem, s, h->pdl, static_cast<const __nv_bfloat16 *>(A),
                     static_cast<const __nv_bfloat16 *>(W0), static_cast<const __nv_bfloat16 *>(W1),
                     static_cast<__nv_bfloat16 *>(out), K, N, h->ex_counts, h->ex_poffsets, h->e_local, h->dev_err);
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
    // decode_mma_kernel: one or two token rows, every expert with rows gets blocks of its own, and a warp walks
    // half a weight row in 512-byte pieces
    constexpr int NT = RP <= 1 ? 1 : 2;
    const bool mma = mma_enabled() && RP <= 2 && (long)T * h->cfg.top_k <= sms && d % 512 == 0 && dff % 512 == 0 &&
                     mma_smem(NT, d) && mma_smem(NT, dff);
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
