// Prefix sums over the per-block expert histograms of the router (one block): shared by the scan kernel of the
// one-GPU path and the fused scan + count-exchange kernel of the expert-parallel path.
#pragma once

#include "common.cuh"

namespace omoe {

// One block.  Histograms are stored expert-major, block_counts[e][b], so a warp
// reads one expert's row with coalesced loads.  Warp w walks experts w, w+32,
// ...: block_base[e][b] becomes the exclusive prefix over blocks b and the
// total goes to counts[e].  Then offsets (exact), poffsets (each expert rounded
// up to kRowAlign) and the expert of every 128-row tile.
// s_cnt [kMaxExperts], s_poff [kMaxExperts + 1]: shared memory of the calling block (any multiple of 32 threads).
__device__ __forceinline__ void scan_body(const int32_t *__restrict__ block_counts, int32_t *__restrict__ block_base,
                                          int n_blocks, int E, int32_t *__restrict__ counts,
                                          int32_t *__restrict__ offsets, int32_t *__restrict__ poffsets,
                                          int32_t *__restrict__ tile_expert, int max_tiles, int32_t *s_cnt,
                                          int32_t *s_poff) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int e = warp; e < E; e += nwarps) {
        const int32_t *row = block_counts + (size_t)e * n_blocks;
        int32_t *out = block_base + (size_t)e * n_blocks;
        int run = 0;
        if ((n_blocks & 3) == 0) {
            // four blocks per lane and step (16-byte loads and stores): a quarter of the dependent round trips
            // to L2, which are all this kernel's time
#pragma unroll 2
            for (int b0 = 0; b0 < n_blocks; b0 += 128) {
                const int b = b0 + lane * 4;
                int4 c4 = make_int4(0, 0, 0, 0);
                if (b < n_blocks) c4 = *reinterpret_cast<const int4 *>(row + b);
                const int sum4 = c4.x + c4.y + c4.z + c4.w;
                int inc = sum4;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    int v = __shfl_up_sync(0xffffffffu, inc, o);
                    if (lane >= o) inc += v;
                }
                if (b < n_blocks) {
                    const int base = run + inc - sum4;
                    *reinterpret_cast<int4 *>(out + b) = make_int4(base, base + c4.x, base + c4.x + c4.y, base + c4.x + c4.y + c4.z);
                }
                run += __shfl_sync(0xffffffffu, inc, 31);
            }
            if (lane == 0) s_cnt[e] = run;
            continue;
        }
#pragma unroll 4
        for (int b0 = 0; b0 < n_blocks; b0 += 32) {
            int b = b0 + lane;
            int c = (b < n_blocks) ? row[b] : 0;
            int inc = c;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                int v = __shfl_up_sync(0xffffffffu, inc, o);
                if (lane >= o) inc += v;
            }
            if (b < n_blocks) out[b] = run + inc - c;
            run += __shfl_sync(0xffffffffu, inc, 31);
        }
        if (lane == 0) s_cnt[e] = run;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int off = 0, poff = 0;
        for (int e = 0; e < E; e++) {
            int c = s_cnt[e];
            counts[e] = c;
            offsets[e] = off;
            poffsets[e] = poff;
            s_poff[e] = poff;
            off += c;
            poff += (c + kRowAlign - 1) / kRowAlign * kRowAlign;
        }
        offsets[E] = off;
        poffsets[E] = poff;
        s_poff[E] = poff;
    }
    __syncthreads();
    const int n_tiles = s_poff[E] / kRowAlign;
    for (int i = threadIdx.x; i < max_tiles; i += blockDim.x) {
        int ex = -1;
        if (i < n_tiles) {
            int row = i * kRowAlign;
            ex = 0;
            while (ex + 1 < E && s_poff[ex + 1] <= row) ex++;
        }
        tile_expert[i] = ex;
    }
}


}  // namespace omoe
