// Ascending in-place sort of a short int32 segment by one warp (keys are distinct).
//   up to 32 keys            bitonic network in registers, one key per lane
//   up to kWarpSortMaxShared bitonic network in shared memory (caller provides the buffer)
//   longer                   selection sort by the warp, in place (rare)
#pragma once
#include "fgc_common.cuh"

namespace fgc {

constexpr int kWarpSortMaxShared = 512;

__device__ __forceinline__ void warp_sort_segment(int *seg, int n, int *keys, int lane)
{
    if (n <= 1) return;
    if (n <= 32) {
        int key = lane < n ? seg[lane] : 0x7fffffff;
#pragma unroll
        for (int k = 2; k <= 32; k <<= 1)
#pragma unroll
            for (int j = k >> 1; j > 0; j >>= 1) {
                const int other = __shfl_xor_sync(FGC_FULL_MASK, key, j);
                const bool up = (lane & k) == 0;          // ascending block
                const bool lower = (lane & j) == 0;       // lower partner keeps the smaller key
                key = (lower == up) ? min(key, other) : max(key, other);
            }
        if (lane < n) seg[lane] = key;
    } else if (n <= kWarpSortMaxShared) {
        int P = 64;
        while (P < n) P <<= 1;
        for (int t = lane; t < P; t += 32) keys[t] = t < n ? seg[t] : 0x7fffffff;
        __syncwarp();
        for (int k = 2; k <= P; k <<= 1)
            for (int j = k >> 1; j > 0; j >>= 1) {
                for (int t = lane; t < P / 2; t += 32) {
                    // t-th compare-exchange of this stage: partner indices a < b = a + j
                    const int a = 2 * j * (t / j) + (t % j), b = a + j;
                    const int ka = keys[a], kb = keys[b];
                    const bool up = (a & k) == 0;
                    if ((ka > kb) == up) { keys[a] = kb; keys[b] = ka; }
                }
                __syncwarp();
            }
        for (int t = lane; t < n; t += 32) seg[t] = keys[t];
        __syncwarp();
    } else {
        for (int p = 0; p < n - 1; p++) {
            int best = 0x7fffffff, where = -1;
            for (int t = p + lane; t < n; t += 32) {
                const int v = seg[t];
                if (v < best) { best = v; where = t; }
            }
            const int gmin = __reduce_min_sync(FGC_FULL_MASK, best);
            const unsigned who = __ballot_sync(FGC_FULL_MASK, best == gmin);
            if (lane == __ffs(who) - 1 && where != p) { seg[where] = seg[p]; seg[p] = gmin; }
            __syncwarp();
        }
    }
}

}  // namespace fgc
