// Ascending in-place sort of a short int32 segment by one warp (keys are distinct).
//   up to 32 keys            bitonic network in registers, one key per lane
//   up to kWarpSortMaxShared bitonic network in shared memory (caller provides the buffer)
//   longer                   bitonic sort by the warp, in place in global memory (rare)
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
        // Bitonic sort in its all-ascending form, in place in global memory, by this one warp:
        // O(n log^2 n / 32) steps (a hub point of a reverse neighbour graph can have a segment of
        // 10^5 entries or more; a quadratic method would keep the GPU busy for minutes).  The
        // sequence is treated as padded to a power of two with +infinity; a compare-exchange
        // whose upper partner lies in the padding never swaps, so it is simply skipped.
        int P = 1;
        while (P < n) P <<= 1;
        for (int k = 2; k <= P; k <<= 1) {
            // flip: element i of a block of k against its mirror image
            for (int t = lane; t < P / 2; t += 32) {
                const int half = k >> 1, blk = t / half, off = t - blk * half;
                const int a = blk * k + off, b = blk * k + (k - 1 - off);
                if (b < n) {
                    const int ka = seg[a], kb = seg[b];
                    if (ka > kb) { seg[a] = kb; seg[b] = ka; }
                }
            }
            __syncwarp();
            for (int j = k >> 2; j > 0; j >>= 1) {
                for (int t = lane; t < P / 2; t += 32) {
                    const int a = 2 * j * (t / j) + (t % j), b = a + j;
                    if (b < n) {
                        const int ka = seg[a], kb = seg[b];
                        if (ka > kb) { seg[a] = kb; seg[b] = ka; }
                    }
                }
                __syncwarp();
            }
        }
    }
}

}  // namespace fgc
