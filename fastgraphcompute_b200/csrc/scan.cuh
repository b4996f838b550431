// In-place exclusive scan of an int32 array in three kernels (tile sums, scan of the tile
// sums by one block, per-tile scan with offset).  The length may live in device memory
// (*n_ptr + n_add) so that a scan can follow a kernel that decides the size, without a host
// round trip: launch enough blocks for the largest possible length, surplus blocks return.
#pragma once
#include "fgc_common.cuh"

namespace fgc {

constexpr int kScanTile = 2048;  // elements per block

__device__ __forceinline__ int scan_length(const int *n_ptr, int n_add)
{
    return n_ptr ? *n_ptr + n_add : n_add;
}


static __global__ void __launch_bounds__(256)
k_scan_tile_sums(const int *__restrict__ counts, const int *__restrict__ n_ptr, int n_add,
                 int *__restrict__ blocksums)
{
    const int n = scan_length(n_ptr, n_add);
    const int base = blockIdx.x * kScanTile;
    if (base >= n) return;
    int s = 0;
#pragma unroll
    for (int k = 0; k < kScanTile / 256; k++) {
        const int i = base + k * 256 + threadIdx.x;
        if (i < n) s += counts[i];
    }
    __shared__ int ws[8];
    s = __reduce_add_sync(FGC_FULL_MASK, s);
    if ((threadIdx.x & 31) == 0) ws[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        int t = 0;
        for (int k = 0; k < 8; k++) t += ws[k];
        blocksums[blockIdx.x] = t;
    }
}

// Tile sums and, by the CTA that finishes last (a ticket counter in *ticket, which must be zero
// at launch and is zero again afterwards; no waiting), the exclusive scan of the tile sums: the
// first two of the three scan kernels in one launch.  Every CTA of the grid takes a ticket,
// also those beyond the array's end.
static __global__ void __launch_bounds__(256)
k_scan_tile_sums_top(const int *__restrict__ counts, const int *__restrict__ n_ptr, int n_add,
                     int *__restrict__ blocksums, int *ticket)
{
    chain_wait();
    chain_release();
    const int n = scan_length(n_ptr, n_add);
    const int base = blockIdx.x * kScanTile;
    __shared__ int ws[8];
    __shared__ int s_last;
    if (base < n) {
        int s = 0;
#pragma unroll
        for (int k = 0; k < kScanTile / 256; k++) {
            const int i = base + k * 256 + threadIdx.x;
            if (i < n) s += counts[i];
        }
        s = __reduce_add_sync(FGC_FULL_MASK, s);
        if ((threadIdx.x & 31) == 0) ws[threadIdx.x >> 5] = s;
        __syncthreads();
        if (threadIdx.x == 0) {
            int t = 0;
            for (int k = 0; k < 8; k++) t += ws[k];
            blocksums[blockIdx.x] = t;
        }
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = atomicAdd(ticket, 1) == (int)gridDim.x - 1;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (threadIdx.x == 0) *ticket = 0;
    // exclusive scan of the tile sums, 256 at a time
    const int n_tiles = (n + kScanTile - 1) / kScanTile;
    __shared__ int carry;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    for (int b0 = 0; b0 < n_tiles; b0 += 256) {
        const int i = b0 + threadIdx.x;
        const int x = i < n_tiles ? ((volatile int *)blocksums)[i] : 0;
        int incl = x;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(FGC_FULL_MASK, incl, o);
            if ((threadIdx.x & 31) >= o) incl += t;
        }
        if ((threadIdx.x & 31) == 31) ws[threadIdx.x >> 5] = incl;
        __syncthreads();
        int warp_off = 0;
        for (int k = 0; k < (int)(threadIdx.x >> 5); k++) warp_off += ws[k];
        const int c = carry;
        if (i < n_tiles) blocksums[i] = c + warp_off + incl - x;
        __syncthreads();
        if (threadIdx.x == 255) carry = c + warp_off + incl;
        __syncthreads();
    }
}

// Single block: exclusive scan of the tile sums.
static __global__ void __launch_bounds__(1024)
k_scan_block_sums(int *__restrict__ blocksums, const int *__restrict__ n_ptr, int n_add)
{
    const int n = (scan_length(n_ptr, n_add) + kScanTile - 1) / kScanTile;
    __shared__ int ws[32];
    __shared__ int carry;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    for (int base = 0; base < n; base += 1024) {
        const int i = base + threadIdx.x;
        const int x = i < n ? blocksums[i] : 0;
        int incl = x;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(FGC_FULL_MASK, incl, o);
            if ((threadIdx.x & 31) >= o) incl += t;
        }
        if ((threadIdx.x & 31) == 31) ws[threadIdx.x >> 5] = incl;
        __syncthreads();
        if (threadIdx.x < 32) {
            int y = ws[threadIdx.x];
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(FGC_FULL_MASK, y, o);
                if (threadIdx.x >= o) y += t;
            }
            ws[threadIdx.x] = y;
        }
        __syncthreads();
        const int warp_off = (threadIdx.x >> 5) ? ws[(threadIdx.x >> 5) - 1] : 0;
        const int c = carry;
        if (i < n) blocksums[i] = c + warp_off + incl - x;
        __syncthreads();
        if (threadIdx.x == 1023) carry = c + warp_off + incl;
        __syncthreads();
    }
}

static __global__ void __launch_bounds__(256)
k_scan_apply(int *__restrict__ counts, const int *__restrict__ n_ptr, int n_add,
             const int *__restrict__ blocksums)
{
    chain_wait();
    chain_release();
    const int n = scan_length(n_ptr, n_add);
    const int base = blockIdx.x * kScanTile;
    if (base >= n) return;
    constexpr int PER = kScanTile / 256;
    int x[PER];
    int s = 0;
    const int first = base + threadIdx.x * PER;
#pragma unroll
    for (int k = 0; k < PER; k++) {
        x[k] = first + k < n ? counts[first + k] : 0;
        s += x[k];
    }
    int incl = s;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(FGC_FULL_MASK, incl, o);
        if ((threadIdx.x & 31) >= o) incl += t;
    }
    __shared__ int ws[8];
    if ((threadIdx.x & 31) == 31) ws[threadIdx.x >> 5] = incl;
    __syncthreads();
    int off = blocksums[blockIdx.x];
    for (int k = 0; k < (int)(threadIdx.x >> 5); k++) off += ws[k];
    int run = off + incl - s;
#pragma unroll
    for (int k = 0; k < PER; k++) {
        if (first + k < n) counts[first + k] = run;
        run += x[k];
    }
}


}  // namespace fgc
