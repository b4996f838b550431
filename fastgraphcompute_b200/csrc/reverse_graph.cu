// Reverse neighbour graph: for every point n the list of (row i, slot k) pairs with
// idx[i,k] == n, as a CSR structure whose segments are sorted by i*K + k.
//
// The backward passes scatter through the neighbour index: point n receives a term from
// every row that lists n as a neighbour.  The reference does this with one fp32 atomicAdd
// per (row, slot, coordinate) (extensions/binned_select_knn_grad_cuda_kernel.cu:58-88), so
// its sums depend on the order in which the atomics land.  With the reverse graph the same
// sums become gathers over a sorted segment, reduced in a fixed order: no float atomics and
// bit-identical results from run to run.
//
// Build: count (integer atomics), exclusive scan, fill (integer atomics for the position
// inside a segment -- that order is arbitrary), then every segment is sorted so that
// nothing of the arbitrary order survives.
#include "reverse_graph.cuh"
#include "segsort.cuh"

namespace fgc {

__global__ void __launch_bounds__(256)
k_rev_count(const int64_t *__restrict__ idx, int64_t total, int n_vert, int *__restrict__ counts)
{
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
        const int64_t n = idx[e];
        if (n >= 0 && n < n_vert) atomicAdd(counts + n, 1);
    }
}

__global__ void __launch_bounds__(256)
k_rev_fill(const int64_t *__restrict__ idx, int64_t total, int n_vert,
           const int *__restrict__ offsets, int *__restrict__ cursor, int *__restrict__ entries)
{
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
        const int64_t n = idx[e];
        if (n >= 0 && n < n_vert) entries[offsets[n] + atomicAdd(cursor + n, 1)] = (int)e;
    }
}

constexpr int kSortWarps = 4;

// One warp per segment: ascending sort of the entries (keys are distinct).
__global__ void __launch_bounds__(kSortWarps * 32)
k_rev_sort(const int *__restrict__ offsets, int *__restrict__ entries, int n_vert)
{
    __shared__ int s_keys[kSortWarps][kWarpSortMaxShared];
    const int lane = threadIdx.x & 31;
    const int wib = threadIdx.x >> 5;
    const int n = blockIdx.x * kSortWarps + wib;
    if (n >= n_vert) return;
    const int beg = offsets[n], deg = offsets[n + 1] - beg;
    warp_sort_segment(entries + beg, deg, s_keys[wib], lane);
}

// --- kNN backward over the reverse graph -------------------------------------------------

constexpr int kBwdSortedWarps = 8;

// One warp per point n:  G[n] = -sum_k 2 g[n,k] (x[idx[n,k]] - x[n])            (own row)
//                               + sum_{(i,k): idx[i,k]=n} 2 g[i,k] (x[n] - x[i])  (reverse segment)
// Lanes stride over the slots / the sorted segment, partial sums are combined by a fixed
// butterfly: the result does not depend on anything but the inputs.
template <int D>
__global__ void __launch_bounds__(kBwdSortedWarps * 32)
k_knn_bwd_sorted(const float *__restrict__ grad_distsq, const int64_t *__restrict__ idx,
                 const float *__restrict__ coords, int n_vert, int K, int n_coords_rt,
                 const int *__restrict__ offsets, const int *__restrict__ entries,
                 float *__restrict__ out)
{
    const int lane = threadIdx.x & 31;
    const int n = blockIdx.x * kBwdSortedWarps + (threadIdx.x >> 5);
    if (n >= n_vert) return;
    const int nc = D > 0 ? D : n_coords_rt;
    constexpr int DM = D > 0 ? D : 1;
    const int beg = offsets[n], end = offsets[n + 1];
    for (int v0 = 0; v0 < nc; v0 += DM) {
        float xn[DM], acc[DM];
#pragma unroll
        for (int v = 0; v < DM; v++) { xn[v] = __ldg(coords + (size_t)n * nc + v0 + v); acc[v] = 0.f; }
        for (int k = lane; k < K; k += 32) {
            const int64_t m = idx[(size_t)n * K + k];
            if (m >= 0 && m < n_vert) {
                const float g2 = 2.f * grad_distsq[(size_t)n * K + k];
#pragma unroll
                for (int v = 0; v < DM; v++) acc[v] -= g2 * (__ldg(coords + (size_t)m * nc + v0 + v) - xn[v]);
            }
        }
        for (int t = beg + lane; t < end; t += 32) {
            const int src = entries[t];
            const int i = src / K;
            const float g2 = 2.f * grad_distsq[src];
#pragma unroll
            for (int v = 0; v < DM; v++) acc[v] += g2 * (xn[v] - __ldg(coords + (size_t)i * nc + v0 + v));
        }
#pragma unroll
        for (int v = 0; v < DM; v++) {
            float s = acc[v];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(FGC_FULL_MASK, s, o);
            if (lane == 0) out[(size_t)n * nc + v0 + v] = s;
        }
    }
}

}  // namespace fgc

extern "C" size_t fgc_reverse_graph_bytes(int64_t n_vert, int32_t K)
{
    if (n_vert < 0 || K < 1 || n_vert * (int64_t)K > 0x7fffffff) return 0;
    return fgc::reverse_graph_layout(n_vert, K).total;
}

extern "C" int fgc_build_reverse_graph(const int64_t *idx, int64_t n_vert, int32_t K, void *rgraph,
                                       size_t rgraph_bytes, fgc_stream_t stream)
{
    FGC_NVTX("fgc_build_reverse_graph");
    using namespace fgc;
    if (n_vert < 0 || K < 1) return FGC_ERR_BAD_ARGUMENT;
    if (n_vert * (int64_t)K > 0x7fffffff) return FGC_ERR_TOO_LARGE;
    const ReverseGraphLayout L = reverse_graph_layout(n_vert, K);
    if (!rgraph || rgraph_bytes < L.total || ((uintptr_t)rgraph & 255)) return FGC_ERR_WORKSPACE;
    if (n_vert == 0) return FGC_OK;
    if (!idx) return FGC_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    char *ws = (char *)rgraph;
    int *offsets = (int *)(ws + L.offsets);
    int *cursor = (int *)(ws + L.cursor);
    int *blocksums = (int *)(ws + L.blocksums);
    int *entries = (int *)(ws + L.entries);
    const int n = (int)n_vert;
    const int64_t total = n_vert * K;
    // offsets and cursor are adjacent: one clear for both
    FGC_RETURN_IF_CUDA(cudaMemsetAsync(offsets, 0, L.blocksums - L.offsets, s));
    int64_t blocks = ceil_div64(total, 256 * 4);
    if (blocks > fgc::sm_count() * 16) blocks = fgc::sm_count() * 16;
    k_rev_count<<<(unsigned)blocks, 256, 0, s>>>(idx, total, n, offsets);
    FGC_CHECK_LAUNCH();
    const int scan_blocks = (int)ceil_div64(n_vert + 1, kScanTile);
    k_scan_tile_sums<<<scan_blocks, 256, 0, s>>>(offsets, nullptr, n + 1, blocksums);
    FGC_CHECK_LAUNCH();
    k_scan_block_sums<<<1, 1024, 0, s>>>(blocksums, nullptr, n + 1);
    FGC_CHECK_LAUNCH();
    k_scan_apply<<<scan_blocks, 256, 0, s>>>(offsets, nullptr, n + 1, blocksums);
    FGC_CHECK_LAUNCH();
    k_rev_fill<<<(unsigned)blocks, 256, 0, s>>>(idx, total, n, offsets, cursor, entries);
    FGC_CHECK_LAUNCH();
    k_rev_sort<<<(unsigned)((n + kSortWarps - 1) / kSortWarps), kSortWarps * 32, 0, s>>>(offsets, entries, n);
    FGC_CHECK_LAUNCH();
    return FGC_OK;
}

extern "C" int fgc_binned_knn_bwd_sorted(const float *grad_distsq, const int64_t *idx,
                                         const float *coords, int64_t n_vert, int32_t K,
                                         int32_t n_coords, const void *rgraph, size_t rgraph_bytes,
                                         float *out_grad_coords, fgc_stream_t stream)
{
    FGC_NVTX("fgc_binned_knn_bwd_sorted");
    using namespace fgc;
    if (n_vert < 0 || K < 1 || n_coords < 1) return FGC_ERR_BAD_ARGUMENT;
    if (n_vert * (int64_t)K > 0x7fffffff) return FGC_ERR_TOO_LARGE;
    const ReverseGraphLayout L = reverse_graph_layout(n_vert, K);
    if (!rgraph || rgraph_bytes < L.total || ((uintptr_t)rgraph & 255)) return FGC_ERR_WORKSPACE;
    if (n_vert == 0) return FGC_OK;
    if (!grad_distsq || !idx || !coords || !out_grad_coords) return FGC_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const char *ws = (const char *)rgraph;
    const int *offsets = (const int *)(ws + L.offsets);
    const int *entries = (const int *)(ws + L.entries);
    const int n = (int)n_vert;
    const unsigned blocks = (unsigned)((n + kBwdSortedWarps - 1) / kBwdSortedWarps);
    const int T = kBwdSortedWarps * 32;
    switch (n_coords) {
    case 2: k_knn_bwd_sorted<2><<<blocks, T, 0, s>>>(grad_distsq, idx, coords, n, K, n_coords, offsets, entries, out_grad_coords); break;
    case 3: k_knn_bwd_sorted<3><<<blocks, T, 0, s>>>(grad_distsq, idx, coords, n, K, n_coords, offsets, entries, out_grad_coords); break;
    case 4: k_knn_bwd_sorted<4><<<blocks, T, 0, s>>>(grad_distsq, idx, coords, n, K, n_coords, offsets, entries, out_grad_coords); break;
    default: k_knn_bwd_sorted<0><<<blocks, T, 0, s>>>(grad_distsq, idx, coords, n, K, n_coords, offsets, entries, out_grad_coords); break;
    }
    FGC_CHECK_LAUNCH();
    return FGC_OK;
}
