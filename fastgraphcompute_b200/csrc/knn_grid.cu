// binned_select_knn forward for sm_100a, part 1: the search grid (this file) --
// part 2, the search itself, is knn_search.cu.
//
// Pipeline (all on the caller's stream, no host synchronisation; 9 launches, 11 while the
// device still has to choose the grid's form for D = 4):
//   k_minmax_setup  fused finite check + min/max of the binned coordinates; clears the cell
//                 table; its last CTA validates the row splits and chooses cell width / grid
//                 shape from the extents and the point count (the grid spans the first
//                 min(D, 4) coordinates)
//   k_histogram   cell id per point, warp-aggregated atomic histogram; the value returned by
//                 the atomic is the point's rank inside its cell.  The ranks also give the
//                 density statistic sum_c c^2 for free, and the kernel's last CTA is the density
//                 pass: it shrinks the cells where the data is clustered; D = 4 data that is
//                 strongly clustered goes back to a grid over three coordinates and gets a
//                 second density pass there
//   k_zero_counts + k_histogram again, for the grid the density pass chose (return at once
//                 when it kept the first grid)
//   k_scan_tile_sums_top, k_scan_apply   exclusive scan of the histogram -> cell boundaries
//   k_fill_ids    counting-sort scatter of the original ids into cell order (arbitrary inside a cell)
//   k_rank_place  ids in ascending order inside every cell (the layout is the same on every
//                 run); coordinates (padded to float4), cell id and direction flag in that order
//   k_sort_large_cells  the same for the few cells too crowded for ranking
//   k_knn         one warp per query point: walks the neighbouring cells in
//                 expanding Chebyshev shells, evaluates 32 candidates per step
//                 (one per lane, 16-byte loads), keeps the K-1 best in registers
//                 and writes the row at its ORIGINAL position with ORIGINAL ids.
//
// What is computed is what the reference's CPU path computes
// (extensions/binned_knn_autograd_kernel.cpp:85-209 with
// extensions/binned_select_knn_cpu.cpp:56-208): per row split, the K-1 nearest
// other points (strict "<" replacement of the current worst, so among equal
// distances the first one visited stays), squared distances accumulated over the
// dimensions in order with one rounding per operation.  The visiting order, the
// grid and the stopping rule are this library's own; they never change which
// points are nearest, only which of several equidistant points is kept.
#include "knn_grid.cuh"
#include "shell_table.cuh"

namespace fgc {

// ---------------------------------------------------------------------------
// grid construction
// ---------------------------------------------------------------------------

__device__ void grid_setup(KnnGrid *g, const int64_t *__restrict__ row_splits, int n_rs, int n_vert,
                           int n_bin_dims, int bins_target, int bins_cap_first, int bins_cap, int bad_rs);

// Fused finite check + min/max of the binned coordinates; clears the cell table (all of its
// capacity: the grid that decides how much of it is used does not exist yet); the CTA that
// finishes last (a ticket counter, no waiting) checks the row splits and chooses the grid.
__global__ void __launch_bounds__(256)
k_minmax_setup(const float *__restrict__ coords, int n_vert, int n_coords, int n_bin_dims, KnnGrid *g,
               int *__restrict__ counts, long long n_counts, const int64_t *__restrict__ row_splits, int n_rs,
               int bins_target, int bins_cap_first, int bins_cap)
{
    chain_wait();
    chain_release();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_counts;
         i += (long long)gridDim.x * blockDim.x)
        counts[i] = 0;
    uint32_t lmin[4] = {0, 0, 0, 0}, lmax[4] = {0, 0, 0, 0};
    uint32_t bad = 0;
    for (int v = blockIdx.x * blockDim.x + threadIdx.x; v < n_vert; v += gridDim.x * blockDim.x) {
        const float *row = coords + (size_t)v * n_coords;
        for (int c = 0; c < n_coords; c++) {
            const float x = __ldg(row + c);
            if (!is_finite_bits(x)) bad = 1;
            if (c < n_bin_dims) {
                const uint32_t k = float_to_ordered(x);
#pragma unroll
                for (int cc = 0; cc < 4; cc++)
                    if (cc == c) { lmin[cc] = max(lmin[cc], ~k); lmax[cc] = max(lmax[cc], k); }
            }
        }
    }
    __shared__ uint32_t s_min[4], s_max[4], s_bad;
    if (threadIdx.x < 4) { s_min[threadIdx.x] = 0; s_max[threadIdx.x] = 0; }
    if (threadIdx.x == 0) s_bad = 0;
    __syncthreads();
#pragma unroll
    for (int c = 0; c < 4; c++) {
        const uint32_t a = __reduce_max_sync(FGC_FULL_MASK, lmin[c]);
        const uint32_t b = __reduce_max_sync(FGC_FULL_MASK, lmax[c]);
        if ((threadIdx.x & 31) == 0) { atomicMax(&s_min[c], a); atomicMax(&s_max[c], b); }
    }
    if (__any_sync(FGC_FULL_MASK, bad) && (threadIdx.x & 31) == 0) atomicOr(&s_bad, 1u);
    __syncthreads();
    if (threadIdx.x < 4) {
        atomicMax(&g->min_key[threadIdx.x], s_min[threadIdx.x]);
        atomicMax(&g->max_key[threadIdx.x], s_max[threadIdx.x]);
    }
    if (threadIdx.x == 0 && s_bad) atomicOr(&g->nonfinite, 1u);
    // the last CTA to arrive sees every CTA's extrema and sets the grid up
    __shared__ int s_last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = atomicAdd(&g->stat_blocks_done, 1) == (int)gridDim.x - 1;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // row_splits must start at 0, end at n_vert and never decrease
    int bad_rs = 0;
    for (int i = 1 + threadIdx.x; i < n_rs; i += blockDim.x)
        if (row_splits[i] < row_splits[i - 1]) bad_rs = 1;
    bad_rs = __syncthreads_or(bad_rs);
    if (threadIdx.x == 0) {
        g->stat_blocks_done = 0;       // the density pass counts its CTAs with the same ticket
        grid_setup(g, row_splits, n_rs, n_vert, n_bin_dims, bins_target, bins_cap_first, bins_cap, bad_rs);
    }
}

// Cells per dimension for a wanted cell width; widens the cells until the table fits.
__device__ inline void fit_shape(const float (&ext)[4], double wd, int bins_cap, int (&n)[4], float &w)
{
    for (int iter = 0; iter < 400; iter++) {
        w = (float)wd;
        const float inv = __fdiv_rn(1.0f, w);
        double prod = 1.0;
        for (int gd = 0; gd < 4; gd++) {
            n[gd] = ext[gd] > 0.f ? (int)floorf(__fmul_rn(ext[gd], inv)) + 1 : 1;
            prod *= (double)n[gd];
        }
        if (prod <= (double)bins_cap) break;
        wd *= 1.05;
    }
}

// One thread.  Chooses the cell width so that a row split of average size gets
// about bins_target cells, bounded by bins_cap cells per row split.
__device__ void grid_setup(KnnGrid *g, const int64_t *__restrict__ row_splits, int n_rs, int n_vert,
                           int n_bin_dims, int bins_target, int bins_cap_first, int bins_cap, int bad_rs)
{
    int status = 0;
    if (atomicOr(&g->nonfinite, 0u)) status |= FGC_STATUS_NONFINITE;
    if (bad_rs || row_splits[0] != 0 || row_splits[n_rs - 1] != (int64_t)n_vert)
        status |= FGC_STATUS_BAD_ROW_SPLITS;
    const int n_events = n_rs - 1;
    const int G = n_bin_dims >= 4 ? 4 : 3;      // grid dimensions in use
    const int sh = G - n_bin_dims;
    float ext[4];
    double vol = 1.0;
    int nz = 0;
    float ext_max = 0.f;
    for (int gd = 0; gd < 4; gd++) {
        if (gd >= G) {
            g->cdim[gd] = -1;
            g->origin[gd] = 0.f;
            ext[gd] = 0.f;
        } else if (gd < sh || (status & FGC_STATUS_NONFINITE)) {
            g->cdim[gd] = gd < sh ? -1 : gd - sh;
            g->origin[gd] = 0.f;
            ext[gd] = 0.f;
        } else {
            const int c = gd - sh;
            const float lo = ordered_to_float(~atomicMax(&g->min_key[c], 0u));
            const float hi = ordered_to_float(atomicMax(&g->max_key[c], 0u));
            g->cdim[gd] = c;
            g->origin[gd] = lo;
            ext[gd] = __fsub_rn(hi, lo);
            if (!(ext[gd] >= 0.f) || !is_finite_bits(ext[gd])) ext[gd] = 0.f;
        }
        if (ext[gd] > 0.f) { vol *= (double)ext[gd]; nz++; }
        ext_max = fmaxf(ext_max, ext[gd]);
    }
    int n[4] = {1, 1, 1, 1};
    float w = 1.f;
    if (nz > 0) {
        if (bins_target < 1) bins_target = 1;
        double wd = pow(vol / (double)bins_target, 1.0 / (double)nz);
        // a degenerate extent ratio can make the width underflow: keep it representable
        if (!(wd > (double)ext_max * 1e-6)) wd = (double)ext_max * 1e-6;
        fit_shape(ext, wd, bins_cap_first, n, w);
    }
    long long B = (long long)n[0] * n[1] * n[2] * n[3];
    if (B > bins_cap_first) {  // cannot happen after the loop above unless the extents are absurd
        n[0] = n[1] = n[2] = n[3] = 1; B = 1; w = fmaxf(ext_max, 1.f) * 2.f;
        status |= FGC_STATUS_INTERNAL;
    }
    g->n[0] = n[0]; g->n[1] = n[1]; g->n[2] = n[2]; g->n[3] = n[3];
    g->gdims = G;
    g->B = (int)B;
    g->n_events = n_events;
    g->total_bins = (int)(B * n_events);
    grid_set_divisors(g);
    g->w = w;
    g->inv_w = __fdiv_rn(1.0f, w);
    g->slack = 4e-6f * fmaxf(ext_max, w);
    g->ext[0] = ext[0]; g->ext[1] = ext[1]; g->ext[2] = ext[2]; g->ext[3] = ext[3];
    g->bins_cap = bins_cap;
    g->status = status;
}

// Density pass.  The first grid is sized from the bounding box, i.e. from the MEAN density.
// Clustered data puts most points into cells far above that mean, and the cost of a query
// grows with the occupancy of the cells around it.  sum_c c^2 / N is the occupancy a typical
// point sees in its own cell; when it is well above the wanted value the grid is rebuilt
// with cells shrunk by the cube root of the ratio (occupancy scales with the cell volume
// where the density is locally smooth).
// pass 0: the density pass on the first grid.  pass 1: a second one, only after pass 0 fell
// back from a grid over four coordinates to one over three (D = 4 only): a dense cell table
// over the four-dimensional bounding box cannot follow strongly clustered data -- the wanted
// cell size would need far more cells than the table holds -- so data that asks for cells more
// than 2.8x finer than the mean density suggests is binned in three coordinates, where the
// same table reaches the wanted size.
__device__ void grid_refine(KnnGrid *g, unsigned long long sum_sq, int n_vert, float seen_target,
                            float seen_target3, int bins_target3, int pass, int allow_fallback)
{
    const float target = pass == 0 ? seen_target : seen_target3;
    const double seen = (double)sum_sq / (double)(n_vert > 0 ? n_vert : 1);
    if (!(seen > 1.5 * (double)target)) return;
    int nz = 0;
    float ext[4], ext_max = 0.f;
    for (int gd = 0; gd < 4; gd++) {
        ext[gd] = g->ext[gd];
        if (ext[gd] > 0.f) nz++;
        ext_max = fmaxf(ext_max, ext[gd]);
    }
    if (nz == 0) return;
    double shrink = pow((double)target / seen, 1.0 / (double)nz);
    int n[4] = {1, 1, 1, 1};
    float w = g->w;
    if (pass == 0 && allow_fallback && g->gdims == 4 && shrink < 0.36) {
        g->gdims = 3;
        g->cdim[3] = -1; g->origin[3] = 0.f; g->ext[3] = 0.f;
        ext[3] = 0.f;
        double vol = 1.0;
        nz = 0; ext_max = 0.f;
        for (int gd = 0; gd < 3; gd++) {
            if (ext[gd] > 0.f) { vol *= (double)ext[gd]; nz++; }
            ext_max = fmaxf(ext_max, ext[gd]);
        }
        if (nz > 0) {
            double wd = pow(vol / (double)(bins_target3 < 1 ? 1 : bins_target3), 1.0 / (double)nz);
            if (!(wd > (double)ext_max * 1e-6)) wd = (double)ext_max * 1e-6;
            fit_shape(ext, wd, g->bins_cap, n, w);
        } else {
            w = 1.f;
        }
        const long long B3 = (long long)n[0] * n[1] * n[2];
        g->n[0] = n[0]; g->n[1] = n[1]; g->n[2] = n[2]; g->n[3] = 1;
        g->B = (int)B3;
        g->total_bins = (int)(B3 * g->n_events);
        grid_set_divisors(g);
        g->w = w;
        g->inv_w = __fdiv_rn(1.0f, w);
        g->slack = 4e-6f * fmaxf(ext_max, w);
        g->fallback3 = 1;
        g->refined = 1;
        g->sum_sq = 0;              // the second density pass starts from scratch
        g->stat_blocks_done = 0;
        return;
    }
    // Never more than 2.2x: data that mixes very dense clusters with a thin background
    // would otherwise pay with long walks through empty cells for the background queries.
    if (shrink < 1.0 / 2.2) shrink = 1.0 / 2.2;
    double wd = (double)g->w * shrink;
    if (!(wd > (double)ext_max * 1e-6)) wd = (double)ext_max * 1e-6;
    fit_shape(ext, wd, g->bins_cap, n, w);
    const long long B = (long long)n[0] * n[1] * n[2] * n[3];
    if (B > g->bins_cap || !(w < g->w)) return;
    g->n[0] = n[0]; g->n[1] = n[1]; g->n[2] = n[2]; g->n[3] = n[3];
    g->B = (int)B;
    g->total_bins = (int)(B * g->n_events);
    grid_set_divisors(g);
    g->w = w;
    g->inv_w = __fdiv_rn(1.0f, w);
    g->slack = 4e-6f * fmaxf(ext_max, w);
    g->refined = pass + 1;
}

__global__ void __launch_bounds__(256)
k_zero_counts(int *__restrict__ counts, const KnnGrid *g, int stage)
{
    chain_wait();
    chain_release();
    if (g->refined < stage) return;      // stage s follows the s-th density pass that changed the grid
    const int n = g->total_bins + 1;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
        counts[i] = 0;
}

// Cell coordinate of a shifted coordinate; identical in every kernel that needs it.
__device__ __forceinline__ int cell_of(float x, float origin, float inv_w, int n)
{
    const float t = __fsub_rn(x, origin);
    int b = (int)floorf(__fmul_rn(t, inv_w));
    b = b < 0 ? 0 : b;
    return b >= n ? n - 1 : b;
}

// refine_pass >= 0: the kernel is also the density pass of that number.  A point that arrives
// as the r-th of its cell adds 2r+1, so that a cell of c points adds c^2 in total: the sum over
// the cells of c^2 comes out of the histogram itself, with no second pass over the table.  The
// CTA that finishes last (a ticket counter, no waiting) decides about the finer grid.
__global__ void __launch_bounds__(256)
k_histogram(const float *__restrict__ coords, int n_vert, int n_coords,
            const int64_t *__restrict__ row_splits, int n_rs, KnnGrid *__restrict__ g,
            int *__restrict__ counts, int *__restrict__ pbin, int *__restrict__ prank,
            int stage, int refine_pass, float seen_target, float seen_target3, int bins_target3,
            int allow_fallback)
{
    chain_wait();
    chain_release();
    if (g->refined < stage) return;
    if (refine_pass == 1 && !g->fallback3) refine_pass = -1;
    const int v = blockIdx.x * blockDim.x + threadIdx.x;
    const bool live = v < n_vert && g->status == 0;
    int flat = 0;
    unsigned long long sq = 0;
    if (live) {
        const float *row = coords + (size_t)v * n_coords;
        int b[4];
#pragma unroll
        for (int gd = 0; gd < 4; gd++) {
            const int c = g->cdim[gd];
            b[gd] = c < 0 ? 0 : cell_of(__ldg(row + c), g->origin[gd], g->inv_w, g->n[gd]);
        }
        const int e = row_split_of(row_splits, n_rs, v);
        // the fourth dimension has one cell (b[3] = 0) in a grid over three coordinates
        flat = e * g->B + ((b[0] * g->n[1] + b[1]) * g->n[2] + b[2]) * g->n[3] + b[3];
    }
    const unsigned active = __ballot_sync(FGC_FULL_MASK, live && FGC_DBG_OK(flat >= 0 && flat < g->total_bins, &g->status));
    if (active >> (threadIdx.x & 31) & 1) {
        // warp-aggregated: one atomic per distinct cell in the warp
        const unsigned peers = __match_any_sync(active, flat);
        const int leader = __ffs(peers) - 1;
        int base = 0;
        if ((int)(threadIdx.x & 31) == leader) base = atomicAdd(counts + flat, __popc(peers));
        base = __shfl_sync(peers, base, leader);
        pbin[v] = flat;
        const int rank = base + __popc(peers & lanemask_lt());
        prank[v] = rank;
        sq = 2ull * (unsigned long long)rank + 1ull;
    }
    if (refine_pass < 0 || g->status != 0) return;     // uniform over the grid
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(FGC_FULL_MASK, sq, o);
    __shared__ unsigned long long s_sq[8];
    if ((threadIdx.x & 31) == 0) s_sq[threadIdx.x >> 5] = sq;
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long t = 0;
        for (int k = 0; k < 8; k++) t += s_sq[k];
        if (t) atomicAdd(&g->sum_sq, t);
        __threadfence();
        const int ticket = atomicAdd(&g->stat_blocks_done, 1);
        if (ticket == (int)gridDim.x - 1) {
            __threadfence();
            g->stat_blocks_done = 0;
            grid_refine(g, atomicAdd(&g->sum_sq, 0ull), n_vert, seen_target, seen_target3, bins_target3,
                        refine_pass, allow_fallback);
        }
    }
}

// Counting-sort scatter, step 1: original ids in cell order.  The position inside a cell is
// the rank the histogram's atomic handed out, i.e. arbitrary.
__global__ void __launch_bounds__(256)
k_fill_ids(int n_vert, const KnnGrid *__restrict__ g, const int *__restrict__ bounds,
           const int *__restrict__ pbin, const int *__restrict__ prank, int *__restrict__ stmp)
{
    chain_wait();
    chain_release();
    const int v = blockIdx.x * blockDim.x + threadIdx.x;
    if (v >= n_vert || g->status != 0) return;
    const int pos = bounds[pbin[v]] + prank[v];
    if (FGC_DBG_OK(pos >= 0 && pos < n_vert, &g->status)) stmp[pos] = v;
}

// Everything that is kept per point in cell order: original id, coordinates padded to
// float4, cell id, direction flag.
__device__ __forceinline__ void place_point(int pos, int v, int bin, const float *__restrict__ coords,
                                            int n_coords, int nv, const int64_t *__restrict__ direction,
                                            int *__restrict__ sorig, float4 *__restrict__ scoords,
                                            int *__restrict__ sbin, uint8_t *__restrict__ sflag)
{
    const float *row = coords + (size_t)v * n_coords;
    for (int q = 0; q < nv; q++) {
        float4 o;
        o.x = 4 * q + 0 < n_coords ? __ldg(row + 4 * q + 0) : 0.f;
        o.y = 4 * q + 1 < n_coords ? __ldg(row + 4 * q + 1) : 0.f;
        o.z = 4 * q + 2 < n_coords ? __ldg(row + 4 * q + 2) : 0.f;
        o.w = 4 * q + 3 < n_coords ? __ldg(row + 4 * q + 3) : 0.f;
        scoords[(size_t)pos * nv + q] = o;
    }
    sorig[pos] = v;
    sbin[pos] = bin;
    if (direction) {
        const int64_t d = direction[v];
        sflag[pos] = (d >= 0 && d <= 2) ? (uint8_t)d : (uint8_t)3;
    }
}

// Step 2: the ids inside every cell in ascending order, so that the cell-ordered layout --
// and with it the order in which the search visits candidates, its choice among equidistant
// candidates and the slot order of its output -- is the same on every run.  One thread per
// point: in a cell of up to kRankMax points the point's place is the number of smaller ids in
// the cell (read from the unordered list of step 1), and everything kept in cell order is
// written there at once.  Points of larger cells keep their arbitrary place for now and
// the cell goes to a work list (k_sort_large_cells).
__global__ void __launch_bounds__(256)
k_rank_place(const float *__restrict__ coords, int n_vert, int n_coords, int nv,
             const int64_t *__restrict__ direction, KnnGrid *__restrict__ g,
             const int *__restrict__ bounds, const int *__restrict__ pbin,
             const int *__restrict__ prank, const int *__restrict__ stmp,
             int *__restrict__ sorig, float4 *__restrict__ scoords, int *__restrict__ sbin,
             uint8_t *__restrict__ sflag, int *__restrict__ biglist, int *__restrict__ hugelist)
{
    chain_wait();
    chain_release();
    const int v = blockIdx.x * blockDim.x + threadIdx.x;
    if (v >= n_vert || g->status != 0) return;
    const int bin = pbin[v];
    const int beg = bounds[bin], len = bounds[bin + 1] - beg;
    if (len <= kRankMax) {
        int rank = 0;
        for (int t = 0; t < len; t++) rank += stmp[beg + t] < v ? 1 : 0;
        if (FGC_DBG_OK(beg >= 0 && rank < len && beg + rank < n_vert, &g->status))
            place_point(beg + rank, v, bin, coords, n_coords, nv, direction, sorig, scoords, sbin, sflag);
    } else {
        const int r = prank[v];
        sorig[beg + r] = v;
        if (r == 0) {
            if (len <= kWarpSortMaxShared) biglist[atomicAdd(&g->n_big_cells, 1)] = bin;
            else hugelist[atomicAdd(&g->n_huge_cells, 1)] = bin;
        }
    }
}

// Step 3: the cells of the work lists.  The first n_warp_blocks CTAs take the cells that one
// warp can sort (in registers / shared memory), the remaining CTAs take the cells beyond
// kWarpSortMaxShared points, one CTA per cell: bitonic sort in its all-ascending form, in
// place in global memory (the sequence is treated as padded to a power of two with
// +infinity; a compare-exchange whose upper partner lies in the padding never swaps, so it
// is simply skipped).  After the sort the same warp / CTA places the cell's points.
constexpr int kSortWarps = 4;

__global__ void __launch_bounds__(kSortWarps * 32)
k_sort_large_cells(const float *__restrict__ coords, int n_coords, int nv,
                   const int64_t *__restrict__ direction, const KnnGrid *__restrict__ g,
                   const int *__restrict__ bounds, const int *__restrict__ biglist,
                   const int *__restrict__ hugelist, int n_warp_blocks,
                   int *__restrict__ sorig, float4 *__restrict__ scoords, int *__restrict__ sbin,
                   uint8_t *__restrict__ sflag)
{
    chain_wait();
    chain_release();
    __shared__ int s_keys[kSortWarps][kWarpSortMaxShared];
    if (g->status != 0) return;
    if ((int)blockIdx.x < n_warp_blocks) {
        const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
        const int n_big = g->n_big_cells;
        for (int w = blockIdx.x * kSortWarps + wib; w < n_big; w += n_warp_blocks * kSortWarps) {
            const int cell = biglist[w];
            const int beg = bounds[cell], n = bounds[cell + 1] - beg;
            warp_sort_segment(sorig + beg, n, s_keys[wib], lane);
            __syncwarp();
            for (int t = lane; t < n; t += 32)
                place_point(beg + t, sorig[beg + t], cell, coords, n_coords, nv, direction, sorig, scoords,
                            sbin, sflag);
            __syncwarp();
        }
        return;
    }
    const int n_huge = g->n_huge_cells;
    const int n_cta = gridDim.x - n_warp_blocks;
    for (int w = blockIdx.x - n_warp_blocks; w < n_huge; w += n_cta) {
        const int cell = hugelist[w];
        const int beg = bounds[cell], n = bounds[cell + 1] - beg;
        int *seg = sorig + beg;
        int P = 1;
        while (P < n) P <<= 1;
        for (int k = 2; k <= P; k <<= 1) {
            // flip: element i of a block of k against its mirror image
            for (int t = threadIdx.x; t < P / 2; t += blockDim.x) {
                const int half = k >> 1, blk = t / half, off = t - blk * half;
                const int a = blk * k + off, b = blk * k + (k - 1 - off);
                if (b < n) {
                    const int ka = seg[a], kb = seg[b];
                    if (ka > kb) { seg[a] = kb; seg[b] = ka; }
                }
            }
            __syncthreads();
            for (int j = k >> 2; j > 0; j >>= 1) {
                for (int t = threadIdx.x; t < P / 2; t += blockDim.x) {
                    const int a = 2 * j * (t / j) + (t % j), b = a + j;
                    if (b < n) {
                        const int ka = seg[a], kb = seg[b];
                        if (ka > kb) { seg[a] = kb; seg[b] = ka; }
                    }
                }
                __syncthreads();
            }
        }
        for (int t = threadIdx.x; t < n; t += blockDim.x)
            place_point(beg + t, seg[t], cell, coords, n_coords, nv, direction, sorig, scoords, sbin, sflag);
        __syncthreads();
    }
}

// Status word and the grid's form ((3 or 4) + 16 * fallback3) to memory the host can read.
__global__ void k_publish_grid_info(const KnnGrid *__restrict__ g, volatile int32_t *info_mapped)
{
    chain_wait();
    chain_release();
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        info_mapped[0] = g->status;
        info_mapped[1] = g->gdims + 16 * g->fallback3;
        __threadfence_system();
    }
}

// One store of the status word to memory the host can read (mapped pinned memory).
__global__ void k_publish_status(const int32_t *__restrict__ status_dev, volatile int32_t *status_mapped)
{
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        *status_mapped = *status_dev;
        __threadfence_system();
    }
}

}  // namespace fgc

extern "C" size_t fgc_knn_workspace_bytes(int64_t n_vert, int32_t n_coords, int64_t n_rs, int32_t K)
{
    if (n_vert < 0 || n_vert > 0x7fffffff || n_coords < 1 || n_rs < 1 || K < 1) return 0;
    return fgc::knn_workspace_layout(n_vert, n_coords, n_rs, K).total;
}

extern "C" int fgc_read_status(const void *workspace_or_params, int32_t *status_host,
                               fgc_stream_t stream)
{
    if (!workspace_or_params || !status_host) return FGC_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    FGC_RETURN_IF_CUDA(cudaMemcpyAsync(status_host, workspace_or_params, sizeof(int32_t),
                                       cudaMemcpyDeviceToHost, s));
    FGC_RETURN_IF_CUDA(cudaStreamSynchronize(s));
    return FGC_OK;
}

extern "C" int fgc_publish_status(const void *workspace_or_params, int32_t *status_mapped,
                                  fgc_stream_t stream)
{
    if (!workspace_or_params || !status_mapped) return FGC_ERR_BAD_ARGUMENT;
    fgc::k_publish_status<<<1, 32, 0, (cudaStream_t)stream>>>((const int32_t *)workspace_or_params, status_mapped);
    FGC_CHECK_LAUNCH();
    return FGC_OK;
}

extern "C" int fgc_knn_publish_grid_info(const void *workspace, int32_t *info_mapped, fgc_stream_t stream)
{
    if (!workspace || !info_mapped) return FGC_ERR_BAD_ARGUMENT;
    FGC_RETURN_IF_CUDA(fgc::launch_chained(fgc::k_publish_grid_info, 1, 32, 0, (cudaStream_t)stream,
                                           (const fgc::KnnGrid *)workspace, info_mapped));
    return FGC_OK;
}

extern "C" int fgc_knn_build_grid(const float *coords, int64_t n_vert, int32_t n_coords,
                                  const int64_t *row_splits, int64_t n_rs, int32_t K,
                                  const int64_t *direction_or_null, float target_occupancy,
                                  void *workspace, size_t workspace_bytes, fgc_stream_t stream)
{
    return fgc_knn_build_grid_dims(coords, n_vert, n_coords, row_splits, n_rs, K, direction_or_null,
                                   target_occupancy, 0, workspace, workspace_bytes, stream);
}

extern "C" int fgc_knn_build_grid_dims(const float *coords, int64_t n_vert, int32_t n_coords,
                                       const int64_t *row_splits, int64_t n_rs, int32_t K,
                                       const int64_t *direction_or_null, float target_occupancy,
                                       int32_t grid_dims, void *workspace, size_t workspace_bytes,
                                       fgc_stream_t stream)
{
    FGC_NVTX("fgc_knn_build_grid_dims");
    using namespace fgc;
    if (grid_dims != 0 && grid_dims != 3 && grid_dims != 4) return FGC_ERR_BAD_ARGUMENT;
    KnnWorkspace L;
    if (!row_splits) return FGC_ERR_BAD_ARGUMENT;
    const int rc = check_knn_args(n_vert, n_coords, n_rs, K, workspace, workspace_bytes, &L);
    if (rc != FGC_OK) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    char *ws = (char *)workspace;
    KnnGrid *grid = (KnnGrid *)(ws + L.header);
    FGC_RETURN_IF_CUDA(cudaMemsetAsync(grid, 0, kGridHeaderBytes + kHardTicketBytes, s));   // header and k_knn_hard's tickets
    if (n_vert == 0) return FGC_OK;
    if (!coords || n_rs < 2) return FGC_ERR_BAD_ARGUMENT;

    int *counts = (int *)(ws + L.counts);
    int *blocksums = (int *)(ws + L.blocksums);
    int *pbin = (int *)(ws + L.pbin);
    int *prank = (int *)(ws + L.prank);
    int *stmp = (int *)(ws + L.stmp);
    int *sorig = (int *)(ws + L.sorig);
    int *biglist = (int *)(ws + L.biglist);
    int *hugelist = (int *)(ws + L.hugelist);
    int *sbin = (int *)(ws + L.sbin);
    uint8_t *sflag = (uint8_t *)(ws + L.sflag);
    float4 *scoords = (float4 *)(ws + L.scoords);

    const int n = (int)n_vert;
    const int n_events = (int)n_rs - 1;
    // D = 4 lets the density pass choose between four and three binned coordinates unless the
    // caller fixes the choice (grid_dims 3 or 4; ignored for every other D)
    const int forced = n_coords == 4 ? grid_dims : 0;
    const int n_bin_dims = forced == 3 ? 3 : (n_coords < 4 ? n_coords : 4);
    // target_occupancy > 0: one fixed grid with that mean occupancy.  Otherwise: mean
    // occupancy K/21 within [1.5, 3] (measured on B200: K = 32 is fastest at 1 to 1.5, K = 64
    // at 3 to 4, K = 128 at 2 to 3; the optimum is flat, +-2 % over a factor of two), then
    // the density pass may shrink the cells so that a typical point sees about seen_target
    // points in its own cell.
    const bool adaptive = !(target_occupancy > 0.f);
    if (adaptive) {
        target_occupancy = (float)K / 21.0f;
        if (target_occupancy < 1.5f) target_occupancy = 1.5f;
        if (target_occupancy > 3.0f) target_occupancy = 3.0f;
    }
    float seen_target = (float)K / 6.0f;
    if (seen_target < 4.f) seen_target = 4.f;
    const float seen_target3 = seen_target * 2.f;    // D = 4 binned in three coordinates
    if (n_coords > n_bin_dims) seen_target *= 2.f;   // coordinates that are not binned thin the cells out
    const int64_t bins_cap64 = L.cap_bins / n_events;
    const int bins_cap = (int)(bins_cap64 < 1 ? 1 : bins_cap64);
    const double bt = (double)n_vert / (double)n_events / (double)target_occupancy;
    int bins_target = bt >= (double)bins_cap ? bins_cap : (int)(bt + 0.5);
    if (bins_target < 1) bins_target = 1;

    const int pt_blocks = (n + 255) / 256;
    const int red_blocks = pt_blocks < fgc::sm_count() * 4 ? pt_blocks : fgc::sm_count() * 4;
    // The cell count is only known on the device.  The first grid may use up to four times the
    // wanted number of cells (its shape is rounded up per dimension): that part of the table is
    // cleared together with the extent reduction; a finer grid of the density pass clears what
    // it needs itself.  The scan grids are sized for the largest table (surplus blocks return
    // at once).
    const int64_t max_entries = (int64_t)bins_cap * n_events + 1;
    const int scan_blocks = (int)ceil_div64(max_entries, kScanTile);
    int bins_cap_first = bins_target > (bins_cap - 64) / 4 ? bins_cap : 4 * bins_target + 64;
    if (!adaptive) bins_cap_first = bins_cap;
    k_minmax_setup<<<red_blocks, 256, 0, s>>>(coords, n, n_coords, n_bin_dims, grid, counts,
                                              (long long)bins_cap_first * n_events + 1, row_splits, (int)n_rs,
                                              bins_target, bins_cap_first, bins_cap);
    FGC_CHECK_LAUNCH();
    const int allow_fallback = adaptive && n_coords == 4 && forced == 0;
    FGC_RETURN_IF_CUDA(launch_chained(k_histogram, pt_blocks, 256, 0, s, coords, n, n_coords, row_splits, (int)n_rs, grid,
                                      counts, pbin, prank, 0, adaptive ? 0 : -1, seen_target, seen_target3,
                                      bins_target, allow_fallback));
    if (adaptive) {
        // the grid of the density pass, when it chose one (both kernels return at once otherwise)
        FGC_RETURN_IF_CUDA(launch_chained(k_zero_counts, fgc::sm_count() * 4, 256, 0, s, counts, grid, 1));
        FGC_RETURN_IF_CUDA(launch_chained(k_histogram, pt_blocks, 256, 0, s, coords, n, n_coords, row_splits, (int)n_rs,
                                          grid, counts, pbin, prank, 1, allow_fallback ? 1 : -1, seen_target,
                                          seen_target3, bins_target, 0));
        if (allow_fallback) {
            // second density pass: ran only when the first one fell back to three coordinates
            FGC_RETURN_IF_CUDA(launch_chained(k_zero_counts, fgc::sm_count() * 4, 256, 0, s, counts, grid, 2));
            FGC_RETURN_IF_CUDA(launch_chained(k_histogram, pt_blocks, 256, 0, s, coords, n, n_coords, row_splits,
                                              (int)n_rs, grid, counts, pbin, prank, 2, -1, seen_target, seen_target3,
                                              bins_target, 0));
        }
    }
    FGC_RETURN_IF_CUDA(launch_chained(k_scan_tile_sums_top, scan_blocks, 256, 0, s, counts, &grid->total_bins, 1,
                                      blocksums, &grid->scan_ticket));
    FGC_RETURN_IF_CUDA(launch_chained(k_scan_apply, scan_blocks, 256, 0, s, counts, &grid->total_bins, 1, blocksums));
    FGC_RETURN_IF_CUDA(launch_chained(k_fill_ids, pt_blocks, 256, 0, s, n, grid, counts, pbin, prank, stmp));
    FGC_RETURN_IF_CUDA(launch_chained(k_rank_place, pt_blocks, 256, 0, s, coords, n, n_coords, L.nv, direction_or_null,
                                      grid, counts, pbin, prank, stmp, sorig, scoords, sbin, sflag, biglist, hugelist));
    const int n_warp_blocks = fgc::sm_count() * 4;
    FGC_RETURN_IF_CUDA(launch_chained(k_sort_large_cells, n_warp_blocks + fgc::sm_count(), kSortWarps * 32, 0, s, coords,
                                      n_coords, L.nv, direction_or_null, grid, counts, biglist, hugelist, n_warp_blocks,
                                      sorig, scoords, sbin, sflag));
    return FGC_OK;
}

extern "C" const int32_t *fgc_knn_cell_order(const void *workspace, int64_t n_vert, int32_t n_coords,
                                             int64_t n_rs, int32_t K)
{
    if (!workspace || n_vert < 0 || n_coords < 1 || n_rs < 1 || K < 1) return nullptr;
    const fgc::KnnWorkspace L = fgc::knn_workspace_layout(n_vert, n_coords, n_rs, K);
    return (const int32_t *)((const char *)workspace + L.sorig);
}

extern "C" int fgc_knn_read_counters(const void *workspace, uint64_t *counters_host,
                                     int32_t *grid_shape_host, float *cell_width_host,
                                     fgc_stream_t stream)
{
    using namespace fgc;
    if (!workspace) return FGC_ERR_BAD_ARGUMENT;
    KnnGrid h;
    cudaStream_t s = (cudaStream_t)stream;
    FGC_RETURN_IF_CUDA(cudaMemcpyAsync(&h, workspace, sizeof(KnnGrid), cudaMemcpyDeviceToHost, s));
    FGC_RETURN_IF_CUDA(cudaStreamSynchronize(s));
    if (counters_host) {
        for (int i = 0; i < 6; i++) counters_host[i] = h.counters[i];
        // facts about the grid build (always available, not only after a counting search)
        counters_host[6] = (uint64_t)h.n_hard;          // queries the last search handed to whole CTAs
        counters_host[7] = (uint64_t)h.n_huge_cells;    // cells above 512 points (sorted by one CTA each)
    }
    if (grid_shape_host) { grid_shape_host[0] = h.n[0]; grid_shape_host[1] = h.n[1]; grid_shape_host[2] = h.n[2] * h.n[3]; }
    if (cell_width_host) *cell_width_host = h.w;
    return FGC_OK;
}
