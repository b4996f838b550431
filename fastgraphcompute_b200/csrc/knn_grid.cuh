// Internal search grid of the kNN: layout of the workspace and the record that
// describes the grid (written on the device, read by every later kernel).
//
// The search grid is private to this library.  The k nearest neighbours of a
// point do not depend on how space is binned, so the grid is chosen for the
// GPU (cell size from the point density, up to three binned dimensions) and not
// from the reference's n_bins / max_bin_dims arguments.
#pragma once
#include "fgc_common.cuh"
#include "scan.cuh"
#include "segsort.cuh"

namespace fgc {

// Grid over the first min(D, 4) coordinate dimensions.  With D <= 3 the grid has three
// dimensions (gdims = 3): grid dimension g uses coordinate dimension cdim[g], unused leading
// grid dimensions have n = 1, and cell (e, b0, b1, b2) of row split e has flat id
// e*B + (b0*n[1] + b1)*n[2] + b2.  With D >= 4 it has four (gdims = 4, cdim[g] = g) and the
// flat id is e*B + ((b0*n[1] + b1)*n[2] + b2)*n[3] + b3.  Either way the cells of one line
// along the last grid dimension are consecutive and, after the counting sort, so are
// their points.
struct KnnGrid {
    int32_t status;        // FGC_STATUS_* bits (first word of the workspace)
    int32_t n_events;
    int32_t n[4];          // cells per grid dimension (1 for an unused one)
    int32_t cdim[4];       // coordinate dimension of grid dimension g, -1 = unused
    int32_t gdims;         // 3 or 4
    int32_t B;             // cells per row split = n[0]*n[1]*n[2]
    int32_t total_bins;    // n_events * B
    float origin[4];       // global minimum of the coordinate
    float w;               // cell width
    float inv_w;           // 1 / w
    float slack;           // absolute safety margin for cell-distance bounds
    uint32_t min_key[4];   // ~ordered(min) per binned coordinate (atomicMax)
    uint32_t max_key[4];   // ordered(max)
    uint32_t nonfinite;    // set when any coordinate is NaN/Inf
    float ext[4];          // extent of the bounding box per grid dimension
    int32_t bins_cap;      // largest cell count per row split the table can hold
    int32_t refined;       // number of density passes that replaced the grid (0, 1 or 2)
    int32_t fallback3;     // 1: D = 4 data too clustered for a table over four coordinates,
                           // the grid was rebuilt over the first three
    int32_t n_big_cells;   // length of the work list of cells sorted by one warp each
    int32_t n_huge_cells;  // length of the work list of cells sorted by one CTA each
    int32_t stat_blocks_done;   // CTAs of the density pass that have added their share
    int32_t n_hard;        // queries whose walk gave up in a large row split (searched by whole CTAs)
    int32_t scan_ticket;   // CTAs of the scan's first kernel that are done (zero between launches)
    unsigned long long sum_sq;   // sum over cells of (points in cell)^2, first grid
    // optional debug counters (filled when a search is launched with count_evals):
    // [0] distance evaluations, [1] 32-candidate steps, [2] list insertions,
    // [3] 32-item metadata batches, [4] shells, [5] queries that scanned their whole row split
    unsigned long long counters[6];
    // division of a cell id by B, n1*n2*n3, n2*n3 and n3 as multiply + shift (grid_set_divisors)
    uint32_t div_m[4];
    uint32_t div_s[4];
};

// x / d for 0 <= x < 2^31 and 1 <= d < 2^31 as (x * m) >> s with m = ceil(2^s / d),
// s = 31 + ceil(log2 d): exact for every such x (m < 2^32, the product fits 64 bits).
__host__ __device__ inline void fast_div_setup(uint32_t d, uint32_t &m, uint32_t &s)
{
    uint32_t l = 0;
    while (l < 31 && (1u << l) < d) l++;
    s = 31 + l;
    m = (uint32_t)((((unsigned long long)1 << s) + d - 1) / d);
}
__device__ __forceinline__ int fast_div(int x, uint32_t m, uint32_t s)
{
    return (int)(((unsigned long long)(uint32_t)x * m) >> s);
}
__host__ __device__ inline void grid_set_divisors(KnnGrid *g)
{
    const uint32_t n1 = (uint32_t)g->n[1], n2 = (uint32_t)g->n[2], n3 = (uint32_t)g->n[3];
    fast_div_setup((uint32_t)g->B, g->div_m[0], g->div_s[0]);
    fast_div_setup(n1 * n2 * n3, g->div_m[1], g->div_s[1]);
    fast_div_setup(n2 * n3, g->div_m[2], g->div_s[2]);
    fast_div_setup(n3, g->div_m[3], g->div_s[3]);
}

// Items of the Chebyshev shell of radius d around a cell, in units of "line segments": a
// segment is a run of consecutive cells along the last grid dimension, i.e. one contiguous
// range of sorted points.  Shell 0 is the cell itself.  For d >= 1 the 8d lines on the rim of
// the (2d+1)x(2d+1) square of leading-dimension offsets contribute their whole 2d+1 cells,
// every interior line contributes its two end cells.
__host__ __device__ inline int shell_items(int d) { return d == 0 ? 1 : 8 * d + 2 * (2 * d - 1) * (2 * d - 1); }
constexpr int kShellTableMaxD = 4;
constexpr int kShellTableEntries = 1 + 10 + 34 + 74 + 130;   // sum of shell_items(0..4)
__host__ __device__ inline int shell_table_offset(int d)
{
    return d == 0 ? 0 : (d == 1 ? 1 : (d == 2 ? 11 : (d == 3 ? 45 : 119)));
}

// Offsets (o0, o1) of the line and cell range [zlo, zhi] (relative to the query's cell) of
// item u of shell d.
__host__ __device__ inline void shell_item_decode(int d, int u, int &o0, int &o1, int &zlo, int &zhi)
{
    o0 = 0; o1 = 0; zlo = 0; zhi = 0;
    if (d == 0) return;
    const int side = 2 * d + 1, half = 2 * d - 1, n_ring = 8 * d;
    if (u < n_ring) {
        if (u < side) { o0 = -d; o1 = u - d; }
        else if (u < 2 * side) { o0 = d; o1 = u - side - d; }
        else {
            const int t = u - 2 * side;
            if (t < half) { o1 = -d; o0 = t - (d - 1); }
            else { o1 = d; o0 = t - half - (d - 1); }
        }
        zlo = -d; zhi = d;
    } else {
        const int c = u - n_ring, t = c >> 1, tq = t / half;
        o0 = tq - (d - 1);
        o1 = t - tq * half - (d - 1);
        zlo = zhi = (c & 1) ? d : -d;
    }
}

// Grids over four coordinates: shell d = the lines whose three leading offsets have Chebyshev
// norm d, each with its whole run of 2d+1 cells, plus the two end cells of every interior line.
// Shells up to kShellTable4MaxD come from a table (nearest first, exact item count); beyond
// that every offset triple of the (2d+1)^3 cube yields two items, the second one of a rim line
// being empty.
constexpr int kShellTable4MaxD = 2;
__host__ __device__ inline int shell_items4(int d)
{
    if (d == 0) return 1;
    const int a = 2 * d + 1, b = 2 * d - 1;
    return d <= kShellTable4MaxD ? a * a * a + b * b * b : 2 * a * a * a;
}
__host__ __device__ inline int shell_table4_offset(int d) { return d == 0 ? 0 : (d == 1 ? 1 : 29); }
__host__ __device__ inline void shell_item_decode4(int d, int u, int &o0, int &o1, int &o2, int &zlo, int &zhi)
{
    const int side = 2 * d + 1;
    const int t = u >> 1, which = u & 1;
    o0 = t / (side * side) - d;
    o1 = (t / side) % side - d;
    o2 = t % side - d;
    const int a0 = o0 < 0 ? -o0 : o0, a1 = o1 < 0 ? -o1 : o1, a2 = o2 < 0 ? -o2 : o2;
    const bool rim = a0 == d || a1 == d || a2 == d;
    if (rim) { zlo = which ? 1 : -d; zhi = which ? 0 : d; }     // second item of a rim line: empty
    else { zlo = zhi = which ? d : -d; }
}

// Cells of up to kRankMax points are put in order by ranking (every point counts the smaller
// ids of its cell); larger cells are sorted by a warp, beyond kWarpSortMaxShared by a CTA.
constexpr int kRankMax = 32;

constexpr size_t kGridHeaderBytes = 256;
// one int per query that k_knn_hard splits over several CTAs (at most as many as the launch has CTAs)
constexpr int kHardTickets = 1024;
constexpr size_t kHardTicketBytes = sizeof(int32_t) * kHardTickets;
static_assert(sizeof(KnnGrid) <= kGridHeaderBytes, "grid header too large");


// Byte offsets of the workspace sections (all 256-byte aligned).
struct KnnWorkspace {
    size_t header, tickets, counts, blocksums, pbin, prank, stmp, sorig, sbin, sflag, biglist, hugelist, scoords, total;
    int64_t cap_bins;   // capacity of the cell table (entries), host decision
    int nv;             // float4 per point in the sorted coordinate array
};

inline KnnWorkspace knn_workspace_layout(int64_t n_vert, int n_coords, int64_t n_rs, int K)
{
    (void)K;
    KnnWorkspace w;
    const int64_t n_events = n_rs > 1 ? n_rs - 1 : 1;
    int64_t cap = 16 * n_vert + 64 * n_events + 1024;
    if (cap > (int64_t)1 << 30) cap = (int64_t)1 << 30;
    if (cap < n_events) cap = n_events;
    w.cap_bins = cap;
    w.nv = (n_coords + 3) / 4;
    size_t off = 0;
    w.header = off; off += kGridHeaderBytes;
    w.tickets = off; off += kHardTicketBytes;     // cleared together with the header
    w.counts = off; off = align_up(off + sizeof(int32_t) * (size_t)(cap + 1), 256);
    w.blocksums = off; off = align_up(off + sizeof(int32_t) * (size_t)((cap + 1) / kScanTile + 2), 256);
    w.pbin = off; off = align_up(off + sizeof(int32_t) * (size_t)n_vert, 256);
    w.prank = off; off = align_up(off + sizeof(int32_t) * (size_t)n_vert, 256);
    w.stmp = off; off = align_up(off + sizeof(int32_t) * (size_t)n_vert, 256);
    w.sorig = off; off = align_up(off + sizeof(int32_t) * (size_t)n_vert, 256);
    w.sbin = off; off = align_up(off + sizeof(int32_t) * (size_t)n_vert, 256);
    w.sflag = off; off = align_up(off + (size_t)n_vert, 256);
    w.biglist = off; off = align_up(off + sizeof(int32_t) * (size_t)(n_vert / (kRankMax + 1) + 1), 256);
    w.hugelist = off; off = align_up(off + sizeof(int32_t) * (size_t)(n_vert / (kWarpSortMaxShared + 1) + 1), 256);
    w.scoords = off; off = align_up(off + sizeof(float4) * (size_t)n_vert * w.nv, 256);
    w.total = off;
    return w;
}

// Argument checks shared by the kNN entry points.
inline int check_knn_args(int64_t n_vert, int32_t n_coords, int64_t n_rs, int32_t K,
                          const void *workspace, size_t workspace_bytes, KnnWorkspace *L)
{
    if (n_vert < 0 || n_rs < 1) return FGC_ERR_BAD_ARGUMENT;
    if (n_vert > 0x7fffffff || n_rs > 0x7fffffff) return FGC_ERR_TOO_LARGE;
    if (n_coords < 2) return n_coords < 1 ? FGC_ERR_BAD_ARGUMENT : FGC_ERR_UNSUPPORTED_DIM;
    if (n_coords > FGC_MAX_KNN_DIMS) return FGC_ERR_UNSUPPORTED_DIM;
    if (K < 1 || K > FGC_MAX_K) return FGC_ERR_UNSUPPORTED_K;
    *L = knn_workspace_layout(n_vert, n_coords, n_rs, K);
    if (!workspace || workspace_bytes < L->total || ((uintptr_t)workspace & 255)) return FGC_ERR_WORKSPACE;
    return FGC_OK;
}

}  // namespace fgc
