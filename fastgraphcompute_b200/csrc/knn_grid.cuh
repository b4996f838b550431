// Internal search grid of the kNN: layout of the workspace and the record that
// describes the grid (written on the device, read by every later kernel).
//
// The search grid is private to this library.  The k nearest neighbours of a
// point do not depend on how space is binned, so the grid is chosen for the
// GPU (cell size from the point density, up to three binned dimensions) and not
// from the reference's n_bins / max_bin_dims arguments.
#pragma once
#include "fgc_common.cuh"

namespace fgc {

// Grid over up to three coordinate dimensions.  Grid dimension g uses
// coordinate dimension cdim[g]; unused leading grid dimensions have n = 1.
// Cell (e, b0, b1, b2) of row split e has flat id e*B + (b0*n[1] + b1)*n[2] + b2,
// so the cells of one (e, b0, b1) line are consecutive and, after the counting
// sort, so are their points.
struct KnnGrid {
    int32_t status;        // FGC_STATUS_* bits (first word of the workspace)
    int32_t n_events;
    int32_t n[3];          // cells per grid dimension
    int32_t cdim[3];       // coordinate dimension of grid dimension g, -1 = unused
    int32_t B;             // cells per row split = n[0]*n[1]*n[2]
    int32_t total_bins;    // n_events * B
    float origin[3];       // global minimum of the coordinate
    float w;               // cell width
    float inv_w;           // 1 / w
    float slack;           // absolute safety margin for cell-distance bounds
    uint32_t min_key[3];   // ~ordered(min) per binned coordinate (atomicMax)
    uint32_t max_key[3];   // ordered(max)
    uint32_t nonfinite;    // set when any coordinate is NaN/Inf
    unsigned long long n_evals;  // distance evaluations (debug counter, optional)
};

constexpr size_t kGridHeaderBytes = 256;
static_assert(sizeof(KnnGrid) <= kGridHeaderBytes, "grid header too large");

constexpr int kScanTile = 2048;  // elements per block in the 3-kernel scan

// Byte offsets of the workspace sections (all 256-byte aligned).
struct KnnWorkspace {
    size_t header, counts, blocksums, pbin, prank, sorig, sbin, sflag, scoords, total;
    int64_t cap_bins;   // capacity of the cell table (entries), host decision
    int nv;             // float4 per point in the sorted coordinate array
};

inline KnnWorkspace knn_workspace_layout(int64_t n_vert, int n_coords, int64_t n_rs, int K)
{
    (void)K;
    KnnWorkspace w;
    const int64_t n_events = n_rs > 1 ? n_rs - 1 : 1;
    int64_t cap = 8 * n_vert + 64 * n_events + 1024;
    if (cap > (int64_t)1 << 30) cap = (int64_t)1 << 30;
    if (cap < n_events) cap = n_events;
    w.cap_bins = cap;
    w.nv = (n_coords + 3) / 4;
    size_t off = 0;
    w.header = off; off += kGridHeaderBytes;
    w.counts = off; off = align_up(off + sizeof(int32_t) * (size_t)(cap + 1), 256);
    w.blocksums = off; off = align_up(off + sizeof(int32_t) * (size_t)((cap + 1) / kScanTile + 2), 256);
    w.pbin = off; off = align_up(off + sizeof(int32_t) * (size_t)n_vert, 256);
    w.prank = off; off = align_up(off + sizeof(int32_t) * (size_t)n_vert, 256);
    w.sorig = off; off = align_up(off + sizeof(int32_t) * (size_t)n_vert, 256);
    w.sbin = off; off = align_up(off + sizeof(int32_t) * (size_t)n_vert, 256);
    w.sflag = off; off = align_up(off + (size_t)n_vert, 256);
    w.scoords = off; off = align_up(off + sizeof(float4) * (size_t)n_vert * w.nv, 256);
    w.total = off;
    return w;
}

}  // namespace fgc
