// Memory layout of the reverse neighbour graph built by fgc_build_reverse_graph
// (reverse_graph.cu): offsets [n_vert+1], cursor, scan scratch, entries [n_vert*K] (i*K + k of
// every pair that lists the point, each segment sorted).
#pragma once
#include "scan.cuh"

namespace fgc {

struct ReverseGraphLayout {
    size_t offsets, cursor, blocksums, entries, total;
};

inline ReverseGraphLayout reverse_graph_layout(int64_t n_vert, int K)
{
    ReverseGraphLayout L;
    size_t off = 0;
    L.offsets = off; off = align_up(off + sizeof(int32_t) * (size_t)(n_vert + 1), 256);
    L.cursor = off; off = align_up(off + sizeof(int32_t) * (size_t)(n_vert + 1), 256);
    L.blocksums = off; off = align_up(off + sizeof(int32_t) * (size_t)((n_vert + 1) / kScanTile + 2), 256);
    L.entries = off; off = align_up(off + sizeof(int32_t) * (size_t)n_vert * K, 256);
    L.total = off;
    return L;
}

}  // namespace fgc
