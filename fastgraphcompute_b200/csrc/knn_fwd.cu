// binned_select_knn forward for sm_100a.
//
// Pipeline (all on the caller's stream, no host synchronisation):
//   k_minmax      fused finite check + min/max of the binned coordinates
//   k_grid_setup  cell width / grid shape from the extents and the point count
//   k_zero_counts clear the cell table
//   k_histogram   cell id per point, warp-aggregated atomic histogram; the value
//                 returned by the atomic is the point's rank inside its cell
//   k_scan_*      exclusive scan of the histogram -> cell boundaries
//   k_scatter     counting-sort scatter: coordinates (padded to float4), original
//                 id, cell id and direction flag in cell order
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

namespace fgc {

// ---------------------------------------------------------------------------
// grid construction
// ---------------------------------------------------------------------------

__global__ void __launch_bounds__(256)
k_minmax(const float *__restrict__ coords, int n_vert, int n_coords, int n_bin_dims, KnnGrid *g)
{
    uint32_t lmin[3] = {0, 0, 0}, lmax[3] = {0, 0, 0};
    uint32_t bad = 0;
    for (int v = blockIdx.x * blockDim.x + threadIdx.x; v < n_vert; v += gridDim.x * blockDim.x) {
        const float *row = coords + (size_t)v * n_coords;
        for (int c = 0; c < n_coords; c++) {
            const float x = __ldg(row + c);
            if (!is_finite_bits(x)) bad = 1;
            if (c < n_bin_dims) {
                const uint32_t k = float_to_ordered(x);
#pragma unroll
                for (int cc = 0; cc < 3; cc++)
                    if (cc == c) { lmin[cc] = max(lmin[cc], ~k); lmax[cc] = max(lmax[cc], k); }
            }
        }
    }
    __shared__ uint32_t s_min[3], s_max[3], s_bad;
    if (threadIdx.x < 3) { s_min[threadIdx.x] = 0; s_max[threadIdx.x] = 0; }
    if (threadIdx.x == 0) s_bad = 0;
    __syncthreads();
#pragma unroll
    for (int c = 0; c < 3; c++) {
        const uint32_t a = __reduce_max_sync(FGC_FULL_MASK, lmin[c]);
        const uint32_t b = __reduce_max_sync(FGC_FULL_MASK, lmax[c]);
        if ((threadIdx.x & 31) == 0) { atomicMax(&s_min[c], a); atomicMax(&s_max[c], b); }
    }
    if (__any_sync(FGC_FULL_MASK, bad) && (threadIdx.x & 31) == 0) atomicOr(&s_bad, 1u);
    __syncthreads();
    if (threadIdx.x < 3) {
        atomicMax(&g->min_key[threadIdx.x], s_min[threadIdx.x]);
        atomicMax(&g->max_key[threadIdx.x], s_max[threadIdx.x]);
    }
    if (threadIdx.x == 0 && s_bad) atomicOr(&g->nonfinite, 1u);
}

// One thread.  Chooses the cell width so that a row split of average size gets
// about bins_target cells, bounded by bins_cap cells per row split.
__global__ void k_grid_setup(KnnGrid *g, const int64_t *__restrict__ row_splits, int n_rs,
                             int n_vert, int n_bin_dims, int bins_target, int bins_cap)
{
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    int status = 0;
    if (g->nonfinite) status |= FGC_STATUS_NONFINITE;
    // row_splits must start at 0, end at n_vert and never decrease
    if (row_splits[0] != 0 || row_splits[n_rs - 1] != (int64_t)n_vert) status |= FGC_STATUS_BAD_ROW_SPLITS;
    for (int i = 1; i < n_rs; i++)
        if (row_splits[i] < row_splits[i - 1]) status |= FGC_STATUS_BAD_ROW_SPLITS;
    const int n_events = n_rs - 1;
    const int sh = 3 - n_bin_dims;
    float ext[3];
    double vol = 1.0;
    int nz = 0;
    float ext_max = 0.f;
    for (int gd = 0; gd < 3; gd++) {
        if (gd < sh || (status & FGC_STATUS_NONFINITE)) {
            g->cdim[gd] = gd < sh ? -1 : gd - sh;
            g->origin[gd] = 0.f;
            ext[gd] = 0.f;
        } else {
            const int c = gd - sh;
            const float lo = ordered_to_float(~g->min_key[c]);
            const float hi = ordered_to_float(g->max_key[c]);
            g->cdim[gd] = c;
            g->origin[gd] = lo;
            ext[gd] = __fsub_rn(hi, lo);
            if (!(ext[gd] >= 0.f) || !is_finite_bits(ext[gd])) ext[gd] = 0.f;
        }
        if (ext[gd] > 0.f) { vol *= (double)ext[gd]; nz++; }
        ext_max = fmaxf(ext_max, ext[gd]);
    }
    int n[3] = {1, 1, 1};
    float w = 1.f;
    if (nz > 0) {
        if (bins_target < 1) bins_target = 1;
        double wd = pow(vol / (double)bins_target, 1.0 / (double)nz);
        // a degenerate extent ratio can make the width underflow: keep it representable
        if (!(wd > (double)ext_max * 1e-6)) wd = (double)ext_max * 1e-6;
        for (int iter = 0; iter < 400; iter++) {
            w = (float)wd;
            const float inv = __fdiv_rn(1.0f, w);
            double prod = 1.0;
            for (int gd = 0; gd < 3; gd++) {
                n[gd] = ext[gd] > 0.f ? (int)floorf(__fmul_rn(ext[gd], inv)) + 1 : 1;
                prod *= (double)n[gd];
            }
            if (prod <= (double)bins_cap) break;
            wd *= 1.05;
        }
    }
    long long B = (long long)n[0] * n[1] * n[2];
    if (B > bins_cap) {  // cannot happen after the loop above unless the extents are absurd
        n[0] = n[1] = n[2] = 1; B = 1; w = fmaxf(ext_max, 1.f) * 2.f;
        status |= FGC_STATUS_INTERNAL;
    }
    g->n[0] = n[0]; g->n[1] = n[1]; g->n[2] = n[2];
    g->B = (int)B;
    g->n_events = n_events;
    g->total_bins = (int)(B * n_events);
    g->w = w;
    g->inv_w = __fdiv_rn(1.0f, w);
    g->slack = 4e-6f * fmaxf(ext_max, w);
    g->status = status;
}

__global__ void __launch_bounds__(256) k_zero_counts(int *__restrict__ counts, const KnnGrid *g)
{
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

__global__ void __launch_bounds__(256)
k_histogram(const float *__restrict__ coords, int n_vert, int n_coords,
            const int64_t *__restrict__ row_splits, int n_rs, const KnnGrid *__restrict__ g,
            int *__restrict__ counts, int *__restrict__ pbin, int *__restrict__ prank)
{
    const int v = blockIdx.x * blockDim.x + threadIdx.x;
    const bool live = v < n_vert && g->status == 0;
    int flat = 0;
    if (live) {
        const float *row = coords + (size_t)v * n_coords;
        int b[3];
#pragma unroll
        for (int gd = 0; gd < 3; gd++) {
            const int c = g->cdim[gd];
            b[gd] = c < 0 ? 0 : cell_of(__ldg(row + c), g->origin[gd], g->inv_w, g->n[gd]);
        }
        const int e = row_split_of(row_splits, n_rs, v);
        flat = e * g->B + (b[0] * g->n[1] + b[1]) * g->n[2] + b[2];
    }
    const unsigned active = __ballot_sync(FGC_FULL_MASK, live);
    if (live) {
        // warp-aggregated: one atomic per distinct cell in the warp
        const unsigned peers = __match_any_sync(active, flat);
        const int leader = __ffs(peers) - 1;
        int base = 0;
        if ((int)(threadIdx.x & 31) == leader) base = atomicAdd(counts + flat, __popc(peers));
        base = __shfl_sync(peers, base, leader);
        pbin[v] = flat;
        prank[v] = base + __popc(peers & lanemask_lt());
    }
}

// --- exclusive scan of counts[0 .. total_bins] in place (three kernels) -------

__global__ void __launch_bounds__(256)
k_scan_tile_sums(const int *__restrict__ counts, const KnnGrid *__restrict__ g,
                 int *__restrict__ blocksums)
{
    const int n = g->total_bins + 1;
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

// Single block: exclusive scan of the tile sums.
__global__ void __launch_bounds__(1024)
k_scan_block_sums(int *__restrict__ blocksums, const KnnGrid *__restrict__ g)
{
    const int n = (g->total_bins + 1 + kScanTile - 1) / kScanTile;
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

__global__ void __launch_bounds__(256)
k_scan_apply(int *__restrict__ counts, const KnnGrid *__restrict__ g,
             const int *__restrict__ blocksums)
{
    const int n = g->total_bins + 1;
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

__global__ void __launch_bounds__(256)
k_scatter(const float *__restrict__ coords, int n_vert, int n_coords, int nv,
          const int64_t *__restrict__ direction, const KnnGrid *__restrict__ g,
          const int *__restrict__ bounds, const int *__restrict__ pbin,
          const int *__restrict__ prank, float4 *__restrict__ scoords, int *__restrict__ sorig,
          int *__restrict__ sbin, uint8_t *__restrict__ sflag)
{
    const int v = blockIdx.x * blockDim.x + threadIdx.x;
    if (v >= n_vert || g->status != 0) return;
    const int b = pbin[v];
    const int pos = bounds[b] + prank[v];
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
    sbin[pos] = b;
    if (direction) {
        const int64_t d = direction[v];
        sflag[pos] = (d >= 0 && d <= 2) ? (uint8_t)d : (uint8_t)3;
    }
}

// ---------------------------------------------------------------------------
// search
// ---------------------------------------------------------------------------

struct KnnArgs {
    const float4 *scoords;
    const int *sorig;
    const int *sbin;
    const uint8_t *sflag;   // nullptr: no direction restriction
    const int *bounds;      // cell boundaries, total_bins + 1 entries
    const KnnGrid *grid;
    int64_t *out_idx;
    float *out_dist;
    int n_vert;
    int K;
    int n_coords;
    int tf_compat;
    int count_evals;
};

constexpr int kKnnWarps = 8;
constexpr uint32_t kInfBits = 0x7f800000u;

// Squared distance over NV float4 chunks; padded components are 0 in both
// operands and add an exact 0.  Order and rounding: acc = acc + (a-b)*(a-b) per
// dimension, dimension 0 first, no fused multiply-add.
template <int NV>
__device__ __forceinline__ float dist_sq(const float4 (&q)[NV], const float4 (&c)[NV], int n_coords)
{
    float acc = 0.f;
#pragma unroll
    for (int v = 0; v < NV; v++) {
        float d;
        d = __fsub_rn(q[v].x, c[v].x); acc = __fadd_rn(acc, __fmul_rn(d, d));
        if (4 * v + 1 < n_coords) { d = __fsub_rn(q[v].y, c[v].y); acc = __fadd_rn(acc, __fmul_rn(d, d)); }
        if (4 * v + 2 < n_coords) { d = __fsub_rn(q[v].z, c[v].z); acc = __fadd_rn(acc, __fmul_rn(d, d)); }
        if (4 * v + 3 < n_coords) { d = __fsub_rn(q[v].w, c[v].w); acc = __fadd_rn(acc, __fmul_rn(d, d)); }
    }
    return acc;
}

// The per-warp neighbour list: slot s = lane*R + r (r < R) is valid when s < K-1.
// Empty valid slots hold +inf, invalid slots hold +0 and are never chosen.  The
// threshold tau is the largest stored distance (compared through the bit
// pattern, which is monotone for non-negative floats), so "unfilled" needs no
// separate bookkeeping: while a slot is empty tau is +inf and every candidate
// replaces the first empty slot; afterwards a candidate replaces the first slot
// that holds tau iff its distance is strictly smaller.
template <int R>
struct NeighbourList {
    float d[R];
    int id[R];
    uint32_t lmax;   // max bit pattern over this lane's slots
    uint32_t tau;    // max over the warp

    __device__ __forceinline__ void init(int lane, int kn)
    {
        lmax = 0;
#pragma unroll
        for (int r = 0; r < R; r++) {
            d[r] = (lane * R + r < kn) ? __uint_as_float(kInfBits) : 0.f;
            id[r] = -1;
            lmax = max(lmax, __float_as_uint(d[r]));
        }
        tau = __reduce_max_sync(FGC_FULL_MASK, lmax);
    }

    // Warp-uniform: insert candidate (dc, jc) if dc < tau.
    __device__ __forceinline__ void offer(int lane, float dc, int jc)
    {
        if (__float_as_uint(dc) < tau) {
            const unsigned holders = __ballot_sync(FGC_FULL_MASK, lmax == tau);
            if (lane == __ffs(holders) - 1) {
                bool done = false;
                uint32_t m = 0;
#pragma unroll
                for (int r = 0; r < R; r++) {
                    if (!done && __float_as_uint(d[r]) == tau) { d[r] = dc; id[r] = jc; done = true; }
                    m = max(m, __float_as_uint(d[r]));
                }
                lmax = m;
            }
            tau = __reduce_max_sync(FGC_FULL_MASK, lmax);
        }
    }
};

template <int NV, int R>
__global__ void __launch_bounds__(kKnnWarps * 32)
k_knn(const KnnArgs a)
{
    __shared__ int s_delta[kKnnWarps][32];
    const int lane = threadIdx.x & 31;
    const int wib = threadIdx.x >> 5;
    const int qi = blockIdx.x * kKnnWarps + wib;   // position in cell order
    const KnnGrid *__restrict__ g = a.grid;
    if (qi >= a.n_vert || g->status != 0) return;

    const int K = a.K, kn = K - 1;
    const int nc = a.n_coords;
    const uint8_t *__restrict__ sflag = a.sflag;
    const int orig_q = __ldg(a.sorig + qi);
    int64_t *__restrict__ out_i = a.out_idx + (size_t)orig_q * K;
    float *__restrict__ out_d = a.out_dist + (size_t)orig_q * K;

    // queries that may not have neighbours keep the default row
    const bool q_inactive = sflag && (sflag[qi] == 0 || sflag[qi] == 2);

    float4 q[NV];
#pragma unroll
    for (int v = 0; v < NV; v++) q[v] = __ldg(a.scoords + (size_t)qi * NV + v);

    NeighbourList<R> list;
    list.init(lane, kn);
    unsigned long long evals = 0;

    // one chunk of up to 32 candidates: lane evaluates sorted position j
    auto process = [&](int j, bool act) {
        float dc = __uint_as_float(kInfBits);
        if (act) {
            float4 c[NV];
#pragma unroll
            for (int v = 0; v < NV; v++) c[v] = __ldg(a.scoords + (size_t)j * NV + v);
            bool ok = j != qi;
            if (sflag) { const uint8_t f = sflag[j]; ok = ok && f != 1 && f != 2; }
            if (ok) dc = dist_sq<NV>(q, c, nc);
        }
        if (a.count_evals) evals += act ? 1 : 0;
        unsigned m = __ballot_sync(FGC_FULL_MASK, __float_as_uint(dc) < list.tau);
        while (m) {
            const int src = __ffs(m) - 1;
            m &= m - 1;
            const float dcs = __shfl_sync(FGC_FULL_MASK, dc, src);
            const int js = __shfl_sync(FGC_FULL_MASK, j, src);
            list.offer(lane, dcs, js);
        }
    };

    if (!q_inactive && kn > 0) {
        const int B = g->B, n0 = g->n[0], n1 = g->n[1], n2 = g->n[2];
        const int flat = __ldg(a.sbin + qi);
        const int e = flat / B;
        int rem = flat - e * B;
        const int b0 = rem / (n1 * n2);
        rem -= b0 * n1 * n2;
        const int b1 = rem / n2;
        const int b2 = rem - b1 * n2;
        const int ev_begin = __ldg(a.bounds + e * B);
        const int ev_end = __ldg(a.bounds + (e + 1) * B);
        const int n_e = ev_end - ev_begin;

        bool brute = n_e <= 512 || n_e <= 8 * K;
        if (!brute) {
            const float w = g->w, slack = g->slack;
            // query position relative to the grid origin, per grid dimension
            float qr[3];
            {
                const float qc[3] = {q[0].x, q[0].y, q[0].z};
#pragma unroll
                for (int gd = 0; gd < 3; gd++) {
                    const int c = g->cdim[gd];
                    const float x = c == 0 ? qc[0] : (c == 1 ? qc[1] : qc[2]);
                    qr[gd] = c < 0 ? 0.f : __fsub_rn(x, g->origin[gd]);
                }
            }
            // lower edge of cell b / upper edge of cell b-1, widened by a relative 1e-6
            auto edge_lo = [&](int b) { return (float)b * w * (1.0f - 1e-6f); };
            auto edge_hi = [&](int b) { return (float)b * w * (1.0f + 1e-6f); };
            // distance from the query to the slab of cells [lo, hi] of grid dimension gd
            auto gap_to = [&](int lo, int hi, int bq, float qrel) {
                float gp = 0.f;
                if (lo > bq) gp = edge_lo(lo) - qrel - slack;
                else if (hi < bq) gp = qrel - edge_hi(hi + 1) - slack;
                return fmaxf(gp, 0.f);
            };
            long long items_done = 0;
            for (int d = 0;; ++d) {
                const int side = 2 * d + 1, half = 2 * d - 1;
                const int n_ring = d == 0 ? 1 : 8 * d;
                const int n_items = d == 0 ? 1 : n_ring + 2 * half * half;
                for (int base = 0; base < n_items; base += 32) {
                    const int u = base + lane;
                    bool valid = u < n_items;
                    int o0 = 0, o1 = 0, zlo = b2, zhi = b2;
                    if (d > 0) {
                        if (u < n_ring) {
                            if (u < side) { o0 = -d; o1 = u - d; }
                            else if (u < 2 * side) { o0 = d; o1 = u - side - d; }
                            else {
                                const int t = u - 2 * side;
                                if (t < half) { o1 = -d; o0 = t - (d - 1); }
                                else { o1 = d; o0 = t - half - (d - 1); }
                            }
                            zlo = b2 - d; zhi = b2 + d;
                        } else {
                            const int cidx = u - n_ring;
                            const int t = cidx >> 1;
                            const int tq = t / half;
                            o0 = tq - (d - 1);
                            o1 = t - tq * half - (d - 1);
                            zlo = zhi = (cidx & 1) ? b2 + d : b2 - d;
                        }
                    }
                    const int g0 = b0 + o0, g1 = b1 + o1;
                    valid = valid && g0 >= 0 && g0 < n0 && g1 >= 0 && g1 < n1;
                    zlo = max(zlo, 0);
                    zhi = min(zhi, n2 - 1);
                    valid = valid && zlo <= zhi;
                    if (valid && list.tau < kInfBits) {
                        const float ga = gap_to(g0, g0, b0, qr[0]);
                        const float gb = gap_to(g1, g1, b1, qr[1]);
                        const float gc = gap_to(zlo, zhi, b2, qr[2]);
                        const float md = ga * ga + gb * gb + gc * gc;
                        if (md > __uint_as_float(list.tau) * 1.00001f) valid = false;
                    }
                    int start = 0, len = 0;
                    if (valid) {
                        const int rowbase = e * B + (g0 * n1 + g1) * n2;
                        start = __ldg(a.bounds + rowbase + zlo);
                        len = __ldg(a.bounds + rowbase + zhi + 1) - start;
                    }
                    const unsigned nzm = __ballot_sync(FGC_FULL_MASK, len > 0);
                    if (nzm == 0) continue;
                    int incl = len;
#pragma unroll
                    for (int o = 1; o < 32; o <<= 1) {
                        const int t = __shfl_up_sync(FGC_FULL_MASK, incl, o);
                        if (lane >= o) incl += t;
                    }
                    const int T = __shfl_sync(FGC_FULL_MASK, incl, 31);
                    const int pprev = incl - len;
                    if (len > 0) s_delta[wib][__popc(nzm & lanemask_lt())] = start - pprev;
                    __syncwarp();
                    int rbase = 0;
                    for (int t = 0; t < T; t += 32) {
                        const int rel = pprev - t;
                        const unsigned contrib = (len > 0 && rel >= 0 && rel < 32) ? (1u << rel) : 0u;
                        const unsigned M = __reduce_or_sync(FGC_FULL_MASK, contrib);
                        const int c = t + lane;
                        const int r = rbase + __popc(M & lanemask_le()) - 1;
                        rbase += __popc(M);
                        const bool act = c < T;
                        const int j = act ? c + s_delta[wib][r] : -1;
                        process(j, act);
                    }
                    __syncwarp();
                }
                items_done += n_items;
                // everything outside the cube of radius d is at least fd away
                float fd = __uint_as_float(kInfBits);
                bool any = false;
                {
                    const int bq[3] = {b0, b1, b2};
                    const int nn[3] = {n0, n1, n2};
#pragma unroll
                    for (int gd = 0; gd < 3; gd++) {
                        const int hi = bq[gd] + d + 1, lo = bq[gd] - d - 1;
                        if (hi <= nn[gd] - 1) { fd = fminf(fd, fmaxf(edge_lo(hi) - qr[gd] - slack, 0.f)); any = true; }
                        if (lo >= 0) { fd = fminf(fd, fmaxf(qr[gd] - edge_hi(lo + 1) - slack, 0.f)); any = true; }
                    }
                }
                if (!any) break;
                if (list.tau < kInfBits && fd * fd > __uint_as_float(list.tau) * 1.00001f) break;
                // walking mostly empty cells: scanning the whole row split is cheaper
                if (items_done * 8 > (long long)n_e) { brute = true; break; }
            }
            if (brute) list.init(lane, kn);
        }
        if (brute) {
            for (int t = 0; t < n_e; t += 32) {
                const int c = t + lane;
                process(ev_begin + c, c < n_e);
            }
        }
    }

    // epilogue: original ids, original row position
    if (lane == 0) { out_i[0] = orig_q; out_d[0] = 0.f; }
    const int64_t pad = a.tf_compat ? (int64_t)orig_q : (int64_t)-1;
#pragma unroll
    for (int r = 0; r < R; r++) {
        const int s = lane * R + r;
        if (s < kn) {
            const bool filled = __float_as_uint(list.d[r]) < kInfBits && list.id[r] >= 0;
            out_i[1 + s] = filled ? (int64_t)__ldg(a.sorig + list.id[r]) : pad;
            out_d[1 + s] = filled ? list.d[r] : 0.f;
        }
    }
    if (a.count_evals) {
        evals = __reduce_add_sync(FGC_FULL_MASK, (unsigned)evals);
        if (lane == 0) atomicAdd((unsigned long long *)&g->n_evals, evals);
    }
}

template <int NV>
static int launch_knn_nv(const KnnArgs &a, cudaStream_t s)
{
    const int kn = a.K - 1;
    const unsigned blocks = (unsigned)((a.n_vert + kKnnWarps - 1) / kKnnWarps);
    const int R = (kn + 31) / 32;
    if (R <= 1) k_knn<NV, 1><<<blocks, kKnnWarps * 32, 0, s>>>(a);
    else if (R <= 2) k_knn<NV, 2><<<blocks, kKnnWarps * 32, 0, s>>>(a);
    else if (R <= 4) k_knn<NV, 4><<<blocks, kKnnWarps * 32, 0, s>>>(a);
    else k_knn<NV, 8><<<blocks, kKnnWarps * 32, 0, s>>>(a);
    return (int)cudaGetLastError();
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

namespace fgc {

static int check_knn_args(int64_t n_vert, int32_t n_coords, const int64_t *row_splits, int64_t n_rs,
                          int32_t K, const void *workspace, size_t workspace_bytes, KnnWorkspace *L)
{
    if (n_vert < 0 || n_rs < 1 || !row_splits) return FGC_ERR_BAD_ARGUMENT;
    if (n_vert > 0x7fffffff || n_rs > 0x7fffffff) return FGC_ERR_TOO_LARGE;
    if (n_coords < 2) return n_coords < 1 ? FGC_ERR_BAD_ARGUMENT : FGC_ERR_UNSUPPORTED_DIM;
    if (n_coords > 8) return FGC_ERR_UNSUPPORTED_DIM;
    if (K < 1 || K > FGC_MAX_K) return FGC_ERR_UNSUPPORTED_K;
    *L = knn_workspace_layout(n_vert, n_coords, n_rs, K);
    if (!workspace || workspace_bytes < L->total || ((uintptr_t)workspace & 255)) return FGC_ERR_WORKSPACE;
    return FGC_OK;
}

}  // namespace fgc

extern "C" int fgc_knn_build_grid(const float *coords, int64_t n_vert, int32_t n_coords,
                                  const int64_t *row_splits, int64_t n_rs, int32_t K,
                                  const int64_t *direction_or_null, float target_occupancy,
                                  void *workspace, size_t workspace_bytes, fgc_stream_t stream)
{
    using namespace fgc;
    KnnWorkspace L;
    const int rc = check_knn_args(n_vert, n_coords, row_splits, n_rs, K, workspace, workspace_bytes, &L);
    if (rc != FGC_OK) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    char *ws = (char *)workspace;
    KnnGrid *grid = (KnnGrid *)(ws + L.header);
    FGC_RETURN_IF_CUDA(cudaMemsetAsync(grid, 0, kGridHeaderBytes, s));
    if (n_vert == 0) return FGC_OK;
    if (!coords || n_rs < 2) return FGC_ERR_BAD_ARGUMENT;

    int *counts = (int *)(ws + L.counts);
    int *blocksums = (int *)(ws + L.blocksums);
    int *pbin = (int *)(ws + L.pbin);
    int *prank = (int *)(ws + L.prank);
    int *sorig = (int *)(ws + L.sorig);
    int *sbin = (int *)(ws + L.sbin);
    uint8_t *sflag = (uint8_t *)(ws + L.sflag);
    float4 *scoords = (float4 *)(ws + L.scoords);

    const int n = (int)n_vert;
    const int n_events = (int)n_rs - 1;
    const int n_bin_dims = n_coords < 3 ? n_coords : 3;
    if (!(target_occupancy > 0.f)) target_occupancy = 2.0f;
    const int64_t bins_cap64 = L.cap_bins / n_events;
    const int bins_cap = (int)(bins_cap64 < 1 ? 1 : bins_cap64);
    const double bt = (double)n_vert / (double)n_events / (double)target_occupancy;
    int bins_target = bt >= (double)bins_cap ? bins_cap : (int)(bt + 0.5);
    if (bins_target < 1) bins_target = 1;

    const int pt_blocks = (n + 255) / 256;
    const int red_blocks = pt_blocks < 148 * 4 ? pt_blocks : 148 * 4;
    k_minmax<<<red_blocks, 256, 0, s>>>(coords, n, n_coords, n_bin_dims, grid);
    FGC_CHECK_LAUNCH();
    k_grid_setup<<<1, 32, 0, s>>>(grid, row_splits, (int)n_rs, n, n_bin_dims, bins_target, bins_cap);
    FGC_CHECK_LAUNCH();
    // The cell count is only known on the device: the scan grids are sized for the
    // largest table k_grid_setup may choose and surplus blocks return at once.
    const int64_t max_entries = (int64_t)bins_cap * n_events + 1;
    const int scan_blocks = (int)ceil_div64(max_entries, kScanTile);
    k_zero_counts<<<148 * 4, 256, 0, s>>>(counts, grid);
    FGC_CHECK_LAUNCH();
    k_histogram<<<pt_blocks, 256, 0, s>>>(coords, n, n_coords, row_splits, (int)n_rs, grid, counts,
                                          pbin, prank);
    FGC_CHECK_LAUNCH();
    k_scan_tile_sums<<<scan_blocks, 256, 0, s>>>(counts, grid, blocksums);
    FGC_CHECK_LAUNCH();
    k_scan_block_sums<<<1, 1024, 0, s>>>(blocksums, grid);
    FGC_CHECK_LAUNCH();
    k_scan_apply<<<scan_blocks, 256, 0, s>>>(counts, grid, blocksums);
    FGC_CHECK_LAUNCH();
    k_scatter<<<pt_blocks, 256, 0, s>>>(coords, n, n_coords, L.nv, direction_or_null, grid, counts,
                                        pbin, prank, scoords, sorig, sbin, sflag);
    FGC_CHECK_LAUNCH();
    return FGC_OK;
}

extern "C" int fgc_knn_search(int64_t n_vert, int32_t n_coords, int64_t n_rs, int32_t K,
                              int32_t has_direction, int32_t tf_compat, int32_t count_evals,
                              int64_t *out_idx, float *out_distsq, void *workspace,
                              size_t workspace_bytes, fgc_stream_t stream)
{
    using namespace fgc;
    KnnWorkspace L;
    static const int64_t dummy_rs = 0;
    const int rc = check_knn_args(n_vert, n_coords, &dummy_rs, n_rs, K, workspace, workspace_bytes, &L);
    if (rc != FGC_OK) return rc;
    if (n_vert == 0) return FGC_OK;
    if (!out_idx || !out_distsq) return FGC_ERR_BAD_ARGUMENT;
    char *ws = (char *)workspace;
    KnnArgs a;
    a.scoords = (const float4 *)(ws + L.scoords);
    a.sorig = (const int *)(ws + L.sorig);
    a.sbin = (const int *)(ws + L.sbin);
    a.sflag = has_direction ? (const uint8_t *)(ws + L.sflag) : nullptr;
    a.bounds = (const int *)(ws + L.counts);
    a.grid = (const KnnGrid *)(ws + L.header);
    a.out_idx = out_idx;
    a.out_dist = out_distsq;
    a.n_vert = (int)n_vert;
    a.K = K;
    a.n_coords = n_coords;
    a.tf_compat = tf_compat;
    a.count_evals = count_evals;
    const int lrc = L.nv == 1 ? launch_knn_nv<1>(a, (cudaStream_t)stream)
                              : launch_knn_nv<2>(a, (cudaStream_t)stream);
    return lrc;
}

extern "C" int fgc_binned_knn_fwd(const float *coords, int64_t n_vert, int32_t n_coords,
                                  const int64_t *row_splits, int64_t n_rs, int32_t K,
                                  const int64_t *direction_or_null, int32_t tf_compat,
                                  float target_occupancy, int64_t *out_idx, float *out_distsq,
                                  void *workspace, size_t workspace_bytes, fgc_stream_t stream)
{
    int rc = fgc_knn_build_grid(coords, n_vert, n_coords, row_splits, n_rs, K, direction_or_null,
                                target_occupancy, workspace, workspace_bytes, stream);
    if (rc != FGC_OK) return rc;
    return fgc_knn_search(n_vert, n_coords, n_rs, K, direction_or_null != nullptr, tf_compat, 0,
                          out_idx, out_distsq, workspace, workspace_bytes, stream);
}

extern "C" int fgc_knn_read_counters(const void *workspace, uint64_t *n_evals_host,
                                     int32_t *grid_shape_host, float *cell_width_host,
                                     fgc_stream_t stream)
{
    using namespace fgc;
    if (!workspace) return FGC_ERR_BAD_ARGUMENT;
    KnnGrid h;
    cudaStream_t s = (cudaStream_t)stream;
    FGC_RETURN_IF_CUDA(cudaMemcpyAsync(&h, workspace, sizeof(KnnGrid), cudaMemcpyDeviceToHost, s));
    FGC_RETURN_IF_CUDA(cudaStreamSynchronize(s));
    if (n_evals_host) *n_evals_host = h.n_evals;
    if (grid_shape_host) { grid_shape_host[0] = h.n[0]; grid_shape_host[1] = h.n[1]; grid_shape_host[2] = h.n[2]; }
    if (cell_width_host) *cell_width_host = h.w;
    return FGC_OK;
}
