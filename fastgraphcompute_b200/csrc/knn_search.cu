// binned_select_knn forward for sm_100a, part 2: the neighbour search on a built grid
// (knn_grid.cu builds it).
//
// One warp per query point.  The warp walks the cells around the query's cell in
// expanding Chebyshev shells.  A shell is described as "items" -- runs of cells along
// the last grid dimension, each a contiguous range of cell-sorted points -- and 32 items
// are looked up at once (one per lane: bounds check, distance-to-box pruning against the
// current K-th distance, two loads of the cell boundaries).  The non-empty ranges of a
// batch are then treated as one flattened candidate stream: every step each lane takes
// the next candidate (a 16-byte load per float4 of coordinates), evaluates the squared
// distance and the warp votes on which candidates beat the current K-th distance.  The
// K-1 best live in registers, spread over the lanes.  The search of a query ends as soon
// as the cube of cells it has covered contains the ball of its K-th distance.
//
// The grid spans the first three coordinates (D <= 3: items are (o0, o1, run)) or the first
// four (D >= 4: items are (o0, o1, o2, run)); for D = 4 the grid build picks one of the two on
// the device (knn_grid.cu: strongly clustered data goes to three) and the kernel branches once.
//
// What is computed is what the reference's CPU path computes
// (extensions/binned_knn_autograd_kernel.cpp:85-209 with
// extensions/binned_select_knn_cpu.cpp:56-208): per row split, the K-1 nearest other
// points, strict "<" replacement of the current worst (so among equal distances the one
// visited first stays), squared distances accumulated over the dimensions in order with
// one rounding per operation.  Visiting order, grid and stopping rule are this library's
// own; they never change which points are nearest, only which of several equidistant
// points is kept.
#include <type_traits>

#include "knn_grid.cuh"
#include "shell_table.cuh"

namespace fgc {

struct KnnArgs {
    const float4 *scoords;
    const int *sorig;
    const int *sbin;
    const uint8_t *sflag;   // nullptr: no direction restriction
    const int *bounds;      // cell boundaries, total_bins + 1 entries
    int *hardlist;          // queries handed over to k_knn_hard (cell-order positions)
    float *hard_parts;      // k_knn_hard: partial lists of queries that several CTAs share
    size_t hard_parts_bytes;
    int *hard_tickets;      // k_knn_hard: finished parts per listed query (zero at launch)
    KnnGrid *grid;
    int64_t *out_idx;
    float *out_dist;
    int n_vert;
    int K;
    int n_coords;
    int tf_compat;
    int count_evals;
};

// Resident CTAs per SM asked of the compiler, per list size (the launch bounds of k_knn).  The
// search fills 85-89 % of the issue slots only when enough warps are resident to cover the
// dependent loads of cell boundaries and candidates, so more resident warps beat fewer
// registers spilled to L1: measured on B200, each step up to these values was faster, and more
// registers with fewer CTAs slower.  The number of warps per CTA (8, 4 or 2 at the same
// residency) makes no measurable difference.
constexpr int kKnnWarps = 8;
constexpr uint32_t kInfBits = 0x7f800000u;
// A query that walks mostly empty cells gives up and scans its whole row split.  In a row split
// of more than kHardMin points that scan is thousands of steps for ONE warp, which then runs on
// alone after every other query has finished; such queries are collected instead and searched
// by a whole CTA each (k_knn_hard).
constexpr int kHardMin = 4096;

// Squared distance over NV float4 chunks.  Order and rounding: acc = acc + (a-b)*(a-b)
// per dimension, dimension 0 first, no fused multiply-add; the first term needs no add.
// The coordinates beyond n_coords are stored as 0 on both sides, so their terms are +0 and adding
// them changes no bit: all 4 NV components are computed, the differences and squares two at a
// time with the packed fp32x2 instructions of sm_100 (same rounding as the scalar ones).
__device__ __forceinline__ void sq_diff_f32x2(float a0, float a1, float b0, float b1, float &s0, float &s1)
{
    unsigned long long d, s;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(pack_f32x2(a0, a1)), "l"(pack_f32x2(b0, b1)));
    asm("mul.rn.f32x2 %0, %1, %1;" : "=l"(s) : "l"(d));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(s0), "=f"(s1) : "l"(s));
}
template <int NV>
__device__ __forceinline__ float dist_sq(const float4 (&q)[NV], const float4 (&c)[NV], int n_coords)
{
    (void)n_coords;
    float acc = 0.f;
#pragma unroll
    for (int v = 0; v < NV; v++) {
        float s0, s1, s2, s3;
        sq_diff_f32x2(q[v].x, q[v].y, c[v].x, c[v].y, s0, s1);
        sq_diff_f32x2(q[v].z, q[v].w, c[v].z, c[v].w, s2, s3);
        acc = v == 0 ? s0 : __fadd_rn(acc, s0);
        acc = __fadd_rn(acc, s1);
        acc = __fadd_rn(acc, s2);
        acc = __fadd_rn(acc, s3);
    }
    return acc;
}

// The per-warp neighbour list: slot s = lane*R + r (r < R) is valid when s < K-1.
// Empty valid slots hold +inf, invalid slots hold +0 and are never chosen.  tau is the
// largest stored distance, compared through the bit pattern (monotone for non-negative
// floats), so while a slot is empty tau is +inf and every candidate goes to the first
// empty slot; afterwards a candidate replaces the first slot that holds tau iff its
// distance is strictly smaller.  With R >= 2 slots fill in slot order (empty slots are a
// suffix, which the bulk placement relies on); with R == 1 any empty slot may be taken.
template <int R>
struct NeighbourList {
    float d[R];
    int id[R];
    uint32_t lmax;   // max bit pattern over this lane's slots
    uint32_t tau;    // max over the warp
    int filled;      // number of occupied slots (warp-uniform)

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
        filled = 0;
    }

    __device__ __forceinline__ void refresh(int lane)
    {
        uint32_t m = 0;
#pragma unroll
        for (int r = 0; r < R; r++) m = max(m, __float_as_uint(d[r]));
        lmax = m;
        tau = __reduce_max_sync(FGC_FULL_MASK, lmax);
    }

    // Warp-uniform: insert candidate (dc, jc) if dc < tau.  Returns 1 if inserted.
    __device__ __forceinline__ int offer(int lane, float dc, int jc)
    {
        if (__float_as_uint(dc) >= tau) return 0;
        // the first lane that holds tau takes the candidate (no find-first needed: it is the
        // holder without a holder below it)
        const bool holds = lmax == tau;
        const unsigned holders = __ballot_sync(FGC_FULL_MASK, holds);
        if (holds && (holders & lanemask_lt()) == 0) {
            bool done = false;
            uint32_t m = 0;
#pragma unroll
            for (int r = 0; r < R; r++) {
                if (!done && __float_as_uint(d[r]) == tau) { d[r] = dc; id[r] = jc; done = true; }
                m = max(m, __float_as_uint(d[r]));
            }
            lmax = m;
        }
        filled += tau == kInfBits ? 1 : 0;
        tau = __reduce_max_sync(FGC_FULL_MASK, lmax);
        return 1;
    }
};


// A step in which at least this many candidates pass the vote is merged into the sorted list as
// a whole (about 150 instructions whatever the count); fewer go in one by one (about 16 each).
// Measured on B200: 8 is best, 5 and 12 are 0.5 to 2 % slower.
constexpr int kBulkMin = 8;
// One stage of a bitonic network over the 32 lanes: partner lane ^ jj; the lane keeps the
// smaller key when want_min; equal keys keep their own entry.
__device__ __forceinline__ void cmpx(float &d, int &id, int jj, bool want_min)
{
    const float od = __shfl_xor_sync(FGC_FULL_MASK, d, jj);
    const int oi = __shfl_xor_sync(FGC_FULL_MASK, id, jj);
    const float nd = want_min ? fminf(d, od) : fmaxf(d, od);
    if (nd != d) id = oi;
    d = nd;
}

// ascending over the lanes
__device__ __forceinline__ void sort32(float &d, int &id, int lane)
{
#pragma unroll
    for (int k = 2; k <= 16; k <<= 1)
#pragma unroll
        for (int jj = k >> 1; jj > 0; jj >>= 1) cmpx(d, id, jj, ((lane & jj) != 0) == ((lane & k) != 0));
#pragma unroll
    for (int jj = 16; jj > 0; jj >>= 1) cmpx(d, id, jj, (lane & jj) == 0);
}

// a bitonic sequence over the lanes into ascending order
__device__ __forceinline__ void merge_bitonic32(float &d, int &id, int lane)
{
#pragma unroll
    for (int jj = 16; jj > 0; jj >>= 1) cmpx(d, id, jj, (lane & jj) == 0);
}

// The neighbour list kept in ascending order across the warp: position s = r*32 + lane holds the
// (s+1)-th smallest distance seen so far, +inf where there is none yet.  All 32R positions are
// kept; the list proper is the first kn of them, so tau is the entry at position kn-1.  A single
// candidate is inserted by a shift, a step with many passing candidates by sorting them and
// merging the sorted sequences.
template <int R>
struct SortedList {
    float d[R];
    int id[R];
    uint32_t tau;

    __device__ __forceinline__ void init(int lane, int kn)
    {
#pragma unroll
        for (int r = 0; r < R; r++) { d[r] = __uint_as_float(kInfBits); id[r] = -1; }
        tau = kn > 0 ? kInfBits : 0u;
    }

    __device__ __forceinline__ void set_tau(int kn)
    {
        const float src = (R == 2 && kn > 32) ? d[R - 1] : d[0];
        tau = __float_as_uint(__shfl_sync(FGC_FULL_MASK, src, (kn - 1) & 31));
    }

    // warp-uniform candidate with dc < tau
    __device__ __forceinline__ void insert(int lane, int kn, float dc, int jc)
    {
        const int p0 = __popc(__ballot_sync(FGC_FULL_MASK, d[0] <= dc));
        if (R == 1 || p0 < 32) {
            float c_d = 0.f; int c_i = 0;
            if (R == 2) {
                c_d = __shfl_sync(FGC_FULL_MASK, d[0], 31);
                c_i = __shfl_sync(FGC_FULL_MASK, id[0], 31);
            }
            const float du = __shfl_up_sync(FGC_FULL_MASK, d[0], 1);
            const int iu = __shfl_up_sync(FGC_FULL_MASK, id[0], 1);
            if (lane > p0) { d[0] = du; id[0] = iu; }
            else if (lane == p0) { d[0] = dc; id[0] = jc; }
            if (R == 2) {
                const float du1 = __shfl_up_sync(FGC_FULL_MASK, d[R - 1], 1);
                const int iu1 = __shfl_up_sync(FGC_FULL_MASK, id[R - 1], 1);
                d[R - 1] = lane == 0 ? c_d : du1;
                id[R - 1] = lane == 0 ? c_i : iu1;
            }
        } else {
            const int p = __popc(__ballot_sync(FGC_FULL_MASK, d[R - 1] <= dc));
            const float du = __shfl_up_sync(FGC_FULL_MASK, d[R - 1], 1);
            const int iu = __shfl_up_sync(FGC_FULL_MASK, id[R - 1], 1);
            if (lane > p) { d[R - 1] = du; id[R - 1] = iu; }
            else if (lane == p) { d[R - 1] = dc; id[R - 1] = jc; }
        }
        set_tau(kn);
    }

    // two ascending sequences of 32 (lo, hi) into one ascending sequence of 64
    __device__ __forceinline__ void merge_halves(int lane)
    {
        float cr = __shfl_sync(FGC_FULL_MASK, d[R - 1], 31 - lane);
        int ir = __shfl_sync(FGC_FULL_MASK, id[R - 1], 31 - lane);
        if (cr < d[0]) {
            const float td = d[0]; const int ti = id[0];
            d[0] = cr; id[0] = ir; cr = td; ir = ti;
        }
        d[R - 1] = cr; id[R - 1] = ir;
#pragma unroll
        for (int jj = 16; jj > 0; jj >>= 1) {
            cmpx(d[0], id[0], jj, (lane & jj) == 0);
            cmpx(d[R - 1], id[R - 1], jj, (lane & jj) == 0);
        }
    }

    // one candidate per lane (+inf where the lane has none): keep the 32R smallest of list and
    // candidates
    __device__ __forceinline__ void merge32(int lane, int kn, float dc, int jc)
    {
        sort32(dc, jc, lane);
        const unsigned lo_has = __ballot_sync(FGC_FULL_MASK, __float_as_uint(d[0]) < kInfBits);
        const unsigned hi_has = R == 2 ? __ballot_sync(FGC_FULL_MASK, __float_as_uint(d[R - 1]) < kInfBits) : 0u;
        if (lo_has == 0) {
            d[0] = dc; id[0] = jc;
        } else if (R == 2 && hi_has == 0) {
            // the upper half is empty: the candidates become the upper half
            d[R - 1] = dc; id[R - 1] = jc;
            merge_halves(lane);
        } else {
            // against the top 32 positions: the elementwise minimum with the reversed candidates is
            // a bitonic sequence of the 32 smallest of the two
            const float cr = __shfl_sync(FGC_FULL_MASK, dc, 31 - lane);
            const int ir = __shfl_sync(FGC_FULL_MASK, jc, 31 - lane);
            if (cr < d[R - 1]) { d[R - 1] = cr; id[R - 1] = ir; }
            merge_bitonic32(d[R - 1], id[R - 1], lane);
            if (R == 2) {
                const float lo_max = __shfl_sync(FGC_FULL_MASK, d[0], 31);
                const float hi_min = __shfl_sync(FGC_FULL_MASK, d[R - 1], 0);
                if (hi_min < lo_max) merge_halves(lane);
            }
        }
        set_tau(kn);
    }
};

// The search of one query by one warp.  G4: the grid spans four coordinates, else three.
template <int NV, int R, bool COUNT, bool G4>
__device__ __forceinline__ void knn_query(const KnnArgs &a)
{
    __shared__ int s_delta[kKnnWarps][32];
    __shared__ float s_bd[kKnnWarps][32];
    __shared__ int s_bj[kKnnWarps][32];
    const int lane = threadIdx.x & 31;
    const int wib = threadIdx.x >> 5;
    const int qi = blockIdx.x * kKnnWarps + wib;   // position in cell order
    KnnGrid *__restrict__ g = a.grid;
    if (qi >= a.n_vert) return;
    if (g->status != 0) {
        // Bad input (non-finite coordinate, malformed row splits): the grid was not built.  Every
        // row gets the defaults of a point without neighbours, so that a caller who does not look
        // at the status word never reads uninitialised indices.
        const int K = a.K;
        const int64_t pad = a.tf_compat ? (int64_t)qi : (int64_t)-1;
        for (int s = lane; s < K; s += 32) {
            a.out_idx[(size_t)qi * K + s] = s == 0 ? (int64_t)qi : pad;
            a.out_dist[(size_t)qi * K + s] = 0.f;
        }
        return;
    }
    if ((g->gdims == 4) != G4) {            // built in the other form: never walk it
        if (threadIdx.x == 0 && blockIdx.x == 0) atomicOr(&g->status, FGC_STATUS_INTERNAL);
        return;
    }

    const int K = a.K, kn = K - 1;
    const int nc = a.n_coords;
    const uint8_t *__restrict__ sflag = a.sflag;
    const int orig_q = __ldg(a.sorig + qi);
    if (!FGC_DBG_OK(orig_q >= 0 && orig_q < a.n_vert, &g->status)) return;
    int64_t *__restrict__ out_i = a.out_idx + (size_t)orig_q * K;
    float *__restrict__ out_d = a.out_dist + (size_t)orig_q * K;

    // queries that may not have neighbours keep the default row
    const bool q_inactive = sflag && (sflag[qi] == 0 || sflag[qi] == 2);

    float4 q[NV];
#pragma unroll
    for (int v = 0; v < NV; v++) q[v] = __ldg(a.scoords + (size_t)qi * NV + v);

    // Sorted list where it was measured faster than the unordered one (B200, uniform, normal and
    // clustered data in 3 to 8 dimensions, K = 8..64): one slot per lane (-2 to -20 %, except
    // uniform 3-D data at K = 32, +7 %: few insertions follow the first sort there), two slots
    // per lane (-10 to -23 % for K = 40, 48 and -1 to -15 % for K = 64 with one float4 per point;
    // -2 to -5 % with more than four coordinates, where it needs the registers of 6 instead of 7
    // resident CTAs).  Four and more slots per lane keep the unordered list.
    constexpr bool SORTED = R <= 2;
    typename std::conditional<SORTED, SortedList<R>, NeighbourList<R>>::type list;
    list.init(lane, kn);
    unsigned cnt_evals = 0, cnt_steps = 0, cnt_ins = 0, cnt_batches = 0, cnt_shells = 0, cnt_brute = 0;

    // one step: lane evaluates the candidate at sorted position j (if act)
    auto process = [&](int j, bool act) {
        float dc = __uint_as_float(kInfBits);
        if (act && FGC_DBG_OK(j >= 0 && j < a.n_vert, &g->status)) {
            float4 c[NV];
#pragma unroll
            for (int v = 0; v < NV; v++) c[v] = __ldg(a.scoords + (size_t)j * NV + v);
            bool ok = j != qi;
            if (sflag) { const uint8_t f = sflag[j]; ok = ok && f != 1 && f != 2; }
            if (ok) dc = dist_sq<NV>(q, c, nc);
        }
        if (COUNT) { cnt_evals += act ? 1 : 0; cnt_steps += 1; }
        unsigned m = __ballot_sync(FGC_FULL_MASK, __float_as_uint(dc) < list.tau);
        if (m == 0) return;
        const int npass = __popc(m);
        if constexpr (SORTED) {
            if (npass >= kBulkMin) {
                list.merge32(lane, kn, (m >> lane & 1) ? dc : __uint_as_float(kInfBits), j);
                if (COUNT) cnt_ins += npass;
                return;
            }
            while (m) {
                const int src = __ffs(m) - 1;
                m &= m - 1;
                const float dcs = __shfl_sync(FGC_FULL_MASK, dc, src);
                const int js = __shfl_sync(FGC_FULL_MASK, j, src);
                if (__float_as_uint(dcs) < list.tau) {
                    list.insert(lane, kn, dcs, js);
                    if (COUNT) cnt_ins += 1;
                }
            }
            return;
        } else {
            if (R >= 2 && list.filled + npass <= kn) {
                // all passing candidates fit into empty slots (tau is +inf here): place them in
                // one go through shared memory instead of one warp-wide insertion each (pays
                // off once a lane holds more than one slot)
                if (m >> lane & 1) {
                    const int rk = __popc(m & lanemask_lt());
                    s_bd[wib][rk] = dc;
                    s_bj[wib][rk] = j;
                }
                __syncwarp();
#pragma unroll
                for (int r = 0; r < R; r++) {
                    const int src = lane * R + r - list.filled;
                    if (src >= 0 && src < npass) { list.d[r] = s_bd[wib][src]; list.id[r] = s_bj[wib][src]; }
                }
                __syncwarp();
                list.filled += npass;
                list.refresh(lane);
                if (COUNT) cnt_ins += npass;
                return;
            }
            while (m) {
                const int src = __ffs(m) - 1;
                m &= m - 1;
                const float dcs = __shfl_sync(FGC_FULL_MASK, dc, src);
                const int js = __shfl_sync(FGC_FULL_MASK, j, src);
                const int ins = list.offer(lane, dcs, js);
                if (COUNT) cnt_ins += ins;
            }
        }
    };

    if (!q_inactive && kn > 0) {
        const int B = g->B, n0 = g->n[0], n1 = g->n[1], n2 = g->n[2], n3 = G4 ? g->n[3] : 1;
        const int flat = __ldg(a.sbin + qi);
        // (divisions by the grid's shape as multiply + shift: the divisors are set with the grid)
        const int e = fast_div(flat, g->div_m[0], g->div_s[0]);
        int rem = flat - e * B;
        const int b0 = fast_div(rem, g->div_m[1], g->div_s[1]);
        rem -= b0 * n1 * n2 * n3;
        const int b1 = fast_div(rem, g->div_m[2], g->div_s[2]);
        rem -= b1 * n2 * n3;
        const int b2 = G4 ? fast_div(rem, g->div_m[3], g->div_s[3]) : rem;
        const int b3 = G4 ? rem - b2 * n3 : 0;
        // the run of an item lies along the last grid dimension
        const int bl = G4 ? b3 : b2, nl = G4 ? n3 : n2;
        constexpr int GD = G4 ? 4 : 3;
        const int ev_begin = __ldg(a.bounds + e * B);
        const int ev_end = __ldg(a.bounds + (e + 1) * B);
        const int n_e = ev_end - ev_begin;

        bool brute = n_e <= 512 || n_e <= 8 * K;
        if (!brute) {
            const float w = g->w, slack = g->slack;
            const float w_lo = w * (1.0f - 1e-6f), w_hi = w * (1.0f + 1e-6f);
            // query position relative to the grid origin, per grid dimension
            float qr[GD];
            {
                const float qc[4] = {q[0].x, q[0].y, q[0].z, q[0].w};
#pragma unroll
                for (int gd = 0; gd < GD; gd++) {
                    const int c = g->cdim[gd];
                    const float x = c == 0 ? qc[0] : (c == 1 ? qc[1] : (c == 2 ? qc[2] : qc[3]));
                    qr[gd] = c < 0 ? 0.f : __fsub_rn(x, g->origin[gd]);
                }
            }
            // Points of cell b have a shifted coordinate >= b*w and < (b+1)*w up to fp32
            // rounding of the cell index computation; the bounds below widen the cell by a
            // relative 1e-6 and an absolute slack so that they hold for every such point.
            // gap_to: lower bound of |x - query| over the points of cells [lo, hi].
            auto gap_to = [&](int lo, int hi, int bq, float qrel) {
                float gp = 0.f;
                if (lo > bq) gp = (float)lo * w_lo - qrel - slack;
                else if (hi < bq) gp = qrel - (float)(hi + 1) * w_hi - slack;
                return fmaxf(gp, 0.f);
            };
            long long items_done = 0;
            // The walk normally starts with the centre cell and shell 1 as ONE batch of 11 items
            // (they are adjacent in the table, centre first): a sparsely filled centre cell never
            // ends a search, and a batch of its own would cost as much as the eleven together.
            // A centre cell that already holds 2K points gives a tight K-th distance that prunes
            // shell 1, so it is walked on its own then.
            const bool merged = __ldg(a.bounds + flat + 1) - __ldg(a.bounds + flat) < 2 * K;
            for (int d = merged ? 1 : 0;; ++d) {
                const bool first = merged && d == 1;
                const int n_items = G4 ? (first ? 1 + shell_items4(1) : shell_items4(d))
                                       : (first ? 1 + shell_items(1) : shell_items(d));
                const int32_t *tab =
                    G4 ? (first ? kShellTable4Data
                                : (d <= kShellTable4MaxD ? kShellTable4Data + shell_table4_offset(d) : nullptr))
                       : (first ? kShellTableData
                                : (d <= kShellTableMaxD ? kShellTableData + shell_table_offset(d) : nullptr));
                for (int base = 0; base < n_items; base += 32) {
                    const int u = base + lane;
                    bool valid = u < n_items;
                    int o0 = 0, o1 = 0, o2 = 0, zlo = 0, zhi = 0;
                    if (valid) {
                        if (tab) {
                            const int32_t t = __ldg(tab + u);
                            if (G4) {
                                o0 = (t & 0xf) - 8;
                                o1 = ((t >> 4) & 0xf) - 8;
                                o2 = ((t >> 8) & 0xf) - 8;
                                zlo = ((t >> 12) & 0xf) - 8;
                                zhi = ((t >> 16) & 0xf) - 8;
                            } else {
                                o0 = (int)(int8_t)(t & 0xff);
                                o1 = (int)(int8_t)((t >> 8) & 0xff);
                                zlo = (int)(int8_t)((t >> 16) & 0xff);
                                zhi = (int)(int8_t)((t >> 24) & 0xff);
                            }
                        } else if (G4) {
                            shell_item_decode4(d, u, o0, o1, o2, zlo, zhi);
                        } else {
                            shell_item_decode(d, u, o0, o1, zlo, zhi);
                        }
                    }
                    const int g0 = b0 + o0, g1 = b1 + o1, g2 = b2 + o2;
                    valid = valid && g0 >= 0 && g0 < n0 && g1 >= 0 && g1 < n1;
                    if (G4) valid = valid && g2 >= 0 && g2 < n2 && zlo <= zhi;
                    zlo = max(bl + zlo, 0);
                    zhi = min(bl + zhi, nl - 1);
                    valid = valid && zlo <= zhi;
                    if (valid && list.tau < kInfBits) {
                        const float ga = gap_to(g0, g0, b0, qr[0]);
                        const float gb = gap_to(g1, g1, b1, qr[1]);
                        const float gc = gap_to(zlo, zhi, bl, qr[GD - 1]);
                        float md = ga * ga + gb * gb + gc * gc;
                        if (G4) { const float gm = gap_to(g2, g2, b2, qr[2]); md += gm * gm; }
                        if (md > __uint_as_float(list.tau) * 1.00001f) valid = false;
                    }
                    int start = 0, len = 0;
                    if (valid) {
                        valid = FGC_DBG_OK(zlo >= 0 && zhi < nl && e >= 0 && e < g->n_events, &g->status);
                    }
                    if (valid) {
                        const int rowbase = G4 ? e * B + ((g0 * n1 + g1) * n2 + g2) * n3 : e * B + (g0 * n1 + g1) * n2;
                        start = __ldg(a.bounds + rowbase + zlo);
                        len = __ldg(a.bounds + rowbase + zhi + 1) - start;
                    }
                    const unsigned nzm = __ballot_sync(FGC_FULL_MASK, len > 0);
                    if (nzm == 0) continue;
                    if (COUNT) cnt_batches += 1;
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
                        // which range does flattened position t + lane belong to: mark the
                        // positions inside this step where a range starts
                        const int rel = pprev - t;
                        const unsigned contrib = (len > 0 && rel >= 0 && rel < 32) ? (1u << rel) : 0u;
                        const unsigned M = __reduce_or_sync(FGC_FULL_MASK, contrib);
                        const int r = rbase + __popc(M & lanemask_le()) - 1;
                        rbase += __popc(M);
                        const int c = t + lane;
                        const bool act = c < T;
                        const int j = act ? c + s_delta[wib][r] : -1;
                        process(j, act);
                    }
                    __syncwarp();
                }
                items_done += n_items;
                if (COUNT) cnt_shells += 1;
                // every point outside the cube of radius d is at least fd away
                float fd = __uint_as_float(kInfBits);
                bool any = false;
                {
                    const int bq[4] = {b0, b1, b2, b3};
                    const int nn[4] = {n0, n1, n2, n3};
#pragma unroll
                    for (int gd = 0; gd < GD; gd++) {
                        const int hi = bq[gd] + d + 1, lo = bq[gd] - d - 1;
                        if (hi <= nn[gd] - 1) { fd = fminf(fd, fmaxf((float)hi * w_lo - qr[gd] - slack, 0.f)); any = true; }
                        if (lo >= 0) { fd = fminf(fd, fmaxf(qr[gd] - (float)(lo + 1) * w_hi - slack, 0.f)); any = true; }
                    }
                }
                if (!any) break;
                if (list.tau < kInfBits && fd * fd > __uint_as_float(list.tau) * 1.00001f) break;
                // walking mostly empty cells: scanning the whole row split is cheaper
                // (giving up earlier costs more than it saves once row splits have millions of points)
                if (items_done * 8 > (long long)n_e) { brute = true; break; }
            }
            if (brute) {
                if (n_e > kHardMin) {
                    // (the list holds n_vert entries and every query appends at most once per
                    // search, so the bound below only guards against a stale counter)
                    int slot = 0;
                    if (lane == 0) {
                        slot = atomicAdd(&g->n_hard, 1);
                        if (slot < a.n_vert) a.hardlist[slot] = qi;
                        if (COUNT) atomicAdd(&g->counters[5], 1ull);
                    }
                    slot = __shfl_sync(FGC_FULL_MASK, slot, 0);
                    if (slot < a.n_vert) return;             // k_knn_hard writes this row
                }
                list.init(lane, kn);
            }
        }
        if (brute) {
            if (COUNT) cnt_brute = 1;
            for (int t = 0; t < n_e; t += 32) {
                const int c = t + lane;
                process(ev_begin + c, c < n_e);
            }
        }
    }

    // epilogue: original ids, original row position
    if (lane == 0) { out_i[0] = orig_q; out_d[0] = 0.f; }
    const int64_t pad = a.tf_compat ? (int64_t)orig_q : (int64_t)-1;
    if constexpr (SORTED) {
        // ascending distances; positions from kn on are not part of the list
#pragma unroll
        for (int r = 0; r < R; r++) {
            const int s = r * 32 + lane;
            if (s < kn) {
                const bool filled = list.d[r] < __uint_as_float(kInfBits) && list.id[r] >= 0;
                out_i[1 + s] = filled ? (int64_t)__ldg(a.sorig + list.id[r]) : pad;
                out_d[1 + s] = filled ? list.d[r] : 0.f;
            }
        }
    } else {
#pragma unroll
        for (int r = 0; r < R; r++) {
            const int s = lane * R + r;
            if (s < kn) {
                const bool filled = __float_as_uint(list.d[r]) < kInfBits && list.id[r] >= 0;
                out_i[1 + s] = filled ? (int64_t)__ldg(a.sorig + list.id[r]) : pad;
                out_d[1 + s] = filled ? list.d[r] : 0.f;
            }
        }
    }
    if (COUNT) {
        cnt_evals = __reduce_add_sync(FGC_FULL_MASK, cnt_evals);
        if (lane == 0) {
            atomicAdd(&g->counters[0], (unsigned long long)cnt_evals);
            atomicAdd(&g->counters[1], (unsigned long long)cnt_steps);
            atomicAdd(&g->counters[2], (unsigned long long)cnt_ins);
            atomicAdd(&g->counters[3], (unsigned long long)cnt_batches);
            atomicAdd(&g->counters[4], (unsigned long long)cnt_shells);
            atomicAdd(&g->counters[5], (unsigned long long)cnt_brute);
        }
    }
}

// The queries that gave up their walk in a large row split: a whole CTA per query, every warp
// scans an interleaved eighth of the candidates with a list of its own, warp 0 then offers the other
// warps' lists to its own.  There are usually a handful of such queries and each scans up to
// hundreds of thousands of points, so while the launch has more CTAs than queries a query is split
// over S CTAs (a contiguous S-th of the row split each): every CTA stores its merged list, the one
// that finishes last (ticket counter, no waiting) offers the S stored lists to a fresh list in part
// order and writes the row.  Same candidates, same strict "<" rule, fixed orders: the result does
// not depend on which CTA picks up what or finishes last.
constexpr int kHardMaxSplit = 32;

template <int NV, int R>
__global__ void __launch_bounds__(kKnnWarps * 32)
k_knn_hard(const KnnArgs a)
{
    chain_wait();
    chain_release();
    __shared__ float s_d[kKnnWarps][R * 32];
    __shared__ int s_i[kKnnWarps][R * 32];
    const int lane = threadIdx.x & 31;
    const int wib = threadIdx.x >> 5;
    KnnGrid *__restrict__ g = a.grid;
    if (g->status != 0) return;
    const int n_hard = min(g->n_hard, a.n_vert);
    if (n_hard == 0) return;
    const int K = a.K, kn = K - 1, nc = a.n_coords;
    const uint8_t *__restrict__ sflag = a.sflag;
    // CTAs per query: what the launch has to spare, what the scratch for the stored lists holds
    constexpr size_t kPartBytes = (size_t)R * 32 * 8;
    long long S = (long long)gridDim.x / n_hard;
    if (S > kHardMaxSplit) S = kHardMaxSplit;
    const long long cap = (long long)(a.hard_parts_bytes / kPartBytes) / n_hard;
    if (S > cap) S = cap;
    if (S < 1 || n_hard > kHardTickets || !a.hard_parts || !a.hard_tickets) S = 1;
    const int split = (int)S;
    const long long units = (long long)n_hard * split;
    float *__restrict__ part_d = a.hard_parts;
    int *__restrict__ part_i = (int *)(a.hard_parts + (size_t)units * R * 32);

    for (long long u = blockIdx.x; u < units; u += gridDim.x) {
        const int h = (int)(u / split), part = (int)(u - (long long)h * split);
        const int qi = a.hardlist[h];
        float4 q[NV];
#pragma unroll
        for (int v = 0; v < NV; v++) q[v] = __ldg(a.scoords + (size_t)qi * NV + v);
        const int B = g->B;
        const int e = __ldg(a.sbin + qi) / B;
        const int ev_begin = __ldg(a.bounds + e * B);
        const int n_e = __ldg(a.bounds + (e + 1) * B) - ev_begin;
        // this CTA's share of the row split
        const int chunk = (int)(((long long)n_e + split - 1) / split);
        const int t_lo = part * chunk, t_hi = min(n_e, t_lo + chunk);
        NeighbourList<R> list;
        list.init(lane, kn);
        auto offer_all = [&](float dc, int j) {
            unsigned m = __ballot_sync(FGC_FULL_MASK, __float_as_uint(dc) < list.tau);
            while (m) {
                const int src = __ffs(m) - 1;
                m &= m - 1;
                list.offer(lane, __shfl_sync(FGC_FULL_MASK, dc, src), __shfl_sync(FGC_FULL_MASK, j, src));
            }
        };
        for (int t = t_lo + wib * 32; t < t_hi; t += kKnnWarps * 32) {
            const int j = ev_begin + t + lane;
            float dc = __uint_as_float(kInfBits);
            if (t + lane < t_hi) {
                float4 c[NV];
#pragma unroll
                for (int v = 0; v < NV; v++) c[v] = __ldg(a.scoords + (size_t)j * NV + v);
                bool ok = j != qi;
                if (sflag) { const uint8_t f = sflag[j]; ok = ok && f != 1 && f != 2; }
                if (ok) dc = dist_sq<NV>(q, c, nc);
            }
            offer_all(dc, j);
        }
#pragma unroll
        for (int r = 0; r < R; r++) {
            s_d[wib][r * 32 + lane] = list.d[r];
            s_i[wib][r * 32 + lane] = list.id[r];
        }
        __syncthreads();
        bool write_row = false;
        if (wib == 0) {
            for (int w = 1; w < kKnnWarps; w++)
#pragma unroll
                for (int r = 0; r < R; r++) {
                    const int j = s_i[w][r * 32 + lane];
                    // slots that are empty or not part of the list carry id -1
                    const float dc = j >= 0 ? s_d[w][r * 32 + lane] : __uint_as_float(kInfBits);
                    offer_all(dc, j);
                }
            write_row = split == 1;
            if (split > 1) {
                // store this part's list, then see whether it was the last one
#pragma unroll
                for (int r = 0; r < R; r++) {
                    part_d[(size_t)u * R * 32 + r * 32 + lane] = list.d[r];
                    part_i[(size_t)u * R * 32 + r * 32 + lane] = list.id[r];
                }
                __threadfence();
                __syncwarp();
                int ticket = 0;
                if (lane == 0) ticket = atomicAdd(&a.hard_tickets[h], 1);
                ticket = __shfl_sync(FGC_FULL_MASK, ticket, 0);
                if (ticket == split - 1) {
                    __threadfence();
                    list.init(lane, kn);
                    for (int p = 0; p < split; p++)
#pragma unroll
                        for (int r = 0; r < R; r++) {
                            const size_t at = ((size_t)h * split + p) * R * 32 + r * 32 + lane;
                            const int j = __ldcg(part_i + at);
                            const float dc = j >= 0 ? __ldcg(part_d + at) : __uint_as_float(kInfBits);
                            offer_all(dc, j);
                        }
                    write_row = true;
                }
            }
            if (write_row) {
                const int orig_q = __ldg(a.sorig + qi);
                int64_t *__restrict__ out_i = a.out_idx + (size_t)orig_q * K;
                float *__restrict__ out_d = a.out_dist + (size_t)orig_q * K;
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
            }
        }
        __syncthreads();
    }
}

// MODE 0: grid over three coordinates (D <= 3); 1: over four (D >= 5); 2: D = 4, where the grid
// build decides on the device between the two -- one launch, one uniform branch (two launches
// of which one returns at once cost the same; out-of-line bodies were slower).
template <int NV, int R, bool COUNT, int MODE>
__global__ void __launch_bounds__(kKnnWarps * 32, (R == 1 ? 8 : (R == 2 ? (NV == 1 ? 7 : 6) : (R == 4 ? 6 : 4))))
k_knn(const KnnArgs a)
{
    chain_wait();
    chain_release();
    if (MODE == 0) knn_query<NV, R, COUNT, false>(a);
    else if (MODE == 1) knn_query<NV, R, COUNT, true>(a);
    else if (a.grid->gdims == 4) knn_query<NV, R, COUNT, true>(a);
    else knn_query<NV, R, COUNT, false>(a);
}

template <int NV, int G4>
static int launch_knn_nv(const KnnArgs &a, cudaStream_t s)
{
    const int kn = a.K - 1;
    const unsigned blocks = (unsigned)((a.n_vert + kKnnWarps - 1) / kKnnWarps);
    const int R = (kn + 31) / 32;
    const int T = kKnnWarps * 32;
    if (a.count_evals) {
        if (R <= 1) FGC_RETURN_IF_CUDA(launch_chained(k_knn<NV, 1, true, G4>, blocks, T, 0, s, a));
        else if (R <= 2) FGC_RETURN_IF_CUDA(launch_chained(k_knn<NV, 2, true, G4>, blocks, T, 0, s, a));
        else if (R <= 4) FGC_RETURN_IF_CUDA(launch_chained(k_knn<NV, 4, true, G4>, blocks, T, 0, s, a));
        else FGC_RETURN_IF_CUDA(launch_chained(k_knn<NV, 8, true, G4>, blocks, T, 0, s, a));
    } else {
        if (R <= 1) FGC_RETURN_IF_CUDA(launch_chained(k_knn<NV, 1, false, G4>, blocks, T, 0, s, a));
        else if (R <= 2) FGC_RETURN_IF_CUDA(launch_chained(k_knn<NV, 2, false, G4>, blocks, T, 0, s, a));
        else if (R <= 4) FGC_RETURN_IF_CUDA(launch_chained(k_knn<NV, 4, false, G4>, blocks, T, 0, s, a));
        else FGC_RETURN_IF_CUDA(launch_chained(k_knn<NV, 8, false, G4>, blocks, T, 0, s, a));
    }
    FGC_CHECK_LAUNCH();
    // the queries that gave up their walk (usually none: the CTAs return at once)
    const unsigned hard_blocks = fgc::sm_count() * 2;
    if (R <= 1) FGC_RETURN_IF_CUDA(launch_chained(k_knn_hard<NV, 1>, hard_blocks, T, 0, s, a));
    else if (R <= 2) FGC_RETURN_IF_CUDA(launch_chained(k_knn_hard<NV, 2>, hard_blocks, T, 0, s, a));
    else if (R <= 4) FGC_RETURN_IF_CUDA(launch_chained(k_knn_hard<NV, 4>, hard_blocks, T, 0, s, a));
    else FGC_RETURN_IF_CUDA(launch_chained(k_knn_hard<NV, 8>, hard_blocks, T, 0, s, a));
    return (int)cudaGetLastError();
}
}  // namespace fgc

extern "C" int fgc_knn_search(int64_t n_vert, int32_t n_coords, int64_t n_rs, int32_t K,
                              int32_t has_direction, int32_t tf_compat, int32_t flags,
                              int64_t *out_idx, float *out_distsq, void *workspace,
                              size_t workspace_bytes, fgc_stream_t stream)
{
    FGC_NVTX("fgc_knn_search");
    using namespace fgc;
    KnnWorkspace L;
    const int rc = check_knn_args(n_vert, n_coords, n_rs, K, workspace, workspace_bytes, &L);
    if (rc != FGC_OK) return rc;
    if (n_vert == 0) return FGC_OK;
    if (!out_idx || !out_distsq) return FGC_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    char *ws = (char *)workspace;
    const bool count = (flags & FGC_SEARCH_COUNT) != 0;
    KnnArgs a;
    a.scoords = (const float4 *)(ws + L.scoords);
    a.sorig = (const int *)(ws + L.sorig);
    a.sbin = (const int *)(ws + L.sbin);
    a.sflag = has_direction ? (const uint8_t *)(ws + L.sflag) : nullptr;
    a.bounds = (const int *)(ws + L.counts);
    a.hardlist = (int *)(ws + L.stmp);        // free since the grid build
    a.hard_parts = (float *)(ws + L.pbin);    // (so is pbin)
    a.hard_parts_bytes = sizeof(int32_t) * (size_t)n_vert;
    a.hard_tickets = (int *)(ws + L.tickets);
    a.grid = (KnnGrid *)(ws + L.header);
    a.out_idx = out_idx;
    a.out_dist = out_distsq;
    a.n_vert = (int)n_vert;
    a.K = K;
    a.n_coords = n_coords;
    a.tf_compat = tf_compat;
    a.count_evals = count;
    // Every search starts its own list of queries for k_knn_hard: a grid may be searched more
    // than once (the build/search split), and a count left by an earlier search would make
    // this one re-scan stale entries and append behind them.
    // The grid build leaves both cleared, so the first search of a grid (FGC_SEARCH_FRESH) needs
    // no clearing and stays in the launch chain of the build.
    if (!(flags & FGC_SEARCH_FRESH)) {
        FGC_RETURN_IF_CUDA(cudaMemsetAsync(&a.grid->n_hard, 0, sizeof(int32_t), s));
        FGC_RETURN_IF_CUDA(cudaMemsetAsync(a.hard_tickets, 0, kHardTicketBytes, s));
    }
    if (n_coords <= 3) return launch_knn_nv<1, 0>(a, s);
    if (L.nv == 1) {
        // D = 4: a caller that fixed the grid's form at build time says so here too and gets the
        // kernel with that one search only (it checks the grid record and refuses a mismatch)
        if (flags & FGC_SEARCH_GRID3) return launch_knn_nv<1, 0>(a, s);
        if (flags & FGC_SEARCH_GRID4) return launch_knn_nv<1, 1>(a, s);
        return launch_knn_nv<1, 2>(a, s);
    }
    if (L.nv == 2) return launch_knn_nv<2, 1>(a, s);
    if (L.nv == 3) return launch_knn_nv<3, 1>(a, s);
    return launch_knn_nv<4, 1>(a, s);
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
    return fgc_knn_search(n_vert, n_coords, n_rs, K, direction_or_null != nullptr, tf_compat, FGC_SEARCH_FRESH,
                          out_idx, out_distsq, workspace, workspace_bytes, stream);
}
