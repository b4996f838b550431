// Neighbour search, tile kernel: one warp per 32 consecutive cell-sorted queries, one query
// per lane.
//
// Queries that are neighbours in cell order sit in the same few cells of one line of the grid
// and need almost the same candidates.  A tile therefore walks ONE region of cells for all of
// its queries -- the lines around the tile's own line, extended along the last grid dimension
// by the tile's own cell span -- and every candidate is loaded once per warp and evaluated by
// all 32 lanes, each against its own query: a 16-byte broadcast read from shared memory and the
// distance arithmetic per candidate, where the warp-per-query kernel (k_knn) spends a warp's
// worth of votes, shuffles and reductions to keep ONE query's list.
//
// The walk is k_knn's: shells of "items" (runs of cells along the last grid dimension, from the
// same tables), 32 items looked up at once (one per lane), the non-empty ranges of a batch
// flattened into one candidate stream.  The stream is consumed 32 candidates at a time: every
// lane fetches one candidate (coalesced 16-byte loads) into shared memory, then all lanes read
// the staged candidates back as broadcasts, four per step, so that four independent distance
// chains are in flight.
//
// A lane keeps its K-1 best in a private max-heap in shared memory (layout [slot][lane]: a
// lane only ever touches its own bank, so the lanes' accesses never conflict whatever slots
// they are at).  The heap starts full of +inf entries, which makes "insert" the one operation
// replace-the-root-and-sift-down from the first candidate on.  Candidates that beat a lane's
// current K-th distance are first appended to a small per-lane buffer; the buffers are merged
// into the heaps by all lanes together, which keeps the divergent heap code out of the
// evaluation loop.
//
// A tile is eligible when its queries share one grid line (same row split, same leading cell
// coordinates) and span at most kTileMaxSpan cells, or lie in a row split small enough to be
// scanned whole.  Queries of other tiles, and queries that are not finished after
// kTileMaxShell shells, are left to k_knn, which skips every query whose `done` flag this
// kernel set.  Same candidates, same strict "<" rule as k_knn: which of several equidistant
// points is kept may differ, nothing else.
#pragma once
#include "knn_grid.cuh"
#include "shell_table.cuh"

namespace fgc {

constexpr int kTileWarps = 4;        // tiles per CTA
constexpr int kTileBuf = 8;          // pending candidates per lane
constexpr int kTileMaxShell = 3;     // shells a tile walks before handing leftovers over
constexpr int kTileMaxSpan = 12;     // largest cell span (last grid dimension) of an eligible tile
constexpr int kTileMaxNeighbours = 64;   // K-1 above this: warp-per-query kernel only

// shared-memory bytes per tile (warp): staged candidates (float4 + id), item offsets, heap
// (distance, id), pending buffers
__host__ __device__ inline size_t tile_smem_bytes(int kn)
{
    return 32 * 16 + 32 * 4 + 32 * 4 + (size_t)kn * 32 * 8 + (size_t)kTileBuf * 32 * 8;
}

struct KnnTileArgs {
    const float4 *scoords;
    const int *sorig;
    const int *sbin;
    const uint8_t *sflag;
    const int *bounds;
    KnnGrid *grid;
    int64_t *out_idx;
    float *out_dist;
    uint8_t *done;          // [n_vert] 1 = row written by this kernel
    int n_vert;
    int K;
    int n_coords;
    int tf_compat;
};

// NC: number of coordinates (2, 3 or 4: one float4 per point).  G4: grid over four coordinates.
template <int NC, bool COUNT, bool G4>
__device__ __forceinline__ void knn_tile(const KnnTileArgs &a, char *tile_base)
{
    constexpr uint32_t kInf = 0x7f800000u;
    constexpr int GD = G4 ? 4 : 3;
    const int lane = threadIdx.x & 31;
    const int qi0 = (blockIdx.x * kTileWarps + (threadIdx.x >> 5)) * 32;
    KnnGrid *__restrict__ g = a.grid;
    if (qi0 >= a.n_vert || g->status != 0) return;
    if ((g->gdims == 4) != G4) return;        // the other form's kernel (or k_knn) takes it

    const int K = a.K, kn = K - 1;
    float4 *st_c = (float4 *)tile_base;                       // staged candidates [32]
    int *st_j = (int *)(tile_base + 32 * 16);                 // their cell-order positions
    int *s_delta = st_j + 32;                                 // item offsets of a batch
    float *hd = (float *)(s_delta + 32);                      // heap distances [kn][32]
    int *hi = (int *)(hd + kn * 32);                          // heap ids
    float *bd = (float *)(hi + kn * 32);                      // pending distances [kTileBuf][32]
    int *bj = (int *)(bd + kTileBuf * 32);                    // pending ids

    const int qi = qi0 + lane;
    const bool valid = qi < a.n_vert;
    const int q_last = min(qi0 + 31, a.n_vert - 1);
    const int B = g->B, n0 = g->n[0], n1 = g->n[1], n2 = g->n[2], n3 = G4 ? g->n[3] : 1;
    const int nl = G4 ? n3 : n2;                              // cells per line
    const int flat_a = __ldg(a.sbin + qi0), flat_b = __ldg(a.sbin + q_last);
    const int e = flat_a / B;
    const int line_a = flat_a / nl, line_b = flat_b / nl;     // global line ids (row split included)
    const int ev_begin = __ldg(a.bounds + e * B);
    const int n_e = __ldg(a.bounds + (e + 1) * B) - ev_begin;
    const bool small_event = (flat_b / B == e) && (n_e <= 512 || n_e <= 8 * K);
    const int za = flat_a - line_a * nl, zb = flat_b - line_b * nl;
    const bool eligible = small_event || (line_a == line_b && zb - za <= kTileMaxSpan);
    if (!eligible) {
        if (valid) a.done[qi] = 0;
        return;
    }
    int rem = line_a - e * (n0 * n1 * (G4 ? n2 : 1));
    const int b0 = rem / (n1 * (G4 ? n2 : 1));
    rem -= b0 * n1 * (G4 ? n2 : 1);
    const int b1 = G4 ? rem / n2 : rem;
    const int b2 = G4 ? rem - b1 * n2 : 0;                    // third leading coordinate (G4 only)

    const uint8_t *__restrict__ sflag = a.sflag;
    const float4 q = __ldg(a.scoords + (valid ? qi : qi0));
    const bool q_inactive = sflag && valid && (sflag[qi] == 0 || sflag[qi] == 2);
    const int bl = valid ? __ldg(a.sbin + qi) - line_a * nl : za;   // own cell along the line

    // the heap starts full of +inf: inserting is always "replace the root, sift down"
    for (int s = 0; s < kn; s++) { hd[s * 32 + lane] = __uint_as_float(kInf); hi[s * 32 + lane] = -1; }
    int nbuf = 0;
    float tau = __uint_as_float(kInf);
    bool fin = !valid || q_inactive || kn == 0;   // nothing (more) to search for this lane
    unsigned c_evals = 0, c_ins = 0;
    __syncwarp();

    auto heap_insert = [&](float d, int j) {
        if (!(d < tau)) return;
        int i = 0;
        for (;;) {
            const int l = 2 * i + 1;
            if (l >= kn) break;
            float dl = hd[l * 32 + lane];
            int c = l;
            if (l + 1 < kn) {
                const float dr = hd[(l + 1) * 32 + lane];
                if (dr > dl) { dl = dr; c = l + 1; }
            }
            if (!(dl > d)) break;
            hd[i * 32 + lane] = dl;
            hi[i * 32 + lane] = hi[c * 32 + lane];
            i = c;
        }
        hd[i * 32 + lane] = d;
        hi[i * 32 + lane] = j;
        tau = hd[lane];
    };
    // merge every lane's pending candidates into its heap (all lanes together)
    auto flush = [&]() {
        const int mx = __reduce_max_sync(FGC_FULL_MASK, nbuf);
        for (int b = 0; b < mx; b++)
            if (b < nbuf) {
                heap_insert(bd[b * 32 + lane], bj[b * 32 + lane]);
                if (COUNT) c_ins++;
            }
        nbuf = 0;
    };
    // All lanes evaluate the n staged candidates; lanes that are finished take none.
    auto eval_staged = [&](int n) {
        const float my_tau_gate = fin ? 0.f : 1.f;    // finished lanes: nothing passes (d >= 0 is never < 0)
        for (int c0 = 0; c0 < n; c0 += 4) {
            if (__any_sync(FGC_FULL_MASK, nbuf > kTileBuf - 4)) flush();
            float dd[4];
            int jj[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int c = min(c0 + u, n - 1);
                const float4 cv = st_c[c];
                jj[u] = st_j[c];
                float d = __fsub_rn(q.x, cv.x);
                float acc = __fmul_rn(d, d);
                d = __fsub_rn(q.y, cv.y); acc = __fadd_rn(acc, __fmul_rn(d, d));
                if (NC > 2) { d = __fsub_rn(q.z, cv.z); acc = __fadd_rn(acc, __fmul_rn(d, d)); }
                if (NC > 3) { d = __fsub_rn(q.w, cv.w); acc = __fadd_rn(acc, __fmul_rn(d, d)); }
                dd[u] = acc;
            }
            if (COUNT) c_evals += fin ? 0 : min(4, n - c0);
            const float gate = fin ? 0.f : tau;
            (void)my_tau_gate;
#pragma unroll
            for (int u = 0; u < 4; u++)
                if (dd[u] < gate && c0 + u < n && jj[u] != qi) {
                    bd[nbuf * 32 + lane] = dd[u];
                    bj[nbuf * 32 + lane] = jj[u];
                    nbuf++;
                }
        }
    };
    // stage the candidate at cell-order position j (act lanes) and evaluate the block
    auto stage_and_eval = [&](int j, bool act, int n) {
        __syncwarp();
        if (act && FGC_DBG_OK(j >= 0 && j < a.n_vert, &g->status)) {
            float4 cv = __ldg(a.scoords + j);
            if (sflag) { const uint8_t f = __ldg(sflag + j); if (f == 1 || f == 2) cv.x = __uint_as_float(kInf); }
            st_c[lane] = cv;
            st_j[lane] = j;
        }
        __syncwarp();
        eval_staged(n);
    };

    if (!__all_sync(FGC_FULL_MASK, fin)) {
        if (small_event) {
            for (int t = 0; t < n_e; t += 32) stage_and_eval(ev_begin + t + lane, t + lane < n_e, min(32, n_e - t));
            flush();
            fin = true;
        } else {
            const float w = g->w, slack = g->slack;
            const float w_lo = w * (1.0f - 1e-6f), w_hi = w * (1.0f + 1e-6f);
            float qr[GD];
            {
                const float qc[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                for (int gd = 0; gd < GD; gd++) {
                    const int c = g->cdim[gd];
                    const float x = c == 0 ? qc[0] : (c == 1 ? qc[1] : (c == 2 ? qc[2] : qc[3]));
                    qr[gd] = c < 0 ? 0.f : __fsub_rn(x, g->origin[gd]);
                }
            }
            // the tile's own box in shifted coordinates (over its valid lanes), for the
            // item-level pruning test: an item is walked when its cells could hold a point within
            // the largest K-th distance any unfinished lane still has
            float box_lo[GD], box_hi[GD];
#pragma unroll
            for (int gd = 0; gd < GD; gd++) {
                float lo = valid ? qr[gd] : __uint_as_float(kInf), hi = valid ? qr[gd] : -__uint_as_float(kInf);
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    lo = fminf(lo, __shfl_xor_sync(FGC_FULL_MASK, lo, o));
                    hi = fmaxf(hi, __shfl_xor_sync(FGC_FULL_MASK, hi, o));
                }
                box_lo[gd] = lo; box_hi[gd] = hi;
            }
            // lower bound of the distance between the tile's box and the cells [lo, hi] of a dimension
            auto gap_box = [&](int lo, int hi, float blo, float bhi) {
                const float c_lo = (float)lo * w_lo - slack, c_hi = (float)(hi + 1) * w_hi + slack;
                float gp = 0.f;
                if (c_lo > bhi) gp = c_lo - bhi;
                else if (c_hi < blo) gp = blo - c_hi;
                return gp;
            };
            const bool merged = __ldg(a.bounds + line_a * nl + zb + 1) - __ldg(a.bounds + line_a * nl + za) < 2 * K;
            for (int d = merged ? 1 : 0; d <= kTileMaxShell; ++d) {
                const bool first_batch = merged && d == 1;
                const int n_items = G4 ? (first_batch ? 1 + shell_items4(1) : shell_items4(d))
                                       : (first_batch ? 1 + shell_items(1) : shell_items(d));
                const int32_t *tab =
                    G4 ? (first_batch ? kShellTable4Data
                                      : (d <= kShellTable4MaxD ? kShellTable4Data + shell_table4_offset(d) : nullptr))
                       : (first_batch ? kShellTableData
                                      : (d <= kShellTableMaxD ? kShellTableData + shell_table_offset(d) : nullptr));
                // the largest K-th distance among the lanes still searching
                const uint32_t tau_max = __reduce_max_sync(FGC_FULL_MASK, fin ? 0u : __float_as_uint(tau));
                for (int base = 0; base < n_items; base += 32) {
                    const int it = base + lane;
                    bool ok = it < n_items;
                    int o0 = 0, o1 = 0, o2 = 0, zlo = 0, zhi = 0;
                    if (ok) {
                        if (tab) {
                            const int32_t t = __ldg(tab + it);
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
                            shell_item_decode4(d, it, o0, o1, o2, zlo, zhi);
                        } else {
                            shell_item_decode(d, it, o0, o1, zlo, zhi);
                        }
                    }
                    const int g0 = b0 + o0, g1 = b1 + o1, g2 = b2 + o2;
                    ok = ok && g0 >= 0 && g0 < n0 && g1 >= 0 && g1 < n1 && zlo <= zhi;
                    if (G4) ok = ok && g2 >= 0 && g2 < n2;
                    // the item's run for the whole tile: offsets below the centre count from the
                    // tile's first cell, offsets above it from its last
                    zlo = max((zlo > 0 ? zb : za) + zlo, 0);
                    zhi = min((zhi < 0 ? za : zb) + zhi, nl - 1);
                    ok = ok && zlo <= zhi;
                    if (ok && tau_max < kInf) {
                        float md = 0.f, gp;
                        gp = gap_box(g0, g0, box_lo[0], box_hi[0]); md += gp * gp;
                        gp = gap_box(g1, g1, box_lo[1], box_hi[1]); md += gp * gp;
                        if (G4) { gp = gap_box(g2, g2, box_lo[2], box_hi[2]); md += gp * gp; }
                        gp = gap_box(zlo, zhi, box_lo[GD - 1], box_hi[GD - 1]); md += gp * gp;
                        if (md > __uint_as_float(tau_max) * 1.00001f) ok = false;
                    }
                    int start = 0, len = 0;
                    if (ok) {
                        const int rowbase = G4 ? e * B + ((g0 * n1 + g1) * n2 + g2) * n3 : e * B + (g0 * n1 + g1) * n2;
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
                    __syncwarp();
                    if (len > 0) s_delta[__popc(nzm & lanemask_lt())] = start - pprev;
                    __syncwarp();
                    int rbase = 0;
                    for (int t = 0; t < T; t += 32) {
                        const int rel = pprev - t;
                        const unsigned contrib = (len > 0 && rel >= 0 && rel < 32) ? (1u << rel) : 0u;
                        const unsigned M = __reduce_or_sync(FGC_FULL_MASK, contrib);
                        const int r = rbase + __popc(M & lanemask_le()) - 1;
                        rbase += __popc(M);
                        const int c = t + lane;
                        const bool act = c < T;
                        const int j = act ? c + s_delta[r] : -1;
                        stage_and_eval(j, act, min(32, T - t));
                    }
                }
                flush();
                // per-lane stopping test: everything outside the covered block of cells (leading
                // coordinates within d of the tile's line, cells za-d .. zb+d along it) is at
                // least fd away
                if (!fin) {
                    float fd = __uint_as_float(kInf);
                    bool any = false;
                    const int lead[3] = {b0, b1, b2};
                    const int nlead[3] = {n0, n1, n2};
#pragma unroll
                    for (int gd = 0; gd < GD - 1; gd++) {
                        if (lead[gd] + d + 1 <= nlead[gd] - 1) { fd = fminf(fd, fmaxf((float)(lead[gd] + d + 1) * w_lo - qr[gd] - slack, 0.f)); any = true; }
                        if (lead[gd] - d - 1 >= 0) { fd = fminf(fd, fmaxf(qr[gd] - (float)(lead[gd] - d) * w_hi - slack, 0.f)); any = true; }
                    }
                    if (zb + d + 1 <= nl - 1) { fd = fminf(fd, fmaxf((float)(zb + d + 1) * w_lo - qr[GD - 1] - slack, 0.f)); any = true; }
                    if (za - d - 1 >= 0) { fd = fminf(fd, fmaxf(qr[GD - 1] - (float)(za - d) * w_hi - slack, 0.f)); any = true; }
                    if (!any) fin = true;
                    else if (__float_as_uint(tau) < kInf && fd * fd > tau * 1.00001f) fin = true;
                }
                if (__all_sync(FGC_FULL_MASK, fin)) break;
            }
        }
    }
    (void)bl;

    // rows of finished queries: every lane writes its own row
    if (valid) a.done[qi] = fin ? 1 : 0;
    if (valid && fin) {
        const int orig_q = __ldg(a.sorig + qi);
        int64_t *__restrict__ out_i = a.out_idx + (size_t)orig_q * K;
        float *__restrict__ out_d = a.out_dist + (size_t)orig_q * K;
        out_i[0] = orig_q;
        out_d[0] = 0.f;
        const int64_t pad = a.tf_compat ? (int64_t)orig_q : (int64_t)-1;
        int w_pos = 1;
        for (int s = 0; s < kn; s++) {
            const int j = hi[s * 32 + lane];
            if (j >= 0) {
                out_i[w_pos] = (int64_t)__ldg(a.sorig + j);
                out_d[w_pos] = hd[s * 32 + lane];
                w_pos++;
            }
        }
        for (; w_pos < K; w_pos++) { out_i[w_pos] = pad; out_d[w_pos] = 0.f; }
    }
    if (COUNT) {
        const unsigned fin_mask = __ballot_sync(FGC_FULL_MASK, fin && valid);
        c_evals = __reduce_add_sync(FGC_FULL_MASK, c_evals);
        c_ins = __reduce_add_sync(FGC_FULL_MASK, c_ins);
        if (lane == 0) {
            atomicAdd(&g->counters[0], (unsigned long long)c_evals);
            atomicAdd(&g->counters[2], (unsigned long long)c_ins);
            atomicAdd(&g->counters[6], (unsigned long long)__popc(fin_mask));
            atomicAdd(&g->counters[7], 1ull);
        }
    }
}

// MODE 0: grid over three coordinates; 1: over four; 2: D = 4, either (decided on the device)
template <int NC, bool COUNT, int MODE>
__global__ void __launch_bounds__(kTileWarps * 32)
k_knn_tile(const KnnTileArgs a)
{
    extern __shared__ __align__(16) char tile_smem[];
    char *base = tile_smem + (size_t)(threadIdx.x >> 5) * tile_smem_bytes(a.K - 1);
    if (MODE == 0) knn_tile<NC, COUNT, false>(a, base);
    else if (MODE == 1) knn_tile<NC, COUNT, true>(a, base);
    else if (a.grid->gdims == 4) knn_tile<NC, COUNT, true>(a, base);
    else knn_tile<NC, COUNT, false>(a, base);
}

}  // namespace fgc
