// Neighbour search, tile variant: one warp per 32 consecutive cell-sorted queries, one
// query per lane.
//
// Queries that are neighbours in cell order sit in the same few cells, so they need almost
// the same candidates.  A tile therefore walks ONE region of cells for all of its queries --
// the lines around the tile's own line, extended along the last grid dimension by the tile's
// own cell span -- and every candidate is loaded once per warp (a broadcast 16-byte load)
// and evaluated by all 32 lanes, each against its own query.  A lane keeps its K-1 best in a
// private max-heap in shared memory (layout [slot][lane] with a stride of 33 words, so the
// lanes' private accesses and the cooperative row read-out are both free of systematic bank
// conflicts).  Candidates that beat a lane's current K-th distance are first appended to a
// small per-lane buffer; the buffers are merged into the heaps warp-synchronously, which
// keeps the divergent heap code out of the evaluation loop.
//
// Compared with one warp per query this removes the warp-wide bookkeeping per query (votes,
// shuffles and reductions to maintain ONE list) at the price of evaluating a candidate region
// that is somewhat larger than any single query needs.  Per-lane pruning of whole items
// against the lane's K-th distance and a per-lane stopping test keep that overhead small.
//
// A tile is eligible when its queries share one grid line (same row split and same leading
// cell coordinates) and span at most kTileMaxSpan cells, or lie in a row split small enough
// to be scanned whole.  Queries of other tiles, and queries that are not finished after
// kTileMaxShell shells, are left to the warp-per-query kernel (k_knn), which skips every
// query whose `done` flag this kernel set.
#pragma once
#include "knn_grid.cuh"

namespace fgc {

constexpr int kTileWarps = 2;       // tiles per CTA
constexpr int kTileBuf = 16;        // pending candidates per lane (merged once a lane holds more than 12)
constexpr int kTileMaxShell = 3;    // shells a tile walks before handing leftovers over
constexpr int kTileMaxSpan = 15;    // largest cell span (last grid dimension) of an eligible tile
constexpr int kTileMaxNeighbours = 128;   // K-1 above this: warp-per-query kernel only
constexpr int kTileStride = 33;     // words between consecutive slots of the per-lane arrays

// shared-memory words per tile (warp)
__host__ __device__ inline int tile_smem_words(int kn)
{
    // staged candidates (2 float4 each) + their flags + item ranges + heaps (distance, id) +
    // pending buffers, rounded to 16 bytes so that every tile's staging area stays aligned
    const int words = 32 * 8 + 8 + 2 * 32 + 2 * kn * kTileStride + 2 * kTileBuf * kTileStride;
    return (words + 3) & ~3;
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

template <int NV>
__device__ __forceinline__ float tile_dist_sq(const float4 (&q)[NV], const float4 (&c)[NV], int n_coords)
{
    float d = __fsub_rn(q[0].x, c[0].x);
    float acc = __fmul_rn(d, d);
    d = __fsub_rn(q[0].y, c[0].y); acc = __fadd_rn(acc, __fmul_rn(d, d));
    if (2 < n_coords) { d = __fsub_rn(q[0].z, c[0].z); acc = __fadd_rn(acc, __fmul_rn(d, d)); }
    if (3 < n_coords) { d = __fsub_rn(q[0].w, c[0].w); acc = __fadd_rn(acc, __fmul_rn(d, d)); }
#pragma unroll
    for (int v = 1; v < NV; v++) {
        if (4 * v + 0 < n_coords) { d = __fsub_rn(q[v].x, c[v].x); acc = __fadd_rn(acc, __fmul_rn(d, d)); }
        if (4 * v + 1 < n_coords) { d = __fsub_rn(q[v].y, c[v].y); acc = __fadd_rn(acc, __fmul_rn(d, d)); }
        if (4 * v + 2 < n_coords) { d = __fsub_rn(q[v].z, c[v].z); acc = __fadd_rn(acc, __fmul_rn(d, d)); }
        if (4 * v + 3 < n_coords) { d = __fsub_rn(q[v].w, c[v].w); acc = __fadd_rn(acc, __fmul_rn(d, d)); }
    }
    return acc;
}

template <int NV, bool COUNT>
__global__ void __launch_bounds__(kTileWarps * 32)
k_knn_tile(const KnnTileArgs a)
{
    extern __shared__ __align__(16) float tile_smem[];
    const int lane = threadIdx.x & 31;
    const int wib = threadIdx.x >> 5;
    const int qi0 = (blockIdx.x * kTileWarps + wib) * 32;
    KnnGrid *__restrict__ g = a.grid;
    if (qi0 >= a.n_vert || g->status != 0) return;

    const int K = a.K, kn = K - 1, nc = a.n_coords;
    float *tile_base = tile_smem + (size_t)wib * tile_smem_words(kn);
    float4 *st_c = (float4 *)tile_base;                            // staged candidates [32][NV]
    uint8_t *st_f = (uint8_t *)(tile_base + 32 * 8);               // their direction flags
    int *s_start = (int *)(tile_base + 32 * 8 + 8);                // item ranges of a batch
    int *s_len = s_start + 32;
    float *hd = (float *)(s_len + 32);                             // heap distances [kn][33]
    int *hi = (int *)(hd + kn * kTileStride);                      // heap ids
    float *bd = (float *)(hi + kn * kTileStride);                  // pending distances [kTileBuf][33]
    int *bj = (int *)(bd + kTileBuf * kTileStride);                // pending ids

    const int qi = qi0 + lane;
    const bool valid = qi < a.n_vert;
    const int q_last = min(qi0 + 31, a.n_vert - 1);
    const int B = g->B, n0 = g->n[0], n1 = g->n[1], n2 = g->n[2];
    const int flat_a = __ldg(a.sbin + qi0), flat_b = __ldg(a.sbin + q_last);
    const int e = flat_a / B;
    const int row_a = flat_a / n2, row_b = flat_b / n2;    // global line ids (row split included)
    const int ev_begin = __ldg(a.bounds + e * B);
    const int n_e = __ldg(a.bounds + (e + 1) * B) - ev_begin;
    const bool small_event = (flat_b / B == e) && (n_e <= 512 || n_e <= 8 * K);
    const int za = flat_a - row_a * n2, zb = flat_b - row_b * n2;
    const bool eligible = small_event || (row_a == row_b && zb - za <= kTileMaxSpan);
    if (!eligible) {
        if (valid) a.done[qi] = 0;
        return;
    }
    int rem = row_a - e * (n0 * n1);
    const int b0 = rem / n1;
    const int b1 = rem - b0 * n1;

    const uint8_t *__restrict__ sflag = a.sflag;
    float4 q[NV];
#pragma unroll
    for (int v = 0; v < NV; v++) q[v] = __ldg(a.scoords + (size_t)(valid ? qi : qi0) * NV + v);
    const bool q_inactive = sflag && valid && (sflag[qi] == 0 || sflag[qi] == 2);
    const int b2 = valid ? __ldg(a.sbin + qi) - row_a * n2 : za;   // own cell along the line

    int cnt = 0, nbuf = 0;
    float tau = __uint_as_float(0x7f800000u);
    bool fin = !valid || q_inactive || kn == 0;   // nothing (more) to search for this lane
    unsigned c_evals = 0, c_ins = 0;

    auto heap_insert = [&](float d, int j) {
        if (cnt < kn) {
            int i = cnt;
            while (i > 0) {
                const int p = (i - 1) >> 1;
                const float dp = hd[p * kTileStride + lane];
                if (dp >= d) break;
                hd[i * kTileStride + lane] = dp;
                hi[i * kTileStride + lane] = hi[p * kTileStride + lane];
                i = p;
            }
            hd[i * kTileStride + lane] = d;
            hi[i * kTileStride + lane] = j;
            cnt++;
            if (cnt == kn) tau = hd[lane];
        } else if (d < tau) {
            int i = 0;
            for (;;) {
                const int l = 2 * i + 1;
                if (l >= kn) break;
                const int r = l + 1;
                float dl = hd[l * kTileStride + lane];
                int c = l;
                if (r < kn) {
                    const float dr = hd[r * kTileStride + lane];
                    if (dr > dl) { dl = dr; c = r; }
                }
                if (dl <= d) break;
                hd[i * kTileStride + lane] = dl;
                hi[i * kTileStride + lane] = hi[c * kTileStride + lane];
                i = c;
            }
            hd[i * kTileStride + lane] = d;
            hi[i * kTileStride + lane] = j;
            tau = hd[lane];
        }
    };
    // merge every lane's pending candidates into its heap (all lanes together)
    auto flush = [&]() {
        const int mx = __reduce_max_sync(FGC_FULL_MASK, nbuf);
        for (int b = 0; b < mx; b++)
            if (b < nbuf) {
                heap_insert(bd[b * kTileStride + lane], bj[b * kTileStride + lane]);
                if (COUNT) c_ins++;
            }
        nbuf = 0;
        __syncwarp();
    };
    // All lanes evaluate candidates [start, start+len); `act` lanes may take them.  32
    // candidates at a time are fetched with one coalesced 16-byte load per lane and staged in
    // shared memory; the next 32 are already in flight while the staged ones are read back
    // as broadcasts, four per step, so that four independent distance chains overlap.
    auto scan_range = [&](int start, int len, bool act) {
        const int end = start + len;
        float4 nxt[NV];
        uint8_t nxt_f = 0;
        if (start + lane < end) {
#pragma unroll
            for (int v = 0; v < NV; v++) nxt[v] = __ldg(a.scoords + (size_t)(start + lane) * NV + v);
            if (sflag) nxt_f = __ldg(sflag + start + lane);
        }
        for (int base = start; base < end; base += 32) {
            const int n = min(32, end - base);
            if (lane < n) {
#pragma unroll
                for (int v = 0; v < NV; v++) st_c[lane * NV + v] = nxt[v];
                st_f[lane] = nxt_f;
            }
            __syncwarp();
            if (base + 32 + lane < end) {
#pragma unroll
                for (int v = 0; v < NV; v++) nxt[v] = __ldg(a.scoords + (size_t)(base + 32 + lane) * NV + v);
                if (sflag) nxt_f = __ldg(sflag + base + 32 + lane);
            }
            for (int c0 = 0; c0 < n; c0 += 4) {
                float dd[4];
                bool ok[4];
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const int c = min(c0 + u, n - 1);
                    float4 cv[NV];
#pragma unroll
                    for (int v = 0; v < NV; v++) cv[v] = st_c[c * NV + v];
                    dd[u] = tile_dist_sq<NV>(q, cv, nc);
                    ok[u] = act && c0 + u < n && base + c != qi;
                    if (sflag) { const uint8_t f = st_f[c]; ok[u] = ok[u] && f != 1 && f != 2; }
                }
                if (COUNT) c_evals += act ? min(4, n - c0) : 0;
#pragma unroll
                for (int u = 0; u < 4; u++)
                    if (ok[u] && dd[u] < tau) {
                        bd[nbuf * kTileStride + lane] = dd[u];
                        bj[nbuf * kTileStride + lane] = base + c0 + u;
                        nbuf++;
                    }
                if (__any_sync(FGC_FULL_MASK, nbuf > kTileBuf - 4)) flush();
            }
            __syncwarp();
        }
    };

    if (!__all_sync(FGC_FULL_MASK, fin)) {
        if (small_event) {
            scan_range(ev_begin, n_e, !fin);
            flush();
            fin = true;
        } else {
            const float w = g->w, slack = g->slack;
            const float w_lo = w * (1.0f - 1e-6f), w_hi = w * (1.0f + 1e-6f);
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
            // lower bound of |x - query| over the points of cells [lo, hi] (see k_knn)
            auto gap_to = [&](int lo, int hi, int bq, float qrel) {
                float gp = 0.f;
                if (lo > bq) gp = (float)lo * w_lo - qrel - slack;
                else if (hi < bq) gp = qrel - (float)(hi + 1) * w_hi - slack;
                return fmaxf(gp, 0.f);
            };
            for (int d = 0; d <= kTileMaxShell; ++d) {
                const int n_items = shell_items(d);
                const int32_t *tab = kShellTableData + shell_table_offset(d);
                for (int base = 0; base < n_items; base += 32) {
                    // lane-parallel lookup of up to 32 item ranges
                    {
                        const int u = base + lane;
                        int start = 0, len = 0;
                        if (u < n_items) {
                            const int32_t t = __ldg(tab + u);
                            const int o0 = (int)(int8_t)(t & 0xff), o1 = (int)(int8_t)((t >> 8) & 0xff);
                            const int zo_lo = (int)(int8_t)((t >> 16) & 0xff), zo_hi = (int)(int8_t)((t >> 24) & 0xff);
                            const int g0 = b0 + o0, g1 = b1 + o1;
                            // rim lines take the tile's span widened by d, interior lines one end cell
                            int zlo = zo_lo == zo_hi && d > 0 ? (zo_lo < 0 ? za - d : zb + d) : za + zo_lo;
                            int zhi = zo_lo == zo_hi && d > 0 ? zlo : zb + zo_hi;
                            zlo = max(zlo, 0);
                            zhi = min(zhi, n2 - 1);
                            if (g0 >= 0 && g0 < n0 && g1 >= 0 && g1 < n1 && zlo <= zhi) {
                                const int rowbase = e * B + (g0 * n1 + g1) * n2;
                                start = __ldg(a.bounds + rowbase + zlo);
                                len = __ldg(a.bounds + rowbase + zhi + 1) - start;
                            }
                        }
                        s_start[lane] = start;
                        s_len[lane] = len;
                    }
                    __syncwarp();
                    const int n_here = min(32, n_items - base);
                    for (int it = 0; it < n_here; it++) {
                        const int len = s_len[it];
                        if (len == 0) continue;
                        // the item's box again (warp-uniform), for the per-lane pruning test
                        const int32_t t = __ldg(tab + base + it);
                        const int o0 = (int)(int8_t)(t & 0xff), o1 = (int)(int8_t)((t >> 8) & 0xff);
                        const int zo_lo = (int)(int8_t)((t >> 16) & 0xff), zo_hi = (int)(int8_t)((t >> 24) & 0xff);
                        int zlo = zo_lo == zo_hi && d > 0 ? (zo_lo < 0 ? za - d : zb + d) : za + zo_lo;
                        int zhi = zo_lo == zo_hi && d > 0 ? zlo : zb + zo_hi;
                        zlo = max(zlo, 0);
                        zhi = min(zhi, n2 - 1);
                        bool act = !fin;
                        if (act && cnt == kn) {
                            const float ga = gap_to(b0 + o0, b0 + o0, b0, qr[0]);
                            const float gb = gap_to(b1 + o1, b1 + o1, b1, qr[1]);
                            const float gc = gap_to(zlo, zhi, b2, qr[2]);
                            if (ga * ga + gb * gb + gc * gc > tau * 1.00001f) act = false;
                        }
                        if (!__any_sync(FGC_FULL_MASK, act)) continue;
                        scan_range(s_start[it], len, act);
                    }
                    __syncwarp();
                }
                flush();
                // per-lane stopping test: everything outside the covered block of cells
                // (lines b0+-d, b1+-d, cells za-d .. zb+d) is at least fd away
                if (!fin) {
                    float fd = __uint_as_float(0x7f800000u);
                    bool any = false;
                    if (b0 + d + 1 <= n0 - 1) { fd = fminf(fd, fmaxf((float)(b0 + d + 1) * w_lo - qr[0] - slack, 0.f)); any = true; }
                    if (b0 - d - 1 >= 0) { fd = fminf(fd, fmaxf(qr[0] - (float)(b0 - d) * w_hi - slack, 0.f)); any = true; }
                    if (b1 + d + 1 <= n1 - 1) { fd = fminf(fd, fmaxf((float)(b1 + d + 1) * w_lo - qr[1] - slack, 0.f)); any = true; }
                    if (b1 - d - 1 >= 0) { fd = fminf(fd, fmaxf(qr[1] - (float)(b1 - d) * w_hi - slack, 0.f)); any = true; }
                    if (zb + d + 1 <= n2 - 1) { fd = fminf(fd, fmaxf((float)(zb + d + 1) * w_lo - qr[2] - slack, 0.f)); any = true; }
                    if (za - d - 1 >= 0) { fd = fminf(fd, fmaxf(qr[2] - (float)(za - d) * w_hi - slack, 0.f)); any = true; }
                    if (!any) fin = true;
                    else if (cnt == kn && fd * fd > tau * 1.00001f) fin = true;
                }
                if (__all_sync(FGC_FULL_MASK, fin)) break;
            }
        }
    }

    // rows of finished queries: written cooperatively, one query after the other
    const unsigned fin_mask = __ballot_sync(FGC_FULL_MASK, fin && valid);
    if (valid) a.done[qi] = fin ? 1 : 0;
    const int orig_l = valid ? __ldg(a.sorig + qi) : 0;
    __syncwarp();
    for (int t = 0; t < 32; t++) {
        if (!(fin_mask >> t & 1)) continue;
        const int orig_q = __shfl_sync(FGC_FULL_MASK, orig_l, t);
        const int cnt_t = __shfl_sync(FGC_FULL_MASK, cnt, t);
        int64_t *__restrict__ out_i = a.out_idx + (size_t)orig_q * K;
        float *__restrict__ out_d = a.out_dist + (size_t)orig_q * K;
        if (lane == 0) { out_i[0] = orig_q; out_d[0] = 0.f; }
        const int64_t pad = a.tf_compat ? (int64_t)orig_q : (int64_t)-1;
        for (int s = lane; s < kn; s += 32) {
            const bool filled = s < cnt_t;
            out_i[1 + s] = filled ? (int64_t)__ldg(a.sorig + hi[s * kTileStride + t]) : pad;
            out_d[1 + s] = filled ? hd[s * kTileStride + t] : 0.f;
        }
    }
    if (COUNT) {
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

}  // namespace fgc
