// Object-condensation index matrices and the gather-with-default that consumes them (sm_100a).
//
//   M[k, :]     ids of the points of object k (points of one row split that share a
//               non-negative truth index), ascending, padded with -1
//   M_not[k, :] ids of all other points of the same row split, ascending, padded with -1
//   objects_per_split[e]
// as extensions/oc_helper.py:128-230 with extensions/oc_helper_cpu.cpp:14-83 and
// extensions/oc_helper_helper.cpp:31-93 of the reference.  The reference finds the objects
// with torch.unique on the host side of its wrapper and then lets every object scan its
// whole row split twice; here one radix sort of (truth index, point id) puts the members of
// every object next to each other, M is a copy of those runs, and M_not is computed
// element-wise: the j-th non-member of an object is  row start + j + t,  t = number of
// members m_0 < m_1 < ... with  m_i - row start - i <= j  (a binary search over the
// object's sorted members), so the big matrix is written once, coalesced, with no scan of
// the row split per object.
//
// The order of the objects (rows of M) is not defined by the reference ("not guaranteed to
// give the identical output in terms of index ordering", oc_helper.py:91-92); here it is
// ascending in (truth index, row split).
#include <cstring>

#include <cub/device/device_radix_sort.cuh>

#include "fgc_common.cuh"
#include "scan.cuh"

namespace fgc {

struct OcHeader {
    int32_t status;     // FGC_STATUS_* bits (first word of the workspace)
    int32_t n_unique;   // number of objects
    int32_t n_maxuq;    // largest object
    int32_t n_maxrs;    // largest row split
    int32_t n_valid;    // points with a non-negative truth index
};

constexpr size_t kOcHeaderBytes = 256;
constexpr uint64_t kOcNoObject = ~0ull;

struct OcWorkspace {
    size_t header, keys_a, keys_b, vals_a, vals_b, flags, blocksums, obj_start, obj_split, cub_temp, total;
    size_t cub_temp_bytes;
};

inline OcWorkspace oc_workspace_layout(int64_t n_vert)
{
    OcWorkspace w;
    const size_t n = (size_t)n_vert;
    size_t off = 0;
    w.header = off; off += kOcHeaderBytes;
    w.keys_a = off; off = align_up(off + 8 * n, 256);
    w.keys_b = off; off = align_up(off + 8 * n, 256);
    w.vals_a = off; off = align_up(off + 4 * n, 256);
    w.vals_b = off; off = align_up(off + 4 * n, 256);
    w.flags = off; off = align_up(off + 4 * (n + 1), 256);
    w.blocksums = off; off = align_up(off + 4 * ((n + 1) / kScanTile + 2), 256);
    w.obj_start = off; off = align_up(off + 4 * (n + 1), 256);
    w.obj_split = off; off = align_up(off + 4 * (n + 1), 256);
    w.cub_temp_bytes = n + ((size_t)1 << 20);   // the sort's own scratch (histograms, tile states)
    w.cub_temp = off; off = align_up(off + w.cub_temp_bytes, 256);
    w.total = off;
    return w;
}

__global__ void k_oc_check(const int64_t *__restrict__ rs, int n_rs, int n_vert, OcHeader *h)
{
    // one warp: row_splits must start at 0, end at n_vert and never decrease
    const int lane = threadIdx.x;
    int bad = 0, longest = 0;
    for (int i = 1 + lane; i < n_rs; i += 32) {
        const int64_t len = rs[i] - rs[i - 1];
        if (len < 0) bad = 1;
        else if (len > longest) longest = (int)(len > 0x7fffffff ? 0x7fffffff : len);
    }
    bad = __any_sync(FGC_FULL_MASK, bad);
    longest = __reduce_max_sync(FGC_FULL_MASK, longest);
    if (lane == 0) {
        if (bad || rs[0] != 0 || rs[n_rs - 1] != (int64_t)n_vert) h->status |= FGC_STATUS_BAD_ROW_SPLITS;
        h->n_maxrs = longest;
    }
}

__global__ void __launch_bounds__(256)
k_oc_keys(const int64_t *__restrict__ asso, int n_vert, uint64_t *__restrict__ keys, int *__restrict__ vals)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_vert) return;
    const int64_t a = asso[i];
    keys[i] = a < 0 ? kOcNoObject : (uint64_t)a;   // points without an object sort to the end
    vals[i] = i;
}

// Position p of the sorted list starts an object when its (truth index, row split) differs
// from its predecessor's.
__device__ __forceinline__ bool oc_is_head(const uint64_t *__restrict__ keys, const int *__restrict__ vals,
                                           const int64_t *__restrict__ rs, int n_rs, int p, int &split)
{
    const uint64_t key = keys[p];
    split = 0;
    if (key == kOcNoObject) return false;
    split = row_split_of(rs, n_rs, vals[p]);
    if (p == 0) return true;
    return keys[p - 1] != key || row_split_of(rs, n_rs, vals[p - 1]) != split;
}

__global__ void __launch_bounds__(256)
k_oc_flags(const uint64_t *__restrict__ keys, const int *__restrict__ vals, const int64_t *__restrict__ rs,
           int n_rs, int n_vert, int *__restrict__ flags, OcHeader *h)
{
    const int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (h->status != 0) return;
    if (p == n_vert) { flags[p] = 0; return; }
    if (p > n_vert) return;
    int split;
    flags[p] = oc_is_head(keys, vals, rs, n_rs, p, split) ? 1 : 0;
    if (keys[p] != kOcNoObject && (p + 1 == n_vert || keys[p + 1] == kOcNoObject)) h->n_valid = p + 1;
}

__global__ void __launch_bounds__(256)
k_oc_objects(const uint64_t *__restrict__ keys, const int *__restrict__ vals, const int64_t *__restrict__ rs,
             int n_rs, int n_vert, const int *__restrict__ scanned, int *__restrict__ obj_start,
             int *__restrict__ obj_split, unsigned long long *__restrict__ objects_per_split, OcHeader *h)
{
    const int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= n_vert || h->status != 0) return;
    if (p == 0) {
        const int n_unique = scanned[n_vert];
        h->n_unique = n_unique;
        obj_start[n_unique] = h->n_valid;
    }
    int split;
    if (oc_is_head(keys, vals, rs, n_rs, p, split)) {
        const int k = scanned[p];
        obj_start[k] = p;
        obj_split[k] = split;
        atomicAdd(objects_per_split + split, 1ull);
    }
}

__global__ void __launch_bounds__(256)
k_oc_largest(const int *__restrict__ obj_start, int n_vert, OcHeader *h)
{
    const int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (h->status != 0 || k >= h->n_unique) return;
    int c = obj_start[k + 1] - obj_start[k];
    c = __reduce_max_sync(__activemask(), c);
    if ((threadIdx.x & 31) == 0 || k == 0) atomicMax(&h->n_maxuq, c);
}

__global__ void __launch_bounds__(256)
k_oc_fill_m(const int *__restrict__ vals, const int *__restrict__ obj_start, int64_t n_unique, int64_t n_maxuq,
            int64_t *__restrict__ M)
{
    const int64_t total = n_unique * n_maxuq;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += stride) {
        const int64_t k = t / n_maxuq, j = t - k * n_maxuq;
        const int beg = obj_start[k], cnt = obj_start[k + 1] - beg;
        M[t] = j < cnt ? (int64_t)vals[beg + j] : (int64_t)-1;
    }
}

// M_not, one warp per run of kOcRun tiles of kOcTile consecutive columns of one row.  The j-th
// non-member is  row start + j + t(j),  t(j) = number of members with at most j non-members
// before them.  t is non-decreasing in j: the warp searches it once for the first column of
// its run (uniform loads) and then walks the member list forward, tile by tile -- every member
// that falls into the tile raises t by one from its column on.  A tile with more than
// kOcLinear members (a dense object) lets every column search between the tile's bounds
// instead.  VEC2: rows are 16-byte aligned (even row length, aligned base) and a lane stores
// two adjacent columns at once.
constexpr int kOcTile = 512;
constexpr int kOcRun = 4;
constexpr int kOcLinear = 16;

template <bool VEC2>
__global__ void __launch_bounds__(256)
k_oc_fill_m_not(const int *__restrict__ vals, const int *__restrict__ obj_start,
                const int *__restrict__ obj_split, const int64_t *__restrict__ rs, int64_t n_unique,
                int n_maxrs, int64_t *__restrict__ M_not)
{
    const int lane = threadIdx.x & 31;
    constexpr int kSpan = kOcTile * kOcRun;
    const int runs_per_row = (n_maxrs + kSpan - 1) / kSpan;
    const int64_t n_runs = n_unique * runs_per_row;
    const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t run = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; run < n_runs; run += n_warps) {
        const int64_t k = run / runs_per_row;
        const int run0 = (int)(run - k * runs_per_row) * kSpan;
        const int beg = obj_start[k], cnt = obj_start[k + 1] - beg;
        const int e = obj_split[k];
        const int64_t row_start = rs[e];
        const int n_non = (int)(rs[e + 1] - row_start) - cnt;
        // member i (a global point id) has  members[i] - row_start - i  non-members before it
        const int *__restrict__ members = vals + beg;
        const int rs32 = (int)row_start;
        auto members_up_to = [&](int j, int lo, int hi) {
            while (lo < hi) {
                const int mid = (lo + hi) >> 1;
                if (members[mid] - rs32 - mid <= j) lo = mid + 1; else hi = mid;
            }
            return lo;
        };
        int64_t *__restrict__ row = M_not + k * (int64_t)n_maxrs;
        int t_first = members_up_to(run0, 0, cnt);
        for (int j0 = run0; j0 < run0 + kSpan && j0 < n_maxrs; j0 += kOcTile) {
            const int j_end = j0 + kOcTile < n_maxrs ? j0 + kOcTile : n_maxrs;
            constexpr int PER = kOcTile / 32;           // columns per lane
            auto column = [&](int u) { return VEC2 ? j0 + 2 * lane + 64 * (u >> 1) + (u & 1) : j0 + lane + 32 * u; };
            int t_of[PER];
#pragma unroll
            for (int u = 0; u < PER; u++) t_of[u] = t_first;
            int t = t_first;
            for (; t < cnt && t - t_first <= kOcLinear; t++) {
                const int b = members[t] - rs32 - t;
                if (b >= j_end) break;
#pragma unroll
                for (int u = 0; u < PER; u++) t_of[u] += column(u) >= b ? 1 : 0;
            }
            if (t - t_first > kOcLinear) {
                t = members_up_to(j_end - 1, t, cnt);
#pragma unroll
                for (int u = 0; u < PER; u++) t_of[u] = members_up_to(column(u), t_first, t);
            }
            if (VEC2) {
#pragma unroll
                for (int u = 0; u < PER; u += 2) {
                    const int j = column(u);
                    if (j < j_end) {    // j_end is even here, so j + 1 < j_end as well
                        longlong2 v;
                        v.x = j < n_non ? row_start + j + t_of[u] : -1;
                        v.y = j + 1 < n_non ? row_start + j + 1 + t_of[u + 1] : -1;
                        *reinterpret_cast<longlong2 *>(row + j) = v;
                    }
                }
            } else {
#pragma unroll
                for (int u = 0; u < PER; u++) {
                    const int j = column(u);
                    if (j < j_end) row[j] = j < n_non ? row_start + j + t_of[u] : -1;
                }
            }
            t_first = t;
        }
    }
}

// out[(v*K + k)*F + f] = idx[v, k] == -1 ? default : feat[idx[v, k]*F + f], on raw words
template <typename W>
__global__ void __launch_bounds__(256)
k_select_with_default(const int64_t *__restrict__ idx, const W *__restrict__ feat, int64_t n_rows_feat,
                      int64_t n_idx, int64_t F, W default_word, W *__restrict__ out)
{
    const int64_t total = n_idx * F;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += stride) {
        const int64_t e = t / F, f = t - e * F;
        const int64_t i = idx[e];
        out[t] = (i >= 0 && i < n_rows_feat) ? feat[i * F + f] : default_word;
    }
}

}  // namespace fgc

extern "C" size_t fgc_oc_workspace_bytes(int64_t n_vert)
{
    if (n_vert < 0 || n_vert > 0x7ffffff0) return 0;
    return fgc::oc_workspace_layout(n_vert).total;
}

extern "C" int fgc_oc_prepare(const int64_t *asso_idx, int64_t n_vert, const int64_t *row_splits, int64_t n_rs,
                              void *workspace, size_t workspace_bytes, int64_t *objects_per_split,
                              fgc_stream_t stream)
{
    FGC_NVTX("fgc_oc_prepare");
    using namespace fgc;
    if (n_vert < 0 || n_rs < 1 || !row_splits || (!objects_per_split && n_rs > 1)) return FGC_ERR_BAD_ARGUMENT;
    if (n_vert > 0x7ffffff0 || n_rs > 0x7fffffff) return FGC_ERR_TOO_LARGE;
    const OcWorkspace L = oc_workspace_layout(n_vert);
    if (!workspace || workspace_bytes < L.total || ((uintptr_t)workspace & 255)) return FGC_ERR_WORKSPACE;
    cudaStream_t s = (cudaStream_t)stream;
    char *ws = (char *)workspace;
    OcHeader *h = (OcHeader *)(ws + L.header);
    FGC_RETURN_IF_CUDA(cudaMemsetAsync(h, 0, kOcHeaderBytes, s));
    if (n_rs > 1)
        FGC_RETURN_IF_CUDA(cudaMemsetAsync(objects_per_split, 0, sizeof(int64_t) * (size_t)(n_rs - 1), s));
    k_oc_check<<<1, 32, 0, s>>>(row_splits, (int)n_rs, (int)n_vert, h);
    FGC_CHECK_LAUNCH();
    if (n_vert == 0) return FGC_OK;
    if (!asso_idx) return FGC_ERR_BAD_ARGUMENT;
    const int n = (int)n_vert;
    const int blocks = (n + 255) / 256;
    uint64_t *keys_a = (uint64_t *)(ws + L.keys_a), *keys_b = (uint64_t *)(ws + L.keys_b);
    int *vals_a = (int *)(ws + L.vals_a), *vals_b = (int *)(ws + L.vals_b);
    k_oc_keys<<<blocks, 256, 0, s>>>(asso_idx, n, keys_a, vals_a);
    FGC_CHECK_LAUNCH();
    // stable LSD radix sort: equal truth indices keep ascending point ids
    cub::DoubleBuffer<uint64_t> dk(keys_a, keys_b);
    cub::DoubleBuffer<int> dv(vals_a, vals_b);
    size_t need = 0;
    FGC_RETURN_IF_CUDA(cub::DeviceRadixSort::SortPairs(nullptr, need, dk, dv, n, 0, 64, s));
    if (need > L.cub_temp_bytes) return FGC_ERR_WORKSPACE;
    FGC_RETURN_IF_CUDA(cub::DeviceRadixSort::SortPairs(ws + L.cub_temp, need, dk, dv, n, 0, 64, s));
    // keep the sorted lists where the fill kernels expect them
    if (dk.Current() != keys_a)
        FGC_RETURN_IF_CUDA(cudaMemcpyAsync(keys_a, dk.Current(), 8 * (size_t)n, cudaMemcpyDeviceToDevice, s));
    if (dv.Current() != vals_a)
        FGC_RETURN_IF_CUDA(cudaMemcpyAsync(vals_a, dv.Current(), 4 * (size_t)n, cudaMemcpyDeviceToDevice, s));
    int *flags = (int *)(ws + L.flags);
    int *blocksums = (int *)(ws + L.blocksums);
    int *obj_start = (int *)(ws + L.obj_start);
    int *obj_split = (int *)(ws + L.obj_split);
    k_oc_flags<<<(n + 1 + 255) / 256, 256, 0, s>>>(keys_a, vals_a, row_splits, (int)n_rs, n, flags, h);
    FGC_CHECK_LAUNCH();
    const int scan_blocks = (int)ceil_div64((int64_t)n + 1, kScanTile);
    k_scan_tile_sums<<<scan_blocks, 256, 0, s>>>(flags, nullptr, n + 1, blocksums);
    FGC_CHECK_LAUNCH();
    k_scan_block_sums<<<1, 1024, 0, s>>>(blocksums, nullptr, n + 1);
    FGC_CHECK_LAUNCH();
    k_scan_apply<<<scan_blocks, 256, 0, s>>>(flags, nullptr, n + 1, blocksums);
    FGC_CHECK_LAUNCH();
    k_oc_objects<<<blocks, 256, 0, s>>>(keys_a, vals_a, row_splits, (int)n_rs, n, flags, obj_start, obj_split,
                                        (unsigned long long *)objects_per_split, h);
    FGC_CHECK_LAUNCH();
    k_oc_largest<<<blocks, 256, 0, s>>>(obj_start, n, h);
    FGC_CHECK_LAUNCH();
    return FGC_OK;
}

extern "C" int fgc_oc_read_sizes(const void *workspace, int32_t *status_host, int64_t sizes_host[3],
                                 fgc_stream_t stream)
{
    using namespace fgc;
    if (!workspace || !status_host || !sizes_host) return FGC_ERR_BAD_ARGUMENT;
    OcHeader h;
    cudaStream_t s = (cudaStream_t)stream;
    FGC_RETURN_IF_CUDA(cudaMemcpyAsync(&h, workspace, sizeof(OcHeader), cudaMemcpyDeviceToHost, s));
    FGC_RETURN_IF_CUDA(cudaStreamSynchronize(s));
    *status_host = h.status;
    sizes_host[0] = h.n_unique;
    sizes_host[1] = h.n_maxuq;
    sizes_host[2] = h.n_maxrs;
    return FGC_OK;
}

extern "C" int fgc_oc_fill(const void *workspace, size_t workspace_bytes, int64_t n_vert,
                           const int64_t *row_splits, int64_t n_unique, int64_t n_maxuq, int64_t n_maxrs,
                           int64_t *out_M, int64_t *out_M_not_or_null, fgc_stream_t stream)
{
    FGC_NVTX("fgc_oc_fill");
    using namespace fgc;
    if (n_vert < 0 || n_unique < 0 || n_maxuq < 0 || n_maxrs < 0 || !row_splits) return FGC_ERR_BAD_ARGUMENT;
    if (n_vert > 0x7ffffff0) return FGC_ERR_TOO_LARGE;
    const OcWorkspace L = oc_workspace_layout(n_vert);
    if (!workspace || workspace_bytes < L.total || ((uintptr_t)workspace & 255)) return FGC_ERR_WORKSPACE;
    cudaStream_t s = (cudaStream_t)stream;
    const char *ws = (const char *)workspace;
    const int *vals = (const int *)(ws + L.vals_a);
    const int *obj_start = (const int *)(ws + L.obj_start);
    const int *obj_split = (const int *)(ws + L.obj_split);
    const int64_t m_total = n_unique * n_maxuq, mn_total = n_unique * n_maxrs;
    if (m_total > 0) {
        if (!out_M) return FGC_ERR_BAD_ARGUMENT;
        int64_t blocks = ceil_div64(m_total, 256);
        if (blocks > fgc::sm_count() * 64) blocks = fgc::sm_count() * 64;
        k_oc_fill_m<<<(unsigned)blocks, 256, 0, s>>>(vals, obj_start, n_unique, n_maxuq, out_M);
        FGC_CHECK_LAUNCH();
    }
    if (out_M_not_or_null && mn_total > 0) {
        if (n_maxrs > 0x7fffffff) return FGC_ERR_TOO_LARGE;
        const int64_t runs = n_unique * ceil_div64(n_maxrs, kOcTile * kOcRun);
        int64_t blocks = ceil_div64(runs, 8);           // 8 warps per CTA, one run of tiles per warp and pass
        if (blocks > fgc::sm_count() * 32) blocks = fgc::sm_count() * 32;
        if ((n_maxrs & 1) == 0 && ((uintptr_t)out_M_not_or_null & 15) == 0)
            k_oc_fill_m_not<true><<<(unsigned)blocks, 256, 0, s>>>(vals, obj_start, obj_split, row_splits, n_unique,
                                                                   (int)n_maxrs, out_M_not_or_null);
        else
            k_oc_fill_m_not<false><<<(unsigned)blocks, 256, 0, s>>>(vals, obj_start, obj_split, row_splits, n_unique,
                                                                    (int)n_maxrs, out_M_not_or_null);
        FGC_CHECK_LAUNCH();
    }
    return FGC_OK;
}

extern "C" int fgc_select_with_default(const int64_t *idx, int64_t n_idx, const void *feat, int64_t n_rows_feat,
                                       int64_t n_feat, int32_t word_bytes, const void *default_word_host,
                                       void *out, fgc_stream_t stream)
{
    FGC_NVTX("fgc_select_with_default");
    using namespace fgc;
    if (n_idx < 0 || n_rows_feat < 0 || n_feat < 0 || !default_word_host) return FGC_ERR_BAD_ARGUMENT;
    if (word_bytes != 4 && word_bytes != 8) return FGC_ERR_BAD_ARGUMENT;
    const int64_t total = n_idx * n_feat;
    if (total == 0) return FGC_OK;
    if (!idx || !out || (!feat && n_rows_feat > 0)) return FGC_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    int64_t blocks = ceil_div64(total, 256);
    if (blocks > fgc::sm_count() * 64) blocks = fgc::sm_count() * 64;
    if (word_bytes == 4) {
        uint32_t w;
        memcpy(&w, default_word_host, 4);
        k_select_with_default<uint32_t><<<(unsigned)blocks, 256, 0, s>>>(
            idx, (const uint32_t *)feat, n_rows_feat, n_idx, n_feat, w, (uint32_t *)out);
    } else {
        uint64_t w;
        memcpy(&w, default_word_host, 8);
        k_select_with_default<uint64_t><<<(unsigned)blocks, 256, 0, s>>>(
            idx, (const uint64_t *)feat, n_rows_feat, n_idx, n_feat, w, (uint64_t *)out);
    }
    FGC_CHECK_LAUNCH();
    return FGC_OK;
}
