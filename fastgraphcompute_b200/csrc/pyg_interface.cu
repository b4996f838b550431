// row_splits <-> PyTorch-Geometric style batch vectors on the device
// (fastgraphcompute/torch_geometric_interface.py:4-74 of the reference, which does it with
// nonzero / repeat_interleave tensor ops).
//
// batch -> row_splits: a point starts a new row split where its batch id differs from its
// predecessor's.  Flags, exclusive scan, scatter: the heads come out in ascending order with
// no sort.  row_splits -> batch: every point finds its row split by binary search.
#include "fgc_common.cuh"
#include "scan.cuh"

namespace fgc {

struct PygLayout {
    size_t header, flags, blocksums, total;
};

static PygLayout pyg_layout(int64_t n)
{
    PygLayout L;
    size_t off = 0;
    L.header = off; off += 256;
    L.flags = off; off = align_up(off + sizeof(int32_t) * (size_t)(n + 1), 256);
    L.blocksums = off; off = align_up(off + sizeof(int32_t) * (size_t)((n + 1) / kScanTile + 2), 256);
    L.total = off;
    return L;
}

static __global__ void __launch_bounds__(256)
k_pyg_flags(const int64_t *__restrict__ batch, int n, int *__restrict__ flags)
{
    const int i = blockIdx.x * 256 + threadIdx.x;
    if (i > n) return;
    // entry n is a sentinel: after the exclusive scan it holds the number of heads
    flags[i] = (i > 0 && i < n && batch[i] != batch[i - 1]) ? 1 : 0;
}

static __global__ void __launch_bounds__(256)
k_pyg_scatter(const int64_t *__restrict__ batch, int n, const int *__restrict__ pos,
              int64_t *__restrict__ row_splits, int32_t *__restrict__ header)
{
    const int i = blockIdx.x * 256 + threadIdx.x;
    if (i > n) return;
    if (i == 0) row_splits[0] = 0;
    if (i == n) {
        const int heads = pos[n];
        row_splits[heads + 1] = n;
        header[0] = heads + 2;          // entries of row_splits
        return;
    }
    if (i > 0 && batch[i] != batch[i - 1]) row_splits[1 + pos[i]] = i;
}

static __global__ void __launch_bounds__(256)
k_pyg_batch(const int64_t *__restrict__ rs, int n_rs, int64_t n, int64_t *__restrict__ batch)
{
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (int64_t)gridDim.x * 256)
        batch[i] = row_split_of(rs, n_rs, i);
}

}  // namespace fgc

extern "C" size_t fgc_pyg_workspace_bytes(int64_t n_points)
{
    if (n_points < 0 || n_points > 0x7ffffffe) return 0;
    return fgc::pyg_layout(n_points).total;
}

extern "C" int fgc_row_splits_from_strict_batch(const int64_t *batch, int64_t n_points,
                                                int64_t *out_row_splits, void *workspace,
                                                size_t workspace_bytes, fgc_stream_t stream)
{
    FGC_NVTX("fgc_row_splits_from_strict_batch");
    using namespace fgc;
    if (n_points < 0 || !out_row_splits) return FGC_ERR_BAD_ARGUMENT;
    if (n_points > 0x7ffffffe) return FGC_ERR_TOO_LARGE;
    if (n_points > 0 && !batch) return FGC_ERR_BAD_ARGUMENT;
    const PygLayout L = pyg_layout(n_points);
    if (!workspace || workspace_bytes < L.total || ((uintptr_t)workspace & 255)) return FGC_ERR_WORKSPACE;
    cudaStream_t s = (cudaStream_t)stream;
    char *ws = (char *)workspace;
    int *flags = (int *)(ws + L.flags);
    int *blocksums = (int *)(ws + L.blocksums);
    const int n = (int)n_points;
    const int blocks = (n + 1 + 255) / 256;
    const int scan_blocks = (int)ceil_div64(n + 1, kScanTile);
    k_pyg_flags<<<blocks, 256, 0, s>>>(batch, n, flags);
    FGC_CHECK_LAUNCH();
    k_scan_tile_sums<<<scan_blocks, 256, 0, s>>>(flags, nullptr, n + 1, blocksums);
    FGC_CHECK_LAUNCH();
    k_scan_block_sums<<<1, 1024, 0, s>>>(blocksums, nullptr, n + 1);
    FGC_CHECK_LAUNCH();
    k_scan_apply<<<scan_blocks, 256, 0, s>>>(flags, nullptr, n + 1, blocksums);
    FGC_CHECK_LAUNCH();
    k_pyg_scatter<<<blocks, 256, 0, s>>>(batch, n, flags, out_row_splits, (int32_t *)(ws + L.header));
    return (int)cudaGetLastError();
}

extern "C" int fgc_pyg_read_count(const void *workspace, int64_t *n_row_splits_host, fgc_stream_t stream)
{
    if (!workspace || !n_row_splits_host) return FGC_ERR_BAD_ARGUMENT;
    int32_t v = 0;
    cudaStream_t s = (cudaStream_t)stream;
    FGC_RETURN_IF_CUDA(cudaMemcpyAsync(&v, workspace, sizeof(v), cudaMemcpyDeviceToHost, s));
    FGC_RETURN_IF_CUDA(cudaStreamSynchronize(s));
    *n_row_splits_host = v;
    return FGC_OK;
}

extern "C" int fgc_strict_batch_from_row_splits(const int64_t *row_splits, int64_t n_rs, int64_t n_points,
                                                int64_t *out_batch, fgc_stream_t stream)
{
    FGC_NVTX("fgc_strict_batch_from_row_splits");
    using namespace fgc;
    if (!row_splits || n_rs < 1 || n_points < 0) return FGC_ERR_BAD_ARGUMENT;
    if (n_rs > 0x7fffffff) return FGC_ERR_TOO_LARGE;
    if (n_points == 0) return FGC_OK;
    if (!out_batch) return FGC_ERR_BAD_ARGUMENT;
    int64_t blocks = ceil_div64(n_points, 256);
    if (blocks > (int64_t)fgc::sm_count() * 16) blocks = (int64_t)fgc::sm_count() * 16;
    k_pyg_batch<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(row_splits, (int)n_rs, n_points, out_batch);
    return (int)cudaGetLastError();
}
