// kNN forward for callers that cannot hand the library a scratch buffer.
//
// Every other entry point takes its scratch memory from the caller, who normally gets it
// from cudaMalloc or from a framework allocator.  Some hosts can do neither at call time:
// an online event filter or an inference service that sizes all of its device memory at
// start-up and forbids later allocations (an allocation synchronises the device and may fail
// once memory is fragmented), or a plugin that only receives input and output pointers from
// its host framework and has no access to that framework's allocator.  For them this file
// keeps one fixed scratch area inside the library image itself: a file-scope __device__ array
// that every GPU which loads the library carries until the process exits.
//
// The price is a size limit (FGC_STATIC_WORKSPACE_BYTES of scratch, i.e. batches of up to a
// few ten thousand points) and one shared area per GPU: two calls that overlap on the same
// GPU -- different streams, or different host threads -- would overwrite each other's grid.
// The area keeps whatever the previous call left; the grid build clears the header and the
// cell table it is about to use, so no stale content is ever read.
#include <mutex>

#include "knn_grid.cuh"

namespace fgc {

static __device__ __align__(256) unsigned char g_static_scratch[FGC_STATIC_WORKSPACE_BYTES];

constexpr int kMaxDevices = 64;
static std::mutex g_static_mutex;
static void *g_static_ptr[kMaxDevices] = {nullptr};

// Device address of g_static_scratch on the current device.  The array's name is only a
// host-side handle; the address a kernel can use comes from cudaGetSymbolAddress, asked once
// per device with that device current and remembered.
static int static_scratch_address(void **out)
{
    int dev = -1;
    FGC_RETURN_IF_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return FGC_ERR_BAD_ARGUMENT;
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (!g_static_ptr[dev]) {
        void *p = nullptr;
        FGC_RETURN_IF_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
        if (!p || ((uintptr_t)p & 255)) return FGC_ERR_WORKSPACE;
        g_static_ptr[dev] = p;
    }
    *out = g_static_ptr[dev];
    return FGC_OK;
}

}  // namespace fgc

extern "C" int fgc_binned_knn_fwd_static(const float *coords, int64_t n_vert, int32_t n_coords,
                                         const int64_t *row_splits, int64_t n_rs, int32_t K,
                                         const int64_t *direction_or_null, int32_t tf_compat,
                                         float target_occupancy, int64_t *out_idx,
                                         float *out_distsq, int32_t *out_status,
                                         fgc_stream_t stream)
{
    using namespace fgc;
    if (!out_status) return FGC_ERR_BAD_ARGUMENT;
    const size_t need = fgc_knn_workspace_bytes(n_vert, n_coords, n_rs, K);
    if (need == 0) return FGC_ERR_BAD_ARGUMENT;
    if (need > (size_t)FGC_STATIC_WORKSPACE_BYTES) return FGC_ERR_STATIC_TOO_LARGE;
    void *scratch = nullptr;
    int rc = static_scratch_address(&scratch);
    if (rc != FGC_OK) return rc;
    rc = fgc_knn_build_grid(coords, n_vert, n_coords, row_splits, n_rs, K, direction_or_null,
                            target_occupancy, scratch, FGC_STATIC_WORKSPACE_BYTES, stream);
    if (rc != FGC_OK) return rc;
    rc = fgc_knn_search(n_vert, n_coords, n_rs, K, direction_or_null != nullptr, tf_compat, FGC_SEARCH_FRESH, out_idx,
                        out_distsq, scratch, FGC_STATIC_WORKSPACE_BYTES, stream);
    if (rc != FGC_OK) return rc;
    // the status word is the first word of the scratch area: hand it to the caller's buffer
    FGC_RETURN_IF_CUDA(cudaMemcpyAsync(out_status, scratch, sizeof(int32_t), cudaMemcpyDeviceToDevice,
                                       (cudaStream_t)stream));
    return FGC_OK;
}
