// Radius cut of a kNN result (sm_100a): the "max_radius" mode of the reference's brute-force
// op select_knn::select_knn (select_knn.cpp:60-62, select_knn_cpu.cpp:98-132,
// select_knn_cuda_kernel.cu:73-132).
//
// That op returns, per point, the K-1 nearest other points of its row split that lie within
// max_radius (squared comparison, boundary included).  The K-1 nearest points within a radius
// are exactly those of the K-1 nearest points overall that lie within it, so the mode is a
// filter on the result of the grid search (which already scans small row splits exhaustively):
// one warp per row drops the slots beyond the radius and closes the gaps, keeping the order of
// the remaining slots; freed slots become pads (-1, or the point itself with tf_compat) with
// distance 0, as the reference's defaults.
#include "fgc_common.cuh"

namespace fgc {

constexpr int kRadiusWarps = 8;
constexpr int kRadiusChunks = (FGC_MAX_K + 31) / 32;

__global__ void __launch_bounds__(kRadiusWarps * 32)
k_knn_radius_filter(int64_t *__restrict__ idx, float *__restrict__ dist, int n_vert, int K,
                    float max_radius_sq, int tf_compat)
{
    const int lane = threadIdx.x & 31;
    const int i = blockIdx.x * kRadiusWarps + (threadIdx.x >> 5);
    if (i >= n_vert) return;
    int64_t *__restrict__ ri = idx + (size_t)i * K;
    float *__restrict__ rd = dist + (size_t)i * K;
    int64_t vi[kRadiusChunks];
    float vd[kRadiusChunks];
    int pos[kRadiusChunks];
    int kept = 0;
#pragma unroll
    for (int c = 0; c < kRadiusChunks; c++) {
        const int s = c * 32 + lane;
        bool keep = false;
        pos[c] = -1;
        if (c * 32 < K) {
            if (s < K) {
                vi[c] = ri[s];
                vd[c] = rd[s];
                const bool pad = s > 0 && (vi[c] < 0 || (tf_compat && vi[c] == (int64_t)i));
                keep = s == 0 || (!pad && vd[c] <= max_radius_sq);
            }
            const unsigned m = __ballot_sync(FGC_FULL_MASK, keep);
            if (keep) pos[c] = kept + __popc(m & lanemask_lt());
            kept += __popc(m);
        }
    }
    __syncwarp();
#pragma unroll
    for (int c = 0; c < kRadiusChunks; c++) {
        if (c * 32 < K) {
            if (pos[c] >= 0) { ri[pos[c]] = vi[c]; rd[pos[c]] = vd[c]; }
            const int s = c * 32 + lane;
            if (s >= kept && s < K) { ri[s] = tf_compat ? (int64_t)i : (int64_t)-1; rd[s] = 0.f; }
        }
    }
}

}  // namespace fgc

extern "C" int fgc_knn_radius_filter(int64_t *idx, float *distsq, int64_t n_vert, int32_t K,
                                     double max_radius, int32_t tf_compat, fgc_stream_t stream)
{
    FGC_NVTX("fgc_knn_radius_filter");
    using namespace fgc;
    if (n_vert < 0 || K < 1) return FGC_ERR_BAD_ARGUMENT;
    if (K > FGC_MAX_K) return FGC_ERR_UNSUPPORTED_K;
    if (n_vert > 0x7fffffff) return FGC_ERR_TOO_LARGE;
    if (!(max_radius > 0.0) || n_vert == 0) return FGC_OK;     // no radius: nothing to cut
    if (!idx || !distsq) return FGC_ERR_BAD_ARGUMENT;
    const int n = (int)n_vert;
    k_knn_radius_filter<<<(n + kRadiusWarps - 1) / kRadiusWarps, kRadiusWarps * 32, 0, (cudaStream_t)stream>>>(
        idx, distsq, n, K, (float)(max_radius * max_radius), tf_compat);   // squared in double, as the reference
    FGC_CHECK_LAUNCH();
    return FGC_OK;
}
