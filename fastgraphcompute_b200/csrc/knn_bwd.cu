// Gradient of the kNN squared distances w.r.t. the coordinates (sm_100a).
//
//   G[i,v] = -sum_k 2 g[i,k] (x[n,v] - x[i,v])        (the row's own term)
//   G[n,v] +=        2 g[i,k] (x[n,v] - x[i,v])        (scattered to n = idx[i,k] >= 0)
// as in extensions/binned_select_knn_grad_cpu.cpp:6-93 (CUDA twin
// extensions/binned_select_knn_grad_cuda_kernel.cu:25-88).
//
// One warp per row: the lanes take the K slots (coalesced idx / grad loads), the
// row's own term is reduced inside the warp and leaves as ONE add per
// coordinate, the neighbour term leaves as one reduction per slot: a 16-byte
// (D = 4; two of them for D = 8) or 8-byte (D = 2) vector reduction, else one fp32
// reduction per coordinate.  (Summing the neighbour terms of 64 cell-adjacent rows per target in a
// shared-memory hash table first, one reduction per distinct target and CTA, was measured
// at twice the time: float adds on shared memory plus the probe cost more than the L2
// reductions they save; without any reductions the kernel would be 22 % faster.)
//
// `order` (optional) is a permutation of the rows: warp w works on row order[w].  Given the
// cell order of the search that produced idx, the warps of a CTA work on rows of one cell or of
// neighbouring cells, whose neighbour sets largely coincide: the scattered 16-byte gathers of
// neighbour coordinates hit in L1, and the reductions of one CTA go to few L2 lines.  The
// gradient does not depend on it (up to the order of the float additions).
#include "fgc_common.cuh"

namespace fgc {

constexpr int kBwdWarps = 8;

template <int D>
__global__ void __launch_bounds__(kBwdWarps * 32)
k_knn_bwd(const float *__restrict__ grad_distsq, const int64_t *__restrict__ idx,
          const float *__restrict__ coords, int n_vert, int K, int n_coords_rt,
          float *__restrict__ out, int vec_ok, const int32_t *__restrict__ order)
{
    const int lane = threadIdx.x & 31;
    const int wi = blockIdx.x * kBwdWarps + (threadIdx.x >> 5);
    if (wi >= n_vert) return;
    const int i = order ? __ldg(order + wi) : wi;
    if (i < 0 || i >= n_vert) return;
    const int nc = D > 0 ? D : n_coords_rt;
    constexpr int DM = D > 0 ? D : 1;
    if (D > 0) {
        float xi[DM], self[DM];
#pragma unroll
        for (int v = 0; v < DM; v++) { xi[v] = __ldg(coords + (size_t)i * nc + v); self[v] = 0.f; }
        for (int k0 = 0; k0 < K; k0 += 32) {
            const int k = k0 + lane;
            if (k < K) {
                const int64_t n = idx[(size_t)i * K + k];
                if (n >= 0 && n < n_vert) {
                    const float g2 = 2.f * grad_distsq[(size_t)i * K + k];
                    float c[DM], xn[DM];
                    if ((D == 4 || D == 8) && vec_ok) {
                        // 16-byte gathers instead of 4-byte ones: the kernel is bound by L1TEX
                        // requests (C2: 0.099 -> 0.080 ms)
#pragma unroll
                        for (int q4 = 0; q4 < DM / 4; q4++) {
                            const float4 t4 = __ldg((const float4 *)(coords + (size_t)n * DM) + q4);
                            xn[(4 * q4) % DM] = t4.x; xn[(4 * q4 + 1) % DM] = t4.y;
                            xn[(4 * q4 + 2) % DM] = t4.z; xn[(4 * q4 + 3) % DM] = t4.w;
                        }
                    } else {
#pragma unroll
                        for (int v = 0; v < DM; v++) xn[v] = __ldg(coords + (size_t)n * nc + v);
                    }
#pragma unroll
                    for (int v = 0; v < DM; v++) {
                        c[v] = g2 * (xn[v] - xi[v]);
                        self[v] -= c[v];
                    }
                    // one vector reduction per neighbour where the row is 8 or 16 bytes wide
                    if ((D == 4 || D == 8) && vec_ok) {
#pragma unroll
                        for (int q4 = 0; q4 < DM / 4; q4++)
                            atomicAdd((float4 *)(out + (size_t)n * DM) + q4,
                                      make_float4(c[(4 * q4) % DM], c[(4 * q4 + 1) % DM], c[(4 * q4 + 2) % DM],
                                                  c[(4 * q4 + 3) % DM]));
                    }
                    else if (D == 2 && vec_ok)
                        atomicAdd((float2 *)(out + (size_t)n * 2), make_float2(c[0], c[1 % DM]));
                    else {
#pragma unroll
                        for (int v = 0; v < DM; v++) atomicAdd(out + (size_t)n * nc + v, c[v]);
                    }
                }
            }
        }
#pragma unroll
        for (int v = 0; v < DM; v++) {
            float s = self[v];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(FGC_FULL_MASK, s, o);
            if (lane == 0) atomicAdd(out + (size_t)i * nc + v, s);
        }
    } else {
        // any number of coordinates: one coordinate at a time
        for (int v = 0; v < nc; v++) {
            const float xi = __ldg(coords + (size_t)i * nc + v);
            float self = 0.f;
            for (int k = lane; k < K; k += 32) {
                const int64_t n = idx[(size_t)i * K + k];
                if (n >= 0 && n < n_vert) {
                    const float c = 2.f * grad_distsq[(size_t)i * K + k] *
                                    (__ldg(coords + (size_t)n * nc + v) - xi);
                    self -= c;
                    atomicAdd(out + (size_t)n * nc + v, c);
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) self += __shfl_xor_sync(FGC_FULL_MASK, self, o);
            if (lane == 0) atomicAdd(out + (size_t)i * nc + v, self);
        }
    }
}

}  // namespace fgc

extern "C" int fgc_binned_knn_bwd(const float *grad_distsq, const int64_t *idx, const float *coords,
                                  int64_t n_vert, int32_t K, int32_t n_coords,
                                  float *out_grad_coords, fgc_stream_t stream)
{
    return fgc_binned_knn_bwd_ordered(grad_distsq, idx, coords, n_vert, K, n_coords, nullptr, out_grad_coords,
                                      stream);
}

extern "C" int fgc_binned_knn_bwd_ordered(const float *grad_distsq, const int64_t *idx, const float *coords,
                                          int64_t n_vert, int32_t K, int32_t n_coords,
                                          const int32_t *order_or_null, float *out_grad_coords,
                                          fgc_stream_t stream)
{
    FGC_NVTX("fgc_binned_knn_bwd");
    using namespace fgc;
    if (n_vert < 0 || K < 1 || n_coords < 1) return FGC_ERR_BAD_ARGUMENT;
    if (n_vert > 0x7fffffff) return FGC_ERR_TOO_LARGE;
    if (n_vert == 0) return FGC_OK;
    if (!grad_distsq || !idx || !coords || !out_grad_coords) return FGC_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    FGC_RETURN_IF_CUDA(cudaMemsetAsync(out_grad_coords, 0, sizeof(float) * (size_t)n_vert * n_coords, s));
    const int n = (int)n_vert;
    const unsigned blocks = (unsigned)((n + kBwdWarps - 1) / kBwdWarps);
    const int T = kBwdWarps * 32;
    const int vec_ok = (((uintptr_t)out_grad_coords | (uintptr_t)coords) & 15) == 0;
    switch (n_coords) {
    case 2: k_knn_bwd<2><<<blocks, T, 0, s>>>(grad_distsq, idx, coords, n, K, n_coords, out_grad_coords, vec_ok, order_or_null); break;
    case 3: k_knn_bwd<3><<<blocks, T, 0, s>>>(grad_distsq, idx, coords, n, K, n_coords, out_grad_coords, vec_ok, order_or_null); break;
    case 4: k_knn_bwd<4><<<blocks, T, 0, s>>>(grad_distsq, idx, coords, n, K, n_coords, out_grad_coords, vec_ok, order_or_null); break;
    case 8: k_knn_bwd<8><<<blocks, T, 0, s>>>(grad_distsq, idx, coords, n, K, n_coords, out_grad_coords, vec_ok, order_or_null); break;
    default: k_knn_bwd<0><<<blocks, T, 0, s>>>(grad_distsq, idx, coords, n, K, n_coords, out_grad_coords, vec_ok, order_or_null); break;
    }
    FGC_CHECK_LAUNCH();
    return FGC_OK;
}
