// Fused GravNet neighbour aggregation for sm_100a (forward and backward).
//
// Forward = steps 4-7 of GravNetOp.forward (fastgraphcompute/gnn_ops.py:90-102):
//   w[i,k]    = exp(-10 * distsq[i,k])
//   val[i,k,:] = (idx[i,k] == -1 ? 0 : prop[idx[i,k],:]) * w[i,k]     (select_with_default,
//                                                      extensions/oc_helper.py:232-271)
//   mean[i,:] = sum_k val / K          max[i,:] = max_k val   (an empty slot counts as 0)
// without materialising the [N,K,P] tensors: one warp per point, lanes over the
// feature channels, every neighbour row is read once (128-byte coalesced) and
// consumed from registers.  argmax keeps the first slot that attains the max.
//
// Backward (what autograd derives for the same lines):
//   coef[i,k,p]   = g_mean[i,p]/K + g_max[i,p]*[k == argmax[i,p]]
//   d_prop[n,p]  += w[i,k]*coef[i,k,p]                      n = idx[i,k] != -1
//   d_distsq[i,k] = -10*w[i,k]*sum_p prop[n,p]*coef[i,k,p]
#include "fgc_common.cuh"

namespace fgc {

constexpr int kGravWarps = 8;

template <int PC>
__global__ void __launch_bounds__(kGravWarps * 32)
k_gravnet_fwd(const float *__restrict__ prop, const int64_t *__restrict__ idx,
              const float *__restrict__ distsq, int n_vert, int K, int P,
              float *__restrict__ out_mean, float *__restrict__ out_max,
              int32_t *__restrict__ out_argmax)
{
    const int lane = threadIdx.x & 31;
    const int i = blockIdx.x * kGravWarps + (threadIdx.x >> 5);
    if (i >= n_vert) return;
    const int pbase = blockIdx.y * 32 * PC + lane;
    float sum[PC], mx[PC];
    int am[PC];
#pragma unroll
    for (int c = 0; c < PC; c++) { sum[c] = 0.f; mx[c] = -INFINITY; am[c] = 0; }
    for (int k0 = 0; k0 < K; k0 += 32) {
        const int k = k0 + lane;
        int n_l = -1;
        float w_l = 0.f;
        if (k < K) {
            const int64_t n64 = idx[(size_t)i * K + k];
            n_l = (n64 >= 0 && n64 < n_vert) ? (int)n64 : -1;
            w_l = expf(__fmul_rn(-10.f, distsq[(size_t)i * K + k]));
        }
        const int cnt = min(32, K - k0);
        for (int kk = 0; kk < cnt; kk++) {
            const int n = __shfl_sync(FGC_FULL_MASK, n_l, kk);
            const float w = __shfl_sync(FGC_FULL_MASK, w_l, kk);
#pragma unroll
            for (int c = 0; c < PC; c++) {
                const int p = pbase + 32 * c;
                if (p < P) {
                    const float x = n >= 0 ? __ldg(prop + (size_t)n * P + p) : 0.f;
                    const float val = __fmul_rn(x, w);
                    sum[c] = __fadd_rn(sum[c], val);
                    if (val > mx[c]) { mx[c] = val; am[c] = k0 + kk; }
                }
            }
        }
    }
#pragma unroll
    for (int c = 0; c < PC; c++) {
        const int p = pbase + 32 * c;
        if (p < P) {
            out_mean[(size_t)i * P + p] = __fdiv_rn(sum[c], (float)K);
            out_max[(size_t)i * P + p] = mx[c];
            if (out_argmax) out_argmax[(size_t)i * P + p] = am[c];
        }
    }
}

template <int PC>
__global__ void __launch_bounds__(kGravWarps * 32)
k_gravnet_bwd(const float *__restrict__ prop, const int64_t *__restrict__ idx,
              const float *__restrict__ distsq, const int32_t *__restrict__ argmax,
              const float *__restrict__ g_mean, const float *__restrict__ g_max, int n_vert,
              int K, int P, float *__restrict__ d_prop, float *__restrict__ d_distsq,
              int accumulate_dd)
{
    const int lane = threadIdx.x & 31;
    const int i = blockIdx.x * kGravWarps + (threadIdx.x >> 5);
    if (i >= n_vert) return;
    const int pbase = blockIdx.y * 32 * PC + lane;
    float gm[PC], gx[PC];
    int am[PC];
#pragma unroll
    for (int c = 0; c < PC; c++) {
        const int p = pbase + 32 * c;
        const bool ok = p < P;
        gm[c] = ok ? __fdiv_rn(g_mean[(size_t)i * P + p], (float)K) : 0.f;
        gx[c] = ok ? g_max[(size_t)i * P + p] : 0.f;
        am[c] = ok ? argmax[(size_t)i * P + p] : -1;
    }
    for (int k0 = 0; k0 < K; k0 += 32) {
        const int k = k0 + lane;
        int n_l = -1;
        float w_l = 0.f;
        if (k < K) {
            const int64_t n64 = idx[(size_t)i * K + k];
            n_l = (n64 >= 0 && n64 < n_vert) ? (int)n64 : -1;
            w_l = expf(__fmul_rn(-10.f, distsq[(size_t)i * K + k]));
        }
        float dd_l = 0.f;
        const int cnt = min(32, K - k0);
        for (int kk = 0; kk < cnt; kk++) {
            const int n = __shfl_sync(FGC_FULL_MASK, n_l, kk);
            if (n < 0) continue;   // warp-uniform
            const float w = __shfl_sync(FGC_FULL_MASK, w_l, kk);
            float dot = 0.f;
#pragma unroll
            for (int c = 0; c < PC; c++) {
                const int p = pbase + 32 * c;
                if (p < P) {
                    const float coef = gm[c] + (am[c] == k0 + kk ? gx[c] : 0.f);
                    dot = fmaf(__ldg(prop + (size_t)n * P + p), coef, dot);
                    if (coef != 0.f) atomicAdd(d_prop + (size_t)n * P + p, w * coef);
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(FGC_FULL_MASK, dot, o);
            if (lane == kk) dd_l = -10.f * w * dot;
        }
        if (k < K) {
            if (accumulate_dd) { if (dd_l != 0.f) atomicAdd(d_distsq + (size_t)i * K + k, dd_l); }
            else d_distsq[(size_t)i * K + k] = dd_l;
        }
    }
}

}  // namespace fgc

extern "C" int fgc_gravnet_aggregate_fwd(const float *prop, const int64_t *idx, const float *distsq,
                                         int64_t n_vert, int32_t K, int32_t P, float *out_mean,
                                         float *out_max, int32_t *out_argmax, fgc_stream_t stream)
{
    using namespace fgc;
    if (n_vert < 0 || K < 1 || P < 1) return FGC_ERR_BAD_ARGUMENT;
    if (n_vert > 0x7fffffff) return FGC_ERR_TOO_LARGE;
    if (n_vert == 0) return FGC_OK;
    if (!prop || !idx || !distsq || !out_mean || !out_max) return FGC_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const int n = (int)n_vert;
    const int T = kGravWarps * 32;
    dim3 grid((unsigned)((n + kGravWarps - 1) / kGravWarps), 1);
    if (P <= 32) k_gravnet_fwd<1><<<grid, T, 0, s>>>(prop, idx, distsq, n, K, P, out_mean, out_max, out_argmax);
    else if (P <= 64) k_gravnet_fwd<2><<<grid, T, 0, s>>>(prop, idx, distsq, n, K, P, out_mean, out_max, out_argmax);
    else {
        grid.y = (unsigned)((P + 127) / 128);
        k_gravnet_fwd<4><<<grid, T, 0, s>>>(prop, idx, distsq, n, K, P, out_mean, out_max, out_argmax);
    }
    FGC_CHECK_LAUNCH();
    return FGC_OK;
}

extern "C" int fgc_gravnet_aggregate_bwd(const float *prop, const int64_t *idx, const float *distsq,
                                         const int32_t *argmax, const float *grad_mean,
                                         const float *grad_max, int64_t n_vert, int32_t K, int32_t P,
                                         float *out_d_prop, float *out_d_distsq, fgc_stream_t stream)
{
    using namespace fgc;
    if (n_vert < 0 || K < 1 || P < 1) return FGC_ERR_BAD_ARGUMENT;
    if (n_vert > 0x7fffffff) return FGC_ERR_TOO_LARGE;
    if (n_vert == 0) return FGC_OK;
    if (!prop || !idx || !distsq || !argmax || !grad_mean || !grad_max || !out_d_prop || !out_d_distsq)
        return FGC_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const int n = (int)n_vert;
    const int T = kGravWarps * 32;
    FGC_RETURN_IF_CUDA(cudaMemsetAsync(out_d_prop, 0, sizeof(float) * (size_t)n_vert * P, s));
    dim3 grid((unsigned)((n + kGravWarps - 1) / kGravWarps), 1);
    if (P <= 32)
        k_gravnet_bwd<1><<<grid, T, 0, s>>>(prop, idx, distsq, argmax, grad_mean, grad_max, n, K, P, out_d_prop, out_d_distsq, 0);
    else if (P <= 64)
        k_gravnet_bwd<2><<<grid, T, 0, s>>>(prop, idx, distsq, argmax, grad_mean, grad_max, n, K, P, out_d_prop, out_d_distsq, 0);
    else {
        grid.y = (unsigned)((P + 127) / 128);
        const int acc = grid.y > 1;
        if (acc) FGC_RETURN_IF_CUDA(cudaMemsetAsync(out_d_distsq, 0, sizeof(float) * (size_t)n_vert * K, s));
        k_gravnet_bwd<4><<<grid, T, 0, s>>>(prop, idx, distsq, argmax, grad_mean, grad_max, n, K, P, out_d_prop, out_d_distsq, acc);
    }
    FGC_CHECK_LAUNCH();
    return FGC_OK;
}
