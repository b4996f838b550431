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
// `order` (optional) is a permutation of the points: warp w works on point order[w].  Given
// the cell order of the kNN that produced idx, neighbouring warps work on neighbouring
// points, whose neighbour rows largely coincide and are then served by L1 instead of L2.
// Results do not depend on it.
//
// Backward (what autograd derives for the same lines):
//   coef[i,k,p]   = g_mean[i,p]/K + g_max[i,p]*[k == argmax[i,p]]
//   d_prop[n,p]  += w[i,k]*coef[i,k,p]                      n = idx[i,k] != -1
//   d_distsq[i,k] = -10*w[i,k]*sum_p prop[n,p]*coef[i,k,p]
#include "fgc_common.cuh"
#include "reverse_graph.cuh"

namespace fgc {

constexpr int kGravWarps = 8;

template <int PC>
__global__ void __launch_bounds__(kGravWarps * 32)
k_gravnet_fwd(const float *__restrict__ prop, const int64_t *__restrict__ idx,
              const float *__restrict__ distsq, int n_vert, int K, int P,
              float *__restrict__ out_mean, float *__restrict__ out_max,
              int32_t *__restrict__ out_argmax, const int32_t *__restrict__ order, int ldo)
{
    const int lane = threadIdx.x & 31;
    const int wi = blockIdx.x * kGravWarps + (threadIdx.x >> 5);
    if (wi >= n_vert) return;
    const int i = order ? __ldg(order + wi) : wi;
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
            out_mean[(size_t)i * ldo + p] = __fdiv_rn(sum[c], (float)K);
            out_max[(size_t)i * ldo + p] = mx[c];
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
              int accumulate_dd, const int32_t *__restrict__ order, int ldg)
{
    const int lane = threadIdx.x & 31;
    const int wi = blockIdx.x * kGravWarps + (threadIdx.x >> 5);
    if (wi >= n_vert) return;
    const int i = order ? __ldg(order + wi) : wi;
    const int pbase = blockIdx.y * 32 * PC + lane;
    float gm[PC], gx[PC];
    int am[PC];
#pragma unroll
    for (int c = 0; c < PC; c++) {
        const int p = pbase + 32 * c;
        const bool ok = p < P;
        gm[c] = ok ? __fdiv_rn(g_mean[(size_t)i * ldg + p], (float)K) : 0.f;
        gx[c] = ok ? g_max[(size_t)i * ldg + p] : 0.f;
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
                    if (d_prop && coef != 0.f) atomicAdd(d_prop + (size_t)n * P + p, w * coef);
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

// ---------------------------------------------------------------------------------------
// Vectorised variants for P % 4 == 0 and P <= 128: a lane holds FOUR consecutive channels
// (16-byte loads, 16-byte vector reductions), LPN = ceil(P/4) rounded up to a power of two
// lanes cover one neighbour row and the 32/LPN lane groups of a warp work on different
// neighbour slots at the same time.  Per neighbour the shuffles, address arithmetic and
// compares are paid once per four channels instead of once per channel.  The groups' partial
// sums and maxima are combined by a fixed butterfly (ties between equal maxima go to the
// lower slot, i.e. "first slot that attains the max" is preserved).
// ---------------------------------------------------------------------------------------

template <int LPN>
__global__ void __launch_bounds__(kGravWarps * 32)
k_gravnet_fwd_v4(const float *__restrict__ prop, const int64_t *__restrict__ idx,
                 const float *__restrict__ distsq, int n_vert, int K, int P,
                 float *__restrict__ out_mean, float *__restrict__ out_max,
                 int32_t *__restrict__ out_argmax, const int32_t *__restrict__ order, int ldo)
{
    constexpr int G = 32 / LPN;
    const int lane = threadIdx.x & 31;
    const int wi = blockIdx.x * kGravWarps + (threadIdx.x >> 5);
    if (wi >= n_vert) return;
    const int i = order ? __ldg(order + wi) : wi;
    const int grp = lane / LPN, c4 = (lane % LPN) * 4;
    const bool chan = c4 < P;
    float sum[4] = {0.f, 0.f, 0.f, 0.f};
    float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
    int am[4] = {0, 0, 0, 0};
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
        for (int kk = 0; kk < cnt; kk += G) {
            const int ks = kk + grp;                     // this group's slot in the chunk
            const int n = __shfl_sync(FGC_FULL_MASK, n_l, ks & 31);
            const float w = __shfl_sync(FGC_FULL_MASK, w_l, ks & 31);
            if (ks < cnt && chan) {
                float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
                if (n >= 0) x = __ldg((const float4 *)(prop + (size_t)n * P + c4));
                const float v[4] = {__fmul_rn(x.x, w), __fmul_rn(x.y, w), __fmul_rn(x.z, w), __fmul_rn(x.w, w)};
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    sum[c] = __fadd_rn(sum[c], v[c]);
                    if (v[c] > mx[c]) { mx[c] = v[c]; am[c] = k0 + ks; }
                }
            }
        }
    }
#pragma unroll
    for (int off = LPN; off < 32; off <<= 1) {
#pragma unroll
        for (int c = 0; c < 4; c++) {
            sum[c] = __fadd_rn(sum[c], __shfl_xor_sync(FGC_FULL_MASK, sum[c], off));
            const float om = __shfl_xor_sync(FGC_FULL_MASK, mx[c], off);
            const int oa = __shfl_xor_sync(FGC_FULL_MASK, am[c], off);
            if (om > mx[c] || (om == mx[c] && oa < am[c])) { mx[c] = om; am[c] = oa; }
        }
    }
    if (grp == 0 && chan) {
        const float kf = (float)K;
        *(float4 *)(out_mean + (size_t)i * ldo + c4) =
            make_float4(__fdiv_rn(sum[0], kf), __fdiv_rn(sum[1], kf), __fdiv_rn(sum[2], kf), __fdiv_rn(sum[3], kf));
        *(float4 *)(out_max + (size_t)i * ldo + c4) = make_float4(mx[0], mx[1], mx[2], mx[3]);
        if (out_argmax) *(int4 *)(out_argmax + (size_t)i * P + c4) = make_int4(am[0], am[1], am[2], am[3]);
    }
}

template <int LPN>
__global__ void __launch_bounds__(kGravWarps * 32)
k_gravnet_bwd_v4(const float *__restrict__ prop, const int64_t *__restrict__ idx,
                 const float *__restrict__ distsq, const int32_t *__restrict__ argmax,
                 const float *__restrict__ g_mean, const float *__restrict__ g_max, int n_vert,
                 int K, int P, float *__restrict__ d_prop, float *__restrict__ d_distsq,
                 const int32_t *__restrict__ order, int ldg)
{
    constexpr int G = 32 / LPN;
    const int lane = threadIdx.x & 31;
    const int wi = blockIdx.x * kGravWarps + (threadIdx.x >> 5);
    if (wi >= n_vert) return;
    const int i = order ? __ldg(order + wi) : wi;
    const int grp = lane / LPN, sub = lane % LPN, c4 = sub * 4;
    const bool chan = c4 < P;
    float gm[4] = {0.f, 0.f, 0.f, 0.f}, gx[4] = {0.f, 0.f, 0.f, 0.f};
    int am[4] = {-1, -1, -1, -1};
    if (chan) {
        const float4 a = *(const float4 *)(g_mean + (size_t)i * ldg + c4);
        const float4 b = *(const float4 *)(g_max + (size_t)i * ldg + c4);
        const int4 m = *(const int4 *)(argmax + (size_t)i * P + c4);
        const float kf = (float)K;
        gm[0] = __fdiv_rn(a.x, kf); gm[1] = __fdiv_rn(a.y, kf); gm[2] = __fdiv_rn(a.z, kf); gm[3] = __fdiv_rn(a.w, kf);
        gx[0] = b.x; gx[1] = b.y; gx[2] = b.z; gx[3] = b.w;
        am[0] = m.x; am[1] = m.y; am[2] = m.z; am[3] = m.w;
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
        const int cnt = min(32, K - k0);
        for (int kk = 0; kk < cnt; kk += G) {
            const int ks = kk + grp;
            const int n = __shfl_sync(FGC_FULL_MASK, n_l, ks & 31);
            const float w = __shfl_sync(FGC_FULL_MASK, w_l, ks & 31);
            const bool live = ks < cnt && n >= 0;
            float dot = 0.f;
            if (live && chan) {
                const float4 x = __ldg((const float4 *)(prop + (size_t)n * P + c4));
                float cf[4];
#pragma unroll
                for (int c = 0; c < 4; c++) cf[c] = gm[c] + (am[c] == k0 + ks ? gx[c] : 0.f);
                dot = x.x * cf[0] + x.y * cf[1] + x.z * cf[2] + x.w * cf[3];
                if (d_prop)
                    atomicAdd((float4 *)(d_prop + (size_t)n * P + c4),
                              make_float4(w * cf[0], w * cf[1], w * cf[2], w * cf[3]));
            }
#pragma unroll
            for (int off = LPN / 2; off > 0; off >>= 1) dot += __shfl_xor_sync(FGC_FULL_MASK, dot, off);
            if (sub == 0 && ks < cnt) d_distsq[(size_t)i * K + k0 + ks] = live ? -10.f * w * dot : 0.f;
        }
    }
}

// ---------------------------------------------------------------------------------------
// d_prop over the reverse neighbour graph: one warp per target row n gathers
//   d_prop[n,:] = sum over (i,k) with idx[i,k] == n of w[i,k] * coef[i,k,:]
// from its sorted segment, lane groups taking consecutive entries, combined by a fixed
// butterfly.  No float atomics: the result is the same on every run.
// ---------------------------------------------------------------------------------------

template <int LPN>
__global__ void __launch_bounds__(kGravWarps * 32)
k_gravnet_dprop_sorted_v4(const float *__restrict__ distsq, const int32_t *__restrict__ argmax,
                          const float *__restrict__ g_mean, const float *__restrict__ g_max,
                          int n_vert, int K, int P, const int *__restrict__ offsets,
                          const int *__restrict__ entries, float *__restrict__ d_prop, int ldg)
{
    constexpr int G = 32 / LPN;
    const int lane = threadIdx.x & 31;
    const int n = blockIdx.x * kGravWarps + (threadIdx.x >> 5);
    if (n >= n_vert) return;
    const int grp = lane / LPN, c4 = (lane % LPN) * 4;
    const bool chan = c4 < P;
    const int beg = offsets[n], end = offsets[n + 1];
    const float kf = (float)K;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int t0 = beg; t0 < end; t0 += G) {
        const int t = t0 + grp;
        if (t < end && chan) {
            const int src = __ldg(entries + t);
            const int i = src / K, k = src - i * K;
            const float w = expf(__fmul_rn(-10.f, __ldg(distsq + src)));
            const float4 a = __ldg((const float4 *)(g_mean + (size_t)i * ldg + c4));
            const float4 b = __ldg((const float4 *)(g_max + (size_t)i * ldg + c4));
            const int4 m = __ldg((const int4 *)(argmax + (size_t)i * P + c4));
            acc[0] += w * (__fdiv_rn(a.x, kf) + (m.x == k ? b.x : 0.f));
            acc[1] += w * (__fdiv_rn(a.y, kf) + (m.y == k ? b.y : 0.f));
            acc[2] += w * (__fdiv_rn(a.z, kf) + (m.z == k ? b.z : 0.f));
            acc[3] += w * (__fdiv_rn(a.w, kf) + (m.w == k ? b.w : 0.f));
        }
    }
#pragma unroll
    for (int off = LPN; off < 32; off <<= 1)
#pragma unroll
        for (int c = 0; c < 4; c++) acc[c] += __shfl_xor_sync(FGC_FULL_MASK, acc[c], off);
    if (grp == 0 && chan)
        *(float4 *)(d_prop + (size_t)n * P + c4) = make_float4(acc[0], acc[1], acc[2], acc[3]);
}

// any P: lanes over channels, entries one after the other
__global__ void __launch_bounds__(kGravWarps * 32)
k_gravnet_dprop_sorted(const float *__restrict__ distsq, const int32_t *__restrict__ argmax,
                       const float *__restrict__ g_mean, const float *__restrict__ g_max, int n_vert,
                       int K, int P, const int *__restrict__ offsets,
                       const int *__restrict__ entries, float *__restrict__ d_prop, int ldg)
{
    const int lane = threadIdx.x & 31;
    const int n = blockIdx.x * kGravWarps + (threadIdx.x >> 5);
    if (n >= n_vert) return;
    const int beg = offsets[n], end = offsets[n + 1];
    const float kf = (float)K;
    for (int p = lane; p < P; p += 32) {
        float acc = 0.f;
        for (int t = beg; t < end; t++) {
            const int src = __ldg(entries + t);
            const int i = src / K, k = src - i * K;
            const float w = expf(__fmul_rn(-10.f, __ldg(distsq + src)));
            acc += w * (__fdiv_rn(__ldg(g_mean + (size_t)i * ldg + p), kf) +
                        (__ldg(argmax + (size_t)i * P + p) == k ? __ldg(g_max + (size_t)i * ldg + p) : 0.f));
        }
        d_prop[(size_t)n * P + p] = acc;
    }
}

}  // namespace fgc

extern "C" int fgc_gravnet_aggregate_fwd_ld(const float *prop, const int64_t *idx, const float *distsq,
                                            int64_t n_vert, int32_t K, int32_t P, float *out_mean,
                                            float *out_max, int64_t ld_out, int32_t *out_argmax,
                                            const int32_t *order_or_null, fgc_stream_t stream)
{
    FGC_NVTX("fgc_gravnet_aggregate_fwd");
    using namespace fgc;
    if (n_vert < 0 || K < 1 || P < 1 || ld_out < P || ld_out > 0x7fffffff) return FGC_ERR_BAD_ARGUMENT;
    const int ldo = (int)ld_out;
    if (n_vert > 0x7fffffff) return FGC_ERR_TOO_LARGE;
    if (n_vert == 0) return FGC_OK;
    if (!prop || !idx || !distsq || !out_mean || !out_max) return FGC_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const int n = (int)n_vert;
    const int T = kGravWarps * 32;
    dim3 grid((unsigned)((n + kGravWarps - 1) / kGravWarps), 1);
    const bool vec = (P % 4 == 0) && (ldo % 4 == 0) && P <= 128 &&
                     (((uintptr_t)prop | (uintptr_t)out_mean | (uintptr_t)out_max | (uintptr_t)out_argmax) & 15) == 0;
    if (vec) {
        if (P <= 16) k_gravnet_fwd_v4<4><<<grid, T, 0, s>>>(prop, idx, distsq, n, K, P, out_mean, out_max, out_argmax, order_or_null, ldo);
        else if (P <= 32) k_gravnet_fwd_v4<8><<<grid, T, 0, s>>>(prop, idx, distsq, n, K, P, out_mean, out_max, out_argmax, order_or_null, ldo);
        else if (P <= 64) k_gravnet_fwd_v4<16><<<grid, T, 0, s>>>(prop, idx, distsq, n, K, P, out_mean, out_max, out_argmax, order_or_null, ldo);
        else k_gravnet_fwd_v4<32><<<grid, T, 0, s>>>(prop, idx, distsq, n, K, P, out_mean, out_max, out_argmax, order_or_null, ldo);
        FGC_CHECK_LAUNCH();
        return FGC_OK;
    }
    if (P <= 32) k_gravnet_fwd<1><<<grid, T, 0, s>>>(prop, idx, distsq, n, K, P, out_mean, out_max, out_argmax, order_or_null, ldo);
    else if (P <= 64) k_gravnet_fwd<2><<<grid, T, 0, s>>>(prop, idx, distsq, n, K, P, out_mean, out_max, out_argmax, order_or_null, ldo);
    else {
        grid.y = (unsigned)((P + 127) / 128);
        k_gravnet_fwd<4><<<grid, T, 0, s>>>(prop, idx, distsq, n, K, P, out_mean, out_max, out_argmax, order_or_null, ldo);
    }
    FGC_CHECK_LAUNCH();
    return FGC_OK;
}

extern "C" int fgc_gravnet_aggregate_fwd(const float *prop, const int64_t *idx, const float *distsq,
                                         int64_t n_vert, int32_t K, int32_t P, float *out_mean,
                                         float *out_max, int32_t *out_argmax,
                                         const int32_t *order_or_null, fgc_stream_t stream)
{
    return fgc_gravnet_aggregate_fwd_ld(prop, idx, distsq, n_vert, K, P, out_mean, out_max, P, out_argmax,
                                        order_or_null, stream);
}

extern "C" int fgc_gravnet_aggregate_bwd_ld(const float *prop, const int64_t *idx, const float *distsq,
                                            const int32_t *argmax, const float *grad_mean,
                                            const float *grad_max, int64_t ld_grad, int64_t n_vert,
                                            int32_t K, int32_t P, float *out_d_prop, float *out_d_distsq,
                                            const int32_t *order_or_null, fgc_stream_t stream)
{
    FGC_NVTX("fgc_gravnet_aggregate_bwd");
    using namespace fgc;
    if (n_vert < 0 || K < 1 || P < 1 || ld_grad < P || ld_grad > 0x7fffffff) return FGC_ERR_BAD_ARGUMENT;
    const int ldg = (int)ld_grad;
    if (n_vert > 0x7fffffff) return FGC_ERR_TOO_LARGE;
    if (n_vert == 0) return FGC_OK;
    if (!prop || !idx || !distsq || !argmax || !grad_mean || !grad_max || !out_d_prop || !out_d_distsq)
        return FGC_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const int n = (int)n_vert;
    const int T = kGravWarps * 32;
    FGC_RETURN_IF_CUDA(cudaMemsetAsync(out_d_prop, 0, sizeof(float) * (size_t)n_vert * P, s));
    dim3 grid((unsigned)((n + kGravWarps - 1) / kGravWarps), 1);
    const bool vec = (P % 4 == 0) && (ldg % 4 == 0) && P <= 128 &&
                     (((uintptr_t)prop | (uintptr_t)grad_mean | (uintptr_t)grad_max | (uintptr_t)argmax |
                       (uintptr_t)out_d_prop) & 15) == 0;
    if (vec) {
        if (P <= 16) k_gravnet_bwd_v4<4><<<grid, T, 0, s>>>(prop, idx, distsq, argmax, grad_mean, grad_max, n, K, P, out_d_prop, out_d_distsq, order_or_null, ldg);
        else if (P <= 32) k_gravnet_bwd_v4<8><<<grid, T, 0, s>>>(prop, idx, distsq, argmax, grad_mean, grad_max, n, K, P, out_d_prop, out_d_distsq, order_or_null, ldg);
        else if (P <= 64) k_gravnet_bwd_v4<16><<<grid, T, 0, s>>>(prop, idx, distsq, argmax, grad_mean, grad_max, n, K, P, out_d_prop, out_d_distsq, order_or_null, ldg);
        else k_gravnet_bwd_v4<32><<<grid, T, 0, s>>>(prop, idx, distsq, argmax, grad_mean, grad_max, n, K, P, out_d_prop, out_d_distsq, order_or_null, ldg);
        FGC_CHECK_LAUNCH();
        return FGC_OK;
    }
    if (P <= 32)
        k_gravnet_bwd<1><<<grid, T, 0, s>>>(prop, idx, distsq, argmax, grad_mean, grad_max, n, K, P, out_d_prop, out_d_distsq, 0, order_or_null, ldg);
    else if (P <= 64)
        k_gravnet_bwd<2><<<grid, T, 0, s>>>(prop, idx, distsq, argmax, grad_mean, grad_max, n, K, P, out_d_prop, out_d_distsq, 0, order_or_null, ldg);
    else {
        grid.y = (unsigned)((P + 127) / 128);
        const int acc = grid.y > 1;
        if (acc) FGC_RETURN_IF_CUDA(cudaMemsetAsync(out_d_distsq, 0, sizeof(float) * (size_t)n_vert * K, s));
        k_gravnet_bwd<4><<<grid, T, 0, s>>>(prop, idx, distsq, argmax, grad_mean, grad_max, n, K, P, out_d_prop, out_d_distsq, acc, order_or_null, ldg);
    }
    FGC_CHECK_LAUNCH();
    return FGC_OK;
}

extern "C" int fgc_gravnet_aggregate_bwd(const float *prop, const int64_t *idx, const float *distsq,
                                         const int32_t *argmax, const float *grad_mean,
                                         const float *grad_max, int64_t n_vert, int32_t K, int32_t P,
                                         float *out_d_prop, float *out_d_distsq,
                                         const int32_t *order_or_null, fgc_stream_t stream)
{
    return fgc_gravnet_aggregate_bwd_ld(prop, idx, distsq, argmax, grad_mean, grad_max, P, n_vert, K, P,
                                        out_d_prop, out_d_distsq, order_or_null, stream);
}

extern "C" int fgc_gravnet_aggregate_bwd_sorted_ld(const float *prop, const int64_t *idx,
                                                   const float *distsq, const int32_t *argmax,
                                                   const float *grad_mean, const float *grad_max,
                                                   int64_t ld_grad, int64_t n_vert, int32_t K, int32_t P,
                                                   const void *rgraph, size_t rgraph_bytes,
                                                   float *out_d_prop, float *out_d_distsq,
                                                   const int32_t *order_or_null, fgc_stream_t stream)
{
    FGC_NVTX("fgc_gravnet_aggregate_bwd_sorted");
    using namespace fgc;
    if (n_vert < 0 || K < 1 || P < 1 || P > 128 || ld_grad < P || ld_grad > 0x7fffffff) return FGC_ERR_BAD_ARGUMENT;
    const int ldg = (int)ld_grad;
    if (n_vert * (int64_t)K > 0x7fffffff) return FGC_ERR_TOO_LARGE;
    const ReverseGraphLayout RL = reverse_graph_layout(n_vert, K);
    if (!rgraph || rgraph_bytes < RL.total || ((uintptr_t)rgraph & 255)) return FGC_ERR_WORKSPACE;
    if (n_vert == 0) return FGC_OK;
    if (!prop || !idx || !distsq || !argmax || !grad_mean || !grad_max || !out_d_prop || !out_d_distsq)
        return FGC_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const int n = (int)n_vert;
    const int T = kGravWarps * 32;
    dim3 grid((unsigned)((n + kGravWarps - 1) / kGravWarps), 1);
    const int *offsets = (const int *)((const char *)rgraph + RL.offsets);
    const int *entries = (const int *)((const char *)rgraph + RL.entries);
    const bool vec = (P % 4 == 0) && (ldg % 4 == 0) &&
                     (((uintptr_t)prop | (uintptr_t)grad_mean | (uintptr_t)grad_max | (uintptr_t)argmax |
                       (uintptr_t)out_d_prop) & 15) == 0;
    // d_distsq: the per-row kernel without its d_prop reductions
    if (vec) {
        if (P <= 16) k_gravnet_bwd_v4<4><<<grid, T, 0, s>>>(prop, idx, distsq, argmax, grad_mean, grad_max, n, K, P, nullptr, out_d_distsq, order_or_null, ldg);
        else if (P <= 32) k_gravnet_bwd_v4<8><<<grid, T, 0, s>>>(prop, idx, distsq, argmax, grad_mean, grad_max, n, K, P, nullptr, out_d_distsq, order_or_null, ldg);
        else if (P <= 64) k_gravnet_bwd_v4<16><<<grid, T, 0, s>>>(prop, idx, distsq, argmax, grad_mean, grad_max, n, K, P, nullptr, out_d_distsq, order_or_null, ldg);
        else k_gravnet_bwd_v4<32><<<grid, T, 0, s>>>(prop, idx, distsq, argmax, grad_mean, grad_max, n, K, P, nullptr, out_d_distsq, order_or_null, ldg);
    } else if (P <= 32) k_gravnet_bwd<1><<<grid, T, 0, s>>>(prop, idx, distsq, argmax, grad_mean, grad_max, n, K, P, nullptr, out_d_distsq, 0, order_or_null, ldg);
    else if (P <= 64) k_gravnet_bwd<2><<<grid, T, 0, s>>>(prop, idx, distsq, argmax, grad_mean, grad_max, n, K, P, nullptr, out_d_distsq, 0, order_or_null, ldg);
    else k_gravnet_bwd<4><<<grid, T, 0, s>>>(prop, idx, distsq, argmax, grad_mean, grad_max, n, K, P, nullptr, out_d_distsq, 0, order_or_null, ldg);
    FGC_CHECK_LAUNCH();
    // d_prop: gathers over the sorted reverse segments
    if (vec) {
        if (P <= 16) k_gravnet_dprop_sorted_v4<4><<<grid, T, 0, s>>>(distsq, argmax, grad_mean, grad_max, n, K, P, offsets, entries, out_d_prop, ldg);
        else if (P <= 32) k_gravnet_dprop_sorted_v4<8><<<grid, T, 0, s>>>(distsq, argmax, grad_mean, grad_max, n, K, P, offsets, entries, out_d_prop, ldg);
        else if (P <= 64) k_gravnet_dprop_sorted_v4<16><<<grid, T, 0, s>>>(distsq, argmax, grad_mean, grad_max, n, K, P, offsets, entries, out_d_prop, ldg);
        else k_gravnet_dprop_sorted_v4<32><<<grid, T, 0, s>>>(distsq, argmax, grad_mean, grad_max, n, K, P, offsets, entries, out_d_prop, ldg);
    } else {
        k_gravnet_dprop_sorted<<<grid, T, 0, s>>>(distsq, argmax, grad_mean, grad_max, n, K, P, offsets, entries, out_d_prop, ldg);
    }
    FGC_CHECK_LAUNCH();
    return FGC_OK;
}

extern "C" int fgc_gravnet_aggregate_bwd_sorted(const float *prop, const int64_t *idx,
                                                const float *distsq, const int32_t *argmax,
                                                const float *grad_mean, const float *grad_max,
                                                int64_t n_vert, int32_t K, int32_t P,
                                                const void *rgraph, size_t rgraph_bytes,
                                                float *out_d_prop, float *out_d_distsq,
                                                const int32_t *order_or_null, fgc_stream_t stream)
{
    return fgc_gravnet_aggregate_bwd_sorted_ld(prop, idx, distsq, argmax, grad_mean, grad_max, P, n_vert, K, P,
                                               rgraph, rgraph_bytes, out_d_prop, out_d_distsq, order_or_null,
                                               stream);
}
