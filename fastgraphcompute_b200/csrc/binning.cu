// bin_by_coordinates for sm_100a: fused finite/min/max pass, device-side
// derivation of the binning parameters, per-point bin assignment with a
// warp-aggregated histogram.
//
// Semantics follow the reference's CPU implementation bit for bit:
//   host derivation  extensions/bin_by_coordinates.cpp:51-120
//   per-point kernel extensions/bin_by_coordinates_cpu.cpp:7-99
// All float steps use explicit round-to-nearest intrinsics (no contraction, no
// fast division) so that bin indices agree with the x86-64 build.
#include "fgc_common.cuh"

namespace fgc {

constexpr int kReduceThreads = 256;

// scratch layout inside fgc_bin_params: [0..7] ~ordered(min), [8..15] ordered(max),
// [16] non-finite flag.  All start at zero, so one memset initialises them and
// both extremes are maintained with atomicMax.
__global__ void __launch_bounds__(kReduceThreads)
k_bin_minmax(const float *__restrict__ coords, int64_t n_vert, int n_coords, fgc_bin_params *prm)
{
    __shared__ uint32_t s_min[FGC_MAX_BIN_DIMS], s_max[FGC_MAX_BIN_DIMS], s_bad;
    if (threadIdx.x < FGC_MAX_BIN_DIMS) { s_min[threadIdx.x] = 0; s_max[threadIdx.x] = 0; }
    if (threadIdx.x == 0) s_bad = 0;
    __syncthreads();
    // Each thread walks whole rows so that a thread's column index is fixed per element.
    const int64_t total = n_vert * (int64_t)n_coords;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    uint32_t bad = 0;
    // thread t handles flat elements t, t+stride, ...; stride is a multiple of n_coords
    // only by accident, so the column is recomputed per element.
    uint32_t lmin[FGC_MAX_BIN_DIMS], lmax[FGC_MAX_BIN_DIMS];
#pragma unroll
    for (int c = 0; c < FGC_MAX_BIN_DIMS; c++) { lmin[c] = 0; lmax[c] = 0; }
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
        const float v = __ldg(coords + e);
        const int c = (int)(e % n_coords);
        if (!is_finite_bits(v)) bad = 1;
        const uint32_t k = float_to_ordered(v);
#pragma unroll
        for (int cc = 0; cc < FGC_MAX_BIN_DIMS; cc++)
            if (cc == c) {
                lmin[cc] = max(lmin[cc], ~k);
                lmax[cc] = max(lmax[cc], k);
            }
    }
#pragma unroll
    for (int c = 0; c < FGC_MAX_BIN_DIMS; c++) {
        uint32_t a = __reduce_max_sync(FGC_FULL_MASK, lmin[c]);
        uint32_t b = __reduce_max_sync(FGC_FULL_MASK, lmax[c]);
        if ((threadIdx.x & 31) == 0 && c < n_coords) {
            atomicMax(&s_min[c], a);
            atomicMax(&s_max[c], b);
        }
    }
    if (__any_sync(FGC_FULL_MASK, bad) && (threadIdx.x & 31) == 0) atomicOr(&s_bad, 1u);
    __syncthreads();
    if (threadIdx.x < n_coords) {
        atomicMax(&prm->scratch[threadIdx.x], s_min[threadIdx.x]);
        atomicMax(&prm->scratch[FGC_MAX_BIN_DIMS + threadIdx.x], s_max[threadIdx.x]);
    }
    if (threadIdx.x == 0 && s_bad) atomicOr(&prm->scratch[2 * FGC_MAX_BIN_DIMS], 1u);
}

// One thread: the D-element derivation of shift, dmax, n_bins and bin_width.
__global__ void k_bin_derive(fgc_bin_params *prm, int64_t n_vert, int n_coords, int pre_normalized,
                             const float *__restrict__ bin_width_in,
                             const int64_t *__restrict__ n_bins_in, int n_bins_len)
{
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    int status = 0;
    if (prm->scratch[2 * FGC_MAX_BIN_DIMS]) status |= FGC_STATUS_NONFINITE;
    float bw_max = -INFINITY;
    const bool have_bw = bin_width_in != nullptr;
    const bool have_nb = n_bins_in != nullptr;
    for (int c = 0; c < FGC_MAX_BIN_DIMS; c++) { prm->shift[c] = 0.f; prm->n_bins[c] = 1; }
    for (int c = 0; c < n_coords; c++) {
        float lo = n_vert > 0 ? ordered_to_float(~prm->scratch[c]) : 0.f;
        float hi = n_vert > 0 ? ordered_to_float(prm->scratch[FGC_MAX_BIN_DIMS + c]) : 0.f;
        float shift = 0.f;
        if (!pre_normalized) {
            shift = lo;
            hi = __fsub_rn(hi, lo);  // max of the shifted column (x - lo is monotone in x)
            lo = __fsub_rn(lo, lo);
        }
        prm->shift[c] = shift;
        float dmax = hi;
        if (lo == hi) dmax = __fadd_rn(dmax, 1.0f);
        dmax = __fadd_rn(dmax, (float)1e-3);
        if (!is_finite_bits(dmax)) dmax = 1.0f;
        if (!(dmax > 0.f)) status |= FGC_STATUS_BAD_DMAX;
        if (have_bw) {
            if (have_nb)
                prm->n_bins[c] = n_bins_in[n_bins_len == 1 ? 0 : c];
            else
                prm->n_bins[c] = (int64_t)__fdiv_rn(dmax, bin_width_in[0]) + 1;
        } else {
            const int64_t nb = n_bins_in[n_bins_len == 1 ? 0 : c];
            prm->n_bins[c] = nb;
            const float bw = __fdiv_rn(dmax, (float)nb);
            if (bw > bw_max) bw_max = bw;
        }
    }
    const float bw = have_bw ? bin_width_in[0] : bw_max;
    prm->bin_width = bw;
    for (int c = 0; c < n_coords; c++)
        if (!(prm->n_bins[c] > 0)) status |= FGC_STATUS_BAD_NBINS;
    if (!(bw > 0.f)) status |= FGC_STATUS_BAD_BINWIDTH;
    prm->n_coords = n_coords;
    prm->status = status;
}

// One thread per point.
__global__ void __launch_bounds__(256)
k_bin_assign(const float *__restrict__ coords, int64_t n_vert, int n_coords,
             const int64_t *__restrict__ row_splits, int n_rs,
             const fgc_bin_params *__restrict__ prm, int calc_n_per_bin, int64_t n_total_bins,
             int64_t *__restrict__ out_bin_idx, int64_t *__restrict__ out_flat,
             unsigned long long *__restrict__ out_n_per_bin)
{
    const int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const bool live = v < n_vert;
    int64_t flat = -1;
    if (live) {
        const float bw = prm->bin_width;
        int64_t stride = 1, f = 0;
        int64_t cidx[FGC_MAX_BIN_DIMS];
#pragma unroll
        for (int c = FGC_MAX_BIN_DIMS - 1; c >= 0; c--) {
            if (c < n_coords) {
                const float x = __fsub_rn(__ldg(coords + v * n_coords + c), prm->shift[c]);
                const float q = __fdiv_rn(x, bw);
                int64_t b = (int64_t)floorf(__fadd_rn(q, 1e-3f));
                const int64_t nb = prm->n_bins[c];
                if (b < 0) b = 0;
                else if (b >= nb) b = nb - 1;
                cidx[c] = b;
                f += b * stride;
                stride *= nb;
            }
        }
        const int rs = row_split_of(row_splits, n_rs, v);
        f += (int64_t)rs * stride;
        if (f < n_total_bins) {
            int64_t *row = out_bin_idx + v * (n_coords + 1);
            row[0] = rs;
#pragma unroll
            for (int c = 0; c < FGC_MAX_BIN_DIMS; c++)
                if (c < n_coords) row[c + 1] = cidx[c];
            out_flat[v] = f;
            flat = f;
        }
    }
    if (calc_n_per_bin) {
        // warp-aggregated histogram: one atomic per distinct bin per warp
        const bool counts = live && flat >= 0;
        const unsigned active = __ballot_sync(FGC_FULL_MASK, counts);
        if (counts) {
            const unsigned peers = __match_any_sync(active, flat);
            const int leader = __ffs(peers) - 1;
            if ((int)(threadIdx.x & 31) == leader)
                atomicAdd(out_n_per_bin + flat, (unsigned long long)__popc(peers));
        }
    }
}

}  // namespace fgc

extern "C" int fgc_bin_prepare(const float *coords, int64_t n_vert, int32_t n_coords,
                               int32_t pre_normalized, const float *bin_width_or_null,
                               const int64_t *n_bins_or_null, int32_t n_bins_len,
                               fgc_bin_params *out_params, fgc_stream_t stream)
{
    FGC_NVTX("fgc_bin_prepare");
    if (!out_params || n_vert < 0 || n_coords < 1 || n_coords > FGC_MAX_BIN_DIMS)
        return FGC_ERR_BAD_ARGUMENT;
    if (n_vert > 0 && !coords) return FGC_ERR_BAD_ARGUMENT;
    if (!bin_width_or_null && !n_bins_or_null) return FGC_ERR_BAD_ARGUMENT;
    if (n_bins_or_null && n_bins_len != 1 && n_bins_len != n_coords) return FGC_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    FGC_RETURN_IF_CUDA(cudaMemsetAsync(out_params, 0, sizeof(fgc_bin_params), s));
    if (n_vert > 0) {
        const int64_t total = n_vert * n_coords;
        int blocks = (int)fgc::ceil_div64(total, (int64_t)fgc::kReduceThreads * 8);
        if (blocks > fgc::sm_count() * 8) blocks = fgc::sm_count() * 8;
        if (blocks < 1) blocks = 1;
        fgc::k_bin_minmax<<<blocks, fgc::kReduceThreads, 0, s>>>(coords, n_vert, n_coords, out_params);
        FGC_CHECK_LAUNCH();
    }
    fgc::k_bin_derive<<<1, 32, 0, s>>>(out_params, n_vert, n_coords, pre_normalized,
                                       bin_width_or_null, n_bins_or_null, n_bins_len);
    FGC_CHECK_LAUNCH();
    return FGC_OK;
}

extern "C" int fgc_bin_assign(const float *coords, int64_t n_vert, int32_t n_coords,
                              const int64_t *row_splits, int64_t n_rs,
                              const fgc_bin_params *params, int32_t calc_n_per_bin,
                              int64_t n_total_bins, int64_t *out_bin_idx, int64_t *out_flat,
                              int64_t *out_n_per_bin, fgc_stream_t stream)
{
    FGC_NVTX("fgc_bin_assign");
    if (!params || n_vert < 0 || n_coords < 1 || n_coords > FGC_MAX_BIN_DIMS || n_rs < 1 ||
        n_rs > 0x7fffffff || !row_splits)
        return FGC_ERR_BAD_ARGUMENT;
    if (n_vert == 0) return FGC_OK;
    if (!coords || !out_bin_idx || !out_flat || (calc_n_per_bin && !out_n_per_bin))
        return FGC_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    const int64_t blocks = fgc::ceil_div64(n_vert, 256);
    if (blocks > 0x7fffffff) return FGC_ERR_TOO_LARGE;
    fgc::k_bin_assign<<<(unsigned)blocks, 256, 0, s>>>(
        coords, n_vert, n_coords, row_splits, (int)n_rs, params, calc_n_per_bin, n_total_bins,
        out_bin_idx, out_flat, (unsigned long long *)out_n_per_bin);
    FGC_CHECK_LAUNCH();
    return FGC_OK;
}
