// The two input projections of a GravNet layer as one pass over x (sm_100a).
//
// GravNetOp.forward starts with two dense layers on the same input (fastgraphcompute/gnn_ops.py:79-82):
//   space     = x @ Ws^T + bs      [N, S]   learned coordinates for the neighbour search
//   propagate = x @ Wp^T + bp      [N, P]   features exchanged between neighbours
// With S + P a few dozen outputs of 64 or so inputs these are tall, skinny products that are
// bound by the traffic of x, and the backward pass -- two weight gradients that reduce over all
// N rows, two input gradients, two bias gradients, each a library GEMM or reduction with its own
// pass over x or over the output gradients -- costs several times the forward.  Here:
//   forward : one kernel, x read once, both outputs written;
//   backward: one kernel, x and the two output gradients read once; it writes
//             dX = dS @ Ws + dP @ Wp and accumulates dW (both weights), db (both biases).
// fp32 throughout with fused multiply-adds (these are dense layers: the bit-exact arithmetic rules
// of the distance code do not apply here; results agree with a library GEMM to rounding).
//
// Layout.  O = S + P outputs, padded to OP = 16 * KO; C = 16 * KC inputs.  A CTA of 256 threads works
// on tiles of 128 rows.  The x tile (and, backward, the tile of output gradients) sits in shared
// memory TRANSPOSED, [channel][row] with 132 floats per channel, so that a thread reads the eight
// (or four) consecutive rows it owns as 16-byte words; the weights sit beside them for the whole
// kernel.  Every thread owns a small register tile (8 rows x KO outputs forward; 8 rows x KC inputs
// for dX; KO outputs x KC inputs for dW), so that one 16-byte shared-memory read feeds 8 to 16
// multiply-adds.
#include "fgc_common.cuh"

namespace fgc {

constexpr int kProjRows = 128;               // rows per tile
constexpr int kProjRowsP = kProjRows + 4;    // padded row count of a transposed tile
constexpr int kProjThreads = 256;

struct ProjShape {
    int C;       // inputs (a multiple of 16)
    int S, P;    // outputs of the two layers
    int O;       // S + P
    int OP;      // O rounded up to a multiple of 16
};

__host__ __device__ inline ProjShape proj_shape(int C, int S, int P)
{
    ProjShape s;
    s.C = C; s.S = S; s.P = P; s.O = S + P;
    s.OP = 16 * ((s.O + 15) / 16);
    return s;
}

inline size_t proj_smem_bytes(const ProjShape &s, bool backward)
{
    size_t words = (size_t)s.OP * s.C + s.OP + (size_t)s.C * kProjRowsP;
    if (backward) words += (size_t)s.OP * kProjRowsP;
    return words * sizeof(float);
}

// x tile, transposed: sXt[c][r] = x[row0 + r][c] (zero beyond the last row); coalesced global reads
// copy (optional): the rows are also written to copy[row * ld_copy + c], the first `width` columns of
// a wider row-major matrix
__device__ __forceinline__ void proj_load_tile_t(float *sT, const float *__restrict__ src, long long row0,
                                                 long long n_rows, int width, float *__restrict__ copy = nullptr,
                                                 long long ld_copy = 0)
{
    if ((width & (width - 1)) == 0 && width >= 4 && width <= 128 && ((uintptr_t)src & 15) == 0 &&
        (!copy || ((((uintptr_t)copy) & 15) == 0 && (ld_copy & 3) == 0))) {
        // rows of 4, 8, ..., 128 floats: one 16-byte load per thread and pass, no divisions
        const int vpr = width >> 2;                       // 16-byte words per row (1..32)
        const int sh = 31 - __clz(vpr);
        const int rows_per_pass = kProjThreads >> sh;
        const int v = threadIdx.x & (vpr - 1), rr = threadIdx.x >> sh;
        for (int r = rr; r < kProjRows; r += rows_per_pass) {
            const long long row = row0 + r;
            float4 val = make_float4(0.f, 0.f, 0.f, 0.f);
            if (row < n_rows) {
                val = __ldg((const float4 *)(src + (size_t)row * width) + v);
                if (copy) *((float4 *)(copy + (size_t)row * ld_copy) + v) = val;
            }
            float *dst = sT + (4 * v) * kProjRowsP + r;
            dst[0] = val.x;
            dst[kProjRowsP] = val.y;
            dst[2 * kProjRowsP] = val.z;
            dst[3 * kProjRowsP] = val.w;
        }
        return;
    }
    const int total = kProjRows * width;
    for (int i = threadIdx.x; i < total; i += kProjThreads) {
        const int r = i / width, c = i - r * width;
        const long long row = row0 + r;
        const float val = row < n_rows ? __ldg(src + (size_t)row * width + c) : 0.f;
        sT[c * kProjRowsP + r] = val;
        if (copy && row < n_rows) copy[(size_t)row * ld_copy + c] = val;
    }
}

// KO = OP / 16 outputs per thread (1..4)
template <int KO>
__global__ void __launch_bounds__(kProjThreads)
k_project_fwd(const float *__restrict__ x, long long n_rows, ProjShape h, const float *__restrict__ Ws,
              const float *__restrict__ bs, const float *__restrict__ Wp, const float *__restrict__ bp,
              float *__restrict__ out_space, float *__restrict__ out_prop, float *__restrict__ x_copy,
              long long ld_copy)
{
    extern __shared__ __align__(16) float proj_smem[];
    float *sW = proj_smem;                       // [C][OP]: transposed weights, a thread's outputs contiguous
    float *sB = sW + h.OP * h.C;                 // [OP]
    float *sX = sB + h.OP;                       // [C][132]
    for (int i = threadIdx.x; i < h.OP * h.C; i += kProjThreads) {
        const int c = i / h.OP, o = i - c * h.OP;
        float v = 0.f;
        if (o < h.S) v = __ldg(Ws + (size_t)o * h.C + c);
        else if (o < h.O) v = __ldg(Wp + (size_t)(o - h.S) * h.C + c);
        sW[i] = v;
    }
    for (int o = threadIdx.x; o < h.OP; o += kProjThreads)
        sB[o] = o < h.S ? (bs ? __ldg(bs + o) : 0.f) : (o < h.O ? (bp ? __ldg(bp + o - h.S) : 0.f) : 0.f);
    const int og = threadIdx.x & 15, rg = threadIdx.x >> 4;     // outputs og*KO.., rows rg*8..
    const long long n_tiles = (n_rows + kProjRows - 1) / kProjRows;
    for (long long tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        __syncthreads();
        proj_load_tile_t(sX, x, tile * kProjRows, n_rows, h.C, x_copy, ld_copy);
        __syncthreads();
        float acc[8][KO];
#pragma unroll
        for (int i = 0; i < 8; i++)
#pragma unroll
            for (int k = 0; k < KO; k++) acc[i][k] = sB[og * KO + k];
        for (int c = 0; c < h.C; c++) {
            const float4 xa = *(const float4 *)(sX + c * kProjRowsP + rg * 8);
            const float4 xb = *(const float4 *)(sX + c * kProjRowsP + rg * 8 + 4);
            const float xv[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
            float w[KO];
#pragma unroll
            for (int k = 0; k < KO; k++) w[k] = sW[c * h.OP + og * KO + k];
#pragma unroll
            for (int i = 0; i < 8; i++)
#pragma unroll
                for (int k = 0; k < KO; k++) acc[i][k] = fmaf(xv[i], w[k], acc[i][k]);
        }
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const long long row = tile * kProjRows + rg * 8 + i;
            if (row < n_rows) {
#pragma unroll
                for (int k = 0; k < KO; k++) {
                    const int o = og * KO + k;
                    if (o < h.S) out_space[(size_t)row * h.S + o] = acc[i][k];
                    else if (o < h.O) out_prop[(size_t)row * h.P + (o - h.S)] = acc[i][k];
                }
            }
        }
    }
}

// Backward: dX, dW (both weights) and db (both biases) from one pass over x and the output
// gradients.  dW / db are accumulated in registers over all tiles of the CTA and then added to the
// global gradients with one atomic per element and CTA.
// KO = OP / 16, KC = C / 16.
template <int KO, int KC>
__global__ void __launch_bounds__(kProjThreads, (KO * KC <= 12 ? 2 : 1))
k_project_bwd(const float *__restrict__ x, long long n_rows, ProjShape h, const float *__restrict__ Ws,
              const float *__restrict__ Wp, const float *__restrict__ d_space, const float *__restrict__ d_prop,
              float *__restrict__ dX, float *__restrict__ dWs, float *__restrict__ dbs,
              float *__restrict__ dWp, float *__restrict__ dbp, const float *__restrict__ dx_add,
              long long ld_add)
{
    extern __shared__ __align__(16) float proj_smem[];
    float *sW = proj_smem;                       // [OP][C] (row o: the C input weights of output o)
    float *sX = sW + h.OP * h.C;                 // [C][132]
    float *sY = sX + h.C * kProjRowsP;           // [OP][132]: output gradients of the tile, transposed
    const int t = threadIdx.x;
    for (int i = t; i < h.OP * h.C; i += kProjThreads) {
        const int o = i / h.C, c = i - o * h.C;
        float v = 0.f;
        if (o < h.S) v = __ldg(Ws + (size_t)o * h.C + c);
        else if (o < h.O) v = __ldg(Wp + (size_t)(o - h.S) * h.C + c);
        sW[i] = v;
    }
    const int lo = t & 15, hi = t >> 4;
    // dW tile of a thread.  C = 64 (KC = 4): outputs og + 8k (k < 2 KO), inputs cg + 8j (j < 8), over
    // the quarter t >> 6 of a tile's rows -- twice the multiply-adds per shared-memory read of the
    // general shape, and strided ownership keeps the 16-byte reads of a warp in different banks.
    // Otherwise: outputs lo*KO.., inputs hi*KC.., all rows.
    constexpr bool W64 = KC == 4;
    constexpr int WO = W64 ? 2 * KO : KO, WC = W64 ? 8 : KC;
    const int og = t & 7, cg = (t >> 3) & 7, rq = t >> 6;
    float accw[WO][WC];
#pragma unroll
    for (int k = 0; k < WO; k++)
#pragma unroll
        for (int j = 0; j < WC; j++) accw[k][j] = 0.f;
    float accb = 0.f;                            // threads t < O: bias gradient of output t
    const long long n_tiles = (n_rows + kProjRows - 1) / kProjRows;
    for (long long tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        __syncthreads();
        const long long row0 = tile * kProjRows;
        proj_load_tile_t(sX, x, row0, n_rows, h.C);
        // output gradients, transposed: channels 0..S-1 from d_space, S..O-1 from d_prop (a missing
        // gradient and the padding channels O..OP-1 are zero)
        if (d_space) proj_load_tile_t(sY, d_space, row0, n_rows, h.S);
        if (d_prop) proj_load_tile_t(sY + h.S * kProjRowsP, d_prop, row0, n_rows, h.P);
        if (!d_space || !d_prop || tile == (long long)blockIdx.x) {
            const int z0 = d_space ? (d_prop ? h.O : h.S) : 0;
            const int z1 = d_space ? h.OP : (d_prop ? h.S : h.OP);
            for (int i = t; i < (z1 - z0) * kProjRowsP; i += kProjThreads) sY[z0 * kProjRowsP + i] = 0.f;
            if (!d_space && d_prop)
                for (int i = t; i < (h.OP - h.O) * kProjRowsP; i += kProjThreads) sY[h.O * kProjRowsP + i] = 0.f;
        }
        __syncthreads();
        // ---- dX[row, c] = sum_o dY[row, o] * W[o, c]: inputs lo*KC.., rows hi*8..
        if (dX) {
            float a[8][KC];
#pragma unroll
            for (int i = 0; i < 8; i++)
#pragma unroll
                for (int j = 0; j < KC; j++) a[i][j] = 0.f;
            for (int o = 0; o < h.O; o++) {
                const float4 ya = *(const float4 *)(sY + o * kProjRowsP + hi * 8);
                const float4 yb = *(const float4 *)(sY + o * kProjRowsP + hi * 8 + 4);
                const float yv[8] = {ya.x, ya.y, ya.z, ya.w, yb.x, yb.y, yb.z, yb.w};
                float w[KC];
                if constexpr (KC % 4 == 0) {
#pragma unroll
                    for (int j = 0; j < KC; j += 4) {
                        const float4 w4 = *(const float4 *)(sW + o * h.C + lo * KC + j);
                        w[j] = w4.x; w[j + 1] = w4.y; w[j + 2] = w4.z; w[j + 3] = w4.w;
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < KC; j++) w[j] = sW[o * h.C + lo * KC + j];
                }
#pragma unroll
                for (int i = 0; i < 8; i++)
#pragma unroll
                    for (int j = 0; j < KC; j++) a[i][j] = fmaf(yv[i], w[j], a[i][j]);
            }
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const long long row = row0 + hi * 8 + i;
                if (row < n_rows) {
                    // dx_add: a second gradient of x (the x columns of the gradient of [x | mean | max])
                    // joins here instead of in a pass of its own
                    if (dx_add) {
                        const float *ad = dx_add + (size_t)row * ld_add + lo * KC;
#pragma unroll
                        for (int j = 0; j < KC; j++) a[i][j] += __ldg(ad + j);
                    }
                    if constexpr (KC % 4 == 0) {
#pragma unroll
                        for (int j = 0; j < KC; j += 4)
                            *(float4 *)(dX + (size_t)row * h.C + lo * KC + j) =
                                make_float4(a[i][j], a[i][j + 1], a[i][j + 2], a[i][j + 3]);
                    } else {
#pragma unroll
                        for (int j = 0; j < KC; j++) dX[(size_t)row * h.C + lo * KC + j] = a[i][j];
                    }
                }
            }
        }
        // ---- dW[o, c] += sum_rows dY[row, o] * x[row, c]: four rows at a time
        for (int r4 = W64 ? rq * 32 : 0; r4 < (W64 ? rq * 32 + 32 : kProjRows); r4 += 4) {
            float4 y4[WO], x4[WC];
#pragma unroll
            for (int k = 0; k < WO; k++)
                y4[k] = *(const float4 *)(sY + (W64 ? og + 8 * k : lo * KO + k) * kProjRowsP + r4);
#pragma unroll
            for (int j = 0; j < WC; j++)
                x4[j] = *(const float4 *)(sX + (W64 ? cg + 8 * j : hi * KC + j) * kProjRowsP + r4);
#pragma unroll
            for (int k = 0; k < WO; k++)
#pragma unroll
                for (int j = 0; j < WC; j++) {
                    float v = accw[k][j];
                    v = fmaf(y4[k].x, x4[j].x, v);
                    v = fmaf(y4[k].y, x4[j].y, v);
                    v = fmaf(y4[k].z, x4[j].z, v);
                    v = fmaf(y4[k].w, x4[j].w, v);
                    accw[k][j] = v;
                }
        }
        if (t < h.O) {
            float sacc = 0.f;
            for (int r = 0; r < kProjRows; r += 4) {
                const float4 y = *(const float4 *)(sY + t * kProjRowsP + r);
                sacc += (y.x + y.y) + (y.z + y.w);
            }
            accb += sacc;
        }
    }
    // ---- the CTA's share goes to the global gradients
#pragma unroll
    for (int k = 0; k < WO; k++) {
        const int o = W64 ? og + 8 * k : lo * KO + k;
#pragma unroll
        for (int j = 0; j < WC; j++) {
            const int c = W64 ? cg + 8 * j : hi * KC + j;
            if (o < h.S) { if (dWs) atomicAdd(dWs + (size_t)o * h.C + c, accw[k][j]); }
            else if (o < h.O) { if (dWp) atomicAdd(dWp + (size_t)(o - h.S) * h.C + c, accw[k][j]); }
        }
    }
    if (t < h.S) { if (dbs) atomicAdd(dbs + t, accb); }
    else if (t < h.O) { if (dbp) atomicAdd(dbp + (t - h.S), accb); }
}

static bool proj_supported(int C, int S, int P)
{
    const int kc = C / 16;
    return C >= 16 && (C % 16) == 0 && (kc <= 4 || kc == 6 || kc == 8) && S >= 1 && P >= 1 && S + P <= 64;
}

}  // namespace fgc

extern "C" int fgc_gravnet_project_supported(int32_t n_in, int32_t n_space, int32_t n_prop)
{
    return fgc::proj_supported(n_in, n_space, n_prop) ? 1 : 0;
}

extern "C" int fgc_gravnet_project_fwd(const float *x, int64_t n_rows, int32_t n_in, int32_t n_space,
                                       int32_t n_prop, const float *w_space, const float *b_space_or_null,
                                       const float *w_prop, const float *b_prop_or_null, float *out_space,
                                       float *out_prop, fgc_stream_t stream)
{
    return fgc_gravnet_project_fwd_cat(x, n_rows, n_in, n_space, n_prop, w_space, b_space_or_null, w_prop,
                                       b_prop_or_null, out_space, out_prop, nullptr, 0, stream);
}

extern "C" int fgc_gravnet_project_fwd_cat(const float *x, int64_t n_rows, int32_t n_in, int32_t n_space,
                                           int32_t n_prop, const float *w_space, const float *b_space_or_null,
                                           const float *w_prop, const float *b_prop_or_null, float *out_space,
                                           float *out_prop, float *x_copy_or_null, int64_t ld_copy,
                                           fgc_stream_t stream)
{
    FGC_NVTX("fgc_gravnet_project_fwd");
    using namespace fgc;
    if (n_rows < 0 || (x_copy_or_null && ld_copy < n_in)) return FGC_ERR_BAD_ARGUMENT;
    if (!proj_supported(n_in, n_space, n_prop)) return FGC_ERR_UNSUPPORTED_DIM;
    if (n_rows == 0) return FGC_OK;
    if (!x || !w_space || !w_prop || !out_space || !out_prop) return FGC_ERR_BAD_ARGUMENT;
    const ProjShape h = proj_shape(n_in, n_space, n_prop);
    const size_t smem = proj_smem_bytes(h, false);
    cudaStream_t s = (cudaStream_t)stream;
    const long long n_tiles = (n_rows + kProjRows - 1) / kProjRows;
    // persistent CTAs: as many as fit on the SMs (about 50 registers, 46 KB of shared memory at C = 64)
    long long blocks = (long long)fgc::sm_count() * (smem <= 54 * 1024 ? 4 : (smem <= 72 * 1024 ? 3 : 2));
    if (blocks > n_tiles) blocks = n_tiles;
#define FGC_PROJ_FWD(V)                                                                                      \
    do {                                                                                                     \
        FGC_RETURN_IF_CUDA(cudaFuncSetAttribute(k_project_fwd<V>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                                (int)smem));                                                 \
        k_project_fwd<V><<<(unsigned)blocks, kProjThreads, smem, s>>>(x, n_rows, h, w_space, b_space_or_null, \
                                                                     w_prop, b_prop_or_null, out_space, out_prop, \
                                                                     x_copy_or_null, (long long)ld_copy); \
    } while (0)
    switch (h.OP / 16) {
    case 1: FGC_PROJ_FWD(1); break;
    case 2: FGC_PROJ_FWD(2); break;
    case 3: FGC_PROJ_FWD(3); break;
    default: FGC_PROJ_FWD(4); break;
    }
#undef FGC_PROJ_FWD
    return (int)cudaGetLastError();
}

extern "C" int fgc_gravnet_project_bwd(const float *x, int64_t n_rows, int32_t n_in, int32_t n_space,
                                       int32_t n_prop, const float *w_space, const float *w_prop,
                                       const float *d_space_or_null, const float *d_prop_or_null,
                                       float *dx_or_null, float *dw_space, float *db_space_or_null,
                                       float *dw_prop, float *db_prop_or_null, fgc_stream_t stream)
{
    return fgc_gravnet_project_bwd_cat(x, n_rows, n_in, n_space, n_prop, w_space, w_prop, d_space_or_null,
                                       d_prop_or_null, nullptr, 0, dx_or_null, dw_space, db_space_or_null,
                                       dw_prop, db_prop_or_null, stream);
}

extern "C" int fgc_gravnet_project_bwd_cat(const float *x, int64_t n_rows, int32_t n_in, int32_t n_space,
                                           int32_t n_prop, const float *w_space, const float *w_prop,
                                           const float *d_space_or_null, const float *d_prop_or_null,
                                           const float *dx_add_or_null, int64_t ld_add, float *dx_or_null,
                                           float *dw_space, float *db_space_or_null, float *dw_prop,
                                           float *db_prop_or_null, fgc_stream_t stream)
{
    FGC_NVTX("fgc_gravnet_project_bwd");
    using namespace fgc;
    if (n_rows < 0 || (dx_add_or_null && ld_add < n_in)) return FGC_ERR_BAD_ARGUMENT;
    if (!proj_supported(n_in, n_space, n_prop)) return FGC_ERR_UNSUPPORTED_DIM;
    if (!w_space || !w_prop || !dw_space || !dw_prop) return FGC_ERR_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    // the weight and bias gradients are accumulated: start them at zero
    FGC_RETURN_IF_CUDA(cudaMemsetAsync(dw_space, 0, sizeof(float) * (size_t)n_space * n_in, s));
    FGC_RETURN_IF_CUDA(cudaMemsetAsync(dw_prop, 0, sizeof(float) * (size_t)n_prop * n_in, s));
    if (db_space_or_null) FGC_RETURN_IF_CUDA(cudaMemsetAsync(db_space_or_null, 0, sizeof(float) * n_space, s));
    if (db_prop_or_null) FGC_RETURN_IF_CUDA(cudaMemsetAsync(db_prop_or_null, 0, sizeof(float) * n_prop, s));
    if (n_rows == 0) return FGC_OK;
    if (!x) return FGC_ERR_BAD_ARGUMENT;
    const ProjShape h = proj_shape(n_in, n_space, n_prop);
    const size_t smem = proj_smem_bytes(h, true);
    const long long n_tiles = (n_rows + kProjRows - 1) / kProjRows;
    // persistent CTAs: two per SM (about 128 registers per thread), one where the tiles need more
    // than half of the SM's shared memory
    long long blocks = (long long)fgc::sm_count() * (smem <= 110 * 1024 ? 2 : 1);
    if (blocks > n_tiles) blocks = n_tiles;
#define FGC_PROJ_BWD(V, Q)                                                                                   \
    do {                                                                                                     \
        FGC_RETURN_IF_CUDA(cudaFuncSetAttribute(k_project_bwd<V, Q>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                                (int)smem));                                                 \
        k_project_bwd<V, Q><<<(unsigned)blocks, kProjThreads, smem, s>>>(                                    \
            x, n_rows, h, w_space, w_prop, d_space_or_null, d_prop_or_null, dx_or_null, dw_space,            \
            db_space_or_null, dw_prop, db_prop_or_null, dx_add_or_null, (long long)ld_add);                  \
    } while (0)
#define FGC_PROJ_BWD_KC(V)                                                                                   \
    do {                                                                                                     \
        switch (n_in / 16) {                                                                                 \
        case 1: FGC_PROJ_BWD(V, 1); break;                                                                   \
        case 2: FGC_PROJ_BWD(V, 2); break;                                                                   \
        case 3: FGC_PROJ_BWD(V, 3); break;                                                                   \
        case 4: FGC_PROJ_BWD(V, 4); break;                                                                   \
        case 6: FGC_PROJ_BWD(V, 6); break;                                                                   \
        case 8: FGC_PROJ_BWD(V, 8); break;                                                                   \
        default: return FGC_ERR_UNSUPPORTED_DIM;                                                             \
        }                                                                                                    \
    } while (0)
    switch (h.OP / 16) {
    case 1: FGC_PROJ_BWD_KC(1); break;
    case 2: FGC_PROJ_BWD_KC(2); break;
    case 3: FGC_PROJ_BWD_KC(3); break;
    default: FGC_PROJ_BWD_KC(4); break;
    }
#undef FGC_PROJ_BWD_KC
#undef FGC_PROJ_BWD
    return (int)cudaGetLastError();
}
