/*
 * fgc_b200.h -- C ABI of libfgc_b200.so, the sm_100a implementation of the
 * FastGraphCompute spatial-graph hot path (coordinate binning, binned kNN
 * forward/backward, index_replacer, GravNet neighbour aggregation).
 *
 * Conventions
 *  - Every pointer is a DEVICE pointer unless its name ends in _host.
 *  - Row-major, contiguous arrays; coordinates fp32, indices int64 (the
 *    reference's public dtypes), row_splits int64 of length n_rs.
 *  - The library never allocates or frees device memory and never retains a
 *    pointer after the call returns.  Outputs and scratch ("workspace") are
 *    provided by the caller; *_workspace_bytes() says how much.
 *  - Work is enqueued on `stream` (a cudaStream_t); calls do not synchronise
 *    unless documented.  The device that owns the pointers must be current.
 *  - Return value: FGC_OK (0), a negative FGC_ERR_* argument error, or a
 *    positive cudaError_t value.  Data-dependent problems (non-finite
 *    coordinates, malformed row_splits) are reported through a status word in
 *    device memory, read with fgc_read_status().
 *  - Re-entrant: concurrent calls on different streams/devices are safe as long
 *    as they use different workspaces.  The library keeps no mutable state
 *    between calls, with one exception: fgc_binned_knn_fwd_static owns a scratch
 *    array per GPU that all of its calls share (see there).
 *
 * Each entry point names the reference interface it replaces
 * (paths relative to the FastGraphCompute repository).
 */
#ifndef FGC_B200_H
#define FGC_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FGC_OK 0
#define FGC_ERR_BAD_ARGUMENT (-1)   /* null pointer, negative size, ... */
#define FGC_ERR_UNSUPPORTED_DIM (-2)/* kNN: n_coords < 2 (the reference raises for < 2 bin dims) or > FGC_MAX_KNN_DIMS */
#define FGC_ERR_UNSUPPORTED_K (-3)  /* K < 1 or K > FGC_MAX_K */
#define FGC_ERR_WORKSPACE (-4)      /* workspace too small / misaligned */
#define FGC_ERR_TOO_LARGE (-5)      /* n_vert or a bin table exceeds 2^31-1 entries */
#define FGC_ERR_STATIC_TOO_LARGE (-6) /* fgc_binned_knn_fwd_static: problem needs more than FGC_STATIC_WORKSPACE_BYTES */

/* bits of the device status word */
#define FGC_STATUS_NONFINITE 1      /* a coordinate is NaN or +-Inf */
#define FGC_STATUS_BAD_ROW_SPLITS 2 /* row_splits not 0-based, not non-decreasing or not ending at n_vert */
#define FGC_STATUS_BAD_DMAX 4       /* binning: max coordinate not > 0 after normalisation */
#define FGC_STATUS_BAD_NBINS 8      /* binning: some n_bins <= 0 */
#define FGC_STATUS_BAD_BINWIDTH 16  /* binning: bin_width <= 0 */
#define FGC_STATUS_INTERNAL 32      /* an internal consistency check failed */
#define FGC_STATUS_DEBUG_BOUNDS 64  /* only in a library built with -DFGC_DEBUG: an index was out of range (the access was skipped) */

#define FGC_MAX_K 257               /* self + 256 neighbours */
#define FGC_MAX_BIN_DIMS 8          /* coordinate dimensions accepted by fgc_bin_* */
#define FGC_MAX_KNN_DIMS 16         /* coordinate dimensions accepted by the kNN (the first 3 are binned) */

typedef struct CUstream_st *fgc_stream_t; /* == cudaStream_t */

/* Library version (major*10000 + minor*100 + patch). */
int fgc_version(void);

/* Text for a return value of this library. */
const char *fgc_error_string(int code);

/* ------------------------------------------------------------------------- */
/* bin_by_coordinates                                                         */
/* ------------------------------------------------------------------------- */

/*
 * Binning parameters derived on the device by fgc_bin_prepare (device-resident
 * record, 256 bytes; copy it to the host to learn n_bins / bin_width / status).
 */
typedef struct fgc_bin_params {
    int32_t status;                    /* FGC_STATUS_* bits, 0 = fine */
    int32_t n_coords;
    float bin_width;                   /* the single, uniform bin width */
    int32_t reserved0;
    float shift[FGC_MAX_BIN_DIMS];     /* subtracted from every coordinate (0 if pre_normalized) */
    int64_t n_bins[FGC_MAX_BIN_DIMS];  /* bins per dimension */
    uint32_t scratch[2 * FGC_MAX_BIN_DIMS + 2];
    uint8_t pad[256 - 16 - 4 * FGC_MAX_BIN_DIMS - 8 * FGC_MAX_BIN_DIMS - 4 * (2 * FGC_MAX_BIN_DIMS + 2)];
} fgc_bin_params;

/*
 * Step 1 of bin_by_coordinates: one fused pass over the coordinates (finite
 * check, per-dimension min and max) and the derivation of shift, dmax, n_bins
 * and bin_width with the reference's fp32 arithmetic.
 * Replaces the host part of bin_by_coordinates (extensions/bin_by_coordinates.cpp:31-120,
 * same steps in extensions/bin_by_coordinates.py:33-104).
 *   bin_width_or_null : [1] fp32 or NULL;  n_bins_or_null : [n_bins_len] int64
 *   (n_bins_len 1 = scalar repeated, or n_coords) or NULL; at least one is needed.
 * out_params is written on the device; no synchronisation.
 */
int fgc_bin_prepare(const float *coords, int64_t n_vert, int32_t n_coords, int32_t pre_normalized,
                    const float *bin_width_or_null, const int64_t *n_bins_or_null,
                    int32_t n_bins_len, fgc_bin_params *out_params, fgc_stream_t stream);

/*
 * Step 2: per-point bin assignment and histogram.
 * Replaces bin_by_coordinates_cuda_fn / calc (extensions/bin_by_coordinates_cuda_kernel.cu:24-172;
 * CPU twin extensions/bin_by_coordinates_cpu.cpp:7-152).
 *   out_bin_idx  [n_vert, n_coords+1] = [row-split index, bin index per dimension]
 *   out_flat     [n_vert]  flat bin id (last dimension fastest, row split slowest)
 *   out_n_per_bin[n_total_bins] (must be zeroed by the caller) or NULL when
 *                calc_n_per_bin == 0
 * n_total_bins = prod(n_bins) * (n_rs - 1) as read back from the parameters.
 */
int fgc_bin_assign(const float *coords, int64_t n_vert, int32_t n_coords,
                   const int64_t *row_splits, int64_t n_rs, const fgc_bin_params *params,
                   int32_t calc_n_per_bin, int64_t n_total_bins, int64_t *out_bin_idx,
                   int64_t *out_flat, int64_t *out_n_per_bin, fgc_stream_t stream);

/* ------------------------------------------------------------------------- */
/* binned_select_knn                                                          */
/* ------------------------------------------------------------------------- */

/* Scratch bytes fgc_binned_knn_fwd needs for this problem size (0 on bad arguments). */
size_t fgc_knn_workspace_bytes(int64_t n_vert, int32_t n_coords, int64_t n_rs, int32_t K);

/*
 * k-nearest-neighbour search inside each row split (forward).
 * Replaces BinnedKNNAutograd::forward (extensions/binned_knn_autograd_kernel.cpp:85-209)
 * including its callees binned_select_knn_cuda_fn (extensions/binned_select_knn_cuda_kernel.cu:252-384),
 * index_replacer_cuda_fn and the un-sort scatters: builds its own bin grid,
 * counting-sorts the points, searches in expanding shells and writes rows in
 * ORIGINAL order with ORIGINAL ids.
 *   out_idx   [n_vert, K] int64: slot 0 = the point itself, then its K-1 nearest
 *             neighbours of the same row split in no particular order, then -1
 *             (or the point's own id when tf_compat != 0) where the row split
 *             has fewer than K eligible points.
 *   out_distsq[n_vert, K] fp32 squared distances (0 for slot 0 and empty slots),
 *             accumulated over the dimensions in order, one rounding per
 *             operation, as extensions/binned_select_knn_cpu.cpp:10-19.
 *   direction_or_null [n_vert] int64: 0 may only BE a neighbour, 1 may only HAVE
 *             neighbours, 2 neither, other values: no restriction.
 *   target_occupancy : mean points per grid cell to aim for (<= 0: library default).
 * The first 4 bytes of the workspace hold the status word (fgc_read_status).
 */
int fgc_binned_knn_fwd(const float *coords, int64_t n_vert, int32_t n_coords,
                       const int64_t *row_splits, int64_t n_rs, int32_t K,
                       const int64_t *direction_or_null, int32_t tf_compat,
                       float target_occupancy, int64_t *out_idx, float *out_distsq,
                       void *workspace, size_t workspace_bytes, fgc_stream_t stream);

/*
 * The two halves of fgc_binned_knn_fwd, for callers that search the same grid more
 * than once or want to time the phases separately.
 *
 * fgc_knn_build_grid: everything up to the search (extent reduction, grid choice,
 * histogram, scan, counting-sort scatter).  Replaces steps 2-8 of
 * BinnedKNNAutograd::forward (extensions/binned_knn_autograd_kernel.cpp:100-145:
 * calculate_optimal_bins, bin_by_coordinates, argsort, index_select, cumsum).
 *
 * fgc_knn_search: the neighbour search proper on a built workspace, including the
 * mapping back to original ids and row order.  Replaces binned_select_knn_cuda_fn
 * (extensions/binned_select_knn_cuda_kernel.cu:252-384) + index_replacer + un-sort
 * scatter (extensions/binned_knn_autograd_kernel.cpp:157-195).  has_direction must say
 * whether the grid was built with a direction array.  flags: FGC_SEARCH_COUNT accumulates
 * the debug counters in the workspace (fgc_knn_read_counters).  A built grid may be searched
 * any number of times (other K is not allowed: the workspace layout depends on the arguments).
 * Two searches of one workspace must not overlap in time (they share the list of queries that
 * gave up their walk and its scratch, which a search clears when it starts -- FGC_SEARCH_FRESH
 * says that this is the first search since the grid was built, which left them cleared; the
 * flag must not be given for a later search).
 *
 * When the status word of the workspace is non-zero after the grid build (non-finite
 * coordinate, malformed row_splits; see fgc_read_status) no neighbour is searched: every row
 * of out_idx / out_distsq gets the defaults of a point without neighbours (itself in slot 0,
 * -1 -- or itself with tf_compat -- elsewhere, distances 0).  The same holds for
 * fgc_binned_knn_fwd and fgc_binned_knn_fwd_static.
 */
int fgc_knn_build_grid(const float *coords, int64_t n_vert, int32_t n_coords,
                       const int64_t *row_splits, int64_t n_rs, int32_t K,
                       const int64_t *direction_or_null, float target_occupancy,
                       void *workspace, size_t workspace_bytes, fgc_stream_t stream);
/*
 * D = 4 only: the grid spans four coordinates unless the data is strongly clustered, in which
 * case the density pass rebuilds it over three (decided on the device).  A caller that knows
 * its data fixes the form: fgc_knn_build_grid_dims(..., grid_dims = 3 or 4, ...) and the
 * matching FGC_SEARCH_GRID3 / FGC_SEARCH_GRID4 flag for fgc_knn_search, which saves the trial
 * histogram and runs a kernel that holds one search only.  grid_dims = 0 and no flag: automatic.
 * fgc_knn_publish_grid_info stores {status word, (3 or 4) + 16 * fell_back} into mapped pinned
 * memory (like fgc_publish_status) so that a host can learn the choice without a copy.
 * No counterparts in the reference.
 */
int fgc_knn_build_grid_dims(const float *coords, int64_t n_vert, int32_t n_coords,
                            const int64_t *row_splits, int64_t n_rs, int32_t K,
                            const int64_t *direction_or_null, float target_occupancy,
                            int32_t grid_dims, void *workspace, size_t workspace_bytes,
                            fgc_stream_t stream);
int fgc_knn_publish_grid_info(const void *workspace, int32_t *info_mapped, fgc_stream_t stream);
#define FGC_SEARCH_COUNT 1     /* flags: accumulate the debug counters */
#define FGC_SEARCH_GRID3 8     /* flags: the grid was built with grid_dims = 3 (D = 4) */
#define FGC_SEARCH_GRID4 16    /* flags: the grid was built with grid_dims = 4 (D = 4) */
#define FGC_SEARCH_FRESH 32    /* flags: first search of this workspace since fgc_knn_build_grid: nothing to clear */
int fgc_knn_search(int64_t n_vert, int32_t n_coords, int64_t n_rs, int32_t K,
                   int32_t has_direction, int32_t tf_compat, int32_t flags,
                   int64_t *out_idx, float *out_distsq, void *workspace,
                   size_t workspace_bytes, fgc_stream_t stream);

/*
 * Diagnostics of a workspace, copied to the host (synchronises the stream): eight 64-bit
 * counters that a search launched with FGC_SEARCH_COUNT accumulates ([0] distance
 * evaluations, [1] 32-candidate steps, [2] list insertions, [3] metadata batches, [4] shells,
 * [5] queries that scanned their whole row split), two facts that need no counting search
 * ([6] queries the last search handed to whole CTAs because their walk gave up in a row split
 * of more than 4096 points, [7] cells of more than 512 points), the grid shape [3] and the
 * cell width.
 * Any output pointer may be NULL.  No counterpart in the reference.
 */
int fgc_knn_read_counters(const void *workspace, uint64_t *counters_host,
                          int32_t *grid_shape_host, float *cell_width_host,
                          fgc_stream_t stream);

/*
 * kNN forward without a caller-provided workspace and without any allocation.
 * (No counterpart in the reference, whose ops allocate through PyTorch.)
 *
 * For hosts that cannot allocate device memory at call time -- services and online event
 * filters that fix their memory budget at start-up, or plugins that are only handed input
 * and output pointers -- the scratch lives in a fixed array inside the library image
 * (FGC_STATIC_WORKSPACE_BYTES per GPU, held by every GPU that loads the library until the
 * process exits).  Same inputs, outputs and results as fgc_binned_knn_fwd, plus
 *   out_status : [1] int32 in device memory, receives the FGC_STATUS_* word of the call.
 *                It is written only when the function returns FGC_OK; after any other
 *                return value its content is whatever it held before.
 * Limits and rules:
 *   - returns FGC_ERR_STATIC_TOO_LARGE when fgc_knn_workspace_bytes(n_vert, n_coords, n_rs, K)
 *     exceeds FGC_STATIC_WORKSPACE_BYTES (that is at about 40 000 points with up to 4
 *     coordinates and about 35 000 with 5 to 8); nothing is launched in that case;
 *   - calls no cudaMalloc/cudaFree or other allocating routine;
 *   - the first call on each GPU looks up the device address of the array
 *     (cudaGetSymbolAddress, with that GPU current).  With CUDA's lazy module loading that
 *     call may also load the library's device code, which places the array in device memory
 *     and can synchronise.  A host that must not see either later makes one warm-up call
 *     per GPU at start-up (n_vert = 0 is enough), outside any stream capture;
 *   - the GPU that owns `stream` and the pointers must be the current device: the array's
 *     address is taken for the current device, not derived from the stream;
 *   - all calls on one GPU share the one array: calls that can overlap on the GPU (different
 *     streams or host threads) race and must be serialised by the caller.  The array keeps
 *     the previous call's contents; each call clears the parts it relies on being zero.
 */
#define FGC_STATIC_WORKSPACE_BYTES (4u << 20)
int fgc_binned_knn_fwd_static(const float *coords, int64_t n_vert, int32_t n_coords,
                              const int64_t *row_splits, int64_t n_rs, int32_t K,
                              const int64_t *direction_or_null, int32_t tf_compat,
                              float target_occupancy, int64_t *out_idx, float *out_distsq,
                              int32_t *out_status, fgc_stream_t stream);

/*
 * Device pointer to the cell order inside a kNN workspace after fgc_knn_build_grid: int32
 * [n_vert], entry p = original id of the p-th point in cell order (a permutation that keeps
 * spatial neighbours together).  NULL on bad arguments.  No counterpart in the reference
 * (its equivalent is the argsort at extensions/binned_knn_autograd_kernel.cpp:118-120).
 */
const int32_t *fgc_knn_cell_order(const void *workspace, int64_t n_vert, int32_t n_coords,
                                  int64_t n_rs, int32_t K);

/*
 * Copies the status word at the start of a workspace / fgc_bin_params to the
 * host and waits for the stream (the only synchronising call of the library).
 */
int fgc_read_status(const void *workspace_or_params, int32_t *status_host, fgc_stream_t stream);

/*
 * The same status word without a copy and without waiting: a one-thread kernel on
 * `stream` stores it to `status_mapped`, which must be page-locked host memory that
 * the device can address (cudaHostAlloc / cudaHostRegister under unified addressing).
 * The host reads it after an event recorded behind this call has completed.  Unlike a
 * device-to-host copy the store does not queue behind bulk copies of other streams, so
 * a host that pipelines batches can check every batch without stalling the pipeline.
 * No counterpart in the reference (its checks synchronise the device).
 */
int fgc_publish_status(const void *workspace_or_params, int32_t *status_mapped, fgc_stream_t stream);

/*
 * Gradient of the squared distances with respect to the coordinates (backward).
 * Replaces binned_select_knn_grad_cuda_fn (extensions/binned_select_knn_grad_cuda_kernel.cu:90-164;
 * CPU twin extensions/binned_select_knn_grad_cpu.cpp:96-164):
 *   G[i] = -sum_k 2 g[i,k] (x[n]-x[i]),  G[n] += 2 g[i,k] (x[n]-x[i]),  n = idx[i,k] >= 0.
 * out_grad_coords [n_vert, n_coords] is overwritten.
 */
int fgc_binned_knn_bwd(const float *grad_distsq, const int64_t *idx, const float *coords,
                       int64_t n_vert, int32_t K, int32_t n_coords, float *out_grad_coords,
                       fgc_stream_t stream);
/*
 * The same with a processing order: order_or_null [n_vert] int32, a permutation of the rows
 * (fgc_knn_cell_order of the forward's workspace, copied before the workspace is reused).
 * Rows that are neighbours in space are then processed by the same CTA, so that consecutive
 * warps meet the same neighbour rows in cache (a few per cent on 200 000 points, K = 32: the
 * ids still address rows in the caller's order).  The gradient is the same up to the order
 * of the float additions.  No counterpart in the reference.
 */
int fgc_binned_knn_bwd_ordered(const float *grad_distsq, const int64_t *idx, const float *coords,
                               int64_t n_vert, int32_t K, int32_t n_coords,
                               const int32_t *order_or_null, float *out_grad_coords,
                               fgc_stream_t stream);

/*
 * Deterministic variant of the backward: sorted-segment reductions instead of float atomics.
 *
 * fgc_build_reverse_graph turns idx [n_vert, K] into a CSR structure that lists, for every
 * point n, the (row, slot) pairs with idx[row, slot] == n, each segment sorted by
 * row*K + slot (scratch: fgc_reverse_graph_bytes, caller-provided, 256-byte aligned;
 * requires n_vert*K < 2^31).  fgc_binned_knn_bwd_sorted computes the same gradient as
 * fgc_binned_knn_bwd by gathering over those segments in a fixed order: bit-identical from
 * run to run, where the atomic version (like the reference's CUDA kernel,
 * extensions/binned_select_knn_grad_cuda_kernel.cu:58-88) depends on the order in which the
 * atomics land.  The graph depends on idx only and can be reused for several backward calls.
 */
size_t fgc_reverse_graph_bytes(int64_t n_vert, int32_t K);
int fgc_build_reverse_graph(const int64_t *idx, int64_t n_vert, int32_t K, void *rgraph,
                            size_t rgraph_bytes, fgc_stream_t stream);
int fgc_binned_knn_bwd_sorted(const float *grad_distsq, const int64_t *idx, const float *coords,
                              int64_t n_vert, int32_t K, int32_t n_coords, const void *rgraph,
                              size_t rgraph_bytes, float *out_grad_coords, fgc_stream_t stream);

/* ------------------------------------------------------------------------- */
/* index_replacer                                                             */
/* ------------------------------------------------------------------------- */

/*
 * out[i] = in[i] < 0 ? in[i] : (in[i] >= n_replacements ? replacements[i] : replacements[in[i]]).
 * Replaces index_replacer_cuda_fn (extensions/index_replacer_cuda_kernel.cu:9-58; CPU twin
 * extensions/index_replacer_cpu.cpp:7-26).  The out-of-range branch reads replacements at
 * the element's POSITION, as the reference does; positions beyond the table keep in[i].
 */
int fgc_index_replacer(const int64_t *to_be_replaced, int64_t n, const int64_t *replacements,
                       int64_t n_replacements, int64_t *out, fgc_stream_t stream);

/* ------------------------------------------------------------------------- */
/* GravNet neighbour aggregation                                              */
/* ------------------------------------------------------------------------- */

/*
 * Fused steps 4-7 of GravNetOp.forward (fastgraphcompute/gnn_ops.py:90-102, with
 * select_with_default of extensions/oc_helper.py:232-271): weights exp(-10 distsq),
 * gather of neighbour rows (-1 -> 0), mean over the K slots (divided by K) and
 * max over the K slots.  out_argmax [n_vert, P] int32 records the slot of the max
 * for the backward pass.  order_or_null [n_vert] int32: optional processing order (a
 * permutation of the points, e.g. fgc_knn_cell_order of the kNN that produced idx); it only
 * improves cache locality, results do not depend on it.
 */
int fgc_gravnet_aggregate_fwd(const float *prop, const int64_t *idx, const float *distsq,
                              int64_t n_vert, int32_t K, int32_t P, float *out_mean,
                              float *out_max, int32_t *out_argmax, const int32_t *order_or_null,
                              fgc_stream_t stream);

/*
 * Backward of the aggregation (what autograd derives for gnn_ops.py:90-102).
 * out_d_prop [n_vert, P] and out_d_distsq [n_vert, K] are overwritten.
 */
int fgc_gravnet_aggregate_bwd(const float *prop, const int64_t *idx, const float *distsq,
                              const int32_t *argmax, const float *grad_mean,
                              const float *grad_max, int64_t n_vert, int32_t K, int32_t P,
                              float *out_d_prop, float *out_d_distsq, const int32_t *order_or_null,
                              fgc_stream_t stream);

/*
 * Deterministic variant of fgc_gravnet_aggregate_bwd (P <= 128): d_prop is gathered over the
 * sorted segments of the reverse neighbour graph of idx (fgc_build_reverse_graph) instead of
 * being scattered with float atomics, d_distsq as before.  Bit-identical from run to run.
 * No counterpart in the reference (torch autograd's index_put accumulation is atomic).
 */
int fgc_gravnet_aggregate_bwd_sorted(const float *prop, const int64_t *idx, const float *distsq,
                                     const int32_t *argmax, const float *grad_mean,
                                     const float *grad_max, int64_t n_vert, int32_t K, int32_t P,
                                     const void *rgraph, size_t rgraph_bytes, float *out_d_prop,
                                     float *out_d_distsq, const int32_t *order_or_null,
                                     fgc_stream_t stream);

/*
 * The three aggregation calls with a row stride (in floats) for tensors that are columns of a
 * wider row-major matrix: ld_out for out_mean / out_max (the aggregation written straight into
 * its columns of the concatenated input [x | mean | max] of the layer's output transformation,
 * gnn_ops.py:106-109), ld_grad for grad_mean / grad_max (the matching columns of that matrix's
 * gradient).  ld >= P; the 16-byte vector kernels need ld % 4 == 0 and 16-byte aligned
 * pointers, other shapes take the scalar kernels.  Everything else as in the calls above.
 */
int fgc_gravnet_aggregate_fwd_ld(const float *prop, const int64_t *idx, const float *distsq,
                                 int64_t n_vert, int32_t K, int32_t P, float *out_mean,
                                 float *out_max, int64_t ld_out, int32_t *out_argmax,
                                 const int32_t *order_or_null, fgc_stream_t stream);
int fgc_gravnet_aggregate_bwd_ld(const float *prop, const int64_t *idx, const float *distsq,
                                 const int32_t *argmax, const float *grad_mean,
                                 const float *grad_max, int64_t ld_grad, int64_t n_vert, int32_t K,
                                 int32_t P, float *out_d_prop, float *out_d_distsq,
                                 const int32_t *order_or_null, fgc_stream_t stream);
int fgc_gravnet_aggregate_bwd_sorted_ld(const float *prop, const int64_t *idx, const float *distsq,
                                        const int32_t *argmax, const float *grad_mean,
                                        const float *grad_max, int64_t ld_grad, int64_t n_vert,
                                        int32_t K, int32_t P, const void *rgraph,
                                        size_t rgraph_bytes, float *out_d_prop, float *out_d_distsq,
                                        const int32_t *order_or_null, fgc_stream_t stream);

/*
 * Radius mode of the reference's brute-force op select_knn::select_knn(coords, row_splits, mask,
 * n_neighbours, max_radius, mask_mode) (select_knn.cpp:60-62; select_knn_cpu.cpp:98-132 /
 * select_knn_cuda_kernel.cu:73-132; the mask arguments are never read there): the K-1 nearest
 * other points of the row split that lie within max_radius.  Run fgc_binned_knn_fwd, then this
 * call on its outputs, in place: slots with distsq > max_radius^2 are dropped, the remaining
 * slots close up in their order, freed slots become pads.  max_radius <= 0: no radius, no-op.
 * The radius is squared in double and rounded to float once (select_knn_cpu.cpp:176-178).
 */
int fgc_knn_radius_filter(int64_t *idx, float *distsq, int64_t n_vert, int32_t K, double max_radius,
                          int32_t tf_compat, fgc_stream_t stream);

/*
 * Object-condensation index matrices -- the consumers of the same row_splits data on the loss
 * side (the reference's oc_helper_matrices: extensions/oc_helper.py:128-230 ->
 * oc_helper_cpu.cpp:117-156 / oc_helper_cuda_kernel.cu, helper oc_helper_helper.cpp:31-93).
 *
 * An object is the set of points of ONE row split that share a non-negative truth index.
 *   M[n_unique, n_maxuq]     point ids of each object, ascending, padded with -1
 *   M_not[n_unique, n_maxrs] ids of all other points of the object's row split, ascending, -1 padded
 *   objects_per_split[n_rs-1]
 * n_unique, n_maxuq (largest object) and n_maxrs (largest row split) are only known on the
 * device, so the work is split like the reference's (which computes them on the host first):
 *   fgc_oc_prepare     sorts (truth index, point id), finds the objects, writes objects_per_split
 *   fgc_oc_read_sizes  status word + {n_unique, n_maxuq, n_maxrs}; waits for the stream
 *   fgc_oc_fill        writes M and, when out_M_not_or_null != NULL, M_not
 * The rows are ordered by (truth index, row split); the reference leaves the order open.
 * asso_idx[n_vert] int64, row_splits[n_rs] int64 (validated: status FGC_STATUS_BAD_ROW_SPLITS).
 */
size_t fgc_oc_workspace_bytes(int64_t n_vert);
int fgc_oc_prepare(const int64_t *asso_idx, int64_t n_vert, const int64_t *row_splits, int64_t n_rs,
                   void *workspace, size_t workspace_bytes, int64_t *objects_per_split,
                   fgc_stream_t stream);
int fgc_oc_read_sizes(const void *workspace, int32_t *status_host, int64_t sizes_host[3],
                      fgc_stream_t stream);
int fgc_oc_fill(const void *workspace, size_t workspace_bytes, int64_t n_vert, const int64_t *row_splits,
                int64_t n_unique, int64_t n_maxuq, int64_t n_maxrs, int64_t *out_M,
                int64_t *out_M_not_or_null, fgc_stream_t stream);

/*
 * out[e, :] = feat[idx[e], :] for idx[e] in [0, n_rows_feat), else the default value
 * (the reference's select_with_default, extensions/oc_helper.py:232-271, which builds the
 * result from a full(), a nonzero() and two advanced-index passes).  idx[n_idx] int64 (the
 * flattened [V, K] index matrix), feat[n_rows_feat, n_feat] of 4- or 8-byte elements
 * (word_bytes), default_word_host: the default value's bit pattern, read on the host at
 * call time; out[n_idx, n_feat] of the same element type.
 */
int fgc_select_with_default(const int64_t *idx, int64_t n_idx, const void *feat, int64_t n_rows_feat,
                            int64_t n_feat, int32_t word_bytes, const void *default_word_host,
                            void *out, fgc_stream_t stream);

/*
 * The two input projections of a GravNet layer in one pass over x
 * (fastgraphcompute/gnn_ops.py:79-82: space = Linear(C -> S)(x), propagate = Linear(C -> P)(x),
 * two library GEMMs in the reference; their autograd backward is six more GEMMs / reductions):
 *   fwd: out_space[n,S] = x @ w_space^T + b_space, out_prop[n,P] = x @ w_prop^T + b_prop
 *   bwd: dx[n,C] = d_space @ w_space + d_prop @ w_prop   (skipped when dx_or_null is NULL),
 *        dw_space[S,C], db_space[S], dw_prop[P,C], db_prop[P] (overwritten; db pointers may be
 *        NULL); a NULL d_space / d_prop counts as zeros.
 * x [n,C] fp32 row-major, weights [out,in] as in torch.nn.Linear.  Supported shapes: C one of
 * 16, 32, 48, 64, 96, 128 and S + P <= 64 (fgc_gravnet_project_supported; FGC_ERR_UNSUPPORTED_DIM otherwise -- the Python
 * layer then uses the library GEMMs).  fp32 with fused multiply-adds; the weight gradients are
 * accumulated with float atomics across CTAs (sums of n terms: equal to a GEMM's to rounding).
 */
int fgc_gravnet_project_supported(int32_t n_in, int32_t n_space, int32_t n_prop);
int fgc_gravnet_project_fwd(const float *x, int64_t n_rows, int32_t n_in, int32_t n_space, int32_t n_prop,
                            const float *w_space, const float *b_space_or_null, const float *w_prop,
                            const float *b_prop_or_null, float *out_space, float *out_prop,
                            fgc_stream_t stream);
int fgc_gravnet_project_bwd(const float *x, int64_t n_rows, int32_t n_in, int32_t n_space, int32_t n_prop,
                            const float *w_space, const float *w_prop, const float *d_space_or_null,
                            const float *d_prop_or_null, float *dx_or_null, float *dw_space,
                            float *db_space_or_null, float *dw_prop, float *db_prop_or_null,
                            fgc_stream_t stream);

/*
 * The two projection calls for a layer that keeps [x | mean | max] as one matrix (gnn_ops.py:106):
 * the forward also writes the rows of x into the first n_in columns of x_copy (row stride ld_copy
 * floats; NULL: no copy), so the concatenation costs no pass of its own; the backward adds the
 * first n_in columns of dx_add (row stride ld_add; the x columns of that matrix's gradient) to
 * dx while it writes it, so the two gradients of x meet without an addition pass.
 */
int fgc_gravnet_project_fwd_cat(const float *x, int64_t n_rows, int32_t n_in, int32_t n_space,
                                int32_t n_prop, const float *w_space, const float *b_space_or_null,
                                const float *w_prop, const float *b_prop_or_null, float *out_space,
                                float *out_prop, float *x_copy_or_null, int64_t ld_copy,
                                fgc_stream_t stream);
int fgc_gravnet_project_bwd_cat(const float *x, int64_t n_rows, int32_t n_in, int32_t n_space,
                                int32_t n_prop, const float *w_space, const float *w_prop,
                                const float *d_space_or_null, const float *d_prop_or_null,
                                const float *dx_add_or_null, int64_t ld_add, float *dx_or_null,
                                float *dw_space, float *db_space_or_null, float *dw_prop,
                                float *db_prop_or_null, fgc_stream_t stream);

/*
 * Conversions between row splits and PyTorch-Geometric style batch vectors on the device
 * (fastgraphcompute/torch_geometric_interface.py:4-42 row_splits_from_strict_batch and :45-74
 * strict_batch_from_row_splits of the reference, which use nonzero / repeat_interleave).
 *
 * fgc_row_splits_from_strict_batch: batch[n_points] int64, the points of one row split
 * contiguous -> out_row_splits (room for n_points + 1 entries; only the first *count are
 * written): 0, every position whose id differs from its predecessor's, n_points.  The count
 * stays in the workspace (fgc_pyg_workspace_bytes(n_points) bytes) until fgc_pyg_read_count
 * copies it to the host (synchronises the stream).  An empty batch gives [0, 0].
 *
 * fgc_strict_batch_from_row_splits: out_batch[i] = index of the row split that holds point i,
 * for i < n_points (= row_splits[n_rs - 1], which the caller knows or reads).
 */
size_t fgc_pyg_workspace_bytes(int64_t n_points);
int fgc_row_splits_from_strict_batch(const int64_t *batch, int64_t n_points, int64_t *out_row_splits,
                                     void *workspace, size_t workspace_bytes, fgc_stream_t stream);
int fgc_pyg_read_count(const void *workspace, int64_t *n_row_splits_host, fgc_stream_t stream);
int fgc_strict_batch_from_row_splits(const int64_t *row_splits, int64_t n_rs, int64_t n_points,
                                     int64_t *out_batch, fgc_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* FGC_B200_H */
