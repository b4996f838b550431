// Shared device/host helpers of libfgc_b200 (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <nvtx3/nvToolsExt.h>

#include "fgc_b200.h"

#define FGC_FULL_MASK 0xffffffffu

// Launch-error check usable inside extern "C" entry points: returns the CUDA
// error code to the caller (never exits, never synchronises).
#define FGC_RETURN_IF_CUDA(expr)                 \
    do {                                         \
        cudaError_t fgc_e_ = (expr);             \
        if (fgc_e_ != cudaSuccess) return (int)fgc_e_; \
    } while (0)

#define FGC_CHECK_LAUNCH() FGC_RETURN_IF_CUDA(cudaGetLastError())

// Bounds checks of the debug build (nvcc -DFGC_DEBUG; fastgraphcompute_b200/build.py --debug
// writes libfgc_b200_debug.so).  FGC_DBG_OK(cond, status_ptr) is `true` in a normal build.  In
// the debug build it evaluates cond and, when it does not hold, sets FGC_STATUS_DEBUG_BOUNDS in
// the status word and yields false, so that the caller skips the access: a bad index is
// recorded and reported through fgc_read_status instead of becoming a memory fault.
#ifdef FGC_DEBUG
#define FGC_DBG_OK(cond, status_ptr) ((cond) ? true : (atomicOr((int *)(status_ptr), FGC_STATUS_DEBUG_BOUNDS), false))
#else
#define FGC_DBG_OK(cond, status_ptr) (true)
#endif

namespace fgc {

// NVTX range around an entry point (header-only NVTX 3: a no-op unless a profiler is attached).
struct NvtxRange {
    explicit NvtxRange(const char *name) { nvtxRangePushA(name); }
    ~NvtxRange() { nvtxRangePop(); }
    NvtxRange(const NvtxRange &) = delete;
    NvtxRange &operator=(const NvtxRange &) = delete;
};
#define FGC_NVTX(name) fgc::NvtxRange fgc_nvtx_range_(name)

// Number of SMs of the current device (148 on a B200), asked once per device and kept.  Grids of
// grid-stride kernels are sized in multiples of it.  A failed query falls back to 148 so that no
// launch path has to handle an error here.
inline int sm_count()
{
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    int n = cached[dev];
    if (n == 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;   // racing writers store the same value
    }
    return n;
}

__host__ __device__ inline int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }
inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// Monotone float -> uint32 key (total order incl. negatives) for atomicMax/Min.
__device__ __forceinline__ uint32_t float_to_ordered(float f)
{
    uint32_t b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__host__ __device__ __forceinline__ float ordered_to_float(uint32_t k)
{
    uint32_t b = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
#ifdef __CUDA_ARCH__
    return __uint_as_float(b);
#else
    union { uint32_t u; float f; } cv;
    cv.u = b;
    return cv.f;
#endif
}

__device__ __forceinline__ bool is_finite_bits(float f)
{
    return (__float_as_uint(f) & 0x7f800000u) != 0x7f800000u;
}

__device__ __forceinline__ uint32_t lanemask_lt()
{
    uint32_t m;
    asm("mov.u32 %0, %%lanemask_lt;" : "=r"(m));
    return m;
}
__device__ __forceinline__ uint32_t lanemask_le()
{
    uint32_t m;
    asm("mov.u32 %0, %%lanemask_le;" : "=r"(m));
    return m;
}

// Two fp32 values in one 64-bit register pair for the packed fp32x2 instructions of sm_100
// (add / sub / mul / fma.rn.f32x2: two IEEE operations per instruction, same rounding as the
// scalar forms).  Worth it where the operands are pairs already (the distance evaluation of the
// search: -3 to -8 %); in the register-tiled projection kernels the packed fma measured slower than
// scalar fmaf (backward 0.58 -> 0.71 ms), so they keep the scalar form.
__device__ __forceinline__ unsigned long long pack_f32x2(float a, float b)
{
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void unpack_f32x2(unsigned long long v, float &a, float &b)
{
    asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
// Programmatic dependent launch (sm_90+): a kernel launched with launch_chained() may be scheduled
// while its predecessor in the stream still runs; its CTAs then sit in chain_wait() until the
// predecessor has finished and its writes are visible.  A predecessor lets that happen by calling
// chain_release() (every CTA, as early as it likes).  Both are no-ops for a kernel launched the
// plain way or without a kernel in front of it.  Used for chains of short kernels, where the
// launch latency of each link is a tenth of its run time.
__device__ __forceinline__ void chain_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void chain_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Index of the row split that contains point v: number of entries rs[1..] <= v
// (what the reference finds by a linear scan, bin_by_coordinates_cpu.cpp:68-74).
__device__ __forceinline__ int row_split_of(const int64_t *__restrict__ rs, int n_rs, int64_t v)
{
    int lo = 1, hi = n_rs;  // first index in [1, n_rs) with rs[idx] > v
    while (lo < hi) {
        int mid = (lo + hi) >> 1;
        if (rs[mid] > v) hi = mid; else lo = mid + 1;
    }
    return lo - 1;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                  Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace fgc
