// index_replacer for sm_100a: out[i] = in[i] < 0 ? in[i]
//                                   : in[i] >= n_repl ? repl[i] : repl[in[i]]
// (extensions/index_replacer_cpu.cpp:7-26, extensions/index_replacer_cuda_kernel.cu:9-28).
// The out-of-range branch indexes the table by the element's POSITION, as the
// reference does; where that position lies beyond the table (the reference
// would read out of bounds there) the input value is kept.
#include "fgc_common.cuh"

namespace fgc {

__global__ void __launch_bounds__(256)
k_index_replacer(const int64_t *__restrict__ in, int64_t n, const int64_t *__restrict__ repl,
                 int64_t n_repl, int64_t *__restrict__ out)
{
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const int64_t r = in[i];
        int64_t o = r;
        if (r >= 0) {
            if (r < n_repl) o = __ldg(repl + r);
            else if (i < n_repl) o = __ldg(repl + i);
        }
        out[i] = o;
    }
}

}  // namespace fgc

extern "C" int fgc_index_replacer(const int64_t *to_be_replaced, int64_t n,
                                  const int64_t *replacements, int64_t n_replacements,
                                  int64_t *out, fgc_stream_t stream)
{
    FGC_NVTX("fgc_index_replacer");
    if (n < 0 || n_replacements < 0) return FGC_ERR_BAD_ARGUMENT;
    if (n == 0) return FGC_OK;
    if (!to_be_replaced || !out || (n_replacements > 0 && !replacements)) return FGC_ERR_BAD_ARGUMENT;
    int64_t blocks = fgc::ceil_div64(n, 256 * 4);
    if (blocks > fgc::sm_count() * 16) blocks = fgc::sm_count() * 16;
    if (blocks < 1) blocks = 1;
    fgc::k_index_replacer<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
        to_be_replaced, n, replacements, n_replacements, out);
    FGC_CHECK_LAUNCH();
    return FGC_OK;
}
