// Version and error text of libfgc_b200.
#include "fgc_common.cuh"

extern "C" int fgc_version(void) { return 100; /* 0.1.0 */ }

extern "C" const char *fgc_error_string(int code)
{
    switch (code) {
    case FGC_OK: return "ok";
    case FGC_ERR_BAD_ARGUMENT: return "bad argument (null pointer, negative size or inconsistent lengths)";
    case FGC_ERR_UNSUPPORTED_DIM: return "unsupported number of coordinate dimensions (the kNN needs 2..16)";
    case FGC_ERR_UNSUPPORTED_K: return "unsupported K (1..257)";
    case FGC_ERR_WORKSPACE: return "workspace missing, too small or not 256-byte aligned";
    case FGC_ERR_TOO_LARGE: return "problem too large for 32-bit point / cell indices";
    case FGC_ERR_STATIC_TOO_LARGE: return "problem too large for the built-in scratch area of fgc_binned_knn_fwd_static";
    default: break;
    }
    if (code > 0) return cudaGetErrorString((cudaError_t)code);
    return "unknown error";
}
