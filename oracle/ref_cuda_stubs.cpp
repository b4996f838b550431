// TEST INFRASTRUCTURE ONLY (oracle side).
//
// The reference's CPU-only source list does not link on its own: its autograd
// orchestrator (fastgraphcompute/extensions/binned_knn_autograd_kernel.cpp:16-52)
// and its binning host wrapper (fastgraphcompute/extensions/bin_by_coordinates.cpp:14-19)
// name four *_cuda_fn symbols unconditionally (and select_knn.cpp:14-21 a fifth,
// select_knn_cuda_fn).  This file defines those
// symbols so that the reference's CPU path can be loaded on a host without the
// reference's CUDA objects.  Each one refuses to run.
#include <torch/extension.h>
#include <tuple>

std::tuple<torch::Tensor, torch::Tensor> binned_select_knn_cuda_fn(
    torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor,
    torch::Tensor, torch::Tensor, bool, bool, int64_t) {
    TORCH_CHECK(false, "oracle build: reference CUDA kNN kernel is not part of the CPU oracle");
    return {};
}

torch::Tensor index_replacer_cuda_fn(torch::Tensor, torch::Tensor) {
    TORCH_CHECK(false, "oracle build: reference CUDA index_replacer is not part of the CPU oracle");
    return {};
}

torch::Tensor binned_select_knn_grad_cuda_fn(torch::Tensor, torch::Tensor, torch::Tensor,
                                             torch::Tensor) {
    TORCH_CHECK(false, "oracle build: reference CUDA kNN gradient is not part of the CPU oracle");
    return {};
}

std::tuple<torch::Tensor, torch::Tensor, torch::Tensor> bin_by_coordinates_cuda_fn(
    torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor, bool) {
    TORCH_CHECK(false, "oracle build: reference CUDA binning kernel is not part of the CPU oracle");
    return {};
}

std::tuple<torch::Tensor, torch::Tensor> select_knn_cuda_fn(torch::Tensor, torch::Tensor, torch::Tensor,
                                                            int64_t, double, int64_t) {
    TORCH_CHECK(false, "oracle build: reference CUDA select_knn kernel is not part of the CPU oracle");
    return {};
}
