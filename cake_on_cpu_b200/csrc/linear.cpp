// PyTorch extension `linear_cpp`: the linear layer of the reference's binding
// (reference src/linear.cpp:12-107, used by python/cake.py:18-49) on this library.
//
//   forward ([cache_sz,] input, weight, bias)               -> output
//   backward([cache_sz,] grad_output, input, weight, bias)  -> {grad_input, grad_weight, grad_bias}
//
// Both call forms of the reference exist: its C++ source takes a leading `cache_sz`
// tensor [L2, L3] (src/linear.cpp:12,52) while its Python module calls without it
// (python/cake.py:22,29).  Here `cache_sz` only feeds cake_query_cntx_torch, as there.
//
// CPU tensors go through cake_sgemm of include/cake.h with host pointers, product for
// product as in the reference (y = x W^T, dX = dY W, dW = dY^T X; the transposed operands
// are made contiguous first, src/linear.cpp:22,76-80).  CUDA tensors never leave the
// device: the same three products run through cakeb200_sgemm_ex on the current stream,
// with W and dY read transposed where they lie and the bias added in the epilogue.
#include <torch/extension.h>

#include <c10/cuda/CUDAStream.h>

#include <vector>

#include "cake.h"

namespace {

void check_f32_2d(const torch::Tensor& t, const char* name) {
    TORCH_CHECK(t.dim() == 2, name, " must be 2-D");
    TORCH_CHECK(t.scalar_type() == torch::kFloat32, name, " must be float32");
}

// C (M x N) = op(A) op(B) (+ bias) on tensors of one device
torch::Tensor product(const torch::Tensor& A, bool trans_a, const torch::Tensor& B, bool trans_b, const torch::Tensor& bias,
                      cake_cntx_t* cntx) {
    const int M = (int) (trans_a ? A.size(1) : A.size(0)), K = (int) (trans_a ? A.size(0) : A.size(1));
    const int N = (int) (trans_b ? B.size(0) : B.size(1));
    TORCH_CHECK((trans_b ? B.size(1) : B.size(0)) == K, "inner dimensions differ");
    auto C = torch::empty({M, N}, A.options());
    if (A.is_cuda()) {
        auto a = A.contiguous(), b = B.contiguous();
        const float* bias_p = bias.defined() ? bias.contiguous().data_ptr<float>() : nullptr;
        const int rc = cakeb200_sgemm_ex(a.data_ptr<float>(), (int) a.size(1), trans_a, b.data_ptr<float>(), (int) b.size(1), trans_b,
                                         C.data_ptr<float>(), N, M, N, K, bias_p, 0, CAKEB200_SCHED_NA, CAKEB200_KERNEL_AUTO,
                                         c10::cuda::getCurrentCUDAStream().stream());
        TORCH_CHECK(rc == CAKEB200_OK, "cakeb200_sgemm_ex: ", cakeb200_last_error());
        return C;
    }
    // host tensors: row-major contiguous operands, as cake_sgemm expects them
    auto a = (trans_a ? A.t() : A).contiguous(), b = (trans_b ? B.t() : B).contiguous();
    const double t = cake_sgemm(a.data_ptr<float>(), b.data_ptr<float>(), C.data_ptr<float>(), M, N, K, /*p=*/1, cntx);
    TORCH_CHECK(t >= 0, "cake_sgemm: ", cakeb200_last_error());
    if (bias.defined()) C.add_(bias);
    return C;
}

cake_cntx_t* context_from(const c10::optional<torch::Tensor>& cache_sz) {
    if (cache_sz.has_value() && cache_sz->defined() && cache_sz->numel() >= 2) {
        auto c = cache_sz->to(torch::kCPU).to(torch::kInt);
        return cake_query_cntx_torch(c[0].item<int>(), c[1].item<int>());
    }
    return cake_query_cntx();
}

torch::Tensor forward_impl(const c10::optional<torch::Tensor>& cache_sz, const torch::Tensor& input, const torch::Tensor& weight,
                           const c10::optional<torch::Tensor>& bias) {
    check_f32_2d(input, "input");
    check_f32_2d(weight, "weight");
    TORCH_CHECK(input.device() == weight.device(), "input and weight live on different devices");
    cake_cntx_t* cntx = context_from(cache_sz);
    torch::Tensor b = (bias.has_value() && bias->defined()) ? *bias : torch::Tensor();
    auto out = product(input, false, weight, true, b, cntx);  // y = x W^T + b
    free(cntx);
    return out;
}

std::vector<torch::Tensor> backward_impl(const c10::optional<torch::Tensor>& cache_sz, const torch::Tensor& grad_output,
                                         const torch::Tensor& input, const torch::Tensor& weight,
                                         const c10::optional<torch::Tensor>& bias) {
    check_f32_2d(grad_output, "grad_output");
    check_f32_2d(input, "input");
    check_f32_2d(weight, "weight");
    cake_cntx_t* cntx = context_from(cache_sz);
    auto grad_input = product(grad_output, false, weight, false, torch::Tensor(), cntx);  // dX = dY W
    auto grad_weight = product(grad_output, true, input, false, torch::Tensor(), cntx);   // dW = dY^T X
    free(cntx);
    torch::Tensor grad_bias = (bias.has_value() && bias->defined()) ? grad_output.sum(0, /*keepdim=*/false) : torch::Tensor();
    return {grad_input, grad_weight, grad_bias};
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    namespace py = pybind11;
    // the call form of python/cake.py:22,29
    m.def("forward",
          [](const torch::Tensor& input, const torch::Tensor& weight, const c10::optional<torch::Tensor>& bias) {
              // three tensors of which the first is 1-D and the last 2-D: (cache_sz, input, weight) without a bias
              if (input.dim() == 1 && weight.dim() == 2 && bias.has_value() && bias->defined() && bias->dim() == 2)
                  return forward_impl(input, weight, *bias, c10::nullopt);
              return forward_impl(c10::nullopt, input, weight, bias);
          },
          "linear forward", py::arg("input"), py::arg("weight"), py::arg("bias") = py::none());
    m.def("backward",
          [](const torch::Tensor& grad_output, const torch::Tensor& input, const torch::Tensor& weight,
             const c10::optional<torch::Tensor>& bias) { return backward_impl(c10::nullopt, grad_output, input, weight, bias); },
          "linear backward", py::arg("grad_output"), py::arg("input"), py::arg("weight"), py::arg("bias") = py::none());
    // the call form of src/linear.cpp:12,52 (leading tensor [L2, L3])
    m.def("forward",
          [](const torch::Tensor& cache_sz, const torch::Tensor& input, const torch::Tensor& weight,
             const c10::optional<torch::Tensor>& bias) { return forward_impl(cache_sz, input, weight, bias); },
          "linear forward with cache sizes", py::arg("cache_sz"), py::arg("input"), py::arg("weight"), py::arg("bias") = py::none());
    m.def("backward",
          [](const torch::Tensor& cache_sz, const torch::Tensor& grad_output, const torch::Tensor& input, const torch::Tensor& weight,
             const c10::optional<torch::Tensor>& bias) { return backward_impl(cache_sz, grad_output, input, weight, bias); },
          "linear backward with cache sizes", py::arg("cache_sz"), py::arg("grad_output"), py::arg("input"), py::arg("weight"),
          py::arg("bias") = py::none());
}
