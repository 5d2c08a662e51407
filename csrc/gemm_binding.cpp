// Torch-facing functions of the tcgen05 GEMM family (standalone GEMM here; the
// fused GEMM -> reduce-scatter and all-gather -> GEMM are bound next to the
// communicator because they need its heap).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <pybind11/pybind11.h>
#include <torch/extension.h>

#include "gemm_decode_sm100.h"
#include "pdl.h"
#include "gemm_sm100.h"

namespace py = pybind11;

namespace {
// One error word per device, zeroed at creation; a non-zero value means a
// pipeline wait ran out inside a GEMM kernel.
at::Tensor& error_word() {
  static std::vector<at::Tensor> words(64);
  int dev = 0;
  cudaGetDevice(&dev);
  if (!words[dev].defined())
    words[dev] = torch::zeros({4}, torch::TensorOptions().dtype(torch::kInt32).device(torch::kCUDA, dev));
  return words[dev];
}
}  // namespace

uint32_t* penny_gemm_error_word() { return reinterpret_cast<uint32_t*>(error_word().data_ptr<int>()); }

void bind_gemm(py::module_& m) {
  // out[M, N] = a[M, K] @ b[N, K]^T (the nn.Linear convention: b is the weight)
  m.def("gemm_bf16", [](at::Tensor a, at::Tensor b, at::Tensor out, int64_t block_n) {
    TORCH_CHECK(a.is_cuda() && b.is_cuda() && out.is_cuda(), "gemm_bf16: CUDA tensors");
    TORCH_CHECK(a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16 &&
                    out.scalar_type() == at::kBFloat16, "gemm_bf16: bf16 only");
    TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && out.dim() == 2, "gemm_bf16: 2-D tensors");
    TORCH_CHECK(a.stride(1) == 1 && b.stride(1) == 1 && out.stride(1) == 1, "gemm_bf16: rows must be contiguous");
    const int64_t M = a.size(0), K = a.size(1), N = b.size(0);
    TORCH_CHECK(b.size(1) == K && out.size(0) == M && out.size(1) == N, "gemm_bf16: shape mismatch");
    const at::cuda::OptionalCUDAGuard guard(a.device());
    cudaError_t rc = penny::sm100::launch_gemm_bf16(
        a.data_ptr(), b.data_ptr(), out.data_ptr(), (int)M, (int)N, (int)K, (int)a.stride(0), (int)b.stride(0),
        (int)out.stride(0), (int)block_n, penny_gemm_error_word(), at::cuda::getCurrentCUDAStream().stream());
    TORCH_CHECK(rc == cudaSuccess, "gemm_bf16: ", cudaGetErrorString(rc));
  }, py::arg("a"), py::arg("b"), py::arg("out"), py::arg("block_n") = 0);
  // Decode-batch linear: out[B, N] = x[B, K] @ w[N, K]^T for B <= 1024 (slabs of 128 rows in one launch).  One CTA per (weight tile, K
  // range); the K ranges of a tile are reduced inside a thread-block cluster through distributed shared
  // memory.  pdl: may start (and load w) while the previous kernel on the stream still runs, so w must not
  // be written by that kernel.  silu_pairs: w's rows are blocks of 64 gate + 64 up rows and out is
  // [B, N / 2] = silu(gate) * up.
  m.def("gemm_decode", [](at::Tensor x, at::Tensor w, at::Tensor out, bool silu_pairs, int64_t splits, bool pdl,
                          int64_t l2_budget, int64_t smem_kb, c10::optional<at::Tensor> push) {
    TORCH_CHECK(x.is_cuda() && w.is_cuda() && out.is_cuda(), "gemm_decode: CUDA tensors");
    TORCH_CHECK(x.scalar_type() == at::kBFloat16 && w.scalar_type() == at::kBFloat16 &&
                    out.scalar_type() == at::kBFloat16, "gemm_decode: bf16 only");
    TORCH_CHECK(x.dim() == 2 && w.dim() == 2 && out.dim() == 2, "gemm_decode: 2-D tensors");
    TORCH_CHECK(x.stride(1) == 1 && w.stride(1) == 1 && out.stride(1) == 1, "gemm_decode: rows must be contiguous");
    const int64_t B = x.size(0), K = x.size(1), N = w.size(0);
    TORCH_CHECK(B >= 1 && B <= penny::sm100::kDecodeMaxBatch, "gemm_decode: 1 <= rows of x <= 1024 (use gemm_bf16 beyond)");
    TORCH_CHECK(!push.has_value() || B <= 128, "gemm_decode: push needs rows of x <= 128");
    TORCH_CHECK(w.size(1) == K && out.size(0) == B && out.size(1) == (silu_pairs ? N / 2 : N),
                "gemm_decode: shape mismatch");
    TORCH_CHECK(splits >= 0 && splits <= 8, "gemm_decode: 0 <= splits <= 8");
    const at::cuda::OptionalCUDAGuard guard(x.device());
    // push: the bytes of a DecodePush from comm_fused_norm_push_target (rows other ranks own go to them)
    penny::sm100::DecodePush pd;
    const penny::sm100::DecodePush* pp = nullptr;
    if (push.has_value()) {
      TORCH_CHECK(push->device().is_cpu() && push->scalar_type() == at::kByte && push->is_contiguous() &&
                      push->numel() == (int64_t)sizeof(pd), "gemm_decode: push must come from comm_fused_norm_push_target");
      memcpy(&pd, push->data_ptr(), sizeof(pd));
      pp = &pd;
    }
    cudaError_t rc = penny::sm100::launch_gemm_decode(
        x.data_ptr(), w.data_ptr(), out.data_ptr(), (int)B, (int)N, (int)K, (int)x.stride(0), (int)w.stride(0),
        (int)out.stride(0), silu_pairs ? 1 : 0, (int)splits, pdl, (long long)l2_budget, (int)smem_kb, pp,
        penny_gemm_error_word(),
        at::cuda::getCurrentCUDAStream().stream());
    TORCH_CHECK(rc == cudaSuccess, "gemm_decode: ", cudaGetErrorString(rc));
  }, py::arg("x"), py::arg("w"), py::arg("out"), py::arg("silu_pairs") = false, py::arg("splits") = 0,
     py::arg("pdl") = true, py::arg("l2_budget") = -1, py::arg("smem_kb") = 0, py::arg("push") = py::none());
  m.def("gemm_decode_splits", [](int64_t B, int64_t N, int64_t K) {
    return penny::sm100::gemm_decode_splits((int)B, (int)N, (int)K);
  });
  m.def("gemm_decode_capacity", [](int64_t B, int64_t splits) {
    return penny::sm100::gemm_decode_capacity((int)B, (int)splits);
  });
  m.def("gemm_decode_stamps", [](int64_t max_ctas) {
    auto t = torch::zeros({max_ctas, 8}, torch::TensorOptions().dtype(torch::kInt64));
    cudaDeviceSynchronize();
    const int n = penny::sm100::gemm_decode_stamps(reinterpret_cast<unsigned long long*>(t.data_ptr<int64_t>()), (int)max_ctas);
    return t.narrow(0, 0, n);
  }, py::arg("max_ctas") = 512, "timestamps of the last gemm_decode launch (needs PENNY_DEC_STAMPS=1)");
  m.def("set_pdl", [](int64_t on) { penny::set_pdl_enabled((int)on); }, py::arg("on"),
        "1 / 0: launch this library's decode kernels with / without programmatic dependent launch; -1: PENNY_PDL decides");
  m.def("pdl_enabled", []() { return penny::pdl_enabled(); });
  m.def("gemm_set_split_tail", [](int64_t on) { penny::sm100::set_split_tail((int)on); }, py::arg("on"),
        "1 / 0: split (or not) the ragged last wave of the CTA-pair GEMM along K; -1: PENNY_GEMM_SPLIT_TAIL decides");
  // Synchronises; returns and clears the error code of the GEMM kernels (0 = fine).
  m.def("gemm_error", []() {
    at::Tensor& w = error_word();
    int v = w[0].item<int>();
    if (v != 0) w.zero_();
    return v;
  });
}
