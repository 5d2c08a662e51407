// Torch-facing functions of the custom all-reduce family.  Names, argument
// order and return types follow the reference's penny_cpp module
// (csrc/torch_interface.cpp:118-140, csrc/custom_all_reduce.cu:14-301) so that
// vLLM / SGLang style callers work unchanged.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>
#include <torch/extension.h>

#include "custom_all_reduce.cuh"

namespace py = pybind11;
using penny::pull::CustomAllreduce;
using fptr_t = int64_t;

namespace {

int dtype_of(const at::Tensor& t) {
  switch (t.scalar_type()) {
    case at::kFloat: return penny::DT_F32;
    case at::kHalf: return penny::DT_F16;
    case at::kBFloat16: return penny::DT_BF16;
    default: TORCH_CHECK(false, "custom allreduce only supports float32, float16 and bfloat16");
  }
}

// Dense in memory from its first element on, even if not contiguous in the
// torch sense (e.g. a slice that runs to the end of its storage).
bool is_weak_contiguous(const at::Tensor& t) {
  if (t.is_contiguous()) return true;
  const int64_t tail = (int64_t)t.storage().nbytes() - t.storage_offset() * (int64_t)t.element_size();
  return tail == t.numel() * (int64_t)t.element_size();
}

// The pull kernels move 16-byte vectors: a dense slice that starts off a 16-byte
// boundary (buf[3:] of a bf16 tensor) must be refused on the host, where it is an
// exception, not on the device, where it would be a misaligned-address fault.
void check_aligned16(const at::Tensor& t, const char* what) {
  TORCH_CHECK((reinterpret_cast<uintptr_t>(t.data_ptr()) & 15u) == 0, "custom allreduce: ", what,
              " must start on a 16-byte boundary (storage offset ", t.storage_offset(), ")");
}

CustomAllreduce* as_fa(fptr_t p) {
  TORCH_CHECK(p != 0, "custom allreduce: null handle");
  return reinterpret_cast<CustomAllreduce*>(p);
}

// Shared prologue of the three collectives: optional staging copy into the
// pre-registered buffer (eager mode), like csrc/custom_all_reduce.cu:63-81.
const void* stage_input(const at::Tensor& inp, fptr_t reg_buffer, int64_t reg_buffer_sz_bytes,
                        cudaStream_t stream) {
  if (reg_buffer == 0) return inp.data_ptr();
  const int64_t bytes = inp.numel() * (int64_t)inp.element_size();
  TORCH_CHECK(bytes <= reg_buffer_sz_bytes, "custom allreduce: input larger than the registered buffer");
  void* reg = reinterpret_cast<void*>(reg_buffer);
  cudaError_t rc = cudaMemcpyAsync(reg, inp.data_ptr(), bytes, cudaMemcpyDeviceToDevice, stream);
  TORCH_CHECK(rc == cudaSuccess, "custom allreduce: staging copy: ", cudaGetErrorString(rc));
  return reg;
}

}  // namespace

void bind_custom_all_reduce(py::module_& m) {
  m.def("init_custom_ar", [](const std::vector<fptr_t>& ipc_ptrs, at::Tensor& rank_data, int64_t rank,
                             bool fully_connected) -> fptr_t {
    const int world = (int)ipc_ptrs.size();
    TORCH_CHECK(world <= 8, "world size > 8 is not supported");
    TORCH_CHECK(world % 2 == 0, "odd numbers of GPUs are not supported");
    TORCH_CHECK(rank >= 0 && rank < world, "invalid rank");
    void* sig[8] = {};
    for (int i = 0; i < world; ++i) sig[i] = reinterpret_cast<void*>(ipc_ptrs[i]);
    return (fptr_t) new CustomAllreduce(sig, rank_data.data_ptr(), (size_t)rank_data.numel(),
                                        (int)rank, world, fully_connected);
  });

  m.def("all_reduce", [](fptr_t fa, at::Tensor& inp, at::Tensor& out, fptr_t reg_buffer,
                         int64_t reg_buffer_sz_bytes) {
    const at::cuda::OptionalCUDAGuard guard(inp.device());
    cudaStream_t stream = at::cuda::getCurrentCUDAStream().stream();
    TORCH_CHECK(inp.scalar_type() == out.scalar_type() && inp.numel() == out.numel(),
                "custom allreduce: in/out mismatch");
    TORCH_CHECK(is_weak_contiguous(inp) && is_weak_contiguous(out), "custom allreduce: tensors must be dense");
    check_aligned16(inp, "input");
    check_aligned16(out, "output");
    const void* src = stage_input(inp, reg_buffer, reg_buffer_sz_bytes, stream);
    as_fa(fa)->allreduce(dtype_of(out), stream, src, out.data_ptr(), (size_t)out.numel());
  });

  m.def("reduce_scatter", [](fptr_t fa, at::Tensor& inp, at::Tensor& out, fptr_t reg_buffer,
                             int64_t reg_buffer_sz_bytes) {
    const at::cuda::OptionalCUDAGuard guard(inp.device());
    cudaStream_t stream = at::cuda::getCurrentCUDAStream().stream();
    TORCH_CHECK(inp.scalar_type() == out.scalar_type(), "custom reduce_scatter: dtype mismatch");
    TORCH_CHECK(is_weak_contiguous(inp) && is_weak_contiguous(out), "custom reduce_scatter: tensors must be dense");
    check_aligned16(inp, "input");
    check_aligned16(out, "output");
    CustomAllreduce* f = as_fa(fa);
    // The output may be as large as the input (reference callers allocate it
    // with empty_like); the shard lands in its first numel / world elements.
    TORCH_CHECK(out.numel() * f->world() >= inp.numel(), "custom reduce_scatter: output too small");
    const void* src = stage_input(inp, reg_buffer, reg_buffer_sz_bytes, stream);
    f->reduce_scatter(dtype_of(out), stream, src, out.data_ptr(), (size_t)inp.numel());
  });

  m.def("all_gather", [](fptr_t fa, at::Tensor& inp, at::Tensor& out, fptr_t reg_buffer,
                         int64_t reg_buffer_sz_bytes) {
    const at::cuda::OptionalCUDAGuard guard(inp.device());
    cudaStream_t stream = at::cuda::getCurrentCUDAStream().stream();
    TORCH_CHECK(inp.scalar_type() == out.scalar_type(), "custom all_gather: dtype mismatch");
    TORCH_CHECK(is_weak_contiguous(inp) && is_weak_contiguous(out), "custom all_gather: tensors must be dense");
    check_aligned16(inp, "input");
    check_aligned16(out, "output");
    CustomAllreduce* f = as_fa(fa);
    TORCH_CHECK(out.numel() >= inp.numel() * f->world(), "custom all_gather: output too small");
    const void* src = stage_input(inp, reg_buffer, reg_buffer_sz_bytes, stream);
    f->all_gather(dtype_of(out), stream, src, out.data_ptr(), (size_t)inp.numel());
  });

  m.def("dispose", [](fptr_t fa) { delete reinterpret_cast<CustomAllreduce*>(fa); });
  m.def("meta_size", []() -> int64_t { return (int64_t)sizeof(penny::pull::PullSignal); });

  m.def("register_buffer", [](fptr_t fa, const std::vector<fptr_t>& ipc_ptrs) {
    CustomAllreduce* f = as_fa(fa);
    TORCH_CHECK((int)ipc_ptrs.size() == f->world(), "register_buffer: one pointer per rank");
    void* p[8] = {};
    for (size_t i = 0; i < ipc_ptrs.size(); ++i) p[i] = reinterpret_cast<void*>(ipc_ptrs[i]);
    f->register_buffer(p);
  });

  m.def("get_graph_buffer_ipc_meta", [](fptr_t fa) {
    auto meta = as_fa(fa)->get_graph_buffer_ipc_meta();
    std::vector<int64_t> bytes(meta.first.begin(), meta.first.end());
    return std::make_tuple(bytes, meta.second);
  });

  m.def("register_graph_buffers", [](fptr_t fa, const std::vector<std::vector<int64_t>>& handles,
                                     const std::vector<std::vector<int64_t>>& offsets) {
    std::vector<std::string> h;
    h.reserve(handles.size());
    for (const auto& v : handles) h.emplace_back(v.begin(), v.end());
    as_fa(fa)->register_graph_buffers(h, offsets);
  });

  m.def("custom_ar_status", [](fptr_t fa, bool clear) {
    uint32_t w[8];
    as_fa(fa)->read_status(w, clear);
    return std::vector<int64_t>(w, w + 8);
  }, py::arg("fa"), py::arg("clear") = true);
  m.def("custom_ar_set_timeout_ms", [](fptr_t fa, int ms) { as_fa(fa)->set_timeout_ms(ms); });
  m.def("custom_ar_set_max_blocks", [](fptr_t fa, int b) { as_fa(fa)->set_max_blocks(b); });

  // cudaMalloc + zero + IPC handle, usable while another stream is capturing
  // (csrc/custom_all_reduce.cu:258-289 of the reference).
  m.def("allocate_shared_buffer_and_handle", [](int64_t size) {
    auto device_index = c10::cuda::current_device();
    at::DeviceGuard device_guard(at::Device(at::DeviceType::CUDA, device_index));
    void* buffer = nullptr;
    cudaStreamCaptureMode mode = cudaStreamCaptureModeRelaxed;
    cudaStream_t stream = c10::cuda::getCurrentCUDAStream().stream();
    TORCH_CHECK(cudaThreadExchangeStreamCaptureMode(&mode) == cudaSuccess, "capture mode");
    cudaError_t rc = cudaMalloc(&buffer, (size_t)size);
    if (rc == cudaSuccess) rc = cudaMemsetAsync(buffer, 0, (size_t)size, stream);
    if (rc == cudaSuccess) rc = cudaStreamSynchronize(stream);
    cudaThreadExchangeStreamCaptureMode(&mode);
    TORCH_CHECK(rc == cudaSuccess, "allocate_shared_buffer: ", cudaGetErrorString(rc));
    auto handle = torch::empty({(int64_t)sizeof(cudaIpcMemHandle_t)},
                               torch::TensorOptions().dtype(torch::kUInt8).device(torch::kCPU));
    rc = cudaIpcGetMemHandle(reinterpret_cast<cudaIpcMemHandle_t*>(handle.data_ptr()), buffer);
    TORCH_CHECK(rc == cudaSuccess, "cudaIpcGetMemHandle: ", cudaGetErrorString(rc));
    return std::make_tuple((fptr_t)buffer, handle);
  });

  m.def("open_mem_handle", [](at::Tensor& mem_handle) -> fptr_t {
    TORCH_CHECK(mem_handle.device().is_cpu() && mem_handle.numel() == (int64_t)sizeof(cudaIpcMemHandle_t),
                "open_mem_handle: expected a 64-byte CPU tensor");
    void* p = nullptr;
    cudaError_t rc = cudaIpcOpenMemHandle(&p, *reinterpret_cast<const cudaIpcMemHandle_t*>(mem_handle.data_ptr()),
                                          cudaIpcMemLazyEnablePeerAccess);
    TORCH_CHECK(rc == cudaSuccess, "cudaIpcOpenMemHandle: ", cudaGetErrorString(rc));
    return (fptr_t)p;
  });

  m.def("free_shared_buffer", [](fptr_t buffer) {
    cudaError_t rc = cudaFree(reinterpret_cast<void*>(buffer));
    TORCH_CHECK(rc == cudaSuccess, "free_shared_buffer: ", cudaGetErrorString(rc));
  });
}
