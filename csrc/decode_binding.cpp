// Torch-facing wrappers of the decode-step kernels.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <pybind11/pybind11.h>
#include <torch/extension.h>

#include "decode_kernels.h"
#include "moe_routing.h"

namespace py = pybind11;
using namespace penny;

namespace {
cudaStream_t cur() { return at::cuda::getCurrentCUDAStream().stream(); }
void need(bool ok, const char* msg) { TORCH_CHECK(ok, "penny: ", msg); }
void ck(cudaError_t rc, const char* what) {
  TORCH_CHECK(rc == cudaSuccess, "penny: ", what, ": ", cudaGetErrorString(rc));
}
bool bf16_cuda(const at::Tensor& t) {
  return t.is_cuda() && t.is_contiguous() && t.scalar_type() == at::kBFloat16;
}
}  // namespace

void bind_decode(py::module_& m) {
  m.def("rope_append", [](at::Tensor qkv, at::Tensor kcache, at::Tensor vcache, at::Tensor positions,
                          int64_t Hq, int64_t Hkv, int64_t D, double theta) {
    need(bf16_cuda(qkv) && bf16_cuda(kcache) && bf16_cuda(vcache), "rope_append expects contiguous bf16 CUDA tensors");
    need(positions.is_cuda() && positions.scalar_type() == at::kInt && positions.is_contiguous(), "positions must be int32 CUDA");
    need(qkv.dim() == 2 && qkv.size(1) == (Hq + 2 * Hkv) * D, "qkv must be [B, (Hq + 2 Hkv) D]");
    need(kcache.dim() == 4 && kcache.size(0) == qkv.size(0) && kcache.size(1) == Hkv && kcache.size(3) == D &&
             vcache.sizes() == kcache.sizes(), "caches must be [B, Hkv, max_len, D]");
    need(positions.numel() == qkv.size(0), "one position per row");
    const at::cuda::OptionalCUDAGuard guard(qkv.device());
    ck(launch_rope_append(qkv.data_ptr(), kcache.data_ptr(), vcache.data_ptr(), positions.data_ptr<int>(),
                          (int)qkv.size(0), (int)Hq, (int)Hkv, (int)D, (int)kcache.size(2), (float)theta, cur()),
       "rope_append");
  });
  m.def("rope_rows", [](at::Tensor qkv, int64_t Hq, int64_t Hkv, int64_t D, int64_t pos0, double theta) {
    need(bf16_cuda(qkv) && qkv.dim() == 2 && qkv.size(1) == (Hq + 2 * Hkv) * D, "rope_rows expects [T, (Hq + 2 Hkv) D] bf16");
    const at::cuda::OptionalCUDAGuard guard(qkv.device());
    ck(launch_rope_rows(qkv.data_ptr(), (int)qkv.size(0), (int)Hq, (int)Hkv, (int)D, (int)pos0, (float)theta, cur()),
       "rope_rows");
  });
  m.def("decode_attn_workspace_bytes", [](int64_t B, int64_t Hq, int64_t splits) {
    return (int64_t)decode_attn_workspace_bytes((int)B, (int)Hq, (int)splits);
  });
  m.def("decode_attention", [](at::Tensor qkv, at::Tensor kcache, at::Tensor vcache, at::Tensor positions,
                               at::Tensor out, at::Tensor workspace, int64_t Hq, int64_t Hkv, int64_t splits,
                               double scale) {
    need(bf16_cuda(qkv) && bf16_cuda(kcache) && bf16_cuda(vcache) && bf16_cuda(out), "decode_attention expects contiguous bf16 CUDA tensors");
    need(positions.is_cuda() && positions.scalar_type() == at::kInt, "positions must be int32 CUDA");
    const int64_t B = qkv.size(0), D = kcache.size(3);
    need(qkv.size(1) == (Hq + 2 * Hkv) * D && out.numel() == B * Hq * D, "decode_attention shapes");
    need(workspace.is_cuda() && (int64_t)workspace.nbytes() >= (int64_t)decode_attn_workspace_bytes((int)B, (int)Hq, (int)splits),
         "workspace too small (decode_attn_workspace_bytes)");
    need(((uintptr_t)workspace.data_ptr() & 15) == 0, "workspace must be 16-byte aligned");
    const at::cuda::OptionalCUDAGuard guard(qkv.device());
    ck(launch_decode_attention(qkv.data_ptr(), kcache.data_ptr(), vcache.data_ptr(), positions.data_ptr<int>(),
                               out.data_ptr(), workspace.data_ptr(), (int)B, (int)Hq, (int)Hkv, (int)D,
                               (int)kcache.size(2), (int)splits, (float)scale, cur()),
       "decode_attention");
  });
  m.def("decode_attn_fused_workspace_bytes", [](int64_t B, int64_t Hq, int64_t Hkv, int64_t splits) {
    return (int64_t)decode_attn_fused_workspace_bytes((int)B, (int)Hq, (int)Hkv, (int)splits);
  });
  // rope + KV append + split-KV attention + merge in one launch; qkv is the raw projection of the new token
  m.def("decode_attention_fused", [](at::Tensor qkv, at::Tensor kcache, at::Tensor vcache, at::Tensor positions,
                                     at::Tensor out, at::Tensor workspace, int64_t Hq, int64_t Hkv, int64_t splits,
                                     double scale, double theta, bool pdl) {
    need(bf16_cuda(qkv) && bf16_cuda(kcache) && bf16_cuda(vcache) && bf16_cuda(out), "decode_attention_fused expects contiguous bf16 CUDA tensors");
    need(positions.is_cuda() && positions.scalar_type() == at::kInt && positions.is_contiguous(), "positions must be int32 CUDA");
    need(kcache.dim() == 4 && vcache.sizes() == kcache.sizes(), "caches must be [B, Hkv, max_len, D]");
    const int64_t B = qkv.size(0), D = kcache.size(3);
    need(qkv.dim() == 2 && qkv.size(1) == (Hq + 2 * Hkv) * D && out.numel() == B * Hq * D && kcache.size(0) == B &&
             kcache.size(1) == Hkv && positions.numel() == B, "decode_attention_fused shapes");
    need(workspace.is_cuda() && (int64_t)workspace.nbytes() >=
                                    (int64_t)decode_attn_fused_workspace_bytes((int)B, (int)Hq, (int)Hkv, (int)splits),
         "workspace too small (decode_attn_fused_workspace_bytes)");
    need(((uintptr_t)workspace.data_ptr() & 15) == 0, "workspace must be 16-byte aligned");
    const at::cuda::OptionalCUDAGuard guard(qkv.device());
    ck(launch_decode_attention_fused(qkv.data_ptr(), kcache.data_ptr(), vcache.data_ptr(), positions.data_ptr<int>(),
                                     out.data_ptr(), workspace.data_ptr(), (int)B, (int)Hq, (int)Hkv, (int)D,
                                     (int)kcache.size(2), (int)splits, (float)scale, (float)theta, pdl, cur()),
       "decode_attention_fused");
  }, py::arg("qkv"), py::arg("kcache"), py::arg("vcache"), py::arg("positions"), py::arg("out"), py::arg("workspace"),
     py::arg("Hq"), py::arg("Hkv"), py::arg("splits"), py::arg("scale"), py::arg("theta"), py::arg("pdl") = true);
  m.def("silu_mul", [](at::Tensor gate_up, at::Tensor out) {
    need(bf16_cuda(gate_up) && bf16_cuda(out) && gate_up.dim() == 2, "silu_mul expects [rows, 2F] bf16");
    const int64_t rows = gate_up.size(0), F = gate_up.size(1) / 2;
    need(out.numel() == rows * F, "silu_mul output must be [rows, F]");
    const at::cuda::OptionalCUDAGuard guard(gate_up.device());
    ck(launch_silu_mul(gate_up.data_ptr(), out.data_ptr(), (int)rows, (int)F, cur()), "silu_mul");
  });
  m.def("argmax_workspace_bytes", [](int64_t rows) { return (int64_t)argmax_workspace_bytes((int)rows); });
  m.def("argmax_rows", [](at::Tensor logits, at::Tensor out_val, at::Tensor out_idx, int64_t index_base,
                          c10::optional<at::Tensor> workspace, c10::optional<at::Tensor> pair) {
    need(bf16_cuda(logits) && logits.dim() == 2, "argmax_rows expects [rows, cols] bf16");
    const int64_t rows = logits.size(0);
    need(out_val.is_cuda() && out_val.scalar_type() == at::kFloat && out_val.numel() == rows, "out_val [rows] fp32");
    need(out_idx.is_cuda() && out_idx.scalar_type() == at::kLong && out_idx.numel() == rows, "out_idx [rows] int64");
    void* ws = nullptr;
    if (workspace.has_value()) {
      need(workspace->is_cuda() && workspace->is_contiguous() &&
               (int64_t)workspace->nbytes() >= (int64_t)argmax_workspace_bytes((int)rows),
           "workspace too small (argmax_workspace_bytes) or not contiguous; it must be zeroed once");
      ws = workspace->data_ptr();
    }
    float* pp = nullptr;
    if (pair.has_value()) {
      need(pair->is_cuda() && pair->scalar_type() == at::kFloat && pair->is_contiguous() && pair->numel() == 2 * rows,
           "pair [2 * rows] fp32");
      pp = pair->data_ptr<float>();
    }
    const at::cuda::OptionalCUDAGuard guard(logits.device());
    ck(launch_argmax(logits.data_ptr(), (int)rows, (int)logits.size(1), out_val.data_ptr<float>(),
                     (long long*)out_idx.data_ptr<int64_t>(), pp, (long long)index_base, ws, cur()),
       "argmax_rows");
  }, py::arg("logits"), py::arg("out_val"), py::arg("out_idx"), py::arg("index_base"),
     py::arg("workspace") = py::none(), py::arg("pair") = py::none());
  // Expert-parallel MoE routing on the device (csrc/moe_routing.cu)
  m.def("moe_route", [](at::Tensor logits, int64_t topk) {
    need(bf16_cuda(logits) && logits.dim() == 2, "moe_route expects [tokens, experts] bf16");
    const int64_t T = logits.size(0), E = logits.size(1);
    const at::cuda::OptionalCUDAGuard guard(logits.device());
    at::Tensor ids = at::empty({T, topk}, logits.options().dtype(at::kInt));
    at::Tensor gates = at::empty({T, topk}, logits.options().dtype(at::kFloat));
    ck(launch_moe_topk(logits.data_ptr(), (int)T, (int)E, (int)topk, ids.data_ptr<int>(), gates.data_ptr<float>(), cur()),
       "moe_route");
    return std::make_tuple(ids, gates);
  });
  m.def("moe_tables", [](at::Tensor ids, int64_t experts) {
    need(ids.is_cuda() && ids.scalar_type() == at::kInt && ids.is_contiguous(), "moe_tables expects contiguous int32 ids");
    const int64_t P = ids.numel();
    const at::cuda::OptionalCUDAGuard guard(ids.device());
    auto opt = ids.options();
    at::Tensor order = at::empty({P}, opt), sorted = at::empty({P}, opt), send_off = at::empty({experts + 1}, opt),
               counts = at::empty({experts}, opt);
    ck(launch_moe_tables(ids.data_ptr<int>(), (int)P, (int)experts, order.data_ptr<int>(), sorted.data_ptr<int>(),
                         send_off.data_ptr<int>(), counts.data_ptr<int>(), cur()),
       "moe_tables");
    return std::make_tuple(order, sorted, send_off, counts);
  });
  m.def("moe_placement", [](at::Tensor counts_all) {
    need(counts_all.is_cuda() && counts_all.scalar_type() == at::kInt && counts_all.is_contiguous() &&
             counts_all.dim() == 2,
         "moe_placement expects [world, experts] int32");
    const int64_t W = counts_all.size(0), E = counts_all.size(1);
    const at::cuda::OptionalCUDAGuard guard(counts_all.device());
    auto opt = counts_all.options();
    at::Tensor dst_base = at::empty({W, E}, opt), rows = at::empty({W}, opt), ranges = at::empty({E, 2}, opt);
    ck(launch_moe_placement(counts_all.data_ptr<int>(), (int)W, (int)E, dst_base.data_ptr<int>(), rows.data_ptr<int>(),
                            ranges.data_ptr<int>(), cur()),
       "moe_placement");
    return std::make_tuple(dst_base, rows, ranges);
  });
  m.def("sample_finish", [](at::Tensor pairs, int64_t world, at::Tensor next_tokens, at::Tensor tokens,
                            at::Tensor positions) {
    const int64_t B = next_tokens.numel();
    need(pairs.is_cuda() && pairs.scalar_type() == at::kFloat && pairs.is_contiguous() && pairs.numel() == world * 2 * B,
         "pairs [world, 2, B] fp32");
    need(next_tokens.scalar_type() == at::kLong && tokens.scalar_type() == at::kLong && tokens.numel() == B &&
             positions.scalar_type() == at::kInt && positions.numel() == B && next_tokens.is_cuda() &&
             tokens.is_cuda() && positions.is_cuda(),
         "next_tokens / tokens [B] int64, positions [B] int32");
    const at::cuda::OptionalCUDAGuard guard(pairs.device());
    ck(launch_sample_finish(pairs.data_ptr<float>(), (int)world, (int)B, (long long*)next_tokens.data_ptr<int64_t>(),
                            (long long*)tokens.data_ptr<int64_t>(), positions.data_ptr<int>(), cur()),
       "sample_finish");
  });

}
