// pybind module `penny_cpp`.
//
// Reference-compatible surface (csrc/torch_interface.cpp:66-141 of the
// reference): get_unique_id, init_with_uid, exchange, nvshmem_register,
// nvshmem_unregister, all_reduce_create / all_reduce_run / all_reduce_destroy,
// and the custom all-reduce family (init_custom_ar ... free_shared_buffer, bound
// in custom_all_reduce_binding.cpp).  The names that mention NVSHMEM keep their
// role – bootstrap token, runtime init, "make this buffer usable" – but are
// backed by the VMM/IPC symmetric heap; registration is a no-op because inputs
// are only ever read by their owner.
//
// New surface: comm_* (explicit communicators, real or single-GPU emulated,
// every algorithm, fused ops).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>
#include <torch/extension.h>

#include <cstdlib>
#include <memory>
#include <mutex>
#include <unordered_map>

#include "comm.h"
#include "schedule.h"

namespace py = pybind11;
using namespace penny;

void bind_custom_all_reduce(py::module_& m);  // custom_all_reduce_binding.cpp
void bind_gemm(py::module_& m);               // gemm_binding.cpp
void bind_decode(py::module_& m);             // decode_binding.cpp
uint32_t* penny_gemm_error_word();            // gemm_binding.cpp

namespace {

int dtype_of(const at::Tensor& t) {
  switch (t.scalar_type()) {
    case at::kFloat: return DT_F32;
    case at::kHalf: return DT_F16;
    case at::kBFloat16: return DT_BF16;
    default: TORCH_CHECK(false, "penny: unsupported dtype ", t.scalar_type(), " (fp32, fp16, bf16)");
  }
}

cudaStream_t current_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

Communicator* as_comm(int64_t h) {
  TORCH_CHECK(h != 0, "penny: null communicator handle");
  return reinterpret_cast<Communicator*>(h);
}

void check_dense(const at::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), "penny: ", name, " must be a CUDA tensor");
  TORCH_CHECK(t.is_contiguous(), "penny: ", name, " must be contiguous");
}

Tuning make_tuning(int blocks, int threads, int nnodes, int routes, bool sym_in, bool sym_out) {
  Tuning t;
  t.blocks = blocks;
  t.threads = threads;
  t.nnodes = nnodes > 0 ? nnodes : 1;
  t.routes = routes;
  t.symmetric_in = sym_in;
  t.symmetric_out = sym_out;
  return t;
}

template <class F>
void with_views(Communicator* c, const std::vector<at::Tensor>& in,
                const std::vector<at::Tensor>& out, F&& f) {
  TORCH_CHECK((int)in.size() == c->views() && (int)out.size() == c->views(),
              "penny: expected ", c->views(), " tensor(s) per argument");
  std::vector<const void*> ip(in.size());
  std::vector<void*> op(out.size());
  for (size_t i = 0; i < in.size(); ++i) {
    check_dense(in[i], "input");
    check_dense(out[i], "output");
    TORCH_CHECK(in[i].scalar_type() == in[0].scalar_type() &&
                    out[i].scalar_type() == in[0].scalar_type(),
                "penny: dtype mismatch");
    ip[i] = in[i].data_ptr();
    op[i] = out[i].data_ptr();
  }
  f(ip.data(), op.data());
}

// ---- global communicator behind the reference-style free functions ----------
std::mutex g_mu;
std::unique_ptr<Communicator> g_comm;

Communicator* global_comm() {
  TORCH_CHECK(g_comm != nullptr, "penny: call init_with_uid (or penny.utils.initialize_distributed) first");
  return g_comm.get();
}

size_t env_size(const char* name, size_t dflt) {
  const char* v = std::getenv(name);
  if (!v || !*v) return dflt;
  return (size_t)std::strtoull(v, nullptr, 10);
}

CommOptions options_from_env() {
  CommOptions o;
  o.heap_bytes = env_size("PENNY_HEAP_BYTES", o.heap_bytes);
  o.timeout_ms = (int)env_size("PENNY_TIMEOUT_MS", (size_t)o.timeout_ms);
  o.multicast = env_size("PENNY_DISABLE_NVLS", 0) == 0;
  const char* hm = std::getenv("PENNY_HEAP_MODE");
  if (hm && std::string(hm) == "ipc") o.heap_mode = HEAP_IPC;
  if (hm && std::string(hm) == "vmm") o.heap_mode = HEAP_VMM;
  return o;
}

// Algorithm object of the reference's create / run / destroy API
// (csrc/common.h:89-118).  packet_size / block_size / routes keep their meaning
// as launch knobs: block_size = threads per block, packet_size = bytes per
// thread per pass (sets the block count), routes = concurrent rings.
struct AlgoHandle {
  at::Tensor buffer;
  int algo;
  Tuning tuning;
};

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "penny_cpp: Blackwell-native collectives (peer-memory kernels over NVLink / NVSwitch)";

  // ------------------------------------------------------------------ bootstrap
  m.def("get_unique_id", []() {
    std::string id = make_unique_id();
    return py::bytearray(id.data(), id.size());
  });
  m.def("init_with_uid", [](py::object uid, int rank, int world_size) {
    std::string id = py::bytes(uid).cast<std::string>();
    std::lock_guard<std::mutex> lk(g_mu);
    TORCH_CHECK(g_comm == nullptr, "penny: already initialised");
    g_comm.reset(new Communicator(id, rank, world_size, options_from_env()));
  });
  m.def("finalize", []() {
    std::lock_guard<std::mutex> lk(g_mu);
    g_comm.reset();
  });
  m.def("is_initialized", []() { return g_comm != nullptr; });
  m.def("global_comm", []() { return (int64_t) reinterpret_cast<intptr_t>(global_comm()); });
  m.def("nvshmem_register", [](at::Tensor) {});
  m.def("nvshmem_unregister", [](at::Tensor) {});

  m.def("exchange", [](at::Tensor buffer, int packet_size, int block_size, int peer) {
    Communicator* c = global_comm();
    check_dense(buffer, "buffer");
    const at::cuda::OptionalCUDAGuard guard(buffer.device());
    Tuning t;
    t.threads = block_size >= 32 ? std::min(block_size, 512) : 0;
    (void)packet_size;
    void* p = buffer.data_ptr();
    c->exchange(dtype_of(buffer), &p, (size_t)buffer.numel(), &peer, t, current_stream());
  });

  m.def("all_reduce_create", [](at::Tensor buffer, int packet_size, int block_size, int nnodes,
                                int routes, int algo) {
    global_comm();
    check_dense(buffer, "buffer");
    TORCH_CHECK(algo >= 0 && algo <= ALGO_NVLS_ONESHOT, "penny: unknown algo ", algo);
    auto* h = new AlgoHandle();
    h->buffer = buffer;
    h->algo = algo;
    h->tuning.threads = block_size >= 32 ? std::min(block_size / 32 * 32, 512) : 0;
    h->tuning.nnodes = nnodes > 0 ? nnodes : 1;
    h->tuning.routes = routes;
    if (packet_size > 0 && h->tuning.threads > 0) {
      size_t bytes = (size_t)buffer.numel() * buffer.element_size();
      size_t per_block = (size_t)packet_size * h->tuning.threads;
      h->tuning.blocks = (int)std::min<size_t>(kMaxBlocks, std::max<size_t>(1, (bytes + per_block - 1) / per_block));
    }
    return (int64_t) reinterpret_cast<intptr_t>(h);
  });
  m.def("all_reduce_run", [](int64_t handle, at::Tensor output) {
    auto* h = reinterpret_cast<AlgoHandle*>(handle);
    TORCH_CHECK(h != nullptr, "penny: null handle");
    Communicator* c = global_comm();
    check_dense(output, "output");
    TORCH_CHECK(output.numel() == h->buffer.numel() && output.scalar_type() == h->buffer.scalar_type(),
                "penny: output must match the buffer given to all_reduce_create");
    const at::cuda::OptionalCUDAGuard guard(output.device());
    const void* in = h->buffer.data_ptr();
    void* out = output.data_ptr();
    Tuning t = h->tuning;
    // ring-type algorithms derive the block count from routes / trees themselves
    if (h->algo == ALGO_RING_STANDARD || h->algo == ALGO_TREE) t.blocks = 0;
    c->all_reduce(h->algo, dtype_of(output), &in, &out, (size_t)output.numel(), t, current_stream());
  });
  m.def("all_reduce_destroy", [](int64_t handle) { delete reinterpret_cast<AlgoHandle*>(handle); });

  // --------------------------------------------------------------- communicators
  m.def("comm_create", [](py::object uid, int rank, int world, int64_t heap_bytes, int heap_mode,
                          bool multicast, int timeout_ms) {
    std::string id = py::bytes(uid).cast<std::string>();
    CommOptions o = options_from_env();
    if (heap_bytes > 0) o.heap_bytes = (size_t)heap_bytes;
    o.heap_mode = heap_mode;
    o.multicast = o.multicast && multicast;
    if (timeout_ms > 0) o.timeout_ms = timeout_ms;
    return (int64_t) reinterpret_cast<intptr_t>(new Communicator(id, rank, world, o));
  }, py::arg("uid"), py::arg("rank"), py::arg("world"), py::arg("heap_bytes") = 0,
     py::arg("heap_mode") = 0, py::arg("multicast") = true, py::arg("timeout_ms") = 0);
  m.def("comm_create_emulated", [](int world, int64_t heap_bytes, int timeout_ms) {
    CommOptions o = options_from_env();
    if (heap_bytes > 0) o.heap_bytes = (size_t)heap_bytes;
    if (timeout_ms > 0) o.timeout_ms = timeout_ms;
    return (int64_t) reinterpret_cast<intptr_t>(new Communicator(world, o));
  }, py::arg("world"), py::arg("heap_bytes") = 0, py::arg("timeout_ms") = 0);
  m.def("comm_destroy", [](int64_t h) { delete as_comm(h); });
  m.def("comm_describe", [](int64_t h) { return as_comm(h)->describe(); });
  m.def("comm_has_multicast", [](int64_t h) { return as_comm(h)->has_multicast(); });
  m.def("comm_rank", [](int64_t h) { return as_comm(h)->rank(); });
  m.def("comm_world", [](int64_t h) { return as_comm(h)->world(); });
  m.def("comm_views", [](int64_t h) { return as_comm(h)->views(); });
  m.def("comm_heap_free", [](int64_t h) { return (int64_t)as_comm(h)->heap_free_bytes(); });
  m.def("comm_barrier", [](int64_t h) { as_comm(h)->host_barrier(); });
  m.def("comm_poison_scratch", [](int64_t h) { as_comm(h)->poison_scratch(); });
  m.def("comm_set_timeout_ms", [](int64_t h, int ms) { as_comm(h)->set_timeout_ms(ms); });
  m.def("comm_pick_algo", [](int64_t h, int dtype, int64_t n, bool symmetric) {
    return as_comm(h)->pick_algo(dtype, (size_t)n, symmetric);
  }, py::arg("comm"), py::arg("dtype"), py::arg("n"), py::arg("symmetric") = false);
  // all-reduce table of one (element size, memory class): [(max_bytes or -1 for "and above", algo id), ...]
  m.def("comm_set_tuning", [](int64_t h, int elem_size, bool symmetric, std::vector<std::pair<int64_t, int>> rows) {
    std::vector<Communicator::TuneEntry> e;
    for (auto& r : rows) e.push_back({r.first < 0 ? ~(size_t)0 : (size_t)r.first, r.second});
    as_comm(h)->set_tuning(elem_size, symmetric, e);
  });

  // A tensor whose storage is a fresh symmetric allocation.  In emulation one
  // tensor per virtual rank is returned (all at the same heap offset).
  m.def("comm_empty", [](int64_t h, std::vector<int64_t> sizes, at::ScalarType dtype) {
    Communicator* c = as_comm(h);
    int64_t numel = 1;
    for (auto s : sizes) numel *= s;
    size_t bytes = (size_t)numel * c10::elementSize(dtype);
    size_t off = c->alloc(std::max<size_t>(bytes, 16));
    int dev = 0;
    cudaGetDevice(&dev);
    auto opts = at::TensorOptions().dtype(dtype).device(at::kCUDA, dev);
    std::vector<at::Tensor> out;
    for (int v = 0; v < c->views(); ++v)
      out.push_back(torch::from_blob(c->local_ptr(off, v), sizes, [](void*) {}, opts));
    return out;
  });
  m.def("comm_heap_offset", [](int64_t h, at::Tensor t, int view) {
    size_t off = as_comm(h)->heap_offset_of(t.data_ptr(), view);
    return off == kNotInHeap ? (int64_t)-1 : (int64_t)off;
  });

  m.def("comm_all_reduce", [](int64_t h, std::vector<at::Tensor> in, std::vector<at::Tensor> out,
                              int algo, int blocks, int threads, int nnodes, int routes,
                              bool sym_in, bool sym_out) {
    Communicator* c = as_comm(h);
    TORCH_CHECK(!in.empty() && in[0].numel() == out[0].numel(), "penny: all_reduce shape mismatch");
    const at::cuda::OptionalCUDAGuard guard(in[0].device());
    with_views(c, in, out, [&](const void* const* ip, void* const* op) {
      c->all_reduce(algo, dtype_of(in[0]), ip, op, (size_t)in[0].numel(),
                    make_tuning(blocks, threads, nnodes, routes, sym_in, sym_out), current_stream());
    });
  }, py::arg("comm"), py::arg("inputs"), py::arg("outputs"), py::arg("algo") = -1,
     py::arg("blocks") = 0, py::arg("threads") = 0, py::arg("nnodes") = 1, py::arg("routes") = 0,
     py::arg("symmetric_in") = false, py::arg("symmetric_out") = false);

  m.def("comm_reduce_scatter", [](int64_t h, std::vector<at::Tensor> in, std::vector<at::Tensor> out,
                                  bool nvls, int blocks, int threads, bool sym_in, bool pipelined) {
    Communicator* c = as_comm(h);
    TORCH_CHECK(!in.empty() && in[0].numel() == out[0].numel() * c->world(),
                "penny: reduce_scatter output must hold numel / world elements");
    const at::cuda::OptionalCUDAGuard guard(in[0].device());
    with_views(c, in, out, [&](const void* const* ip, void* const* op) {
      c->reduce_scatter(dtype_of(in[0]), ip, op, (size_t)in[0].numel(), nvls,
                        make_tuning(blocks, threads, 1, 0, sym_in, false), current_stream(), pipelined);
    });
  }, py::arg("comm"), py::arg("inputs"), py::arg("outputs"), py::arg("nvls") = false,
     py::arg("blocks") = 0, py::arg("threads") = 0, py::arg("symmetric_in") = false,
     py::arg("pipelined") = false);

  m.def("comm_all_gather", [](int64_t h, std::vector<at::Tensor> in, std::vector<at::Tensor> out,
                              bool nvls, int blocks, int threads, bool sym_out) {
    Communicator* c = as_comm(h);
    TORCH_CHECK(!in.empty() && out[0].numel() == in[0].numel() * c->world(),
                "penny: all_gather output must hold numel * world elements");
    const at::cuda::OptionalCUDAGuard guard(in[0].device());
    with_views(c, in, out, [&](const void* const* ip, void* const* op) {
      c->all_gather(dtype_of(in[0]), ip, op, (size_t)in[0].numel(), nvls,
                    make_tuning(blocks, threads, 1, 0, false, sym_out), current_stream());
    });
  }, py::arg("comm"), py::arg("inputs"), py::arg("outputs"), py::arg("nvls") = false,
     py::arg("blocks") = 0, py::arg("threads") = 0, py::arg("symmetric_out") = false);

  m.def("comm_all_to_all", [](int64_t h, std::vector<at::Tensor> in, std::vector<at::Tensor> out,
                              int blocks, int threads, bool sym_out, bool pipelined) {
    Communicator* c = as_comm(h);
    TORCH_CHECK(!in.empty() && out[0].numel() == in[0].numel() && in[0].numel() % c->world() == 0,
                "penny: all_to_all needs equal chunks");
    const at::cuda::OptionalCUDAGuard guard(in[0].device());
    with_views(c, in, out, [&](const void* const* ip, void* const* op) {
      c->all_to_all(dtype_of(in[0]), ip, op, (size_t)in[0].numel() / c->world(),
                    make_tuning(blocks, threads, 1, 0, false, sym_out), current_stream(), pipelined);
    });
  }, py::arg("comm"), py::arg("inputs"), py::arg("outputs"), py::arg("blocks") = 0,
     py::arg("threads") = 0, py::arg("symmetric_out") = false, py::arg("pipelined") = false);

  m.def("comm_exchange", [](int64_t h, std::vector<at::Tensor> bufs, std::vector<int> peers,
                            int blocks, int threads) {
    Communicator* c = as_comm(h);
    TORCH_CHECK((int)bufs.size() == c->views() && peers.size() == bufs.size(),
                "penny: expected ", c->views(), " buffer(s) and peer(s)");
    std::vector<void*> p;
    for (auto& b : bufs) {
      check_dense(b, "buffer");
      p.push_back(b.data_ptr());
    }
    const at::cuda::OptionalCUDAGuard guard(bufs[0].device());
    c->exchange(dtype_of(bufs[0]), p.data(), (size_t)bufs[0].numel(), peers.data(),
                make_tuning(blocks, threads, 1, 0, false, false), current_stream());
  }, py::arg("comm"), py::arg("buffers"), py::arg("peers"), py::arg("blocks") = 0,
     py::arg("threads") = 0);

  m.def("comm_fused_ar_rmsnorm", [](int64_t h, std::vector<at::Tensor> in,
                                    std::vector<at::Tensor> residual, at::Tensor weight,
                                    std::vector<at::Tensor> out, std::vector<at::Tensor> residual_out,
                                    double eps, int proto, int blocks, int threads, bool symmetric,
                                    int symmetric_out_arg, bool pushed) {
    Communicator* c = as_comm(h);
    const int nv = c->views();
    // symmetric: the inputs sit at one heap offset on every rank; symmetric_out: the outputs do
    // (-1 = same answer as for the inputs)
    const bool symmetric_out = symmetric_out_arg < 0 ? symmetric : symmetric_out_arg != 0;
    TORCH_CHECK((int)in.size() == nv && (int)out.size() == nv, "penny: expected ", nv, " tensor(s)");
    TORCH_CHECK(residual.empty() || (int)residual.size() == nv, "penny: residual views");
    TORCH_CHECK(residual_out.empty() || (int)residual_out.size() == nv, "penny: residual_out views");
    TORCH_CHECK(in[0].dim() == 2, "penny: fused norm expects [rows, hidden]");
    const int rows = (int)in[0].size(0), hidden = (int)in[0].size(1);
    check_dense(weight, "weight");
    TORCH_CHECK(weight.numel() == hidden && weight.scalar_type() == in[0].scalar_type(),
                "penny: weight must be [hidden] of the input dtype");
    std::vector<const void*> ip(nv), rp(nv);
    std::vector<void*> op(nv), rop(nv);
    // every row is moved as 16-byte vectors: refuse a misaligned base here, on
    // the host, rather than fault on the device
    auto aligned16 = [](const at::Tensor& t, const char* what) {
      TORCH_CHECK((reinterpret_cast<uintptr_t>(t.data_ptr()) & 15u) == 0, "penny: fused norm ", what,
                  " must start on a 16-byte boundary");
    };
    aligned16(weight, "weight");
    for (int v = 0; v < nv; ++v) {
      check_dense(in[v], "input");
      check_dense(out[v], "output");
      TORCH_CHECK(out[v].numel() == in[v].numel(), "penny: output shape");
      aligned16(in[v], "input");
      aligned16(out[v], "output");
      ip[v] = in[v].data_ptr();
      op[v] = out[v].data_ptr();
      if (!residual.empty()) {
        check_dense(residual[v], "residual");
        aligned16(residual[v], "residual");
        rp[v] = residual[v].data_ptr();
      }
      if (!residual_out.empty()) {
        check_dense(residual_out[v], "residual_out");
        aligned16(residual_out[v], "residual_out");
        rop[v] = residual_out[v].data_ptr();
      }
    }
    const at::cuda::OptionalCUDAGuard guard(in[0].device());
    c->fused_ar_rmsnorm(dtype_of(in[0]), proto, ip.data(), residual.empty() ? nullptr : rp.data(),
                        weight.data_ptr(), op.data(), residual_out.empty() ? nullptr : rop.data(),
                        rows, hidden, (float)eps,
                        make_tuning(blocks, threads, 1, 0, symmetric, symmetric_out), current_stream(), pushed);
  }, py::arg("comm"), py::arg("inputs"), py::arg("residual"), py::arg("weight"),
     py::arg("outputs"), py::arg("residual_out"), py::arg("eps") = 1e-5, py::arg("proto") = 0,
     py::arg("blocks") = 0, py::arg("threads") = 0, py::arg("symmetric") = false,
     py::arg("symmetric_out") = -1, py::arg("pushed") = false);
  // The epilogue target (a DecodePush, as bytes in a CPU tensor) for gemm_decode(push=...) feeding
  // comm_fused_ar_rmsnorm(proto = LL two-shot, pushed = true) on a [rows, hidden] bf16 tensor.
  m.def("comm_fused_norm_push_target", [](int64_t h, int64_t rows, int64_t hidden, int64_t view) {
    const penny::sm100::DecodePush p = as_comm(h)->fused_norm_push_target((int)rows, (int)hidden, 2, (int)view);
    auto t = torch::empty({(int64_t)sizeof(p)}, torch::TensorOptions().dtype(torch::kUInt8));
    memcpy(t.data_ptr(), &p, sizeof(p));
    return t;
  }, py::arg("comm"), py::arg("rows"), py::arg("hidden"), py::arg("view") = 0);

  // out = rmsnorm(x + residual) * weight without communication (world size 1)
  m.def("add_rmsnorm", [](at::Tensor x, c10::optional<at::Tensor> residual, at::Tensor weight,
                          at::Tensor out, c10::optional<at::Tensor> residual_out, double eps) {
    check_dense(x, "x");
    check_dense(out, "out");
    check_dense(weight, "weight");
    TORCH_CHECK(x.dim() == 2 && out.numel() == x.numel() && weight.numel() == x.size(1),
                "penny: add_rmsnorm shapes");
    FusedNormArgs a;
    memset(&a, 0, sizeof(a));
    a.in = x.data_ptr();
    a.residual = residual.has_value() ? residual->data_ptr() : nullptr;
    a.weight = weight.data_ptr();
    a.out = out.data_ptr();
    a.residual_out = residual_out.has_value() ? residual_out->data_ptr() : nullptr;
    a.rows = (int)x.size(0);
    a.hidden = (int)x.size(1);
    a.eps = (float)eps;
    const int es = (int)x.element_size();
    const int threads = std::min(512, std::max(32, (a.hidden * es / 16 + 31) / 32 * 32));
    const at::cuda::OptionalCUDAGuard guard(x.device());
    cudaError_t rc = launch_add_rmsnorm(dtype_of(x), a, std::min(a.rows, 2048), threads, current_stream());
    TORCH_CHECK(rc == cudaSuccess, "penny: add_rmsnorm: ", cudaGetErrorString(rc));
  }, py::arg("x"), py::arg("residual"), py::arg("weight"), py::arg("out"),
     py::arg("residual_out"), py::arg("eps") = 1e-5);

  // MoE dispatch: x rows -> the owners of their experts.  Every list has one entry
  // per view.  recv / meta are symmetric heap tensors ([cap_rows, hidden], [cap_rows] int32).
  m.def("comm_moe_dispatch", [](int64_t h, std::vector<at::Tensor> x, std::vector<at::Tensor> order,
                                std::vector<at::Tensor> expert_of_sorted, std::vector<at::Tensor> send_off,
                                std::vector<at::Tensor> dst_base, std::vector<at::Tensor> dst_row_of_pair,
                                std::vector<at::Tensor> recv, std::vector<at::Tensor> meta, int topk,
                                int experts, int blocks) {
    Communicator* c = as_comm(h);
    const int nv = c->views();
    TORCH_CHECK((int)x.size() == nv && (int)recv.size() == nv && (int)meta.size() == nv, "comm_moe_dispatch: views");
    MoeArgs a[kMaxRanks];
    memset(a, 0, sizeof(a));
    for (int v = 0; v < nv; ++v) {
      check_dense(x[v], "x");
      TORCH_CHECK(x[v].dim() == 2 && recv[v].dim() == 2 && recv[v].size(1) == x[v].size(1), "comm_moe_dispatch: shapes");
      for (const at::Tensor* t : {&order[v], &expert_of_sorted[v], &send_off[v], &dst_base[v], &dst_row_of_pair[v], &meta[v]})
        TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kInt && t->is_contiguous(), "comm_moe_dispatch: int32 CUDA tables");
      a[v].x = x[v].data_ptr();
      a[v].order = order[v].data_ptr<int>();
      a[v].expert_of_sorted = expert_of_sorted[v].data_ptr<int>();
      a[v].send_off = send_off[v].data_ptr<int>();
      a[v].dst_base = dst_base[v].data_ptr<int>();
      a[v].dst_row_of_pair = dst_row_of_pair[v].data_ptr<int>();
      a[v].recv_off = c->heap_offset_of(recv[v].data_ptr(), v);
      a[v].meta_off = c->heap_offset_of(meta[v].data_ptr(), v);
      TORCH_CHECK(a[v].recv_off != kNotInHeap && a[v].meta_off != kNotInHeap,
                  "comm_moe_dispatch: recv and meta must be symmetric heap tensors");
      TORCH_CHECK(a[v].recv_off == a[0].recv_off && a[v].meta_off == a[0].meta_off, "comm_moe_dispatch: offsets differ");
      a[v].tokens = (int)x[v].size(0);
      a[v].topk = topk;
      a[v].hidden = (int)x[v].size(1);
      a[v].experts = experts;
      a[v].cap_rows = (int)recv[v].size(0);
    }
    const at::cuda::OptionalCUDAGuard guard(x[0].device());
    Tuning t;
    t.blocks = blocks;
    c->moe_dispatch(dtype_of(x[0]), a, t, current_stream());
  }, py::arg("comm"), py::arg("x"), py::arg("order"), py::arg("expert_of_sorted"), py::arg("send_off"),
     py::arg("dst_base"), py::arg("dst_row_of_pair"), py::arg("recv"), py::arg("meta"), py::arg("topk"),
     py::arg("experts"), py::arg("blocks") = 0);

  // MoE combine: expert outputs y (rows as received) -> out[t] = sum_k gates[t, k] * y[t, k].
  m.def("comm_moe_combine", [](int64_t h, std::vector<at::Tensor> y, std::vector<at::Tensor> out,
                               std::vector<at::Tensor> topk_ids, std::vector<at::Tensor> gates,
                               std::vector<at::Tensor> meta, std::vector<at::Tensor> dst_row_of_pair,
                               std::vector<at::Tensor> comb, std::vector<int> recv_rows, int experts,
                               int blocks) {
    Communicator* c = as_comm(h);
    const int nv = c->views();
    TORCH_CHECK((int)y.size() == nv && (int)out.size() == nv && (int)comb.size() == nv && (int)recv_rows.size() == nv,
                "comm_moe_combine: views");
    MoeArgs a[kMaxRanks];
    memset(a, 0, sizeof(a));
    for (int v = 0; v < nv; ++v) {
      check_dense(y[v], "y");
      check_dense(out[v], "out");
      TORCH_CHECK(topk_ids[v].scalar_type() == at::kInt && gates[v].scalar_type() == at::kFloat &&
                      meta[v].scalar_type() == at::kInt && dst_row_of_pair[v].scalar_type() == at::kInt,
                  "comm_moe_combine: table dtypes (int32 ids/meta/rows, fp32 gates)");
      TORCH_CHECK(topk_ids[v].is_contiguous() && gates[v].is_contiguous(), "comm_moe_combine: contiguous tables");
      a[v].x = y[v].data_ptr();
      a[v].out = out[v].data_ptr();
      a[v].topk_ids = topk_ids[v].data_ptr<int>();
      a[v].gates = gates[v].data_ptr<float>();
      a[v].meta = meta[v].data_ptr<int>();
      a[v].dst_row_of_pair = dst_row_of_pair[v].data_ptr<int>();
      a[v].comb_off = c->heap_offset_of(comb[v].data_ptr(), v);
      TORCH_CHECK(a[v].comb_off != kNotInHeap && a[v].comb_off == c->heap_offset_of(comb[0].data_ptr(), 0),
                  "comm_moe_combine: comb must be a symmetric heap tensor");
      a[v].tokens = (int)out[v].size(0);
      a[v].topk = (int)(topk_ids[v].numel() / out[v].size(0));
      a[v].hidden = (int)out[v].size(1);
      a[v].experts = experts;
      a[v].recv_rows = recv_rows[v];
      TORCH_CHECK(y[v].size(0) >= recv_rows[v] && comb[v].size(0) >= (int64_t)a[v].tokens * a[v].topk,
                  "comm_moe_combine: buffer sizes");
    }
    const at::cuda::OptionalCUDAGuard guard(y[0].device());
    Tuning t;
    t.blocks = blocks;
    c->moe_combine(dtype_of(out[0]), a, t, current_stream());
  }, py::arg("comm"), py::arg("y"), py::arg("out"), py::arg("topk_ids"), py::arg("gates"), py::arg("meta"),
     py::arg("dst_row_of_pair"), py::arg("comb"), py::arg("recv_rows"), py::arg("experts"), py::arg("blocks") = 0);

  // out[M / world, N] = this rank's row shard of sum_r a_r[M, K_r] @ b_r[N, K_r]^T
  m.def("comm_gemm_rs", [](int64_t h, at::Tensor a, at::Tensor b, at::Tensor out) {
    Communicator* c = as_comm(h);
    TORCH_CHECK(a.is_cuda() && a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16 &&
                    out.scalar_type() == at::kBFloat16, "comm_gemm_rs: bf16 CUDA tensors");
    TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && out.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1 &&
                    out.stride(1) == 1, "comm_gemm_rs: 2-D tensors with contiguous rows");
    const int64_t M = a.size(0), K = a.size(1), N = b.size(0);
    TORCH_CHECK(b.size(1) == K && out.size(0) * c->world() == M && out.size(1) == N, "comm_gemm_rs: shapes");
    const at::cuda::OptionalCUDAGuard guard(a.device());
    c->gemm_reduce_scatter(a.data_ptr(), b.data_ptr(), out.data_ptr(), (int)M, (int)N, (int)K,
                           (int)a.stride(0), (int)b.stride(0), (int)out.stride(0), penny_gemm_error_word(),
                           current_stream());
  });
  // out[M, N] = all_gather(a_shard)[M, K] @ b[N, K]^T
  m.def("comm_ag_gemm", [](int64_t h, at::Tensor a_shard, at::Tensor b, at::Tensor out, int side_ctas) {
    Communicator* c = as_comm(h);
    TORCH_CHECK(a_shard.is_cuda() && a_shard.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16 &&
                    out.scalar_type() == at::kBFloat16, "comm_ag_gemm: bf16 CUDA tensors");
    TORCH_CHECK(a_shard.dim() == 2 && b.dim() == 2 && out.dim() == 2 && a_shard.stride(1) == 1 &&
                    b.stride(1) == 1 && out.stride(1) == 1, "comm_ag_gemm: 2-D tensors with contiguous rows");
    const int64_t M = a_shard.size(0) * c->world(), K = a_shard.size(1), N = b.size(0);
    TORCH_CHECK(b.size(1) == K && out.size(0) == M && out.size(1) == N, "comm_ag_gemm: shapes");
    const at::cuda::OptionalCUDAGuard guard(a_shard.device());
    c->all_gather_gemm(a_shard.data_ptr(), b.data_ptr(), out.data_ptr(), (int)M, (int)N, (int)K,
                       (int)a_shard.stride(0), (int)b.stride(0), (int)out.stride(0), side_ctas,
                       penny_gemm_error_word(), current_stream());
  }, py::arg("comm"), py::arg("a_shard"), py::arg("b"), py::arg("out"), py::arg("side_ctas") = 0);

  m.def("comm_wait_selftest", [](int64_t h) { as_comm(h)->wait_selftest(current_stream()); });
  m.def("comm_status", [](int64_t h, int view, bool clear) {
    StatusRecord s = as_comm(h)->read_status(view, clear);
    py::dict d;
    d["code"] = s.code;
    d["rank"] = s.rank;
    d["peer"] = s.peer;
    d["block"] = s.block;
    d["want"] = s.want;
    d["seen"] = s.seen;
    return d;
  }, py::arg("comm"), py::arg("view") = 0, py::arg("clear") = true);

  // ------------------------------------------------------------------- schedule
  m.def("sched_ring_rank_at", &ring_rank_at);
  m.def("sched_ring_stride", &ring_stride);

  m.attr("ALGO_RING_STANDARD") = (int)ALGO_RING_STANDARD;
  m.attr("ALGO_RING_SIMPLE") = (int)ALGO_RING_SIMPLE;
  m.attr("ALGO_ONESHOT") = (int)ALGO_ONESHOT;
  m.attr("ALGO_TWOSHOT") = (int)ALGO_TWOSHOT;
  m.attr("ALGO_DOUBLE_RING") = (int)ALGO_DOUBLE_RING;
  m.attr("ALGO_TREE") = (int)ALGO_TREE;
  m.attr("ALGO_NVLS") = (int)ALGO_NVLS;
  m.attr("ALGO_ONESHOT_LL") = (int)ALGO_ONESHOT_LL;
  m.attr("ALGO_NVLS_ONESHOT") = (int)ALGO_NVLS_ONESHOT;
  m.attr("ALGO_AUTO") = (int)ALGO_AUTO;
  m.attr("PROTO_LL") = (int)FUSED_PROTO_LL;
  m.attr("PROTO_FLAG") = (int)FUSED_PROTO_FLAG;
  m.attr("PROTO_NVLS") = (int)FUSED_PROTO_NVLS;
  m.attr("PROTO_NVLS_ONESHOT") = (int)FUSED_PROTO_NVLS_ONESHOT;
  m.attr("PROTO_LL_TWOSHOT") = (int)FUSED_PROTO_LL_TWOSHOT;

  bind_custom_all_reduce(m);
  bind_gemm(m);
  bind_decode(m);
}
