// C[M, N] = A[M, K] * B[N, K]^T  (bf16 in, fp32 accumulate in TMEM, bf16 out)
// for sm_100a: a persistent, warp-specialised tcgen05 kernel.
//
//   warp 0      TMA producer: one elected thread streams [128 x 64] A tiles and
//               [BN x 64] B tiles (128-byte swizzle) into a kStages-deep ring
//   warp 1      MMA issuer: one elected thread issues tcgen05.mma (M=128, N=BN,
//               K=16) into one of two TMEM accumulators; tcgen05.commit hands
//               ring slots back to the producer and accumulators to the epilogue
//   warps 2-5   epilogue: tcgen05.ld the finished accumulator (each warp its
//               own 32-lane quarter), convert to bf16, transpose through a small
//               swizzled staging buffer and store full 128-byte row segments –
//               overlapped with the MMAs of the next tile
//   warps 6-9   copy warps: idle here; in the fused kernels they move operand
//               shards between GPUs while the other warps compute
// One CTA per SM; tiles are handed out round-robin with the M index fastest so
// that CTAs working at the same time share a B tile in L2.
//
// Large problems run the CTA-pair variant instead (gemm_kernel_pair_sm100.cuh:
// cta_group::2, 256 x 256 tiles over two SMs, a third less shared-memory fill
// traffic per FLOP); block_n = 512 selects it explicitly.
//
// The same main loop is the body of the fused kernels (GEMM -> reduce-scatter,
// all-gather -> GEMM): they differ in where the epilogue writes and in what the
// producer waits for.  Those variants live in gemm_fused_sm100.cu and
// instantiate gemm_persistent<> / gemm_persistent_pair<> with their own policies.
#include "gemm_sm100.h"

#include <cuda.h>

#include <atomic>
#include <cstdlib>
#include <map>
#include <mutex>
#include <stdexcept>
#include <string>

#include "gemm_kernel_pair_sm100.cuh"
#include "kernel_setup.h"
#include "gemm_kernel_sm100.cuh"

namespace penny {
namespace sm100 {

namespace {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                              CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                              CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, []() {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult st;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &st) == cudaSuccess &&
        st == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(p);
    else
      (void)cudaGetLastError();
  });
  return fn;
}

}  // namespace

// Row-major [rows, cols] bf16 matrix, box = [box_rows x 64 columns], 128-byte swizzle.
cudaError_t make_tile_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols,
                          uint64_t row_stride_elems, uint32_t box_rows) {
  EncodeFn fn = encode_fn();
  if (fn == nullptr) return cudaErrorNotSupported;
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || (row_stride_elems * 2) % 16 != 0 ||
      box_rows == 0 || box_rows > 256)
    return cudaErrorInvalidValue;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {row_stride_elems * 2};
  cuuint32_t box[2] = {(cuuint32_t)kBlockK, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

// Plain GEMM: C row-major in this GPU's memory, nothing to wait for.
struct StoreLocal : PolicyBase {
  __nv_bfloat16* c;
  int ldc;
  __device__ __forceinline__ void store16(const State&, int row, int col, const uint4& v, int M,
                                          int N) const {
    store16_local(c, ldc, row, col, v, M, N);
  }
};

template <int BN>
cudaError_t launch_gemm_bn(const void* a, const void* b, void* c, int M, int N, int K, int lda,
                           int ldb, int ldc, int sms, uint32_t* error_word, cudaStream_t stream) {
  CUtensorMap ma, mb;
  cudaError_t rc = make_tile_map(&ma, a, (uint64_t)M, (uint64_t)K, (uint64_t)lda, kBlockM);
  if (rc != cudaSuccess) return rc;
  rc = make_tile_map(&mb, b, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, BN);
  if (rc != cudaSuccess) return rc;
  using Kernel = GemmKernel<BN>;
  rc = kernel_setup(reinterpret_cast<const void*>(gemm_persistent<BN, StoreLocal>), Kernel::kSmemBytes).rc;
  if (rc != cudaSuccess) return rc;
  const int tiles_m = (M + kBlockM - 1) / kBlockM, tiles_n = (N + BN - 1) / BN;
  const int grid = std::min(sms, tiles_m * tiles_n);
  GemmShape shape{M, N, K, tiles_m, tiles_n, 0, tiles_m * tiles_n, 1, 16};
  StoreLocal ep;
  ep.c = reinterpret_cast<__nv_bfloat16*>(c);
  ep.ldc = ldc;
  gemm_persistent<BN, StoreLocal><<<grid, kGemmThreads, Kernel::kSmemBytes, stream>>>(
      ma, mb, shape, ep, error_word);
  return cudaGetLastError();
}

namespace {
std::atomic<int> g_split_tail{-1};  // -1: take PENNY_GEMM_SPLIT_TAIL (default off)
}
void set_split_tail(int on) { g_split_tail.store(on < 0 ? -1 : (on != 0)); }
bool split_tail_enabled() {
  const int v = g_split_tail.load();
  if (v >= 0) return v != 0;
  static const bool on = []() {
    const char* e = getenv("PENNY_GEMM_SPLIT_TAIL");
    return e != nullptr && e[0] == '1';
  }();
  return on;
}

bool pair_kernel_enabled() {
  static const bool on = []() {
    const char* e = getenv("PENNY_GEMM_PAIR");
    return !(e != nullptr && e[0] == '0');
  }();
  return on;
}

namespace {
// fp32 partial tiles + arrival counters of the split last wave: one per
// (device, stream), so that launches on different streams never share it.
struct SplitScratch {
  float* ws = nullptr;
  unsigned* counters = nullptr;
};
constexpr int kMaxSplit = 4;

SplitScratch* split_scratch(int dev, cudaStream_t stream, int pairs) {
  static std::mutex mu;
  static std::map<std::pair<int, cudaStream_t>, SplitScratch> table;
  std::lock_guard<std::mutex> lock(mu);
  auto it = table.find({dev, stream});
  if (it != table.end()) return &it->second;
  // never allocate while the stream is being captured: the caller falls back to unsplit tiles
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
    (void)cudaGetLastError();
    return nullptr;
  }
  SplitScratch sc;
  const size_t ws_bytes = (size_t)pairs * 2 * kBlockM * PairGemmKernel::kTileN * sizeof(float);
  if (cudaMalloc(&sc.ws, ws_bytes) != cudaSuccess) {
    (void)cudaGetLastError();
    return nullptr;
  }
  if (cudaMalloc(&sc.counters, (size_t)pairs * 2 * sizeof(unsigned)) != cudaSuccess ||
      cudaMemset(sc.counters, 0, (size_t)pairs * 2 * sizeof(unsigned)) != cudaSuccess) {
    (void)cudaGetLastError();
    cudaFree(sc.ws);
    return nullptr;
  }
  return &(table[{dev, stream}] = sc);
}
}  // namespace

// 256 x 256 tiles on CTA pairs (cta_group::2).  A ragged last wave is split along
// K over the idle pairs (at most kMaxSplit ranges per tile; gemm_tile_order.h).
cudaError_t launch_gemm_pair(const void* a, const void* b, void* c, int M, int N, int K, int lda,
                             int ldb, int ldc, int sms, uint32_t* error_word, cudaStream_t stream) {
  CUtensorMap ma, mb;
  cudaError_t rc = make_tile_map(&ma, a, (uint64_t)M, (uint64_t)K, (uint64_t)lda, kBlockM);
  if (rc != cudaSuccess) return rc;
  rc = make_tile_map(&mb, b, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, PairGemmKernel::kTileN / 2);
  if (rc != cudaSuccess) return rc;
  const KernelSetup ks = kernel_setup(reinterpret_cast<const void*>(gemm_persistent_pair<StoreLocal>),
                                      PairGemmKernel::kSmemBytes, kGemmThreads);
  if (ks.rc != cudaSuccess) return ks.rc;
  const int pairs = ks.pairs;
  const int tiles_m = (M + kBlockM - 1) / kBlockM;
  const int tiles_n = (N + PairGemmKernel::kTileN - 1) / PairGemmKernel::kTileN;
  const int ptiles = ((tiles_m + 1) / 2) * tiles_n;
  GemmShape shape{M, N, K, tiles_m, tiles_n, 0, tiles_m * tiles_n, 1, 16};
  int npairs = std::min(pairs, ptiles);
  plan_split_tail(shape, pairs, (K + kBlockK - 1) / kBlockK, split_tail_enabled() ? kMaxSplit : 1);
  if (shape.split_s > 1) {
    int dev = 0;
    cudaGetDevice(&dev);
    SplitScratch* sc = split_scratch(dev, stream, pairs);
    if (sc != nullptr) {
      shape.split_ws = sc->ws;
      shape.split_counters = sc->counters;
      npairs = pairs;  // the plan assumes the full grid
    } else {
      shape.split_s = 1;
      shape.split_first = ptiles;
    }
  }
  StoreLocal ep;
  ep.c = reinterpret_cast<__nv_bfloat16*>(c);
  ep.ldc = ldc;
  gemm_persistent_pair<StoreLocal><<<2 * npairs, kGemmThreads, PairGemmKernel::kSmemBytes, stream>>>(
      ma, mb, shape, ep, error_word);
  return cudaGetLastError();
}

// Estimated time of each kernel variant in units of one 128 x 256 tile on one
// SM: waves x relative tile cost.  The single-CTA kernels are fill-bound (more
// so the narrower the tile; factors from measured 8192^3 and 4096 x 768 x 4096
// runs); a pair tile takes the time of one 128 x 256 tile.  The number of
// resident pairs differs between parts (GPCs with an odd SM count strand one).
int choose_block_n(int M, int N, int K, int sms, int pairs) {
  const int tiles_m = (M + kBlockM - 1) / kBlockM;
  auto waves = [](long long tiles, int slots) { return (double)((tiles + slots - 1) / slots); };
  auto single = [&](int bn, double eff) {
    return waves((long long)tiles_m * ((N + bn - 1) / bn), sms) * (bn / 256.0) * eff;
  };
  double best = single(128, 1.45);
  int pick = 128;
  if (N > 128 && single(192, 1.20) < best) best = single(192, 1.20), pick = 192;
  if (N > 192 && single(256, 1.12) < best) best = single(256, 1.12), pick = 256;
  if (pair_kernel_enabled() && N > 128 && pairs > 0) {
    GemmShape s{M, N, K, tiles_m, (N + 255) / 256, 0, 0, 1, 16};
    const int num_kb = (K + kBlockK - 1) / kBlockK;
    plan_split_tail(s, pairs, num_kb, split_tail_enabled() ? kMaxSplit : 1);
    const int ptiles = pair_tile_count(s);
    double cost;
    if (s.split_s > 1) cost = s.split_first / pairs + 1.0 / s.split_s + 0.1;
    else cost = waves(ptiles, pairs);
    if (K < 1024) cost *= 1.25;  // short K: the epilogue of a 256-row tile is not hidden (measured at K = 512)
    if (cost < best) best = cost, pick = 512;
  }
  return pick;
}

cudaError_t launch_gemm_bf16(const void* a, const void* b, void* c, int M, int N, int K, int lda,
                             int ldb, int ldc, int block_n, uint32_t* error_word,
                             cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || K % 8 != 0 || lda % 8 != 0 || ldb % 8 != 0)
    return cudaErrorInvalidValue;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (block_n == 0) {
    const KernelSetup ks = kernel_setup(reinterpret_cast<const void*>(gemm_persistent_pair<StoreLocal>),
                                        PairGemmKernel::kSmemBytes, kGemmThreads);
    const int pairs = ks.rc == cudaSuccess ? ks.pairs : 0;
    block_n = choose_block_n(M, N, K, sms, pairs);
  }
  if (block_n == 512) return launch_gemm_pair(a, b, c, M, N, K, lda, ldb, ldc, sms, error_word, stream);
  if (block_n == 192) return launch_gemm_bn<192>(a, b, c, M, N, K, lda, ldb, ldc, sms, error_word, stream);
  if (block_n == 256) return launch_gemm_bn<256>(a, b, c, M, N, K, lda, ldb, ldc, sms, error_word, stream);
  if (block_n == 128) return launch_gemm_bn<128>(a, b, c, M, N, K, lda, ldb, ldc, sms, error_word, stream);
  return cudaErrorInvalidValue;
}

}  // namespace sm100
}  // namespace penny
