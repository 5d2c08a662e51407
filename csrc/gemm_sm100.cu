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
// The same main loop is the body of the fused kernels (GEMM -> reduce-scatter,
// all-gather -> GEMM): they differ in where the epilogue writes and in what the
// producer waits for.  Those variants live in gemm_rs_sm100.cu / ag_gemm_sm100.cu
// and instantiate gemm_persistent<> with their own policies.
#include "gemm_sm100.h"

#include <cuda.h>

#include <mutex>
#include <stdexcept>
#include <string>

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
  static bool attr = false;
  if (!attr) {
    rc = cudaFuncSetAttribute(gemm_persistent<BN, StoreLocal>,
                              cudaFuncAttributeMaxDynamicSharedMemorySize, Kernel::kSmemBytes);
    if (rc != cudaSuccess) return rc;
    attr = true;
  }
  const int tiles_m = (M + kBlockM - 1) / kBlockM, tiles_n = (N + BN - 1) / BN;
  const int grid = std::min(sms, tiles_m * tiles_n);
  GemmShape shape{M, N, K, tiles_m, tiles_n, 0, tiles_m * tiles_n, 1};
  StoreLocal ep;
  ep.c = reinterpret_cast<__nv_bfloat16*>(c);
  ep.ldc = ldc;
  gemm_persistent<BN, StoreLocal><<<grid, kGemmThreads, Kernel::kSmemBytes, stream>>>(
      ma, mb, shape, ep, error_word);
  return cudaGetLastError();
}

cudaError_t launch_gemm_bf16(const void* a, const void* b, void* c, int M, int N, int K, int lda,
                             int ldb, int ldc, int block_n, uint32_t* error_word,
                             cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || K % 8 != 0 || lda % 8 != 0 || ldb % 8 != 0)
    return cudaErrorInvalidValue;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (block_n == 0) block_n = (N >= 256 && (long long)((M + 127) / 128) * ((N + 255) / 256) >= sms / 2) ? 256 : 128;
  if (block_n == 256) return launch_gemm_bn<256>(a, b, c, M, N, K, lda, ldb, ldc, sms, error_word, stream);
  if (block_n == 128) return launch_gemm_bn<128>(a, b, c, M, N, K, lda, ldb, ldc, sms, error_word, stream);
  return cudaErrorInvalidValue;
}

}  // namespace sm100
}  // namespace penny
