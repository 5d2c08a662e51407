// NVLS collectives: the reduction and the broadcast happen inside the NVSwitch.
//
// c.mc is the multicast alias of the symmetric heap: a multimem.ld_reduce on
// mc + off returns the sum of the word at heap offset `off` of EVERY rank (the
// switch pulls the replicas and adds them, fp32 accumulate), a multimem.st on
// mc + off writes all replicas at once.
//
//   NvlsTwoShot   rank r reduces chunk r with ld_reduce and multicasts the
//                 result: each GPU's links carry S/N + S bytes instead of the
//                 2 * S * (N-1)/N of any peer-to-peer algorithm.  Input and output
//                 in the heap at the same offset on every rank.
//                 Tensors elsewhere are staged by the communicator with two copies
//                 (a variant that staged inside the kernel measured 3-7 us slower
//                 at 8 ranks than the two copy launches it saved).
//   NvlsOneShot   stage the input into this call's scratch half, ONE barrier, then
//                 every rank ld_reduces the whole buffer into its own output.  No
//                 second barrier: the next call uses the other half, and a rank can
//                 only reach the call after that once every peer has left this one.
//   NvlsReduceScatter / NvlsAllGather   the two halves on their own.
//
// Unless staged, the input (and for two-shot / all-gather the output) must live in
// the heap at the same offset on every rank, and both barriers are needed: the first
// says "my input is complete", the second "the switch has finished reading my input
// and my writes have landed", so a buffer may be reused right after the call.
// The reference has no NVLS path (it predates it: NVSHMEM puts + signals only).
#include "algos.h"
#include "launch.cuh"
#include "schedule.h"

namespace penny {

template <typename T>
__device__ __forceinline__ V16 multimem_ld_reduce(const void* p);
template <>
__device__ __forceinline__ V16 multimem_ld_reduce<float>(const void* p) {
  V16 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3])
               : "l"(p)
               : "memory");
  return v;
}
template <>
__device__ __forceinline__ V16 multimem_ld_reduce<__nv_bfloat16>(const void* p) {
  V16 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3])
               : "l"(p)
               : "memory");
  return v;
}
template <>
__device__ __forceinline__ V16 multimem_ld_reduce<__half>(const void* p) {
  V16 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3])
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st(void* p, const V16& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p),
               "r"(v.w[0]), "r"(v.w[1]), "r"(v.w[2]), "r"(v.w[3])
               : "memory");
}

template <typename T>
struct NvlsTwoShot {
  static __device__ void body(const CommCtx& c, int rank, const CollArgs& a, const Blk& b, u64 seq,
                              int& s_abort) {
    constexpr size_t E = 16 / sizeof(T);
    const size_t V = ceil_div(a.n, E);
    const Span mine = split_span(V, c.world, rank);
    const size_t stride = (size_t)b.nblocks * b.nthreads;
    PK_BLOCK_BARRIER(c, rank, CH_BARRIER, b, flag_value(seq, 1), s_abort);
    if (s_abort) return;
    const size_t len = mine.end - mine.begin;
    for (size_t j0 = (size_t)b.bid * b.nthreads + threadIdx.x; j0 < len; j0 += kBatch * stride) {
      V16 r[kBatch];
#pragma unroll
      for (int u = 0; u < kBatch; ++u)
        if (j0 + u * stride < len)
          r[u] = multimem_ld_reduce<T>(c.mc + a.in_heap_off + (mine.begin + j0 + u * stride) * 16);
#pragma unroll
      for (int u = 0; u < kBatch; ++u)
        if (j0 + u * stride < len)
          multimem_st(c.mc + a.out_heap_off + (mine.begin + j0 + u * stride) * 16, r[u]);
    }
    PK_BLOCK_BARRIER(c, rank, CH_BARRIER, b, flag_value(seq, 2), s_abort);
  }
  static __device__ void run(const CommCtx& c, int rank, const CollArgs& a, const Blk& b) {
    run_collective<NvlsTwoShot<T>, CollArgs>(c, rank, a, b);
  }
};

// scratch: both halves of [V] staged vectors
PK_HD size_t nvls_oneshot_scratch_bytes(size_t n, int elem_size) { return 2 * vecs_for(n, elem_size) * 16; }

template <typename T>
struct NvlsOneShot {
  static __device__ void body(const CommCtx& c, int rank, const CollArgs& a, const Blk& b, u64 seq,
                              int& s_abort) {
    constexpr size_t E = 16 / sizeof(T);
    const T* in = reinterpret_cast<const T*>(a.in);
    T* out = reinterpret_cast<T*>(a.out);
    const size_t V = ceil_div(a.n, E);
    const size_t base = scratch_half(a.scratch_off, a.scratch_bytes, seq);
    const size_t stride = (size_t)b.nblocks * b.nthreads;
    const size_t first = (size_t)b.bid * b.nthreads + threadIdx.x;
    for (size_t v = first; v < V; v += stride) st16(c.heap[rank] + base + v * 16, load_user_vec<T>(in, v, a.n));
    PK_BLOCK_BARRIER(c, rank, CH_BARRIER, b, flag_value(seq, 1), s_abort);
    if (s_abort) return;
    for (size_t v0 = first; v0 < V; v0 += kBatch * stride) {
      V16 r[kBatch];
#pragma unroll
      for (int u = 0; u < kBatch; ++u)
        if (v0 + u * stride < V) r[u] = multimem_ld_reduce<T>(c.mc + base + (v0 + u * stride) * 16);
#pragma unroll
      for (int u = 0; u < kBatch; ++u)
        if (v0 + u * stride < V) store_user_vec<T>(out, v0 + u * stride, a.n, r[u]);
    }
  }
  static __device__ void run(const CommCtx& c, int rank, const CollArgs& a, const Blk& b) {
    run_collective<NvlsOneShot<T>, CollArgs>(c, rank, a, b);
  }
};

// a.n = whole input; rank r gets the sum of shard r (a.n / world elements).
template <typename T>
struct NvlsReduceScatter {
  static __device__ void body(const CommCtx& c, int rank, const CollArgs& a, const Blk& b, u64 seq,
                              int& s_abort) {
    constexpr size_t E = 16 / sizeof(T);
    T* out = reinterpret_cast<T*>(a.out);
    const size_t shard = a.n / c.world;
    const size_t SV = ceil_div(shard, E);
    const size_t stride = (size_t)b.nblocks * b.nthreads;
    const size_t in_off = a.in_heap_off + (size_t)rank * shard * sizeof(T);  // 16-byte aligned
    PK_BLOCK_BARRIER(c, rank, CH_BARRIER, b, flag_value(seq, 1), s_abort);
    if (s_abort) return;
    for (size_t j = (size_t)b.bid * b.nthreads + threadIdx.x; j < SV; j += stride)
      store_user_vec<T>(out, j, shard, multimem_ld_reduce<T>(c.mc + in_off + j * 16));
    PK_BLOCK_BARRIER(c, rank, CH_BARRIER, b, flag_value(seq, 2), s_abort);
  }
  static __device__ void run(const CommCtx& c, int rank, const CollArgs& a, const Blk& b) {
    run_collective<NvlsReduceScatter<T>, CollArgs>(c, rank, a, b);
  }
};

// a.n = one shard (its byte size a multiple of 16); the output lives in the heap.
template <typename T>
struct NvlsAllGather {
  static __device__ void body(const CommCtx& c, int rank, const CollArgs& a, const Blk& b, u64 seq,
                              int& s_abort) {
    constexpr size_t E = 16 / sizeof(T);
    const T* in = reinterpret_cast<const T*>(a.in);
    const size_t SV = ceil_div(a.n, E);
    const size_t stride = (size_t)b.nblocks * b.nthreads;
    const size_t out_off = a.out_heap_off + (size_t)rank * a.n * sizeof(T);
    PK_BLOCK_BARRIER(c, rank, CH_BARRIER, b, flag_value(seq, 1), s_abort);
    if (s_abort) return;
    for (size_t j = (size_t)b.bid * b.nthreads + threadIdx.x; j < SV; j += stride)
      multimem_st(c.mc + out_off + j * 16, load_user_vec<T>(in, j, a.n));
    PK_BLOCK_BARRIER(c, rank, CH_BARRIER, b, flag_value(seq, 2), s_abort);
  }
  static __device__ void run(const CommCtx& c, int rank, const CollArgs& a, const Blk& b) {
    run_collective<NvlsAllGather<T>, CollArgs>(c, rank, a, b);
  }
};

static bool nvls_ok(const CommCtx& c, const LaunchCfg& cfg) {
  return c.mc != nullptr && cfg.emu_world <= 0;
}

size_t nvls_oneshot_scratch(size_t n, int elem_size) { return nvls_oneshot_scratch_bytes(n, elem_size); }

cudaError_t launch_all_reduce_nvls(int dtype, int kind, const CommCtx& c, const CollArgs* a,
                                   const LaunchCfg& cfg) {
  if (!nvls_ok(c, cfg)) return cudaErrorNotSupported;
  if (kind == NVLS_TWOSHOT && (a[0].in_heap_off == kNotInHeap || a[0].out_heap_off == kNotInHeap))
    return cudaErrorNotSupported;
  cudaError_t rc = cudaErrorInvalidValue;
  PENNY_DISPATCH_DTYPE(dtype, T, {
    rc = kind == NVLS_ONESHOT ? launch_body<NvlsOneShot<T>, CollArgs>(c, a, cfg)
                              : launch_body<NvlsTwoShot<T>, CollArgs>(c, a, cfg);
  });
  return rc;
}

cudaError_t launch_reduce_scatter_nvls(int dtype, const CommCtx& c, const CollArgs* a,
                                       const LaunchCfg& cfg) {
  if (!nvls_ok(c, cfg) || a[0].in_heap_off == kNotInHeap) return cudaErrorNotSupported;
  cudaError_t rc = cudaErrorInvalidValue;
  PENNY_DISPATCH_DTYPE(dtype, T, rc = (launch_body<NvlsReduceScatter<T>, CollArgs>(c, a, cfg)));
  return rc;
}

cudaError_t launch_all_gather_nvls(int dtype, const CommCtx& c, const CollArgs* a,
                                   const LaunchCfg& cfg) {
  if (!nvls_ok(c, cfg) || a[0].out_heap_off == kNotInHeap) return cudaErrorNotSupported;
  cudaError_t rc = cudaErrorInvalidValue;
  PENNY_DISPATCH_DTYPE(dtype, T, rc = (launch_body<NvlsAllGather<T>, CollArgs>(c, a, cfg)));
  return rc;
}

}  // namespace penny
