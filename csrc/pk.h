// Penny-B200 kernel primitives: one source for the device build (sm_100a) and
// for the host protocol simulator (threads + atomics).
//
// Every collective body in this library is written against this header only:
//   * CommCtx       – the peer-mapped symmetric heap as one rank sees it
//   * Blk           – which block of the launch the body is running as
//   * PK_FOR_THREADS / PK_SYNC – "all threads of the block run this, then meet"
//   * st_release_sys / ld_acquire_sys / wait_flag_ge – cross-GPU flags with a
//     bounded wait that records a status record instead of hanging
//   * ld16/st16 + Vec16<T> – 16-byte vectors reduced in fp32
//
// Compiled with -DPENNY_HOST_SIM the same bodies run on the CPU: a block is a
// std::thread that walks its "threads" sequentially, flags are __atomic
// builtins, and the heap is ordinary host memory.  That is how the flag
// protocols are checked (including under ThreadSanitizer) without a GPU.
//
// The role of this layer in the reference is played by NVSHMEM's device API
// (nvshmemx_putmem_signal_nbi_block / nvshmem_signal_wait_until, e.g.
// csrc/all_reduce_ring_standard.cu:101-107) and by the raw flag helpers of
// csrc/custom_all_reduce.cuh:164-253; those waits are unbounded, these are not.
#pragma once

#include <stddef.h>
#include <stdint.h>
#include <string.h>

// A plain C++ translation unit (no nvcc) gets the host flavour of everything.
#if !defined(__CUDACC__) && !defined(PENNY_HOST_SIM)
#define PENNY_HOST_SIM 1
#endif

#if defined(PENNY_HOST_SIM)
#include <chrono>
#include <thread>
#endif

#if defined(__CUDACC__) && !defined(PENNY_HOST_SIM)
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#define PK_HD __host__ __device__ __forceinline__
#define PK_DEV __device__ __forceinline__
#else
#define PK_HD inline
#define PK_DEV inline
#endif

namespace penny {

constexpr int kMaxRanks = 8;
// Flag rows per channel.  A launch may use at most this many blocks.
constexpr int kMaxBlocks = 512;
// Independent flag arrays, so that one call can run several kinds of
// handshake side by side (see SignalPad).
constexpr int kNumChannels = 5;

enum Channel : int {
  CH_BARRIER = 0,  // all-to-all "I am here" flags (start / end barriers)
  CH_DATA = 1,     // point-to-point "step s has landed" counters (rings, tree)
  CH_CREDIT = 2,   // receiver -> sender "slot is free again" credits (double ring)
  CH_USER = 3,     // pairwise exchange
  CH_FUSED = 4,    // fused GEMM / MoE tile flags
};

enum DType : int { DT_F32 = 0, DT_F16 = 1, DT_BF16 = 2 };
PK_HD int dtype_size(int dt) { return dt == DT_F32 ? 4 : 2; }

// Error codes written to CommCtx::status[0] by a wait that ran out.
enum StatusCode : uint32_t {
  ST_OK = 0,
  ST_TIMEOUT_BARRIER = 1,
  ST_TIMEOUT_DATA = 2,
  ST_TIMEOUT_CREDIT = 3,
  ST_TIMEOUT_LL = 4,
  ST_TIMEOUT_TILE = 5,
  ST_TIMEOUT_SELFTEST = 6,
  ST_BAD_ARGS = 7,
};
constexpr int kStatusWords = 16;

// Layout of the first bytes of every rank's heap (identical on all ranks).
//   call_seq             : number of collective calls this communicator has
//                          finished; read by every block at kernel entry and
//                          bumped by the last block to leave.  It lives in device
//                          memory, not in a kernel argument, so a replayed CUDA
//                          graph keeps counting.
//   flag[ch][block][src] : written only by block `block` of rank `src`.
// A flag value is flag_value(seq, step): 64-bit, unique per (call, step) and
// monotone, so flags are never reset and a stale value can never satisfy a
// later wait.  Collectives run one at a time per communicator (one stream).
struct SignalPad {
  // [SEQ_ALL]  collectives in which every rank depends on every rank
  // [SEQ_PAIR] pairwise exchange, which must not flip the scratch halves of the
  //            others: two ranks could otherwise drift two such calls apart
  unsigned long long call_seq[2];
  uint32_t done[2];
  uint32_t _pad[10];
  unsigned long long flag[kNumChannels][kMaxBlocks][kMaxRanks];
};
constexpr size_t kSignalPadBytes = (sizeof(SignalPad) + 4095) / 4096 * 4096;
// The status words follow the pad; user allocations start at kHeapReserved.
constexpr size_t kStatusOffset = kSignalPadBytes;
constexpr size_t kHeapReserved = kSignalPadBytes + 4096;
constexpr int kStepsPerCall = 64;
enum SeqKind : int { SEQ_ALL = 0, SEQ_PAIR = 1 };

// What a kernel needs to reach every peer.  heap[r] is rank r's heap as mapped
// into THIS process; mc is the NVLS multicast alias of the same range (or null).
struct CommCtx {
  char* heap[kMaxRanks];
  char* mc;
  int rank;
  int world;
  unsigned long long timeout_ns;
  uint32_t* status;  // kStatusWords words in this rank's own device memory
};

struct Blk {
  int bid;       // block index inside the collective
  int nblocks;   // blocks taking part
  int nthreads;  // threads per block
};

#if defined(PENNY_HOST_SIM)
#define PK_FOR_THREADS(blk, tid) for (int tid = 0; tid < (blk).nthreads; ++tid)
#define PK_SYNC(blk) ((void)0)
#define PK_SHARED(type, name) type name
#else
#define PK_FOR_THREADS(blk, tid) \
  for (int tid = threadIdx.x, _pk_once = 1; _pk_once; _pk_once = 0)
#define PK_SYNC(blk) __syncthreads()
#define PK_SHARED(type, name) __shared__ type name
#endif

PK_HD SignalPad* pad_of(const CommCtx& c, int r) {
  return reinterpret_cast<SignalPad*>(c.heap[r]);
}

// ---------------------------------------------------------------------------
// flags
// ---------------------------------------------------------------------------
#if defined(PENNY_HOST_SIM)
typedef unsigned long long u64;
PK_DEV void st_release_sys(u64* p, u64 v) { __atomic_store_n(p, v, __ATOMIC_RELEASE); }
PK_DEV u64 ld_acquire_sys(const u64* p) { return __atomic_load_n(p, __ATOMIC_ACQUIRE); }
PK_DEV uint32_t atomic_inc_dev(uint32_t* p) { return __atomic_fetch_add(p, 1u, __ATOMIC_ACQ_REL); }
PK_DEV void fence_dev() { __atomic_thread_fence(__ATOMIC_SEQ_CST); }
PK_DEV void fence_sys() { __atomic_thread_fence(__ATOMIC_SEQ_CST); }
PK_DEV uint64_t now_ns() {
  return (uint64_t)std::chrono::duration_cast<std::chrono::nanoseconds>(
             std::chrono::steady_clock::now().time_since_epoch())
      .count();
}
PK_DEV void spin_pause() { std::this_thread::yield(); }
PK_DEV uint32_t status_cas(uint32_t* p, uint32_t expect, uint32_t v) {
  __atomic_compare_exchange_n(p, &expect, v, false, __ATOMIC_ACQ_REL, __ATOMIC_ACQUIRE);
  return expect;
}
#else
typedef unsigned long long u64;
PK_DEV void st_release_sys(u64* p, u64 v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
PK_DEV u64 ld_acquire_sys(const u64* p) {
  u64 v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
PK_DEV uint32_t atomic_inc_dev(uint32_t* p) { return atomicAdd(p, 1u); }
PK_DEV void fence_dev() { __threadfence(); }
PK_DEV void fence_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
PK_DEV uint64_t now_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
PK_DEV void spin_pause() {}
PK_DEV uint32_t status_cas(uint32_t* p, uint32_t expect, uint32_t v) {
  return atomicCAS(p, expect, v);
}
#endif

// First failure wins.
PK_DEV void report_status(const CommCtx& c, uint32_t code, int peer, int bid, u64 want, u64 seen) {
  if (c.status == nullptr) return;
  if (status_cas(&c.status[0], 0u, code) == 0u) {
    c.status[1] = (uint32_t)c.rank;
    c.status[2] = (uint32_t)peer;
    c.status[3] = (uint32_t)bid;
    c.status[4] = (uint32_t)want;
    c.status[5] = (uint32_t)(want >> 32);
    c.status[6] = (uint32_t)seen;
    c.status[7] = (uint32_t)(seen >> 32);
  }
}

// Wait until *p >= want.  Gives up after c.timeout_ns and returns false after
// recording {code, rank, peer, block, want, seen}; never traps, never hangs.
PK_DEV bool wait_flag_ge(const u64* p, u64 want, const CommCtx& c, uint32_t code, int peer,
                         int bid) {
  u64 seen = ld_acquire_sys(p);
  if (seen >= want) return true;
  const uint64_t t0 = now_ns();
  for (uint32_t spin = 1;; ++spin) {
    seen = ld_acquire_sys(p);
    if (seen >= want) return true;
    if ((spin & 31u) == 0u) {
      if (now_ns() - t0 > c.timeout_ns) {
        report_status(c, code, peer, bid, want, seen);
        return false;
      }
      spin_pause();
    }
  }
}

// ---------------------------------------------------------------------------
// 16-byte vectors
// ---------------------------------------------------------------------------
struct alignas(16) V16 {
  uint32_t w[4];
};

#if defined(PENNY_HOST_SIM)
// Host stand-ins for the 16-bit float types: same bit layouts, conversions by
// the usual round-to-nearest-even rules.
struct HostBF16 {
  uint16_t bits;
};
struct HostF16 {
  uint16_t bits;
};
inline float to_f32(float v) { return v; }
inline float to_f32(HostBF16 v) {
  uint32_t u = (uint32_t)v.bits << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
inline void from_f32(float f, float& o) { o = f; }
inline void from_f32(float f, HostBF16& o) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) {
    o.bits = 0x7fc0;
    return;
  }
  u += 0x7fffu + ((u >> 16) & 1u);
  o.bits = (uint16_t)(u >> 16);
}
float host_half_to_float(uint16_t h);
uint16_t host_float_to_half(float f);
inline float to_f32(HostF16 v) { return host_half_to_float(v.bits); }
inline void from_f32(float f, HostF16& o) { o.bits = host_float_to_half(f); }
using bf16_t = HostBF16;
using f16_t = HostF16;
PK_DEV V16 ld16(const void* p) {
  V16 v;
  memcpy(&v, p, 16);
  return v;
}
PK_DEV void st16(void* p, const V16& v) { memcpy(p, &v, 16); }
PK_DEV V16 ld16_volatile(const void* p) {
  V16 v;
  const uint64_t* q = reinterpret_cast<const uint64_t*>(p);
  uint64_t a = __atomic_load_n(q, __ATOMIC_ACQUIRE);
  uint64_t b = __atomic_load_n(q + 1, __ATOMIC_ACQUIRE);
  memcpy(&v.w[0], &a, 8);
  memcpy(&v.w[2], &b, 8);
  return v;
}
PK_DEV void st16_volatile(void* p, const V16& v) {
  uint64_t a, b;
  memcpy(&a, &v.w[0], 8);
  memcpy(&b, &v.w[2], 8);
  uint64_t* q = reinterpret_cast<uint64_t*>(p);
  __atomic_store_n(q, a, __ATOMIC_RELEASE);
  __atomic_store_n(q + 1, b, __ATOMIC_RELEASE);
}
#else
using bf16_t = __nv_bfloat16;
using f16_t = __half;
PK_DEV float to_f32(float v) { return v; }
PK_DEV float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
PK_DEV float to_f32(__half v) { return __half2float(v); }
PK_DEV void from_f32(float f, float& o) { o = f; }
PK_DEV void from_f32(float f, __nv_bfloat16& o) { o = __float2bfloat16_rn(f); }
PK_DEV void from_f32(float f, __half& o) { o = __float2half_rn(f); }
PK_DEV V16 ld16(const void* p) {
  V16 v;
  asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3])
               : "l"(p)
               : "memory");
  return v;
}
PK_DEV void st16(void* p, const V16& v) {
  asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.w[0]), "r"(v.w[1]),
               "r"(v.w[2]), "r"(v.w[3])
               : "memory");
}
// Used by the flag-in-data protocol: must not be cached or reordered.
PK_DEV V16 ld16_volatile(const void* p) {
  V16 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3])
               : "l"(p)
               : "memory");
  return v;
}
PK_DEV void st16_volatile(void* p, const V16& v) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.w[0]),
               "r"(v.w[1]), "r"(v.w[2]), "r"(v.w[3])
               : "memory");
}
#endif

template <typename T>
struct VecTraits {
  static constexpr int kElems = 16 / (int)sizeof(T);
};

template <typename T>
PK_DEV void unpack_add(const V16& v, float (&acc)[16 / sizeof(T)]) {
  T e[16 / sizeof(T)];
  memcpy(e, &v, 16);
#pragma unroll
  for (int i = 0; i < (int)(16 / sizeof(T)); ++i) acc[i] += to_f32(e[i]);
}
template <typename T>
PK_DEV void unpack_set(const V16& v, float (&acc)[16 / sizeof(T)]) {
  T e[16 / sizeof(T)];
  memcpy(e, &v, 16);
#pragma unroll
  for (int i = 0; i < (int)(16 / sizeof(T)); ++i) acc[i] = to_f32(e[i]);
}
template <typename T>
PK_DEV V16 pack(const float (&acc)[16 / sizeof(T)]) {
  T e[16 / sizeof(T)];
#pragma unroll
  for (int i = 0; i < (int)(16 / sizeof(T)); ++i) from_f32(acc[i], e[i]);
  V16 v;
  memcpy(&v, e, 16);
  return v;
}

// Vector v of a user array of n elements of T.  The last vector may be ragged
// and the array may start off a 16-byte boundary: such vectors are read /
// written element by element so that nothing outside [0, n) is touched.
// Internal (heap) buffers are always whole, aligned vectors.
template <typename T>
PK_DEV V16 load_user_vec(const T* base, size_t v, size_t n) {
  constexpr size_t E = 16 / sizeof(T);
  if ((v + 1) * E <= n && (reinterpret_cast<uintptr_t>(base + v * E) & 15u) == 0)
    return ld16(base + v * E);
  T e[E];
#pragma unroll
  for (size_t i = 0; i < E; ++i) {
    float z = 0.f;
    T zt;
    from_f32(z, zt);
    e[i] = (v * E + i < n) ? base[v * E + i] : zt;
  }
  V16 out;
  memcpy(&out, e, 16);
  return out;
}
template <typename T>
PK_DEV void store_user_vec(T* base, size_t v, size_t n, const V16& val) {
  constexpr size_t E = 16 / sizeof(T);
  if ((v + 1) * E <= n && (reinterpret_cast<uintptr_t>(base + v * E) & 15u) == 0) {
    st16(base + v * E, val);
    return;
  }
  T e[E];
  memcpy(e, &val, 16);
#pragma unroll
  for (size_t i = 0; i < E; ++i)
    if (v * E + i < n) base[v * E + i] = e[i];
}

// Vectors a thread keeps in flight per pass of a copy loop: the loads of a
// batch are issued back to back before the first dependent store.
constexpr int kBatch = 4;

PK_HD size_t ceil_div(size_t a, size_t b) { return (a + b - 1) / b; }
PK_HD size_t round_up(size_t a, size_t b) { return ceil_div(a, b) * b; }

// ---------------------------------------------------------------------------
// call sequence + block-level synchronisation with the same block on every peer
// ---------------------------------------------------------------------------

// Every thread of every block reads the call number at entry.  It cannot change
// before the last block of this launch has gone through end_call.
PK_DEV u64 begin_call(const CommCtx& c, int rank, int kind) {
  return pad_of(c, rank)->call_seq[kind];
}

// Once per block, on every path out of a collective body.
PK_DEV void end_call(const CommCtx& c, int rank, const Blk& b, u64 seq, int kind) {
  PK_SYNC(b);
  PK_FOR_THREADS(b, tid) {
    if (tid == 0) {
      SignalPad* pad = pad_of(c, rank);
      fence_dev();
      if (atomic_inc_dev(&pad->done[kind]) == (uint32_t)b.nblocks - 1u) {
        pad->done[kind] = 0;
        fence_dev();
        pad->call_seq[kind] = seq + 1;
      }
    }
  }
}

PK_HD u64 flag_value(u64 seq, int step) { return seq * kStepsPerCall + (u64)step; }

// Scratch is lent to a call in two halves; call `seq` uses half seq & 1.  A peer
// can run at most one call ahead of this rank (it cannot finish call k before
// every rank has entered call k), so the half it writes is never the half this
// rank is still reading, whatever layout either call uses inside its half.
PK_HD size_t scratch_half(size_t scratch_off, size_t scratch_bytes, u64 seq) {
  return scratch_off + (size_t)(seq & 1ull) * (scratch_bytes / 2);
}

// Thread `t`: tell `peer` that this block reached (seq, step) on channel ch.
// Everything the block wrote before the preceding PK_SYNC becomes visible to a
// peer that acquires the flag (release is cumulative over the barrier).
PK_DEV void signal_peer(const CommCtx& c, int rank, int peer, int ch, const Blk& b, u64 val) {
  st_release_sys(&pad_of(c, peer)->flag[ch][b.bid][rank], val);
}
PK_DEV bool wait_peer(const CommCtx& c, int rank, int peer, int ch, const Blk& b, u64 val,
                      uint32_t code) {
  return wait_flag_ge(&pad_of(c, rank)->flag[ch][b.bid][peer], val, c, code, peer, b.bid);
}

// Full barrier among block b of every rank: signal all, wait for all.
// s_abort is set (for the whole block) if any wait timed out.
#define PK_BLOCK_BARRIER(c, rank, ch, b, val, s_abort)                              \
  do {                                                                              \
    PK_SYNC(b);                                                                     \
    PK_FOR_THREADS(b, _t) {                                                         \
      if (_t < (c).world && _t != (rank)) signal_peer(c, rank, _t, ch, b, val);     \
    }                                                                               \
    PK_FOR_THREADS(b, _t) {                                                         \
      if (_t < (c).world && _t != (rank)) {                                         \
        if (!wait_peer(c, rank, _t, ch, b, val, ST_TIMEOUT_BARRIER)) (s_abort) = 1; \
      }                                                                             \
    }                                                                               \
    PK_SYNC(b);                                                                     \
  } while (0)

// Wrapper used by every collective: zero the abort flag, read the call number,
// run Body::body, bump the call number.
template <class Body, class Args, int KIND = SEQ_ALL>
PK_DEV void run_collective(const CommCtx& c, int rank, const Args& a, const Blk& b) {
  PK_SHARED(int, s_abort);
  PK_FOR_THREADS(b, tid) {
    if (tid == 0) s_abort = 0;
  }
  const u64 seq = begin_call(c, rank, KIND);
  PK_SYNC(b);
  Body::body(c, rank, a, b, seq, s_abort);
  end_call(c, rank, b, seq, KIND);
}

}  // namespace penny
