// Programmatic dependent launch: the kernels of a decode step are launched so
// that kernel k + 1 may become resident while kernel k is still running.  Its
// prologue (barrier set-up, TMEM allocation, tensor-map fetch, and the loads of
// operands that no earlier kernel writes: weights, KV-cache tiles) then overlaps
// the tail of kernel k; only its first access to data that kernel k produces
// waits for kernel k to finish.  Inside a CUDA graph the launch attribute
// becomes a programmatic edge, so a captured step keeps the overlap.
//
// Rules every kernel launched through launch_kernel_ex(pdl = true) follows:
//   * pdl_launch_dependents() early (any thread; the next kernel is released
//     once every CTA has issued it or exited);
//   * pdl_wait() in EVERY thread before that thread's first global-memory access
//     to anything a preceding kernel may write or still read (outputs included);
//     it returns at once when there is nothing to wait for, and is a no-op in a
//     launch without the attribute;
//   * a kernel never exits without having waited, so "kernel k finished" implies
//     "everything before k finished".
// A kernel launched without the attribute after one of these serialises as
// usual (it starts when its predecessor has completed).
//
// The reference launches everything with plain <<< >>> on one stream; its
// kernels are separated by full launch gaps (e.g. csrc/custom_all_reduce.cuh:
// 803-841 chooses and launches one kernel per call).
#pragma once
#include <cuda_runtime.h>

namespace penny {

#if defined(__CUDACC__)
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
#endif

// Process-wide switch (PENNY_PDL=0 turns the attribute off everywhere; the
// kernels then run strictly one after the other).  set_pdl_enabled(-1) returns to
// the environment's choice.
bool pdl_enabled();
void set_pdl_enabled(int on);

// cudaLaunchKernelEx with an optional cluster shape and the programmatic
// stream-serialization attribute.  cluster_x <= 1: no cluster.
template <typename... KArgs, typename... Args>
cudaError_t launch_kernel_ex(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                             cudaStream_t stream, bool pdl, int cluster_x, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n = 0;
  if (cluster_x > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = (unsigned)cluster_x;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  if (pdl && pdl_enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = (unsigned)n;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace penny
