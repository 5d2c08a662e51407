// One-time, per-DEVICE setup of a kernel.  Function attributes (the dynamic
// shared-memory limit) belong to the device the call is made on, so a process
// that drives several GPUs has to raise the limit on each of them; a plain
// `static bool done` would only cover the first.  Thread-safe.
#pragma once
#include <cuda_runtime.h>

#include <map>
#include <mutex>
#include <utility>

namespace penny {

struct KernelSetup {
  cudaError_t rc = cudaSuccess;
  int pairs = 0;  // resident clusters of two CTAs (only when asked for)
};

// Raises `kernel`'s dynamic shared-memory limit to smem_bytes on the current
// device (once) and, if threads_for_pairs > 0, asks how many clusters of two
// CTAs of that many threads can be resident at a time (0 if the query fails).
inline KernelSetup kernel_setup(const void* kernel, int smem_bytes, int threads_for_pairs = 0) {
  static std::mutex mu;
  static std::map<std::pair<int, const void*>, KernelSetup> done;
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lock(mu);
  auto it = done.find({dev, kernel});
  if (it != done.end()) return it->second;
  KernelSetup ks;
  ks.rc = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
  if (ks.rc != cudaSuccess) {
    (void)cudaGetLastError();
    return ks;  // not cached: the caller reports the error, a later call may retry
  }
  if (threads_for_pairs > 0) {
    int sms = 0;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)sms & ~1u, 1, 1);
    cfg.blockDim = dim3((unsigned)threads_for_pairs, 1, 1);
    cfg.dynamicSmemBytes = (size_t)smem_bytes;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n <= 0) {
      (void)cudaGetLastError();
      n = sms / 2 - 2;  // conservative: a GPC with an odd SM count strands one SM
    }
    ks.pairs = n < sms / 2 ? n : sms / 2;
  }
  done[{dev, kernel}] = ks;
  return ks;
}

}  // namespace penny
