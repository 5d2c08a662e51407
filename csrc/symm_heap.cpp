#include "symm_heap.h"

#include <cuda.h>
#include <cuda_runtime.h>
#include <unistd.h>

#include <stdexcept>
#include <vector>

namespace penny {

namespace {

void* drv_symbol(const char* name) {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult st;
  cudaError_t rc = cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &st);
  if (rc != cudaSuccess || st != cudaDriverEntryPointSuccess || fn == nullptr) {
    (void)cudaGetLastError();
    throw std::runtime_error(std::string("penny heap: CUDA driver symbol not available: ") + name);
  }
  return fn;
}
#define DRV(name) reinterpret_cast<decltype(&name)>(drv_symbol(#name))

std::string drv_err(CUresult r) { return "CUresult " + std::to_string((int)r); }

void ck(CUresult r, const char* what) {
  if (r != CUDA_SUCCESS) throw std::runtime_error(std::string("penny heap: ") + what + ": " + drv_err(r));
}
void ckrt(cudaError_t r, const char* what) {
  if (r != cudaSuccess) {
    (void)cudaGetLastError();
    throw std::runtime_error(std::string("penny heap: ") + what + ": " + cudaGetErrorString(r));
  }
}

CUmemAllocationProp local_prop(int device) {
  CUmemAllocationProp prop = {};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return prop;
}

}  // namespace

SymmHeap::SymmHeap(Bootstrap* bs, int rank, int world, size_t bytes, int mode, bool want_multicast)
    : bs_(bs), rank_(rank), world_(world), bytes_(bytes), mode_(mode) {
  if (world < 1 || world > kMaxRanks) throw std::runtime_error("penny heap: world must be 1..8");
  ckrt(cudaGetDevice(&device_), "cudaGetDevice");
  ckrt(cudaFree(0), "context init");
  if (mode_ == HEAP_EMU) {
    create_emu();
    return;
  }
  if (bs_ == nullptr) throw std::runtime_error("penny heap: a bootstrap is required");
  if (mode_ == HEAP_AUTO || mode_ == HEAP_VMM) {
    // every rank must take the same path: agree on VMM support first
    int ok = 1;
    try {
      int fd_ok = 0;
      CUdevice dev;
      ck(DRV(cuDeviceGet)(&dev, device_), "cuDeviceGet");
      ck(DRV(cuDeviceGetAttribute)(
             &fd_ok, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, dev),
         "cuDeviceGetAttribute");
      ok = fd_ok ? 1 : 0;
    } catch (const std::exception&) {
      ok = 0;
    }
    std::vector<int> all(world_);
    bs_->all_gather(&ok, sizeof(ok), all.data());
    for (int v : all) ok = ok && v;
    if (ok) {
      mode_ = HEAP_VMM;
      create_vmm(want_multicast);
      return;
    }
    if (mode_ == HEAP_VMM) throw std::runtime_error("penny heap: VMM fd export not supported");
    mode_ = HEAP_IPC;
  }
  mc_note_ = "multicast needs the VMM heap";
  create_ipc();
}

SymmHeap::~SymmHeap() {
  try {
    destroy();
  } catch (...) {
  }
}

void SymmHeap::create_emu() {
  bytes_ = round_up(bytes_, 4096);
  for (int r = 0; r < world_; ++r) {
    void* p = nullptr;
    ckrt(cudaMalloc(&p, bytes_), "cudaMalloc (emulated rank heap)");
    ckrt(cudaMemset(p, 0, bytes_), "cudaMemset");
    base_[r] = (char*)p;
  }
  ckrt(cudaDeviceSynchronize(), "sync");
  mc_note_ = "multicast is not available in single-GPU emulation";
}

void SymmHeap::create_ipc() {
  bytes_ = round_up(bytes_, 2u << 20);
  void* p = nullptr;
  ckrt(cudaMalloc(&p, bytes_), "cudaMalloc (heap)");
  ckrt(cudaMemset(p, 0, bytes_), "cudaMemset");
  ckrt(cudaDeviceSynchronize(), "sync");
  base_[rank_] = (char*)p;
  cudaIpcMemHandle_t mine;
  ckrt(cudaIpcGetMemHandle(&mine, p), "cudaIpcGetMemHandle");
  std::vector<cudaIpcMemHandle_t> all(world_);
  bs_->all_gather(&mine, sizeof(mine), all.data());
  for (int r = 0; r < world_; ++r) {
    if (r == rank_) continue;
    void* q = nullptr;
    ckrt(cudaIpcOpenMemHandle(&q, all[r], cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
    base_[r] = (char*)q;
  }
  bs_->barrier();
}

void SymmHeap::create_vmm(bool want_multicast) {
  auto p_getgran = DRV(cuMemGetAllocationGranularity);
  auto p_create = DRV(cuMemCreate);
  auto p_export = DRV(cuMemExportToShareableHandle);
  auto p_import = DRV(cuMemImportFromShareableHandle);
  auto p_reserve = DRV(cuMemAddressReserve);
  auto p_map = DRV(cuMemMap);
  auto p_setaccess = DRV(cuMemSetAccess);

  CUmemAllocationProp prop = local_prop(device_);
  size_t gran = 0;
  ck(p_getgran(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED), "granularity");
  if (gran < (2u << 20)) gran = 2u << 20;
  // sized so that the multicast binding (which has its own granularity) fits too
  size_t mc_gran = 0;
  if (want_multicast) {
    try {
      CUmulticastObjectProp mp = {};
      mp.numDevices = (unsigned)world_;
      mp.size = round_up(bytes_, gran);
      mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
      if (DRV(cuMulticastGetGranularity)(&mc_gran, &mp, CU_MULTICAST_GRANULARITY_MINIMUM) !=
          CUDA_SUCCESS)
        mc_gran = 0;
    } catch (const std::exception&) {
      mc_gran = 0;
    }
  }
  // all ranks must use one size
  size_t want = round_up(bytes_, gran > mc_gran ? gran : mc_gran);
  std::vector<size_t> sizes(world_);
  bs_->all_gather(&want, sizeof(want), sizes.data());
  for (size_t s : sizes)
    if (s > want) want = s;
  bytes_ = want;

  CUmemGenericAllocationHandle mine;
  ck(p_create(&mine, bytes_, &prop, 0), "cuMemCreate");
  mem_handle_[rank_] = mine;
  int fd = -1;
  ck(p_export(&fd, mine, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0), "cuMemExportToShareableHandle");
  for (int p = 0; p < world_; ++p)
    if (p != rank_) bs_->send_fd(p, fd);
  for (int p = 0; p < world_; ++p) {
    if (p == rank_) continue;
    int pfd = bs_->recv_fd(p);
    CUmemGenericAllocationHandle h;
    ck(p_import(&h, (void*)(uintptr_t)pfd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR),
       "cuMemImportFromShareableHandle");
    close(pfd);
    mem_handle_[p] = h;
  }
  close(fd);

  CUmemAccessDesc access = {};
  access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  access.location.id = device_;
  access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  for (int r = 0; r < world_; ++r) {
    CUdeviceptr va = 0;
    ck(p_reserve(&va, bytes_, gran, 0, 0), "cuMemAddressReserve");
    ck(p_map(va, bytes_, 0, mem_handle_[r], 0), "cuMemMap");
    ck(p_setaccess(va, bytes_, &access, 1), "cuMemSetAccess");
    base_[r] = (char*)va;
  }
  ckrt(cudaMemset(base_[rank_], 0, bytes_), "cudaMemset");
  ckrt(cudaDeviceSynchronize(), "sync");
  bs_->barrier();
  if (want_multicast)
    setup_multicast();
  else
    mc_note_ = "multicast not requested";
}

// Every stage is followed by an agreement round, so that either all ranks end
// up with a multicast mapping or none does.
void SymmHeap::setup_multicast() {
  auto agree = [&](int ok) {
    std::vector<int> all(world_);
    bs_->all_gather(&ok, sizeof(ok), all.data());
    for (int v : all) ok = ok && v;
    return ok != 0;
  };
  int ok = 1;
  std::string why;
  CUdevice dev = 0;
  try {
    ck(DRV(cuDeviceGet)(&dev, device_), "cuDeviceGet");
    int sup = 0;
    ck(DRV(cuDeviceGetAttribute)(&sup, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev), "attr");
    if (!sup) {
      ok = 0;
      why = "device reports no multicast support";
    }
  } catch (const std::exception& e) {
    ok = 0;
    why = e.what();
  }
  if (!agree(ok)) {
    mc_note_ = why.empty() ? "a peer reports no multicast support" : why;
    return;
  }

  // stage 1: rank 0 creates and exports, the others import
  CUmemGenericAllocationHandle mc = 0;
  int fd = -1;
  try {
    if (rank_ == 0) {
      CUmulticastObjectProp mp = {};
      mp.numDevices = (unsigned)world_;
      mp.size = bytes_;
      mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
      ck(DRV(cuMulticastCreate)(&mc, &mp), "cuMulticastCreate");
      ck(DRV(cuMemExportToShareableHandle)(&fd, mc, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0),
         "export multicast");
    }
  } catch (const std::exception& e) {
    ok = 0;
    why = e.what();
  }
  if (!agree(ok)) {
    if (mc) DRV(cuMemRelease)(mc);
    if (fd >= 0) close(fd);
    mc_note_ = why.empty() ? "rank 0 could not create the multicast object" : why;
    return;
  }
  if (rank_ == 0) {
    for (int p = 1; p < world_; ++p) bs_->send_fd(p, fd);
    close(fd);
  } else {
    int pfd = bs_->recv_fd(0);
    try {
      ck(DRV(cuMemImportFromShareableHandle)(&mc, (void*)(uintptr_t)pfd,
                                             CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR),
         "import multicast");
    } catch (const std::exception& e) {
      ok = 0;
      why = e.what();
    }
    close(pfd);
  }
  // stage 2: add devices (all of them before anyone binds)
  if (ok) {
    try {
      ck(DRV(cuMulticastAddDevice)(mc, dev), "cuMulticastAddDevice");
    } catch (const std::exception& e) {
      ok = 0;
      why = e.what();
    }
  }
  if (!agree(ok)) {
    if (mc) DRV(cuMemRelease)(mc);
    mc_note_ = why.empty() ? "a peer could not join the multicast object" : why;
    return;
  }
  // stage 3: bind + map
  CUdeviceptr va = 0;
  bool mapped = false;
  try {
    ck(DRV(cuMulticastBindMem)(mc, 0, mem_handle_[rank_], 0, bytes_, 0), "cuMulticastBindMem");
    mc_bound_ = true;
    ck(DRV(cuMemAddressReserve)(&va, bytes_, 2u << 20, 0, 0), "reserve multicast va");
    ck(DRV(cuMemMap)(va, bytes_, 0, mc, 0), "map multicast");
    mapped = true;
    CUmemAccessDesc access = {};
    access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    access.location.id = device_;
    access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    ck(DRV(cuMemSetAccess)(va, bytes_, &access, 1), "access multicast");
  } catch (const std::exception& e) {
    ok = 0;
    why = e.what();
  }
  mc_handle_ = mc;
  if (!agree(ok)) {
    if (mapped) DRV(cuMemUnmap)(va, bytes_);
    if (va) DRV(cuMemAddressFree)(va, bytes_);
    if (mc_bound_) DRV(cuMulticastUnbind)(mc, dev, 0, bytes_);
    mc_bound_ = false;
    DRV(cuMemRelease)(mc);
    mc_handle_ = 0;
    mc_note_ = why.empty() ? "a peer could not bind the multicast object" : why;
    return;
  }
  mc_base_ = (char*)va;
  mc_note_ = "multicast bound";
}

void SymmHeap::destroy() {
  if (destroyed_) return;
  destroyed_ = true;
  (void)cudaDeviceSynchronize();
  if (mode_ == HEAP_EMU) {
    for (int r = 0; r < world_; ++r)
      if (base_[r]) cudaFree(base_[r]);
    return;
  }
  // nobody unbinds while a peer may still have a kernel touching this memory
  if (bs_) {
    try {
      bs_->barrier();
    } catch (...) {
    }
  }
  if (mode_ == HEAP_IPC) {
    for (int r = 0; r < world_; ++r) {
      if (!base_[r]) continue;
      if (r == rank_)
        cudaFree(base_[r]);
      else
        cudaIpcCloseMemHandle(base_[r]);
    }
    return;
  }
  try {
    auto p_unmap = DRV(cuMemUnmap);
    auto p_free = DRV(cuMemAddressFree);
    auto p_release = DRV(cuMemRelease);
    if (mc_base_) {
      p_unmap((CUdeviceptr)mc_base_, bytes_);
      p_free((CUdeviceptr)mc_base_, bytes_);
      mc_base_ = nullptr;
    }
    if (mc_handle_) {
      if (mc_bound_) {
        CUdevice dev;
        if (DRV(cuDeviceGet)(&dev, device_) == CUDA_SUCCESS)
          DRV(cuMulticastUnbind)(mc_handle_, dev, 0, bytes_);
      }
      p_release(mc_handle_);
      mc_handle_ = 0;
    }
    for (int r = 0; r < world_; ++r) {
      if (base_[r]) {
        p_unmap((CUdeviceptr)base_[r], bytes_);
        p_free((CUdeviceptr)base_[r], bytes_);
        base_[r] = nullptr;
      }
      if (mem_handle_[r]) {
        p_release(mem_handle_[r]);
        mem_handle_[r] = 0;
      }
    }
  } catch (...) {
  }
}

}  // namespace penny
