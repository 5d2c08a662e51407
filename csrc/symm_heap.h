// Symmetric heap: one equally sized allocation per rank, every rank's piece
// mapped into every process, optionally bound to one NVLS multicast object.
//
//   VMM   cuMemCreate (exportable as a POSIX fd) -> fds passed over the
//         bootstrap sockets -> cuMemImportFromShareableHandle + cuMemMap on
//         every peer.  Required for NVLS: the same allocations are bound to a
//         multicast object (cuMulticastCreate/AddDevice/BindMem) whose mapping
//         is the address multimem.* instructions operate on.
//   IPC   cudaMalloc + cudaIpcGetMemHandle/OpenMemHandle.  No multicast.
//   EMU   `world` allocations on the current GPU of ONE process: the virtual
//         ranks of the single-GPU emulation.
//
// This replaces NVSHMEM's symmetric heap in the reference (nvshmem_malloc +
// nvshmemx_buffer_register, csrc/common.h:24-40) and generalises its
// cudaIpc-based shared buffers (csrc/custom_all_reduce.cu:258-301).
//
// The driver API is reached through cudaGetDriverEntryPoint, so the library
// does not link libcuda and can be imported on a machine without a GPU.
#pragma once
#include <stddef.h>

#include <string>

#include "bootstrap.h"
#include "pk.h"

namespace penny {

enum HeapMode : int { HEAP_AUTO = 0, HEAP_VMM = 1, HEAP_IPC = 2, HEAP_EMU = 3 };

class SymmHeap {
 public:
  // Collective over the bootstrap (bs may be null only for HEAP_EMU).
  SymmHeap(Bootstrap* bs, int rank, int world, size_t bytes, int mode, bool want_multicast);
  ~SymmHeap();
  SymmHeap(const SymmHeap&) = delete;
  SymmHeap& operator=(const SymmHeap&) = delete;

  char* base(int r) const { return base_[r]; }
  char* mc_base() const { return mc_base_; }
  size_t bytes() const { return bytes_; }
  int mode() const { return mode_; }
  bool has_multicast() const { return mc_base_ != nullptr; }
  const std::string& multicast_note() const { return mc_note_; }

  // Unbind / unmap everything.  Safe to call twice.  Every rank must get here
  // before any rank's process exits while the multicast object is still bound.
  void destroy();

 private:
  void create_vmm(bool want_multicast);
  void create_ipc();
  void create_emu();
  void setup_multicast();

  Bootstrap* bs_;
  int rank_, world_, device_ = 0;
  size_t bytes_;
  int mode_;
  char* base_[kMaxRanks] = {};
  char* mc_base_ = nullptr;
  std::string mc_note_;
  bool destroyed_ = false;
  // opaque driver handles (CUmemGenericAllocationHandle is an unsigned long long)
  unsigned long long mem_handle_[kMaxRanks] = {};
  unsigned long long mc_handle_ = 0;
  bool mc_bound_ = false;
};

}  // namespace penny
