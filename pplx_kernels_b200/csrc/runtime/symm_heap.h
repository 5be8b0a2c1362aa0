// Symmetric device memory: every rank allocates a buffer of the same size and
// maps all peers' buffers into its own address space, so that a kernel can
// address "the same offset on rank r" with one table of base pointers.
//
// Role parity: replaces both mechanisms of the reference -- the per-peer
// cudaMalloc + cudaIpc{Get,Open}MemHandle buffers of AllToAllIntraNode
// (intranode.cpp:63-122) and NVSHMEM's symmetric heap (`nvshmem_malloc`,
// internode.cpp:36-68, bindings/nvshmem.cpp:49-62).  Inside one NVSwitch box all
// peers are reachable by load/store, so one implementation serves both API
// flavours.  Handles are exchanged through a `Bootstrap`.
//
// With PPLX_B200_VMM=1 the buffers come from the driver's virtual memory management API
// instead (runtime/vmm.h): file-descriptor handles passed between the ranks over unix
// sockets, and -- with PPLX_B200_MULTIMEM=1 on NVSwitch systems -- one multicast mapping of
// the whole allocation, through which a kernel reaches the same offset on ALL ranks with
// one `multimem` instruction.  Both are off by default: a process that dies while its
// memory is bound to a multicast object can raise NVLink errors on its peers' GPUs, so jobs
// that must survive the loss of a rank leave them off.
//
// A second construction path, `SymmetricAllocation::create_local_world`, places
// several ranks' buffers on ONE device inside one process.  It exists so that
// the multi-rank protocol can be exercised where fewer GPUs than ranks are
// available: all ranks then run inside a single cooperative grid.
#pragma once

#include <cstddef>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include <cuda_runtime.h>

#include "bootstrap.h"
#include "vmm.h"

namespace pplx {

class SymmetricAllocation {
 public:
  ~SymmetricAllocation();
  SymmetricAllocation(const SymmetricAllocation&) = delete;
  SymmetricAllocation& operator=(const SymmetricAllocation&) = delete;

  void* local() const { return peers_[rank_]; }
  void* peer(int r) const { return peers_[r]; }
  const std::vector<void*>& peers() const { return peers_; }
  size_t bytes() const { return bytes_; }
  int rank() const { return rank_; }
  int world() const { return static_cast<int>(peers_.size()); }
  // The multicast alias of the allocation (same offsets), or nullptr.
  void* multicast() const { return vmm_ ? vmm_->multicast() : nullptr; }
  bool from_vmm() const { return vmm_ != nullptr; }
  // Why multicast was asked for but is not there (empty otherwise).
  std::string multicast_note() const { return vmm_ ? vmm_->multicast_note() : std::string(); }

  // Collective over `bs`: allocates `bytes` zero-filled bytes on the current
  // device and maps every peer's buffer.
  static std::shared_ptr<SymmetricAllocation> create(Bootstrap& bs, size_t bytes);

  // `n` ranks on the current device of this process.
  static std::vector<std::shared_ptr<SymmetricAllocation>> create_local_world(int n, size_t bytes);

 private:
  SymmetricAllocation() = default;
  std::vector<void*> peers_;
  std::vector<bool> ipc_opened_;
  std::shared_ptr<void> local_owner_;  // frees the local buffer
  std::unique_ptr<VmmArena> vmm_;      // owns everything instead, when in use
  size_t bytes_ = 0;
  int rank_ = 0;
  int device_ = 0;
};

// World barrier on a stream, built on a symmetric flag array and a monotonically
// increasing epoch (no reset, so it can be captured in a CUDA graph and
// replayed).  Counterpart of nvshmemx_barrier_all_on_stream
// (bindings/nvshmem.cpp:66-69).
class StreamBarrier {
 public:
  explicit StreamBarrier(Bootstrap& bs);
  ~StreamBarrier();
  void run(cudaStream_t stream);
  struct Status read_status() const;

 private:
  std::shared_ptr<SymmetricAllocation> flags_;
  uint32_t* epoch_ = nullptr;
  struct Status* status_ = nullptr;
  uint64_t timeout_ns_;
};

}  // namespace pplx
