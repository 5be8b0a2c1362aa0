// Device memory from the driver's virtual memory management API, shareable between the
// processes of one box as POSIX file descriptors, and NVLink multicast objects over it.
//
// Role parity: the reference obtains peer-visible memory from cudaIpc handles
// (intranode.cpp:63-122) or from NVSHMEM's symmetric heap (internode.cpp:36-68), whose
// NVLink transport is built on exactly these driver calls; NVSHMEM is not available here, so
// the library makes them itself.  What they add over cudaMalloc + cudaIpc:
//   * a physical allocation can be bound to a MULTICAST object: one store to the multicast
//     address lands in the memory of every rank (`multimem.st`), one reduction is applied
//     at every rank (`multimem.red`) -- the NVSwitch replicates, not the SM;
//   * the handle is a file descriptor, which a process can pass to exactly the peers it
//     chooses (SCM_RIGHTS over a unix socket) instead of a token any process may open.
//
// The driver entry points are resolved through the runtime (cudaGetDriverEntryPoint), so the
// library does not link against libcuda.
#pragma once

#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

#include "bootstrap.h"

namespace pplx {

// What the current device and driver offer.  `reason` says what is missing.
struct VmmSupport {
  bool vmm = false;        // cuMemCreate with POSIX file descriptor handles
  bool multicast = false;  // cuMulticastCreate (NVSwitch multicast and reductions)
  std::string reason;
};
VmmSupport query_vmm_support(int device);

// Collective: every rank passes one file descriptor (or -1 for "none") to every other rank
// of the box.  Returns, per rank, a descriptor owned by the caller (-1 where the peer sent
// none, and at the caller's own index).  The descriptors travel as SCM_RIGHTS messages over
// abstract unix-domain sockets whose names are exchanged through `bs`; every rank first
// connects to all peers, then serves the connections it received, then reads its answers,
// so no rank waits for a peer that waits for it.
std::vector<int> exchange_fds(Bootstrap& bs, int my_fd, int timeout_ms = 60000);

// One rank's share of a symmetric allocation made of driver allocations.
class VmmArena {
 public:
  VmmArena() = default;
  ~VmmArena();
  VmmArena(const VmmArena&) = delete;
  VmmArena& operator=(const VmmArena&) = delete;

  // Collective over `bs`.  Allocates at least `bytes` zero-filled bytes on the current
  // device, maps every peer's allocation, and -- with `want_multicast`, where every rank
  // sits on a GPU of its own that supports it -- binds all of them to one multicast object
  // and maps that too.  Throws the same error on every rank if any rank fails; a failure of
  // the multicast part alone leaves the arena without multicast (`multicast_note` says why).
  void create(Bootstrap& bs, size_t bytes, bool want_multicast);

  void* peer(int r) const { return reinterpret_cast<void*>(peer_va_[r]); }
  void* multicast() const { return reinterpret_cast<void*>(mc_va_); }
  const std::string& multicast_note() const { return multicast_note_; }
  size_t mapped_bytes() const { return size_; }
  int world() const { return static_cast<int>(peer_va_.size()); }

 private:
  void destroy() noexcept;
  void drop_multicast() noexcept;
  std::string multicast_note_;
  std::vector<uint64_t> peer_va_;      // CUdeviceptr per rank (own allocation at own index)
  std::vector<uint64_t> peer_handle_;  // CUmemGenericAllocationHandle per rank
  uint64_t mc_va_ = 0;
  uint64_t mc_handle_ = 0;
  bool mc_bound_ = false;
  size_t size_ = 0;  // rounded up to the allocation (and multicast) granularity
  int rank_ = 0;
  int device_ = 0;
};

}  // namespace pplx
