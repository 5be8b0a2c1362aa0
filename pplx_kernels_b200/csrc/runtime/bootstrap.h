// Host-side exchange of small blobs between the ranks of one job.  Used only at
// set-up time, to swap memory handles.
//
// Role parity: `Distributed` / `DistributedNVSHMEM` (csrc/core/distributed.h:9-40,
// distributed.cpp:7-33) and the unique-id bootstrap the reference gets from
// NVSHMEM (bindings/nvshmem.cpp:17-41).  Here the unique id names an abstract
// unix-domain socket that rank 0 listens on; the other ranks of the box connect
// to it and rank 0 relays every gather.  A torch ProcessGroup based
// implementation lives with the bindings.
#pragma once

#include <cstddef>
#include <cstdint>
#include <memory>
#include <string>
#include <vector>

namespace pplx {

class Bootstrap {
 public:
  virtual ~Bootstrap() = default;
  virtual int rank() const = 0;
  virtual int world() const = 0;

  // Every rank contributes `bytes` bytes; `out` receives world * bytes, rank order.
  virtual void all_gather(const void* in, void* out, size_t bytes) = 0;

  // Blob j of `in` (bytes_each long) ends up as blob `rank` ... of rank j's `out`.
  virtual void all_to_all(const void* in, void* out, size_t bytes_each);

  void barrier();
};

// world == 1.
class SingleBootstrap final : public Bootstrap {
 public:
  int rank() const override { return 0; }
  int world() const override { return 1; }
  void all_gather(const void* in, void* out, size_t bytes) override;
};

constexpr size_t kUniqueIdBytes = 128;

struct UniqueId {
  uint8_t bytes[kUniqueIdBytes];
};

// Creates the rendezvous socket (this process becomes the future rank 0) and
// returns the id to hand to the other ranks by any out-of-band means.
UniqueId create_unique_id();

// Star-topology bootstrap over the socket named by a unique id.
class SocketBootstrap final : public Bootstrap {
 public:
  SocketBootstrap(const UniqueId& uid, int rank, int world, int timeout_ms = 60000);
  ~SocketBootstrap() override;
  int rank() const override { return rank_; }
  int world() const override { return world_; }
  void all_gather(const void* in, void* out, size_t bytes) override;

 private:
  int rank_;
  int world_;
  int timeout_ms_;
  int listen_fd_ = -1;          // rank 0 only
  std::vector<int> peer_fds_;   // rank 0: fd per rank (own slot -1); others: [0] = hub
};

}  // namespace pplx
