// Process-global symmetric-memory runtime behind the `nvshmem_*` Python names.
//
// Role parity: the NVSHMEM host calls the reference wraps in
// csrc/bindings/nvshmem.cpp:17-98 (unique id, init, finalize, my_pe, n_pes,
// malloc, barrier_all, barrier_all_on_stream, alltoall).  NVSHMEM itself is not
// used; the calls are served by SymmetricAllocation + StreamBarrier.
#pragma once

#include <map>
#include <memory>
#include <mutex>

#include <cuda_runtime.h>

#include "bootstrap.h"
#include "symm_heap.h"

namespace pplx {

class Runtime {
 public:
  static Runtime& instance();

  void init(std::shared_ptr<Bootstrap> bs);
  void finalize();
  bool initialized() const { return bootstrap_ != nullptr; }
  int my_pe() const;
  int n_pes() const;
  Bootstrap& bootstrap();

  // Collective.  The returned allocation stays registered until `release`.
  std::shared_ptr<SymmetricAllocation> malloc(size_t bytes);
  void release(void* local_ptr);
  // Allocation that contains [ptr, ptr + bytes), or null.
  std::shared_ptr<SymmetricAllocation> find(const void* ptr, size_t bytes) const;

  void barrier_on_stream(cudaStream_t stream);
  void barrier_all();

  // dest and src are symmetric, world chunks of `chunk_bytes` each.
  void alltoall(void* dest, const void* src, size_t chunk_bytes, cudaStream_t stream);

 private:
  Runtime() = default;
  mutable std::mutex mu_;
  std::shared_ptr<Bootstrap> bootstrap_;
  std::unique_ptr<StreamBarrier> barrier_;
  std::map<const void*, std::shared_ptr<SymmetricAllocation>> allocs_;
};

}  // namespace pplx
