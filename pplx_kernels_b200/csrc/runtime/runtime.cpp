#include "runtime.h"

#include <algorithm>

#include "../core/status.h"
#include "../core/utils.h"
#include "../kernels/collectives.h"
#include "all_to_all.h"

namespace pplx {

Runtime& Runtime::instance() {
  static Runtime rt;
  return rt;
}

void Runtime::init(std::shared_ptr<Bootstrap> bs) {
  std::lock_guard<std::mutex> lock(mu_);
  PPLX_CHECK(bootstrap_ == nullptr, "runtime already initialised; call finalize first");
  PPLX_CHECK(bs->world() <= kMaxWorld, "at most " << kMaxWorld << " ranks are supported");
  bootstrap_ = std::move(bs);
  barrier_ = std::make_unique<StreamBarrier>(*bootstrap_);
}

void Runtime::finalize() {
  std::lock_guard<std::mutex> lock(mu_);
  if (bootstrap_ == nullptr) return;
  cudaDeviceSynchronize();
  // Peers may still be reading our memory until they reach this point too.
  bootstrap_->barrier();
  allocs_.clear();
  barrier_.reset();
  bootstrap_->barrier();
  bootstrap_.reset();
}

int Runtime::my_pe() const {
  PPLX_CHECK(bootstrap_ != nullptr, "runtime not initialised");
  return bootstrap_->rank();
}

int Runtime::n_pes() const {
  PPLX_CHECK(bootstrap_ != nullptr, "runtime not initialised");
  return bootstrap_->world();
}

Bootstrap& Runtime::bootstrap() {
  PPLX_CHECK(bootstrap_ != nullptr, "runtime not initialised (call nvshmem_init first)");
  return *bootstrap_;
}

std::shared_ptr<SymmetricAllocation> Runtime::malloc(size_t bytes) {
  std::lock_guard<std::mutex> lock(mu_);
  PPLX_CHECK(bootstrap_ != nullptr, "runtime not initialised");
  auto a = SymmetricAllocation::create(*bootstrap_, round_up<size_t>(std::max<size_t>(bytes, 16), 256));
  allocs_[a->local()] = a;
  return a;
}

void Runtime::release(void* local_ptr) {
  std::lock_guard<std::mutex> lock(mu_);
  allocs_.erase(local_ptr);
}

std::shared_ptr<SymmetricAllocation> Runtime::find(const void* ptr, size_t bytes) const {
  std::lock_guard<std::mutex> lock(mu_);
  auto it = allocs_.upper_bound(ptr);
  if (it == allocs_.begin()) return nullptr;
  --it;
  const uint8_t* base = static_cast<const uint8_t*>(it->first);
  const uint8_t* p = static_cast<const uint8_t*>(ptr);
  if (p >= base && p + bytes <= base + it->second->bytes()) return it->second;
  return nullptr;
}

void Runtime::barrier_on_stream(cudaStream_t stream) {
  PPLX_CHECK(barrier_ != nullptr, "runtime not initialised");
  barrier_->run(stream);
}

void Runtime::barrier_all() {
  barrier_on_stream(nullptr);
  CUDA_CHECK(cudaStreamSynchronize(nullptr));
  const Status s = barrier_->read_status();
  if (s.code != kOk) throw Error("pplx_kernels_b200: " + describe_status(s));
}

void Runtime::alltoall(void* dest, const void* src, size_t chunk_bytes, cudaStream_t stream) {
  const int world = n_pes();
  auto d = find(dest, chunk_bytes * world);
  PPLX_CHECK(d != nullptr, "alltoall: dest must come from nvshmem_malloc");
  PPLX_CHECK(chunk_bytes % 16 == 0 && reinterpret_cast<uintptr_t>(dest) % 16 == 0 &&
                 reinterpret_cast<uintptr_t>(src) % 16 == 0,
             "alltoall: buffers and per-rank chunks must be multiples of 16 bytes");
  const size_t off = static_cast<const uint8_t*>(dest) - static_cast<const uint8_t*>(d->local());
  AllToAllCopyParams a{};
  for (int r = 0; r < world; ++r) a.peer_dst[r] = static_cast<uint8_t*>(d->peer(r)) + off;
  a.src = static_cast<const uint8_t*>(src);
  a.chunk_bytes = chunk_bytes;
  a.rank = my_pe();
  a.world = world;
  // Enough blocks to keep every SM storing: about two waves over all peers.
  const int per_peer = std::max(1, 2 * get_sm_count() / world);
  const int blocks = static_cast<int>(
      std::clamp<size_t>(chunk_bytes / (16 * 512 * 4), 1, static_cast<size_t>(per_peer)));
  CUDA_CHECK(launch_alltoall_copy(a, blocks, stream));
  barrier_on_stream(stream);
}

}  // namespace pplx
