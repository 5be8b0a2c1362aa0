#include "symm_heap.h"

#include <cstring>

#include <unistd.h>

#include "../core/buffer.h"
#include "../core/status.h"
#include "../core/utils.h"
#include "../kernels/collectives.h"

namespace pplx {

namespace {

struct CudaFreeDeleter {
  void operator()(void* p) const {
    if (p) cudaFree(p);
  }
};

std::shared_ptr<void> alloc_zeroed(size_t bytes) {
  void* p = nullptr;
  CUDA_CHECK(cudaMalloc(&p, bytes));
  std::shared_ptr<void> owner(p, CudaFreeDeleter{});
  CUDA_CHECK(cudaMemset(p, 0, bytes));
  CUDA_CHECK(cudaDeviceSynchronize());
  return owner;
}

struct HandleBlob {
  cudaIpcMemHandle_t handle;
  int32_t device;
  int32_t pid;
  uint64_t bytes;
  char pci_bus_id[32];  // "0000:1b:00.0": identifies the GPU whatever each rank's device order
};

// Fails with a readable message when the peer's GPU is visible to this process but not
// reachable by loads and stores (no NVLink / PCIe P2P path).  A GPU this process cannot
// see at all (a narrowed CUDA_VISIBLE_DEVICES) is left to cudaIpcOpenMemHandle to judge.
void check_peer_reachable(int my_device, const HandleBlob& peer, int peer_rank) {
  if (peer.pci_bus_id[0] == '\0') return;
  int peer_device = -1;
  if (cudaDeviceGetByPCIBusId(&peer_device, peer.pci_bus_id) != cudaSuccess) {
    cudaGetLastError();  // not visible here: clear the sticky-free error and move on
    return;
  }
  if (peer_device == my_device) return;  // ranks that share a GPU
  int can = 0;
  if (cudaDeviceCanAccessPeer(&can, my_device, peer_device) != cudaSuccess) {
    cudaGetLastError();
    return;
  }
  PPLX_CHECK(can != 0, "peer access between device " << my_device << " and device " << peer_device
                           << " (rank " << peer_rank << ", " << peer.pci_bus_id
                           << ") is not available: all ranks of one object must sit in one "
                              "NVLink / PCIe peer-to-peer domain");
}

}  // namespace

SymmetricAllocation::~SymmetricAllocation() {
  for (size_t r = 0; r < peers_.size(); ++r) {
    if (ipc_opened_[r] && peers_[r] != nullptr) cudaIpcCloseMemHandle(peers_[r]);
  }
}

std::shared_ptr<SymmetricAllocation> SymmetricAllocation::create(Bootstrap& bs, size_t bytes) {
  PPLX_CHECK(bytes > 0, "empty symmetric allocation");
  const int world = bs.world();
  const int rank = bs.rank();
  auto alloc = std::shared_ptr<SymmetricAllocation>(new SymmetricAllocation());
  alloc->bytes_ = bytes;
  alloc->rank_ = rank;
  alloc->device_ = current_device();
  alloc->peers_.assign(world, nullptr);
  alloc->ipc_opened_.assign(world, false);
  const bool want_multicast = env_long("PPLX_B200_MULTIMEM", 0) != 0;
  if (world > 1 && (want_multicast || env_long("PPLX_B200_VMM", 0) != 0)) {
    // All ranks read the same environment, so they take this branch together.
    alloc->vmm_ = std::make_unique<VmmArena>();
    alloc->vmm_->create(bs, bytes, want_multicast);
    for (int r = 0; r < world; ++r) alloc->peers_[r] = alloc->vmm_->peer(r);
    bs.barrier();
    return alloc;
  }
  alloc->local_owner_ = alloc_zeroed(bytes);
  alloc->peers_[rank] = alloc->local_owner_.get();
  if (world == 1) return alloc;

  HandleBlob mine{};
  CUDA_CHECK(cudaIpcGetMemHandle(&mine.handle, alloc->local_owner_.get()));
  mine.device = alloc->device_;
  if (cudaDeviceGetPCIBusId(mine.pci_bus_id, sizeof(mine.pci_bus_id), alloc->device_) !=
      cudaSuccess) {
    cudaGetLastError();
    mine.pci_bus_id[0] = '\0';
  }
  mine.pid = static_cast<int32_t>(::getpid());
  mine.bytes = bytes;
  std::vector<HandleBlob> all(world);
  bs.all_gather(&mine, all.data(), sizeof(HandleBlob));
  for (int r = 0; r < world; ++r) {
    if (r == rank) continue;
    PPLX_CHECK(all[r].bytes == bytes, "symmetric allocation sizes differ: rank "
                                          << r << " has " << all[r].bytes << ", this rank "
                                          << bytes);
    PPLX_CHECK(all[r].pid != mine.pid,
               "two ranks share a process; use create_local_world for that");
    check_peer_reachable(alloc->device_, all[r], r);
    void* p = nullptr;
    CUDA_CHECK(cudaIpcOpenMemHandle(&p, all[r].handle, cudaIpcMemLazyEnablePeerAccess));
    alloc->peers_[r] = p;
    alloc->ipc_opened_[r] = true;
  }
  // No rank may touch a peer before that peer finished zero-filling.
  bs.barrier();
  return alloc;
}

std::vector<std::shared_ptr<SymmetricAllocation>> SymmetricAllocation::create_local_world(
    int n, size_t bytes) {
  PPLX_CHECK(n >= 1 && bytes > 0, "bad local world");
  std::vector<std::shared_ptr<void>> owners;
  std::vector<void*> ptrs;
  for (int r = 0; r < n; ++r) {
    owners.push_back(alloc_zeroed(bytes));
    ptrs.push_back(owners.back().get());
  }
  std::vector<std::shared_ptr<SymmetricAllocation>> out;
  for (int r = 0; r < n; ++r) {
    auto alloc = std::shared_ptr<SymmetricAllocation>(new SymmetricAllocation());
    alloc->bytes_ = bytes;
    alloc->rank_ = r;
    alloc->device_ = current_device();
    alloc->peers_ = ptrs;
    alloc->ipc_opened_.assign(n, false);
    // Every rank's view keeps all buffers alive.
    alloc->local_owner_ = std::make_shared<std::vector<std::shared_ptr<void>>>(owners);
    out.push_back(std::move(alloc));
  }
  return out;
}

StreamBarrier::StreamBarrier(Bootstrap& bs) {
  static_assert(sizeof(uint32_t) * (kBarrierMcWord + 1) <= kBarrierFlagBytes &&
                    sizeof(uint32_t) * kMaxWorld <= sizeof(uint32_t) * kBarrierMcWord,
                "barrier flag layout");
  flags_ = SymmetricAllocation::create(bs, kBarrierFlagBytes);
  CUDA_CHECK(cudaMalloc(&epoch_, sizeof(uint32_t)));
  CUDA_CHECK(cudaMemset(epoch_, 0, sizeof(uint32_t)));
  CUDA_CHECK(cudaMalloc(&status_, sizeof(Status)));
  CUDA_CHECK(cudaMemset(status_, 0, sizeof(Status)));
  timeout_ns_ = static_cast<uint64_t>(env_long("PPLX_B200_TIMEOUT_MS", 20000)) * 1000000ull;
}

StreamBarrier::~StreamBarrier() {
  if (epoch_) cudaFree(epoch_);
  if (status_) cudaFree(status_);
}

void StreamBarrier::run(cudaStream_t stream) {
  BarrierParams b{};
  PPLX_CHECK(flags_->world() <= kMaxWorld, "world too large");
  for (int r = 0; r < flags_->world(); ++r) b.peer[r] = static_cast<uint8_t*>(flags_->peer(r));
  b.mc = static_cast<uint8_t*>(flags_->multicast());
  b.epoch = epoch_;
  b.status = status_;
  b.timeout_ns = timeout_ns_;
  b.rank = flags_->rank();
  b.world = flags_->world();
  CUDA_CHECK(launch_barrier(b, stream));
}

Status StreamBarrier::read_status() const {
  Status s{};
  CUDA_CHECK(cudaMemcpy(&s, status_, sizeof(Status), cudaMemcpyDeviceToHost));
  return s;
}

}  // namespace pplx
