#include "vmm.h"

#include <cerrno>
#include <chrono>
#include <cstdio>
#include <cstring>
#include <mutex>

#include <poll.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <cuda.h>
#include <cuda_runtime.h>

#include "../core/utils.h"

namespace pplx {
namespace {

// ---- driver entry points, resolved once through the runtime ---------------------------------

struct DriverApi {
  decltype(&cuGetErrorString) GetErrorString = nullptr;
  decltype(&cuDeviceGetAttribute) DeviceGetAttribute = nullptr;
  decltype(&cuMemGetAllocationGranularity) MemGetAllocationGranularity = nullptr;
  decltype(&cuMemCreate) MemCreate = nullptr;
  decltype(&cuMemRelease) MemRelease = nullptr;
  decltype(&cuMemExportToShareableHandle) MemExportToShareableHandle = nullptr;
  decltype(&cuMemImportFromShareableHandle) MemImportFromShareableHandle = nullptr;
  decltype(&cuMemAddressReserve) MemAddressReserve = nullptr;
  decltype(&cuMemAddressFree) MemAddressFree = nullptr;
  decltype(&cuMemMap) MemMap = nullptr;
  decltype(&cuMemUnmap) MemUnmap = nullptr;
  decltype(&cuMemSetAccess) MemSetAccess = nullptr;
  decltype(&cuMulticastCreate) MulticastCreate = nullptr;
  decltype(&cuMulticastAddDevice) MulticastAddDevice = nullptr;
  decltype(&cuMulticastBindMem) MulticastBindMem = nullptr;
  decltype(&cuMulticastUnbind) MulticastUnbind = nullptr;
  decltype(&cuMulticastGetGranularity) MulticastGetGranularity = nullptr;
  bool vmm_ok = false;
  bool multicast_ok = false;
  std::string missing;
};

template <typename Fn>
bool resolve(const char* name, Fn& fn, std::string& missing) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess || p == nullptr) {
    cudaGetLastError();
    if (!missing.empty()) missing += ", ";
    missing += name;
    return false;
  }
  fn = reinterpret_cast<Fn>(p);
  return true;
}

const DriverApi& driver() {
  static DriverApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    bool v = true, m = true;
    v &= resolve("cuGetErrorString", api.GetErrorString, api.missing);
    v &= resolve("cuDeviceGetAttribute", api.DeviceGetAttribute, api.missing);
    v &= resolve("cuMemGetAllocationGranularity", api.MemGetAllocationGranularity, api.missing);
    v &= resolve("cuMemCreate", api.MemCreate, api.missing);
    v &= resolve("cuMemRelease", api.MemRelease, api.missing);
    v &= resolve("cuMemExportToShareableHandle", api.MemExportToShareableHandle, api.missing);
    v &= resolve("cuMemImportFromShareableHandle", api.MemImportFromShareableHandle, api.missing);
    v &= resolve("cuMemAddressReserve", api.MemAddressReserve, api.missing);
    v &= resolve("cuMemAddressFree", api.MemAddressFree, api.missing);
    v &= resolve("cuMemMap", api.MemMap, api.missing);
    v &= resolve("cuMemUnmap", api.MemUnmap, api.missing);
    v &= resolve("cuMemSetAccess", api.MemSetAccess, api.missing);
    m &= resolve("cuMulticastCreate", api.MulticastCreate, api.missing);
    m &= resolve("cuMulticastAddDevice", api.MulticastAddDevice, api.missing);
    m &= resolve("cuMulticastBindMem", api.MulticastBindMem, api.missing);
    m &= resolve("cuMulticastUnbind", api.MulticastUnbind, api.missing);
    m &= resolve("cuMulticastGetGranularity", api.MulticastGetGranularity, api.missing);
    api.vmm_ok = v;
    api.multicast_ok = v && m;
  });
  return api;
}

std::string cu_error(CUresult r) {
  const char* s = nullptr;
  const DriverApi& d = driver();
  if (d.GetErrorString != nullptr && d.GetErrorString(r, &s) == CUDA_SUCCESS && s != nullptr)
    return std::string(s) + " (CUresult " + std::to_string(static_cast<int>(r)) + ")";
  return "CUresult " + std::to_string(static_cast<int>(r));
}

}  // namespace

VmmSupport query_vmm_support(int device) {
  VmmSupport s;
  const DriverApi& d = driver();
  if (!d.vmm_ok) {
    s.reason = "driver entry points not found: " + d.missing;
    return s;
  }
  int vmm = 0, fd = 0, mc = 0;
  if (d.DeviceGetAttribute(&vmm, CU_DEVICE_ATTRIBUTE_VIRTUAL_MEMORY_MANAGEMENT_SUPPORTED, device) !=
          CUDA_SUCCESS ||
      d.DeviceGetAttribute(&fd, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED,
                           device) != CUDA_SUCCESS) {
    s.reason = "device attributes could not be read";
    return s;
  }
  s.vmm = vmm != 0 && fd != 0;
  if (!s.vmm) {
    s.reason = "the device does not export allocations as POSIX file descriptors";
    return s;
  }
  if (!d.multicast_ok) {
    s.reason = "multicast entry points not found: " + d.missing;
  } else if (d.DeviceGetAttribute(&mc, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, device) !=
                 CUDA_SUCCESS ||
             mc == 0) {
    s.reason = "the device reports no NVSwitch multicast support";
  } else {
    s.multicast = true;
  }
  return s;
}

// ---- file descriptors between the processes of one box ---------------------------------------

namespace {

struct FdGuard {
  std::vector<int> fds;
  ~FdGuard() {
    for (int fd : fds)
      if (fd >= 0) ::close(fd);
  }
  int add(int fd) {
    fds.push_back(fd);
    return fd;
  }
};

socklen_t abstract_address(const char* name, sockaddr_un* addr) {
  std::memset(addr, 0, sizeof(*addr));
  addr->sun_family = AF_UNIX;
  const size_t n = std::strlen(name);
  PPLX_CHECK(n + 1 < sizeof(addr->sun_path), "socket name too long");
  addr->sun_path[0] = '\0';
  std::memcpy(addr->sun_path + 1, name, n);
  return static_cast<socklen_t>(offsetof(sockaddr_un, sun_path) + 1 + n);
}

void wait_readable(int fd, int timeout_ms, const char* what) {
  pollfd p{fd, POLLIN, 0};
  int rc;
  do {
    rc = ::poll(&p, 1, timeout_ms);
  } while (rc < 0 && errno == EINTR);
  PPLX_CHECK(rc > 0, "exchange_fds: timed out waiting for " << what);
}

// One byte of payload, and the descriptor as ancillary data when there is one.
void send_fd(int sock, int fd) {
  char payload = fd >= 0 ? 1 : 0;
  iovec iov{&payload, 1};
  alignas(cmsghdr) char control[CMSG_SPACE(sizeof(int))];
  msghdr msg{};
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  if (fd >= 0) {
    std::memset(control, 0, sizeof(control));
    msg.msg_control = control;
    msg.msg_controllen = sizeof(control);
    cmsghdr* c = CMSG_FIRSTHDR(&msg);
    c->cmsg_level = SOL_SOCKET;
    c->cmsg_type = SCM_RIGHTS;
    c->cmsg_len = CMSG_LEN(sizeof(int));
    std::memcpy(CMSG_DATA(c), &fd, sizeof(int));
  }
  ssize_t rc;
  do {
    rc = ::sendmsg(sock, &msg, MSG_NOSIGNAL);
  } while (rc < 0 && errno == EINTR);
  PPLX_CHECK(rc == 1, "exchange_fds: sendmsg failed: " << std::strerror(errno));
}

int recv_fd(int sock, int timeout_ms) {
  wait_readable(sock, timeout_ms, "a peer's descriptor");
  char payload = 0;
  iovec iov{&payload, 1};
  alignas(cmsghdr) char control[CMSG_SPACE(sizeof(int))];
  std::memset(control, 0, sizeof(control));
  msghdr msg{};
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = control;
  msg.msg_controllen = sizeof(control);
  ssize_t rc;
  do {
    rc = ::recvmsg(sock, &msg, MSG_CMSG_CLOEXEC);
  } while (rc < 0 && errno == EINTR);
  PPLX_CHECK(rc == 1, "exchange_fds: recvmsg failed: " << std::strerror(errno));
  if (payload == 0) return -1;
  for (cmsghdr* c = CMSG_FIRSTHDR(&msg); c != nullptr; c = CMSG_NXTHDR(&msg, c)) {
    if (c->cmsg_level == SOL_SOCKET && c->cmsg_type == SCM_RIGHTS) {
      int fd = -1;
      std::memcpy(&fd, CMSG_DATA(c), sizeof(int));
      return fd;
    }
  }
  PPLX_CHECK(false, "exchange_fds: a peer announced a descriptor but none arrived");
  return -1;
}

}  // namespace

std::vector<int> exchange_fds(Bootstrap& bs, int my_fd, int timeout_ms) {
  const int world = bs.world(), rank = bs.rank();
  std::vector<int> out(world, -1);
  if (world == 1) return out;
  static std::mutex mu;
  static unsigned counter = 0;
  FdGuard guard;

  // Listen first, then tell the others where.
  char name[64];
  {
    std::lock_guard<std::mutex> lock(mu);
    std::snprintf(name, sizeof(name), "pplx-b200-fd-%d-%u", static_cast<int>(::getpid()),
                  counter++);
  }
  const int listener = guard.add(::socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0));
  PPLX_CHECK(listener >= 0, "exchange_fds: socket: " << std::strerror(errno));
  sockaddr_un addr;
  socklen_t len = abstract_address(name, &addr);
  PPLX_CHECK(::bind(listener, reinterpret_cast<sockaddr*>(&addr), len) == 0,
             "exchange_fds: bind: " << std::strerror(errno));
  PPLX_CHECK(::listen(listener, world) == 0, "exchange_fds: listen: " << std::strerror(errno));
  std::vector<char> names(static_cast<size_t>(world) * sizeof(name));
  bs.all_gather(name, names.data(), sizeof(name));

  // Connect to every peer (completes against the backlog, before the peer accepts) and say
  // who is calling.
  std::vector<int> outgoing(world, -1);
  for (int r = 0; r < world; ++r) {
    if (r == rank) continue;
    const int s = guard.add(::socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0));
    PPLX_CHECK(s >= 0, "exchange_fds: socket: " << std::strerror(errno));
    len = abstract_address(names.data() + static_cast<size_t>(r) * sizeof(name), &addr);
    PPLX_CHECK(::connect(s, reinterpret_cast<sockaddr*>(&addr), len) == 0,
               "exchange_fds: connect to rank " << r << ": " << std::strerror(errno));
    const int32_t me = rank;
    PPLX_CHECK(::send(s, &me, sizeof(me), MSG_NOSIGNAL) == sizeof(me),
               "exchange_fds: send: " << std::strerror(errno));
    outgoing[r] = s;
  }
  // Serve the world - 1 callers.
  for (int i = 0; i < world - 1; ++i) {
    wait_readable(listener, timeout_ms, "a peer to connect");
    const int c = guard.add(::accept4(listener, nullptr, nullptr, SOCK_CLOEXEC));
    PPLX_CHECK(c >= 0, "exchange_fds: accept: " << std::strerror(errno));
    wait_readable(c, timeout_ms, "a peer's rank");
    int32_t who = -1;
    PPLX_CHECK(::recv(c, &who, sizeof(who), MSG_WAITALL) == sizeof(who) && who >= 0 &&
                   who < world && who != rank,
               "exchange_fds: bad greeting");
    send_fd(c, my_fd);
  }
  // Collect the answers.  Should one of them fail, the descriptors already received are closed.
  try {
    for (int r = 0; r < world; ++r) {
      if (r != rank) out[r] = recv_fd(outgoing[r], timeout_ms);
    }
    // Nobody closes a socket a peer may still read from.
    bs.barrier();
  } catch (...) {
    for (int fd : out)
      if (fd >= 0) ::close(fd);
    throw;
  }
  return out;
}

// ---- the arena -------------------------------------------------------------------------------

namespace {

// Every rank reports the outcome of a step; all of them throw if any of them failed, so that
// no rank is left waiting in the next collective.
void agree(Bootstrap& bs, CUresult mine, const char* step) {
  const int32_t code = static_cast<int32_t>(mine);
  std::vector<int32_t> all(bs.world());
  bs.all_gather(&code, all.data(), sizeof(code));
  for (int r = 0; r < bs.world(); ++r) {
    PPLX_CHECK(all[r] == 0, "VMM arena: " << step << " failed on rank " << r << ": "
                                          << cu_error(static_cast<CUresult>(all[r])));
  }
}

// The same for a step that may fail without ending the set-up: false (and a note) on every
// rank if any rank failed.
bool all_ok(Bootstrap& bs, CUresult mine, const char* step, std::string* note) {
  const int32_t code = static_cast<int32_t>(mine);
  std::vector<int32_t> all(bs.world());
  bs.all_gather(&code, all.data(), sizeof(code));
  for (int r = 0; r < bs.world(); ++r) {
    if (all[r] != 0) {
      *note = std::string(step) + " failed on rank " + std::to_string(r) + ": " +
              cu_error(static_cast<CUresult>(all[r]));
      return false;
    }
  }
  return true;
}

CUmemAllocationProp device_prop(int device) {
  CUmemAllocationProp prop{};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return prop;
}

// Reserves an address range, maps `handle` there and opens it for `device`.
CUresult map_for(const DriverApi& d, CUmemGenericAllocationHandle handle, size_t size,
                 size_t align, int device, CUdeviceptr* va) {
  *va = 0;
  CUresult rc = d.MemAddressReserve(va, size, align, 0, 0);
  if (rc != CUDA_SUCCESS) return rc;
  rc = d.MemMap(*va, size, 0, handle, 0);
  if (rc != CUDA_SUCCESS) {
    d.MemAddressFree(*va, size);
    *va = 0;
    return rc;
  }
  CUmemAccessDesc access{};
  access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  access.location.id = device;
  access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  rc = d.MemSetAccess(*va, size, &access, 1);
  if (rc != CUDA_SUCCESS) {
    d.MemUnmap(*va, size);
    d.MemAddressFree(*va, size);
    *va = 0;
  }
  return rc;
}

}  // namespace

VmmArena::~VmmArena() { destroy(); }

void VmmArena::drop_multicast() noexcept {
  const DriverApi& d = driver();
  if (!d.multicast_ok) return;
  if (mc_va_ != 0) {
    d.MemUnmap(mc_va_, size_);
    d.MemAddressFree(mc_va_, size_);
    mc_va_ = 0;
  }
  if (mc_handle_ != 0) {
    if (mc_bound_) d.MulticastUnbind(mc_handle_, device_, 0, size_);
    d.MemRelease(mc_handle_);
    mc_handle_ = 0;
    mc_bound_ = false;
  }
}

void VmmArena::destroy() noexcept {
  const DriverApi& d = driver();
  if (!d.vmm_ok) return;
  // The multicast mapping goes first, then the binding, then the memory it was bound to.
  drop_multicast();
  for (size_t r = 0; r < peer_va_.size(); ++r) {
    if (peer_va_[r] != 0) {
      d.MemUnmap(peer_va_[r], size_);
      d.MemAddressFree(peer_va_[r], size_);
    }
    if (r < peer_handle_.size() && peer_handle_[r] != 0) d.MemRelease(peer_handle_[r]);
  }
  peer_va_.clear();
  peer_handle_.clear();
}

void VmmArena::create(Bootstrap& bs, size_t bytes, bool want_multicast) {
  const DriverApi& d = driver();
  const int world = bs.world();
  rank_ = bs.rank();
  device_ = current_device();
  CUDA_CHECK(cudaFree(nullptr));  // the runtime's context exists before the driver is called

  // Do all ranks agree on what can be done?
  const VmmSupport support = query_vmm_support(device_);
  struct Caps {
    int32_t vmm, multicast;
    char pci_bus_id[32];
  } mine{support.vmm ? 1 : 0, support.multicast && want_multicast ? 1 : 0, {}};
  if (cudaDeviceGetPCIBusId(mine.pci_bus_id, sizeof(mine.pci_bus_id), device_) != cudaSuccess) {
    cudaGetLastError();
    std::snprintf(mine.pci_bus_id, sizeof(mine.pci_bus_id), "rank-%d", rank_);
  }
  std::vector<Caps> caps(world);
  bs.all_gather(&mine, caps.data(), sizeof(Caps));
  bool multicast = world > 1;
  for (int r = 0; r < world; ++r) {
    PPLX_CHECK(caps[r].vmm != 0, "VMM arena: rank " << r << " cannot use it"
                                                    << (r == rank_ ? ": " + support.reason : ""));
    multicast = multicast && caps[r].multicast != 0;
    // A multicast object takes every GPU once.
    for (int q = 0; q < r; ++q)
      if (std::strncmp(caps[q].pci_bus_id, caps[r].pci_bus_id, sizeof(mine.pci_bus_id)) == 0)
        multicast = false;
  }

  // Size: a multiple of the allocation granularity, and of the multicast granularity.
  const CUmemAllocationProp prop = device_prop(device_);
  size_t gran = 0;
  CUresult rc = d.MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED);
  CUmulticastObjectProp mc_prop{};
  if (rc == CUDA_SUCCESS && multicast) {
    mc_prop.numDevices = static_cast<unsigned>(world);
    mc_prop.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    mc_prop.size = round_up<size_t>(bytes, gran);
    size_t mc_gran = 0;
    rc = d.MulticastGetGranularity(&mc_gran, &mc_prop, CU_MULTICAST_GRANULARITY_RECOMMENDED);
    if (rc == CUDA_SUCCESS && mc_gran > gran) gran = mc_gran;
  }
  agree(bs, rc, "querying the granularity");
  size_ = round_up<size_t>(bytes, gran);
  mc_prop.size = size_;

  // This rank's memory, and a descriptor for it.
  peer_va_.assign(world, 0);
  peer_handle_.assign(world, 0);
  CUmemGenericAllocationHandle own = 0;
  int own_fd = -1;
  rc = d.MemCreate(&own, size_, &prop, 0);
  if (rc == CUDA_SUCCESS) {
    peer_handle_[rank_] = own;
    rc = d.MemExportToShareableHandle(&own_fd, own, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  }
  if (rc == CUDA_SUCCESS) {
    CUdeviceptr va = 0;
    rc = map_for(d, own, size_, gran, device_, &va);
    peer_va_[rank_] = va;
  }
  agree(bs, rc, "allocating");
  CUDA_CHECK(cudaMemset(reinterpret_cast<void*>(peer_va_[rank_]), 0, size_));
  CUDA_CHECK(cudaDeviceSynchronize());

  // Everybody's memory, mapped here.
  std::vector<int> fds = exchange_fds(bs, own_fd);
  ::close(own_fd);
  rc = CUDA_SUCCESS;
  for (int r = 0; r < world; ++r) {
    if (r == rank_) continue;
    if (rc == CUDA_SUCCESS) {
      CUmemGenericAllocationHandle h = 0;
      rc = d.MemImportFromShareableHandle(&h, reinterpret_cast<void*>(static_cast<uintptr_t>(fds[r])),
                                          CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
      if (rc == CUDA_SUCCESS) {
        peer_handle_[r] = h;
        CUdeviceptr va = 0;
        rc = map_for(d, h, size_, gran, device_, &va);
        peer_va_[r] = va;
      }
    }
    if (fds[r] >= 0) ::close(fds[r]);
  }
  agree(bs, rc, "mapping the peers' memory");
  if (!multicast) {
    if (want_multicast && world > 1)
      multicast_note_ = support.multicast ? "not every rank has a GPU of its own with multicast"
                                          : support.reason;
    return;
  }

  // One multicast object over all of it: rank 0 creates, everybody adds its GPU, and only
  // when all GPUs are in may memory be bound.
  CUmemGenericAllocationHandle mc = 0;
  int mc_fd = -1;
  rc = CUDA_SUCCESS;
  if (rank_ == 0) {
    rc = d.MulticastCreate(&mc, &mc_prop);
    if (rc == CUDA_SUCCESS)
      rc = d.MemExportToShareableHandle(&mc_fd, mc, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  }
  if (!all_ok(bs, rc, "creating the multicast object", &multicast_note_)) {
    if (mc != 0) d.MemRelease(mc);
    if (mc_fd >= 0) ::close(mc_fd);
    return;
  }
  fds = exchange_fds(bs, mc_fd);
  if (mc_fd >= 0) ::close(mc_fd);
  if (rank_ != 0) {
    rc = d.MemImportFromShareableHandle(&mc, reinterpret_cast<void*>(static_cast<uintptr_t>(fds[0])),
                                        CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  }
  for (int fd : fds)
    if (fd >= 0) ::close(fd);
  if (rc == CUDA_SUCCESS) {
    mc_handle_ = mc;
    rc = d.MulticastAddDevice(mc, device_);
  }
  else if (mc != 0 && rank_ == 0) {
    d.MemRelease(mc);
  }
  if (!all_ok(bs, rc, "adding the devices to the multicast object", &multicast_note_)) {
    drop_multicast();
    return;
  }
  rc = d.MulticastBindMem(mc, 0, own, 0, size_, 0);
  mc_bound_ = rc == CUDA_SUCCESS;
  if (!all_ok(bs, rc, "binding memory to the multicast object", &multicast_note_)) {
    drop_multicast();
    return;
  }
  CUdeviceptr mc_va = 0;
  rc = map_for(d, mc, size_, gran, device_, &mc_va);
  mc_va_ = mc_va;
  if (!all_ok(bs, rc, "mapping the multicast object", &multicast_note_)) drop_multicast();
}

}  // namespace pplx
