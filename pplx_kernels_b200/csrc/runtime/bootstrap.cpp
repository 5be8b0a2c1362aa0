#include "bootstrap.h"

#include <cerrno>
#include <chrono>
#include <cstring>
#include <mutex>
#include <random>
#include <thread>
#include <unordered_map>

#include <poll.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include "../core/utils.h"

namespace pplx {

long env_long(const char* name, long fallback) {
  const char* v = std::getenv(name);
  if (v == nullptr || *v == '\0') return fallback;
  char* end = nullptr;
  const long r = std::strtol(v, &end, 10);
  return (end != nullptr && *end == '\0') ? r : fallback;
}

void Bootstrap::all_to_all(const void* in, void* out, size_t bytes_each) {
  const int w = world();
  std::vector<uint8_t> all(static_cast<size_t>(w) * w * bytes_each);
  all_gather(in, all.data(), static_cast<size_t>(w) * bytes_each);
  for (int src = 0; src < w; ++src) {
    std::memcpy(static_cast<uint8_t*>(out) + src * bytes_each,
                all.data() + (static_cast<size_t>(src) * w + rank()) * bytes_each, bytes_each);
  }
}

void Bootstrap::barrier() {
  uint8_t token = 0;
  std::vector<uint8_t> all(world());
  all_gather(&token, all.data(), 1);
}

void SingleBootstrap::all_gather(const void* in, void* out, size_t bytes) {
  std::memcpy(out, in, bytes);
}

namespace {

constexpr char kMagic[8] = {'P', 'P', 'L', 'X', 'B', '2', '0', '0'};

struct UidLayout {
  char magic[8];
  uint64_t nonce;
  uint32_t pid;
  char name[64];  // abstract socket name (without the leading NUL)
};
static_assert(sizeof(UidLayout) <= kUniqueIdBytes, "unique id too large");

std::mutex g_mu;
std::unordered_map<uint64_t, int> g_listeners;  // nonce -> listening fd

sockaddr_un make_addr(const char* name, socklen_t* len) {
  sockaddr_un addr{};
  addr.sun_family = AF_UNIX;
  const size_t n = std::strlen(name);
  PPLX_CHECK(n + 1 < sizeof(addr.sun_path), "socket name too long");
  addr.sun_path[0] = '\0';
  std::memcpy(addr.sun_path + 1, name, n);
  *len = static_cast<socklen_t>(offsetof(sockaddr_un, sun_path) + 1 + n);
  return addr;
}

void write_all(int fd, const void* buf, size_t n) {
  const uint8_t* p = static_cast<const uint8_t*>(buf);
  while (n > 0) {
    const ssize_t r = ::send(fd, p, n, MSG_NOSIGNAL);
    if (r < 0) {
      if (errno == EINTR) continue;
      PPLX_CHECK(false, "bootstrap send failed: " << std::strerror(errno));
    }
    p += r;
    n -= static_cast<size_t>(r);
  }
}

void read_all(int fd, void* buf, size_t n, int timeout_ms) {
  uint8_t* p = static_cast<uint8_t*>(buf);
  while (n > 0) {
    pollfd pfd{fd, POLLIN, 0};
    const int pr = ::poll(&pfd, 1, timeout_ms);
    if (pr < 0 && errno == EINTR) continue;
    PPLX_CHECK(pr > 0, "bootstrap receive timed out after " << timeout_ms
                                                             << " ms (a peer did not answer)");
    const ssize_t r = ::recv(fd, p, n, 0);
    if (r < 0 && errno == EINTR) continue;
    PPLX_CHECK(r > 0, "bootstrap peer closed the connection");
    p += r;
    n -= static_cast<size_t>(r);
  }
}

}  // namespace

UniqueId create_unique_id() {
  std::random_device rd;
  const uint64_t nonce = (static_cast<uint64_t>(rd()) << 32) ^ rd() ^
                         static_cast<uint64_t>(
                             std::chrono::steady_clock::now().time_since_epoch().count());
  UidLayout u{};
  std::memcpy(u.magic, kMagic, sizeof(kMagic));
  u.nonce = nonce;
  u.pid = static_cast<uint32_t>(::getpid());
  std::snprintf(u.name, sizeof(u.name), "pplx-b200-%u-%016llx", u.pid,
                static_cast<unsigned long long>(nonce));

  const int fd = ::socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
  PPLX_CHECK(fd >= 0, "socket(): " << std::strerror(errno));
  socklen_t len = 0;
  sockaddr_un addr = make_addr(u.name, &len);
  PPLX_CHECK(::bind(fd, reinterpret_cast<sockaddr*>(&addr), len) == 0,
             "bind(): " << std::strerror(errno));
  PPLX_CHECK(::listen(fd, 128) == 0, "listen(): " << std::strerror(errno));
  {
    std::lock_guard<std::mutex> lock(g_mu);
    g_listeners[nonce] = fd;
  }
  UniqueId id{};
  std::memcpy(id.bytes, &u, sizeof(u));
  return id;
}

SocketBootstrap::SocketBootstrap(const UniqueId& uid, int rank, int world, int timeout_ms)
    : rank_(rank), world_(world), timeout_ms_(timeout_ms) {
  PPLX_CHECK(world >= 1 && rank >= 0 && rank < world, "bad rank/world " << rank << "/" << world);
  UidLayout u{};
  std::memcpy(&u, uid.bytes, sizeof(u));
  if (world == 1) {
    // Nothing to exchange; release the listener if this process made one.
    std::lock_guard<std::mutex> lock(g_mu);
    auto it = g_listeners.find(u.nonce);
    if (it != g_listeners.end()) {
      ::close(it->second);
      g_listeners.erase(it);
    }
    return;
  }
  PPLX_CHECK(std::memcmp(u.magic, kMagic, sizeof(kMagic)) == 0,
             "unique id was not produced by get_unique_id()");
  u.name[sizeof(u.name) - 1] = '\0';

  if (rank == 0) {
    {
      std::lock_guard<std::mutex> lock(g_mu);
      auto it = g_listeners.find(u.nonce);
      PPLX_CHECK(it != g_listeners.end(),
                 "rank 0 must be the process that called get_unique_id()");
      listen_fd_ = it->second;
      g_listeners.erase(it);
    }
    peer_fds_.assign(world, -1);
    for (int n = 1; n < world; ++n) {
      pollfd pfd{listen_fd_, POLLIN, 0};
      const int pr = ::poll(&pfd, 1, timeout_ms_);
      PPLX_CHECK(pr > 0, "bootstrap: only " << n - 1 << " of " << world - 1
                                             << " peers connected before the timeout");
      const int fd = ::accept4(listen_fd_, nullptr, nullptr, SOCK_CLOEXEC);
      PPLX_CHECK(fd >= 0, "accept(): " << std::strerror(errno));
      int32_t peer_rank = -1;
      read_all(fd, &peer_rank, sizeof(peer_rank), timeout_ms_);
      PPLX_CHECK(peer_rank > 0 && peer_rank < world && peer_fds_[peer_rank] < 0,
                 "bootstrap: unexpected hello from rank " << peer_rank);
      peer_fds_[peer_rank] = fd;
    }
  } else {
    const int fd = ::socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
    PPLX_CHECK(fd >= 0, "socket(): " << std::strerror(errno));
    socklen_t len = 0;
    sockaddr_un addr = make_addr(u.name, &len);
    const auto deadline =
        std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms_);
    while (::connect(fd, reinterpret_cast<sockaddr*>(&addr), len) != 0) {
      PPLX_CHECK(std::chrono::steady_clock::now() < deadline,
                 "bootstrap: could not reach rank 0: " << std::strerror(errno));
      std::this_thread::sleep_for(std::chrono::milliseconds(5));
    }
    const int32_t me = rank;
    write_all(fd, &me, sizeof(me));
    peer_fds_.assign(1, fd);
  }
}

SocketBootstrap::~SocketBootstrap() {
  for (int fd : peer_fds_)
    if (fd >= 0) ::close(fd);
  if (listen_fd_ >= 0) ::close(listen_fd_);
}

void SocketBootstrap::all_gather(const void* in, void* out, size_t bytes) {
  if (world_ == 1) {
    std::memcpy(out, in, bytes);
    return;
  }
  uint8_t* o = static_cast<uint8_t*>(out);
  if (rank_ == 0) {
    std::memcpy(o, in, bytes);
    for (int r = 1; r < world_; ++r) read_all(peer_fds_[r], o + r * bytes, bytes, timeout_ms_);
    for (int r = 1; r < world_; ++r) write_all(peer_fds_[r], o, bytes * world_);
  } else {
    write_all(peer_fds_[0], in, bytes);
    read_all(peer_fds_[0], o, bytes * world_, timeout_ms_);
  }
}

}  // namespace pplx
