// Symmetric heap: the same-sized allocation on every rank of a group, each rank's piece mapped into
// every other rank's address space (peer loads and stores over NVLink), plus one multicast mapping of
// all pieces for `multimem.*` instructions (reduction and broadcast inside the NVSwitch).
//
// Three parts, all host code:
//   * `DriverApi`   - the handful of virtual-memory and multicast driver calls the heap needs, as a table of
//                     functions.  `cuda_driver()` (symmetric_heap_cuda.cpp) fills it from the CUDA driver;
//                     tests fill it with a host implementation over memfd + mmap, which gives real shared
//                     memory between processes, so the exchange protocol is exercised without a GPU.
//   * `FdChannel`   - moves file descriptors (the shareable handles) between the ranks of one machine over
//                     unix datagram sockets in the abstract namespace (SCM_RIGHTS).  Every receive has a
//                     time limit; a peer that never shows up makes the call fail, not hang.
//   * `SymmetricHeap` - the collective `allocate` / `release` built from the two.
//
// Layout of one allocation on every rank: a single reserved range of `world * size` bytes, rank r's
// piece at `base + r * size` (so a peer pointer is plain arithmetic), and a second range of `size`
// bytes mapping the multicast object when the group has one.
//
// The reference reaches peers through NCCL only (csrc/nccl/nccl.cpp:33-76: ncclCommInitRank and
// ncclAllReduce); this heap is what the fused collective kernels of this library stand on instead.
#pragma once

#include <poll.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <cerrno>
#include <chrono>
#include <cstdint>
#include <cstring>
#include <deque>
#include <functional>
#include <stdexcept>
#include <string>
#include <thread>
#include <utility>
#include <vector>

namespace nt::symm {

using Handle = uint64_t;   // a driver allocation or multicast handle
using Address = uint64_t;  // a virtual address

struct DriverApi {
  // Allocation granularity of `device`'s memory (multicast_devices == 0) or of a multicast object over that
  // many devices.
  std::function<size_t(int device, int multicast_devices)> granularity;
  std::function<bool(int device)> multicast_supported;
  std::function<Handle(int device, size_t bytes)> create;           // physical memory, shareable as an fd
  std::function<int(Handle)> export_fd;                             // caller closes the fd
  std::function<Handle(int fd)> import_fd;                          // does not close the fd
  std::function<void(Handle)> release;                              // drop one reference to a handle
  std::function<Address(size_t bytes, size_t alignment)> reserve;   // address range, nothing mapped
  std::function<void(Address, size_t bytes)> unreserve;
  std::function<void(Address, size_t bytes, Handle, int device)> map;  // map + read/write access for device
  std::function<void(Address, size_t bytes)> unmap;
  std::function<Handle(int n_devices, size_t bytes)> multicast_create;
  std::function<void(Handle mc, int device)> multicast_add_device;
  std::function<void(Handle mc, Handle memory, size_t bytes)> multicast_bind;  // whole piece at offset 0
  std::function<void(Handle mc, int device, size_t bytes)> multicast_unbind;
};

// The CUDA driver behind the table (symmetric_heap_cuda.cpp).
const DriverApi& cuda_driver();

inline size_t round_up(size_t v, size_t to) { return (v + to - 1) / to * to; }

class Timeout : public std::runtime_error {
 public:
  using std::runtime_error::runtime_error;
};

// ---------------------------------------------------------------------------------------------------
struct Message {
  uint32_t magic = 0x4e545348;  // "NTSH"
  int32_t src = -1;
  uint32_t kind = 0;
  uint32_t flags = 0;
  uint64_t seq = 0;
};

struct Received {
  Message msg;
  int fd = -1;  // -1 when the message carried none
};

class FdChannel {
 public:
  FdChannel(const std::string& job, int rank, int world, int timeout_ms)
      : job_(job), rank_(rank), world_(world), timeout_ms_(timeout_ms) {
    sock_ = ::socket(AF_UNIX, SOCK_DGRAM | SOCK_CLOEXEC, 0);
    if (sock_ < 0) throw std::runtime_error(std::string("symmetric heap: socket(): ") + std::strerror(errno));
    int on = 1;  // the kernel then attaches the sender's pid / uid / gid to every message we receive
    if (::setsockopt(sock_, SOL_SOCKET, SO_PASSCRED, &on, sizeof(on)) != 0) {
      int err = errno;
      ::close(sock_);
      throw std::runtime_error(std::string("symmetric heap: SO_PASSCRED: ") + std::strerror(err));
    }
    sockaddr_un addr;
    socklen_t len = address_of(rank, &addr);
    if (::bind(sock_, reinterpret_cast<sockaddr*>(&addr), len) != 0) {
      int err = errno;
      ::close(sock_);
      throw std::runtime_error("symmetric heap: cannot bind the socket of rank " + std::to_string(rank) + " of job '" +
                               job + "': " + std::strerror(err));
    }
  }
  FdChannel(const FdChannel&) = delete;
  FdChannel& operator=(const FdChannel&) = delete;
  ~FdChannel() {
    for (auto& r : pending_)
      if (r.fd >= 0) ::close(r.fd);
    if (sock_ >= 0) ::close(sock_);
  }

  int rank() const { return rank_; }
  int world() const { return world_; }
  int timeout_ms() const { return timeout_ms_; }

  // Send a message, with `fd` attached when it is >= 0.  A peer whose socket does not exist yet is
  // retried until the time limit.
  void send(int dst, uint32_t kind, uint64_t seq, uint32_t flags, int fd) {
    Message m;
    m.src = rank_;
    m.kind = kind;
    m.seq = seq;
    m.flags = flags;
    sockaddr_un addr;
    socklen_t len = address_of(dst, &addr);
    iovec iov{&m, sizeof(m)};
    alignas(cmsghdr) char control[CMSG_SPACE(sizeof(int))];
    msghdr hdr{};
    hdr.msg_name = &addr;
    hdr.msg_namelen = len;
    hdr.msg_iov = &iov;
    hdr.msg_iovlen = 1;
    if (fd >= 0) {
      std::memset(control, 0, sizeof(control));
      hdr.msg_control = control;
      hdr.msg_controllen = sizeof(control);
      cmsghdr* c = CMSG_FIRSTHDR(&hdr);
      c->cmsg_level = SOL_SOCKET;
      c->cmsg_type = SCM_RIGHTS;
      c->cmsg_len = CMSG_LEN(sizeof(int));
      std::memcpy(CMSG_DATA(c), &fd, sizeof(int));
    }
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms_);
    for (;;) {
      ssize_t n = ::sendmsg(sock_, &hdr, MSG_DONTWAIT);
      if (n == static_cast<ssize_t>(sizeof(m))) return;
      int err = errno;
      bool retry = n < 0 && (err == ECONNREFUSED || err == ENOENT || err == EAGAIN || err == EWOULDBLOCK || err == EINTR ||
                             err == ENOBUFS);
      if (!retry)
        throw std::runtime_error("symmetric heap: send to rank " + std::to_string(dst) + ": " + std::strerror(err));
      if (std::chrono::steady_clock::now() > deadline)
        throw Timeout("symmetric heap: rank " + std::to_string(dst) + " did not take a message from rank " +
                      std::to_string(rank_) + " within " + std::to_string(timeout_ms_) + " ms (" + std::strerror(err) + ")");
      std::this_thread::sleep_for(std::chrono::milliseconds(2));
    }
  }

  // The message of (kind, seq) from `src`; others that arrive meanwhile are kept for their own callers.
  Received receive(int src, uint32_t kind, uint64_t seq) {
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms_);
    for (;;) {
      for (auto it = pending_.begin(); it != pending_.end(); ++it)
        if (it->msg.src == src && it->msg.kind == kind && it->msg.seq == seq) {
          Received r = *it;
          pending_.erase(it);
          return r;
        }
      auto left = std::chrono::duration_cast<std::chrono::milliseconds>(deadline - std::chrono::steady_clock::now()).count();
      if (left <= 0)
        throw Timeout("symmetric heap: rank " + std::to_string(rank_) + " waited " + std::to_string(timeout_ms_) +
                      " ms for message kind " + std::to_string(kind) + " #" + std::to_string(seq) + " of rank " +
                      std::to_string(src));
      pollfd p{sock_, POLLIN, 0};
      int ready = ::poll(&p, 1, static_cast<int>(left));
      if (ready < 0 && errno != EINTR) throw std::runtime_error(std::string("symmetric heap: poll(): ") + std::strerror(errno));
      if (ready > 0) take_one();
    }
  }

 private:
  socklen_t address_of(int rank, sockaddr_un* addr) const {
    std::memset(addr, 0, sizeof(*addr));
    addr->sun_family = AF_UNIX;
    std::string name = "nt-symm/" + job_ + "/" + std::to_string(rank);
    if (name.size() + 1 > sizeof(addr->sun_path)) throw std::runtime_error("symmetric heap: job name too long");
    std::memcpy(addr->sun_path + 1, name.data(), name.size());  // leading NUL: abstract namespace, no file to clean up
    return static_cast<socklen_t>(offsetof(sockaddr_un, sun_path) + 1 + name.size());
  }

  void take_one() {
    Received r;
    iovec iov{&r.msg, sizeof(r.msg)};
    alignas(cmsghdr) char control[CMSG_SPACE(sizeof(int)) + CMSG_SPACE(sizeof(ucred))];
    msghdr hdr{};
    hdr.msg_iov = &iov;
    hdr.msg_iovlen = 1;
    hdr.msg_control = control;
    hdr.msg_controllen = sizeof(control);
    ssize_t n = ::recvmsg(sock_, &hdr, MSG_DONTWAIT | MSG_CMSG_CLOEXEC);
    if (n < 0) {
      if (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR) return;
      throw std::runtime_error(std::string("symmetric heap: recvmsg(): ") + std::strerror(errno));
    }
    bool same_user = false;  // the abstract socket name space is open to every local process: take our own user's only
    for (cmsghdr* c = CMSG_FIRSTHDR(&hdr); c != nullptr; c = CMSG_NXTHDR(&hdr, c)) {
      if (c->cmsg_level != SOL_SOCKET) continue;
      if (c->cmsg_type == SCM_RIGHTS) std::memcpy(&r.fd, CMSG_DATA(c), sizeof(int));
      if (c->cmsg_type == SCM_CREDENTIALS) {
        ucred who;
        std::memcpy(&who, CMSG_DATA(c), sizeof(who));
        same_user = who.uid == ::geteuid();
      }
    }
    bool ok = same_user && n == static_cast<ssize_t>(sizeof(Message)) && r.msg.magic == Message().magic && r.msg.src >= 0 &&
              r.msg.src < world_ && r.msg.src != rank_;
    if (!ok) {  // not one of ours: drop it, and the descriptor with it
      if (r.fd >= 0) ::close(r.fd);
      return;
    }
    pending_.push_back(r);
  }

  std::string job_;
  int rank_, world_, timeout_ms_;
  int sock_ = -1;
  std::deque<Received> pending_;
};

// ---------------------------------------------------------------------------------------------------
struct Allocation {
  uint64_t id = 0;
  size_t size = 0;          // bytes of one rank's piece (the request rounded up to the granularity)
  Address base = 0;         // rank r's piece is at base + r * size
  Address multicast = 0;    // 0: the group has no multicast mapping
  Handle local = 0, mc = 0;
  Address piece(int rank) const { return base + static_cast<Address>(rank) * size; }
};

class SymmetricHeap {
 public:
  enum Kind : uint32_t { kMemory = 1, kMulticast = 2, kBarrier = 3 };

  SymmetricHeap(const DriverApi& api, const std::string& job, int rank, int world, int device, int timeout_ms)
      : api_(api), channel_(job, rank, world, timeout_ms), rank_(rank), world_(world), device_(device) {
    if (world < 1 || rank < 0 || rank >= world) throw std::invalid_argument("symmetric heap: bad rank / world");
  }

  int rank() const { return rank_; }
  int world() const { return world_; }

  // Collective: every rank calls with the same arguments, in the same order as its other calls.
  Allocation allocate(size_t bytes, bool want_multicast) {
    if (bytes == 0) throw std::invalid_argument("symmetric heap: empty allocation");
    Allocation a;
    a.id = ++seq_;
    bool mc_here = want_multicast && world_ > 1 && api_.multicast_supported(device_);
    size_t gran = api_.granularity(device_, 0);
    if (mc_here) gran = std::max(gran, api_.granularity(device_, world_));
    a.size = round_up(bytes, gran);
    int mapped = 0;
    Cleanup undo;  // runs in reverse unless dismissed

    a.local = api_.create(device_, a.size);
    undo.add([&] { api_.release(a.local); });
    {
      int fd = api_.export_fd(a.local);
      FdGuard guard(fd);
      for (int p = 0; p < world_; ++p)
        if (p != rank_) channel_.send(p, kMemory, a.id, mc_here ? 1u : 0u, fd);
    }
    a.base = api_.reserve(a.size * world_, gran);
    undo.add([&] { api_.unreserve(a.base, a.size * world_); });
    bool mc_everywhere = mc_here;
    undo.add([&] {
      for (int r = 0; r < mapped; ++r) api_.unmap(a.piece(r), a.size);
    });
    for (int r = 0; r < world_; ++r) {
      if (r == rank_) {
        api_.map(a.piece(r), a.size, a.local, device_);
      } else {
        Received got = channel_.receive(r, kMemory, a.id);
        FdGuard guard(got.fd);
        if (got.fd < 0) throw std::runtime_error("symmetric heap: rank " + std::to_string(r) + " sent no handle");
        mc_everywhere = mc_everywhere && (got.msg.flags & 1u);
        Handle h = api_.import_fd(got.fd);
        try {
          api_.map(a.piece(r), a.size, h, device_);
        } catch (...) {
          api_.release(h);
          throw;
        }
        api_.release(h);  // the mapping keeps the memory alive
      }
      mapped = r + 1;
    }
    // Every rank has seen every flag, so all take the same branch below.
    if (want_multicast && world_ > 1 && !mc_everywhere) mc_here = false;
    if (mc_here) {
      if (rank_ == 0) {
        a.mc = api_.multicast_create(world_, a.size);
        undo.add([&] { api_.release(a.mc); });
        int fd = api_.export_fd(a.mc);
        FdGuard guard(fd);
        for (int p = 1; p < world_; ++p) channel_.send(p, kMulticast, a.id, 0, fd);
      } else {
        Received got = channel_.receive(0, kMulticast, a.id);
        FdGuard guard(got.fd);
        if (got.fd < 0) throw std::runtime_error("symmetric heap: rank 0 sent no multicast handle");
        a.mc = api_.import_fd(got.fd);
        undo.add([&] { api_.release(a.mc); });
      }
      api_.multicast_add_device(a.mc, device_);
      barrier();  // the driver wants every device added before the first bind
      api_.multicast_bind(a.mc, a.local, a.size);
      undo.add([&] { api_.multicast_unbind(a.mc, device_, a.size); });
      barrier();
      a.multicast = api_.reserve(a.size, gran);
      undo.add([&] { api_.unreserve(a.multicast, a.size); });
      api_.map(a.multicast, a.size, a.mc, device_);
      undo.add([&] { api_.unmap(a.multicast, a.size); });
    }
    barrier();  // nobody uses a peer's piece before that peer has mapped its own
    undo.dismiss();
    return a;
  }

  // Collective.  The caller has made sure no kernel still uses the memory on any rank.
  void release(Allocation& a) {
    barrier();
    if (a.multicast) {
      api_.unmap(a.multicast, a.size);
      api_.unreserve(a.multicast, a.size);
      api_.multicast_unbind(a.mc, device_, a.size);
      api_.release(a.mc);
    }
    for (int r = 0; r < world_; ++r) api_.unmap(a.piece(r), a.size);
    api_.unreserve(a.base, a.size * world_);
    api_.release(a.local);
    a = Allocation();
  }

  // All ranks of the group; bounded by the channel's time limit.
  void barrier() {
    uint64_t n = ++barrier_seq_;
    for (int p = 0; p < world_; ++p)
      if (p != rank_) channel_.send(p, kBarrier, n, 0, -1);
    for (int p = 0; p < world_; ++p)
      if (p != rank_) channel_.receive(p, kBarrier, n);
  }

 private:
  struct FdGuard {
    explicit FdGuard(int fd) : fd(fd) {}
    ~FdGuard() {
      if (fd >= 0) ::close(fd);
    }
    int fd;
  };
  class Cleanup {
   public:
    void add(std::function<void()> f) { steps_.push_back(std::move(f)); }
    void dismiss() { steps_.clear(); }
    ~Cleanup() {
      for (auto it = steps_.rbegin(); it != steps_.rend(); ++it) {
        try {
          (*it)();
        } catch (...) {  // already unwinding; nothing better to do with a second failure
        }
      }
    }

   private:
    std::vector<std::function<void()>> steps_;
  };

  const DriverApi& api_;
  FdChannel channel_;
  int rank_, world_, device_;
  uint64_t seq_ = 0, barrier_seq_ = 0;
};

}  // namespace nt::symm
