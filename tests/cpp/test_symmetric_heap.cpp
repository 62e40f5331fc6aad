// Host test of the symmetric heap (csrc/runtime/symmetric_heap.h): the ranks are forked processes and the
// driver table is a host implementation over memfd + mmap, so "peer memory" is real shared memory and the
// whole exchange (descriptor passing, mapping, multicast set-up order, barriers, time limits, clean-up after
// a failure) runs without a GPU.      g++ -std=c++17 -I nanotitan_b200/csrc/runtime tests/cpp/test_symmetric_heap.cpp
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <sys/wait.h>

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <map>

#include "symmetric_heap.h"

using namespace nt::symm;

namespace {

constexpr size_t kMemGranule = 64 << 10, kMcGranule = 128 << 10, kHeader = 4096;

struct McHeader {  // lives behind the payload of a multicast object's memfd, shared by all ranks
  std::atomic<int> devices_wanted, devices_added, bound;
};

struct FakeDriver {
  struct Entry {
    int fd;
    size_t bytes;
    bool multicast;
  };
  std::map<Handle, Entry> handles;
  std::map<Address, std::pair<void*, size_t>> ranges;  // aligned start -> raw mmap
  Handle next = 1;
  bool multicast_ok = true;
  int multicast_calls = 0, live_maps = 0;

  static McHeader* header(const Entry& e) {
    void* p = mmap(nullptr, kHeader, PROT_READ | PROT_WRITE, MAP_SHARED, e.fd, static_cast<off_t>(e.bytes));
    if (p == MAP_FAILED) throw std::runtime_error("fake driver: cannot map the multicast header");
    return static_cast<McHeader*>(p);  // leaked on purpose: one page per call in a short test
  }

  Handle adopt(int fd) {
    struct stat st;
    if (fstat(fd, &st) != 0) throw std::runtime_error("fake driver: fstat");
    bool mc = (static_cast<size_t>(st.st_size) % kMemGranule) == kHeader;
    size_t bytes = static_cast<size_t>(st.st_size) - (mc ? kHeader : 0);
    handles[next] = Entry{fd, bytes, mc};
    return next++;
  }

  DriverApi api() {
    DriverApi a;
    a.granularity = [](int, int mc_devices) { return mc_devices > 0 ? kMcGranule : kMemGranule; };
    a.multicast_supported = [this](int) { return multicast_ok; };
    a.create = [this](int, size_t bytes) {
      if (bytes % kMemGranule) throw std::runtime_error("fake driver: size is not a multiple of the granularity");
      int fd = memfd_create("nt-symm-test", MFD_CLOEXEC);
      if (fd < 0 || ftruncate(fd, static_cast<off_t>(bytes)) != 0) throw std::runtime_error("fake driver: memfd");
      return adopt(fd);
    };
    a.export_fd = [this](Handle h) { return dup(handles.at(h).fd); };
    a.import_fd = [this](int fd) { return adopt(dup(fd)); };
    a.release = [this](Handle h) {
      close(handles.at(h).fd);
      handles.erase(h);
    };
    a.reserve = [this](size_t bytes, size_t align) {
      size_t raw_len = bytes + align;
      void* raw = mmap(nullptr, raw_len, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE, -1, 0);
      if (raw == MAP_FAILED) throw std::runtime_error("fake driver: reserve");
      Address start = round_up(reinterpret_cast<Address>(raw), align);
      ranges[start] = {raw, raw_len};
      return start;
    };
    a.unreserve = [this](Address start, size_t) {
      auto r = ranges.at(start);
      munmap(r.first, r.second);
      ranges.erase(start);
    };
    a.map = [this](Address at, size_t bytes, Handle h, int) {
      const Entry& e = handles.at(h);
      if (bytes > e.bytes) throw std::runtime_error("fake driver: mapping larger than the allocation");
      if (e.multicast && header(e)->bound.load() != header(e)->devices_wanted.load())
        throw std::runtime_error("fake driver: multicast object mapped before every device bound its memory");
      void* p = mmap(reinterpret_cast<void*>(at), bytes, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_FIXED, e.fd, 0);
      if (p == MAP_FAILED) throw std::runtime_error("fake driver: map");
      ++live_maps;
    };
    a.unmap = [this](Address at, size_t bytes) {
      mmap(reinterpret_cast<void*>(at), bytes, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_FIXED | MAP_NORESERVE, -1, 0);
      --live_maps;
    };
    a.multicast_create = [this](int n, size_t bytes) {
      ++multicast_calls;
      if (bytes % kMcGranule) throw std::runtime_error("fake driver: multicast size is not a multiple of its granularity");
      int fd = memfd_create("nt-symm-test-mc", MFD_CLOEXEC);
      if (fd < 0 || ftruncate(fd, static_cast<off_t>(bytes + kHeader)) != 0) throw std::runtime_error("fake driver: memfd");
      Handle h = adopt(fd);
      header(handles.at(h))->devices_wanted.store(n);
      return h;
    };
    a.multicast_add_device = [this](Handle mc, int) {
      ++multicast_calls;
      header(handles.at(mc))->devices_added.fetch_add(1);
    };
    a.multicast_bind = [this](Handle mc, Handle mem, size_t bytes) {
      ++multicast_calls;
      McHeader* h = header(handles.at(mc));
      if (h->devices_added.load() != h->devices_wanted.load())
        throw std::runtime_error("fake driver: memory bound before every device was added");
      if (handles.at(mem).bytes != bytes) throw std::runtime_error("fake driver: bind size differs from the allocation");
      h->bound.fetch_add(1);
    };
    a.multicast_unbind = [this](Handle mc, int, size_t) {
      ++multicast_calls;
      header(handles.at(mc))->bound.fetch_sub(1);
    };
    return a;
  }
};

#define EXPECT(cond)                                                          \
  do {                                                                        \
    if (!(cond)) {                                                            \
      std::fprintf(stderr, "rank %d: %s:%d: %s\n", rank, __FILE__, __LINE__, #cond); \
      return 1;                                                               \
    }                                                                         \
  } while (0)

uint32_t* words(Address a) { return reinterpret_cast<uint32_t*>(a); }

int exchange_case(const std::string& job, int rank, int world) {
  FakeDriver drv;
  DriverApi api = drv.api();
  SymmetricHeap heap(api, job, rank, world, /*device=*/rank, /*timeout_ms=*/10000);
  Allocation a = heap.allocate(100000, true);
  EXPECT(a.size == kMcGranule);  // 100000 bytes rounded up to the larger of the two granularities
  EXPECT(a.base % kMcGranule == 0 && a.multicast != 0);
  const size_t n = a.size / 4;
  for (size_t i = 0; i < n; ++i) words(a.piece(rank))[i] = static_cast<uint32_t>(rank * 1000003u + i);
  heap.barrier();
  for (int r = 0; r < world; ++r)
    for (size_t i = 0; i < n; i += 97) EXPECT(words(a.piece(r))[i] == static_cast<uint32_t>(r * 1000003u + i));
  heap.barrier();
  words(a.piece((rank + 1) % world))[rank] = 0xabc00000u + rank;  // a store into the neighbour's piece
  heap.barrier();
  int left = (rank + world - 1) % world;
  EXPECT(words(a.piece(rank))[left] == 0xabc00000u + left);
  if (rank == 0) words(a.multicast)[5] = 77;  // every rank maps the same multicast object
  heap.barrier();
  EXPECT(words(a.multicast)[5] == 77);

  Allocation b = heap.allocate(kMemGranule, false);  // a second allocation, no multicast asked for
  EXPECT(b.multicast == 0 && b.size == kMemGranule && b.base != a.base && b.id == a.id + 1);
  words(b.piece((rank + 1) % world))[0] = 5 + rank;
  heap.barrier();
  EXPECT(words(b.piece(rank))[0] == static_cast<uint32_t>(5 + left));
  heap.release(b);
  heap.release(a);
  EXPECT(drv.handles.empty() && drv.ranges.empty() && drv.live_maps == 0);
  EXPECT(a.base == 0 && a.size == 0);
  return 0;
}

int no_multicast_on_one_rank_case(const std::string& job, int rank, int world) {
  FakeDriver drv;
  drv.multicast_ok = rank != 1;
  DriverApi api = drv.api();
  SymmetricHeap heap(api, job, rank, world, rank, 10000);
  Allocation a = heap.allocate(1 << 20, true);
  EXPECT(a.multicast == 0 && drv.multicast_calls == 0);  // all ranks agree to go without
  words(a.piece((rank + 1) % world))[3] = 900 + rank;
  heap.barrier();
  EXPECT(words(a.piece(rank))[3] == static_cast<uint32_t>(900 + (rank + world - 1) % world));
  heap.release(a);
  EXPECT(drv.handles.empty() && drv.ranges.empty() && drv.live_maps == 0);
  return 0;
}

int absent_peer_case(const std::string& job, int rank, int /*world*/) {
  if (rank != 0) return 0;  // the peers never start
  FakeDriver drv;
  DriverApi api = drv.api();
  SymmetricHeap heap(api, job, 0, 2, 0, /*timeout_ms=*/300);
  auto t0 = std::chrono::steady_clock::now();
  bool timed_out = false;
  try {
    heap.allocate(4096, true);
  } catch (const Timeout&) {
    timed_out = true;
  }
  auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
  EXPECT(timed_out && ms >= 250 && ms < 5000);
  EXPECT(drv.handles.empty() && drv.ranges.empty() && drv.live_maps == 0);  // the failed call cleaned up after itself
  return 0;
}

int fake_driver_checks_order_case(const std::string&, int rank, int) {
  // The stand-in driver must refuse what the real one refuses, or the cases above prove nothing.
  FakeDriver drv;
  DriverApi api = drv.api();
  Handle mc = api.multicast_create(2, kMcGranule);
  Handle mem = api.create(0, kMcGranule);
  api.multicast_add_device(mc, 0);
  bool refused = false;
  try {
    api.multicast_bind(mc, mem, kMcGranule);  // the second device was never added
  } catch (const std::runtime_error&) {
    refused = true;
  }
  EXPECT(refused);
  api.multicast_add_device(mc, 1);
  api.multicast_bind(mc, mem, kMcGranule);
  Address at = api.reserve(kMcGranule, kMcGranule);
  refused = false;
  try {
    api.map(at, kMcGranule, mc, 0);  // only one of two devices has bound its memory
  } catch (const std::runtime_error&) {
    refused = true;
  }
  EXPECT(refused);
  return 0;
}

int single_rank_case(const std::string& job, int rank, int) {
  if (rank != 0) return 0;
  FakeDriver drv;
  DriverApi api = drv.api();
  SymmetricHeap heap(api, job, 0, 1, 0, 1000);
  Allocation a = heap.allocate(10, true);
  EXPECT(a.size == kMemGranule && a.multicast == 0 && a.piece(0) == a.base);
  words(a.base)[0] = 1;
  heap.release(a);
  EXPECT(drv.handles.empty() && drv.live_maps == 0);
  return 0;
}

bool run_ranks(const char* name, int world, int (*body)(const std::string&, int, int)) {
  std::string job = std::string(name) + "-" + std::to_string(getpid());
  std::vector<pid_t> kids;
  for (int r = 0; r < world; ++r) {
    pid_t pid = fork();
    if (pid == 0) {
      int rc = 1;
      try {
        rc = body(job, r, world);
      } catch (const std::exception& e) {
        std::fprintf(stderr, "rank %d: exception: %s\n", r, e.what());
      }
      _exit(rc);
    }
    kids.push_back(pid);
  }
  bool ok = true;
  for (pid_t pid : kids) {
    int status = 0;
    waitpid(pid, &status, 0);
    ok = ok && WIFEXITED(status) && WEXITSTATUS(status) == 0;
  }
  std::printf("%-32s %s\n", name, ok ? "ok" : "FAILED");
  return ok;
}

}  // namespace

int main() {
  bool ok = true;
  ok &= run_ranks("exchange-3-ranks", 3, exchange_case);
  ok &= run_ranks("exchange-8-ranks", 8, exchange_case);
  ok &= run_ranks("one-rank-without-multicast", 3, no_multicast_on_one_rank_case);
  ok &= run_ranks("absent-peer-times-out", 1, absent_peer_case);
  ok &= run_ranks("single-rank", 1, single_rank_case);
  ok &= run_ranks("stand-in-driver-refuses-misuse", 1, fake_driver_checks_order_case);
  std::printf(ok ? "ALL PASSED\n" : "SOME FAILED\n");
  return ok ? 0 : 1;
}
