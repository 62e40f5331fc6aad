// The symmetric heap (symmetric_heap.h) behind the Python module: heaps are kept in a process-wide table and
// named by small integers; an allocation comes back as a byte tensor over this rank's piece together with every
// rank's address of it and the multicast address.
#include <ATen/ATen.h>

#include <map>
#include <memory>
#include <mutex>

#include "kernels/ops.h"
#include "symmetric_heap.h"

namespace nt {
namespace {

struct OpenHeap {
  std::unique_ptr<symm::SymmetricHeap> heap;
  std::map<int64_t, symm::Allocation> live;
  int device;
};

std::mutex& table_mutex() {
  static std::mutex mu;
  return mu;
}
std::map<int64_t, OpenHeap>& table() {
  static std::map<int64_t, OpenHeap> heaps;
  return heaps;
}

OpenHeap& find(int64_t id) {
  auto it = table().find(id);
  TORCH_CHECK(it != table().end(), "symmetric heap ", id, " is not open");
  return it->second;
}

}  // namespace

int64_t symm_heap_open(const std::string& job, int64_t rank, int64_t world, int64_t device, int64_t timeout_ms) {
  std::lock_guard<std::mutex> lock(table_mutex());
  static int64_t next = 1;
  OpenHeap h;
  h.heap = std::make_unique<symm::SymmetricHeap>(symm::cuda_driver(), job, static_cast<int>(rank), static_cast<int>(world),
                                                 static_cast<int>(device), static_cast<int>(timeout_ms));
  h.device = static_cast<int>(device);
  table().emplace(next, std::move(h));
  return next++;
}

std::tuple<at::Tensor, std::vector<int64_t>, int64_t, int64_t> symm_heap_alloc(int64_t heap, int64_t bytes, bool multicast) {
  std::lock_guard<std::mutex> lock(table_mutex());
  OpenHeap& h = find(heap);
  TORCH_CHECK(bytes > 0, "symmetric heap: empty allocation");
  symm::Allocation a = h.heap->allocate(static_cast<size_t>(bytes), multicast);
  std::vector<int64_t> peers;
  for (int r = 0; r < h.heap->world(); ++r) peers.push_back(static_cast<int64_t>(a.piece(r)));
  at::Tensor mine = at::from_blob(reinterpret_cast<void*>(a.piece(h.heap->rank())), {bytes}, [](void*) {},
                                  at::TensorOptions().dtype(at::kByte).device(at::kCUDA, h.device));
  int64_t id = static_cast<int64_t>(a.id);
  int64_t mc = static_cast<int64_t>(a.multicast);
  h.live.emplace(id, a);
  return {mine, peers, mc, id};
}

void symm_heap_free(int64_t heap, int64_t allocation) {
  std::lock_guard<std::mutex> lock(table_mutex());
  OpenHeap& h = find(heap);
  auto it = h.live.find(allocation);
  TORCH_CHECK(it != h.live.end(), "symmetric heap: allocation ", allocation, " is not live");
  h.heap->release(it->second);
  h.live.erase(it);
}

void symm_heap_close(int64_t heap) {
  std::lock_guard<std::mutex> lock(table_mutex());
  OpenHeap& h = find(heap);
  TORCH_CHECK(h.live.empty(), "symmetric heap: ", h.live.size(), " allocation(s) still live");
  table().erase(heap);
}

}  // namespace nt
