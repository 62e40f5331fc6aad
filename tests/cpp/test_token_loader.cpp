// Host test of the token window loader (csrc/runtime/token_loader.h).
//     g++ -std=c++17 -I nanotitan_b200/csrc/runtime tests/cpp/test_token_loader.cpp -lpthread
#include <cstdio>
#include <cstdlib>
#include <numeric>

#include "token_loader.h"

#define EXPECT(cond)                                                 \
  do {                                                               \
    if (!(cond)) {                                                   \
      std::fprintf(stderr, "%s:%d: %s\n", __FILE__, __LINE__, #cond); \
      return 1;                                                      \
    }                                                                \
  } while (0)

int main() {
  char path[] = "/tmp/nt-token-loader-XXXXXX";
  int fd = mkstemp(path);
  EXPECT(fd >= 0);
  const int64_t S = 7, B = 3, n_tokens = 7 * 10 + 1 + 4;  // ten whole windows and a ragged tail
  std::vector<uint16_t> tokens(n_tokens);
  for (int64_t i = 0; i < n_tokens; ++i) tokens[i] = static_cast<uint16_t>((i * 7919) % 65521);
  EXPECT(write(fd, tokens.data(), tokens.size() * 2) == static_cast<ssize_t>(tokens.size() * 2));
  close(fd);
  {
    const int depth = 3;
    nt::TokenWindowLoader loader(path, S, B, depth, /*threads=*/2);
    EXPECT(loader.num_sequences() == 10 && loader.slot_elements() == 2 * B * S);
    std::vector<int64_t> ring(depth * loader.slot_elements(), -1);
    loader.set_ring(ring.data());
    for (int epoch = 0; epoch < 3; ++epoch) {
      std::vector<int64_t> order(10);
      std::iota(order.begin(), order.end(), 0);
      for (int64_t i = 0; i < 10; ++i) std::swap(order[i], order[(i * 3 + epoch) % 10]);
      loader.start(order.data(), 10);
      EXPECT(loader.batches_in_epoch() == 3);  // the tenth sample does not fill a batch
      std::vector<int> held;
      for (int64_t b = 0;; ++b) {
        int slot = loader.next(5000);
        if (slot < 0) {
          EXPECT(b == 3);
          break;
        }
        EXPECT(slot == b % depth);
        const int64_t* x = ring.data() + slot * loader.slot_elements();
        const int64_t* y = x + B * S;
        for (int64_t r = 0; r < B; ++r)
          for (int64_t j = 0; j < S; ++j) {
            int64_t at = order[b * B + r] * S + j;
            EXPECT(x[r * S + j] == tokens[at] && y[r * S + j] == tokens[at + 1]);
          }
        held.push_back(slot);
        if (held.size() == 2) {  // the consumer keeps two batches in flight, as a training loop that runs ahead does
          loader.release(held.front());
          held.erase(held.begin());
        }
      }
      for (int s : held) loader.release(s);
    }
    // a slot that is never released stalls the ring; the wait gives up instead of hanging
    std::vector<int64_t> order(9);
    std::iota(order.begin(), order.end(), 0);
    nt::TokenWindowLoader small(path, S, 1, 2, 1);
    std::vector<int64_t> ring2(2 * small.slot_elements());
    small.set_ring(ring2.data());
    small.start(order.data(), 9);
    EXPECT(small.next(2000) == 0 && small.next(2000) == 1);
    bool gave_up = false;
    try {
      small.next(200);
    } catch (const std::runtime_error&) {
      gave_up = true;
    }
    EXPECT(gave_up);
    bool refused = false;
    try {
      small.release(0);
      small.release(0);
    } catch (const std::logic_error&) {
      refused = true;
    }
    EXPECT(refused);
    int64_t bad[1] = {10};
    refused = false;
    try {
      small.start(bad, 1);
    } catch (const std::out_of_range&) {
      refused = true;
    }
    EXPECT(refused);
  }
  unlink(path);
  std::printf("ALL PASSED\n");
  return 0;
}
