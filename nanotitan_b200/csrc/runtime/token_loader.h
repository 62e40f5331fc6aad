// Batches of next-token training windows, cut from a memory-mapped uint16 token file by background threads into a
// ring of caller-owned (pinned) int64 buffers.
//
// Sample i of a file is the window tokens[i*S, i*S + S]: inputs are its first S tokens, targets the last S (the
// reference's dataset rule, src/data/dataset.py:8-27).  The reference builds batches with a torch DataLoader, one
// Python __getitem__ per sample in worker processes; here a step's batch is one widening copy per sample straight
// into the buffer the host-to-device copy reads, so the loader keeps up with a GPU that consumes a batch every few
// tens of milliseconds without occupying CPU cores with interpreters.
//
// Ring protocol: batch b goes to slot b % depth.  A worker may write the slot once the consumer has released batch
// b - depth; the consumer takes batches in order with `next()` and hands slots back with `release()`.  All waits
// have a time limit.
#pragma once

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <mutex>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

namespace nt {

class TokenWindowLoader {
 public:
  TokenWindowLoader(const std::string& path, int64_t seq_len, int64_t batch, int depth, int threads)
      : seq_len_(seq_len), batch_(batch), depth_(depth), threads_(threads) {
    if (seq_len < 1 || batch < 1 || depth < 2 || threads < 1) throw std::invalid_argument("token loader: bad geometry");
    fd_ = ::open(path.c_str(), O_RDONLY | O_CLOEXEC);
    if (fd_ < 0) throw std::runtime_error("token loader: cannot open " + path);
    struct stat st;
    if (::fstat(fd_, &st) != 0 || st.st_size < 4) {
      ::close(fd_);
      throw std::runtime_error("token loader: " + path + " is empty");
    }
    bytes_ = static_cast<size_t>(st.st_size);
    void* p = ::mmap(nullptr, bytes_, PROT_READ, MAP_SHARED, fd_, 0);
    if (p == MAP_FAILED) {
      ::close(fd_);
      throw std::runtime_error("token loader: cannot map " + path);
    }
    tokens_ = static_cast<const uint16_t*>(p);
    n_tokens_ = static_cast<int64_t>(bytes_ / 2);
    n_sequences_ = (n_tokens_ - 1) / seq_len_;  // one more token than inputs, for the shifted targets
  }
  TokenWindowLoader(const TokenWindowLoader&) = delete;
  TokenWindowLoader& operator=(const TokenWindowLoader&) = delete;
  ~TokenWindowLoader() {
    stop();
    ::munmap(const_cast<uint16_t*>(tokens_), bytes_);
    ::close(fd_);
  }

  int64_t num_sequences() const { return n_sequences_; }
  int64_t slot_elements() const { return 2 * batch_ * seq_len_; }  // inputs then targets
  int64_t batches_in_epoch() const { return n_batches_; }

  // `ring` holds depth * slot_elements() int64 values and outlives the loader's use of it.
  void set_ring(int64_t* ring) { ring_ = ring; }

  // Begin an epoch over `order` (sample indices in visiting order); a trailing partial batch is dropped.
  void start(const int64_t* order, int64_t n) {
    if (ring_ == nullptr) throw std::logic_error("token loader: no ring buffer set");
    stop();
    for (int64_t i = 0; i < n; ++i)
      if (order[i] < 0 || order[i] >= n_sequences_)
        throw std::out_of_range("token loader: sample " + std::to_string(order[i]) + " of " + std::to_string(n_sequences_));
    order_.assign(order, order + n);
    n_batches_ = n / batch_;
    owner_.assign(depth_, 0);
    ready_.assign(depth_, -1);
    for (int s = 0; s < depth_; ++s) owner_[s] = s;
    next_fill_.store(0);
    consumed_ = 0;
    stopping_ = false;
    error_.clear();
    for (int t = 0; t < threads_; ++t) workers_.emplace_back([this] { work(); });
  }

  // Slot of the next batch, or -1 when the epoch is over.
  int next(int timeout_ms) {
    std::unique_lock<std::mutex> lock(mu_);
    if (consumed_ >= n_batches_) return -1;
    const int64_t b = consumed_;
    const int s = static_cast<int>(b % depth_);
    bool ok = cv_.wait_for(lock, std::chrono::milliseconds(timeout_ms), [&] { return ready_[s] == b || !error_.empty(); });
    if (!error_.empty()) throw std::runtime_error("token loader: " + error_);
    if (!ok) throw std::runtime_error("token loader: batch " + std::to_string(b) + " was not ready within " +
                                      std::to_string(timeout_ms) + " ms (was a slot never released?)");
    ++consumed_;
    return s;
  }

  // The consumer is done with the batch in `slot` (its host-to-device copy has completed).
  void release(int slot) {
    {
      std::lock_guard<std::mutex> lock(mu_);
      if (slot < 0 || slot >= depth_) throw std::out_of_range("token loader: bad slot");
      if (ready_[slot] != owner_[slot] || ready_[slot] >= consumed_)
        throw std::logic_error("token loader: slot released twice or before it was taken");
      owner_[slot] += depth_;
    }
    cv_.notify_all();
  }

  void stop() {
    {
      std::lock_guard<std::mutex> lock(mu_);
      stopping_ = true;
    }
    cv_.notify_all();
    for (auto& w : workers_) w.join();
    workers_.clear();
  }

 private:
  void work() {
    try {
      for (;;) {
        const int64_t b = next_fill_.fetch_add(1);
        if (b >= n_batches_) return;
        const int s = static_cast<int>(b % depth_);
        {
          std::unique_lock<std::mutex> lock(mu_);
          cv_.wait(lock, [&] { return owner_[s] == b || stopping_; });
          if (stopping_) return;
        }
        int64_t* x = ring_ + static_cast<int64_t>(s) * slot_elements();
        int64_t* y = x + batch_ * seq_len_;
        for (int64_t r = 0; r < batch_; ++r) {
          const uint16_t* src = tokens_ + order_[b * batch_ + r] * seq_len_;
          int64_t* xr = x + r * seq_len_;
          int64_t* yr = y + r * seq_len_;
          int64_t prev = src[0];
          for (int64_t j = 0; j < seq_len_; ++j) {  // each token is read once: it is input j+1 and target j
            const int64_t cur = src[j + 1];
            xr[j] = prev;
            yr[j] = cur;
            prev = cur;
          }
        }
        {
          std::lock_guard<std::mutex> lock(mu_);
          ready_[s] = b;
        }
        cv_.notify_all();
      }
    } catch (const std::exception& e) {
      std::lock_guard<std::mutex> lock(mu_);
      error_ = e.what();
      cv_.notify_all();
    }
  }

  int64_t seq_len_, batch_;
  int depth_, threads_;
  int fd_ = -1;
  size_t bytes_ = 0;
  const uint16_t* tokens_ = nullptr;
  int64_t n_tokens_ = 0, n_sequences_ = 0, n_batches_ = 0;
  int64_t* ring_ = nullptr;
  std::vector<int64_t> order_;
  std::mutex mu_;
  std::condition_variable cv_;
  std::vector<int64_t> owner_, ready_;  // per slot: batch allowed to write it / batch it holds
  std::atomic<int64_t> next_fill_{0};
  int64_t consumed_ = 0;
  bool stopping_ = false;
  std::string error_;
  std::vector<std::thread> workers_;
};

}  // namespace nt
