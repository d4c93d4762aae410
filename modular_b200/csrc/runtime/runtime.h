// Host-side native runtime: work-stealing thread pool with futures, bounded MPSC ring,
// levelled logger, profiling ranges (Chrome trace + optional NVTX), content-addressable
// blob cache, chained KV-block hashing and a crash backtrace handler.
//
// These are the counterparts of the reference's native support libraries
// (AsyncRT/lib/Runtime/ThreadPoolWorkQueue.cpp, AsyncRT/include/AsyncRT/Support/
// LockFreeRingBuffer.h, Support/lib/Log.cpp, Support/include/Support/Profiling/Ranges.h,
// Cache/lib/BlobCache.cpp, Init/lib/DevelopmentSignalHandler.cpp, and the block hasher
// in max/python/max/_core_mojo/mojo_module.mojo), sized for what a serving process needs.
#pragma once
#include <pybind11/pybind11.h>

#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <deque>
#include <functional>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

namespace mb {

// ---------------------------------------------------------------- futures + pool
class TaskState {
 public:
  void set_done(bool ok, std::string err = {});
  bool wait(double timeout_s = -1.0);  // false on timeout
  bool done() const { return done_.load(std::memory_order_acquire); }
  bool ok() const { return ok_; }
  const std::string& error() const { return err_; }

 private:
  std::mutex mu_;
  std::condition_variable cv_;
  std::atomic<bool> done_{false};
  bool ok_ = true;
  std::string err_;
};
using Future = std::shared_ptr<TaskState>;

class ThreadPool {
 public:
  explicit ThreadPool(int n_threads, bool pin_threads = false);
  ~ThreadPool();
  Future submit(std::function<void()> fn);
  // Splits [0, n) into chunks and runs fn(begin, end) on the pool; blocks until done.
  void parallel_for(size_t n, size_t grain, const std::function<void(size_t, size_t)>& fn);
  int size() const { return static_cast<int>(workers_.size()); }
  uint64_t steals() const { return steals_.load(); }

 private:
  struct Queue {
    std::mutex mu;
    std::deque<std::pair<std::function<void()>, Future>> q;
  };
  void worker_loop(int id);
  bool pop_or_steal(int id, std::pair<std::function<void()>, Future>& out);
  std::vector<std::unique_ptr<Queue>> queues_;
  std::vector<std::thread> workers_;
  std::mutex sleep_mu_;
  std::condition_variable sleep_cv_;
  std::atomic<int64_t> pending_{0};
  std::atomic<uint64_t> next_{0}, steals_{0};
  std::atomic<bool> stop_{false};
};

// ---------------------------------------------------------------- MPSC ring
// Bounded multi-producer / single-consumer queue of 64-bit payloads (Vyukov-style
// sequence numbers; no locks, no allocation after construction).
class MpscRing {
 public:
  explicit MpscRing(size_t capacity_pow2);
  bool push(uint64_t v);
  bool pop(uint64_t* v);
  size_t capacity() const { return mask_ + 1; }

 private:
  struct Cell {
    std::atomic<uint64_t> seq;
    uint64_t val;
  };
  std::unique_ptr<Cell[]> cells_;
  size_t mask_;
  alignas(64) std::atomic<uint64_t> head_{0};
  alignas(64) uint64_t tail_ = 0;
};

// ---------------------------------------------------------------- logging
enum LogLevel { LOG_TRACE = 0, LOG_DEBUG, LOG_INFO, LOG_WARN, LOG_ERROR, LOG_OFF };
void log_set_level(int level);
int log_get_level();
void log_write(int level, const char* channel, const char* msg);

// ---------------------------------------------------------------- profiling ranges
void prof_enable(bool on, bool nvtx);
bool prof_enabled();
void prof_push(const char* name);
void prof_pop();
std::string prof_dump_chrome_trace(bool clear);

// ---------------------------------------------------------------- hashing
uint64_t hash64(const void* data, size_t n, uint64_t seed);
// Chained hashes of consecutive `block` token groups: h[i] = H(h[i-1] || tokens of block i).
std::vector<uint64_t> hash_token_blocks(const int64_t* tokens, size_t n_tokens, size_t block,
                                        uint64_t parent, uint64_t seed);

// ---------------------------------------------------------------- blob cache
class BlobCache {
 public:
  BlobCache(std::string dir, size_t mem_limit_bytes);
  void put(const std::string& key, const std::string& blob);
  bool get(const std::string& key, std::string* out);
  static std::string content_key(const std::string& blob);
  uint64_t hits_mem = 0, hits_disk = 0, misses = 0;

 private:
  std::string path_of(const std::string& key) const;
  std::string dir_;
  size_t limit_, used_ = 0;
  std::mutex mu_;
  std::deque<std::pair<std::string, std::string>> mem_;  // FIFO eviction
};

void install_crash_handler();
void bind_runtime(pybind11::module_& m);

}  // namespace mb
