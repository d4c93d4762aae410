#include "runtime.h"

#include <execinfo.h>
#include <pthread.h>
#include <pybind11/functional.h>
#include <pybind11/stl.h>
#include <signal.h>
#include <sys/stat.h>
#include <unistd.h>

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <sstream>

#include <dlfcn.h>

namespace py = pybind11;

namespace mb {

// ================================================================ futures + pool
void TaskState::set_done(bool ok, std::string err) {
  {
    std::lock_guard<std::mutex> g(mu_);
    ok_ = ok;
    err_ = std::move(err);
    done_.store(true, std::memory_order_release);
  }
  cv_.notify_all();
}

bool TaskState::wait(double timeout_s) {
  std::unique_lock<std::mutex> g(mu_);
  if (timeout_s < 0) {
    cv_.wait(g, [&] { return done_.load(); });
    return true;
  }
  return cv_.wait_for(g, std::chrono::duration<double>(timeout_s), [&] { return done_.load(); });
}

ThreadPool::ThreadPool(int n_threads, bool pin_threads) {
  if (n_threads < 1) n_threads = 1;
  for (int i = 0; i < n_threads; ++i) queues_.emplace_back(new Queue());
  for (int i = 0; i < n_threads; ++i) {
    workers_.emplace_back([this, i] { worker_loop(i); });
    if (pin_threads) {
      cpu_set_t set;
      CPU_ZERO(&set);
      CPU_SET(i % std::max(1u, std::thread::hardware_concurrency()), &set);
      pthread_setaffinity_np(workers_.back().native_handle(), sizeof(set), &set);
    }
  }
}

ThreadPool::~ThreadPool() {
  stop_.store(true);
  {
    std::lock_guard<std::mutex> g(sleep_mu_);
  }
  sleep_cv_.notify_all();
  for (auto& t : workers_) t.join();
}

Future ThreadPool::submit(std::function<void()> fn) {
  Future f = std::make_shared<TaskState>();
  const size_t qi = next_.fetch_add(1) % queues_.size();
  {
    std::lock_guard<std::mutex> g(queues_[qi]->mu);
    queues_[qi]->q.emplace_back(std::move(fn), f);
  }
  pending_.fetch_add(1);
  {
    std::lock_guard<std::mutex> g(sleep_mu_);
  }
  sleep_cv_.notify_one();
  return f;
}

bool ThreadPool::pop_or_steal(int id, std::pair<std::function<void()>, Future>& out) {
  {
    Queue& q = *queues_[id];
    std::lock_guard<std::mutex> g(q.mu);
    if (!q.q.empty()) {
      out = std::move(q.q.front());  // own queue: FIFO
      q.q.pop_front();
      return true;
    }
  }
  const int n = static_cast<int>(queues_.size());
  for (int k = 1; k < n; ++k) {
    Queue& q = *queues_[(id + k) % n];
    std::lock_guard<std::mutex> g(q.mu);
    if (!q.q.empty()) {
      out = std::move(q.q.back());  // steal from the other end
      q.q.pop_back();
      steals_.fetch_add(1);
      return true;
    }
  }
  return false;
}

void ThreadPool::worker_loop(int id) {
  std::pair<std::function<void()>, Future> item;
  while (true) {
    if (pop_or_steal(id, item)) {
      pending_.fetch_sub(1);
      try {
        item.first();
        item.second->set_done(true);
      } catch (const std::exception& e) {
        item.second->set_done(false, e.what());
      } catch (...) {
        item.second->set_done(false, "unknown exception");
      }
      item.first = nullptr;
      item.second.reset();
      continue;
    }
    std::unique_lock<std::mutex> g(sleep_mu_);
    if (stop_.load() && pending_.load() <= 0) return;
    sleep_cv_.wait_for(g, std::chrono::milliseconds(50),
                       [&] { return stop_.load() || pending_.load() > 0; });
    if (stop_.load() && pending_.load() <= 0) return;
  }
}

void ThreadPool::parallel_for(size_t n, size_t grain, const std::function<void(size_t, size_t)>& fn) {
  if (n == 0) return;
  if (grain == 0) grain = (n + workers_.size() - 1) / workers_.size();
  std::vector<Future> fs;
  for (size_t b = 0; b < n; b += grain) {
    const size_t e = std::min(n, b + grain);
    fs.push_back(submit([=, &fn] { fn(b, e); }));
  }
  std::string err;
  for (auto& f : fs) {
    f->wait();
    if (!f->ok() && err.empty()) err = f->error();
  }
  if (!err.empty()) throw std::runtime_error(err);
}

// ================================================================ MPSC ring
MpscRing::MpscRing(size_t cap) {
  size_t c = 2;
  while (c < cap) c <<= 1;
  cells_.reset(new Cell[c]);
  mask_ = c - 1;
  for (size_t i = 0; i < c; ++i) cells_[i].seq.store(i, std::memory_order_relaxed);
}

bool MpscRing::push(uint64_t v) {
  uint64_t pos = head_.load(std::memory_order_relaxed);
  while (true) {
    Cell& c = cells_[pos & mask_];
    const uint64_t seq = c.seq.load(std::memory_order_acquire);
    const int64_t dif = static_cast<int64_t>(seq) - static_cast<int64_t>(pos);
    if (dif == 0) {
      if (head_.compare_exchange_weak(pos, pos + 1, std::memory_order_relaxed)) {
        c.val = v;
        c.seq.store(pos + 1, std::memory_order_release);
        return true;
      }
    } else if (dif < 0) {
      return false;  // full
    } else {
      pos = head_.load(std::memory_order_relaxed);
    }
  }
}

bool MpscRing::pop(uint64_t* v) {
  Cell& c = cells_[tail_ & mask_];
  const uint64_t seq = c.seq.load(std::memory_order_acquire);
  if (static_cast<int64_t>(seq) - static_cast<int64_t>(tail_ + 1) < 0) return false;  // empty
  *v = c.val;
  c.seq.store(tail_ + mask_ + 1, std::memory_order_release);
  ++tail_;
  return true;
}

// ================================================================ logging
static std::atomic<int> g_log_level{-1};
static const char* kLevelNames[] = {"TRACE", "DEBUG", "INFO", "WARN", "ERROR"};

int log_get_level() {
  int lv = g_log_level.load(std::memory_order_relaxed);
  if (lv >= 0) return lv;
  lv = LOG_WARN;
  if (const char* e = getenv("MB200_LOG_LEVEL")) {
    for (int i = 0; i < 5; ++i)
      if (strcasecmp(e, kLevelNames[i]) == 0) lv = i;
    if (strcasecmp(e, "OFF") == 0) lv = LOG_OFF;
  }
  g_log_level.store(lv);
  return lv;
}
void log_set_level(int level) { g_log_level.store(level); }
void log_write(int level, const char* channel, const char* msg) {
  if (level < log_get_level() || level >= LOG_OFF) return;
  const auto now = std::chrono::system_clock::now().time_since_epoch();
  const double t = std::chrono::duration<double>(now).count();
  fprintf(stderr, "[%.3f] %-5s [%s] %s\n", t, kLevelNames[level], channel, msg);
}

// ================================================================ profiling ranges
struct TraceEvent {
  std::string name;
  uint64_t ts_us, dur_us;
  uint32_t tid;
};
static std::atomic<bool> g_prof_on{false};
static bool g_prof_nvtx = false;
static std::mutex g_prof_mu;
static std::vector<TraceEvent> g_events;
struct OpenRange {
  std::string name;
  uint64_t t0;
};
static thread_local std::vector<OpenRange> tl_open;
typedef int (*NvtxPushFn)(const char*);
typedef int (*NvtxPopFn)(void);
static NvtxPushFn g_nvtx_push = nullptr;
static NvtxPopFn g_nvtx_pop = nullptr;

static uint64_t now_us() {
  return std::chrono::duration_cast<std::chrono::microseconds>(
             std::chrono::steady_clock::now().time_since_epoch())
      .count();
}
void prof_enable(bool on, bool nvtx) {
  if (on && nvtx && !g_nvtx_push) {
    // NVTX v2 C symbols live in libnvToolsExt; absent on many boxes, in which case the
    // ranges are still recorded for the Chrome trace.
    if (void* h = dlopen("libnvToolsExt.so.1", RTLD_NOW | RTLD_GLOBAL)) {
      g_nvtx_push = reinterpret_cast<NvtxPushFn>(dlsym(h, "nvtxRangePushA"));
      g_nvtx_pop = reinterpret_cast<NvtxPopFn>(dlsym(h, "nvtxRangePop"));
    }
  }
  g_prof_nvtx = nvtx && g_nvtx_push && g_nvtx_pop;
  g_prof_on.store(on, std::memory_order_release);
}
bool prof_enabled() { return g_prof_on.load(std::memory_order_relaxed); }
void prof_push(const char* name) {
  if (!g_prof_on.load(std::memory_order_relaxed)) return;  // off-cost: one relaxed load
  tl_open.push_back({name, now_us()});
  if (g_prof_nvtx) g_nvtx_push(name);
}
void prof_pop() {
  if (tl_open.empty()) return;
  OpenRange r = std::move(tl_open.back());
  tl_open.pop_back();
  if (g_prof_nvtx) g_nvtx_pop();
  const uint64_t t1 = now_us();
  std::lock_guard<std::mutex> g(g_prof_mu);
  g_events.push_back({std::move(r.name), r.t0, t1 - r.t0,
                      static_cast<uint32_t>(std::hash<std::thread::id>()(std::this_thread::get_id()))});
}
std::string prof_dump_chrome_trace(bool clear) {
  std::lock_guard<std::mutex> g(g_prof_mu);
  std::ostringstream os;
  os << "{\"traceEvents\":[";
  for (size_t i = 0; i < g_events.size(); ++i) {
    const auto& e = g_events[i];
    if (i) os << ",";
    os << "{\"name\":\"";
    for (char ch : e.name) {
      if (ch == '"' || ch == '\\') os << '\\';
      os << ch;
    }
    os << "\",\"ph\":\"X\",\"pid\":" << getpid() << ",\"tid\":" << (e.tid & 0xffff)
       << ",\"ts\":" << e.ts_us << ",\"dur\":" << e.dur_us << "}";
  }
  os << "]}";
  if (clear) g_events.clear();
  return os.str();
}

// ================================================================ hashing
static inline uint64_t rotl(uint64_t x, int r) { return (x << r) | (x >> (64 - r)); }
static inline uint64_t fmix(uint64_t k) {
  k ^= k >> 33; k *= 0xff51afd7ed558ccdull;
  k ^= k >> 33; k *= 0xc4ceb9fe1a85ec53ull;
  k ^= k >> 33;
  return k;
}
// 64-bit multiply-rotate hash over 8-byte words (wyhash/murmur family construction).
uint64_t hash64(const void* data, size_t n, uint64_t seed) {
  const uint8_t* p = static_cast<const uint8_t*>(data);
  uint64_t h = seed ^ (n * 0x9E3779B97F4A7C15ull);
  size_t i = 0;
  for (; i + 8 <= n; i += 8) {
    uint64_t k;
    memcpy(&k, p + i, 8);
    k *= 0x87c37b91114253d5ull; k = rotl(k, 31); k *= 0x4cf5ad432745937full;
    h ^= k; h = rotl(h, 27) * 5 + 0x52dce729;
  }
  uint64_t k = 0;
  for (size_t j = 0; i + j < n; ++j) k |= static_cast<uint64_t>(p[i + j]) << (8 * j);
  if (n & 7) {
    k *= 0x87c37b91114253d5ull; k = rotl(k, 31); k *= 0x4cf5ad432745937full;
    h ^= k;
  }
  return fmix(h);
}

std::vector<uint64_t> hash_token_blocks(const int64_t* tokens, size_t n_tokens, size_t block,
                                        uint64_t parent, uint64_t seed) {
  std::vector<uint64_t> out;
  if (block == 0) return out;
  out.reserve(n_tokens / block);
  uint64_t h = parent;
  for (size_t b = 0; b + block <= n_tokens; b += block) {
    h = hash64(tokens + b, block * sizeof(int64_t), h ^ seed);
    out.push_back(h);
  }
  return out;
}

// ================================================================ blob cache
BlobCache::BlobCache(std::string dir, size_t mem_limit) : dir_(std::move(dir)), limit_(mem_limit) {
  if (!dir_.empty()) mkdir(dir_.c_str(), 0755);
}
std::string BlobCache::content_key(const std::string& blob) {
  char buf[40];
  snprintf(buf, sizeof(buf), "%016llx%016llx",
           static_cast<unsigned long long>(hash64(blob.data(), blob.size(), 0x1234)),
           static_cast<unsigned long long>(hash64(blob.data(), blob.size(), 0xabcdef)));
  return buf;
}
std::string BlobCache::path_of(const std::string& key) const {
  std::string safe;
  for (char c : key) safe += (isalnum(static_cast<unsigned char>(c)) || c == '-' || c == '_') ? c : '_';
  return dir_ + "/" + safe + ".blob";
}
void BlobCache::put(const std::string& key, const std::string& blob) {
  std::lock_guard<std::mutex> g(mu_);
  mem_.emplace_back(key, blob);
  used_ += blob.size();
  while (used_ > limit_ && mem_.size() > 1) {
    used_ -= mem_.front().second.size();
    mem_.pop_front();
  }
  if (!dir_.empty()) {
    const std::string tmp = path_of(key) + ".tmp" + std::to_string(getpid());
    std::ofstream f(tmp, std::ios::binary);
    f.write(blob.data(), blob.size());
    f.close();
    rename(tmp.c_str(), path_of(key).c_str());  // atomic publish
  }
}
bool BlobCache::get(const std::string& key, std::string* out) {
  std::lock_guard<std::mutex> g(mu_);
  for (auto it = mem_.rbegin(); it != mem_.rend(); ++it)
    if (it->first == key) {
      *out = it->second;
      ++hits_mem;
      return true;
    }
  if (!dir_.empty()) {
    std::ifstream f(path_of(key), std::ios::binary);
    if (f) {
      std::stringstream ss;
      ss << f.rdbuf();
      *out = ss.str();
      mem_.emplace_back(key, *out);
      used_ += out->size();
      ++hits_disk;
      return true;
    }
  }
  ++misses;
  return false;
}

// ================================================================ crash handler
static void crash_handler(int sig) {
  void* frames[64];
  const int n = backtrace(frames, 64);
  const char* msg = "\n*** modular_b200: fatal signal, native backtrace follows ***\n";
  (void)!write(2, msg, strlen(msg));
  backtrace_symbols_fd(frames, n, 2);
  signal(sig, SIG_DFL);
  raise(sig);
}
void install_crash_handler() {
  signal(SIGSEGV, crash_handler);
  signal(SIGABRT, crash_handler);
  signal(SIGBUS, crash_handler);
  signal(SIGFPE, crash_handler);
}

// ================================================================ bindings
void bind_runtime(py::module_& m) {
  py::class_<TaskState, Future>(m, "Future")
      .def("done", &TaskState::done)
      .def("ok", &TaskState::ok)
      .def("error", &TaskState::error)
      .def("wait", [](TaskState& s, double timeout) {
        py::gil_scoped_release rel;
        return s.wait(timeout);
      }, py::arg("timeout") = -1.0);

  // Joining the workers must not hold the GIL: a queued Python task may be waiting for it.
  struct PoolDeleter {
    void operator()(ThreadPool* p) const {
      py::gil_scoped_release rel;
      delete p;
    }
  };
  py::class_<ThreadPool, std::unique_ptr<ThreadPool, PoolDeleter>>(m, "ThreadPool")
      .def(py::init<int, bool>(), py::arg("n_threads"), py::arg("pin_threads") = false)
      .def("size", &ThreadPool::size)
      .def("steals", &ThreadPool::steals)
      .def("submit", [](ThreadPool& p, py::function fn) {
        auto holder = std::make_shared<py::function>(std::move(fn));
        return p.submit([holder] {
          // A Python exception must be turned into a plain C++ one while the GIL is still held: its message
          // and its destructor both touch Python objects, and the pool's catch block runs without the GIL.
          std::string failure;
          bool failed = false;
          {
            py::gil_scoped_acquire acq;
            try {
              (*holder)();
            } catch (py::error_already_set& e) {
              failure = e.what();
              failed = true;
              e.restore();
              PyErr_Clear();
            }
            holder->release().dec_ref();
          }
          if (failed) throw std::runtime_error(failure);
        });
      })
      // dst/src are raw addresses (e.g. tensor.data_ptr()); copies run without the GIL.
      .def("parallel_memcpy", [](ThreadPool& p, uintptr_t dst, uintptr_t src, size_t nbytes) {
        py::gil_scoped_release rel;
        p.parallel_for(nbytes, 4u << 20, [=](size_t b, size_t e) {
          memcpy(reinterpret_cast<char*>(dst) + b, reinterpret_cast<const char*>(src) + b, e - b);
        });
      })
      .def("submit_memcpy", [](ThreadPool& p, uintptr_t dst, uintptr_t src, size_t nbytes) {
        return p.submit([=] {
          memcpy(reinterpret_cast<void*>(dst), reinterpret_cast<const void*>(src), nbytes);
        });
      });

  py::class_<MpscRing>(m, "MpscRing")
      .def(py::init<size_t>())
      .def("push", &MpscRing::push)
      .def("pop", [](MpscRing& r) -> py::object {
        uint64_t v;
        if (r.pop(&v)) return py::int_(v);
        return py::none();
      })
      .def("capacity", &MpscRing::capacity);

  m.def("log_set_level", &log_set_level);
  m.def("log_get_level", &log_get_level);
  m.def("log_write", &log_write);
  m.def("prof_enable", &prof_enable, py::arg("on"), py::arg("nvtx") = false);
  m.def("prof_enabled", &prof_enabled);
  m.def("prof_push", &prof_push);
  m.def("prof_pop", &prof_pop);
  m.def("prof_dump_chrome_trace", &prof_dump_chrome_trace, py::arg("clear") = true);
  m.def("hash64", [](py::bytes b, uint64_t seed) {
    std::string s = b;
    return hash64(s.data(), s.size(), seed);
  });
  m.def("hash_token_blocks", [](py::buffer tokens, size_t block, uint64_t parent, uint64_t seed) {
    py::buffer_info info = tokens.request();
    if (info.itemsize != 8) throw std::runtime_error("hash_token_blocks expects int64 tokens");
    return hash_token_blocks(static_cast<const int64_t*>(info.ptr), static_cast<size_t>(info.size),
                             block, parent, seed);
  });
  py::class_<BlobCache>(m, "BlobCache")
      .def(py::init<std::string, size_t>(), py::arg("dir"), py::arg("mem_limit_bytes") = (64u << 20))
      .def("put", [](BlobCache& c, const std::string& k, py::bytes b) { c.put(k, std::string(b)); })
      .def("get", [](BlobCache& c, const std::string& k) -> py::object {
        std::string out;
        if (c.get(k, &out)) return py::bytes(out);
        return py::none();
      })
      .def_static("content_key", [](py::bytes b) { return BlobCache::content_key(std::string(b)); })
      .def_readonly("hits_mem", &BlobCache::hits_mem)
      .def_readonly("hits_disk", &BlobCache::hits_disk)
      .def_readonly("misses", &BlobCache::misses);
  m.def("install_crash_handler", &install_crash_handler);
}

}  // namespace mb
