#include "resource_pool.h"

#include <cuda_runtime.h>

#include <atomic>

namespace bagua {

namespace {
std::atomic<int> g_guard{-1};  // -1: not decided yet (environment), 0 / 1

// Offset of the first byte of `p[0..n)` that is not the guard pattern, or -1.
long first_damaged(const unsigned char* p, size_t n) {
  for (size_t i = 0; i < n; ++i)
    if (p[i] != MemoryPool::kGuardPattern) return (long)i;
  return -1;
}
}  // namespace

void MemoryPool::set_guard(bool on) { g_guard.store(on ? 1 : 0); }
bool MemoryPool::guard() {
  int g = g_guard.load();
  if (g < 0) {
    g = env_long("BAGUA_B200_POOL_GUARD", 0) != 0 ? 1 : 0;
    int expected = -1;
    g_guard.compare_exchange_strong(expected, g);
    g = g_guard.load();
  }
  return g == 1;
}

void log_write(LogLevel l, const char* file, int line, const std::string& msg) {
  static const char* names[] = {"TRACE", "DEBUG", "INFO", "WARN", "ERROR", "OFF"};
  static std::mutex mu;
  const char* base = std::strrchr(file, '/');
  std::lock_guard<std::mutex> g(mu);
  std::fprintf(stderr, "[bagua-b200 %s %s:%d] %s\n", names[(int)l], base ? base + 1 : file, line, msg.c_str());
}

PoolBlock::~PoolBlock() {
  if (pool_ && ptr_) pool_->give_back(ptr_, cls_, tag_);
}

size_t MemoryPool::size_class(size_t bytes) {
  size_t c = kMinClass;
  while (c < bytes) c <<= 1;
  return c;
}

MemoryPool& MemoryPool::for_device(int device) {
  BAGUA_CHECK(device >= -1 && device < kMaxDevices, MemPool, "device index " << device << " out of range");
  static std::array<std::unique_ptr<MemoryPool>, kMaxDevices + 1> pools;
  static std::mutex mu;
  std::lock_guard<std::mutex> g(mu);
  auto& p = pools[(size_t)(device + 1)];
  if (!p) p = std::make_unique<MemoryPool>(device);
  return *p;
}

std::shared_ptr<PoolBlock> MemoryPool::pull(size_t bytes, uint64_t tag) {
  const size_t cls = size_class(bytes == 0 ? 1 : bytes);
  void* ptr = nullptr;
  {
    std::lock_guard<std::mutex> g(mu_);
    stats_.pulls++;
    auto it = free_.find({cls, tag});
    if (it != free_.end() && !it->second.empty()) {
      ptr = it->second.back();
      it->second.pop_back();
    }
  }
  if (!ptr) {
    const bool guarded = guard();
    const size_t raw = cls + (guarded ? 2 * kGuardBytes : 0);
    if (device_ >= 0) {
      int prev = -1;
      cudaGetDevice(&prev);
      if (prev != device_) cudaSetDevice(device_);
      cudaError_t e = cudaMalloc(&ptr, raw);
      if (e != cudaSuccess) {
        // give cached blocks back to the device and retry once
        release_cached();
        e = cudaMalloc(&ptr, raw);
      }
      if (e == cudaSuccess && guarded) {
        cudaMemset(ptr, kGuardPattern, kGuardBytes);
        e = cudaMemset(static_cast<char*>(ptr) + kGuardBytes + cls, kGuardPattern, kGuardBytes);
      }
      if (prev >= 0 && prev != device_) cudaSetDevice(prev);
      if (e != cudaSuccess) {
        cudaGetLastError();
        throw BaguaError(ErrorKind::MemPool, "cudaMalloc of " + std::to_string(cls) + " bytes on device " +
                                                 std::to_string(device_) + " failed: " + cudaGetErrorString(e));
      }
    } else {
      ptr = std::aligned_alloc(256, align_up(raw, 256));
      if (!ptr) throw BaguaError(ErrorKind::MemPool, "host allocation of " + std::to_string(cls) + " bytes failed");
      if (guarded) {
        std::memset(ptr, kGuardPattern, kGuardBytes);
        std::memset(static_cast<char*>(ptr) + kGuardBytes + cls, kGuardPattern, kGuardBytes);
      }
    }
    std::lock_guard<std::mutex> g(mu_);
    if (guarded) {
      ptr = static_cast<char*>(ptr) + kGuardBytes;  // still 256-byte aligned
      guarded_[ptr] = cls;
    }
    stats_.device_allocs++;
    stats_.bytes_reserved += cls;
  }
  {
    std::lock_guard<std::mutex> g(mu_);
    stats_.bytes_in_use += cls;
  }
  return std::make_shared<PoolBlock>(this, ptr, bytes, cls, tag);
}

void MemoryPool::give_back(void* ptr, size_t cls, uint64_t tag) {
  std::lock_guard<std::mutex> g(mu_);
  if (device_ < 0 && guarded_.count(ptr)) {
    // host memory can be looked at right away: a block is checked every time it comes back
    const unsigned char* p = static_cast<const unsigned char*>(ptr);
    if ((first_damaged(p - kGuardBytes, kGuardBytes) >= 0 || first_damaged(p + cls, kGuardBytes) >= 0) &&
        reported_.insert(ptr).second) {
      stats_.guard_violations++;
      BAGUA_LOG(Error, "host pool block of " << cls << " bytes came back with an overwritten guard region");
    }
  }
  free_[{cls, tag}].push_back(ptr);
  stats_.bytes_in_use -= cls;
}

void MemoryPool::release_cached() {
  std::map<std::pair<size_t, uint64_t>, std::vector<void*>> taken;
  {
    std::lock_guard<std::mutex> g(mu_);
    taken.swap(free_);
    for (auto& kv : taken) {
      stats_.bytes_reserved -= kv.first.first * kv.second.size();
      for (void*& p : kv.second)
        if (guarded_.erase(p)) {  // the allocation starts at the front guard
          reported_.erase(p);
          p = static_cast<char*>(p) - kGuardBytes;
        }
    }
  }
  for (auto& kv : taken)
    for (void* p : kv.second) {
      if (device_ >= 0)
        cudaFree(p);  // implicit device synchronisation makes this safe for any stream
      else
        std::free(p);
    }
}

MemoryPool::~MemoryPool() {
  // Device memory is reclaimed by the driver at process exit; calling cudaFree from a
  // static destructor can run after the runtime has shut down.
  if (device_ < 0) release_cached();
}

size_t MemoryPool::check_guards() {
  std::vector<std::pair<void*, size_t>> blocks;
  {
    std::lock_guard<std::mutex> g(mu_);
    blocks.assign(guarded_.begin(), guarded_.end());
  }
  if (blocks.empty()) return 0;
  int prev = -1;
  if (device_ >= 0) {
    cudaGetDevice(&prev);
    if (prev != device_) cudaSetDevice(device_);
    BAGUA_CUDA_CHECK(cudaDeviceSynchronize());
  }
  size_t damaged = 0;
  unsigned char front[kGuardBytes], back[kGuardBytes];
  for (auto& [ptr, cls] : blocks) {
    const unsigned char* f = static_cast<const unsigned char*>(ptr) - kGuardBytes;
    const unsigned char* b = static_cast<const unsigned char*>(ptr) + cls;
    if (device_ >= 0) {
      BAGUA_CUDA_CHECK(cudaMemcpy(front, f, kGuardBytes, cudaMemcpyDeviceToHost));
      BAGUA_CUDA_CHECK(cudaMemcpy(back, b, kGuardBytes, cudaMemcpyDeviceToHost));
      f = front;
      b = back;
    }
    const long bad_front = first_damaged(f, kGuardBytes), bad_back = first_damaged(b, kGuardBytes);
    if (bad_front < 0 && bad_back < 0) continue;
    ++damaged;
    std::lock_guard<std::mutex> g(mu_);
    if (reported_.insert(ptr).second) {
      stats_.guard_violations++;
      BAGUA_LOG(Error, "pool block of " << cls << " bytes on device " << device_ << ": guard region overwritten "
                                        << (bad_front >= 0 ? "before the block, " : "behind the block, ")
                                        << (bad_front >= 0 ? (long)kGuardBytes - bad_front : bad_back)
                                        << (bad_front >= 0 ? " bytes in front of its start" : " bytes past its capacity"));
    }
  }
  if (device_ >= 0 && prev >= 0 && prev != device_) cudaSetDevice(prev);
  return damaged;
}

PoolStats MemoryPool::stats() const {
  std::lock_guard<std::mutex> g(mu_);
  return stats_;
}

EventLease::~EventLease() {
  if (pool_ && ev_) pool_->give_back(ev_);
}

EventPool& EventPool::instance() {
  static EventPool* p = new EventPool();  // leaked on purpose: see ~MemoryPool
  return *p;
}

std::unique_ptr<EventLease> EventPool::take() {
  int dev = 0;
  BAGUA_CUDA_CHECK(cudaGetDevice(&dev));
  {
    std::lock_guard<std::mutex> g(mu_);
    auto& v = free_[dev];
    if (!v.empty()) {
      cudaEvent_t ev = v.back();
      v.pop_back();
      return std::make_unique<EventLease>(this, ev);
    }
  }
  cudaEvent_t ev;
  BAGUA_CUDA_CHECK(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
  {
    std::lock_guard<std::mutex> g(mu_);
    owner_[ev] = dev;
  }
  return std::make_unique<EventLease>(this, ev);
}

void EventPool::give_back(cudaEvent_t ev) {
  std::lock_guard<std::mutex> g(mu_);
  free_[owner_[ev]].push_back(ev);
}

size_t EventPool::cached() const {
  std::lock_guard<std::mutex> g(mu_);
  size_t n = 0;
  for (auto& kv : free_) n += kv.second.size();
  return n;
}

EventPool::~EventPool() {}

}  // namespace bagua
