#include "resource_pool.h"

#include <cuda_runtime.h>

namespace bagua {

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
    if (device_ >= 0) {
      int prev = -1;
      cudaGetDevice(&prev);
      if (prev != device_) cudaSetDevice(device_);
      cudaError_t e = cudaMalloc(&ptr, cls);
      if (e != cudaSuccess) {
        // give cached blocks back to the device and retry once
        release_cached();
        e = cudaMalloc(&ptr, cls);
      }
      if (prev >= 0 && prev != device_) cudaSetDevice(prev);
      if (e != cudaSuccess) {
        cudaGetLastError();
        throw BaguaError(ErrorKind::MemPool, "cudaMalloc of " + std::to_string(cls) + " bytes on device " +
                                                 std::to_string(device_) + " failed: " + cudaGetErrorString(e));
      }
    } else {
      ptr = std::aligned_alloc(256, align_up(cls, 256));
      if (!ptr) throw BaguaError(ErrorKind::MemPool, "host allocation of " + std::to_string(cls) + " bytes failed");
    }
    std::lock_guard<std::mutex> g(mu_);
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
  free_[{cls, tag}].push_back(ptr);
  stats_.bytes_in_use -= cls;
}

void MemoryPool::release_cached() {
  std::map<std::pair<size_t, uint64_t>, std::vector<void*>> taken;
  {
    std::lock_guard<std::mutex> g(mu_);
    taken.swap(free_);
    for (auto& kv : taken) stats_.bytes_reserved -= kv.first.first * kv.second.size();
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
