// Engine-wide counters (what `_C.stats()` reports).  The reference has no counters; its
// observability is log lines (bagua-core-internal/src/lib.rs:228-240).
#pragma once

#include <atomic>
#include <cstdint>

namespace bagua {

struct EngineStats {
  std::atomic<uint64_t> buckets_scheduled{0};
  std::atomic<uint64_t> ops_executed{0};
  std::atomic<uint64_t> fused_launches{0};
  std::atomic<uint64_t> library_fallbacks{0};
  std::atomic<uint64_t> staged_copies{0};
  std::atomic<uint64_t> bytes_communicated{0};
  static EngineStats& global();
};

}  // namespace bagua
