// Stress test of the host runtime (scheduler, channels, pools, buckets) meant to be built
// with -fsanitize=thread or -fsanitize=address: several producer threads mark tensors ready
// while the worker thread executes callback ops and a waiter drains completions.
// Exit code 0 = all invariants held (and the sanitizer, if any, stayed silent).
#include <atomic>
#include <cstdio>
#include <thread>

#include "comm/communicator.h"
#include "ops/comm_op.h"
#include "pool/resource_pool.h"
#include "runtime/backend.h"
#include "protocol_model.h"
#include "tensor/tensor.h"

using namespace bagua;

namespace {
struct HostTensor : RawTensor {
  explicit HostTensor(int64_t n) : buf((size_t)n, 0.f) {}
  void* data_ptr() const override { return (void*)buf.data(); }
  int64_t num_elements() const override { return (int64_t)buf.size(); }
  int64_t num_elements_allocated() const override { return (int64_t)buf.size(); }
  int device_id() const override { return -1; }
  DType dtype() const override { return DType::F32; }
  std::vector<float> buf;
};
}  // namespace

int main() {
  const int kBuckets = 8, kTensorsPerBucket = 4, kRounds = 200;
  CommBackend backend(4, -1);  // small capacity: exercises back-pressure
  std::vector<BucketPtr> buckets;
  std::vector<std::vector<TensorPtr>> tensors((size_t)kBuckets);
  std::atomic<int> executed{0};
  std::vector<int> order;
  std::mutex order_mu;
  for (int b = 0; b < kBuckets; ++b) {
    for (int t = 0; t < kTensorsPerBucket; ++t)
      tensors[b].push_back(std::make_shared<BaguaTensor>("t" + std::to_string(b) + "_" + std::to_string(t),
                                                         std::make_shared<HostTensor>(64)));
    auto bucket = std::make_shared<BaguaBucket>("b" + std::to_string(b), tensors[b]);
    bucket->append_op(make_callback_op(
        [&, b](const std::string&) {
          executed++;
          std::lock_guard<std::mutex> g(order_mu);
          order.push_back(b);
          // pool traffic from the worker thread
          auto blk = MemoryPool::for_device(-1).pull(1000 + 37 * b, /*stream_tag=*/(uint64_t)b % 3);
          std::memset(blk->ptr(), b, 1000);
        },
        "stress"));
    buckets.push_back(bucket);
  }
  backend.register_ordered_buckets(buckets);

  size_t waited = 0;
  for (int round = 0; round < kRounds; ++round) {
    // four producer threads mark disjoint tensors ready in a scrambled order
    std::vector<std::thread> producers;
    for (int p = 0; p < 4; ++p)
      producers.emplace_back([&, p] {
        for (int b = kBuckets - 1; b >= 0; --b)
          for (int t = 0; t < kTensorsPerBucket; ++t)
            if ((b + t) % 4 == p) backend.mark_communication_ready(tensors[b][t], 0);
        // pool traffic from producer threads as well
        auto blk = MemoryPool::for_device(-1).pull(4096, (uint64_t)p);
        std::memset(blk->ptr(), p, 4096);
      });
    for (auto& th : producers) th.join();
    waited += backend.wait_pending_comm_ops();
  }
  int failures = 0;
  if (executed.load() != kBuckets * kRounds || (int)waited != kBuckets * kRounds) {
    std::fprintf(stderr, "executed %d, waited %zu, expected %d\n", executed.load(), waited, kBuckets * kRounds);
    ++failures;
  }
  for (size_t i = 0; i < order.size(); ++i)
    if (order[i] != (int)(i % kBuckets)) {
      std::fprintf(stderr, "bucket order violated at %zu: got %d\n", i, order[i]);
      ++failures;
      break;
    }
  // the signalling-protocol model (atomics only) must also be clean under the sanitizer
  for (uint32_t seed = 0; seed < 6; ++seed) {
    ProtocolModelResult r =
        run_protocol_model(4, 2, 30, seed, /*use_done_chain=*/true, /*slow_rank=*/-1, /*mix=*/seed >= 3);
    if (r.errors || r.timeouts) {
      std::fprintf(stderr, "protocol model: %llu errors, %llu timeouts\n", (unsigned long long)r.errors,
                   (unsigned long long)r.timeouts);
      ++failures;
    }
  }
  std::printf("runtime stress: %d bucket executions, %zu waited, %d failures\n", executed.load(), waited, failures);
  return failures ? 1 : 0;
}
