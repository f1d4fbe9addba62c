// Host-thread model of the fused kernels' signalling protocol (see protocol_model.cc).
#pragma once

#include "common.h"

namespace bagua {

struct ProtocolModelResult {
  uint64_t errors = 0;    // payload words that did not hold the expected value
  uint64_t timeouts = 0;  // bounded waits that ran out
  uint64_t ops = 0;
};

// nranks in [2, 8], blocks in [1, 8].  slow_rank >= 0 makes that rank linger before the
// final copy-out of every two-shot op and fixes sizes so that consecutive ops overlap in
// staging (the adversarial schedule); -1 = random jitter only.  mix = false alternates the
// two all-reduce layouts; mix = true draws every op from all kernels of the communicator
// (all-reduces, all-gather, all-to-all, reduce-scatter, their direct-peer-access variants,
// broadcasts, barrier).
ProtocolModelResult run_protocol_model(int nranks, int blocks, int n_ops, uint32_t seed, bool use_done_chain,
                                       int slow_rank, bool mix = false);

}  // namespace bagua
