// Command-line front end of the signalling-protocol model (protocol_model.cc), driven by
// tests/test_cpu_protocol_model.py:
//   protocol_model <nranks> <blocks> <n_ops> <seed> <use_done_chain 0|1> <slow_rank> <mix 0|1>
// prints one line: {"errors": E, "timeouts": T, "ops": N}
#include <cstdio>
#include <cstdlib>

#include "protocol_model.h"

int main(int argc, char** argv) {
  if (argc != 8) {
    std::fprintf(stderr, "usage: %s nranks blocks n_ops seed use_done_chain slow_rank mix\n", argv[0]);
    return 2;
  }
  try {
    const bagua::ProtocolModelResult r =
        bagua::run_protocol_model(std::atoi(argv[1]), std::atoi(argv[2]), std::atoi(argv[3]),
                                  (uint32_t)std::strtoul(argv[4], nullptr, 10), std::atoi(argv[5]) != 0,
                                  std::atoi(argv[6]), std::atoi(argv[7]) != 0);
    std::printf("{\"errors\": %llu, \"timeouts\": %llu, \"ops\": %llu}\n", (unsigned long long)r.errors,
                (unsigned long long)r.timeouts, (unsigned long long)r.ops);
  } catch (const std::exception& e) {
    std::fprintf(stderr, "protocol model: %s\n", e.what());
    return 1;
  }
  return 0;
}
