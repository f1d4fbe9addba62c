// Symmetric-heap slabs with an NVSwitch multicast mapping (NVLS).
//
// A slab is one physical allocation per rank made with the driver's virtual-memory-
// management API, shared between the processes of one node as POSIX file descriptors, and
// bound to one multicast object.  Every rank ends up with
//   * base[q]  – an ordinary (unicast) mapping of rank q's memory, usable exactly like the
//                CUDA-IPC slabs of the symmetric heap (peer loads and stores), and
//   * mc_base  – the multicast mapping: a `multimem.st` to mc_base + off lands at offset
//                off of every rank's memory, a `multimem.ld_reduce` from it returns the
//                element-wise sum over all ranks, computed inside the switch.
// An all-reduce on such memory moves S bytes per GPU and direction instead of 2(N-1)/N·S.
//
// The driver entry points are looked up at run time (cudaGetDriverEntryPoint), so the
// extension does not link against libcuda and still loads on a machine without a driver.
// Everything here is collective over the communicator's transport, and every step ends
// with an agreement round: either all ranks get the slab or none does, in which case the
// caller falls back to CUDA-IPC slabs.
#pragma once

#include <cuda_runtime_api.h>

#include <string>

#include "transport.h"

namespace bagua {

constexpr int kMulticastMaxRanks = 8;

struct MulticastSlab {
  char* base[kMulticastMaxRanks] = {};
  char* mc_base = nullptr;
  size_t bytes = 0;
  void* impl = nullptr;  // driver handles, for teardown
};

// The CUDA runtime calls and the driver lookup that the setup uses, as a table: with a stand-in
// for it the whole sequence — above all the agreement between ranks after every step and the
// clean-up when a step fails — runs on a machine without a GPU (tests/cpp/nvls_setup.cc).
struct MulticastPlatform {
  bool (*select_device)(int device);
  void* (*driver_entry)(const char* name);  // nullptr: the driver does not have it
  void* (*scratch_alloc)(size_t bytes);     // memory the transport can all-gather through; nullptr on failure
  void (*scratch_free)(void* p);
  bool (*to_scratch)(void* dst, const void* src, size_t bytes, cudaStream_t stream);
  bool (*from_scratch)(void* dst, const void* src, size_t bytes, cudaStream_t stream);  // finished on return
  bool (*clear)(void* mapped, size_t bytes, cudaStream_t stream);                       // zero-fill, finished on return
};
// nullptr restores the CUDA runtime.  Call while no setup is running.
void set_multicast_platform(const MulticastPlatform* platform);

// Collective.  `bytes` is rounded up to the multicast granularity.  Returns false on every
// rank alike, with the first failing step in `why`, and leaves nothing allocated.
bool create_multicast_slab(Transport& transport, int rank, int nranks, int device, cudaStream_t stream, size_t bytes,
                           MulticastSlab* out, std::string* why);

// Unbinds, unmaps and releases.  Local; call on every rank before the transport goes away.
void destroy_multicast_slab(MulticastSlab& slab);

// Unbinds and unmaps every slab this process still holds (their pointers dangle afterwards)
// and returns how many there were.  For process exit: a process should not die while its
// memory is still bound to a multicast object that other GPUs use.
int release_all_multicast_slabs();

}  // namespace bagua
