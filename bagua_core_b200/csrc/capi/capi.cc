#include "bagua_core_c.h"

#include "../comm/communicator.h"

struct BaguaSingleCommunicatorC {
  std::shared_ptr<bagua::SingleCommunicator> inner;
};

namespace {
thread_local std::string g_last_error;
}

extern "C" {

BaguaSingleCommunicatorC* bagua_single_communicator_c_create(size_t rank, size_t nranks, size_t device_id,
                                                             uint64_t stream_ptr, const char* nccl_unique_id_str) {
  if (!nccl_unique_id_str) {
    g_last_error = "nccl_unique_id_str is NULL";
    return nullptr;
  }
  try {
    // A "c10d:<group>" id selects the host transport, for which the device id is unused.
    const std::string uid(nccl_unique_id_str);
    const int dev = bagua::is_c10d_unique_id(uid) ? -1 : (int)device_id;
    auto* obj = new BaguaSingleCommunicatorC();
    obj->inner = std::make_shared<bagua::SingleCommunicator>((int)rank, (int)nranks, dev, stream_ptr, uid);
    return obj;
  } catch (const std::exception& e) {
    g_last_error = e.what();
    return nullptr;
  }
}

void bagua_single_communicator_c_destroy(BaguaSingleCommunicatorC** ptr) {
  if (!ptr || !*ptr) return;
  delete *ptr;
  *ptr = nullptr;
}

int32_t bagua_single_communicator_c_nranks(BaguaSingleCommunicatorC** ptr, size_t* nranks) {
  if (!ptr || !*ptr || !nranks) return -1;
  *nranks = (size_t)(*ptr)->inner->nranks();
  return 0;
}
int32_t bagua_single_communicator_c_rank(BaguaSingleCommunicatorC** ptr, size_t* rank) {
  if (!ptr || !*ptr || !rank) return -1;
  *rank = (size_t)(*ptr)->inner->rank();
  return 0;
}
int32_t bagua_single_communicator_c_device_id(BaguaSingleCommunicatorC** ptr, size_t* device_id) {
  if (!ptr || !*ptr || !device_id) return -1;
  *device_id = (size_t)(*ptr)->inner->device_id();
  return 0;
}
int32_t bagua_core_c_generate_nccl_unique_id_str(char* buf, size_t buf_len) {
  if (!buf) return -1;
  try {
    std::string s = bagua::nccl_generate_unique_id_b64();
    if (s.size() + 1 > buf_len) {
      g_last_error = "buffer too small for the unique id";
      return -2;
    }
    std::memcpy(buf, s.c_str(), s.size() + 1);
    return (int32_t)s.size();
  } catch (const std::exception& e) {
    g_last_error = e.what();
    return -2;
  }
}
const char* bagua_core_c_last_error(void) { return g_last_error.c_str(); }

}  // extern "C"
