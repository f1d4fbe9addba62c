/* C interface to the communicator (opaque handle).
 *
 * Counterpart of the reference's C binding stub (bagua-core-c/src/lib.rs:5-69):
 * create / destroy / nranks of a single communicator.  Here the symbols really are
 * exported from the shared object (the reference declares them without #[no_mangle]),
 * and `rank` / `device_id` accessors are added.  Return codes: 0 success, -1 null
 * pointer, -2 the call raised an error (text available from
 * bagua_core_c_last_error()).
 */
#ifndef BAGUA_CORE_C_H_
#define BAGUA_CORE_C_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BAGUA_C_API __attribute__((visibility("default")))

typedef struct BaguaSingleCommunicatorC BaguaSingleCommunicatorC;

/* Blocks until all `nranks` ranks have joined.  Returns NULL on failure. */
BAGUA_C_API BaguaSingleCommunicatorC* bagua_single_communicator_c_create(size_t rank, size_t nranks,
                                                                         size_t device_id, uint64_t stream_ptr,
                                                                         const char* nccl_unique_id_str);
/* Frees the communicator and sets *ptr to NULL.  A NULL handle is ignored. */
BAGUA_C_API void bagua_single_communicator_c_destroy(BaguaSingleCommunicatorC** ptr);
BAGUA_C_API int32_t bagua_single_communicator_c_nranks(BaguaSingleCommunicatorC** ptr, size_t* nranks);
BAGUA_C_API int32_t bagua_single_communicator_c_rank(BaguaSingleCommunicatorC** ptr, size_t* rank);
BAGUA_C_API int32_t bagua_single_communicator_c_device_id(BaguaSingleCommunicatorC** ptr, size_t* device_id);
/* Writes a fresh base64 NCCL unique id (NUL-terminated) into buf; returns its length or -2. */
BAGUA_C_API int32_t bagua_core_c_generate_nccl_unique_id_str(char* buf, size_t buf_len);
BAGUA_C_API const char* bagua_core_c_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* BAGUA_CORE_C_H_ */
