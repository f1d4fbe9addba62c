/* MinMaxUInt8 compression for callers that must not allocate device memory.
 *
 * This entry point has no counterpart in the reference: there, every compress call
 * pulls its output and its reduction scratch from a cudaMalloc-backed pool
 * (bagua-core-internal/src/datatypes/mod.rs:327-345).
 *
 * Who needs it: code that runs where an allocation is not an option — inside a
 * framework allocator callback, in a process whose device memory is already fully handed
 * out to another pool, or in a latency-critical loop where a cudaMalloc (which
 * synchronises the device) would stall every stream.  Such callers own their input and output buffers already; what they
 * cannot provide is the small scratch the kernels need for per-block partial minima and
 * maxima.  Here that scratch is a fixed 64 KiB array that lives in the library's device
 * image (each GPU that loads the library holds its own copy until the process exits).
 *
 * Contract
 *  - fp32 input of `num_elements` values, split into `n_chunks` equal chunks
 *    (num_elements % n_chunks == 0); output layout and numerics are exactly those of
 *    `BaguaTensorPy.compress("MinMaxUInt8", n_chunks, -1)`; `out_bytes` must be at least
 *    bagua_no_alloc_compressed_size(num_elements, n_chunks).
 *  - `in`, `out` are device pointers on the CURRENT device (`in` aligned to 4 bytes, else
 *    BAGUA_NO_ALLOC_ERR_INVALID); `stream` is a stream of that device.  The work is
 *    enqueued; nothing is synchronised.
 *  - Limit: n_chunks * blocks_per_chunk partial results must fit the scratch, i.e. at
 *    most BAGUA_NO_ALLOC_MAX_PARTIALS (8192) — in practice n_chunks <= 8192.  Larger
 *    requests are refused with BAGUA_NO_ALLOC_ERR_TOO_LARGE and nothing is launched.
 *  - The call makes no cudaMalloc / cudaFree and uses no allocating library routine.
 *  - The first call on each device looks up the device address of the scratch array
 *    (cudaGetSymbolAddress) — make that first call before any stream capture begins.
 *  - All calls on one device share the one scratch array: two calls whose kernels can
 *    overlap on the GPU (different streams without an ordering between them) race on it.
 *    Calls on one stream are safe back to back.  Nothing in the scratch needs to start
 *    at zero: every slot a call reads was written earlier by the same call.
 *
 * Return value: 0 on success, a negative BAGUA_NO_ALLOC_ERR_* code otherwise;
 * bagua_no_alloc_last_error() gives the text for the calling thread.
 */
#ifndef BAGUA_NO_ALLOC_H_
#define BAGUA_NO_ALLOC_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BAGUA_NO_ALLOC_API __attribute__((visibility("default")))

#define BAGUA_NO_ALLOC_MAX_PARTIALS 8192
#define BAGUA_NO_ALLOC_SCRATCH_BYTES (BAGUA_NO_ALLOC_MAX_PARTIALS * 8)

#define BAGUA_NO_ALLOC_ERR_INVALID (-1)   /* null pointer, bad sizes, output too small */
#define BAGUA_NO_ALLOC_ERR_TOO_LARGE (-2) /* needs more scratch than the fixed array holds */
#define BAGUA_NO_ALLOC_ERR_CUDA (-3)      /* a CUDA call failed (text in last_error) */

/* `stream` is a cudaStream_t passed as an opaque pointer (NULL = default stream). */
BAGUA_NO_ALLOC_API int bagua_no_alloc_compress_minmax_u8_f32(const float* in, int64_t num_elements, int n_chunks,
                                                             uint8_t* out, size_t out_bytes, void* stream);
BAGUA_NO_ALLOC_API size_t bagua_no_alloc_compressed_size(int64_t num_elements, int n_chunks);
BAGUA_NO_ALLOC_API const char* bagua_no_alloc_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* BAGUA_NO_ALLOC_H_ */
