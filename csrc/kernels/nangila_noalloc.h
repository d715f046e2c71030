/* Entry points of libnangila_kernels.so that never allocate.
 *
 * Who this is for: code that wants a checksum of a device buffer but is not in a position to get
 * scratch memory for it — a plugin running inside somebody else's process under a "no allocations
 * after start-up" rule, a callback on a thread where cudaMalloc would deadlock with the caller's own
 * allocator lock, a library that was handed a fixed memory budget it has already spent. The ordinary
 * nangila_crc32() needs a caller-provided chunk table; here the table is a fixed array inside the
 * library image.
 *
 * This header has no counterpart in the reference implementation.
 */
#pragma once
#include <cuda_runtime_api.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Largest buffer nangila_crc32_noalloc() accepts: 64 MiB. The built-in table is sized for it
 * (131073 words, about 512 KiB) and every GPU that loads the library carries that table until the
 * process exits, whether the function is ever called or not. */
int64_t nangila_crc32_noalloc_max_bytes(void);

/* IEEE CRC32 (the zlib one) of `nbytes` bytes at device address `data`, written to the device word
 * `*out`; queued on `stream`, returns a cudaError_t value (0 = queued). Same result as nangila_crc32().
 *
 * - Calls no cudaMalloc / cudaFree / allocating library routine, and does not synchronize.
 * - nbytes > nangila_crc32_noalloc_max_bytes() is refused with cudaErrorInvalidValue (nothing queued).
 * - The first call on each device looks up the table's address on that device (once; the device
 *   must be current, as for any launch). Make that first call outside any stream capture.
 * - All calls on a device share the one table. Calls whose kernels may overlap on the GPU (different
 *   streams without an ordering between them) race on it and can return wrong checksums; calls on
 *   one stream, or otherwise ordered, are fine. The table keeps whatever the last call left in it;
 *   each call overwrites every entry it later reads, so that content never matters. */
int nangila_crc32_noalloc(const void* data, int64_t nbytes, uint32_t* out, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
