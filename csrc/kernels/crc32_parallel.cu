// Parallel IEEE CRC32 (polynomial 0xEDB88320, initial value and final XOR 0xFFFFFFFF) of a device
// buffer. Step 1: every thread computes the standard CRC of its own 512-byte chunk with a table in
// shared memory. Step 2: one block combines neighbouring chunks pairwise, doubling the span each
// round, using crc(A||B) = crc(A) * x^(8 len B) mod P  xor  crc(B) in GF(2)[x].
//
// Replaces compute_crc32_kernel (nangila-cuda/src/kernels/crc32.cu:56-72), which walks the whole
// payload with a single thread, and matches the host table CRC (nangila-core/src/packet.rs:241-274).
#include <cuda_runtime.h>

#include <atomic>

#include "nangila_kernels.h"
#include "nangila_noalloc.h"

namespace nangila {
namespace {

constexpr uint32_t kPoly = 0xEDB88320u;
constexpr int kChunk = 512;

// a * b mod P with the reflected bit order (bit 31 is x^0).
__host__ __device__ inline uint32_t mulmod(uint32_t a, uint32_t b) {
  uint32_t m = 1u << 31, p = 0;
  for (;;) {
    if (a & m) {
      p ^= b;
      if ((a & (m - 1)) == 0) break;
    }
    m >>= 1;
    b = (b & 1u) ? (b >> 1) ^ kPoly : b >> 1;
  }
  return p;
}
// x^(8 * nbytes) mod P
__host__ __device__ inline uint32_t x_pow_bytes(uint64_t nbytes) {
  uint32_t result = 1u << 31;  // x^0
  uint32_t sq = 1u << 30;      // x^1
  sq = mulmod(sq, sq);         // x^2
  sq = mulmod(sq, sq);         // x^4
  sq = mulmod(sq, sq);         // x^8 = one byte
  while (nbytes) {
    if (nbytes & 1u) result = mulmod(sq, result);
    sq = mulmod(sq, sq);
    nbytes >>= 1;
  }
  return result;
}

__global__ void __launch_bounds__(128) crc_chunks_kernel(const uint8_t* __restrict__ data, int64_t nbytes,
                                                        uint32_t* __restrict__ crcs, int64_t nchunks) {
  __shared__ uint32_t table[256];
  for (int i = threadIdx.x; i < 256; i += blockDim.x) {
    uint32_t c = uint32_t(i);
#pragma unroll
    for (int k = 0; k < 8; ++k) c = (c & 1u) ? (kPoly ^ (c >> 1)) : (c >> 1);
    table[i] = c;
  }
  __syncthreads();
  const int64_t chunk = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (chunk >= nchunks) return;
  const int64_t begin = chunk * kChunk;
  const int64_t end = begin + kChunk < nbytes ? begin + kChunk : nbytes;
  uint32_t c = 0xFFFFFFFFu;
  int64_t i = begin;
  if ((reinterpret_cast<uintptr_t>(data) & 3u) == 0) {
    for (; i + 4 <= end; i += 4) {
      uint32_t w = *reinterpret_cast<const uint32_t*>(data + i);
#pragma unroll
      for (int b = 0; b < 4; ++b) c = table[(c ^ (w >> (8 * b))) & 0xffu] ^ (c >> 8);
    }
  }
  for (; i < end; ++i) c = table[(c ^ data[i]) & 0xffu] ^ (c >> 8);
  crcs[chunk] = c ^ 0xFFFFFFFFu;
}

__global__ void __launch_bounds__(1024) crc_combine_kernel(uint32_t* crcs, int64_t nchunks, int64_t nbytes,
                                                          uint32_t* out) {
  // lengths: every chunk holds kChunk bytes except the last one
  for (int64_t span = 1; span < nchunks; span <<= 1) {
    for (int64_t i = int64_t(threadIdx.x) * 2 * span; i + span < nchunks; i += int64_t(blockDim.x) * 2 * span) {
      const int64_t rbegin = (i + span) * kChunk;
      int64_t rend = (i + 2 * span) * kChunk;
      if (rend > nbytes) rend = nbytes;
      crcs[i] = mulmod(x_pow_bytes(uint64_t(rend - rbegin)), crcs[i]) ^ crcs[i + span];
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) *out = nchunks > 0 ? crcs[0] : 0u;
}

}  // namespace
}  // namespace nangila

extern "C" int64_t nangila_crc32_scratch_words(int64_t nbytes) { return (nbytes + nangila::kChunk - 1) / nangila::kChunk + 1; }

// out: one uint32 on the device. scratch: nangila_crc32_scratch_words(nbytes) uint32 words.
extern "C" int nangila_crc32(const void* data, int64_t nbytes, uint32_t* scratch, uint32_t* out, cudaStream_t stream) {
  using namespace nangila;
  if (out == nullptr || nbytes < 0 || (nbytes > 0 && (data == nullptr || scratch == nullptr)))
    return int(cudaErrorInvalidValue);
  if (nbytes == 0) return int(cudaMemsetAsync(out, 0, 4, stream));
  const int64_t nchunks = (nbytes + kChunk - 1) / kChunk;
  crc_chunks_kernel<<<unsigned((nchunks + 127) / 128), 128, 0, stream>>>(static_cast<const uint8_t*>(data), nbytes,
                                                                       scratch, nchunks);
  crc_combine_kernel<<<1, 1024, 0, stream>>>(scratch, nchunks, nbytes, out);
  return int(cudaGetLastError());
}

// ---------------------------------------------------------------------------------------------------
// Allocation-free entry point (declared in nangila_noalloc.h; the reference has nothing like it).
//
// The chunk table that nangila_crc32() takes from its caller lives here in a fixed array inside the
// library image, so a caller that has no way to obtain device memory can still checksum a buffer: it
// hands over only the data pointer and the 4-byte result location.
namespace nangila {
namespace {

constexpr int64_t kNoAllocMaxBytes = int64_t(64) << 20;                    // largest buffer accepted
constexpr int64_t kNoAllocWords = kNoAllocMaxBytes / kChunk + 1;           // 131073 words = 512 KiB + 4
static __device__ __align__(256) uint32_t g_crc_scratch[kNoAllocWords];

constexpr int kMaxDevices = 64;
// device address of g_crc_scratch, per device ordinal; host threads that race on the first call store the same value
std::atomic<uint32_t*> g_scratch_addr[kMaxDevices];

}  // namespace
}  // namespace nangila

extern "C" int64_t nangila_crc32_noalloc_max_bytes(void) { return nangila::kNoAllocMaxBytes; }

extern "C" int nangila_crc32_noalloc(const void* data, int64_t nbytes, uint32_t* out, cudaStream_t stream) {
  using namespace nangila;
  if (out == nullptr || nbytes < 0 || (nbytes > 0 && data == nullptr)) return int(cudaErrorInvalidValue);
  if (nbytes > kNoAllocMaxBytes) return int(cudaErrorInvalidValue);  // beyond the built-in table: refuse
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return int(e);
  if (dev < 0 || dev >= kMaxDevices) return int(cudaErrorInvalidDevice);
  if (g_scratch_addr[dev].load(std::memory_order_acquire) == nullptr) {
    // In host code `g_crc_scratch` is only a handle for the symbol, not an address a kernel could
    // use; the address inside the current device's copy of the image has to be asked for.
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_crc_scratch);
    if (e != cudaSuccess) return int(e);
    g_scratch_addr[dev].store(static_cast<uint32_t*>(p), std::memory_order_release);
  }
  uint32_t* scratch = g_scratch_addr[dev].load(std::memory_order_acquire);
  if (nbytes == 0) {
    // nothing to hash: the result is 0; written by a kernel so that no memset node is needed either
    crc_combine_kernel<<<1, 32, 0, stream>>>(scratch, 0, 0, out);
    return int(cudaGetLastError());
  }
  const int64_t nchunks = (nbytes + kChunk - 1) / kChunk;
  // Every table entry the second kernel reads is written by the first one in this same call, so
  // nothing left over from an earlier call can leak into the result and nothing needs clearing.
  crc_chunks_kernel<<<unsigned((nchunks + 127) / 128), 128, 0, stream>>>(static_cast<const uint8_t*>(data), nbytes,
                                                                       scratch, nchunks);
  crc_combine_kernel<<<1, 1024, 0, stream>>>(scratch, nchunks, nbytes, out);
  return int(cudaGetLastError());
}
