// 64-bit hash of a device buffer for cross-rank agreement checks of the predictor state, without
// copying the state to the host: h = sum over 32-bit words w_i of mix64(seed, i, w_i) (mod 2^64).
// The sum is commutative, so any launch geometry gives the same value and ranks holding the same
// bytes get the same hash.
//
// Role in the reference: Predictor::state_hash (nangila-core/src/predictor.rs:455-477) hashed on the
// host and compared across ranks every 100 steps (python/nangila/ddp.py:385-412). The host core keeps
// the reference's SipHash; this device hash is what the CUDA path compares.
#include <cuda_runtime.h>

#include "nangila_kernels.h"

namespace nangila {
namespace {

__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
  z ^= z >> 30;
  z *= 0xBF58476D1CE4E5B9ull;
  z ^= z >> 27;
  z *= 0x94D049BB133111EBull;
  z ^= z >> 31;
  return z;
}

__global__ void __launch_bounds__(256) state_hash_kernel(const uint32_t* __restrict__ words, int64_t nwords,
                                                        const uint8_t* __restrict__ tail, int ntail,
                                                        unsigned long long seed, unsigned long long* out) {
  unsigned long long acc = 0;
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < nwords; i += stride)
    acc += mix64(seed + (unsigned long long)(i)*0x9E3779B97F4A7C15ull + words[i]);
  if (blockIdx.x == 0 && threadIdx.x == 0 && ntail > 0) {
    uint32_t w = 0;
    for (int b = 0; b < ntail; ++b) w |= uint32_t(tail[b]) << (8 * b);
    acc += mix64(seed + (unsigned long long)(nwords)*0x9E3779B97F4A7C15ull + w);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  __shared__ unsigned long long red[8];
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned long long a = 0;
    for (int i = 0; i < 8; ++i) a += red[i];
    atomicAdd(out, a);
  }
}

}  // namespace
}  // namespace nangila

// *out must be zero (or hold the hash of preceding buffers, to chain several buffers into one value).
extern "C" int nangila_state_hash(const void* data, int64_t nbytes, uint64_t seed, uint64_t* out, cudaStream_t stream) {
  if (data == nullptr || out == nullptr || nbytes < 0 || (reinterpret_cast<uintptr_t>(data) & 3u) != 0)
    return int(cudaErrorInvalidValue);
  if (nbytes == 0) return 0;
  const int64_t nwords = nbytes / 4;
  const int ntail = int(nbytes % 4);
  int64_t blocks = (nwords + 255) / 256;
  blocks = blocks < 1 ? 1 : (blocks > 148 * 8 ? 148 * 8 : blocks);
  nangila::state_hash_kernel<<<int(blocks), 256, 0, stream>>>(
      static_cast<const uint32_t*>(data), nwords, static_cast<const uint8_t*>(data) + nwords * 4, ntail, seed,
      reinterpret_cast<unsigned long long*>(out));
  return int(cudaGetLastError());
}
