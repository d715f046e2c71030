// Pieces of the three-pass radix select over the bit pattern of |x| (bits [30:20], [19:9], [8:0])
// shared by the DGC kernel and the absmax / percentile kernel.
#pragma once
#include <cstdint>

namespace nangila {
namespace rsel {

constexpr int kBins0 = 2048, kBins1 = 2048, kBins2 = 512;

// Scanning bins from the top, find the bin that holds the `want`-th largest element (1-based) and
// reduce `want` to the rank inside that bin. The first warp of the CTA scans; the result is broadcast
// through `sh` (2 words of shared memory). `hist` must be complete (grid barrier before the call).
__device__ inline void select_bin(const uint32_t* hist, int nbins, uint32_t& want, uint32_t& bin, uint32_t* sh) {
  if (threadIdx.x < 32) {
    uint32_t remaining = want;
    uint32_t found = 0;
    bool done = false;
    for (int base = nbins - 32; base >= 0 && !done; base -= 32) {
      uint32_t c = hist[base + 31 - threadIdx.x];  // lane 0 = highest bin of this group
      uint32_t incl = c;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        uint32_t t = __shfl_up_sync(0xffffffffu, incl, off);
        if (threadIdx.x >= off) incl += t;
      }
      uint32_t total = __shfl_sync(0xffffffffu, incl, 31);
      if (total >= remaining) {
        uint32_t hit = __ballot_sync(0xffffffffu, incl >= remaining);
        int lane = __ffs(hit) - 1;
        uint32_t before = __shfl_sync(0xffffffffu, incl - c, lane);
        found = uint32_t(base + 31 - lane);
        remaining -= before;
        done = true;
      } else {
        remaining -= total;
      }
    }
    if (threadIdx.x == 0) {
      sh[0] = found;
      sh[1] = remaining;
    }
  }
  __syncthreads();
  bin = sh[0];
  want = sh[1];
  __syncthreads();
}

}  // namespace rsel
}  // namespace nangila
