// Cross-GPU signalling primitives used inside the fused kernels: system-scope release stores and
// acquire loads on flag words that live in peer-mapped (symmetric) memory, and a wait that always
// ends — when the flag does not arrive within the time limit the waiter records what it was waiting
// for in a status block and returns false, so the kernel can drain and exit and the host can read
// the status. Nothing here traps, asserts or spins without a limit.
//
// Flags carry epochs (one per launch of a bucket's kernel, strictly increasing), so a value left
// over from an earlier launch can never satisfy a later wait and flags never need clearing.
#pragma once
#include <cstdint>

namespace nangila {
namespace comm {

// Status block layout (uint32 words) written by the first waiter that gives up.
enum StatusWord : int {
  kStatusCode = 0,    // 0 = ok, else one of StatusCode
  kStatusRank = 1,    // rank that gave up
  kStatusPeer = 2,    // rank it was waiting for (or 0xffffffff)
  kStatusEpoch = 3,   // epoch it expected
  kStatusSeen = 4,    // last flag value it saw
  kStatusPhase = 5,   // kernel phase (1, 2, 3)
  kStatusChunk = 6,   // chunk / task index
  kStatusBarrier = 7, // counter of the in-kernel grid barrier (kernels launched without a cooperative launch)
  kStatusWords = 8,
};
enum StatusCode : uint32_t {
  kOk = 0,
  kTimeoutPhase2 = 2,   // owner did not get every rank's contribution
  kTimeoutPhase3 = 3,   // reduced chunk did not arrive from its owner
  kTimeoutGrid = 4,     // grid-wide barrier inside one GPU did not complete
  kTimeoutBulk = 6,     // a bulk copy into shared memory did not complete
  kBadArgument = 5,
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_gpu_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// True when `seen` is at or past `epoch` (wrap-around safe for 32-bit epochs).
__device__ __forceinline__ bool epoch_reached(uint32_t seen, uint32_t epoch) {
  return int32_t(seen - epoch) >= 0;
}

__device__ __forceinline__ void report_failure(uint32_t* status, uint32_t code, uint32_t rank, uint32_t peer,
                                               uint32_t epoch, uint32_t seen, uint32_t phase, uint32_t chunk) {
  if (atomicCAS(&status[kStatusCode], 0u, code) == 0u) {
    status[kStatusRank] = rank;
    status[kStatusPeer] = peer;
    status[kStatusEpoch] = epoch;
    status[kStatusSeen] = seen;
    status[kStatusPhase] = phase;
    status[kStatusChunk] = chunk;
    __threadfence_system();
  }
}

// Wait until *flag reaches `epoch`. Gives up after `timeout_ns` or as soon as another waiter of this
// kernel has already reported a failure (status[0] != 0). Returns true on success.
__device__ __forceinline__ bool wait_flag(const uint32_t* flag, uint32_t epoch, uint64_t timeout_ns,
                                          uint32_t* status, uint32_t code, uint32_t rank, uint32_t peer,
                                          uint32_t phase, uint32_t chunk) {
  uint32_t seen = ld_acquire_sys(flag);
  if (epoch_reached(seen, epoch)) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  for (;;) {
    __nanosleep(spins < 64 ? 32 : 256);
    seen = ld_acquire_sys(flag);
    if (epoch_reached(seen, epoch)) return true;
    if ((++spins & 15u) == 0u) {
      if (*reinterpret_cast<volatile uint32_t*>(&status[kStatusCode]) != 0u) return false;
      if (globaltimer_ns() - t0 > timeout_ns) {
        report_failure(status, code, rank, peer, epoch, seen, phase, chunk);
        return false;
      }
    }
  }
}

// Barrier among all CTAs of one launch WITHOUT a cooperative launch, so the kernel can start while other
// work still holds part of the GPU and share it afterwards. It needs every CTA of the launch to become
// resident at some point, which holds when the grid is no larger than what the device can hold at once
// (the launchers clamp to that) and the other kernels on the device terminate on their own. `word` is a
// counter in global memory that is zero when the kernel starts and only grows: barrier number k is
// complete when it reaches k * nblocks. Every thread of every CTA must call sync() the same number of
// times. Returns false, on every CTA, once any waiter of this kernel has given up (time limit or a failure
// recorded elsewhere in the status block); the caller then returns.
struct GridBarrier {
  uint32_t* word;
  uint32_t nblocks;
  uint32_t k;
  __device__ __forceinline__ GridBarrier(uint32_t* w, uint32_t n) : word(w), nblocks(n), k(0u) {}
  __device__ __forceinline__ bool sync(uint64_t timeout_ns, uint32_t* status, uint32_t rank, uint32_t epoch) {
    k += 1u;
    __syncthreads();
    int ok = 1;
    if (threadIdx.x == 0) {
      __threadfence();
      red_release_gpu_add(word, 1u);
      const uint32_t target = k * nblocks;
      uint64_t t0 = 0;
      uint32_t spins = 0, seen;
      while (int32_t((seen = ld_acquire_gpu(word)) - target) < 0) {
        __nanosleep(spins < 32 ? 20 : 200);
        if ((++spins & 31u) == 0u) {
          if (*reinterpret_cast<volatile uint32_t*>(&status[kStatusCode]) != 0u) {
            ok = 0;
            break;
          }
          const uint64_t now = globaltimer_ns();
          if (t0 == 0) t0 = now;
          if (now - t0 > timeout_ns) {
            report_failure(status, kTimeoutGrid, rank, 0xffffffffu, epoch, seen, k, 0u);
            ok = 0;
            break;
          }
        }
      }
    }
    return __syncthreads_and(ok) != 0;
  }
};

}  // namespace comm
}  // namespace nangila
