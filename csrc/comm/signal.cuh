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

}  // namespace comm
}  // namespace nangila
