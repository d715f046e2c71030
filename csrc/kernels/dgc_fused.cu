// Fused Deep-Gradient-Compression exchange for sm_100a: momentum correction, exact top-k threshold
// by radix select, compaction of (index, value) pairs with momentum-factor masking, the sparse
// all-gather over NVLink peer memory and the scatter-accumulate into the dense bucket — one
// cooperative launch per bucket, no NCCL collective.
//
// What it replaces in the reference: DGCCompressor::compress (nangila-core/src/dgc.rs:104-149:
// residual accumulation, top-k by a full sort of |v|, zeroing of the sent entries), decompress
// (:151-174: scatter into zeros) and the all-gather + mean the DDP hook would put around them
// (python/nangila/ddp.py:299-339). Momentum correction and momentum-factor masking are the parts of
// the DGC paper the reference leaves out (dgc.rs:36-38); `momentum = 0` gives the reference's plain
// accumulation.
//
// Phases (grid-wide barriers between them; all CTAs are co-resident because the launch is
// cooperative):
//   0  clear the scratch histograms / cursor
//   1  u = m u + g ; v = v + u ; histogram of bits [30:20] of |v|
//   2  histogram of bits [19:9] among elements whose top bits equal the selected bin
//   3  histogram of bits [8:0]  among elements matching both        -> threshold bit pattern tau
//   4  compaction: every element with |v| >= tau is appended to the local send list (bounded by the
//      list capacity), u and v are zeroed there; the dense bucket is zeroed
//   5  the list is copied into every rank's receive slot for this rank, then a flag is released
//   6  wait (bounded) for every rank's list, add value / W into the bucket, list by list in rank order
// The selection is exact: tau is the k-th largest |v|. Elements equal to tau are all selected, so
// with ties the list can be longer than k (it is cut at the capacity; what is cut stays in v).
#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "nangila_kernels.h"
#include "quant.cuh"
#include "radix_select.cuh"
#include "signal.cuh"

namespace cg = cooperative_groups;

namespace nangila {
namespace {

using namespace comm;
using namespace rsel;

constexpr int kThreads = 256;

// scratch layout (uint32 words)
constexpr int kHist0 = 0, kHist1 = kHist0 + kBins0, kHist2 = kHist1 + kBins1;
constexpr int kCursor = kHist2 + kBins2;  // number of selected entries
constexpr int kScratchWords = kCursor + 8;

template <typename T>
__device__ __forceinline__ float ldf(const T* p, int64_t i) { return dev::Vec16<T>::to_float(p[i]); }


template <typename T>
__global__ void __launch_bounds__(kThreads, 2) dgc_fused_kernel(const __grid_constant__ NangilaDgcParams p) {
  cg::grid_group grid = cg::this_grid();
  const int vr = blockIdx.y;
  const int me = p.rank0 + vr;
  const int W = p.world;
  const int64_t n = p.n;
  T* __restrict__ grad = static_cast<T*>(p.grad[vr]);
  float* __restrict__ u = p.u[vr];
  float* __restrict__ v = p.v[vr];
  uint32_t* scratch = p.scratch[vr];
  uint32_t* status = p.status[vr];
  uint8_t* myreg = p.region[me];
  const uint32_t cap = p.capacity;
  const uint64_t slot_bytes = 16 + uint64_t(cap) * 8;
  // Two sets of receive slots, used alternately by epoch parity: a rank that runs one launch ahead
  // writes the other set while a slower peer may still be scattering from this one; it cannot get
  // two launches ahead because its wait in phase 6 needs the peer's flag of the launch in between.
  const uint64_t recv_base = p.recv_off + uint64_t(p.epoch & 1u) * uint64_t(W) * slot_bytes;
  // local send list lives in this rank's own receive slot for itself
  uint8_t* myslot = myreg + recv_base + uint64_t(me) * slot_bytes;
  uint32_t* my_idx = reinterpret_cast<uint32_t*>(myslot + 16);
  float* my_val = reinterpret_cast<float*>(myslot + 16 + uint64_t(cap) * 4);

  __shared__ uint32_t sh_hist[kBins0];
  __shared__ uint32_t sh_sel[2];
  const int64_t tid0 = int64_t(blockIdx.x) * kThreads + threadIdx.x;
  const int64_t stride = int64_t(gridDim.x) * kThreads;

  // ---- phase 0 ----
  for (int i = int(tid0); i < kScratchWords; i += int(stride)) scratch[i] = 0u;
  grid.sync();

  // ---- phase 1: momentum correction + histogram of bits [30:20] ----
  for (int i = threadIdx.x; i < kBins0; i += kThreads) sh_hist[i] = 0u;
  __syncthreads();
  for (int64_t i = tid0; i < n; i += stride) {
    float g = dev::sanitize(ldf(grad, i));
    float un = __fmaf_rn(p.momentum, u[i], g);
    float vn = v[i] + un;
    u[i] = un;
    v[i] = vn;
    atomicAdd(&sh_hist[(__float_as_uint(vn) & 0x7fffffffu) >> 20], 1u);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < kBins0; i += kThreads)
    if (sh_hist[i]) atomicAdd(&scratch[kHist0 + i], sh_hist[i]);
  grid.sync();
  uint32_t want = p.k, bin0, bin1, bin2;
  select_bin(scratch + kHist0, kBins0, want, bin0, sh_sel);

  // ---- phase 2: bits [19:9] ----
  for (int i = threadIdx.x; i < kBins1; i += kThreads) sh_hist[i] = 0u;
  __syncthreads();
  for (int64_t i = tid0; i < n; i += stride) {
    uint32_t b = __float_as_uint(v[i]) & 0x7fffffffu;
    if ((b >> 20) == bin0) atomicAdd(&sh_hist[(b >> 9) & 0x7ffu], 1u);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < kBins1; i += kThreads)
    if (sh_hist[i]) atomicAdd(&scratch[kHist1 + i], sh_hist[i]);
  grid.sync();
  select_bin(scratch + kHist1, kBins1, want, bin1, sh_sel);

  // ---- phase 3: bits [8:0] ----
  for (int i = threadIdx.x; i < kBins2; i += kThreads) sh_hist[i] = 0u;
  __syncthreads();
  const uint32_t prefix = (bin0 << 11) | bin1;
  for (int64_t i = tid0; i < n; i += stride) {
    uint32_t b = __float_as_uint(v[i]) & 0x7fffffffu;
    if ((b >> 9) == prefix) atomicAdd(&sh_hist[b & 0x1ffu], 1u);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < kBins2; i += kThreads)
    if (sh_hist[i]) atomicAdd(&scratch[kHist2 + i], sh_hist[i]);
  grid.sync();
  select_bin(scratch + kHist2, kBins2, want, bin2, sh_sel);
  const uint32_t tau = (prefix << 9) | bin2;  // bit pattern of the k-th largest |v|

  // ---- phase 4: compaction + masking + clear the dense bucket ----
  for (int64_t i0 = int64_t(blockIdx.x) * kThreads; i0 < n; i0 += stride) {
    const int64_t i = i0 + threadIdx.x;
    bool sel = false;
    float val = 0.0f;
    if (i < n) {
      val = v[i];
      uint32_t b = __float_as_uint(val) & 0x7fffffffu;
      sel = b >= tau && (p.k > 0) && b != 0u;
      grad[i] = dev::Vec16<T>::from_float(0.0f);
    }
    // warp-aggregated append
    uint32_t mask = __ballot_sync(0xffffffffu, sel);
    if (mask) {
      int lane = threadIdx.x & 31;
      uint32_t base = 0;
      if (lane == __ffs(mask) - 1) base = atomicAdd(&scratch[kCursor], uint32_t(__popc(mask)));
      base = __shfl_sync(0xffffffffu, base, __ffs(mask) - 1);
      if (sel) {
        uint32_t pos = base + uint32_t(__popc(mask & ((1u << lane) - 1u)));
        if (pos < cap) {
          my_idx[pos] = uint32_t(i);
          my_val[pos] = val;
          v[i] = 0.0f;
          u[i] = 0.0f;
        }
      }
    }
  }
  grid.sync();
  const uint32_t count = min(scratch[kCursor], cap);
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    *reinterpret_cast<uint32_t*>(myslot) = count;
    p.out_count[vr][0] = count;
    p.out_count[vr][1] = tau;
  }

  // ---- phase 5: copy the list into every other rank's slot for this rank, release flags ----
  for (int d = 1; d < W; ++d) {
    const int r = (me + d) % W;
    uint8_t* dst = p.region[r] + recv_base + uint64_t(me) * slot_bytes;
    uint32_t* d_idx = reinterpret_cast<uint32_t*>(dst + 16);
    float* d_val = reinterpret_cast<float*>(dst + 16 + uint64_t(cap) * 4);
    for (int64_t j = tid0; j < count; j += stride) {
      d_idx[j] = my_idx[j];
      d_val[j] = my_val[j];
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) *reinterpret_cast<uint32_t*>(dst) = count;
  }
  __threadfence_system();
  grid.sync();
  if (blockIdx.x == 0 && threadIdx.x < W) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint32_t*>(p.region[threadIdx.x] + p.flag_off) + me, p.epoch);
  }

  // ---- phase 6: wait for every rank's list and accumulate it ----
  // The lists are added in rank order with a grid barrier after each, so every rank performs the same
  // floating-point additions in the same order and all replicas end up with identical bits. Indices
  // inside one list are unique, so no atomics are needed. A CTA whose wait fails keeps taking part in
  // the barriers (skipping the work) so that nobody is left waiting for it.
  const float inv_w = 1.0f / float(W);
  bool alive = true;
  for (int r = 0; r < W; ++r) {
    bool ok = true;
    if (alive && threadIdx.x == 0)
      ok = wait_flag(reinterpret_cast<const uint32_t*>(myreg + p.flag_off) + r, p.epoch, p.timeout_ns, status,
                     kTimeoutPhase2, uint32_t(me), uint32_t(r), 6u, 0u);
    alive = __syncthreads_and(ok ? 1 : 0) && alive;
    if (alive) {
      const uint8_t* src = myreg + recv_base + uint64_t(r) * slot_bytes;
      const uint32_t cnt = min(*reinterpret_cast<const uint32_t*>(src), cap);
      const uint32_t* s_idx = reinterpret_cast<const uint32_t*>(src + 16);
      const float* s_val = reinterpret_cast<const float*>(src + 16 + uint64_t(cap) * 4);
      for (int64_t j = tid0; j < cnt; j += stride) {
        const uint32_t idx = s_idx[j];
        if (idx < n) grad[idx] = dev::Vec16<T>::from_float(__fmaf_rn(s_val[j], inv_w, ldf(grad, idx)));
      }
    }
    grid.sync();
  }
}

}  // namespace
}  // namespace nangila

extern "C" uint64_t nangila_dgc_region_bytes(uint32_t capacity, int32_t world, uint64_t* recv_off, uint64_t* flag_off) {
  auto align = [](uint64_t x) { return (x + 255) & ~uint64_t(255); };
  uint64_t off = 0;
  if (recv_off) *recv_off = off;
  off = align(off + 2 * uint64_t(world) * (16 + uint64_t(capacity) * 8));
  if (flag_off) *flag_off = off;
  off = align(off + uint64_t(world) * 4);
  return off;
}

extern "C" uint32_t nangila_dgc_scratch_words(void) { return nangila::kScratchWords; }

extern "C" int nangila_dgc_launch(const NangilaDgcParams* p, cudaStream_t stream) {
  using namespace nangila;
  if (p == nullptr || p->n <= 0 || p->n > 0x7fffffffll || p->world < 1 || p->world > NANGILA_MAX_RANKS ||
      p->nvr < 1 || p->nvr > NANGILA_MAX_VRANKS || p->rank0 < 0 || p->rank0 + p->nvr > p->world ||
      (p->nvr > 1 && p->nvr != p->world) || p->epoch == 0 || p->grid_x < 1 || p->capacity == 0 ||
      p->capacity % 4 != 0 || p->k > p->capacity || !(p->momentum >= 0.0f && p->momentum < 1.0f))
    return int(cudaErrorInvalidValue);
  const void* fn;
  switch (p->grad_dtype) {
    case NANGILA_F32: fn = reinterpret_cast<const void*>(&dgc_fused_kernel<float>); break;
    case NANGILA_BF16: fn = reinterpret_cast<const void*>(&dgc_fused_kernel<__nv_bfloat16>); break;
    case NANGILA_F16: fn = reinterpret_cast<const void*>(&dgc_fused_kernel<__half>); break;
    default: return int(cudaErrorInvalidValue);
  }
  dim3 grid(unsigned(p->grid_x), unsigned(p->nvr)), block(kThreads);
  void* args[] = {const_cast<NangilaDgcParams*>(p)};
  return int(cudaLaunchCooperativeKernel(fn, grid, block, args, 0, stream));
}
