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
// Phases (grid-wide barriers between them: hardware barriers of a cooperative launch in the single-GPU
// loopback world, counter barriers with a time limit otherwise, see comm/signal.cuh):
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

#include "launch_util.cuh"
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
constexpr int kCandCount = kCursor + 1;   // candidates collected in phase 1, summed over the CTAs
constexpr int kCandOverflow = kCursor + 4;  // non-zero if a CTA ran out of room for its candidates
constexpr int kScratchWords = kCursor + 8;  // the candidate list (index, bits pairs) follows

template <typename T>
__device__ __forceinline__ float ldf(const T* p, int64_t i) { return dev::Vec16<T>::to_float(p[i]); }

// Four consecutive elements (the bucket and the fp32 state are at least 16-byte aligned and the
// vector index is a multiple of 4, so 8- and 16-byte accesses are aligned).
template <typename T>
__device__ __forceinline__ void ld4(const T* p, int64_t i, float (&x)[4]) {
  if constexpr (sizeof(T) == 4) {
    const float4 a = *reinterpret_cast<const float4*>(p + i);
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
  } else {
    const uint2 a = *reinterpret_cast<const uint2*>(p + i);
    const T* h = reinterpret_cast<const T*>(&a);
#pragma unroll
    for (int k = 0; k < 4; ++k) x[k] = dev::Vec16<T>::to_float(h[k]);
  }
}
template <typename T>
__device__ __forceinline__ void st4_zero(T* p, int64_t i) {
  if constexpr (sizeof(T) == 4) *reinterpret_cast<float4*>(p + i) = make_float4(0.f, 0.f, 0.f, 0.f);
  else *reinterpret_cast<uint2*>(p + i) = make_uint2(0u, 0u);
}

// One vote per distinct bin of the warp: gradients cluster in a handful of exponent bins, and 32 lanes
// adding to the same shared-memory word would be serialised. `active` lanes hold a valid `bin`.
__device__ __forceinline__ void hist_add(uint32_t* hist, uint32_t bin, bool active) {
  const uint32_t live = __ballot_sync(0xffffffffu, active);
  if (!active) return;
  const uint32_t peers = __match_any_sync(live, bin);
  if ((threadIdx.x & 31) == __ffs(peers) - 1) atomicAdd(&hist[bin], uint32_t(__popc(peers)));
}

template <typename T>
__global__ void __launch_bounds__(kThreads, 3) dgc_fused_kernel(const __grid_constant__ NangilaDgcParams p) {
  cg::grid_group grid = cg::this_grid();
  const int vr = blockIdx.y;
  // Grid-wide barriers: the hardware one when several ranks are emulated in one (cooperative) launch; with a
  // real process group a counter barrier over the CTAs of this launch, so the kernel needs no cooperative
  // launch, can start while backward still holds part of the GPU, and runs with a capped number of CTAs.
  const bool coop = p.nvr > 1;
  GridBarrier soft(p.status[vr] + kStatusBarrier, gridDim.x);
  auto gsync = [&]() -> bool {
    if (coop) {
      grid.sync();
      return true;
    }
    return soft.sync(p.timeout_ns, p.status[vr], uint32_t(p.rank0 + vr), p.epoch);
  };
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
  __shared__ uint32_t sh_cand_cnt;  // candidates this CTA has appended to its segment of the list
  const int64_t tid0 = int64_t(blockIdx.x) * kThreads + threadIdx.x;
  const int64_t stride = int64_t(gridDim.x) * kThreads;
  // The dense passes walk the bucket in groups of 4 elements; every warp keeps all 32 lanes in the loop
  // (the loop bound is rounded up per warp) so that the warp-wide votes below are well defined.
  const int64_t n4 = n / 4;                          // whole groups
  const int64_t groups = (n + 3) / 4;                // including the ragged last one
  const int64_t groups_rounded = (groups + 31) / 32 * 32;

  // Candidates. Between two calls on the same bucket the threshold moves little, so phase 1 also
  // collects every entry with |v| >= 0.96 * (previous threshold) into a short list (unsent entries
  // pile up just below the threshold, so the band has to be narrow). If that list holds
  // at least k entries and did not overflow, the k largest entries of the bucket are all in it and the
  // three selection passes and the compaction run over the list (a few thousand entries) instead of
  // the dense state; otherwise (first call, threshold moved a lot) the dense passes run as before.
  const uint32_t tau_prev = p.out_count[vr][1];
  const uint32_t cand_cap = p.cand_capacity;
  const uint32_t cand_thr = (cand_cap > 0 && tau_prev > 0 && tau_prev < 0x7f800000u)
                                ? __float_as_uint(__uint_as_float(tau_prev) * 0.96f)
                                : 0xffffffffu;  // nothing qualifies
  const uint32_t seg_cap = cand_cap / gridDim.x;  // entries per CTA
  uint32_t* cand_idx = scratch + kScratchWords + uint64_t(blockIdx.x) * seg_cap;
  uint32_t* cand_bits = cand_idx + cand_cap;

  // ---- phase 0 ----
  for (int i = int(tid0); i < kScratchWords; i += int(stride)) scratch[i] = 0u;
  if (threadIdx.x == 0) sh_cand_cnt = 0u;
  if (!gsync()) return;

  // ---- phase 1: momentum correction + histogram of bits [30:20] ----
  for (int i = threadIdx.x; i < kBins0; i += kThreads) sh_hist[i] = 0u;
  __syncthreads();
  for (int64_t q = tid0; q < groups_rounded; q += stride) {
    float vn[4];
    int valid = 0;
    if (q < n4) {
      float g[4];
      ld4<T>(grad, q * 4, g);
      float4 uu = *reinterpret_cast<const float4*>(u + q * 4);
      float4 vv = *reinterpret_cast<const float4*>(v + q * 4);
      uu.x = __fmaf_rn(p.momentum, uu.x, dev::sanitize(g[0]));
      uu.y = __fmaf_rn(p.momentum, uu.y, dev::sanitize(g[1]));
      uu.z = __fmaf_rn(p.momentum, uu.z, dev::sanitize(g[2]));
      uu.w = __fmaf_rn(p.momentum, uu.w, dev::sanitize(g[3]));
      vv.x += uu.x; vv.y += uu.y; vv.z += uu.z; vv.w += uu.w;
      *reinterpret_cast<float4*>(u + q * 4) = uu;
      *reinterpret_cast<float4*>(v + q * 4) = vv;
      st4_zero<T>(grad, q * 4);  // the dense result starts from zero; phase 6 scatters into it
      vn[0] = vv.x; vn[1] = vv.y; vn[2] = vv.z; vn[3] = vv.w;
      valid = 4;
    } else if (q < groups) {
      for (int k = 0; k < 4; ++k) {
        const int64_t i = q * 4 + k;
        vn[k] = 0.0f;
        if (i < n) {
          const float un = __fmaf_rn(p.momentum, u[i], dev::sanitize(ldf(grad, i)));
          vn[k] = v[i] + un;
          u[i] = un;
          v[i] = vn[k];
          grad[i] = dev::Vec16<T>::from_float(0.0f);
          valid = k + 1;
        }
      }
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const uint32_t b = __float_as_uint(vn[k]) & 0x7fffffffu;
      hist_add(sh_hist, b >> 20, k < valid);
      const bool cand = k < valid && b >= cand_thr;
      const uint32_t mask = __ballot_sync(0xffffffffu, cand);
      if (mask) {
        const int lane = threadIdx.x & 31;
        uint32_t base = 0;
        if (lane == __ffs(mask) - 1) base = atomicAdd(&sh_cand_cnt, uint32_t(__popc(mask)));
        base = __shfl_sync(0xffffffffu, base, __ffs(mask) - 1);
        if (cand) {
          const uint32_t pos = base + uint32_t(__popc(mask & ((1u << lane) - 1u)));
          if (pos < seg_cap) {
            cand_idx[pos] = uint32_t(q * 4 + k);
            cand_bits[pos] = b;
          }
        }
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < kBins0; i += kThreads)
    if (sh_hist[i]) atomicAdd(&scratch[kHist0 + i], sh_hist[i]);
  const uint32_t my_cand = min(sh_cand_cnt, seg_cap);  // entries of this CTA's segment
  if (threadIdx.x == 0) {
    atomicAdd(&scratch[kCandCount], my_cand);
    if (sh_cand_cnt > seg_cap) atomicOr(&scratch[kCandOverflow], 1u);
  }
  if (!gsync()) return;
  uint32_t want = p.k, bin0, bin1, bin2;
  select_bin(scratch + kHist0, kBins0, want, bin0, sh_sel);

  const uint32_t ncand = scratch[kCandCount];
  const bool from_list = seg_cap > 0 && ncand >= p.k && scratch[kCandOverflow] == 0u;  // same on every CTA
  uint32_t tau;
  if (from_list) {
    // ---- phases 2-4 over the candidate list ----
    for (int i = threadIdx.x; i < kBins1; i += kThreads) sh_hist[i] = 0u;
    __syncthreads();
    const uint32_t nc_rounded = (my_cand + 31u) / 32u * 32u;  // this CTA scans its own segment
    for (uint32_t j = threadIdx.x; j < nc_rounded; j += kThreads) {
      const uint32_t b = j < my_cand ? cand_bits[j] : 0xffffffffu;
      hist_add(sh_hist, (b >> 9) & 0x7ffu, b != 0xffffffffu && (b >> 20) == bin0);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < kBins1; i += kThreads)
      if (sh_hist[i]) atomicAdd(&scratch[kHist1 + i], sh_hist[i]);
    if (!gsync()) return;
    select_bin(scratch + kHist1, kBins1, want, bin1, sh_sel);
    for (int i = threadIdx.x; i < kBins2; i += kThreads) sh_hist[i] = 0u;
    __syncthreads();
    const uint32_t prefix = (bin0 << 11) | bin1;
    for (uint32_t j = threadIdx.x; j < nc_rounded; j += kThreads) {
      const uint32_t b = j < my_cand ? cand_bits[j] : 0xffffffffu;
      hist_add(sh_hist, b & 0x1ffu, b != 0xffffffffu && (b >> 9) == prefix);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < kBins2; i += kThreads)
      if (sh_hist[i]) atomicAdd(&scratch[kHist2 + i], sh_hist[i]);
    if (!gsync()) return;
    select_bin(scratch + kHist2, kBins2, want, bin2, sh_sel);
    tau = (prefix << 9) | bin2;
    for (uint32_t j = threadIdx.x; j < nc_rounded; j += kThreads) {
      const uint32_t b = j < my_cand ? cand_bits[j] : 0xffffffffu;
      const bool sel = b != 0xffffffffu && b >= tau && (p.k > 0) && b != 0u;
      const uint32_t mask = __ballot_sync(0xffffffffu, sel);
      if (mask) {
        const int lane = threadIdx.x & 31;
        uint32_t base = 0;
        if (lane == __ffs(mask) - 1) base = atomicAdd(&scratch[kCursor], uint32_t(__popc(mask)));
        base = __shfl_sync(0xffffffffu, base, __ffs(mask) - 1);
        if (sel) {
          const uint32_t pos = base + uint32_t(__popc(mask & ((1u << lane) - 1u)));
          if (pos < cap) {
            const uint32_t i = cand_idx[j];
            my_idx[pos] = i;
            my_val[pos] = v[i];
            v[i] = 0.0f;
            u[i] = 0.0f;
          }
        }
      }
    }
  } else {
    // bit patterns of |v| for one group (0 beyond the end: never selected, never counted)
    auto load_bits = [&](int64_t q, uint32_t (&b)[4]) {
      if (q < n4) {
        const uint4 a = *reinterpret_cast<const uint4*>(v + q * 4);
        b[0] = a.x & 0x7fffffffu; b[1] = a.y & 0x7fffffffu; b[2] = a.z & 0x7fffffffu; b[3] = a.w & 0x7fffffffu;
      } else {
  #pragma unroll
        for (int k = 0; k < 4; ++k) b[k] = (q * 4 + k < n) ? (__float_as_uint(v[q * 4 + k]) & 0x7fffffffu) : 0xffffffffu;
      }
    };

    // ---- phase 2: bits [19:9] ----
    for (int i = threadIdx.x; i < kBins1; i += kThreads) sh_hist[i] = 0u;
    __syncthreads();
    for (int64_t q = tid0; q < groups_rounded; q += stride) {
      uint32_t b[4] = {0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu};
      if (q < groups) load_bits(q, b);
  #pragma unroll
      for (int k = 0; k < 4; ++k) hist_add(sh_hist, (b[k] >> 9) & 0x7ffu, b[k] != 0xffffffffu && (b[k] >> 20) == bin0);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < kBins1; i += kThreads)
      if (sh_hist[i]) atomicAdd(&scratch[kHist1 + i], sh_hist[i]);
    if (!gsync()) return;
    select_bin(scratch + kHist1, kBins1, want, bin1, sh_sel);

    // ---- phase 3: bits [8:0] ----
    for (int i = threadIdx.x; i < kBins2; i += kThreads) sh_hist[i] = 0u;
    __syncthreads();
    const uint32_t prefix = (bin0 << 11) | bin1;
    for (int64_t q = tid0; q < groups_rounded; q += stride) {
      uint32_t b[4] = {0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu};
      if (q < groups) load_bits(q, b);
  #pragma unroll
      for (int k = 0; k < 4; ++k) hist_add(sh_hist, b[k] & 0x1ffu, b[k] != 0xffffffffu && (b[k] >> 9) == prefix);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < kBins2; i += kThreads)
      if (sh_hist[i]) atomicAdd(&scratch[kHist2 + i], sh_hist[i]);
    if (!gsync()) return;
    select_bin(scratch + kHist2, kBins2, want, bin2, sh_sel);
    tau = (prefix << 9) | bin2;  // bit pattern of the k-th largest |v|

    // ---- phase 4: compaction + masking ----
    for (int64_t q = tid0; q < groups_rounded; q += stride) {
      uint32_t b[4] = {0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu};
      if (q < groups) load_bits(q, b);
      const int lane = threadIdx.x & 31;
  #pragma unroll
      for (int k = 0; k < 4; ++k) {
        const bool sel = b[k] != 0xffffffffu && b[k] >= tau && (p.k > 0) && b[k] != 0u;
        // warp-aggregated append
        const uint32_t mask = __ballot_sync(0xffffffffu, sel);
        if (mask) {
          uint32_t base = 0;
          if (lane == __ffs(mask) - 1) base = atomicAdd(&scratch[kCursor], uint32_t(__popc(mask)));
          base = __shfl_sync(0xffffffffu, base, __ffs(mask) - 1);
          if (sel) {
            const uint32_t pos = base + uint32_t(__popc(mask & ((1u << lane) - 1u)));
            if (pos < cap) {
              const int64_t i = q * 4 + k;
              my_idx[pos] = uint32_t(i);
              my_val[pos] = v[i];
              v[i] = 0.0f;
              u[i] = 0.0f;
            }
          }
        }
      }
    }
  }
  if (!gsync()) return;
  const uint32_t count = min(scratch[kCursor], cap);
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    *reinterpret_cast<uint32_t*>(myslot) = count;
    p.out_count[vr][0] = count;
    p.out_count[vr][1] = tau;
    scratch[kCursor + 2] = from_list ? 1u : 0u;  // which selection path ran (telemetry)
    scratch[kCursor + 3] = ncand;
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
  if (!gsync()) return;
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
    if (!gsync()) return;
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
      (p->nvr > 1 && p->nvr != p->world) || p->epoch == 0 || p->capacity == 0 ||
      p->capacity % 4 != 0 || p->k > p->capacity || (p->cand_capacity != 0 && p->cand_capacity < p->k) || !(p->momentum >= 0.0f && p->momentum < 1.0f))
    return int(cudaErrorInvalidValue);
  const void* fn;
  switch (p->grad_dtype) {
    case NANGILA_F32: fn = reinterpret_cast<const void*>(&dgc_fused_kernel<float>); break;
    case NANGILA_BF16: fn = reinterpret_cast<const void*>(&dgc_fused_kernel<__nv_bfloat16>); break;
    case NANGILA_F16: fn = reinterpret_cast<const void*>(&dgc_fused_kernel<__half>); break;
    default: return int(cudaErrorInvalidValue);
  }
  int grid_x = 0;
  const cudaError_t ce = clamp_grid(fn, kThreads, 0, p->grid_x, p->nvr, &grid_x);
  if (ce != cudaSuccess) return int(ce);
  dim3 grid(unsigned(grid_x), unsigned(p->nvr)), block(kThreads);
  void* args[] = {const_cast<NangilaDgcParams*>(p)};
  if (p->nvr > 1) return int(cudaLaunchCooperativeKernel(fn, grid, block, args, 0, stream));
  // real process group: plain launch; the counter of the in-kernel grid barrier starts from zero
  const cudaError_t me = cudaMemsetAsync(p->status[0] + comm::kStatusBarrier, 0, sizeof(uint32_t), stream);
  if (me != cudaSuccess) return int(me);
  return int(cudaLaunchKernel(fn, grid, block, args, 0, stream));
}
