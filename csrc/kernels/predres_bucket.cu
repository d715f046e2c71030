// Fused prediction-residual bucket exchange for sm_100a: predict-subtract, error feedback,
// block-scaled INT4 quantization, the cross-GPU exchange over NVLink peer memory, dequantize-
// accumulate, re-quantized broadcast, reconstruction and history update — one launch per bucket, no
// NCCL collective. See nangila_kernels.h for the phase description.
//
// What it replaces in the reference: predict_subtract_quantize[_vec4] (nangila-cuda/src/kernels/
// predict.cu:130-238), the size + data all-gathers around it (python/nangila/ddp.py:249-260,
// nangila_ddp/src/ddp_hook.cpp:260-288), W launches of dequantize_add_reconstruct[_vec4]
// (reconstruct.cu:42-131), the mean (ddp.py:272-273) and the history rotation
// (ddp_hook.cpp:325-326).
//
// Work decomposition. The bucket is cut into chunks of `chunk_elems`; chunk c is owned by rank
// c % W. Every CTA walks a fixed task list (task t belongs to CTA t % gridDim.x, in increasing t):
// first all phase-1 chunks, then the owned phase-2 chunks, then all phase-3 chunks. Phase-1 tasks
// never wait, so every rank always gets through them and every later wait is eventually served as
// long as each rank's CTAs become resident; in the single-GPU loopback world that is guaranteed by
// a cooperative launch. Waits are bounded (comm/signal.cuh).
//
// Data always moves by stores into the consumer's memory ("push"): phase 1 writes the packed chunk
// into the owner's slot [owned index][source rank]; phase 2 writes the reduced chunk into every
// rank's slot [chunk]. A flag in the consumer's memory is released after each chunk. Because every
// chunk's reduction needs all ranks, a rank that has finished launch k of a bucket knows that all
// ranks have finished reading what it wrote in launch k-1, so the slots need no double buffering.
#include <algorithm>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "nangila_kernels.h"
#include "quant.cuh"
#include "signal.cuh"

namespace nangila {
namespace {

using namespace dev;
using namespace comm;

constexpr int kThreads = 256;
constexpr int kElemsPerIter = kThreads * kElemsPerThread;  // 4096

// packed nibbles, then one bf16 scale per 64 elements, then a 16-byte trailer whose first word is the
// sender's prediction gain (phase 1) or the mean gain of all senders (phase 2)
__host__ __device__ inline uint64_t compressed_trailer_off(int chunk) {
  return uint64_t(chunk) / 2 + uint64_t(chunk) / kQuantBlock * 2;
}
__host__ __device__ inline uint64_t compressed_slot_bytes(int chunk) { return compressed_trailer_off(chunk) + 16; }

template <typename T, typename S, bool COMPRESSED>
__global__ void __launch_bounds__(kThreads, 2)
predres_bucket_kernel(const __grid_constant__ NangilaPredResParams p) {
  const int vr = blockIdx.y;
  const int me = p.rank0 + vr;
  const int W = p.world;
  const int C = p.chunk_elems;
  const int iters = C / kElemsPerIter;
  const int NC = p.nchunks;
  const int owned_max = (NC + W - 1) / W;
  const int my_owned = NC > me ? (NC - me + W - 1) / W : 0;
  const int64_t n = p.n;
  const int tid = threadIdx.x;
  const uint64_t slot = COMPRESSED ? compressed_slot_bytes(C) : uint64_t(C) * sizeof(T);
  const uint32_t epoch = p.epoch;
  const float mu = p.mu;
  const float kappa = p.pred_gain[vr];  // this rank's prediction gain for the bucket, in [0, 1]

  T* __restrict__ grad = static_cast<T*>(p.grad[vr]);
  S* __restrict__ prev = static_cast<S*>(p.prev[vr]);
  const S* __restrict__ curr = static_cast<const S*>(p.curr[vr]);
  S* __restrict__ ef = static_cast<S*>(p.ef[vr]);
  S* __restrict__ ef2 = static_cast<S*>(p.ef2[vr]);
  uint32_t* status = p.status[vr];
  uint8_t* myreg = p.region[me];

  const uint32_t key1 = make_key(p.seed, p.step, p.bucket_id, uint32_t(me), 1u);
  const uint32_t key2 = make_key(p.seed, p.step, p.bucket_id, 0u, 2u);
  const bool stochastic = p.stochastic != 0;

  float sum_e2 = 0.0f, sum_g2 = 0.0f, sum_xp = 0.0f, sum_pp = 0.0f, sum_f2 = 0.0f;

  const int T1 = owned_max * W;
  const int ntasks = T1 + my_owned + NC;
  for (int task = blockIdx.x; task < ntasks; task += gridDim.x) {
    if (*reinterpret_cast<volatile uint32_t*>(&status[kStatusCode]) != 0u) break;

    if (task < T1) {
      // ---------------- phase 1: quantize own residual, push to the chunk's owner -----------------
      const int k = task / W, d = task % W;
      const int o = (me + 1 + d) % W;  // remote owners first, own chunk last in each round
      const int c = k * W + o;
      if (c >= NC) continue;
      const int j = c / W;
      uint8_t* dst = p.region[o] + p.recv1_off + (uint64_t(j) * W + me) * slot;
      for (int it = 0; it < iters; ++it) {
        const int64_t base = int64_t(c) * C + int64_t(it) * kElemsPerIter + tid * kElemsPerThread;
        float g[16];
        load16_guarded<T>(grad, base, n, g);
#pragma unroll
        for (int i = 0; i < 16; ++i) g[i] = sanitize(g[i]);
        if constexpr (COMPRESSED) {
          float pv[16], cu[16];
          load16_guarded<S>(prev, base, n, pv);
          load16_guarded<S>(curr, base, n, cu);
          float e[16];
          if (ef != nullptr) {
            load16_guarded<S>(ef, base, n, e);
#pragma unroll
            for (int i = 0; i < 16; ++i) e[i] += g[i];
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) e[i] = g[i];
          }
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float pred = __fmaf_rn(mu, cu[i] - pv[i], cu[i]);
            sum_g2 = __fmaf_rn(g[i], g[i], sum_g2);
            sum_xp = __fmaf_rn(e[i], pred, sum_xp);  // <g + ef, g_hat>
            sum_pp = __fmaf_rn(pred, pred, sum_pp);  // <g_hat, g_hat>
            e[i] = __fmaf_rn(-kappa, pred, e[i]);
            sum_e2 = __fmaf_rn(e[i], e[i], sum_e2);
          }
          uint2 packed;
          uint32_t sb;
          float deq[16];
          quantize16(e, key1, uint32_t(base >> 1), stochastic, packed, sb, deq);
          if (ef != nullptr) {
            store16_guarded<S>(ef, base, n, e);
#pragma unroll
            for (int i = 0; i < 16; ++i) sum_f2 = __fmaf_rn(e[i], e[i], sum_f2);
          }
          *reinterpret_cast<uint2*>(dst + uint64_t(it) * (kElemsPerIter / 2) + tid * 8) = packed;
          if ((tid & (kLanesPerBlock - 1)) == 0)
            *reinterpret_cast<uint16_t*>(dst + uint64_t(C) / 2 +
                                         (uint64_t(it) * (kElemsPerIter / kQuantBlock) + tid / kLanesPerBlock) * 2) =
                uint16_t(sb);
        } else {
          Vec16<T>::store(reinterpret_cast<T*>(dst) + int64_t(it) * kElemsPerIter + tid * kElemsPerThread, g);
        }
      }
      if (COMPRESSED && tid == 0) *reinterpret_cast<float*>(dst + compressed_trailer_off(C)) = kappa;
      __syncthreads();
      if (tid == 0) {
        __threadfence_system();
        st_release_sys(reinterpret_cast<uint32_t*>(p.region[o] + p.flag1_off) + (uint64_t(j) * W + me), epoch);
      }
    } else if (task < T1 + my_owned) {
      // ---------------- phase 2: owner reduces the W contributions and broadcasts ------------------
      const int j = task - T1;
      const int c = j * W + me;
      bool ok = true;
      if (tid < W)
        ok = wait_flag(reinterpret_cast<const uint32_t*>(myreg + p.flag1_off) + (uint64_t(j) * W + tid), epoch,
                       p.timeout_ns, status, kTimeoutPhase2, uint32_t(me), uint32_t(tid), 2u, uint32_t(c));
      if (!__syncthreads_and(ok ? 1 : 0)) break;
      const float inv_w = 1.0f / float(W);
      if (COMPRESSED && tid < W) {
        // mean prediction gain of the senders: every rank applies the same value in phase 3
        float kbar = 0.0f;
        for (int r = 0; r < W; ++r)
          kbar += *reinterpret_cast<const float*>(myreg + p.recv1_off + (uint64_t(j) * W + r) * slot +
                                                  compressed_trailer_off(C));
        *reinterpret_cast<float*>(p.region[tid] + p.recv2_off + uint64_t(c) * slot + compressed_trailer_off(C)) =
            kbar * inv_w;
      }
      for (int it = 0; it < iters; ++it) {
        float acc[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[i] = 0.0f;
        for (int r = 0; r < W; ++r) {
          const uint8_t* src = myreg + p.recv1_off + (uint64_t(j) * W + r) * slot;
          if constexpr (COMPRESSED) {
            const uint2 pk = *reinterpret_cast<const uint2*>(src + uint64_t(it) * (kElemsPerIter / 2) + tid * 8);
            const uint32_t sb = *reinterpret_cast<const uint16_t*>(
                src + uint64_t(C) / 2 + (uint64_t(it) * (kElemsPerIter / kQuantBlock) + tid / kLanesPerBlock) * 2);
            dequant16_add(pk, bf16_bits_to_float(sb), acc);
          } else {
            float v[16];
            Vec16<T>::load(reinterpret_cast<const T*>(src) + int64_t(it) * kElemsPerIter + tid * kElemsPerThread, v);
#pragma unroll
            for (int i = 0; i < 16; ++i) acc[i] += v[i];
          }
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[i] *= inv_w;
        if constexpr (COMPRESSED) {
          const int64_t obase = int64_t(j) * C + int64_t(it) * kElemsPerIter + tid * kElemsPerThread;
          if (ef2 != nullptr) {
            float f[16];
            Vec16<S>::load(ef2 + obase, f);
#pragma unroll
            for (int i = 0; i < 16; ++i) acc[i] += f[i];
          }
          const int64_t base = int64_t(c) * C + int64_t(it) * kElemsPerIter + tid * kElemsPerThread;
          uint2 packed;
          uint32_t sb;
          float deq[16];
          quantize16(acc, key2, uint32_t(base >> 1), stochastic, packed, sb, deq);
          if (ef2 != nullptr) Vec16<S>::store(ef2 + obase, acc);
          for (int r = 0; r < W; ++r) {
            const int rr = (me + 1 + r) % W;
            uint8_t* dst = p.region[rr] + p.recv2_off + uint64_t(c) * slot;
            *reinterpret_cast<uint2*>(dst + uint64_t(it) * (kElemsPerIter / 2) + tid * 8) = packed;
            if ((tid & (kLanesPerBlock - 1)) == 0)
              *reinterpret_cast<uint16_t*>(dst + uint64_t(C) / 2 +
                                           (uint64_t(it) * (kElemsPerIter / kQuantBlock) + tid / kLanesPerBlock) * 2) =
                  uint16_t(sb);
          }
        } else {
          for (int r = 0; r < W; ++r) {
            const int rr = (me + 1 + r) % W;
            uint8_t* dst = p.region[rr] + p.recv2_off + uint64_t(c) * slot;
            Vec16<T>::store(reinterpret_cast<T*>(dst) + int64_t(it) * kElemsPerIter + tid * kElemsPerThread, acc);
          }
        }
      }
      __syncthreads();
      if (tid < W) {
        __threadfence_system();
        st_release_sys(reinterpret_cast<uint32_t*>(p.region[tid] + p.flag2_off) + c, epoch);
      }
    } else {
      // ---------------- phase 3: reconstruct, write bucket and history ------------------------------
      const int c = task - T1 - my_owned;
      bool ok = true;
      if (tid == 0)
        ok = wait_flag(reinterpret_cast<const uint32_t*>(myreg + p.flag2_off) + c, epoch, p.timeout_ns, status,
                       kTimeoutPhase3, uint32_t(me), uint32_t(c % W), 3u, uint32_t(c));
      if (!__syncthreads_and(ok ? 1 : 0)) break;
      const uint8_t* src = myreg + p.recv2_off + uint64_t(c) * slot;
      const float kbar = COMPRESSED ? *reinterpret_cast<const float*>(src + compressed_trailer_off(C)) : 0.0f;
      for (int it = 0; it < iters; ++it) {
        const int64_t base = int64_t(c) * C + int64_t(it) * kElemsPerIter + tid * kElemsPerThread;
        if (base >= n) continue;
        float out[16];
        if constexpr (COMPRESSED) {
          float pv[16], cu[16];
          load16_guarded<S>(prev, base, n, pv);
          load16_guarded<S>(curr, base, n, cu);
#pragma unroll
          for (int i = 0; i < 16; ++i) out[i] = kbar * __fmaf_rn(mu, cu[i] - pv[i], cu[i]);
          const uint2 pk = *reinterpret_cast<const uint2*>(src + uint64_t(it) * (kElemsPerIter / 2) + tid * 8);
          const uint32_t sb = *reinterpret_cast<const uint16_t*>(
              src + uint64_t(C) / 2 + (uint64_t(it) * (kElemsPerIter / kQuantBlock) + tid / kLanesPerBlock) * 2);
          dequant16_add(pk, bf16_bits_to_float(sb), out);
        } else {
          Vec16<T>::load(reinterpret_cast<const T*>(src) + int64_t(it) * kElemsPerIter + tid * kElemsPerThread, out);
        }
        store16_guarded<T>(grad, base, n, out);
        store16_guarded<S>(prev, base, n, out);  // becomes g(t) after the caller swaps prev and curr
      }
    }
  }

  // per-rank telemetry: five atomics per CTA
  if (p.stats[vr] != nullptr && COMPRESSED) {
    __shared__ float red[5][kThreads / 32];
    float v[5] = {sum_e2, sum_g2, sum_xp, sum_pp, sum_f2};
#pragma unroll
    for (int k = 0; k < 5; ++k) {
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) v[k] += __shfl_xor_sync(0xffffffffu, v[k], off);
      if ((tid & 31) == 0) red[k][tid >> 5] = v[k];
    }
    __syncthreads();
    if (tid < 5) {
      float a = 0.0f;
#pragma unroll
      for (int i = 0; i < kThreads / 32; ++i) a += red[tid][i];
      atomicAdd(&p.stats[vr][tid], a);
    }
  }
}

template <typename T, typename S>
cudaError_t launch_ts(const NangilaPredResParams& p, cudaStream_t stream) {
  dim3 grid(unsigned(p.grid_x), unsigned(p.nvr));
  dim3 block(kThreads);
  void* args[] = {const_cast<NangilaPredResParams*>(&p)};
  const void* fn = p.mode == 0 ? reinterpret_cast<const void*>(&predres_bucket_kernel<T, S, true>)
                               : reinterpret_cast<const void*>(&predres_bucket_kernel<T, S, false>);
  if (p.nvr > 1) return cudaLaunchCooperativeKernel(fn, grid, block, args, 0, stream);
  return cudaLaunchKernel(fn, grid, block, args, 0, stream);
}

}  // namespace
}  // namespace nangila

extern "C" uint64_t nangila_predres_region_bytes(int64_t n, int32_t world, int32_t chunk_elems, int32_t grad_dtype,
                                                 uint64_t* recv1_off, uint64_t* recv2_off, uint64_t* flag1_off,
                                                 uint64_t* flag2_off) {
  auto align = [](uint64_t x) { return (x + 255) & ~uint64_t(255); };
  const uint64_t esize = grad_dtype == NANGILA_F32 ? 4 : 2;
  const uint64_t nchunks = uint64_t((n + chunk_elems - 1) / chunk_elems);
  const uint64_t owned_max = (nchunks + world - 1) / world;
  const uint64_t slot = std::max<uint64_t>(nangila::compressed_slot_bytes(chunk_elems), uint64_t(chunk_elems) * esize);
  uint64_t off = 0;
  if (recv1_off) *recv1_off = off;
  off = align(off + owned_max * world * slot);
  if (recv2_off) *recv2_off = off;
  off = align(off + nchunks * slot);
  if (flag1_off) *flag1_off = off;
  off = align(off + owned_max * world * 4);
  if (flag2_off) *flag2_off = off;
  off = align(off + nchunks * 4);
  return off;
}

extern "C" int nangila_predres_launch(const NangilaPredResParams* p, cudaStream_t stream) {
  using namespace nangila;
  if (p == nullptr || p->n <= 0 || p->world < 1 || p->world > NANGILA_MAX_RANKS || p->nvr < 1 ||
      p->nvr > NANGILA_MAX_VRANKS || p->rank0 < 0 || p->rank0 + p->nvr > p->world || p->chunk_elems <= 0 ||
      p->chunk_elems % kElemsPerIter != 0 || p->epoch == 0 || p->grid_x < 1 ||
      p->nchunks != int32_t((p->n + p->chunk_elems - 1) / p->chunk_elems) || !(p->mu >= 0.0f && p->mu <= 1.0f) ||
      false)
    return int(cudaErrorInvalidValue);
  if (p->nvr > 1 && p->nvr != p->world) return int(cudaErrorInvalidValue);
  for (int v = 0; v < p->nvr; ++v)
    if (!(p->pred_gain[v] >= 0.0f && p->pred_gain[v] <= 1.0f)) return int(cudaErrorInvalidValue);
  cudaError_t e;
  const bool s32 = p->state_dtype == NANGILA_F32;
  if (!s32 && p->state_dtype != NANGILA_BF16) return int(cudaErrorInvalidValue);
  switch (p->grad_dtype) {
    case NANGILA_F32:
      e = s32 ? launch_ts<float, float>(*p, stream) : launch_ts<float, __nv_bfloat16>(*p, stream);
      break;
    case NANGILA_BF16:
      e = s32 ? launch_ts<__nv_bfloat16, float>(*p, stream) : launch_ts<__nv_bfloat16, __nv_bfloat16>(*p, stream);
      break;
    case NANGILA_F16:
      e = s32 ? launch_ts<__half, float>(*p, stream) : launch_ts<__half, __nv_bfloat16>(*p, stream);
      break;
    default: return int(cudaErrorInvalidValue);
  }
  return int(e);
}
