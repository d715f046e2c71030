// Quantizing parameter all-gather for fully-sharded training (sm_100a): every rank quantizes its
// parameter shard to INT8 (default) or INT4 with one bf16 scale per 64 elements, stores the packed
// chunks straight into every rank's staging slots over NVLink, and every rank dequantizes all W
// shards directly into the unsharded parameter buffer the next layer reads. One launch replaces
// all-gather + copy-out; 1.03 (INT8) or 0.53 (INT4) bytes per element cross the links instead of 2.
//
// The owner of a shard also consumes the dequantized form of its own shard, so all ranks compute
// with bit-identical parameters. Rounding is to nearest (parameters must not pick up random noise).
//
// The reference leaves the FSDP parameter all-gather untouched (python/nangila/fsdp.py:80-236 only
// hooks the gradient path).
//
// Staging slots are double-buffered by launch parity: a rank may start launch t+1 while a slower
// peer still dequantizes launch t, but it cannot finish t+1 (and so cannot start t+2) before that
// peer has started t+1, because it needs the peer's flags of t+1.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "launch_util.cuh"
#include "nangila_kernels.h"
#include "quant.cuh"
#include "signal.cuh"

namespace nangila {
namespace {

using namespace dev;
using namespace comm;

constexpr int kThreads = 256;
constexpr int kE = 8;
constexpr int kPerIter = kThreads * kE;  // 2048

__host__ __device__ inline uint64_t ag_slot_bytes(int chunk, int bits) {
  return uint64_t(chunk) * bits / 8 + uint64_t(chunk) / kQuantBlock * 2;
}

template <typename T, int BITS>
__global__ void __launch_bounds__(kThreads, 4) fsdp_ag_kernel(const __grid_constant__ NangilaAgParams p) {
  const int vr = blockIdx.y;
  const int me = p.rank0 + vr;
  const int W = p.world;
  const int C = p.chunk_elems;
  const int iters = C / kPerIter;
  const int64_t shard = p.shard_elems;
  const int cps = int((shard + C - 1) / C);
  const int tid = threadIdx.x;
  const uint64_t slot = ag_slot_bytes(C, BITS);
  const uint64_t set_bytes = uint64_t(W) * cps * slot;
  const uint64_t recv = p.recv_off + uint64_t(p.epoch & 1u) * set_bytes;
  const T* __restrict__ in = static_cast<const T*>(p.in_shard[vr]);
  T* __restrict__ out = static_cast<T*>(p.out_full[vr]);
  uint32_t* status = p.status[vr];
  uint8_t* myreg = p.region[me];
  constexpr float kQmax = BITS == 8 ? 127.0f : 7.0f;
  constexpr float kInvQmax = BITS == 8 ? 0.0078740157f : 0.14285715f;

  const int ntasks = cps + W * cps;
  for (int task = blockIdx.x; task < ntasks; task += gridDim.x) {
    if (*reinterpret_cast<volatile uint32_t*>(&status[kStatusCode]) != 0u) break;
    if (task < cps) {
      // ---- quantize chunk `task` of my shard and store it into every rank's slot [me][task] ----
      const int j = task;
      for (int it = 0; it < iters; ++it) {
        const int64_t local = int64_t(j) * C + int64_t(it) * kPerIter + tid * kE;
        float x[kE];
        load8_guarded<T>(in, local, shard, x);
        float amax = 0.0f;
#pragma unroll
        for (int i = 0; i < kE; ++i) {
          x[i] = sanitize(x[i]);
          amax = fmaxf(amax, fabsf(x[i]));
        }
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
        uint32_t sb = bf16_ceil_bits(__fmul_rn(amax, kInvQmax));
        const float s = bf16_bits_to_float(sb);
        const bool live = s > 1e-30f;
        const float inv = live ? __frcp_rn(s) : 0.0f;
        if (!live) sb = 0;
        uint32_t w0 = 0, w1 = 0;
#pragma unroll
        for (int i = 0; i < kE; ++i) {
          const int q = int(fminf(fmaxf(rintf(x[i] * inv), -kQmax - 1.0f), kQmax));
          if (BITS == 8) {
            if (i < 4) w0 |= (uint32_t(q) & 0xffu) << (8 * i); else w1 |= (uint32_t(q) & 0xffu) << (8 * (i - 4));
          } else {
            w0 |= (uint32_t(q) & 0xfu) << (4 * i);
          }
        }
        int rr = me + 1 == W ? 0 : me + 1;  // peers first, this rank last; no division in the loop
        for (int r = 0; r < W; ++r, rr = (rr + 1 == W ? 0 : rr + 1)) {
          uint8_t* dst = p.region[rr] + recv + (uint64_t(me) * cps + j) * slot;
          if (BITS == 8) reinterpret_cast<uint2*>(dst + uint64_t(it) * kPerIter)[tid] = make_uint2(w0, w1);
          else reinterpret_cast<uint32_t*>(dst + uint64_t(it) * (kPerIter / 2))[tid] = w0;
          if ((tid & 7) == 0)
            reinterpret_cast<uint16_t*>(dst + uint64_t(C) * BITS / 8)[it * (kPerIter / kQuantBlock) + tid / 8] = uint16_t(sb);
        }
      }
      __syncthreads();
      if (tid < W) {
        __threadfence_system();
        st_release_sys(reinterpret_cast<uint32_t*>(p.region[tid] + p.flag_off) + (uint64_t(me) * cps + j), p.epoch);
      }
    } else {
      // ---- dequantize chunk j of owner o into the unsharded buffer ----
      const int idx = task - cps;
      const int o = (me + idx / cps) % W;  // own shard first
      const int j = idx % cps;
      bool ok = true;
      if (tid == 0)
        ok = wait_flag(reinterpret_cast<const uint32_t*>(myreg + p.flag_off) + (uint64_t(o) * cps + j), p.epoch,
                       p.timeout_ns, status, kTimeoutPhase3, uint32_t(me), uint32_t(o), 3u, uint32_t(j));
      if (!__syncthreads_and(ok ? 1 : 0)) break;
      const uint8_t* src = myreg + recv + (uint64_t(o) * cps + j) * slot;
      // The packed words and scales of kB iterations are fetched before any of them is expanded: the
      // stores to `out` may alias the slot as far as the compiler knows, so without this every load
      // would wait for the previous iteration's stores.
      constexpr int kB = 4;
      for (int it0 = 0; it0 < iters; it0 += kB) {
        uint2 w[kB];
        uint16_t sc[kB];
#pragma unroll
        for (int b = 0; b < kB; ++b) {
          const int it = it0 + b;
          w[b] = make_uint2(0u, 0u);
          sc[b] = 0;
          if (it < iters && int64_t(j) * C + int64_t(it) * kPerIter + tid * kE < shard) {
            sc[b] = reinterpret_cast<const uint16_t*>(src + uint64_t(C) * BITS / 8)[it * (kPerIter / kQuantBlock) + tid / 8];
            if (BITS == 8) w[b] = reinterpret_cast<const uint2*>(src + uint64_t(it) * kPerIter)[tid];
            else w[b].x = reinterpret_cast<const uint32_t*>(src + uint64_t(it) * (kPerIter / 2))[tid];
          }
        }
#pragma unroll
        for (int b = 0; b < kB; ++b) {
          const int it = it0 + b;
          const int64_t local = int64_t(j) * C + int64_t(it) * kPerIter + tid * kE;
          if (it >= iters || local >= shard) continue;
          const float s = bf16_bits_to_float(sc[b]);
          float y[kE];
          if (BITS == 8) {
#pragma unroll
            for (int i = 0; i < kE; ++i) {
              const uint32_t ww = i < 4 ? w[b].x : w[b].y;
              y[i] = float(int(ww << (24 - 8 * (i & 3))) >> 24) * s;
            }
          } else {
#pragma unroll
            for (int i = 0; i < kE; ++i) y[i] = float(int(w[b].x << (28 - 4 * i)) >> 28) * s;
          }
          store8_guarded<T>(out + int64_t(o) * shard, local, shard, y);
        }
      }
    }
  }
}

}  // namespace
}  // namespace nangila

extern "C" uint64_t nangila_ag_region_bytes(int64_t shard_elems, int32_t world, int32_t chunk_elems, int32_t bits,
                                            uint64_t* recv_off, uint64_t* flag_off) {
  auto align = [](uint64_t x) { return (x + 255) & ~uint64_t(255); };
  const uint64_t cps = uint64_t((shard_elems + chunk_elems - 1) / chunk_elems);
  uint64_t off = 0;
  if (recv_off) *recv_off = off;
  off = align(off + 2 * uint64_t(world) * cps * nangila::ag_slot_bytes(chunk_elems, bits));
  if (flag_off) *flag_off = off;
  off = align(off + uint64_t(world) * cps * 4);
  return off;
}

extern "C" int nangila_ag_launch(const NangilaAgParams* p, cudaStream_t stream) {
  using namespace nangila;
  if (p == nullptr || p->shard_elems <= 0 || p->shard_elems % 8 != 0 || p->world < 1 || p->world > NANGILA_MAX_RANKS ||
      p->nvr < 1 || p->nvr > NANGILA_MAX_VRANKS || p->rank0 < 0 || p->rank0 + p->nvr > p->world ||
      (p->nvr > 1 && p->nvr != p->world) || p->chunk_elems <= 0 || p->chunk_elems % kPerIter != 0 || p->epoch == 0 ||
      (p->bits != 8 && p->bits != 4))
    return int(cudaErrorInvalidValue);
  const void* fn = nullptr;
#define NANGILA_AG_PICK(TYPE)                                                                  \
  fn = p->bits == 8 ? reinterpret_cast<const void*>(&fsdp_ag_kernel<TYPE, 8>)                  \
                    : reinterpret_cast<const void*>(&fsdp_ag_kernel<TYPE, 4>)
  switch (p->dtype) {
    case NANGILA_F32: NANGILA_AG_PICK(float); break;
    case NANGILA_BF16: NANGILA_AG_PICK(__nv_bfloat16); break;
    case NANGILA_F16: NANGILA_AG_PICK(__half); break;
    default: return int(cudaErrorInvalidValue);
  }
#undef NANGILA_AG_PICK
  int grid_x = 0;
  const cudaError_t ce = clamp_grid(fn, kThreads, 0, p->grid_x, p->nvr, &grid_x);
  if (ce != cudaSuccess) return int(ce);
  dim3 grid(unsigned(grid_x), unsigned(p->nvr)), block(kThreads);
  void* args[] = {const_cast<NangilaAgParams*>(p)};
  if (p->nvr > 1) return int(cudaLaunchCooperativeKernel(fn, grid, block, args, 0, stream));
  return int(cudaLaunchKernel(fn, grid, block, args, 0, stream));
}
