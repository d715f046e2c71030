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
#include <type_traits>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "launch_util.cuh"
#include "nangila_kernels.h"
#include "ptx_sm100.cuh"
#include "quant.cuh"
#include "signal.cuh"

namespace nangila {
namespace {

using namespace dev;
using namespace comm;

constexpr int kThreads = 256;
constexpr int kE = kElems8;                       // elements per thread per iteration
constexpr int kElemsPerIter = kThreads * kE;      // 2048

// packed nibbles, then one bf16 scale per 64 elements, then a 16-byte trailer whose first word is the
// sender's prediction gain (phase 1) or the mean gain of all senders (phase 2)
__host__ __device__ inline uint64_t compressed_trailer_off(int chunk) {
  return uint64_t(chunk) / 2 + uint64_t(chunk) / kQuantBlock * 2;
}
__host__ __device__ inline uint64_t compressed_slot_bytes(int chunk) { return compressed_trailer_off(chunk) + 16; }

// Slot layout (compressed modes), warp-major so that everything one warp needs from a chunk is
// contiguous and can be fetched with one bulk copy: packed nibbles [warp][iteration][lane] (4 bytes per
// lane = 8 elements), then bf16 scales [warp][iteration][4] (one per 64 elements), then the trailer.
__device__ __forceinline__ uint32_t* packed_ptr(uint8_t* slot, int C, int it, int tid) {
  const int iters = C / kElemsPerIter;
  return reinterpret_cast<uint32_t*>(slot) + ((tid >> 5) * iters + it) * 32 + (tid & 31);
}
__device__ __forceinline__ uint16_t* scale_ptr(uint8_t* slot, int C, int it, int tid) {
  const int iters = C / kElemsPerIter;
  return reinterpret_cast<uint16_t*>(slot + uint64_t(C) / 2) + ((tid >> 5) * iters + it) * 4 + ((tid & 31) >> 3);
}

struct TaskInfo {
  int phase;      // 1, 2, 3 or 0 (padding task: nothing to do)
  int c;          // chunk id (flag index)
  int j;          // index of the chunk among its owner's chunks
  int o;          // owner rank
  int64_t base;   // first element of the chunk in the bucket
  int64_t limit;  // elements at or beyond this index do not belong to the chunk's range
};
// All-reduce modes: chunk c covers [c C, (c+1) C) and belongs to rank c % W.
// Reduce-scatter mode: the bucket is W equal shards; rank o owns shard o, cut into `cps` chunks.
// Gather mode: every rank pushes each of its packed chunks to all ranks and later sums all W
// contributions of every chunk itself: tasks are NC quantize tasks followed by NC sum tasks.
template <bool RS, bool GATHER>
__device__ __forceinline__ TaskInfo decode_task(int task, int me, int W, int NC, int T1, int my_owned, int C,
                                                int64_t n, int cps, int64_t shard) {
  TaskInfo t;
  if (GATHER) {
    t.phase = task < NC ? 1 : 2;
    t.c = t.j = task < NC ? task : task - NC;
    t.o = me;
    t.base = int64_t(t.c) * C;
    t.limit = n;
    return t;
  }
  if (task < T1) {
    const int k = task / W, d = task % W;
    t.o = (me + 1 + d) % W;  // remote owners first, own chunk last in each round
    t.j = k;
    t.c = RS ? t.o * cps + k : k * W + t.o;
    t.phase = t.c < NC ? 1 : 0;
  } else if (task < T1 + my_owned) {
    t.j = task - T1;
    t.o = me;
    t.c = RS ? me * cps + t.j : t.j * W + me;
    t.phase = 2;
  } else {
    t.c = task - T1 - my_owned;
    t.j = t.c / W;
    t.o = t.c % W;
    t.phase = 3;
  }
  if (RS) {
    t.base = int64_t(t.o) * shard + int64_t(t.j) * C;
    t.limit = int64_t(t.o + 1) * shard;
  } else {
    t.base = int64_t(t.c) * C;
    t.limit = n;
  }
  return t;
}

struct Stats {
  float e2 = 0.0f, g2 = 0.0f, xp = 0.0f, pp = 0.0f, f2 = 0.0f;
};

// Phase 1 of the compressed modes for one chunk: x = g + ef - kappa * g_hat, block-INT4 quantize, new
// error memory, packed nibbles and scales stored into the owner's slot `dst`.
// LEAN: the rank's gain is zero and no statistics were asked for, so neither the history nor the
// five running sums are touched. GUARD: the chunk straddles the end of the range.
template <typename T, typename S, bool LEAN, bool GUARD, bool SINGLE>
__device__ __forceinline__ void phase1_compressed(T* __restrict__ grad, S* __restrict__ prev,
                                                  const S* __restrict__ curr, S* __restrict__ ef, uint8_t* dst,
                                                  int64_t tbase, int64_t lim, int iters, int C, int tid, float mu,
                                                  float kappa, bool use_history, uint32_t key1, bool stochastic,
                                                  Stats& st, int ndst, uint8_t* const* regions, uint64_t dst_off,
                                                  bool keep_history) {
#pragma unroll 2
  for (int it = 0; it < iters; ++it) {
    const int64_t base = tbase + int64_t(it) * kElemsPerIter + tid * kE;
    float g[kE], e[kE];
    load8<T, GUARD>(grad, base, lim, g);
    if (ef != nullptr) {
      load8<S, GUARD>(ef, base, lim, e);
#pragma unroll
      for (int i = 0; i < kE; ++i) {
        g[i] = sanitize(g[i]);
        e[i] += g[i];
      }
    } else {
#pragma unroll
      for (int i = 0; i < kE; ++i) e[i] = g[i] = sanitize(g[i]);
    }
    [[maybe_unused]] float pred[kE];
    if constexpr (!LEAN) {
      float pv[kE], cu[kE];
      if (use_history) {
        load8<S, GUARD>(prev, base, lim, pv);
        load8<S, GUARD>(curr, base, lim, cu);
      } else {
#pragma unroll
        for (int i = 0; i < kE; ++i) pv[i] = cu[i] = 0.0f;
      }
#pragma unroll
      for (int i = 0; i < kE; ++i) {
        pred[i] = __fmaf_rn(mu, cu[i] - pv[i], cu[i]);
        st.g2 = __fmaf_rn(g[i], g[i], st.g2);
        st.xp = __fmaf_rn(e[i], pred[i], st.xp);  // <g + ef, g_hat>
        st.pp = __fmaf_rn(pred[i], pred[i], st.pp);  // <g_hat, g_hat>
        e[i] = __fmaf_rn(-kappa, pred[i], e[i]);
        st.e2 = __fmaf_rn(e[i], e[i], st.e2);
      }
    }
    [[maybe_unused]] float out[kE];
    if constexpr (SINGLE) {
#pragma unroll
      for (int i = 0; i < kE; ++i) out[i] = e[i];
    }
    uint32_t packed, sb;
    quantize8(e, key1, uint32_t(base >> 1), stochastic, packed, sb);
    if (ef != nullptr) {
      store8<S, GUARD>(ef, base, lim, e);
      if constexpr (!LEAN) {
#pragma unroll
        for (int i = 0; i < kE; ++i) st.f2 = __fmaf_rn(e[i], e[i], st.f2);
      }
    }
    if constexpr (SINGLE) {
#pragma unroll
      for (int i = 0; i < kE; ++i) out[i] -= e[i];
      if constexpr (!LEAN) {
#pragma unroll
        for (int i = 0; i < kE; ++i) out[i] = __fmaf_rn(kappa, pred[i], out[i]);
      }
      store8<T, GUARD>(grad, base, lim, out);
      if (keep_history) store8<S, GUARD>(prev, base, lim, out);
    } else if (ndst == 1) {
      *packed_ptr(dst, C, it, tid) = packed;
      if ((tid & (kLanes8 - 1)) == 0) *scale_ptr(dst, C, it, tid) = uint16_t(sb);
    } else {
      // gather mode: the same words go to this chunk's slot [source = me] on every rank
      for (int r = 0; r < ndst; ++r) {
        uint8_t* d = regions[r] + dst_off;
        *packed_ptr(d, C, it, tid) = packed;
        if ((tid & (kLanes8 - 1)) == 0) *scale_ptr(d, C, it, tid) = uint16_t(sb);
      }
    }
  }
}

// Packed-bf16 fast path: bf16 gradients with bf16 state in the variants that neither read the history nor
// keep statistics (the gain is zero, which is where a run spends nearly all its calls once the controller
// has found nothing to predict).
template <typename T, typename S, bool LEAN>
constexpr bool kFastBf16 = LEAN && std::is_same_v<T, __nv_bfloat16> && std::is_same_v<S, __nv_bfloat16>;

constexpr int kWarpElems = 32 * kE;  // elements one warp handles per iteration (contiguous)
constexpr int kRingBytesPerWarp = 6144;

template <typename T, typename S, bool LEAN>
struct Ring {
  static constexpr int GB = kWarpElems * int(sizeof(T));
  static constexpr int SB = kWarpElems * int(sizeof(S));
  static constexpr int STAGE = GB + SB * (LEAN ? 1 : 3);  // grad, error memory, [prev, curr]
  static constexpr int D = (kRingBytesPerWarp / STAGE) < 2 ? 2 : (kRingBytesPerWarp / STAGE);
  static constexpr int BYTES_PER_WARP = D * STAGE;
};
constexpr int kMaxDepth = 6;

// Phase 1 for a chunk that lies wholly inside the range, with the inputs streamed through a per-warp
// ring in shared memory: lane 0 issues bulk copies (cp.async.bulk, completion on an mbarrier) D
// iterations ahead, so the warp never waits on a global load once the ring is primed and far more
// bytes are in flight than registers could hold. Each warp owns its ring and its barriers; `kuse`
// counts the stage uses of this warp since the start of the kernel (stage = kuse % D, parity from
// kuse / D). Returns false if a copy did not complete in time (the caller reports the failure).
// SINGLE (a world of one rank): nothing is exchanged; the dequantized value is written straight back to
// the bucket and the history, so the whole step is this one pass.
template <typename T, typename S, bool LEAN, bool SINGLE>
__device__ __forceinline__ bool phase1_bulk(T* __restrict__ grad, S* __restrict__ prev,
                                            const S* __restrict__ curr, S* __restrict__ ef, uint8_t* dst,
                                            int64_t tbase, int iters, int C, int tid, float mu, float kappa,
                                            bool use_history, uint32_t key1, bool stochastic, Stats& st,
                                            uint8_t* ring, uint64_t* bars, uint32_t& kuse, uint64_t timeout_ns,
                                            int ndst, uint8_t* const* regions, uint64_t dst_off, bool keep_history) {
  using R = Ring<T, S, LEAN>;
  constexpr int D = R::D;
  const int lane = tid & 31, warp = tid >> 5;
  const bool has_ef = ef != nullptr;
  const bool hist = !LEAN && use_history;
  const uint32_t bytes = uint32_t(R::GB + (has_ef ? R::SB : 0) + (hist ? 2 * R::SB : 0));
  auto issue = [&](int it, uint32_t k) {
    if (lane == 0) {
      uint8_t* sdst = ring + (k % D) * R::STAGE;
      uint64_t* bar = bars + (k % D);
      const int64_t e0 = tbase + int64_t(it) * kElemsPerIter + warp * kWarpElems;
      sm100::mbar_arrive_expect_tx(bar, bytes);
      sm100::bulk_load(sdst, grad + e0, R::GB, bar);
      if (has_ef) sm100::bulk_load(sdst + R::GB, ef + e0, R::SB, bar);
      if (hist) {
        sm100::bulk_load(sdst + R::GB + R::SB, prev + e0, R::SB, bar);
        sm100::bulk_load(sdst + R::GB + 2 * R::SB, curr + e0, R::SB, bar);
      }
    }
  };
  const uint32_t k0 = kuse;
  const int primed = iters < D ? iters : D;
  for (int i = 0; i < primed; ++i) issue(i, k0 + uint32_t(i));
  int issued = primed;
  bool ok = true;
  for (int it = 0; it < iters; ++it) {
    const uint32_t k = k0 + uint32_t(it);
    if (!__all_sync(0xffffffffu, sm100::mbar_wait(bars + (k % D), (k / D) & 1u, timeout_ns))) {
      ok = false;
      kuse = k;
      // drain what is still in flight (bounded) so that no copy lands after the CTA has gone
      for (int j = it + 1; j < issued; ++j) {
        const uint32_t kj = k0 + uint32_t(j);
        sm100::mbar_wait(bars + (kj % D), (kj / D) & 1u, timeout_ns);
      }
      break;
    }
    const uint8_t* sp = ring + (k % D) * R::STAGE;
    const int64_t base = tbase + int64_t(it) * kElemsPerIter + tid * kE;
    if constexpr (kFastBf16<T, S, LEAN>) {
      // packed bf16 arithmetic (quant.cuh): two elements per instruction, no FP32 round trip
      const uint4 gv = *reinterpret_cast<const uint4*>(sp + lane * 16);
      uint4 ev = make_uint4(0u, 0u, 0u, 0u);
      if (has_ef) ev = *reinterpret_cast<const uint4*>(sp + R::GB + lane * 16);
      uint32_t x[4] = {gv.x, gv.y, gv.z, gv.w};
      if (has_ef) {
        const uint32_t ew[4] = {ev.x, ev.y, ev.z, ev.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) x[j] = as_u32(__hadd2(as_bf162(x[j]), as_bf162(ew[j])));
      }
      if (!__any_sync(0xffffffffu, maybe_nonfinite8(x))) {
        __syncwarp();  // every lane has read the stage: lane 0 may refill it
        if (it + D < iters) {
          issue(it + D, k + uint32_t(D));
          issued = it + D + 1;
        }
        uint32_t packed, sb, qs[4];
        quantize8_bf16(x, packed, sb, qs);
        if (has_ef) *reinterpret_cast<uint4*>(ef + base) = make_uint4(x[0], x[1], x[2], x[3]);
        if constexpr (SINGLE) {
          const uint4 o = make_uint4(qs[0], qs[1], qs[2], qs[3]);
          *reinterpret_cast<uint4*>(grad + base) = o;
          if (keep_history) *reinterpret_cast<uint4*>(prev + base) = o;
        } else if (ndst == 1) {
          *packed_ptr(dst, C, it, tid) = packed;
          if ((tid & (kLanes8 - 1)) == 0) *scale_ptr(dst, C, it, tid) = uint16_t(sb);
        } else {
          for (int r = 0; r < ndst; ++r) {
            uint8_t* d = regions[r] + dst_off;
            *packed_ptr(d, C, it, tid) = packed;
            if ((tid & (kLanes8 - 1)) == 0) *scale_ptr(d, C, it, tid) = uint16_t(sb);
          }
        }
        continue;
      }
      // a NaN / Inf somewhere in the warp's slice (or magnitudes >= 2): the FP32 path below sanitises it
    }
    float g[kE], e[kE], pv[kE], cu[kE];
    Vec8<T>::load(reinterpret_cast<const T*>(sp) + lane * kE, g);
    if (has_ef) Vec8<S>::load(reinterpret_cast<const S*>(sp + R::GB) + lane * kE, e);
    if constexpr (!LEAN) {
      if (hist) {
        Vec8<S>::load(reinterpret_cast<const S*>(sp + R::GB + R::SB) + lane * kE, pv);
        Vec8<S>::load(reinterpret_cast<const S*>(sp + R::GB + 2 * R::SB) + lane * kE, cu);
      } else {
#pragma unroll
        for (int i = 0; i < kE; ++i) pv[i] = cu[i] = 0.0f;
      }
    }
    __syncwarp();  // every lane has read the stage: lane 0 may refill it
    if (it + D < iters) {
      issue(it + D, k + uint32_t(D));
      issued = it + D + 1;
    }
    if (has_ef) {
#pragma unroll
      for (int i = 0; i < kE; ++i) {
        g[i] = sanitize(g[i]);
        e[i] += g[i];
      }
    } else {
#pragma unroll
      for (int i = 0; i < kE; ++i) e[i] = g[i] = sanitize(g[i]);
    }
    if constexpr (!LEAN) {
#pragma unroll
      for (int i = 0; i < kE; ++i) {
        const float pred = __fmaf_rn(mu, cu[i] - pv[i], cu[i]);
        st.g2 = __fmaf_rn(g[i], g[i], st.g2);
        st.xp = __fmaf_rn(e[i], pred, st.xp);
        st.pp = __fmaf_rn(pred, pred, st.pp);
        e[i] = __fmaf_rn(-kappa, pred, e[i]);
        st.e2 = __fmaf_rn(e[i], e[i], st.e2);
      }
    }
    float out[kE];
    if constexpr (SINGLE) {
#pragma unroll
      for (int i = 0; i < kE; ++i) out[i] = e[i];
    }
    uint32_t packed, sb;
    quantize8(e, key1, uint32_t(base >> 1), stochastic, packed, sb);
    if (has_ef) {
      Vec8<S>::store(ef + base, e);
      if constexpr (!LEAN) {
#pragma unroll
        for (int i = 0; i < kE; ++i) st.f2 = __fmaf_rn(e[i], e[i], st.f2);
      }
    }
    if constexpr (SINGLE) {
#pragma unroll
      for (int i = 0; i < kE; ++i) out[i] -= e[i];  // q * scale
      if constexpr (!LEAN) {
#pragma unroll
        for (int i = 0; i < kE; ++i) out[i] = __fmaf_rn(kappa, __fmaf_rn(mu, cu[i] - pv[i], cu[i]), out[i]);
      }
      Vec8<T>::store(grad + base, out);
      if (keep_history) Vec8<S>::store(prev + base, out);  // becomes g(t) after the caller swaps prev and curr
    } else if (ndst == 1) {
      *packed_ptr(dst, C, it, tid) = packed;
      if ((tid & (kLanes8 - 1)) == 0) *scale_ptr(dst, C, it, tid) = uint16_t(sb);
    } else {
      // gather mode: the same words go to this chunk's slot [source = me] on every rank
      for (int r = 0; r < ndst; ++r) {
        uint8_t* d = regions[r] + dst_off;
        *packed_ptr(d, C, it, tid) = packed;
        if ((tid & (kLanes8 - 1)) == 0) *scale_ptr(d, C, it, tid) = uint16_t(sb);
      }
    }
  }
  if (ok) kuse = k0 + uint32_t(iters);
  return ok;
}

constexpr int kWarps = kThreads / 32;
constexpr int kSlots = 4;  // completion counters in flight per CTA

// The eight warps of a CTA work on the same task but never meet at a block barrier: each warp waits
// for the task's input flag itself, processes its own 256-element slices of every iteration, and then
// bumps the task's completion counter in shared memory. Whichever warp arrives last publishes the
// task's flag (system-scope fence + release store). A block barrier here would leave every warp idle,
// with no loads in flight, until the slowest one and the fence were done. A warp may run at most
// kSlots - 1 tasks ahead of the slowest warp of its CTA (the counters are reused round-robin).
// MODE 0: exact all-reduce; 1: compressed all-reduce; 2: compressed reduce-scatter (phases 1 and 2
// only: the owner writes the mean of its shard to out_shard, nothing is broadcast, no history);
// 3: compressed all-reduce, lean phase 1 (this rank's gain is zero and no statistics are wanted);
// 4 / 5: world of one rank, full / lean: phase 1 alone quantizes, reconstructs and writes the result;
// 6 / 7: gather mode, full / lean (small worlds): phase 1 pushes the packed chunk to every rank, and
// every rank sums the W contributions of every chunk itself: one quantization, two phases.
template <typename T, typename S, int MODE>
__global__ void __launch_bounds__(kThreads, 4)
predres_bucket_kernel(const __grid_constant__ NangilaPredResParams p) {
  constexpr bool COMPRESSED = MODE != 0;
  constexpr bool RS = MODE == 2;
  constexpr bool LEAN = MODE == 2 || MODE == 3 || MODE == 5 || MODE == 7;
  constexpr bool SINGLE = MODE == 4 || MODE == 5;
  constexpr bool GATHER = MODE == 6 || MODE == 7;
  const int vr = blockIdx.y;
  const int me = p.rank0 + vr;
  const int W = p.world;
  const int C = p.chunk_elems;
  const int iters = C / kElemsPerIter;
  const int NC = p.nchunks;
  const int64_t n = p.n;
  const int64_t shard = RS ? n / W : 0;
  const int cps = RS ? NC / W : 0;
  const int owned_max = RS ? cps : (NC + W - 1) / W;
  const int my_owned = RS ? cps : (NC > me ? (NC - me + W - 1) / W : 0);
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const uint64_t slot = COMPRESSED ? compressed_slot_bytes(C) : uint64_t(C) * sizeof(T);
  const uint32_t epoch = p.epoch;
  uint32_t* status = p.status[vr];
  uint8_t* myreg = p.region[me];
  const int T1 = owned_max * W;
  const int ntasks = GATHER ? 2 * NC : SINGLE ? T1 : T1 + my_owned + (RS ? 0 : NC);
  // Reduce-scatter has no phase 3 to prove that the owner is done reading, so its slots alternate
  // between two sets by launch parity (a rank cannot get two launches ahead of a peer: its phase 2 of
  // the launch in between needs that peer's flags).
  // (gather mode alternates for the same reason: a rank may start the next launch while a peer still sums)
  const uint64_t recv1 = p.recv1_off + (RS       ? uint64_t(epoch & 1u) * uint64_t(cps) * W * slot
                                        : GATHER ? uint64_t(epoch & 1u) * uint64_t(NC) * W * slot
                                                 : 0);

  __shared__ int s_count[kSlots];   // warps that have finished the task in this slot
  __shared__ int s_done;            // tasks of this CTA whose flag has been published
  __shared__ float red[5][kWarps];
  __shared__ __align__(8) uint64_t s_bars[kWarps][kMaxDepth];  // per-warp ring barriers (phase 1)
  __shared__ __align__(8) uint64_t s_bat[kWarps][2];            // per-warp batch barriers (phases 2 and 3)
  extern __shared__ __align__(128) uint8_t s_ring[];           // kWarps * Ring::BYTES_PER_WARP (compressed modes)
  if (tid < kSlots) s_count[tid] = 0;
  if (tid == 0) s_done = 0;
  if (COMPRESSED && tid < kWarps * kMaxDepth) sm100::mbar_init(&s_bars[0][0] + tid, 1);
  if (COMPRESSED && tid < kWarps * 2) sm100::mbar_init(&s_bat[0][0] + tid, 1);
  if (COMPRESSED) sm100::fence_barrier_init();
  __syncthreads();
  uint32_t ring_uses = 0;  // stage uses of this warp's ring so far
  // Phases 2 and 3 fetch their (small, strided) inputs in batches of `ib` iterations with bulk copies
  // into the two halves of the warp's ring: batch b+1 is in flight while batch b is processed.
  constexpr int kRingBytes = COMPRESSED ? Ring<T, S, LEAN>::BYTES_PER_WARP : 0;
  constexpr int kHalf = (kRingBytes / 2) & ~127;
  constexpr int kIterBytes = 32 * 4 + 4 * 2;  // packed words + scales of one warp for one iteration
  constexpr int kStateBytes = kWarpElems * int(sizeof(S));
  const int warp = tid >> 5;
  uint8_t* const wring = s_ring + warp * kRingBytes;
  uint64_t* const wbat = &s_bat[warp][0];
  uint32_t bat_parity = 0u;  // bit h: parity of the next phase of this warp's batch barrier h
  bool failed = false;

  const float mu = p.mu;
  const float kappa = RS ? 0.0f : p.pred_gain[vr];  // this rank's prediction gain for the bucket, in [0, 1]
  T* __restrict__ grad = static_cast<T*>(p.grad[vr]);
  S* __restrict__ prev = static_cast<S*>(p.prev[vr]);
  const S* __restrict__ curr = static_cast<const S*>(p.curr[vr]);
  S* __restrict__ ef = static_cast<S*>(p.ef[vr]);
  S* __restrict__ ef2 = static_cast<S*>(p.ef2[vr]);
  const uint32_t key1 = make_key(p.seed, p.step, p.bucket_id, uint32_t(me), 1u);
  const uint32_t key2 = make_key(p.seed, p.step, p.bucket_id, 0u, 2u);
  const bool stochastic = p.stochastic != 0;
  // With a zero gain the history only matters for the statistics that steer the gain; the host asks
  // for them on probe steps (p.measure) and the loads are skipped otherwise.
  const bool use_history = !RS && (kappa != 0.0f || p.measure != 0);
  // The new history may be left unwritten only where nothing will read it: the caller asks for that
  // while the gain is 0 and no probe is near. A non-zero gain or a probe always writes it.
  const bool keep_history = !COMPRESSED || p.skip_history == 0 || use_history;
  Stats acc_stats;

  // Phases of the epoch this launch runs (see NangilaPredResParams::phase_mask): tasks are ordered by
  // phase, so a contiguous set of phases is a contiguous task range.
  const int pm = (p.phase_mask & 7) == 0 ? 7 : (p.phase_mask & 7);
  const int end1 = GATHER ? NC : T1;
  const int end2 = GATHER ? 2 * NC : SINGLE ? T1 : T1 + my_owned;
  const int task_begin = (pm & 1) ? 0 : (pm & 2) ? end1 : end2;
  const int task_end = (pm & 4) ? ntasks : (pm & 2) ? end2 : end1;

  int local = 0;  // number of the task within this CTA
  for (int task = task_begin + int(blockIdx.x); task < task_end; task += gridDim.x, ++local) {
    const TaskInfo t = decode_task<RS, GATHER>(task, me, W, NC, T1, my_owned, C, n, cps, shard);
    const int c = t.c, j = t.j;
    const int64_t lim = t.limit;
    // ---- entry (per warp): stop if this rank has failed; do not run too far ahead; wait for inputs ----
    int ok = 1;
    if (lane == 0) {
      if (*reinterpret_cast<volatile uint32_t*>(&status[kStatusCode]) != 0u) ok = 0;
      const uint64_t t0 = globaltimer_ns();
      while (ok && local - *reinterpret_cast<volatile int*>(&s_done) >= kSlots) {
        __nanosleep(64);
        if (*reinterpret_cast<volatile uint32_t*>(&status[kStatusCode]) != 0u) ok = 0;
        else if (globaltimer_ns() - t0 > p.timeout_ns) {
          report_failure(status, kTimeoutGrid, uint32_t(me), 0xffffffffu, epoch, 0u, uint32_t(t.phase), uint32_t(c));
          ok = 0;
        }
      }
      if (ok && t.phase == 3) {
        ok = wait_flag(reinterpret_cast<const uint32_t*>(myreg + p.flag2_off) + c, epoch, p.timeout_ns, status,
                       kTimeoutPhase3, uint32_t(me), uint32_t(t.o), 3u, uint32_t(c));
      }
    }
    ok = __shfl_sync(0xffffffffu, ok, 0);
    if (ok && t.phase == 2) {
      // one lane per source rank: the W flags are polled side by side
      int mine = 1;
      for (int r = lane; r < W; r += 32)
        mine = mine && wait_flag(reinterpret_cast<const uint32_t*>(myreg + p.flag1_off) + (uint64_t(j) * W + r), epoch,
                                 p.timeout_ns, status, kTimeoutPhase2, uint32_t(me), uint32_t(r), 2u, uint32_t(c));
      ok = __all_sync(0xffffffffu, mine);
    }
    if (!ok) break;
    if (COMPRESSED && t.phase != 1) {
      // the flags were acquired through the generic proxy; the bulk copies below read through the
      // async proxy
      __syncwarp();
      asm volatile("fence.proxy.async.global;" ::: "memory");
    }

    if (t.phase == 1) {
      // ---------------- phase 1: quantize own residual, push to the chunk's owner -------------------
      const uint64_t dst_off = recv1 + (uint64_t(j) * W + me) * slot;
      uint8_t* dst = p.region[t.o] + dst_off;
      const int ndst = GATHER ? W : 1;
      const bool full = t.base + C <= lim;  // whole chunk inside the range: no per-access bounds checks
      if constexpr (COMPRESSED) {
        if (full) {
          using R = Ring<T, S, LEAN>;
          const int warp = tid >> 5;
          if (!phase1_bulk<T, S, LEAN, SINGLE>(grad, prev, curr, ef, dst, t.base, iters, C, tid, mu, kappa, use_history, key1,
                                       stochastic, acc_stats, s_ring + warp * R::BYTES_PER_WARP, &s_bars[warp][0],
                                       ring_uses, p.timeout_ns, ndst, p.region, dst_off, keep_history)) {
            if (lane == 0)
              report_failure(status, kTimeoutBulk, uint32_t(me), 0xffffffffu, epoch, 0u, 1u, uint32_t(c));
            break;
          }
        } else
          phase1_compressed<T, S, LEAN, true, SINGLE>(grad, prev, curr, ef, dst, t.base, lim, iters, C, tid, mu, kappa,
                                              use_history, key1, stochastic, acc_stats, ndst, p.region, dst_off,
                                              keep_history);
        if (!SINGLE && !GATHER && tid == 0) *reinterpret_cast<float*>(dst + compressed_trailer_off(C)) = kappa;
        if (GATHER && tid < W) *reinterpret_cast<float*>(p.region[tid] + dst_off + compressed_trailer_off(C)) = kappa;
      } else {
#pragma unroll 2
        for (int it = 0; it < iters; ++it) {
          const int64_t base = t.base + int64_t(it) * kElemsPerIter + tid * kE;
          float g[kE];
          if (full) Vec8<T>::load(grad + base, g);
          else load8_guarded<T>(grad, base, lim, g);
#pragma unroll
          for (int i = 0; i < kE; ++i) g[i] = sanitize(g[i]);
          Vec8<T>::store(reinterpret_cast<T*>(dst) + int64_t(it) * kElemsPerIter + tid * kE, g);
        }
      }
    } else if (t.phase == 2) {
      // ---------------- phase 2: owner reduces the W contributions and broadcasts --------------------
      const float inv_w = 1.0f / float(W);
      uint8_t* src0 = myreg + recv1 + uint64_t(j) * W * slot;
      [[maybe_unused]] float gbar = kappa;  // gather mode: the gain applied to the prediction
      if (GATHER && p.uniform_gain == 0) {
        gbar = 0.0f;
        for (int r = 0; r < W; ++r)
          gbar += *reinterpret_cast<const float*>(src0 + uint64_t(r) * slot + compressed_trailer_off(C));
        gbar *= inv_w;
      }
      if (COMPRESSED && !RS && !GATHER && tid < W) {
        // mean prediction gain of the senders: every rank applies the same value in phase 3
        float kbar = 0.0f;
        for (int r = 0; r < W; ++r)
          kbar += *reinterpret_cast<const float*>(src0 + uint64_t(r) * slot + compressed_trailer_off(C));
        *reinterpret_cast<float*>(p.region[tid] + p.recv2_off + uint64_t(c) * slot + compressed_trailer_off(C)) =
            kbar * inv_w;
      }
      const uint64_t off2 = p.recv2_off + uint64_t(c) * slot;  // this chunk's broadcast slot in every region
      // what happens to the sum of one iteration (8 elements of this lane)
      auto finish = [&](int it, float (&acc)[kE]) {
#pragma unroll
        for (int i = 0; i < kE; ++i) acc[i] *= RS ? p.out_scale : inv_w;
        if constexpr (RS) {
          // reduce-scatter: the mean of this rank's shard is the result; nothing is broadcast
          const int64_t local_i = int64_t(j) * C + int64_t(it) * kElemsPerIter + tid * kE;
          store8_guarded<T>(static_cast<T*>(p.out_shard[vr]), local_i, shard, acc);
        } else if constexpr (GATHER) {
          // the mean of the W dequantized residuals plus the prediction is the result on every rank
          const int64_t base = t.base + int64_t(it) * kElemsPerIter + tid * kE;
          if (base < n) {
            if (gbar != 0.0f) {
              float pv[kE], cu[kE];
              load8_guarded<S>(prev, base, n, pv);
              load8_guarded<S>(curr, base, n, cu);
#pragma unroll
              for (int i = 0; i < kE; ++i) acc[i] = __fmaf_rn(gbar, __fmaf_rn(mu, cu[i] - pv[i], cu[i]), acc[i]);
            }
            store8_guarded<T>(grad, base, n, acc);
            if (keep_history) store8_guarded<S>(prev, base, n, acc);  // becomes g(t) after the caller swaps prev and curr
          }
        } else if constexpr (COMPRESSED) {
          const int64_t obase = int64_t(j) * C + int64_t(it) * kElemsPerIter + tid * kE;
          if (ef2 != nullptr) {
            float f[kE];
            Vec8<S>::load(ef2 + obase, f);
#pragma unroll
            for (int i = 0; i < kE; ++i) acc[i] += f[i];
          }
          const int64_t base = t.base + int64_t(it) * kElemsPerIter + tid * kE;
          uint32_t packed, sb;
          quantize8(acc, key2, uint32_t(base >> 1), stochastic, packed, sb);
          if (ef2 != nullptr) Vec8<S>::store(ef2 + obase, acc);
          // peers first, this rank last; no division in the loop
          int rr = me + 1 == W ? 0 : me + 1;
          for (int r = 0; r < W; ++r) {
            uint8_t* dst = p.region[rr] + off2;
            *packed_ptr(dst, C, it, tid) = packed;
            if ((tid & (kLanes8 - 1)) == 0) *scale_ptr(dst, C, it, tid) = uint16_t(sb);
            rr = rr + 1 == W ? 0 : rr + 1;
          }
        } else {
          int rr = me + 1 == W ? 0 : me + 1;
          for (int r = 0; r < W; ++r) {
            Vec8<T>::store(reinterpret_cast<T*>(p.region[rr] + off2) + int64_t(it) * kElemsPerIter + tid * kE, acc);
            rr = rr + 1 == W ? 0 : rr + 1;
          }
        }
      };
      // packed-bf16 form of the same (quant.cuh): the mean's factor 1 / W (or out_scale) is folded into each
      // rank's block scale, so the sum of the dequantized codes is already the result
      [[maybe_unused]] const bool fast2 = kFastBf16<T, S, LEAN> && t.base + C <= lim && (!GATHER || gbar == 0.0f) &&
                                          (RS || GATHER || ef2 == nullptr);
      [[maybe_unused]] auto finish_fast = [&](int it, uint32_t (&acc)[4]) {
        if constexpr (kFastBf16<T, S, LEAN>) {
          const uint4 o = make_uint4(acc[0], acc[1], acc[2], acc[3]);
          if constexpr (RS) {
            const int64_t local_i = int64_t(j) * C + int64_t(it) * kElemsPerIter + tid * kE;
            *reinterpret_cast<uint4*>(static_cast<T*>(p.out_shard[vr]) + local_i) = o;
          } else if constexpr (GATHER) {
            const int64_t base = t.base + int64_t(it) * kElemsPerIter + tid * kE;
            *reinterpret_cast<uint4*>(grad + base) = o;
            if (keep_history) *reinterpret_cast<uint4*>(prev + base) = o;
          } else {
            uint32_t packed, sb, qs[4];
            quantize8_bf16(acc, packed, sb, qs);
            int rr = me + 1 == W ? 0 : me + 1;
            for (int r = 0; r < W; ++r) {
              uint8_t* dst = p.region[rr] + off2;
              *packed_ptr(dst, C, it, tid) = packed;
              if ((tid & (kLanes8 - 1)) == 0) *scale_ptr(dst, C, it, tid) = uint16_t(sb);
              rr = rr + 1 == W ? 0 : rr + 1;
            }
          }
        }
      };
      [[maybe_unused]] const float mulw = RS ? p.out_scale : inv_w;
      bool batched = false;
      if constexpr (COMPRESSED) {
        const int ib = min(iters, kHalf / (W * kIterBytes)) & ~1;
        if ((iters & 1) == 0 && ib >= 2) {
          batched = true;
          const int nb = (iters + ib - 1) / ib;
          auto issue = [&](int b) {
            if (lane == 0) {
              const int h = b & 1, it0 = b * ib, m = min(ib, iters - it0);
              uint8_t* buf = wring + h * kHalf;
              sm100::mbar_arrive_expect_tx(wbat + h, uint32_t(W * m * kIterBytes));
              for (int r = 0; r < W; ++r) {
                uint8_t* src = src0 + uint64_t(r) * slot;
                sm100::bulk_load(buf + r * ib * 128, packed_ptr(src, C, it0, warp * 32), uint32_t(m * 128), wbat + h);
                sm100::bulk_load(buf + W * ib * 128 + r * ib * 8, scale_ptr(src, C, it0, warp * 32), uint32_t(m * 8),
                                 wbat + h);
              }
            }
          };
          issue(0);
          for (int b = 0; b < nb; ++b) {
            if (b + 1 < nb) issue(b + 1);
            const int h = b & 1, it0 = b * ib, m = min(ib, iters - it0);
            if (!__all_sync(0xffffffffu, sm100::mbar_wait(wbat + h, (bat_parity >> h) & 1u, p.timeout_ns))) {
              if (b + 1 < nb) sm100::mbar_wait(wbat + (h ^ 1), (bat_parity >> (h ^ 1)) & 1u, p.timeout_ns);
              failed = true;
              break;
            }
            bat_parity ^= 1u << h;
            const uint8_t* buf = wring + h * kHalf;
            for (int i = 0; i < m; ++i) {
              if constexpr (kFastBf16<T, S, LEAN>) {
                if (fast2) {
                  uint32_t acc2[4] = {0u, 0u, 0u, 0u};
#pragma unroll 4
                  for (int r = 0; r < W; ++r) {
                    const uint32_t pk = reinterpret_cast<const uint32_t*>(buf + r * ib * 128)[i * 32 + lane];
                    const uint16_t sc = reinterpret_cast<const uint16_t*>(buf + W * ib * 128 + r * ib * 8)[i * 4 + (lane >> 3)];
                    dequant8_bf16_fma(pk, bf16_rn_bits(bf16_bits_to_float(sc) * mulw), acc2);
                  }
                  finish_fast(it0 + i, acc2);
                  continue;
                }
              }
              float acc[kE];
#pragma unroll
              for (int q = 0; q < kE; ++q) acc[q] = 0.0f;
#pragma unroll 4
              for (int r = 0; r < W; ++r) {
                const uint32_t pk = reinterpret_cast<const uint32_t*>(buf + r * ib * 128)[i * 32 + lane];
                const uint16_t sc = reinterpret_cast<const uint16_t*>(buf + W * ib * 128 + r * ib * 8)[i * 4 + (lane >> 3)];
                dequant8_add(pk, bf16_bits_to_float(sc), acc);
              }
              finish(it0 + i, acc);
            }
            __syncwarp();  // the half may be refilled by the issue two batches later
          }
        }
      }
      if (!batched) {
#pragma unroll 2
        for (int it = 0; it < iters; ++it) {
          float acc[kE];
#pragma unroll
          for (int i = 0; i < kE; ++i) acc[i] = 0.0f;
          if constexpr (COMPRESSED) {
#pragma unroll 4
            for (int r = 0; r < W; ++r) {
              uint8_t* src = src0 + uint64_t(r) * slot;
              dequant8_add(*packed_ptr(src, C, it, tid), bf16_bits_to_float(*scale_ptr(src, C, it, tid)), acc);
            }
          } else {
#pragma unroll 4
            for (int r = 0; r < W; ++r) {
              float v[kE];
              Vec8<T>::load(reinterpret_cast<const T*>(src0 + uint64_t(r) * slot) + int64_t(it) * kElemsPerIter + tid * kE, v);
#pragma unroll
              for (int i = 0; i < kE; ++i) acc[i] += v[i];
            }
          }
          finish(it, acc);
        }
      }
    } else if (t.phase == 3) {
      // ---------------- phase 3: reconstruct, write bucket and history -------------------------------
      uint8_t* src = myreg + p.recv2_off + uint64_t(c) * slot;
      // with uniform gains the owner's mean equals this rank's own gain: no dependent load before the copies
      const float kbar = !COMPRESSED        ? 0.0f
                         : p.uniform_gain != 0 ? kappa
                                               : *reinterpret_cast<const float*>(src + compressed_trailer_off(C));
      // one iteration of this lane once its packed word and scale are known
      auto emit = [&](auto guard_tag, int it, uint32_t pk, uint16_t sc, const uint8_t* hist_smem) {
        constexpr bool GUARD = decltype(guard_tag)::value;
        const int64_t base = t.base + int64_t(it) * kElemsPerIter + tid * kE;
        if (GUARD && base >= n) return;
        float out[kE];
        if constexpr (COMPRESSED) {
          if (kbar != 0.0f) {
            float pv[kE], cu[kE];
            if (hist_smem != nullptr) {
              Vec8<S>::load(reinterpret_cast<const S*>(hist_smem) + lane * kE, pv);
              Vec8<S>::load(reinterpret_cast<const S*>(hist_smem + kStateBytes) + lane * kE, cu);
            } else {
              load8<S, GUARD>(prev, base, n, pv);
              load8<S, GUARD>(curr, base, n, cu);
            }
#pragma unroll
            for (int q = 0; q < kE; ++q) out[q] = kbar * __fmaf_rn(mu, cu[q] - pv[q], cu[q]);
          } else {
#pragma unroll
            for (int q = 0; q < kE; ++q) out[q] = 0.0f;
          }
          dequant8_add(pk, bf16_bits_to_float(sc), out);
        } else {
          Vec8<T>::load(reinterpret_cast<const T*>(src) + int64_t(it) * kElemsPerIter + tid * kE, out);
        }
        store8<T, GUARD>(grad, base, n, out);
        if (keep_history) store8<S, GUARD>(prev, base, n, out);  // becomes g(t) after the caller swaps prev and curr
      };
      const bool whole = t.base + C <= n;
      bool batched = false;
      if constexpr (COMPRESSED) {
        // the history rides along only for whole chunks (a bulk copy may not run past the bucket's end)
        const bool hist = kbar != 0.0f && whole;
        const int per_it = kIterBytes + (hist ? 2 * kStateBytes : 0);
        const int ib = min(iters, kHalf / per_it) & ~1;
        if ((iters & 1) == 0 && ib >= 2) {
          batched = true;
          const int nb = (iters + ib - 1) / ib;
          auto issue = [&](int b) {
            if (lane == 0) {
              const int h = b & 1, it0 = b * ib, m = min(ib, iters - it0);
              uint8_t* buf = wring + h * kHalf;
              sm100::mbar_arrive_expect_tx(wbat + h, uint32_t(m * per_it));
              sm100::bulk_load(buf, packed_ptr(src, C, it0, warp * 32), uint32_t(m * 128), wbat + h);
              sm100::bulk_load(buf + ib * 128, scale_ptr(src, C, it0, warp * 32), uint32_t(m * 8), wbat + h);
              if (hist) {
                for (int i = 0; i < m; ++i) {
                  const int64_t e0 = t.base + int64_t(it0 + i) * kElemsPerIter + warp * kWarpElems;
                  uint8_t* hb = buf + ib * kIterBytes + i * 2 * kStateBytes;
                  sm100::bulk_load(hb, prev + e0, uint32_t(kStateBytes), wbat + h);
                  sm100::bulk_load(hb + kStateBytes, curr + e0, uint32_t(kStateBytes), wbat + h);
                }
              }
            }
          };
          issue(0);
          for (int b = 0; b < nb; ++b) {
            if (b + 1 < nb) issue(b + 1);
            const int h = b & 1, it0 = b * ib, m = min(ib, iters - it0);
            if (!__all_sync(0xffffffffu, sm100::mbar_wait(wbat + h, (bat_parity >> h) & 1u, p.timeout_ns))) {
              if (b + 1 < nb) sm100::mbar_wait(wbat + (h ^ 1), (bat_parity >> (h ^ 1)) & 1u, p.timeout_ns);
              failed = true;
              break;
            }
            bat_parity ^= 1u << h;
            const uint8_t* buf = wring + h * kHalf;
            for (int i = 0; i < m; ++i) {
              const uint32_t pk = reinterpret_cast<const uint32_t*>(buf)[i * 32 + lane];
              const uint16_t sc = reinterpret_cast<const uint16_t*>(buf + ib * 128)[i * 4 + (lane >> 3)];
              if constexpr (kFastBf16<T, S, LEAN>) {
                if (whole && kbar == 0.0f) {  // packed-bf16 form: q * scale straight into the bucket's type
                  uint32_t o[4] = {0u, 0u, 0u, 0u};
                  dequant8_bf16_fma(pk, sc, o);
                  const int64_t base = t.base + int64_t(it0 + i) * kElemsPerIter + tid * kE;
                  const uint4 ov = make_uint4(o[0], o[1], o[2], o[3]);
                  *reinterpret_cast<uint4*>(grad + base) = ov;
                  if (keep_history) *reinterpret_cast<uint4*>(prev + base) = ov;
                  continue;
                }
              }
              const uint8_t* hs = hist ? buf + ib * kIterBytes + i * 2 * kStateBytes : nullptr;
              if (whole) emit(std::false_type{}, it0 + i, pk, sc, hs);
              else emit(std::true_type{}, it0 + i, pk, sc, hs);
            }
            __syncwarp();
          }
        }
      }
      if (!batched) {
        for (int it = 0; it < iters; ++it) {
          uint32_t pk = 0u;
          uint16_t sc = 0;
          if constexpr (COMPRESSED) {
            pk = *packed_ptr(src, C, it, tid);
            sc = *scale_ptr(src, C, it, tid);
          }
          if (whole) emit(std::false_type{}, it, pk, sc, nullptr);
          else emit(std::true_type{}, it, pk, sc, nullptr);
        }
      }
    }
    if (failed) {
      if (lane == 0)
        report_failure(status, kTimeoutBulk, uint32_t(me), 0xffffffffu, epoch, 0u, uint32_t(t.phase), uint32_t(c));
      break;
    }

    // ---- exit (per warp): count this warp in; the last warp of the CTA publishes the task ----
    __syncwarp();
    if (lane == 0) {
      __threadfence_block();
      const int sl = local % kSlots;
      if (atomicAdd(&s_count[sl], 1) == kWarps - 1) {
        s_count[sl] = 0;
        if (t.phase == 1 && GATHER) {
          __threadfence_system();
          for (int r = 0; r < W; ++r)
            st_release_sys(reinterpret_cast<uint32_t*>(p.region[r] + p.flag1_off) + (uint64_t(j) * W + me), epoch);
        } else if (t.phase == 1 && !SINGLE) {
          __threadfence_system();
          st_release_sys(reinterpret_cast<uint32_t*>(p.region[t.o] + p.flag1_off) + (uint64_t(j) * W + me), epoch);
        } else if (t.phase == 2 && !RS && !GATHER) {
          __threadfence_system();
          for (int r = 0; r < W; ++r)
            st_release_sys(reinterpret_cast<uint32_t*>(p.region[(me + 1 + r) % W] + p.flag2_off) + c, epoch);
        }
        __threadfence_block();
        atomicAdd(&s_done, 1);
      }
    }
  }

  // per-rank telemetry: five atomics per CTA
  if (p.stats[vr] != nullptr && COMPRESSED && !LEAN && (pm & 1)) {
    float v[5] = {acc_stats.e2, acc_stats.g2, acc_stats.xp, acc_stats.pp, acc_stats.f2};
#pragma unroll
    for (int k = 0; k < 5; ++k) {
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) v[k] += __shfl_xor_sync(0xffffffffu, v[k], off);
      if (lane == 0) red[k][tid >> 5] = v[k];
    }
    __syncthreads();
    if (tid < 5) {
      float a = 0.0f;
#pragma unroll
      for (int i = 0; i < kWarps; ++i) a += red[tid][i];
      atomicAdd(&p.stats[vr][tid], a);
    }
  }
}

template <typename T, typename S, int MODE>
cudaError_t launch_mode(const NangilaPredResParams& p, cudaStream_t stream) {
  constexpr bool LEAN = MODE == 2 || MODE == 3 || MODE == 5 || MODE == 7;
  constexpr int smem = MODE == 0 ? 0 : kWarps * Ring<T, S, LEAN>::BYTES_PER_WARP;
  static_assert(Ring<T, S, LEAN>::D <= kMaxDepth, "ring depth");
  const void* fn = reinterpret_cast<const void*>(&predres_bucket_kernel<T, S, MODE>);
  // every CTA of a rank must be resident: an owner's wait may depend on a contribution that sits in a
  // CTA which has not started yet
  int grid_x = 0;
  cudaError_t e = clamp_grid(fn, kThreads, size_t(smem), p.grid_x, p.nvr, &grid_x);
  if (e != cudaSuccess) return e;
  dim3 grid{unsigned(grid_x), unsigned(p.nvr)};
  dim3 block{unsigned(kThreads)};
  void* args[] = {const_cast<NangilaPredResParams*>(&p)};
  if (p.nvr > 1) return cudaLaunchCooperativeKernel(fn, grid, block, args, size_t(smem), stream);
  return cudaLaunchKernel(fn, grid, block, args, size_t(smem), stream);
}

template <typename T, typename S>
cudaError_t launch_ts(const NangilaPredResParams& p, cudaStream_t stream) {
  bool lean = p.mode == 0 && p.measure == 0;
  for (int v = 0; v < p.nvr; ++v) lean = lean && p.pred_gain[v] == 0.0f;
  if (p.mode == 0 && p.world == 1) return lean ? launch_mode<T, S, 5>(p, stream) : launch_mode<T, S, 4>(p, stream);
  if (p.mode == 0 && p.gather != 0) return lean ? launch_mode<T, S, 7>(p, stream) : launch_mode<T, S, 6>(p, stream);
  if (p.mode == 0) return lean ? launch_mode<T, S, 3>(p, stream) : launch_mode<T, S, 1>(p, stream);
  if (p.mode == 1) return launch_mode<T, S, 0>(p, stream);
  return launch_mode<T, S, 2>(p, stream);
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
  // gather mode (small worlds): every rank holds all W slots of every chunk, twice (launch parity)
  const bool gather_ok = world >= 2 && world <= NANGILA_GATHER_MAX_WORLD;
  const uint64_t cslot = nangila::compressed_slot_bytes(chunk_elems);
  uint64_t off = 0;
  if (recv1_off) *recv1_off = off;
  off = align(off + std::max<uint64_t>(owned_max * world * slot, gather_ok ? 2 * nchunks * world * cslot : 0));
  if (recv2_off) *recv2_off = off;
  off = align(off + nchunks * slot);
  if (flag1_off) *flag1_off = off;
  off = align(off + std::max<uint64_t>(owned_max, gather_ok ? nchunks : 0) * world * 4);
  if (flag2_off) *flag2_off = off;
  off = align(off + nchunks * 4);
  return off;
}

// Reduce-scatter mode (mode 2): only the phase-1 slots and flags are needed.
extern "C" uint64_t nangila_rs_region_bytes(int64_t n, int32_t world, int32_t chunk_elems, uint64_t* recv1_off,
                                            uint64_t* flag1_off, int32_t* nchunks) {
  auto align = [](uint64_t x) { return (x + 255) & ~uint64_t(255); };
  const int64_t shard = n / world;
  const uint64_t cps = uint64_t((shard + chunk_elems - 1) / chunk_elems);
  if (nchunks) *nchunks = int32_t(cps * world);
  uint64_t off = 0;
  if (recv1_off) *recv1_off = off;
  off = align(off + 2 * cps * world * nangila::compressed_slot_bytes(chunk_elems));
  if (flag1_off) *flag1_off = off;
  off = align(off + cps * world * 4);
  return off;
}

extern "C" int nangila_predres_resident_ctas(void) {
  using namespace nangila;
  // every compressed variant has the same launch bounds and the same 48 KB of dynamic shared memory
  const void* fn = reinterpret_cast<const void*>(&predres_bucket_kernel<__nv_bfloat16, __nv_bfloat16, 3>);
  int resident = 0;
  const size_t smem = size_t(kWarps) * Ring<__nv_bfloat16, __nv_bfloat16, true>::BYTES_PER_WARP;
  if (resident_ctas(fn, kThreads, smem, &resident) != cudaSuccess) return -1;
  return resident;
}

extern "C" int32_t nangila_predres_chunk_elems(int64_t n, int32_t resident) {
  // Each phase walks the chunks in waves of `resident` CTAs. A chunk count just above a multiple of that
  // leaves most of the GPU idle in the last wave (800 chunks on 592 CTAs: 68 % busy), so the chunk size is
  // derived from the wave count instead of being a fixed power of two.
  constexpr int64_t kMaxChunk = 131072, kGrain = 4096;  // an even number of 2048-element iterations
  if (n <= 0) return int32_t(kGrain);
  const int64_t g = resident > 0 ? resident : 1;
  const int64_t waves = std::max<int64_t>(1, (n + g * kMaxChunk - 1) / (g * kMaxChunk));
  const int64_t per = (n + g * waves - 1) / (g * waves);
  const int64_t chunk = std::max(kGrain, (per + kGrain - 1) / kGrain * kGrain);
  return int32_t(std::min(chunk, kMaxChunk));
}

extern "C" int nangila_predres_launch(const NangilaPredResParams* p, cudaStream_t stream) {
  using namespace nangila;
  if (p == nullptr || p->n <= 0 || p->world < 1 || p->world > NANGILA_MAX_RANKS || p->nvr < 1 ||
      p->nvr > NANGILA_MAX_VRANKS || p->rank0 < 0 || p->rank0 + p->nvr > p->world || p->chunk_elems <= 0 ||
      p->chunk_elems % kElemsPerIter != 0 || p->epoch == 0 || p->mode < 0 || p->mode > 2 ||
      !(p->mu >= 0.0f && p->mu <= 1.0f) || p->phase_mask < 0 || p->phase_mask > 7 || p->phase_mask == 5)
    return int(cudaErrorInvalidValue);
  if (p->mode == 2) {
    // reduce-scatter: W equal shards whose length keeps 16-byte vector accesses aligned
    if (p->n % p->world != 0 || (p->n / p->world) % 8 != 0) return int(cudaErrorInvalidValue);
    const int64_t shard = p->n / p->world;
    if (p->nchunks != int32_t(p->world * ((shard + p->chunk_elems - 1) / p->chunk_elems)))
      return int(cudaErrorInvalidValue);
    for (int v = 0; v < p->nvr; ++v)
      if (p->out_shard[v] == nullptr) return int(cudaErrorInvalidValue);
  } else if (p->nchunks != int32_t((p->n + p->chunk_elems - 1) / p->chunk_elems)) {
    return int(cudaErrorInvalidValue);
  }
  if (p->nvr > 1 && p->nvr != p->world) return int(cudaErrorInvalidValue);
  if (p->gather != 0 && (p->world < 2 || p->world > NANGILA_GATHER_MAX_WORLD)) return int(cudaErrorInvalidValue);
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
