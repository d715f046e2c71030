// PowerSGD on Blackwell tensor cores (sm_100a).
//
// For one gradient matrix M (m x n, row-major; M = gradient + error memory, bf16) and rank r <= 16:
//   prep         M <- bf16(grad + error memory)
//   GEMM A       P_local  = M  * Q        (m x 16)   tcgen05.mma, A = M  tiles (K-major),  B = Q^T (16 x n)
//   exchange     P = mean over ranks of P_local; Gram-Schmidt on the columns of P (in-kernel)
//   GEMM B       Q'_local = M^T * P       (n x 16)   tcgen05.mma, A = M^T tiles (MN-major), B = P^T (16 x m)
//   exchange     Q' = mean over ranks of Q'_local; orthonormalised copy kept as the next warm start
//   reconstruct  grad <- P Q'^T ; error memory <- M - P Q'^T
// Both GEMMs run as 128 x 16 output tiles: operands are staged in shared memory by TMA
// (cp.async.bulk.tensor, 128-byte swizzle, no cluster multicast) through a 4-stage mbarrier pipeline,
// one elected thread issues tcgen05.mma with the accumulator in tensor memory, and the epilogue reads
// it back with tcgen05.ld. M is read straight from its row-major storage in both GEMMs: the second
// one feeds the tensor core an MN-major A operand instead of materialising a transpose.
// The exchanges store each rank's factor into every rank's slot over NVLink and every rank then adds
// the W slots in rank order, so all replicas hold bit-identical P and Q'.
//
// What it replaces in the reference: PowerSGDCompressor::compress / decompress
// (nangila-core/src/power_sgd.rs:46-193: ndarray GEMMs on the host, per-rank factors shipped and W
// dense reconstructions averaged). Here P and Q' are averaged across ranks (standard PowerSGD).
#include <algorithm>
#include <cstring>
#include <cooperative_groups.h>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "nangila_kernels.h"
#include "ptx_sm100.cuh"
#include "quant.cuh"
#include "signal.cuh"

namespace nangila {
namespace {
namespace cg = cooperative_groups;

using namespace sm100;
using namespace comm;

constexpr int kTileRows = 128;   // UMMA M
constexpr int kCols = 16;        // UMMA N: rank padded to 16
constexpr int kSlabK = 64;       // bf16 elements per 128-byte swizzle row
constexpr int kStages = 4;
constexpr int kABytes = kTileRows * kSlabK * 2;  // 16 KiB
constexpr int kBBytes = kCols * kSlabK * 2;      // 2 KiB
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kGemmThreads = 128;
constexpr int kTmemCols = 32;
constexpr int kGemmSmem = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers and flags*/;

// One CTA computes out[row0 .. row0+127][0..15] (+)= sum over its K range.
//  A_MN = false: tmA is a map of M (inner dim = K), box {64, 128}; the A stage is one box.
//  A_MN = true : tmA is a map of M whose inner dim is the OUTPUT row dimension, box {64, 64}; the A
//                stage is two boxes (output rows 0..63 and 64..127) of 64 K-rows each.
//  tmB always maps B^T (16 x K, inner dim = K), box {64, 16}.
template <bool A_MN>
__global__ void __launch_bounds__(kGemmThreads)
psgd_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 float* __restrict__ out, int rows_out, int k_total, int k_per_split, int use_atomics,
                 uint32_t* status, uint64_t timeout_ns, const __grid_constant__ NangilaPsgdPush push) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
  uint64_t* empty = full + kStages;
  uint64_t* accum_done = empty + kStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_done + 1);
  uint32_t* failed = tmem_slot + 1;
  uint32_t* last_of_tile = failed + 1;   // this CTA completed its row tile (epilogue push)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row0 = blockIdx.x * kTileRows;
  const int k_begin = blockIdx.y * k_per_split;
  const int k_end = min(k_total, k_begin + k_per_split);
  const int nslabs = (k_end - k_begin + kSlabK - 1) / kSlabK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(accum_done, 1);
    *failed = 0;
    fence_barrier_init();
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmB);
  }
  if (warp == 0) tmem_alloc(tmem_slot, kTmemCols);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (nslabs > 0) {
    if (warp == 0 && lane == 0) {
      // ---------------- TMA producer ----------------
      for (int i = 0; i < nslabs; ++i) {
        const int s = i % kStages;
        if (i >= kStages && !mbar_wait(&empty[s], uint32_t((i / kStages - 1) & 1), timeout_ns)) {
          *failed = 1;
          break;
        }
        uint8_t* a_dst = smem + s * kStageBytes;
        uint8_t* b_dst = a_dst + kABytes;
        const int k0 = k_begin + i * kSlabK;
        mbar_arrive_expect_tx(&full[s], kStageBytes);
        if (A_MN) {
          tma_load_2d(a_dst, &tmA, row0, k0, &full[s]);
          tma_load_2d(a_dst + kABytes / 2, &tmA, row0 + 64, k0, &full[s]);
        } else {
          tma_load_2d(a_dst, &tmA, k0, row0, &full[s]);
        }
        tma_load_2d(b_dst, &tmB, k0, 0, &full[s]);
      }
    } else if (warp == 1 && lane == 0) {
      // ---------------- MMA issuer ----------------
      constexpr uint32_t idesc = make_idesc_bf16(kTileRows, kCols, A_MN, false);
      bool ok = true;
      for (int i = 0; i < nslabs && ok; ++i) {
        const int s = i % kStages;
        if (!mbar_wait(&full[s], uint32_t((i / kStages) & 1), timeout_ns)) {
          *failed = 1;
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t a_addr = smem_u32(smem + s * kStageBytes);
        const uint32_t b_addr = a_addr + kABytes;
#pragma unroll
        for (int kk = 0; kk < kSlabK / 16; ++kk) {
          // K-major: 16 elements along K = 32 bytes inside the swizzle row.
          // MN-major: 16 K-rows = two groups of 8 rows of 128 bytes.
          const uint64_t a_desc = A_MN ? make_smem_desc(a_addr + kk * 2048, kABytes / 2, 1024)
                                       : make_smem_desc(a_addr + kk * 32, 16, 1024);
          const uint64_t b_desc = make_smem_desc(b_addr + kk * 32, 16, 1024);
          umma_bf16(tmem_base, a_desc, b_desc, idesc, (i > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&empty[s]);  // frees the stage once these MMAs have read it
      }
      if (ok) umma_commit(accum_done);
    }
    __syncwarp();
    // ---------------- epilogue: all four warps ----------------
    bool ok = mbar_wait(accum_done, 0, timeout_ns);
    if (*reinterpret_cast<volatile uint32_t*>(failed) != 0u) ok = false;
    ok = __all_sync(0xffffffffu, ok);  // tcgen05.ld needs the whole warp
    if (ok) {
      tc_fence_after_sync();
      float v[16];
      tmem_ld_32x32b_x16(tmem_base + (uint32_t(warp * 32) << 16), v);
      const int row = row0 + warp * 32 + lane;
      if (row < rows_out) {
        float* dst = out + int64_t(row) * kCols;
        if (use_atomics) {
#pragma unroll
          for (int c = 0; c < kCols; ++c) atomicAdd(dst + c, v[c]);
        } else {
#pragma unroll
          for (int c = 0; c < kCols; c += 4) *reinterpret_cast<float4*>(dst + c) = make_float4(v[c], v[c + 1], v[c + 2], v[c + 3]);
        }
      }
    } else if (threadIdx.x == 0) {
      report_failure(status, kTimeoutGrid, 0u, 0xffffffffu, 0u, 0u, 7u, uint32_t(blockIdx.x));
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, kTmemCols);

  // ---------------- exchange started from the epilogue ----------------
  // Whichever of a tile's K splits arrives last finds the complete tile in `out` (its own part went there above,
  // the others' were fenced before they counted themselves in) and stores it into every rank's slot for this
  // rank. A CTA whose pipeline failed still counts itself in, so that nobody waits for it; the status block says
  // that the data is not to be trusted.
  if (push.counters != nullptr) {
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) *last_of_tile = atomicAdd(&push.counters[blockIdx.x], 1u) == gridDim.y - 1 ? 1u : 0u;
    __syncthreads();
    if (*last_of_tile != 0u) {
      __threadfence();
      const uint32_t epoch = push.epoch_dev != nullptr ? *push.epoch_dev : push.epoch;
      const int W = push.world, r = push.rank;
      const uint64_t slot_bytes = (uint64_t(rows_out) * r * 4 + 255) & ~uint64_t(255);
      const uint64_t base = push.recv_off + uint64_t(epoch & 1u) * W * slot_bytes + uint64_t(push.me) * slot_bytes;
      const int row = row0 + warp * 32 + lane;
      if (row < rows_out) {
        float v[kCols];
#pragma unroll
        for (int c = 0; c < kCols; c += 4) {
          const float4 a = __ldcg(reinterpret_cast<const float4*>(out + int64_t(row) * kCols + c));
          v[c] = a.x; v[c + 1] = a.y; v[c + 2] = a.z; v[c + 3] = a.w;
        }
        for (int d = 0; d < W; ++d) {
          float* dst = reinterpret_cast<float*>(push.region[(push.me + d) % W] + base);
          for (int c = 0; c < r; ++c) dst[int64_t(c) * rows_out + row] = v[c];   // adjacent rows: adjacent addresses
        }
      }
      __threadfence_system();
      __syncthreads();
      if (threadIdx.x == 0) {
        const uint32_t tiles = gridDim.x;
        if (atomicAdd(&push.counters[tiles], 1u) == tiles - 1) {
          __threadfence_system();  // every tile's stores were fenced before its CTA counted itself in
          for (int d = 0; d < W; ++d)
            st_release_sys(reinterpret_cast<uint32_t*>(push.region[d] + push.flag_off) + push.me, epoch);
        }
      }
    }
  }
}

// ---- prep / reconstruct (element-wise) -----------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) psgd_prep_kernel(const T* __restrict__ grad, const __nv_bfloat16* __restrict__ ef,
                                                       __nv_bfloat16* __restrict__ mef, int64_t numel,
                                                       float* __restrict__ z0, int64_t n0, float* __restrict__ z1,
                                                       int64_t n1) {
  const int64_t t0 = int64_t(blockIdx.x) * 256 + threadIdx.x, stride = int64_t(gridDim.x) * 256;
  for (int64_t i = t0; i < numel; i += stride)
    mef[i] = __float2bfloat16_rn(dev::sanitize(dev::Vec16<T>::to_float(grad[i])) + __bfloat162float(ef[i]));
  // the two projections accumulate into these with atomics (split K): clear them here, not in launches of their own
  for (int64_t i = t0; i < n0; i += stride) z0[i] = 0.0f;
  for (int64_t i = t0; i < n1; i += stride) z1[i] = 0.0f;
}
// grad = P Q^T (rank r), ef = (m + ef) - grad. P and Q are the averaged factors, COLUMN-major
// (P[k * m + row], Q[k * n + col]). Each thread owns 8 consecutive columns and walks down the rows of
// its CTA's share; for r <= 4 its 8 x r slice of Q stays in registers, so per row it reads 16 bytes of
// m + ef and r broadcast values of P and writes the 8 results twice (bucket, error memory).
template <typename T, int RQ>
__global__ void __launch_bounds__(256) psgd_reconstruct_kernel(T* __restrict__ grad, __nv_bfloat16* __restrict__ ef,
                                                              const __nv_bfloat16* __restrict__ mef,
                                                              const float* __restrict__ P, const float* __restrict__ Q,
                                                              int m, int n, int r) {
  const int col = (blockIdx.x * 256 + threadIdx.x) * 8;
  if (col >= n) return;  // n is a multiple of 8
  float q[RQ > 0 ? RQ : 1][8];
  if constexpr (RQ > 0) {
#pragma unroll
    for (int k = 0; k < RQ; ++k) {
      if (k < r) dev::Vec8<float>::load(Q + int64_t(k) * n + col, q[k]);
      else {
#pragma unroll
        for (int j = 0; j < 8; ++j) q[k][j] = 0.0f;
      }
    }
  }
  for (int row = blockIdx.y; row < m; row += gridDim.y) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
    if constexpr (RQ > 0) {
#pragma unroll
      for (int k = 0; k < RQ; ++k) {
        const float pk = k < r ? P[int64_t(k) * m + row] : 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = __fmaf_rn(pk, q[k][j], acc[j]);
      }
    } else {
      for (int k = 0; k < r; ++k) {
        const float pk = P[int64_t(k) * m + row];
        float qk[8];
        dev::Vec8<float>::load(Q + int64_t(k) * n + col, qk);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = __fmaf_rn(pk, qk[j], acc[j]);
      }
    }
    const int64_t i = int64_t(row) * n + col;
    float x[8], o[8];
    dev::Vec8<__nv_bfloat16>::load(mef + i, x);
    // the error memory must see the value as the bucket will hold it (rounded to the bucket's type)
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = dev::Vec16<T>::to_float(dev::Vec16<T>::from_float(acc[j]));
    dev::Vec8<T>::store(grad + i, o);
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] -= o[j];
    dev::Vec8<__nv_bfloat16>::store(ef + i, x);
  }
}

// ---- cross-rank mean of a (rows x 16) factor + orthonormalisation ----------------------------------------
// One thread-block CLUSTER of kXCtas CTAs per rank; every CTA owns a slice of the rows. local: this
// rank's factor as the GEMM leaves it (rows x 16 fp32, row-major, columns >= r ignored). Everything after
// that is COLUMN-major (element (row, c) at [c * rows + row]) so that every pass is a coalesced stream:
// mean_out (16 x rows fp32): the averaged factor, orthonormalised in place when orth_mean != 0;
// t_out (16 x rows bf16): the orthonormalised averaged factor (rows r..15 zero): the B operand of the
// next GEMM.
// Orthonormalisation is Gram-Schmidt through the Gram matrix (Q = W R^-1 with R^T R = W^T W, the
// Cholesky factor), applied twice ("CholeskyQR2"): each round is one pass that accumulates the r x r Gram
// matrix, a cluster-wide sum over distributed shared memory in a fixed order (every CTA gets the same
// bits), a 16 x 16 factorisation done redundantly by every CTA, and one pass that applies R^-1. A column
// whose pivot vanishes (rank-deficient factor) becomes zero, as a column of norm 0 stays in classical
// Gram-Schmidt. The second round removes the orthogonality loss of the first.
constexpr int kXCtas = 8;
constexpr int kXThreads = 512;
constexpr int kPairs = kCols * (kCols + 1) / 2;

// RMAX: compile-time bound on the rank (4 keeps the 10 pair sums and the row in registers).
template <int RMAX>
__global__ void __launch_bounds__(kXThreads) psgd_exchange_kernel(const __grid_constant__ NangilaPsgdExchangeParams p) {
  constexpr int kAcc = RMAX * (RMAX + 1) / 2;
  cg::cluster_group cluster = cg::this_cluster();
  const int g = int(cluster.block_rank());
  const int vr = blockIdx.x / kXCtas;
  const int me = p.rank0 + vr;
  const int W = p.world, rows = p.rows, r = p.rank;
  const int tid = threadIdx.x;
  const uint64_t slot_bytes = (uint64_t(rows) * r * 4 + 255) & ~uint64_t(255);
  const uint32_t epoch = p.epoch_dev != nullptr ? *p.epoch_dev : p.epoch;
  const uint64_t base = p.recv_off + uint64_t(epoch & 1u) * W * slot_bytes;  // two slot sets, by launch parity
  uint32_t* status = p.status[vr];
  const float* local = p.local[vr];
  float* mean = p.mean_out[vr];
  // this CTA's rows
  const int per = (rows + kXCtas - 1) / kXCtas;
  const int r0 = min(rows, g * per), r1 = min(rows, r0 + per);
  __shared__ float s_warp[kXThreads / 32][kPairs];  // per-warp partial sums (summed in warp order: no float atomics)
  __shared__ float s_part[kPairs];          // this CTA's partial Gram matrix (lower triangle, packed)
  __shared__ float s_gram[kPairs];          // cluster-wide sum
  __shared__ float s_rinv[kCols][kCols];    // R^-1 (upper triangular); a zero column for a vanished pivot
  __shared__ int s_ok;

  // 1. store my rows of my factor (r columns, column-major) into every rank's slot [me] (unless the GEMM's
  //    epilogue has done that already)
  if (p.pushed == 0) {
    for (int d = 0; d < W; ++d) {
      float* dst = reinterpret_cast<float*>(p.region[(me + d) % W] + base + uint64_t(me) * slot_bytes);
      for (int c = 0; c < r; ++c)
        for (int i = r0 + tid; i < r1; i += kXThreads) dst[int64_t(c) * rows + i] = local[int64_t(i) * kCols + c];
    }
    __threadfence_system();
  }
  cluster.sync();
  if (p.pushed == 0 && g == 0 && tid < W) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint32_t*>(p.region[tid] + p.flag_off) + me, epoch);
  }
  // 2. wait for every rank's factor (every CTA polls for itself; on failure all of them still take part in
  //    the cluster barriers below, doing no work)
  if (tid == 0) s_ok = 1;
  __syncthreads();
  if (tid < W) {
    if (!wait_flag(reinterpret_cast<const uint32_t*>(p.region[me] + p.flag_off) + tid, epoch, p.timeout_ns, status,
                   kTimeoutPhase2, uint32_t(me), uint32_t(tid), 8u, 0u))
      s_ok = 0;
  }
  __syncthreads();
  const bool ok = s_ok != 0;
  // 3. mean in rank order (identical on every rank); columns >= r are zero
  float* work = p.orth_mean ? mean : p.scratch[vr];
  if (ok) {
    const float inv_w = 1.0f / float(W);
    for (int c = 0; c < kCols; ++c)
      for (int i = r0 + tid; i < r1; i += kXThreads) {
        float acc = 0.0f;
        if (c < r)
          for (int src = 0; src < W; ++src)
            acc += reinterpret_cast<const float*>(p.region[me] + base + uint64_t(src) * slot_bytes)[int64_t(c) * rows + i];
        acc *= inv_w;
        mean[int64_t(c) * rows + i] = acc;
        if (!p.orth_mean && c < r) work[int64_t(c) * rows + i] = acc;
      }
  }
  __syncthreads();
  // 4. two rounds of Cholesky-QR on `work`
  for (int round = 0; round < 2; ++round) {
    for (int i = tid; i < (kXThreads / 32) * kPairs; i += kXThreads) (&s_warp[0][0])[i] = 0.0f;
    __syncthreads();
    if (ok) {
      // every thread owns whole rows: all pair products of a row come from registers
      float acc[kAcc];
#pragma unroll
      for (int q = 0; q < kAcc; ++q) acc[q] = 0.0f;
      for (int i = r0 + tid; i < r1; i += kXThreads) {
        float w[RMAX];
#pragma unroll
        for (int c = 0; c < RMAX; ++c) w[c] = c < r ? work[int64_t(c) * rows + i] : 0.0f;
        int q = 0;
#pragma unroll
        for (int c = 0; c < RMAX; ++c)
#pragma unroll
          for (int j = 0; j <= c; ++j, ++q) acc[q] = __fmaf_rn(w[c], w[j], acc[q]);
      }
#pragma unroll
      for (int q = 0; q < kAcc; ++q) {
        float v = acc[q];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        if ((tid & 31) == 0) s_warp[tid >> 5][q] = v;
      }
    }
    __syncthreads();
    for (int q = tid; q < kPairs; q += kXThreads) {
      float v = 0.0f;
      for (int w = 0; w < kXThreads / 32; ++w) v += s_warp[w][q];  // fixed order: the same bits on every rank
      s_part[q] = v;
    }
    cluster.sync();  // every CTA's partial matrix is complete
    for (int q = tid; q < kPairs; q += kXThreads) {
      float v = 0.0f;
      for (int b = 0; b < kXCtas; ++b) v += *cluster.map_shared_rank(&s_part[q], b);  // fixed order
      s_gram[q] = v;
    }
    __syncthreads();
    if (tid == 0) {
      // Cholesky of the r x r Gram matrix: L L^T; then R^-1 = (L^T)^-1 by back substitution
      float L[kCols][kCols];
      bool dead[kCols];
      for (int c = 0; c < r; ++c) {
        for (int j = 0; j <= c; ++j) {
          float sum = s_gram[c * (c + 1) / 2 + j];
          for (int k = 0; k < j; ++k) sum -= L[c][k] * L[j][k];
          if (j < c) {
            L[c][j] = dead[j] ? 0.0f : sum / L[j][j];
          } else {
            const float diag = s_gram[c * (c + 1) / 2 + c];
            dead[c] = !(sum > 1e-20f) || !(sum > 1e-7f * diag);  // pivot vanished: dependent (or zero) column
            L[c][c] = dead[c] ? 1.0f : sqrtf(sum);
          }
        }
      }
      // X = R^-1 where R = L^T (upper triangular): X[j][c] for j <= c
      for (int c = 0; c < kCols; ++c)
        for (int j = 0; j < kCols; ++j) s_rinv[j][c] = 0.0f;
      for (int c = 0; c < r; ++c) {
        if (dead[c]) continue;  // column of zeros
        s_rinv[c][c] = 1.0f / L[c][c];
        for (int j = c - 1; j >= 0; --j) {
          if (dead[j]) continue;
          float sum = 0.0f;
          for (int k = j + 1; k <= c; ++k) sum += L[k][j] * s_rinv[k][c];  // R[j][k] = L[k][j]
          s_rinv[j][c] = -sum / L[j][j];
        }
      }
    }
    __syncthreads();
    if (ok) {
      for (int i = r0 + tid; i < r1; i += kXThreads) {
        float w[RMAX];
#pragma unroll
        for (int c = 0; c < RMAX; ++c) w[c] = c < r ? work[int64_t(c) * rows + i] : 0.0f;
#pragma unroll
        for (int c = 0; c < RMAX; ++c) {
          if (c < r) {
            float o = 0.0f;
#pragma unroll
            for (int j = 0; j <= c; ++j) o = __fmaf_rn(w[j], s_rinv[j][c], o);
            work[int64_t(c) * rows + i] = o;
          }
        }
      }
    }
    cluster.sync();  // nobody reads a neighbour's s_part after this; safe to clear it in the next round
  }
  // 5. bf16 copy for the next GEMM's B operand (same layout)
  if (ok) {
    __nv_bfloat16* t_out = static_cast<__nv_bfloat16*>(p.t_out[vr]);
    for (int c = 0; c < kCols; ++c)
      for (int i = r0 + tid; i < r1; i += kXThreads)
        t_out[int64_t(c) * rows + i] = __float2bfloat16_rn(c < r ? work[int64_t(c) * rows + i] : 0.0f);
  }
}

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn encode_fn() {
  static EncodeFn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess) f = nullptr;
    return reinterpret_cast<EncodeFn>(f);
  }();
  return fn;
}
// bf16 matrix with `inner` contiguous elements per row, `outer` rows, row pitch in elements.
bool make_map(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer, uint64_t pitch_elems, uint32_t box_inner,
              uint32_t box_outer) {
  EncodeFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {pitch_elems * 2};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int pick_splits(int tiles, int k_total) {
  int want = 148 / (tiles > 0 ? tiles : 1);
  int max_splits = (k_total + 4 * kSlabK - 1) / (4 * kSlabK);  // at least four slabs per split
  int s = want < 1 ? 1 : (want > max_splits ? max_splits : want);
  return s < 1 ? 1 : s;
}

}  // namespace
}  // namespace nangila

// out (rows x 16 fp32) = M * Bt^T  (transposed = 0: M is m x n, rows = m, contraction over n;
// transposed = 1: out = M^T * Bt^T, rows = n, contraction over m). Bt is 16 x K bf16, K contiguous.
// `out` must be zero-filled when the launch splits K (it always may: zero it).
extern "C" int nangila_psgd_gemm(const void* M, int32_t m, int32_t n, const void* Bt, int32_t transposed, float* out,
                                 uint32_t* status, uint64_t timeout_ns, cudaStream_t stream) {
  return nangila_psgd_gemm_push(M, m, n, Bt, transposed, out, nullptr, status, timeout_ns, stream);
}

extern "C" int nangila_psgd_gemm_push(const void* M, int32_t m, int32_t n, const void* Bt, int32_t transposed, float* out,
                                      const NangilaPsgdPush* push_in, uint32_t* status, uint64_t timeout_ns,
                                      cudaStream_t stream) {
  using namespace nangila;
  NangilaPsgdPush push;
  std::memset(&push, 0, sizeof push);
  if (push_in != nullptr) {
    push = *push_in;
    if (push.counters == nullptr || push.world < 1 || push.world > NANGILA_MAX_RANKS || push.me < 0 || push.me >= push.world ||
        push.rank < 1 || push.rank > 16 || (push.epoch == 0 && push.epoch_dev == nullptr))
      return int(cudaErrorInvalidValue);
    for (int r = 0; r < push.world; ++r)
      if (push.region[r] == nullptr) return int(cudaErrorInvalidValue);
  }
  if (!M || !Bt || !out || !status || m <= 0 || n <= 0 || (n % 8) != 0 || (m % 8) != 0 ||
      (reinterpret_cast<uintptr_t>(M) & 15u) || (reinterpret_cast<uintptr_t>(Bt) & 15u) ||
      (reinterpret_cast<uintptr_t>(out) & 15u))
    return int(cudaErrorInvalidValue);
  CUtensorMap tmA, tmB;
  const int rows = transposed ? n : m;
  const int k_total = transposed ? m : n;
  bool ok;
  if (transposed) ok = make_map(&tmA, M, uint64_t(n), uint64_t(m), uint64_t(n), 64, 64);   // inner = output rows
  else ok = make_map(&tmA, M, uint64_t(n), uint64_t(m), uint64_t(n), 64, 128);             // inner = K
  ok = ok && make_map(&tmB, Bt, uint64_t(k_total), 16, uint64_t(k_total), 64, 16);
  if (!ok) return int(cudaErrorNotSupported);
  const int tiles = (rows + kTileRows - 1) / kTileRows;
  const int splits = pick_splits(tiles, k_total);
  int k_per_split = (k_total + splits - 1) / splits;
  k_per_split = (k_per_split + kSlabK - 1) / kSlabK * kSlabK;
  const int nsplit = (k_total + k_per_split - 1) / k_per_split;
  dim3 grid{unsigned(tiles), unsigned(nsplit), 1u}, block{unsigned(kGemmThreads), 1u, 1u};
  cudaError_t e;
  if (transposed) {
    static bool attr1 = false;
    if (!attr1) {
      cudaFuncSetAttribute(psgd_gemm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmem);
      attr1 = true;
    }
    psgd_gemm_kernel<true><<<grid, block, kGemmSmem, stream>>>(tmA, tmB, out, rows, k_total, k_per_split, nsplit > 1, status,
                                                              timeout_ns, push);
  } else {
    static bool attr0 = false;
    if (!attr0) {
      cudaFuncSetAttribute(psgd_gemm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmem);
      attr0 = true;
    }
    psgd_gemm_kernel<false><<<grid, block, kGemmSmem, stream>>>(tmA, tmB, out, rows, k_total, k_per_split, nsplit > 1, status,
                                                               timeout_ns, push);
  }
  e = cudaGetLastError();
  return int(e);
}

extern "C" int nangila_psgd_prep(const void* grad, int32_t dtype, const void* ef, void* mef, int64_t numel, float* z0,
                                 int64_t n0, float* z1, int64_t n1,
                                 cudaStream_t stream) {
  using namespace nangila;
  if (!grad || !ef || !mef || numel <= 0) return int(cudaErrorInvalidValue);
  const int blocks = int(std::min<int64_t>((numel + 255) / 256, 148 * 8));
  auto* e = static_cast<const __nv_bfloat16*>(ef);
  auto* o = static_cast<__nv_bfloat16*>(mef);
  switch (dtype) {
    case NANGILA_F32: psgd_prep_kernel<float><<<blocks, 256, 0, stream>>>(static_cast<const float*>(grad), e, o, numel, z0, n0, z1, n1); break;
    case NANGILA_BF16: psgd_prep_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(grad), e, o, numel, z0, n0, z1, n1); break;
    case NANGILA_F16: psgd_prep_kernel<__half><<<blocks, 256, 0, stream>>>(static_cast<const __half*>(grad), e, o, numel, z0, n0, z1, n1); break;
    default: return int(cudaErrorInvalidValue);
  }
  return int(cudaGetLastError());
}

extern "C" int nangila_psgd_reconstruct(void* grad, int32_t dtype, void* ef, const void* mef, const float* P,
                                        const float* Q, int32_t m, int32_t n, int32_t r, cudaStream_t stream) {
  using namespace nangila;
  if (!grad || !ef || !mef || !P || !Q || m <= 0 || n <= 0 || r <= 0 || r > 16) return int(cudaErrorInvalidValue);
  if (n % 8 != 0) return int(cudaErrorInvalidValue);
  const unsigned gx = unsigned((n / 8 + 255) / 256);
  const unsigned gy = unsigned(std::max<int64_t>(1, std::min<int64_t>(m, (148 * 8 + gx - 1) / gx)));
  const dim3 grid{gx, gy};
  auto* e = static_cast<__nv_bfloat16*>(ef);
  auto* f = static_cast<const __nv_bfloat16*>(mef);
#define NANGILA_RECON(T, RQ) psgd_reconstruct_kernel<T, RQ><<<grid, 256, 0, stream>>>(static_cast<T*>(grad), e, f, P, Q, m, n, r)
  switch (dtype) {
    case NANGILA_F32: if (r <= 4) NANGILA_RECON(float, 4); else NANGILA_RECON(float, 0); break;
    case NANGILA_BF16: if (r <= 4) NANGILA_RECON(__nv_bfloat16, 4); else NANGILA_RECON(__nv_bfloat16, 0); break;
    case NANGILA_F16: if (r <= 4) NANGILA_RECON(__half, 4); else NANGILA_RECON(__half, 0); break;
    default: return int(cudaErrorInvalidValue);
  }
#undef NANGILA_RECON
  return int(cudaGetLastError());
}

extern "C" uint64_t nangila_psgd_exchange_region_bytes(int32_t rows, int32_t rank, int32_t world, uint64_t* recv_off,
                                                       uint64_t* flag_off) {
  auto align = [](uint64_t x) { return (x + 255) & ~uint64_t(255); };
  const uint64_t slot = align(uint64_t(rows) * rank * 4);
  uint64_t off = 0;
  if (recv_off) *recv_off = off;
  off = align(off + 2 * uint64_t(world) * slot);
  if (flag_off) *flag_off = off;
  off = align(off + uint64_t(world) * 4);
  return off;
}

extern "C" int nangila_psgd_exchange(const NangilaPsgdExchangeParams* p, cudaStream_t stream) {
  using namespace nangila;
  if (!p || p->rows <= 0 || p->rank <= 0 || p->rank > 16 || p->world < 1 || p->world > NANGILA_MAX_RANKS || p->nvr < 1 ||
      p->nvr > NANGILA_MAX_VRANKS || (p->nvr > 1 && p->nvr != p->world) || (p->epoch == 0 && p->epoch_dev == nullptr))
    return int(cudaErrorInvalidValue);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3{unsigned(p->nvr * kXCtas), 1u, 1u};
  cfg.blockDim = dim3{unsigned(kXThreads), 1u, 1u};
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  attrs[0].id = cudaLaunchAttributeClusterDimension;
  attrs[0].val.clusterDim.x = kXCtas;
  attrs[0].val.clusterDim.y = 1;
  attrs[0].val.clusterDim.z = 1;
  // several emulated ranks in one launch wait for one another: ask for a cooperative launch so that
  // all their clusters are resident together
  attrs[1].id = cudaLaunchAttributeCooperative;
  attrs[1].val.cooperative = 1;
  cfg.attrs = attrs;
  cfg.numAttrs = p->nvr > 1 ? 2 : 1;
  const NangilaPsgdExchangeParams params = *p;
  cudaError_t e = p->rank <= 4 ? cudaLaunchKernelEx(&cfg, psgd_exchange_kernel<4>, params)
                               : cudaLaunchKernelEx(&cfg, psgd_exchange_kernel<kCols>, params);
  return int(e);
}
