// C interface of libnangila_kernels.so: every sm_100a kernel of the framework behind a plain C
// launcher that takes raw device pointers and a stream, so it can be driven from the torch glue,
// from ctypes, or from another runtime. All launchers return a cudaError_t value (0 = success);
// none of them allocates, frees or synchronizes.
#pragma once
#include <cuda_runtime_api.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NANGILA_MAX_RANKS 16   /* ranks in one exchange group */
#define NANGILA_GATHER_MAX_WORLD 4
#define NANGILA_MAX_VRANKS 8   /* ranks emulated inside ONE launch (single-GPU loopback world) */

enum NangilaDType { NANGILA_F32 = 0, NANGILA_F16 = 1, NANGILA_BF16 = 2 };

/* ---- fused prediction-residual bucket exchange -------------------------------------------------
 * One launch per gradient bucket does, for every rank r of the group:
 *   phase 1  e = g + ef - kappa g_hat,  g_hat = curr + mu (curr - prev); block-INT4 quantize e; store the
 *            packed chunk into the chunk owner's receive slot over NVLink; ef <- e - deq(q)
 *   phase 2  (owner of a chunk) wait for all ranks' slots, dequantize-accumulate, average, add the
 *            owner's second error memory, re-quantize, store the result into every rank's slot
 *   phase 3  wait for the reduced chunk, out = mean(kappa) g_hat + deq; write the bucket and the new history.
 * mode 1 (uncompressed) moves the raw values instead and produces the exact mean; it is used for
 * warm-up, Safe-Mode fallback and forced re-synchronisation, and also maintains the history.
 *
 * Multi-GPU: nvr = 1, rank0 = this rank, `region[r]` = rank r's mapping of the bucket's symmetric
 * region. Single-GPU loopback: nvr = world, rank0 = 0, grid.y = nvr, launched cooperatively.
 * grid_x is clamped to the number of CTAs of the chosen variant that the device can hold at once
 * (occupancy x SM count, divided by nvr); grid_x <= 0 asks for exactly that number.
 */
typedef struct NangilaPredResParams {
  void* grad[NANGILA_MAX_VRANKS];      /* in/out: bucket, n elements of grad_dtype */
  void* prev[NANGILA_MAX_VRANKS];      /* in: g(t-1); out: new g(t) (caller swaps prev/curr after) */
  void* curr[NANGILA_MAX_VRANKS];      /* in: g(t) */
  void* ef[NANGILA_MAX_VRANKS];        /* in/out: error feedback, n elements of state_dtype (may be NULL) */
  void* ef2[NANGILA_MAX_VRANKS];       /* in/out: owner-side error memory, owned_chunks*chunk elems (may be NULL) */
  float* stats[NANGILA_MAX_VRANKS];    /* += {sum e^2, sum g^2, <g+ef, g_hat>, <g_hat, g_hat>, sum ef_new^2}; >= 8 floats; may be NULL */
  uint32_t* status[NANGILA_MAX_VRANKS];/* 8 words, see comm/signal.cuh; must be zero before launch */
  uint8_t* region[NANGILA_MAX_RANKS];  /* symmetric region of every rank of the group */
  uint64_t recv1_off, recv2_off, flag1_off, flag2_off; /* byte offsets inside a region */
  int64_t n;                           /* elements in the bucket */
  int32_t world, rank0, nvr;
  int32_t chunk_elems;                 /* multiple of 2048 */
  int32_t nchunks;                     /* ceil(n / chunk_elems) */
  int32_t grad_dtype, state_dtype;     /* NangilaDType; state is F32 or BF16 */
  int32_t mode;                        /* 0 compressed all-reduce, 1 exact all-reduce, 2 compressed reduce-scatter */
  int32_t stochastic;                  /* 0: round to nearest (tests), 1: stochastic rounding */
  int32_t measure;                     /* 1: accumulate <g+ef,g_hat>, <g_hat,g_hat> even when the gain is 0 */
  int32_t gather;                      /* 1 (compressed all-reduce, 2 <= world <= NANGILA_GATHER_MAX_WORLD): every rank
                                          receives every rank's packed chunks and sums them itself: one
                                          quantization and two phases instead of two and three */
  int32_t uniform_gain;                /* 1: every rank of the group passes the same pred_gain (the host
                                          keeps the controllers in step), so phase 3 need not read the
                                          owner's mean from the chunk trailer before fetching the history */
  uint32_t epoch;                      /* strictly increasing per launch on this bucket, never 0 */
  uint32_t seed, step, bucket_id;
  float mu;
  float pred_gain[NANGILA_MAX_VRANKS]; /* kappa in [0,1]: e = g + ef - kappa * g_hat; ranks may differ, the
                                          reconstruction uses the mean of all ranks' values */
  uint64_t timeout_ns;
  int32_t grid_x;                      /* CTAs per rank */
  void* out_shard[NANGILA_MAX_VRANKS]; /* mode 2: n / world elements of grad_dtype, this rank's reduced shard */
  float out_scale;                     /* mode 2: result = sum of all ranks' values * out_scale (1/W for a mean) */
  int32_t phase_mask;                  /* 0 or 7: all phases in this launch. Otherwise a contiguous set of bits
                                          (1: phase 1, 2: phase 2, 4: phase 3): the launch runs only those phases
                                          of the epoch. The caller queues the remaining phases of the same epoch
                                          later on the same stream with otherwise identical parameters, which lets
                                          it put other buckets' non-waiting phase 1 in between. */
  int32_t skip_history;                /* 1: do not write the new history (allowed while the gain is 0 and no probe
                                          is near: nothing reads it); the caller still swaps prev / curr */
} NangilaPredResParams;

/* Bytes one rank's symmetric region must have for a bucket. */
uint64_t nangila_predres_region_bytes(int64_t n, int32_t world, int32_t chunk_elems, int32_t grad_dtype,
                                      uint64_t* recv1_off, uint64_t* recv2_off, uint64_t* flag1_off,
                                      uint64_t* flag2_off);
uint64_t nangila_rs_region_bytes(int64_t n, int32_t world, int32_t chunk_elems, uint64_t* recv1_off,
                                 uint64_t* flag1_off, int32_t* nchunks);
int nangila_predres_launch(const NangilaPredResParams* p, cudaStream_t stream);
/* CTAs of the compressed variants that the current device holds at once (occupancy x SM count): what a host
 * sizes chunks against so that every phase is a whole number of equally loaded waves. <= 0 on error. */
int nangila_predres_resident_ctas(void);
/* Chunk size (elements, a multiple of 4096) for a bucket of n elements: the smallest that covers the bucket
 * with at most `waves x resident` chunks, waves = the least that keeps a chunk at or below 131072 elements. */
int32_t nangila_predres_chunk_elems(int64_t n, int32_t resident_ctas);

/* ---- quantizing parameter all-gather (fsdp_ag_dequant.cu) ------------------------------------------------ */
typedef struct NangilaAgParams {
  const void* in_shard[NANGILA_MAX_VRANKS]; /* this rank's shard, shard_elems of dtype */
  void* out_full[NANGILA_MAX_VRANKS];       /* world * shard_elems of dtype */
  uint32_t* status[NANGILA_MAX_VRANKS];
  uint8_t* region[NANGILA_MAX_RANKS];
  uint64_t recv_off, flag_off;
  int64_t shard_elems;                      /* multiple of 8 */
  int32_t world, rank0, nvr, dtype;
  int32_t chunk_elems;                      /* multiple of 2048 */
  int32_t bits;                             /* 8 or 4 */
  uint32_t epoch;
  uint64_t timeout_ns;
  int32_t grid_x;
} NangilaAgParams;
uint64_t nangila_ag_region_bytes(int64_t shard_elems, int32_t world, int32_t chunk_elems, int32_t bits,
                                 uint64_t* recv_off, uint64_t* flag_off);
int nangila_ag_launch(const NangilaAgParams* p, cudaStream_t stream);

/* ---- PowerSGD on tcgen05 tensor cores (powersgd_tcgen05.cu) ------------------------------------------------ */
/* out (rows x 16 fp32, zero-filled by the caller) += M * Bt^T (transposed = 0, rows = m) or M^T * Bt^T
 * (transposed = 1, rows = n). M: m x n bf16 row-major, m and n multiples of 8. Bt: 16 x K bf16. */
int nangila_psgd_gemm(const void* M, int32_t m, int32_t n, const void* Bt, int32_t transposed, float* out,
                      uint32_t* status, uint64_t timeout_ns, cudaStream_t stream);
/* The same GEMM with the cross-rank exchange of its result started from the epilogue: the CTA that completes a
 * 128-row tile of `out` (the last of the tile's K splits to arrive) stores the tile's first `rank` columns, column-major,
 * into slot [me] of EVERY rank's exchange region (peer stores over NVLink, this rank's own region included), and the CTA
 * that completes the last tile releases the flags. nangila_psgd_exchange() is then launched with `pushed = 1` and only
 * waits, averages and orthonormalises. `counters`: tiles + 1 zero words (arrivals per tile, finished tiles). */
typedef struct NangilaPsgdPush {
  uint8_t* region[NANGILA_MAX_RANKS];
  uint64_t recv_off, flag_off;             /* layout of nangila_psgd_exchange_region_bytes(rows, rank, world) */
  int32_t world, me, rank;
  uint32_t epoch;
  const uint32_t* epoch_dev;               /* if not NULL the epoch is read from this device word */
  uint32_t* counters;
} NangilaPsgdPush;
int nangila_psgd_gemm_push(const void* M, int32_t m, int32_t n, const void* Bt, int32_t transposed, float* out,
                           const NangilaPsgdPush* push, uint32_t* status, uint64_t timeout_ns, cudaStream_t stream);
/* mef = grad + ef; also clears z0[0..n0) and z1[0..n1) (the projections' accumulators; either may be NULL / 0) */
int nangila_psgd_prep(const void* grad, int32_t dtype, const void* ef, void* mef, int64_t numel, float* z0, int64_t n0,
                      float* z1, int64_t n1, cudaStream_t stream);
int nangila_psgd_reconstruct(void* grad, int32_t dtype, void* ef, const void* mef, const float* P, const float* Q,
                             int32_t m, int32_t n, int32_t r, cudaStream_t stream);
typedef struct NangilaPsgdExchangeParams {
  const float* local[NANGILA_MAX_VRANKS];   /* rows x 16 fp32: this rank's factor */
  float* mean_out[NANGILA_MAX_VRANKS];      /* rows x 16 fp32: mean over ranks (orthonormalised if orth_mean) */
  float* scratch[NANGILA_MAX_VRANKS];       /* rows x 16 fp32, needed when orth_mean == 0 */
  void* t_out[NANGILA_MAX_VRANKS];          /* 16 x rows bf16: orthonormalised mean, transposed */
  uint32_t* status[NANGILA_MAX_VRANKS];
  uint8_t* region[NANGILA_MAX_RANKS];
  uint64_t recv_off, flag_off;
  int32_t rows, rank, world, rank0, nvr, orth_mean;
  int32_t pushed;                           /* 1: the factors are already in the slots and the flags released (or being
                                               released) by nangila_psgd_gemm_push(); `local` is not read */
  uint32_t epoch;
  uint64_t timeout_ns;
  const uint32_t* epoch_dev;                /* if not NULL the epoch is read from this device word instead of `epoch`:
                                               a launch recorded in a CUDA graph then sees a new epoch at every replay
                                               (the graph increments the word before the first exchange) */
} NangilaPsgdExchangeParams;
uint64_t nangila_psgd_exchange_region_bytes(int32_t rows, int32_t rank, int32_t world, uint64_t* recv_off,
                                            uint64_t* flag_off);
int nangila_psgd_exchange(const NangilaPsgdExchangeParams* p, cudaStream_t stream);

/* ---- fused DGC exchange (see dgc_fused.cu) ------------------------------------------------------------
 * u = m u + g; v += u; exact k-th largest |v| by radix select; (index, value) compaction with masking
 * of u and v; sparse all-gather into every rank's receive slots; scatter-add value / W into the
 * bucket. nvr > 1 (loopback world): cooperative launch. nvr == 1: plain launch with counter barriers between
 * the phases (status[0][7] is the counter; the launcher clears it); grid_x is clamped to device residency. */
typedef struct NangilaDgcParams {
  void* grad[NANGILA_MAX_VRANKS];       /* in: gradient; out: dense mean of the selected entries */
  float* u[NANGILA_MAX_VRANKS];         /* momentum-corrected velocity, n floats */
  float* v[NANGILA_MAX_VRANKS];         /* accumulated (unsent) gradient, n floats */
  uint32_t* scratch[NANGILA_MAX_VRANKS];/* nangila_dgc_scratch_words() + 2 * cand_capacity words, any content */
  uint32_t* status[NANGILA_MAX_VRANKS]; /* 8 words, zero before launch */
  uint32_t* out_count[NANGILA_MAX_VRANKS]; /* [0] entries sent by this rank, [1] threshold bit pattern */
  uint8_t* region[NANGILA_MAX_RANKS];
  uint64_t recv_off, flag_off;
  int64_t n;
  int32_t world, rank0, nvr, grad_dtype;
  uint32_t k;                           /* entries to keep: ceil(n (1 - sparsity)) */
  uint32_t capacity;                    /* list capacity per rank, multiple of 4, >= k */
  uint32_t cand_capacity;               /* candidate list entries behind the scratch words (0: always take the
                                           dense selection passes) */
  uint32_t epoch;
  float momentum;                       /* momentum-correction factor m in [0, 1) */
  uint64_t timeout_ns;
  int32_t grid_x;
} NangilaDgcParams;
uint64_t nangila_dgc_region_bytes(uint32_t capacity, int32_t world, uint64_t* recv_off, uint64_t* flag_off);
uint32_t nangila_dgc_scratch_words(void);
int nangila_dgc_launch(const NangilaDgcParams* p, cudaStream_t stream);

/* ---- Sculptor calibration statistics (sculptor_stats.cu) -----------------------------------------------
 * Descriptor arrays live in DEVICE memory. */
typedef struct NangilaLayerDesc {
  const void* data;
  int64_t numel;
  int32_t dtype;
  int32_t pad_;
} NangilaLayerDesc;
typedef struct NangilaPairDesc {
  const void* data_i;
  const void* data_j;
  float* state;          /* 5 * numel floats: mean_i, mean_j, m2_i, m2_j, co-moment */
  int64_t numel;
  int32_t dtype;
  int32_t count_after;   /* number of samples including the one being added */
} NangilaPairDesc;
int nangila_sculptor_layer_sumsq(const NangilaLayerDesc* layers, int32_t nlayers, int64_t max_numel, double* out,
                                 cudaStream_t stream);
int nangila_sculptor_pair_update(const NangilaPairDesc* pairs, int32_t npairs, int64_t max_numel, cudaStream_t stream);
int nangila_sculptor_pair_finalize(const NangilaPairDesc* pairs, int32_t npairs, int64_t max_numel, double* out,
                                   cudaStream_t stream);

/* ---- state hash, parallel CRC32, absmax / percentile ------------------------------------------------------ */
int nangila_state_hash(const void* data, int64_t nbytes, uint64_t seed, uint64_t* out, cudaStream_t stream);
int64_t nangila_crc32_scratch_words(int64_t nbytes);
int nangila_crc32(const void* data, int64_t nbytes, uint32_t* scratch, uint32_t* out, cudaStream_t stream);
uint32_t nangila_absmax_scratch_words(void);
int nangila_absmax_hist(const void* x, int32_t dtype, int64_t n, uint32_t k, float qmax, uint32_t* scratch, float* out,
                        uint32_t* hist256, cudaStream_t stream);

/* ---- single-scale compatibility kernels (reference signature: predict.cu / reconstruct.cu) ------- */
int nangila_predict_quantize_gamma(const float* grad, const float* g_curr, const float* g_prev, float mu,
                                   float gamma, uint8_t* out, int64_t n, uint32_t step, uint32_t layer_id,
                                   cudaStream_t stream);
int nangila_dequant_reconstruct_gamma(const uint8_t* packed, const float* g_curr, const float* g_prev, float mu,
                                      float gamma, float* out, int64_t n, cudaStream_t stream);

/* ---- device-side packet codec in the host core's wire format (packet_codec.cu) ---------------------------
 * payload = f32 -64 | u32 numel | u32 ndim = 1 | u32 numel | f32 kappa | f32 scale[ceil(n/64)] | u8 packed[ceil(n/2)].
 * encode: x = grad + ef - kappa (curr + mu (curr - prev)); scale = amax / 7 per 64 elements; round to nearest; ef <- x - q scale.
 * gain >= 0 fixes kappa; gain < 0 derives it on the device as clip(<grad + ef, g_hat> / <g_hat, g_hat>, 0, 1) (no
 * scratch needed: the sums sit in the payload's first bytes until the encoder has read them). curr / prev / ef are
 * FP32 and may be NULL (no history: kappa = 0; no error memory). `payload` must be 4-byte aligned and hold
 * nangila_packet_payload_bytes(n) bytes. */
int64_t nangila_packet_payload_bytes(int64_t n);
int nangila_packet_encode(const void* grad, int32_t dtype, const float* curr, const float* prev, float* ef, float mu,
                          float gain, int64_t n, uint8_t* payload, cudaStream_t stream);
/* decode: out = q scale + kappa (curr + mu (curr - prev)); gain < 0 takes kappa from the payload. `ndim` is the
 * payload's dimension count (its third word), which fixes where the gain, scales and nibbles start. */
int nangila_packet_decode(const uint8_t* payload, int64_t payload_bytes, int32_t ndim, const float* curr, const float* prev,
                          float mu, float gain, int64_t n, float* out, cudaStream_t stream);
/* runtime helpers for callers that bind this library without linking the CUDA runtime themselves */
int nangila_copy_to_host(void* dst, const void* src, int64_t nbytes, cudaStream_t stream);   /* copies, then synchronises */
int nangila_copy_to_device(void* dst, const void* src, int64_t nbytes, cudaStream_t stream); /* asynchronous */
int nangila_stream_sync(cudaStream_t stream);

/* ---- fused softmax cross-entropy over bf16 logits with padded columns (fused_ce.cu) ---------------- */
int nangila_ce_forward(const void* logits, const int64_t* targets, float* losses, float* lse, int64_t rows, int v, int64_t stride,
                       cudaStream_t stream);
int nangila_ce_backward(const void* logits, const int64_t* targets, const float* lse, const float* grad_out, void* grad, int64_t rows,
                        int v, int64_t stride, cudaStream_t stream);

/* ---- column sums of a [R, C] bf16 matrix and of its product with a second one (colsum.cu) -------- */
int64_t nangila_colsum_scratch_floats(int C);
int nangila_colsum(const void* a, const void* b, int64_t R, int C, float* scratch, float* out, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
