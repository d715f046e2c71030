// C++ DDP communication hook (`nangila._cuda.NangilaDDPHook`).
//
// The whole per-bucket path of the prediction-residual compressor runs here without touching the
// interpreter beyond the hook call itself: bucket state lookup, stream hand-over, ONE launch of the
// fused bucket kernel on a dedicated high-priority stream, and a CUDA-aware future that DDP's
// reducer waits on without a host synchronisation. The prediction-gain controller (lagged by one
// step, fed from a pinned host copy of the kernels' statistics) and the safe-mode monitor run in
// `step()` / `report_validation_loss()`.
//
// Phase deferral. With more than one rank the compressed exchange of a bucket is queued as separate
// launches of the same kernel, one per phase: phase 1 (quantize and push, never waits for a peer) at once,
// the phases that wait for peers' flags only when the NEXT bucket arrives (or, for the last bucket of
// the iteration, right away). Nothing consumes a bucket before the end of backward, so the delay is free,
// and by the time a waiting phase starts the peers have usually delivered: the kernel no longer sits on
// the SMs spinning while ranks are skewed. The bucket's future completes after its last phase.
//
// Two ways in. `run(bucket)` is what a Python comm hook calls (DDP then wants a Python future). With
// `register_native(reducer)` the hook is installed on DDP's reducer as a C++ CommHookInterface: the reducer
// calls it from the autograd thread without entering the interpreter at all; Python is touched only when
// a bucket is seen for the first time (its symmetric memory comes from a Python allocator).
//
// Counterpart of nangila::NangilaDDPHook in the reference (nangila_ddp/src/ddp_hook.cpp:45-372),
// which per bucket ran a compress kernel, two all-gathers with host synchronisation, one reconstruct
// kernel per rank, an accumulate / divide and two history copies.
#include <ATen/cuda/CUDAContext.h>
#include <ATen/cuda/CUDAEvent.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/csrc/distributed/c10d/comm.hpp>
#include <torch/csrc/distributed/c10d/reducer.hpp>
#include <torch/csrc/jit/python/pybind_utils.h>
#include <torch/extension.h>

#include <nvtx3/nvToolsExt.h>

#include <cstdlib>
#include <cstring>
#include <deque>
#include <map>
#include <memory>
#include <mutex>
#include <optional>
#include <string>
#include <vector>

#include "core/config.hpp"
#include "core/safe_mode.hpp"
#include "nangila_kernels.h"

namespace py = pybind11;

namespace {

constexpr int kStatsWidth = 8;

int grad_dtype_code(const at::Tensor& t) {
  switch (t.scalar_type()) {
    case at::kFloat: return NANGILA_F32;
    case at::kHalf: return NANGILA_F16;
    case at::kBFloat16: return NANGILA_BF16;
    default: TORCH_CHECK(false, "nangila: unsupported gradient dtype ", t.scalar_type());
  }
}

double env_double(const char* name, double fallback) {
  const char* v = std::getenv(name);
  return (v && *v) ? std::atof(v) : fallback;
}

struct Bucket {
  int64_t n = 0;
  int grad_dtype = 0;
  int32_t chunk = 0;
  int32_t nchunks = 0;
  uint64_t r1 = 0, r2 = 0, f1 = 0, f2 = 0;
  std::vector<uint8_t*> region;  // one pointer per rank, this bucket's exchange region
  at::Tensor prev, curr, ef;
  int slot = 0;
  double pred_gain = 1.0;
  double miss_ema = -1.0;
  int cooldown = 0;
  uint32_t epoch = 0;
  uint64_t calls = 0;
  uint64_t compressed_calls = 0;
  uint64_t probe_every = 0;  // calls between history probes while the gain is 0 (0: not initialised)
  uint64_t next_probe = 0;
  uint64_t last_probe = 0;
  double totals[4] = {0, 0, 0, 0};
  // NANGILA_TIMING=1: events around the most recent launch of this bucket
  std::shared_ptr<at::cuda::CUDAEvent> t0, t1;
};

// A bucket whose later phases are still to be queued.
struct Pending {
  NangilaPredResParams p;
  int next_bit;   // phase bit to launch next (2 or 4)
  int last_bit;   // final phase bit of this exchange (2 in gather mode, 4 otherwise)
  std::shared_ptr<torch::jit::PythonFutureWrapper> fut;      // Python entry: the future's value is a Python object
  c10::intrusive_ptr<c10::ivalue::Future> native_fut;        // native entry: the value is the bucket tensor
  at::Tensor tensor;
  Bucket* bucket;
};

class DdpHook {
 public:
  DdpHook(int64_t num_layers, int64_t warmup_steps)
      : num_layers_(num_layers), warmup_steps_(warmup_steps), safe_mode_(std::nullopt) {
    momentum_ = 0.9;
    timeout_s_ = env_double("NANGILA_WAIT_TIMEOUT_MS", 2000.0) / 1e3;
    const char* fixed = std::getenv("NANGILA_PRED_GAIN");
    adaptive_ = !(fixed && *fixed);
    fixed_gain_ = adaptive_ ? 1.0 : std::atof(fixed);
    probe_every_ = std::max<int64_t>(1, int64_t(env_double("NANGILA_PROBE_EVERY", 8)));
    chunk_override_ = int32_t(env_double("NANGILA_CHUNK", 0));
    ctas_ = int32_t(env_double("NANGILA_COMM_CTAS", 0));
    ctas_wait_ = int32_t(env_double("NANGILA_COMM_CTAS_WAIT", 0));
    defer_ = env_double("NANGILA_DEFER", 1) != 0;
    dry_run_ = env_double("NANGILA_DRY_RUN", 0) != 0;
    timing_ = env_double("NANGILA_TIMING", 0) != 0;
    nvtx_ = env_double("NANGILA_NVTX", 0) != 0;
    // gather mode (every rank sums all contributions itself) only pays at two ranks: at four, the three-phase
    // form with deferred waiting phases was 3 % faster per step and the gather kernel alone slower than NCCL
    gather_max_world_ = std::min<int32_t>(NANGILA_GATHER_MAX_WORLD, int32_t(env_double("NANGILA_GATHER_MAX_WORLD", 2)));
  }

  // `allocate(bytes)` returns the addresses (one per rank, as ints) of a fresh zero-initialised
  // block of symmetric memory; it is called once per bucket, never on the steady-state path.
  void attach(int64_t rank, int64_t world, py::function allocate) {
    TORCH_CHECK(world >= 1 && world <= NANGILA_MAX_RANKS, "nangila: world size out of range");
    TORCH_CHECK(rank >= 0 && rank < world, "nangila: bad rank");
    rank_ = int32_t(rank);
    world_ = int32_t(world);
    allocate_ = std::move(allocate);
    attached_ = true;
  }

  void configure(double momentum, bool error_feedback, bool stochastic, int64_t seed, int64_t max_buckets) {
    TORCH_CHECK(buckets_.empty(), "nangila: configure() must precede the first bucket");
    momentum_ = momentum;
    error_feedback_ = error_feedback;
    stochastic_ = stochastic;
    seed_ = uint32_t(seed);
    max_buckets_ = int(max_buckets);
  }

  // The hook body: `bucket` is a torch.distributed.GradBucket. Returns a torch.futures.Future.
  py::object run(py::object bucket) {
    at::Tensor tensor = bucket.attr("buffer")().cast<at::Tensor>();
    const int64_t index = bucket.attr("index")().cast<int64_t>();
    const bool is_last = bucket.attr("is_last")().cast<bool>();
    return run_tensor(index, tensor, is_last);
  }

  // Create the device state of a bucket without launching anything (checkpoint restore fills it in).
  void ensure_bucket(py::object bucket) {
    at::Tensor tensor = bucket.attr("buffer")().cast<at::Tensor>();
    const int64_t index = bucket.attr("index")().cast<int64_t>();
    TORCH_CHECK(attached_, "nangila: attach() was not called");
    TORCH_CHECK(tensor.is_cuda() && tensor.is_contiguous(), "nangila: the C++ hook needs a contiguous CUDA bucket");
    c10::cuda::CUDAGuard guard(tensor.device());
    std::lock_guard<std::mutex> lock(mutex_);
    ensure_device(tensor);
    bucket_for(index, tensor);
  }

  // `is_last`: no further bucket follows in this iteration, so nothing may stay deferred.
  py::object run_tensor(int64_t index, at::Tensor tensor, bool is_last) {
    std::shared_ptr<torch::jit::PythonFutureWrapper> wrapper;
    run_impl(index, std::move(tensor), is_last, &wrapper, nullptr);
    return py::cast(wrapper);
  }

  // Entry of the reducer-level hook: no interpreter involved.
  c10::intrusive_ptr<c10::ivalue::Future> run_native(int64_t index, at::Tensor tensor, bool is_last) {
    c10::intrusive_ptr<c10::ivalue::Future> fut;
    run_impl(index, std::move(tensor), is_last, nullptr, &fut);
    return fut;
  }

  // Installs this hook on a DDP reducer (``ddp_model.reducer``) as a C++ communication hook.
  static void register_native(std::shared_ptr<DdpHook> self, py::object reducer);

  void run_impl(int64_t index, at::Tensor tensor, bool is_last, std::shared_ptr<torch::jit::PythonFutureWrapper>* py_out,
                c10::intrusive_ptr<c10::ivalue::Future>* native_out) {
    TORCH_CHECK(attached_, "nangila: attach() was not called");
    TORCH_CHECK(tensor.is_cuda() && tensor.is_contiguous(), "nangila: the C++ hook needs a contiguous CUDA bucket");
    TORCH_CHECK((reinterpret_cast<uintptr_t>(tensor.data_ptr()) & 15u) == 0, "nangila: bucket must be 16-byte aligned");
    c10::cuda::CUDAGuard guard(tensor.device());
    std::vector<Pending> finished;  // futures to complete once the state lock is released
    std::shared_ptr<torch::jit::PythonFutureWrapper> wrapper;
    c10::intrusive_ptr<c10::ivalue::Future> native_fut;
    {
    std::lock_guard<std::mutex> lock(mutex_);
    ensure_device(tensor);
    Bucket& b = bucket_for(index, tensor);
    const bool compressed = is_compression_enabled();
    b.epoch += 1;
    b.calls += 1;
    b.compressed_calls += compressed ? 1 : 0;
    launches_ += 1;
    const int64_t nbytes = tensor.numel() * tensor.element_size();
    original_bytes_ += nbytes;
    compressed_bytes_ += compressed ? int64_t(double(tensor.numel()) * (0.5 + 2.0 / 64.0)) : nbytes;

    NangilaPredResParams p;
    std::memset(&p, 0, sizeof p);
    p.n = b.n;
    p.world = world_;
    p.rank0 = rank_;
    p.nvr = 1;
    p.chunk_elems = b.chunk;
    p.nchunks = b.nchunks;
    p.grad_dtype = b.grad_dtype;
    p.state_dtype = b.grad_dtype == NANGILA_F32 ? NANGILA_F32 : NANGILA_BF16;
    p.mode = compressed ? 0 : 1;
    p.stochastic = stochastic_ ? 1 : 0;
    // probes that keep finding nothing to predict are spaced out (8, 16, ... 64 calls); see adapt()
    if (b.probe_every == 0) {
      b.probe_every = uint64_t(probe_every_);
      b.next_probe = b.probe_every;
    }
    p.measure = 0;
    if (b.calls >= b.next_probe) {
      p.measure = 1;
      b.last_probe = b.calls;
      b.next_probe = b.calls + b.probe_every;
    }
    // the history is read by a probe and by a non-zero gain only: while the gain is 0 it is written on the
    // two calls before a probe (the predictor needs two steps) and the two after it (until the controller
    // has seen the probe's statistics), and left alone in between
    p.skip_history = (compressed && b.pred_gain == 0.0 && p.measure == 0 && b.calls + 2 < b.next_probe &&
                      b.calls > b.last_probe + 2) ? 1 : 0;
    p.gather = (compressed && world_ >= 2 && world_ <= gather_max_world_) ? 1 : 0;
    p.uniform_gain = 1;  // the statistics are summed over the group before the controller reads them
    p.epoch = b.epoch;
    p.seed = seed_;
    p.step = uint32_t(step_);
    p.bucket_id = uint32_t(index);
    p.mu = float(momentum_);
    p.pred_gain[0] = float(b.pred_gain);
    p.timeout_ns = uint64_t(timeout_s_ * 1e9);
    p.grid_x = grid_for(b, false);
    p.recv1_off = b.r1;
    p.recv2_off = b.r2;
    p.flag1_off = b.f1;
    p.flag2_off = b.f2;
    p.grad[0] = tensor.data_ptr();
    p.prev[0] = b.prev.data_ptr();
    p.curr[0] = b.curr.data_ptr();
    p.ef[0] = error_feedback_ ? b.ef.data_ptr() : nullptr;
    p.stats[0] = stats_dev_.data_ptr<float>() + size_t(b.slot) * kStatsWidth;
    p.status[0] = reinterpret_cast<uint32_t*>(status_.data_ptr<int32_t>());
    for (int r = 0; r < world_; ++r) p.region[r] = b.region[size_t(r)];

    // hand the bucket over to the exchange stream: it starts when the producer stream has written
    // the gradients, and the future's completion event orders the consumer after the kernel
    c10::cuda::CUDAStream producer = c10::cuda::getCurrentCUDAStream(tensor.device().index());
    ready_.record(producer);
    ready_.block(*stream_);
    if (nvtx_) nvtxRangePushA(compressed ? "nangila.bucket.int4" : "nangila.bucket.exact");
    if (timing_) {
      if (!b.t0) {
        b.t0 = std::make_shared<at::cuda::CUDAEvent>(cudaEventDefault);
        b.t1 = std::make_shared<at::cuda::CUDAEvent>(cudaEventDefault);
      }
      b.t0->record(*stream_);
    }
    // split into per-phase launches when there are peers to wait for; otherwise one fused launch
    // (two launches of the gather form gained nothing over the fused one at two ranks, so it stays fused)
    const bool split = defer_ && compressed && world_ > 1 && p.gather == 0;
    p.phase_mask = split ? 1 : 0;
    // NANGILA_DRY_RUN=1 (diagnostics): everything but the launch, to time the host side of the hook on its own
    const int err = dry_run_ ? 0 : nangila_predres_launch(&p, stream_->stream());
    if (nvtx_) nvtxRangePop();
    TORCH_CHECK(err == 0, "nangila: predres_launch failed: ", cudaGetErrorString(static_cast<cudaError_t>(err)));
    std::swap(b.prev, b.curr);

    apply_restore(index, b, tensor);
    if (py_out != nullptr) {
      // DDP's Python-hook adapter expects the future's value to be a Python object (the bucket tensor).
      auto fut = c10::make_intrusive<c10::ivalue::Future>(c10::PyObjectType::get(), std::vector<c10::Device>{tensor.device()});
      wrapper = std::make_shared<torch::jit::PythonFutureWrapper>(fut);
    } else {
      native_fut = c10::make_intrusive<c10::ivalue::Future>(c10::TensorType::get(), std::vector<c10::Device>{tensor.device()});
    }
    // older buckets advance by one phase each (oldest first); then this one joins the queue
    advance_pending(finished, /*drain=*/false);
    if (split) {
      Pending q;
      q.p = p;
      q.p.grid_x = grid_for(b, true);
      q.next_bit = 2;
      q.last_bit = p.gather != 0 ? 2 : 4;
      q.fut = wrapper;
      q.native_fut = native_fut;
      q.tensor = tensor;
      q.bucket = &b;
      pending_.push_back(std::move(q));
    } else {
      if (timing_) b.t1->record(*stream_);
      Pending q;
      q.fut = wrapper;
      q.native_fut = native_fut;
      q.tensor = tensor;
      q.bucket = &b;
      finished.push_back(std::move(q));
    }
    if (is_last) advance_pending(finished, /*drain=*/true);
    }  // state lock released: completing a future below drops and re-takes the GIL

    // Completing a future while the exchange stream is current records the stream's event in it, so
    // the reducer's wait orders its own stream after everything queued on the exchange stream so far,
    // which includes the bucket's last phase.
    complete(finished);
    if (py_out != nullptr) *py_out = wrapper;
    if (native_out != nullptr) *native_out = native_fut;
  }

  // Once per optimizer step, after the last bucket was queued.
  void step() {
    std::vector<Pending> finished;
    {
    std::lock_guard<std::mutex> lock(mutex_);
    step_ += 1;
    if (!stream_) return;
    c10::cuda::CUDAGuard guard(device_);
    advance_pending(finished, /*drain=*/true);  // nothing should be left; a caller that bypassed is_last ends here
    if (stats_pending_) {
      stats_event_.synchronize();
      const float* host = stats_host_.data_ptr<float>();
      for (auto& kv : buckets_) adapt(kv.second, host + size_t(kv.second.slot) * kStatsWidth);
    }
    {
      c10::cuda::CUDAStreamGuard sg(*stream_);
      stats_host_.copy_(stats_dev_, /*non_blocking=*/true);
      stats_dev_.zero_();
      stats_event_.record(*stream_);
      stats_pending_ = true;
    }
    }
    if (!finished.empty()) {
      c10::cuda::CUDAGuard guard(device_);
      complete(finished);
    }
  }

  int64_t current_step() const { return step_; }
  bool is_compression_enabled() const {
    return step_ >= warmup_steps_ && step_ >= exact_until_ && !paused_ && !paused_override_;
  }
  // Resume: gradients are exchanged uncompressed before `step` (a new DDP instance lays its buckets out in
  // construction order for one iteration); saved bucket state given to restore_bucket() is copied into a
  // bucket the first time it appears with the saved size at or after that step.
  void set_exact_until(int64_t step) { exact_until_ = step; }
  void restore_bucket(int64_t index, at::Tensor prev, at::Tensor curr, c10::optional<at::Tensor> ef) {
    std::lock_guard<std::mutex> lock(mutex_);
    restore_[index] = Restore{std::move(prev), std::move(curr), std::move(ef)};
  }
  void fast_forward(int64_t to_step) { step_ = std::max(step_, to_step); }
  // Uncompressed exchange while set (safe-mode fallback, history re-seed after a failure).
  void set_paused(bool paused) { paused_override_ = paused; }

  void enable_safe_mode(double divergence_threshold, int64_t check_interval, int64_t consecutive_failures, int64_t recovery_cooldown) {
    nangila::SafeModeConfig cfg;
    cfg.divergence_threshold = float(divergence_threshold);
    cfg.check_interval = size_t(check_interval);
    cfg.max_consecutive_failures = uint32_t(consecutive_failures);
    cfg.recovery_cooldown = size_t(recovery_cooldown);
    safe_mode_.emplace(cfg);
  }
  // Returns the monitor's action code: 0 continue, 1 fall back, 2 recovery complete, 3 no check this step, 4 canary.
  int report_validation_loss(double loss) {
    if (!safe_mode_) return 3;
    if (!safe_mode_->should_check(size_t(step_))) return 3;
    const nangila::SafeModeAction a = safe_mode_->check(size_t(step_), float(loss));
    paused_ = !safe_mode_->should_compress();
    return int(a);
  }

  // Blocks until the exchange stream is idle; raises if a kernel gave up waiting for a peer.
  void check_status() {
    if (!stream_) return;
    {
      std::vector<Pending> finished;
      {
        std::lock_guard<std::mutex> lock(mutex_);
        c10::cuda::CUDAGuard guard(device_);
        advance_pending(finished, /*drain=*/true);
      }
      if (!finished.empty()) {
        c10::cuda::CUDAGuard guard(device_);
        complete(finished);
      }
    }
    stream_->synchronize();
    at::Tensor host = status_.cpu();
    const int32_t* w = host.data_ptr<int32_t>();
    if (w[0] != 0) {
      const int code = w[0];
      std::string what = code == 2   ? "timeout in phase 2: a chunk owner did not receive every rank's contribution"
                         : code == 3 ? "timeout in phase 3: a reduced chunk did not arrive from its owner"
                         : code == 4 ? "timeout in an intra-GPU grid barrier"
                                     : "code " + std::to_string(code);
      const int r = w[1], peer = w[2], ep = w[3], seen = w[4], ph = w[5], ch = w[6];
      status_.zero_();
      TORCH_CHECK(false, "nangila: fused exchange failed on rank ", r, " (", what, "); waiting for rank ", peer, ", epoch ", ep,
                  " (last seen ", seen, "), phase ", ph, ", chunk ", ch);
    }
  }

  py::dict get_stats() const {
    py::dict d;
    d["step"] = step_;
    d["compression_enabled"] = is_compression_enabled();
    d["num_layers"] = num_layers_;
    d["num_buckets"] = int64_t(buckets_.size());
    d["kernel_launches"] = launches_;
    d["total_original_bytes"] = original_bytes_;
    d["total_compressed_bytes"] = compressed_bytes_;
    d["compression_ratio"] = compressed_bytes_ > 0 ? double(original_bytes_) / double(compressed_bytes_) : 1.0;
    py::dict gains;
    for (auto& kv : buckets_) gains[py::int_(kv.first)] = kv.second.pred_gain;
    d["prediction_gain"] = gains;
    if (timing_) {
      // device time of each bucket's most recent launch, where it has completed (nothing is synchronised)
      py::dict ms;
      for (auto& kv : buckets_)
        if (kv.second.t1 && kv.second.t1->query()) ms[py::int_(kv.first)] = kv.second.t0->elapsed_time(*kv.second.t1);
      d["bucket_kernel_ms"] = ms;
    }
    return d;
  }
  int64_t launches() const { return launches_; }
  // The device table of per-bucket statistics and the exchange stream, so that the caller can sum the
  // table over the process group (on that stream) before step() copies it to the host. Every rank then
  // derives the same prediction gains.
  py::object stats_tensor() const { return stats_dev_.defined() ? py::cast(stats_dev_) : py::none(); }
  int64_t stream_ptr() const { return stream_ ? int64_t(reinterpret_cast<intptr_t>(stream_->stream())) : 0; }
  static std::string version() { return "0.1.0"; }

  // History / error-feedback tensors of a bucket, for checkpointing and tests.
  py::dict bucket_state(int64_t index) {
    auto it = buckets_.find(index);
    TORCH_CHECK(it != buckets_.end(), "nangila: unknown bucket ", index);
    py::dict d;
    d["n"] = it->second.n;
    d["epoch"] = it->second.epoch;
    d["prev"] = it->second.prev;
    d["curr"] = it->second.curr;
    if (error_feedback_) d["ef"] = it->second.ef;
    d["pred_gain"] = it->second.pred_gain;
    return d;
  }

 private:
  struct Restore {
    at::Tensor prev, curr;
    c10::optional<at::Tensor> ef;
  };
  // Copies saved state into the bucket (on the exchange stream, before its kernel). Caller holds the lock.
  void apply_restore(int64_t index, Bucket& b, const at::Tensor& tensor) {
    if (restore_.empty() || step_ < exact_until_) return;
    auto it = restore_.find(index);
    if (it == restore_.end()) return;
    if (it->second.prev.numel() == b.n && it->second.curr.numel() == b.n) {
      c10::cuda::CUDAStreamGuard sg(*stream_);
      b.prev.copy_(it->second.prev.to(b.prev.scalar_type()), /*non_blocking=*/true);
      b.curr.copy_(it->second.curr.to(b.curr.scalar_type()), /*non_blocking=*/true);
      if (error_feedback_ && it->second.ef.has_value() && it->second.ef->numel() == b.n)
        b.ef.copy_(it->second.ef->to(b.ef.scalar_type()), /*non_blocking=*/true);
    }
    (void)tensor;
    restore_.erase(it);
  }

  // Queue the next phase of every deferred bucket (oldest first); with `drain`, keep going until nothing
  // is deferred. Buckets whose last phase has been queued move to `finished`. Caller holds the lock.
  void advance_pending(std::vector<Pending>& finished, bool drain) {
    do {
      const size_t count = pending_.size();
      for (size_t i = 0; i < count; ++i) {
        Pending q = std::move(pending_.front());
        pending_.pop_front();
        q.p.phase_mask = q.next_bit;
        launches_ += 1;
        const int err = nangila_predres_launch(&q.p, stream_->stream());
        TORCH_CHECK(err == 0, "nangila: predres_launch failed: ", cudaGetErrorString(static_cast<cudaError_t>(err)));
        if (q.next_bit == q.last_bit) {
          if (timing_ && q.bucket->t1) q.bucket->t1->record(*stream_);
          finished.push_back(std::move(q));
        } else {
          q.next_bit <<= 1;
          pending_.push_back(std::move(q));
        }
      }
    } while (drain && !pending_.empty());
  }

  void complete(std::vector<Pending>& finished) {
    if (finished.empty()) return;
    c10::cuda::CUDAStreamGuard sg(*stream_);
    for (auto& q : finished) {
      if (q.native_fut) q.native_fut->markCompleted(c10::IValue(q.tensor));
      else q.fut->markCompleted(py::cast(q.tensor));
    }
    finished.clear();
  }

  void ensure_device(const at::Tensor& t) {
    if (stream_) return;
    device_ = t.device();
    // NANGILA_STREAM_PRIORITY=0 puts the exchange on a normal-priority stream (default: high priority)
    stream_.emplace(c10::cuda::getStreamFromPool(/*isHighPriority=*/env_double("NANGILA_STREAM_PRIORITY", -1) < 0, device_.index()));
    auto f32 = at::TensorOptions().dtype(at::kFloat).device(device_);
    stats_dev_ = at::zeros({max_buckets_, kStatsWidth}, f32);
    stats_host_ = at::zeros({max_buckets_, kStatsWidth}, at::TensorOptions().dtype(at::kFloat).pinned_memory(true));
    status_ = at::zeros({8}, at::TensorOptions().dtype(at::kInt).device(device_));
  }

  Bucket& bucket_for(int64_t index, const at::Tensor& t) {
    const int code = grad_dtype_code(t);
    auto it = buckets_.find(index);
    if (it != buckets_.end() && it->second.n == t.numel() && it->second.grad_dtype == code) return it->second;
    Bucket b;
    b.n = t.numel();
    b.grad_dtype = code;
    // sized against the CTAs the device holds at once, so that each phase is whole, equally loaded waves
    int32_t c;
    if (chunk_override_ > 0) {
      c = chunk_override_;
    } else {
      if (resident_ <= 0) resident_ = nangila_predres_resident_ctas();
      c = nangila_predres_chunk_elems(b.n, resident_);
    }
    b.chunk = c;
    b.nchunks = int32_t((b.n + c - 1) / c);
    const uint64_t total = nangila_predres_region_bytes(b.n, world_, c, code, &b.r1, &b.r2, &b.f1, &b.f2);
    {
      py::gil_scoped_acquire gil;
      py::list ptrs = allocate_(py::int_(total)).cast<py::list>();
      TORCH_CHECK(int(py::len(ptrs)) == world_, "nangila: the allocator must return one address per rank");
      for (auto h : ptrs) b.region.push_back(reinterpret_cast<uint8_t*>(static_cast<uintptr_t>(h.cast<uint64_t>())));
    }
    auto opts = at::TensorOptions().device(t.device()).dtype(code == NANGILA_F32 ? at::kFloat : at::kBFloat16);
    b.prev = at::zeros({b.n}, opts);
    b.curr = at::zeros({b.n}, opts);
    if (error_feedback_) b.ef = at::zeros({b.n}, opts);
    b.slot = it != buckets_.end() ? it->second.slot : (next_slot_++ % max_buckets_);
    b.pred_gain = fixed_gain_;
    stats_dev_[b.slot].zero_();
    buckets_[index] = std::move(b);
    return buckets_[index];
  }

  // CTAs for a launch: no more than there are chunks; the launcher clamps to what the device can hold at
  // once. `waiting`: a launch of phases 2 / 3 only (NANGILA_COMM_CTAS_WAIT), which may spend time polling flags.
  int32_t grid_for(const Bucket& b, bool waiting) const {
    const int64_t owned = (b.nchunks + world_ - 1) / world_;
    const int64_t want = owned * world_;  // = chunks of the bucket, rounded up to whole rounds
    const int64_t cap = waiting && ctas_wait_ > 0 ? ctas_wait_ : ctas_ > 0 ? ctas_ : (int64_t(1) << 20);
    return int32_t(std::max<int64_t>(1, std::min(want, cap)));
  }

  // Least-squares prediction gain from the previous step's inner products (see the kernel's
  // statistics layout: {sum e^2, sum g^2, <g + ef, g_hat>, <g_hat, g_hat>, sum ef^2}).
  void adapt(Bucket& b, const float* row) {
    const double e2 = row[0], g2 = row[1], xp = row[2], pp = row[3], f2 = row[4];
    if (g2 <= 0.0) return;
    b.totals[0] += e2; b.totals[1] += g2; b.totals[2] += xp; b.totals[3] += pp;
    b.miss_ema = b.miss_ema < 0.0 ? e2 / g2 : 0.7 * b.miss_ema + 0.3 * e2 / g2;
    if (!adaptive_) return;
    if (b.cooldown > 0) { b.cooldown -= 1; return; }
    if (f2 > 2.0 * g2) { b.pred_gain = 0.0; b.cooldown = 20; return; }
    if (pp <= 0.0) return;  // not a probe step
    const double best = std::min(std::max(xp / pp, 0.0), 1.0);
    const double gain = 0.5 * b.pred_gain + 0.5 * best;
    b.pred_gain = gain >= 0.2 ? gain : 0.0;
    if (b.probe_every != 0)
      b.probe_every = b.pred_gain > 0.0 ? uint64_t(probe_every_) : std::min<uint64_t>(2 * b.probe_every, std::max<uint64_t>(64, uint64_t(probe_every_)));  // below 0.2 (< 4 % less residual energy) the history loads cost more than they save
  }

  int64_t num_layers_;
  int64_t warmup_steps_;
  int64_t step_ = 0;
  int64_t exact_until_ = 0;
  std::map<int64_t, Restore> restore_;
  bool paused_ = false;
  bool paused_override_ = false;
  std::optional<nangila::SafeMode> safe_mode_;
  bool attached_ = false;
  int32_t rank_ = 0, world_ = 1;
  py::function allocate_;
  double momentum_;
  bool error_feedback_ = true;
  bool stochastic_ = true;
  uint32_t seed_ = 42;
  int max_buckets_ = 512;
  double timeout_s_;
  bool adaptive_;
  double fixed_gain_;
  int64_t probe_every_;
  int32_t chunk_override_;
  int32_t ctas_;
  int32_t ctas_wait_ = 0;
  bool defer_ = true;
  bool dry_run_ = false;
  int resident_ = 0;  // CTAs of the bucket kernel the device holds at once (queried once)
  std::deque<Pending> pending_;
  int32_t gather_max_world_;
  bool timing_ = false;
  bool nvtx_ = false;
  std::mutex mutex_;
  std::map<int64_t, Bucket> buckets_;
  int next_slot_ = 0;
  c10::Device device_{c10::kCPU};
  std::optional<c10::cuda::CUDAStream> stream_;
  at::cuda::CUDAEvent ready_;
  at::cuda::CUDAEvent stats_event_;
  bool stats_pending_ = false;
  at::Tensor stats_dev_, stats_host_, status_;
  int64_t launches_ = 0;
  int64_t original_bytes_ = 0;
  int64_t compressed_bytes_ = 0;
};

}  // namespace

// The reducer-level hook: what DDP's reducer calls for every ready bucket when the hook was installed with
// register_native(). It shares ownership of the DdpHook with the Python object.
class NativeCommHook : public c10d::CommHookInterface {
 public:
  explicit NativeCommHook(std::shared_ptr<DdpHook> owner) : owner_(std::move(owner)) {}
  ~NativeCommHook() override {
    // the DdpHook holds Python objects (the allocator callback): release it with the interpreter lock, and not
    // at all once the interpreter is gone
    if (Py_IsInitialized()) {
      py::gil_scoped_acquire gil;
      owner_.reset();
    } else {
      new std::shared_ptr<DdpHook>(std::move(owner_));  // deliberately leaked at process exit
    }
  }
  c10::intrusive_ptr<c10::ivalue::Future> runHook(c10d::GradBucket& bucket) override {
    return owner_->run_native(int64_t(bucket.getIndex()), bucket.getBufferRef(), bucket.isLast());
  }
  at::Tensor parseHookResult(const c10::IValue& result) override { return result.toTensor(); }

 private:
  std::shared_ptr<DdpHook> owner_;
};

void DdpHook::register_native(std::shared_ptr<DdpHook> self, py::object reducer) {
  auto r = reducer.cast<std::shared_ptr<c10d::Reducer>>();
  TORCH_CHECK(r != nullptr, "nangila: register_native() wants ddp_model.reducer");
  r->register_comm_hook(std::make_unique<NativeCommHook>(std::move(self)));
}

void register_ddp_hook(py::module_& m) {
  py::class_<DdpHook, std::shared_ptr<DdpHook>>(m, "NangilaDDPHook")
      .def(py::init<int64_t, int64_t>(), py::arg("num_layers"), py::arg("warmup_steps"))
      .def("attach", &DdpHook::attach, py::arg("rank"), py::arg("world"), py::arg("allocate"))
      .def("configure", &DdpHook::configure, py::arg("momentum") = 0.9, py::arg("error_feedback") = true,
           py::arg("stochastic") = true, py::arg("seed") = 42, py::arg("max_buckets") = 512)
      .def("run", &DdpHook::run, py::arg("bucket"))
      .def("run_tensor", &DdpHook::run_tensor, py::arg("index"), py::arg("tensor"), py::arg("is_last") = true)
      .def("ensure_bucket", &DdpHook::ensure_bucket, py::arg("bucket"))
      .def("register_native", &DdpHook::register_native, py::arg("reducer"))
      .def("set_exact_until", &DdpHook::set_exact_until)
      .def("restore_bucket", &DdpHook::restore_bucket, py::arg("index"), py::arg("prev"), py::arg("curr"), py::arg("ef") = py::none())
      .def("step", &DdpHook::step)
      .def("current_step", &DdpHook::current_step)
      .def("is_compression_enabled", &DdpHook::is_compression_enabled)
      .def("fast_forward", &DdpHook::fast_forward)
      .def("set_paused", &DdpHook::set_paused)
      .def("enable_safe_mode", &DdpHook::enable_safe_mode, py::arg("divergence_threshold") = 0.1, py::arg("check_interval") = 100,
           py::arg("consecutive_failures") = 3, py::arg("recovery_cooldown") = 1000)
      .def("report_validation_loss", &DdpHook::report_validation_loss)
      .def("check_status", &DdpHook::check_status)
      .def("get_stats", &DdpHook::get_stats)
      .def("get_kernel_launches", &DdpHook::launches)
      .def("stats_tensor", &DdpHook::stats_tensor)
      .def("stream_ptr", &DdpHook::stream_ptr)
      .def("bucket_state", &DdpHook::bucket_state)
      .def_static("version", &DdpHook::version);
}
