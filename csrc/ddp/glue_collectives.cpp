// Bindings of the kernels other than the prediction-residual bucket exchange; kept in its own
// translation unit so the glue compiles in parallel.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <algorithm>
#include <cstring>
#include <vector>

#include "nangila_kernels.h"

namespace py = pybind11;

namespace {

int dtype_code(const at::Tensor& t) {
  switch (t.scalar_type()) {
    case at::kFloat: return NANGILA_F32;
    case at::kHalf: return NANGILA_F16;
    case at::kBFloat16: return NANGILA_BF16;
    default: TORCH_CHECK(false, "nangila: unsupported dtype ", t.scalar_type());
  }
}
void check_launch(int err, const char* what) {
  TORCH_CHECK(err == 0, "nangila: ", what, " failed: ", cudaGetErrorString(static_cast<cudaError_t>(err)));
}
uint8_t* as_ptr(int64_t v) { return reinterpret_cast<uint8_t*>(static_cast<uintptr_t>(v)); }

py::tuple dgc_region_layout(int64_t capacity, int64_t world) {
  uint64_t r, f;
  uint64_t total = nangila_dgc_region_bytes(uint32_t(capacity), int32_t(world), &r, &f);
  return py::make_tuple(total, r, f, nangila_dgc_scratch_words());
}

void dgc_launch(const std::vector<at::Tensor>& grad, const std::vector<at::Tensor>& u, const std::vector<at::Tensor>& v,
                const std::vector<at::Tensor>& scratch, const std::vector<at::Tensor>& status,
                const std::vector<at::Tensor>& out_count, const std::vector<int64_t>& region_ptrs, int64_t recv_off,
                int64_t flag_off, int64_t rank0, int64_t k, int64_t capacity, int64_t epoch, double momentum,
                double timeout_s, int64_t grid_x) {
  const size_t nvr = grad.size();
  TORCH_CHECK(nvr >= 1 && nvr <= NANGILA_MAX_VRANKS && u.size() == nvr && v.size() == nvr && scratch.size() == nvr &&
                  status.size() == nvr && out_count.size() == nvr, "nangila: per-rank list length mismatch");
  const size_t world = region_ptrs.size();
  TORCH_CHECK(world >= 1 && world <= NANGILA_MAX_RANKS, "nangila: bad world size");
  NangilaDgcParams p;
  std::memset(&p, 0, sizeof p);
  p.n = grad[0].numel();
  p.world = int32_t(world);
  p.rank0 = int32_t(rank0);
  p.nvr = int32_t(nvr);
  p.grad_dtype = dtype_code(grad[0]);
  p.k = uint32_t(k);
  p.capacity = uint32_t(capacity);
  p.epoch = uint32_t(epoch);
  p.momentum = float(momentum);
  p.timeout_ns = uint64_t(timeout_s * 1e9);
  p.grid_x = int32_t(grid_x);
  p.recv_off = uint64_t(recv_off);
  p.flag_off = uint64_t(flag_off);
  for (size_t i = 0; i < nvr; ++i) {
    TORCH_CHECK(grad[i].is_cuda() && grad[i].is_contiguous() && grad[i].numel() == p.n, "nangila: grad");
    TORCH_CHECK(u[i].scalar_type() == at::kFloat && v[i].scalar_type() == at::kFloat && u[i].numel() == p.n &&
                    v[i].numel() == p.n && u[i].is_contiguous() && v[i].is_contiguous(), "nangila: u/v must be fp32[n]");
    TORCH_CHECK(scratch[i].scalar_type() == at::kInt && scratch[i].numel() >= int64_t(nangila_dgc_scratch_words()), "scratch");
    TORCH_CHECK(status[i].scalar_type() == at::kInt && status[i].numel() >= 8, "status");
    TORCH_CHECK(out_count[i].scalar_type() == at::kInt && out_count[i].numel() >= 2, "out_count");
    p.grad[i] = grad[i].data_ptr();
    p.u[i] = u[i].data_ptr<float>();
    p.v[i] = v[i].data_ptr<float>();
    p.scratch[i] = reinterpret_cast<uint32_t*>(scratch[i].data_ptr<int32_t>());
    // whatever follows the fixed scratch words is the candidate list (index, bits pairs)
    const int64_t extra = (scratch[i].numel() - int64_t(nangila_dgc_scratch_words())) / 2;
    if (i == 0 || extra < int64_t(p.cand_capacity)) p.cand_capacity = uint32_t(std::max<int64_t>(extra, 0));
    p.status[i] = reinterpret_cast<uint32_t*>(status[i].data_ptr<int32_t>());
    p.out_count[i] = reinterpret_cast<uint32_t*>(out_count[i].data_ptr<int32_t>());
  }
  for (size_t r = 0; r < world; ++r) p.region[r] = as_ptr(region_ptrs[r]);
  c10::cuda::CUDAGuard guard(grad[0].device());
  check_launch(nangila_dgc_launch(&p, at::cuda::getCurrentCUDAStream()), "dgc_launch");
}

// ---- small reductions ---------------------------------------------------------------------------------
at::Tensor state_hash(const std::vector<at::Tensor>& tensors, int64_t seed) {
  TORCH_CHECK(!tensors.empty(), "nangila: state_hash needs at least one tensor");
  auto out = at::zeros({1}, tensors[0].options().dtype(at::kLong));
  c10::cuda::CUDAGuard guard(tensors[0].device());
  uint64_t s = uint64_t(seed);
  for (const at::Tensor& t : tensors) {
    TORCH_CHECK(t.is_cuda() && t.is_contiguous(), "nangila: state_hash wants contiguous CUDA tensors");
    check_launch(nangila_state_hash(t.data_ptr(), t.numel() * t.element_size(), s,
                                    reinterpret_cast<uint64_t*>(out.data_ptr<int64_t>()),
                                    at::cuda::getCurrentCUDAStream()), "state_hash");
    s = s * 0x9E3779B97F4A7C15ull + 0x632BE59BD9B4E019ull;  // a different stream of hashes per tensor
  }
  return out;
}
at::Tensor crc32_device(const at::Tensor& t) {
  TORCH_CHECK(t.is_cuda() && t.is_contiguous(), "nangila: crc32 wants a contiguous CUDA tensor");
  const int64_t nbytes = t.numel() * t.element_size();
  auto scratch = at::empty({nangila_crc32_scratch_words(nbytes)}, t.options().dtype(at::kInt));
  auto out = at::zeros({1}, t.options().dtype(at::kInt));
  c10::cuda::CUDAGuard guard(t.device());
  check_launch(nangila_crc32(t.data_ptr(), nbytes, reinterpret_cast<uint32_t*>(scratch.data_ptr<int32_t>()),
                             reinterpret_cast<uint32_t*>(out.data_ptr<int32_t>()), at::cuda::getCurrentCUDAStream()),
               "crc32");
  return out;
}
// ---- device-side packet codec (host wire format) -------------------------------------------------------------
int64_t packet_payload_bytes(int64_t n) { return nangila_packet_payload_bytes(n); }
// Encodes `grad` into payload[0 : packet_payload_bytes(n)] (uint8, 4-byte aligned). gain < 0: derive kappa on the device.
void packet_encode(const at::Tensor& grad, const c10::optional<at::Tensor>& curr, const c10::optional<at::Tensor>& prev,
                   const c10::optional<at::Tensor>& ef, double mu, double gain, at::Tensor payload) {
  TORCH_CHECK(grad.is_cuda() && grad.is_contiguous(), "nangila: packet_encode wants a contiguous CUDA gradient");
  const int64_t n = grad.numel();
  TORCH_CHECK(payload.is_cuda() && payload.scalar_type() == at::kByte && payload.is_contiguous() &&
                  payload.numel() >= nangila_packet_payload_bytes(n), "nangila: payload buffer too small");
  auto f32 = [&](const c10::optional<at::Tensor>& t, const char* what) -> float* {
    if (!t.has_value()) return nullptr;
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kFloat && t->is_contiguous() && t->numel() == n, "nangila: ", what,
                " must be a contiguous FP32 CUDA tensor of the gradient's size");
    return t->data_ptr<float>();
  };
  c10::cuda::CUDAGuard guard(grad.device());
  check_launch(nangila_packet_encode(grad.data_ptr(), dtype_code(grad), f32(curr, "curr"), f32(prev, "prev"), f32(ef, "ef"),
                                     float(mu), float(gain), n, payload.data_ptr<uint8_t>(), at::cuda::getCurrentCUDAStream()),
               "packet_encode");
}
void packet_decode(const at::Tensor& payload, int64_t ndim, const c10::optional<at::Tensor>& curr,
                   const c10::optional<at::Tensor>& prev, double mu, double gain, at::Tensor out) {
  TORCH_CHECK(payload.is_cuda() && payload.scalar_type() == at::kByte && payload.is_contiguous(), "nangila: payload must be uint8 CUDA");
  TORCH_CHECK(out.is_cuda() && out.scalar_type() == at::kFloat && out.is_contiguous(), "nangila: out must be FP32 CUDA");
  const int64_t n = out.numel();
  const float* c = curr.has_value() ? curr->data_ptr<float>() : nullptr;
  const float* p = prev.has_value() ? prev->data_ptr<float>() : nullptr;
  if (c) TORCH_CHECK(curr->numel() == n && prev.has_value() && prev->numel() == n, "nangila: history size mismatch");
  c10::cuda::CUDAGuard guard(out.device());
  check_launch(nangila_packet_decode(payload.data_ptr<uint8_t>(), payload.numel(), int32_t(ndim), c, p, float(mu), float(gain), n,
                                     out.data_ptr<float>(), at::cuda::getCurrentCUDAStream()), "packet_decode");
}

// returns (float[4] = {max|x|, k-th largest |x|, gamma, non-finite count}, int32[256] histogram of |x|/max)
py::tuple absmax_hist(const at::Tensor& x, int64_t k, double qmax) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous(), "nangila: absmax_hist wants a contiguous CUDA tensor");
  auto scratch = at::empty({int64_t(nangila_absmax_scratch_words())}, x.options().dtype(at::kInt));
  auto out = at::zeros({4}, x.options().dtype(at::kFloat));
  auto hist = at::zeros({256}, x.options().dtype(at::kInt));
  c10::cuda::CUDAGuard guard(x.device());
  check_launch(nangila_absmax_hist(x.data_ptr(), dtype_code(x), x.numel(), uint32_t(k), float(qmax),
                                   reinterpret_cast<uint32_t*>(scratch.data_ptr<int32_t>()), out.data_ptr<float>(),
                                   reinterpret_cast<uint32_t*>(hist.data_ptr<int32_t>()),
                                   at::cuda::getCurrentCUDAStream()), "absmax_hist");
  return py::make_tuple(out, hist);
}

// ---- Sculptor statistics ---------------------------------------------------------------------------------
template <class Desc>
at::Tensor to_device_descs(const std::vector<Desc>& v, const at::Device& dev) {
  auto host = at::empty({int64_t(v.size() * sizeof(Desc))}, at::TensorOptions().dtype(at::kByte));
  std::memcpy(host.data_ptr(), v.data(), v.size() * sizeof(Desc));
  return host.to(dev);
}
at::Tensor sculptor_layer_sumsq(const std::vector<at::Tensor>& layers) {
  TORCH_CHECK(!layers.empty(), "nangila: no layers");
  std::vector<NangilaLayerDesc> d(layers.size());
  int64_t mx = 1;
  for (size_t i = 0; i < layers.size(); ++i) {
    TORCH_CHECK(layers[i].is_cuda() && layers[i].is_contiguous(), "nangila: layers must be contiguous CUDA tensors");
    d[i] = NangilaLayerDesc{layers[i].data_ptr(), layers[i].numel(), dtype_code(layers[i]), 0};
    mx = std::max<int64_t>(mx, layers[i].numel());
  }
  c10::cuda::CUDAGuard guard(layers[0].device());
  at::Tensor descs = to_device_descs(d, layers[0].device());
  auto out = at::zeros({int64_t(layers.size())}, layers[0].options().dtype(at::kDouble));
  check_launch(nangila_sculptor_layer_sumsq(reinterpret_cast<const NangilaLayerDesc*>(descs.data_ptr()),
                                            int32_t(layers.size()), mx, out.data_ptr<double>(),
                                            at::cuda::getCurrentCUDAStream()), "sculptor_layer_sumsq");
  return out;
}
std::vector<NangilaPairDesc> pair_descs(const std::vector<at::Tensor>& xi, const std::vector<at::Tensor>& xj,
                                        const std::vector<at::Tensor>& state, const std::vector<int64_t>& count_after,
                                        int64_t* mx) {
  TORCH_CHECK(xi.size() == xj.size() && xi.size() == state.size() && xi.size() == count_after.size() && !xi.empty(),
              "nangila: pair list length mismatch");
  std::vector<NangilaPairDesc> d(xi.size());
  *mx = 1;
  for (size_t i = 0; i < xi.size(); ++i) {
    TORCH_CHECK(xi[i].numel() == xj[i].numel() && xi[i].scalar_type() == xj[i].scalar_type() && xi[i].is_contiguous() &&
                    xj[i].is_contiguous(), "nangila: pair members must match in size and dtype");
    TORCH_CHECK(state[i].scalar_type() == at::kFloat && state[i].numel() == 5 * xi[i].numel() && state[i].is_contiguous(),
                "nangila: pair state must be float[5 * numel]");
    d[i] = NangilaPairDesc{xi[i].data_ptr(), xj[i].data_ptr(), state[i].data_ptr<float>(), xi[i].numel(),
                           dtype_code(xi[i]), int32_t(count_after[i])};
    *mx = std::max<int64_t>(*mx, xi[i].numel());
  }
  return d;
}
void sculptor_pair_update(const std::vector<at::Tensor>& xi, const std::vector<at::Tensor>& xj,
                          const std::vector<at::Tensor>& state, const std::vector<int64_t>& count_after) {
  int64_t mx;
  auto d = pair_descs(xi, xj, state, count_after, &mx);
  c10::cuda::CUDAGuard guard(xi[0].device());
  at::Tensor descs = to_device_descs(d, xi[0].device());
  check_launch(nangila_sculptor_pair_update(reinterpret_cast<const NangilaPairDesc*>(descs.data_ptr()), int32_t(d.size()),
                                            mx, at::cuda::getCurrentCUDAStream()), "sculptor_pair_update");
}
at::Tensor sculptor_pair_finalize(const std::vector<at::Tensor>& state, const std::vector<int64_t>& count) {
  std::vector<at::Tensor> dummy;
  TORCH_CHECK(!state.empty() && state.size() == count.size(), "nangila: pair list length mismatch");
  std::vector<NangilaPairDesc> d(state.size());
  int64_t mx = 1;
  for (size_t i = 0; i < state.size(); ++i) {
    const int64_t n = state[i].numel() / 5;
    d[i] = NangilaPairDesc{nullptr, nullptr, state[i].data_ptr<float>(), n, NANGILA_F32, int32_t(count[i])};
    mx = std::max<int64_t>(mx, n);
  }
  c10::cuda::CUDAGuard guard(state[0].device());
  at::Tensor descs = to_device_descs(d, state[0].device());
  auto out = at::zeros({int64_t(state.size()), 8}, state[0].options().dtype(at::kDouble));
  check_launch(nangila_sculptor_pair_finalize(reinterpret_cast<const NangilaPairDesc*>(descs.data_ptr()),
                                              int32_t(d.size()), mx, out.data_ptr<double>(),
                                              at::cuda::getCurrentCUDAStream()), "sculptor_pair_finalize");
  return out;
}

// ---- fully-sharded collectives -------------------------------------------------------------------------
py::tuple rs_region_layout(int64_t n, int64_t world, int64_t chunk_elems) {
  uint64_t r1, f1;
  int32_t nchunks;
  uint64_t total = nangila_rs_region_bytes(n, int32_t(world), int32_t(chunk_elems), &r1, &f1, &nchunks);
  return py::make_tuple(total, r1, f1, nchunks);
}
// Compressed reduce-scatter: `input[v]` holds world equal shards; `output[v]` receives the reduced shard.
void rs_launch(const std::vector<at::Tensor>& input, const std::vector<at::Tensor>& output,
               const std::vector<c10::optional<at::Tensor>>& ef, const std::vector<at::Tensor>& status,
               const std::vector<int64_t>& region_ptrs, int64_t recv1_off, int64_t flag1_off, int64_t nchunks,
               int64_t rank0, int64_t chunk_elems, bool stochastic, int64_t epoch, int64_t seed, int64_t step,
               int64_t bucket_id, double out_scale, double timeout_s, int64_t grid_x) {
  const size_t nvr = input.size();
  const size_t world = region_ptrs.size();
  TORCH_CHECK(nvr >= 1 && nvr <= NANGILA_MAX_VRANKS && output.size() == nvr && ef.size() == nvr && status.size() == nvr,
              "nangila: per-rank list length mismatch");
  TORCH_CHECK(world >= 1 && world <= NANGILA_MAX_RANKS, "nangila: bad world size");
  NangilaPredResParams p;
  std::memset(&p, 0, sizeof p);
  p.n = input[0].numel();
  p.world = int32_t(world);
  p.rank0 = int32_t(rank0);
  p.nvr = int32_t(nvr);
  p.chunk_elems = int32_t(chunk_elems);
  p.nchunks = int32_t(nchunks);
  p.grad_dtype = dtype_code(input[0]);
  p.state_dtype = NANGILA_BF16;
  p.mode = 2;
  p.stochastic = stochastic ? 1 : 0;
  p.epoch = uint32_t(epoch);
  p.seed = uint32_t(seed);
  p.step = uint32_t(step);
  p.bucket_id = uint32_t(bucket_id);
  p.mu = 0.0f;
  p.out_scale = float(out_scale);
  p.timeout_ns = uint64_t(timeout_s * 1e9);
  p.grid_x = int32_t(grid_x);
  p.recv1_off = uint64_t(recv1_off);
  p.flag1_off = uint64_t(flag1_off);
  for (size_t v = 0; v < nvr; ++v) {
    TORCH_CHECK(input[v].is_cuda() && input[v].is_contiguous() && input[v].numel() == p.n, "nangila: rs input");
    TORCH_CHECK(output[v].is_cuda() && output[v].is_contiguous() && output[v].numel() * int64_t(world) == p.n &&
                    output[v].scalar_type() == input[v].scalar_type(), "nangila: rs output must be one shard of the input dtype");
    TORCH_CHECK((reinterpret_cast<uintptr_t>(input[v].data_ptr()) & 15u) == 0 &&
                    (reinterpret_cast<uintptr_t>(output[v].data_ptr()) & 15u) == 0, "nangila: rs buffers must be 16-byte aligned");
    p.grad[v] = input[v].data_ptr();
    p.out_shard[v] = output[v].data_ptr();
    if (ef[v].has_value()) {
      TORCH_CHECK(ef[v]->scalar_type() == at::kBFloat16 && ef[v]->numel() == p.n && ef[v]->is_contiguous(), "nangila: rs ef must be bf16[n]");
      p.ef[v] = ef[v]->data_ptr();
    }
    p.status[v] = reinterpret_cast<uint32_t*>(status[v].data_ptr<int32_t>());
  }
  for (size_t r = 0; r < world; ++r) p.region[r] = as_ptr(region_ptrs[r]);
  c10::cuda::CUDAGuard guard(input[0].device());
  check_launch(nangila_predres_launch(&p, at::cuda::getCurrentCUDAStream()), "rs_launch");
}

py::tuple ag_region_layout(int64_t shard_elems, int64_t world, int64_t chunk_elems, int64_t bits) {
  uint64_t r, f;
  uint64_t total = nangila_ag_region_bytes(shard_elems, int32_t(world), int32_t(chunk_elems), int32_t(bits), &r, &f);
  return py::make_tuple(total, r, f);
}
void ag_launch(const std::vector<at::Tensor>& input, const std::vector<at::Tensor>& output,
               const std::vector<at::Tensor>& status, const std::vector<int64_t>& region_ptrs, int64_t recv_off,
               int64_t flag_off, int64_t rank0, int64_t chunk_elems, int64_t bits, int64_t epoch, double timeout_s,
               int64_t grid_x) {
  const size_t nvr = input.size();
  const size_t world = region_ptrs.size();
  TORCH_CHECK(nvr >= 1 && nvr <= NANGILA_MAX_VRANKS && output.size() == nvr && status.size() == nvr, "nangila: list length mismatch");
  NangilaAgParams p;
  std::memset(&p, 0, sizeof p);
  p.shard_elems = input[0].numel();
  p.world = int32_t(world);
  p.rank0 = int32_t(rank0);
  p.nvr = int32_t(nvr);
  p.dtype = dtype_code(input[0]);
  p.chunk_elems = int32_t(chunk_elems);
  p.bits = int32_t(bits);
  p.epoch = uint32_t(epoch);
  p.timeout_ns = uint64_t(timeout_s * 1e9);
  p.grid_x = int32_t(grid_x);
  p.recv_off = uint64_t(recv_off);
  p.flag_off = uint64_t(flag_off);
  for (size_t v = 0; v < nvr; ++v) {
    TORCH_CHECK(input[v].is_cuda() && input[v].is_contiguous() && input[v].numel() == p.shard_elems, "nangila: ag input");
    TORCH_CHECK(output[v].is_cuda() && output[v].is_contiguous() && output[v].numel() == p.shard_elems * int64_t(world) &&
                    output[v].scalar_type() == input[v].scalar_type(), "nangila: ag output must hold world shards of the input dtype");
    TORCH_CHECK((reinterpret_cast<uintptr_t>(input[v].data_ptr()) & 15u) == 0 &&
                    (reinterpret_cast<uintptr_t>(output[v].data_ptr()) & 15u) == 0, "nangila: ag buffers must be 16-byte aligned");
    p.in_shard[v] = input[v].data_ptr();
    p.out_full[v] = output[v].data_ptr();
    p.status[v] = reinterpret_cast<uint32_t*>(status[v].data_ptr<int32_t>());
  }
  for (size_t r = 0; r < world; ++r) p.region[r] = as_ptr(region_ptrs[r]);
  c10::cuda::CUDAGuard guard(input[0].device());
  check_launch(nangila_ag_launch(&p, at::cuda::getCurrentCUDAStream()), "ag_launch");
}

// ---- PowerSGD (tcgen05) ----------------------------------------------------------------------------------
// out (rows x 16 fp32) = M * Bt^T or M^T * Bt^T; zero-fills `out` first (the kernel may split K).
// With `counters` (int32, tiles + 1 zero words) the GEMM's epilogue also starts the cross-rank exchange of its result:
// see nangila_psgd_gemm_push(). The remaining push_* arguments describe the exchange region of this factor.
void psgd_gemm(const at::Tensor& M, const at::Tensor& Bt, bool transposed, at::Tensor out, at::Tensor status,
               double timeout_s, bool zero_out, const c10::optional<at::Tensor>& counters,
               const std::vector<int64_t>& push_region_ptrs, int64_t push_recv_off, int64_t push_flag_off, int64_t push_me,
               int64_t push_rank, int64_t push_epoch, const c10::optional<at::Tensor>& push_epoch_word) {
  TORCH_CHECK(M.is_cuda() && M.dim() == 2 && M.scalar_type() == at::kBFloat16 && M.is_contiguous(), "nangila: M must be a contiguous bf16 matrix");
  const int64_t m = M.size(0), n = M.size(1);
  const int64_t k = transposed ? m : n, rows = transposed ? n : m;
  TORCH_CHECK(Bt.scalar_type() == at::kBFloat16 && Bt.is_contiguous() && Bt.numel() == 16 * k, "nangila: Bt must be bf16[16, K]");
  TORCH_CHECK(out.scalar_type() == at::kFloat && out.is_contiguous() && out.numel() == rows * 16, "nangila: out must be fp32[rows, 16]");
  c10::cuda::CUDAGuard guard(M.device());
  if (zero_out) out.zero_();  // split-K partial sums are added with atomics
  NangilaPsgdPush push;
  std::memset(&push, 0, sizeof push);
  const bool pushing = counters.has_value();
  if (pushing) {
    const int64_t tiles = (rows + 127) / 128;
    TORCH_CHECK(counters->is_cuda() && counters->scalar_type() == at::kInt && counters->is_contiguous() && counters->numel() >= tiles + 1,
                "nangila: counters must be an int32 CUDA tensor of tiles + 1 words");
    TORCH_CHECK(!push_region_ptrs.empty() && int64_t(push_region_ptrs.size()) <= NANGILA_MAX_RANKS, "nangila: bad push regions");
    push.counters = reinterpret_cast<uint32_t*>(counters->data_ptr<int32_t>());
    push.world = int32_t(push_region_ptrs.size());
    push.me = int32_t(push_me);
    push.rank = int32_t(push_rank);
    push.recv_off = uint64_t(push_recv_off);
    push.flag_off = uint64_t(push_flag_off);
    push.epoch = uint32_t(push_epoch);
    if (push_epoch_word.has_value()) {
      TORCH_CHECK(push_epoch_word->is_cuda() && push_epoch_word->scalar_type() == at::kInt, "nangila: the epoch word must be an int32 CUDA tensor");
      push.epoch_dev = reinterpret_cast<const uint32_t*>(push_epoch_word->data_ptr<int32_t>());
    }
    for (size_t r = 0; r < push_region_ptrs.size(); ++r) push.region[r] = as_ptr(push_region_ptrs[r]);
  }
  check_launch(nangila_psgd_gemm_push(M.data_ptr(), int32_t(m), int32_t(n), Bt.data_ptr(), transposed ? 1 : 0, out.data_ptr<float>(),
                                      pushing ? &push : nullptr, reinterpret_cast<uint32_t*>(status.data_ptr<int32_t>()),
                                      uint64_t(timeout_s * 1e9), at::cuda::getCurrentCUDAStream()), "psgd_gemm");
}
void psgd_prep(const at::Tensor& grad, const at::Tensor& ef, at::Tensor mef, c10::optional<at::Tensor> clear0,
               c10::optional<at::Tensor> clear1) {
  TORCH_CHECK(grad.is_cuda() && grad.is_contiguous() && ef.scalar_type() == at::kBFloat16 && mef.scalar_type() == at::kBFloat16 &&
                  ef.numel() == grad.numel() && mef.numel() == grad.numel(), "nangila: psgd_prep shapes");
  c10::cuda::CUDAGuard guard(grad.device());
  float *z0 = nullptr, *z1 = nullptr;
  int64_t n0 = 0, n1 = 0;
  if (clear0.has_value()) {
    TORCH_CHECK(clear0->scalar_type() == at::kFloat && clear0->is_contiguous(), "nangila: clear0 must be fp32");
    z0 = clear0->data_ptr<float>();
    n0 = clear0->numel();
  }
  if (clear1.has_value()) {
    TORCH_CHECK(clear1->scalar_type() == at::kFloat && clear1->is_contiguous(), "nangila: clear1 must be fp32");
    z1 = clear1->data_ptr<float>();
    n1 = clear1->numel();
  }
  check_launch(nangila_psgd_prep(grad.data_ptr(), dtype_code(grad), ef.data_ptr(), mef.data_ptr(), grad.numel(), z0, n0, z1, n1,
                                 at::cuda::getCurrentCUDAStream()), "psgd_prep");
}
void psgd_reconstruct(at::Tensor grad, at::Tensor ef, const at::Tensor& mef, const at::Tensor& P, const at::Tensor& Q,
                      int64_t m, int64_t n, int64_t r) {
  TORCH_CHECK(grad.is_cuda() && grad.is_contiguous() && grad.numel() == m * n && P.numel() == m * 16 && Q.numel() == n * 16 &&
                  P.scalar_type() == at::kFloat && Q.scalar_type() == at::kFloat, "nangila: psgd_reconstruct shapes");
  c10::cuda::CUDAGuard guard(grad.device());
  check_launch(nangila_psgd_reconstruct(grad.data_ptr(), dtype_code(grad), ef.data_ptr(), mef.data_ptr(), P.data_ptr<float>(),
                                        Q.data_ptr<float>(), int32_t(m), int32_t(n), int32_t(r),
                                        at::cuda::getCurrentCUDAStream()), "psgd_reconstruct");
}
py::tuple psgd_exchange_layout(int64_t rows, int64_t rank, int64_t world) {
  uint64_t r, f;
  uint64_t total = nangila_psgd_exchange_region_bytes(int32_t(rows), int32_t(rank), int32_t(world), &r, &f);
  return py::make_tuple(total, r, f);
}
void psgd_exchange(const std::vector<at::Tensor>& local, const std::vector<at::Tensor>& mean_out,
                   const std::vector<at::Tensor>& scratch, const std::vector<at::Tensor>& t_out,
                   const std::vector<at::Tensor>& status, const std::vector<int64_t>& region_ptrs, int64_t recv_off,
                   int64_t flag_off, int64_t rows, int64_t rank, int64_t rank0, bool orth_mean, int64_t epoch,
                   double timeout_s, const c10::optional<at::Tensor>& epoch_word, bool pushed) {
  const size_t nvr = local.size();
  TORCH_CHECK(nvr >= 1 && nvr <= NANGILA_MAX_VRANKS && mean_out.size() == nvr && scratch.size() == nvr && t_out.size() == nvr &&
                  status.size() == nvr, "nangila: list length mismatch");
  NangilaPsgdExchangeParams p;
  std::memset(&p, 0, sizeof p);
  p.rows = int32_t(rows);
  p.rank = int32_t(rank);
  p.world = int32_t(region_ptrs.size());
  p.rank0 = int32_t(rank0);
  p.nvr = int32_t(nvr);
  p.orth_mean = orth_mean ? 1 : 0;
  p.pushed = pushed ? 1 : 0;
  p.epoch = uint32_t(epoch);
  if (epoch_word.has_value()) {
    TORCH_CHECK(epoch_word->is_cuda() && epoch_word->scalar_type() == at::kInt && epoch_word->numel() >= 1,
                "nangila: the epoch word must be an int32 CUDA tensor");
    p.epoch_dev = reinterpret_cast<const uint32_t*>(epoch_word->data_ptr<int32_t>());
  }
  p.timeout_ns = uint64_t(timeout_s * 1e9);
  p.recv_off = uint64_t(recv_off);
  p.flag_off = uint64_t(flag_off);
  for (size_t v = 0; v < nvr; ++v) {
    TORCH_CHECK(local[v].scalar_type() == at::kFloat && local[v].numel() == rows * 16 && mean_out[v].numel() == rows * 16 &&
                    scratch[v].numel() == rows * 16 && t_out[v].scalar_type() == at::kBFloat16 && t_out[v].numel() == rows * 16,
                "nangila: psgd_exchange buffers must be [rows, 16]");
    p.local[v] = local[v].data_ptr<float>();
    p.mean_out[v] = mean_out[v].data_ptr<float>();
    p.scratch[v] = scratch[v].data_ptr<float>();
    p.t_out[v] = t_out[v].data_ptr();
    p.status[v] = reinterpret_cast<uint32_t*>(status[v].data_ptr<int32_t>());
  }
  for (size_t r = 0; r < region_ptrs.size(); ++r) p.region[r] = as_ptr(region_ptrs[r]);
  c10::cuda::CUDAGuard guard(local[0].device());
  check_launch(nangila_psgd_exchange(&p, at::cuda::getCurrentCUDAStream()), "psgd_exchange");
}

}  // namespace

void register_more(py::module_& m) {
  m.def("packet_payload_bytes", &packet_payload_bytes);
  m.def("packet_encode", &packet_encode, py::arg("grad"), py::arg("curr"), py::arg("prev"), py::arg("ef"), py::arg("mu"),
        py::arg("gain"), py::arg("payload"));
  m.def("packet_decode", &packet_decode, py::arg("payload"), py::arg("ndim"), py::arg("curr"), py::arg("prev"), py::arg("mu"),
        py::arg("gain"), py::arg("out"));
  m.def("dgc_region_layout", &dgc_region_layout);
  m.def("dgc_launch", &dgc_launch, py::arg("grad"), py::arg("u"), py::arg("v"), py::arg("scratch"), py::arg("status"),
        py::arg("out_count"), py::arg("region_ptrs"), py::arg("recv_off"), py::arg("flag_off"), py::arg("rank0"),
        py::arg("k"), py::arg("capacity"), py::arg("epoch"), py::arg("momentum"), py::arg("timeout_s"),
        py::arg("grid_x"));
  m.def("psgd_gemm", &psgd_gemm, py::arg("M"), py::arg("Bt"), py::arg("transposed"), py::arg("out"), py::arg("status"),
        py::arg("timeout_s"), py::arg("zero_out") = true, py::arg("counters") = py::none(),
        py::arg("push_region_ptrs") = std::vector<int64_t>{}, py::arg("push_recv_off") = 0, py::arg("push_flag_off") = 0,
        py::arg("push_me") = 0, py::arg("push_rank") = 0, py::arg("push_epoch") = 0, py::arg("push_epoch_word") = py::none());
  m.def("psgd_prep", &psgd_prep, py::arg("grad"), py::arg("ef"), py::arg("mef"), py::arg("clear0") = py::none(),
        py::arg("clear1") = py::none());
  m.def("psgd_reconstruct", &psgd_reconstruct);
  m.def("psgd_exchange_layout", &psgd_exchange_layout);
  m.def("psgd_exchange", &psgd_exchange, py::arg("local"), py::arg("mean_out"), py::arg("scratch"), py::arg("t_out"),
        py::arg("status"), py::arg("region_ptrs"), py::arg("recv_off"), py::arg("flag_off"), py::arg("rows"), py::arg("rank"),
        py::arg("rank0"), py::arg("orth_mean"), py::arg("epoch"), py::arg("timeout_s"), py::arg("epoch_word") = py::none(),
        py::arg("pushed") = false);
  m.def("rs_region_layout", &rs_region_layout);
  m.def("rs_launch", &rs_launch);
  m.def("ag_region_layout", &ag_region_layout);
  m.def("ag_launch", &ag_launch);
  m.def("state_hash", &state_hash, py::arg("tensors"), py::arg("seed") = 0);
  m.def("crc32", &crc32_device);
  m.def("absmax_hist", &absmax_hist, py::arg("x"), py::arg("k"), py::arg("qmax") = 7.0);
  m.def("sculptor_layer_sumsq", &sculptor_layer_sumsq);
  m.def("sculptor_pair_update", &sculptor_pair_update);
  m.def("sculptor_pair_finalize", &sculptor_pair_finalize);
}
