// torch glue (`nangila._cuda`): tensor-typed entry points over the C launchers of
// libnangila_kernels.so. Every function queues work on the current CUDA stream of the tensors'
// device and returns without synchronizing.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

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
void check_cuda_contig(const at::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), "nangila: ", name, " must be a CUDA tensor");
  TORCH_CHECK(t.is_contiguous(), "nangila: ", name, " must be contiguous");
  TORCH_CHECK((reinterpret_cast<uintptr_t>(t.data_ptr()) & 15u) == 0, "nangila: ", name, " must be 16-byte aligned");
}
void check_launch(int err, const char* what) {
  TORCH_CHECK(err == 0, "nangila: ", what, " failed: ", cudaGetErrorString(static_cast<cudaError_t>(err)));
}

py::tuple predres_region_layout(int64_t n, int64_t world, int64_t chunk_elems, int64_t grad_dtype) {
  uint64_t r1, r2, f1, f2;
  uint64_t total = nangila_predres_region_bytes(n, int32_t(world), int32_t(chunk_elems), int32_t(grad_dtype), &r1, &r2, &f1, &f2);
  return py::make_tuple(total, r1, r2, f1, f2);
}

// One launch of the fused bucket kernel. The per-rank lists have one entry per rank emulated in this
// launch: exactly one for a real multi-GPU group, `world` entries for the single-GPU loopback world.
void predres_launch(const std::vector<at::Tensor>& grad, const std::vector<at::Tensor>& prev,
                    const std::vector<at::Tensor>& curr, const std::vector<c10::optional<at::Tensor>>& ef,
                    const std::vector<c10::optional<at::Tensor>>& ef2, const std::vector<c10::optional<at::Tensor>>& stats,
                    const std::vector<at::Tensor>& status, const std::vector<int64_t>& region_ptrs,
                    int64_t recv1_off, int64_t recv2_off, int64_t flag1_off, int64_t flag2_off, int64_t rank0,
                    int64_t chunk_elems, int64_t mode, bool stochastic, bool measure, int64_t epoch, int64_t seed, int64_t step,
                    int64_t bucket_id, double mu, const std::vector<double>& pred_gain, double timeout_s, int64_t grid_x,
                    bool uniform_gain, bool gather, int64_t phase_mask, bool skip_history) {
  const size_t nvr = grad.size();
  TORCH_CHECK(nvr >= 1 && nvr <= NANGILA_MAX_VRANKS, "nangila: bad number of emulated ranks");
  TORCH_CHECK(prev.size() == nvr && curr.size() == nvr && ef.size() == nvr && ef2.size() == nvr &&
                  stats.size() == nvr && status.size() == nvr, "nangila: per-rank list length mismatch");
  const size_t world = region_ptrs.size();
  TORCH_CHECK(world >= 1 && world <= NANGILA_MAX_RANKS, "nangila: bad world size");
  NangilaPredResParams p;
  std::memset(&p, 0, sizeof p);
  const int64_t n = grad[0].numel();
  p.n = n;
  p.world = int32_t(world);
  p.rank0 = int32_t(rank0);
  p.nvr = int32_t(nvr);
  p.chunk_elems = int32_t(chunk_elems);
  p.nchunks = int32_t((n + chunk_elems - 1) / chunk_elems);
  p.grad_dtype = dtype_code(grad[0]);
  p.state_dtype = dtype_code(prev[0]);
  p.mode = int32_t(mode);
  p.stochastic = stochastic ? 1 : 0;
  p.measure = measure ? 1 : 0;
  p.uniform_gain = uniform_gain ? 1 : 0;
  p.gather = gather ? 1 : 0;
  p.phase_mask = int32_t(phase_mask);
  p.skip_history = skip_history ? 1 : 0;
  p.epoch = uint32_t(epoch);
  p.seed = uint32_t(seed);
  p.step = uint32_t(step);
  p.bucket_id = uint32_t(bucket_id);
  p.mu = float(mu);
  TORCH_CHECK(pred_gain.size() == nvr, "nangila: one prediction gain per emulated rank");
  for (size_t v = 0; v < nvr; ++v) p.pred_gain[v] = float(pred_gain[v]);
  p.timeout_ns = uint64_t(timeout_s * 1e9);
  p.grid_x = int32_t(grid_x);
  p.recv1_off = uint64_t(recv1_off);
  p.recv2_off = uint64_t(recv2_off);
  p.flag1_off = uint64_t(flag1_off);
  p.flag2_off = uint64_t(flag2_off);
  const int64_t owned_max = (p.nchunks + int64_t(world) - 1) / int64_t(world);
  for (size_t v = 0; v < nvr; ++v) {
    check_cuda_contig(grad[v], "grad");
    check_cuda_contig(prev[v], "prev");
    check_cuda_contig(curr[v], "curr");
    TORCH_CHECK(grad[v].numel() == n && prev[v].numel() == n && curr[v].numel() == n, "nangila: size mismatch");
    TORCH_CHECK(dtype_code(grad[v]) == p.grad_dtype && dtype_code(prev[v]) == p.state_dtype &&
                    dtype_code(curr[v]) == p.state_dtype, "nangila: dtype mismatch");
    p.grad[v] = grad[v].data_ptr();
    p.prev[v] = prev[v].data_ptr();
    p.curr[v] = curr[v].data_ptr();
    if (ef[v].has_value()) {
      check_cuda_contig(*ef[v], "ef");
      TORCH_CHECK(ef[v]->numel() == n && dtype_code(*ef[v]) == p.state_dtype, "nangila: ef mismatch");
      p.ef[v] = ef[v]->data_ptr();
    }
    if (ef2[v].has_value()) {
      check_cuda_contig(*ef2[v], "ef2");
      TORCH_CHECK(ef2[v]->numel() >= owned_max * chunk_elems && dtype_code(*ef2[v]) == p.state_dtype,
                  "nangila: ef2 must hold owned_chunks * chunk_elems elements of the state dtype");
      p.ef2[v] = ef2[v]->data_ptr();
    }
    if (stats[v].has_value()) {
      TORCH_CHECK(stats[v]->is_cuda() && stats[v]->scalar_type() == at::kFloat && stats[v]->numel() >= 8, "nangila: stats");
      p.stats[v] = stats[v]->data_ptr<float>();
    }
    TORCH_CHECK(status[v].is_cuda() && status[v].scalar_type() == at::kInt && status[v].numel() >= 8, "nangila: status");
    p.status[v] = reinterpret_cast<uint32_t*>(status[v].data_ptr<int32_t>());
  }
  for (size_t r = 0; r < world; ++r) p.region[r] = reinterpret_cast<uint8_t*>(static_cast<uintptr_t>(region_ptrs[r]));
  c10::cuda::CUDAGuard guard(grad[0].device());
  check_launch(nangila_predres_launch(&p, at::cuda::getCurrentCUDAStream()), "predres_launch");
}

void predict_quantize_gamma(const at::Tensor& grad, const at::Tensor& curr, const at::Tensor& prev, double mu,
                            double gamma, at::Tensor out, int64_t step, int64_t layer_id) {
  TORCH_CHECK(grad.is_cuda() && grad.scalar_type() == at::kFloat && grad.is_contiguous(), "grad: fp32 CUDA contiguous");
  TORCH_CHECK(curr.scalar_type() == at::kFloat && prev.scalar_type() == at::kFloat && out.scalar_type() == at::kByte, "dtypes");
  TORCH_CHECK(out.numel() >= (grad.numel() + 1) / 2, "out too small");
  c10::cuda::CUDAGuard guard(grad.device());
  check_launch(nangila_predict_quantize_gamma(grad.data_ptr<float>(), curr.data_ptr<float>(), prev.data_ptr<float>(),
                                              float(mu), float(gamma), out.data_ptr<uint8_t>(), grad.numel(),
                                              uint32_t(step), uint32_t(layer_id), at::cuda::getCurrentCUDAStream()),
               "predict_quantize_gamma");
}
void dequant_reconstruct_gamma(const at::Tensor& packed, const at::Tensor& curr, const at::Tensor& prev, double mu,
                               double gamma, at::Tensor out) {
  TORCH_CHECK(packed.is_cuda() && packed.scalar_type() == at::kByte && out.scalar_type() == at::kFloat, "dtypes");
  TORCH_CHECK(packed.numel() >= (out.numel() + 1) / 2, "packed too small");
  c10::cuda::CUDAGuard guard(out.device());
  check_launch(nangila_dequant_reconstruct_gamma(packed.data_ptr<uint8_t>(), curr.data_ptr<float>(),
                                                 prev.data_ptr<float>(), float(mu), float(gamma), out.data_ptr<float>(),
                                                 out.numel(), at::cuda::getCurrentCUDAStream()),
               "dequant_reconstruct_gamma");
}

// Raw-pointer forms with the reference's positional signature (python.rs:592-751).
int raw_predict_and_quantize(uint64_t gradient_ptr, uint64_t g_current_ptr, uint64_t g_previous_ptr, float momentum,
                             float gamma, uint64_t output_ptr, int64_t n, uint64_t stream_ptr, uint32_t step,
                             uint32_t layer_id) {
  return nangila_predict_quantize_gamma(reinterpret_cast<const float*>(gradient_ptr),
                                        reinterpret_cast<const float*>(g_current_ptr),
                                        reinterpret_cast<const float*>(g_previous_ptr), momentum, gamma,
                                        reinterpret_cast<uint8_t*>(output_ptr), n, step, layer_id,
                                        reinterpret_cast<cudaStream_t>(stream_ptr));
}
int raw_dequantize_and_reconstruct(uint64_t packed_ptr, uint64_t g_current_ptr, uint64_t g_previous_ptr, float momentum,
                                   float gamma, uint64_t output_ptr, int64_t n, uint64_t stream_ptr) {
  return nangila_dequant_reconstruct_gamma(reinterpret_cast<const uint8_t*>(packed_ptr),
                                           reinterpret_cast<const float*>(g_current_ptr),
                                           reinterpret_cast<const float*>(g_previous_ptr), momentum, gamma,
                                           reinterpret_cast<float*>(output_ptr), n,
                                           reinterpret_cast<cudaStream_t>(stream_ptr));
}
int stream_synchronize(uint64_t stream_ptr) { return int(cudaStreamSynchronize(reinterpret_cast<cudaStream_t>(stream_ptr))); }
std::string error_string(int code) { return cudaGetErrorString(static_cast<cudaError_t>(code)); }

}  // namespace

void register_more(py::module_& m);
void register_ddp_hook(py::module_& m);  // ddp_hook.cpp  // other glue translation units append their bindings here

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "nangila torch glue over the sm_100a kernels";
  m.def("predres_region_layout", &predres_region_layout);
  m.def("predres_resident_ctas", []() { return nangila_predres_resident_ctas(); });
  m.def("predres_chunk_elems", [](int64_t n, int64_t resident) { return nangila_predres_chunk_elems(n, int32_t(resident)); });
  m.def("predres_launch", &predres_launch, py::arg("grad"), py::arg("prev"), py::arg("curr"), py::arg("ef"),
        py::arg("ef2"), py::arg("stats"), py::arg("status"), py::arg("region_ptrs"), py::arg("recv1_off"),
        py::arg("recv2_off"), py::arg("flag1_off"), py::arg("flag2_off"), py::arg("rank0"), py::arg("chunk_elems"),
        py::arg("mode"), py::arg("stochastic"), py::arg("measure"), py::arg("epoch"), py::arg("seed"), py::arg("step"),
        py::arg("bucket_id"), py::arg("mu"), py::arg("pred_gain"), py::arg("timeout_s"), py::arg("grid_x"),
        py::arg("uniform_gain") = false, py::arg("gather") = false, py::arg("phase_mask") = 0,
        py::arg("skip_history") = false);
  m.def("predict_quantize_gamma", &predict_quantize_gamma);
  m.def("dequant_reconstruct_gamma", &dequant_reconstruct_gamma);
  m.def("raw_predict_and_quantize", &raw_predict_and_quantize);
  m.def("raw_dequantize_and_reconstruct", &raw_dequantize_and_reconstruct);
  m.def("stream_synchronize", &stream_synchronize);
  m.def("error_string", &error_string);
  register_more(m);
  register_ddp_hook(m);
}
