// pybind11 module `nangila._C`: the host-side core exposed with the class, method and keyword
// names of the reference's Python extension module.
//
// Parity: nangila-hook/src/python.rs:16-97 (SyncMode), :100-126 (CompressorType), :129-195
// (NangilaConfig), :198-248 (Sculptor), :251-557 (NangilaHook), :560-751 (free functions),
// :754-766 (module, __version__ = "0.1.0").
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "checkpoint.hpp"
#include "compressor.hpp"
#include "config.hpp"
#include "dtype.hpp"
#include "hook.hpp"
#include "mask.hpp"
#include "metrics.hpp"
#include "packet.hpp"
#include "predictor.hpp"
#include "q8_23.hpp"
#include "quantizer.hpp"
#include "safe_mode.hpp"
#include "sculptor.hpp"
#include "siphash.hpp"
#include "topology_report.hpp"

namespace py = pybind11;
using namespace nangila;
using farray = py::array_t<float, py::array::c_style | py::array::forcecast>;

namespace {

Tensor to_tensor(const farray& a) {
  py::buffer_info bi = a.request();
  std::vector<size_t> shape;
  for (auto d : bi.shape) shape.push_back(size_t(d));
  if (shape.empty()) shape.push_back(1);
  const float* p = static_cast<const float*>(bi.ptr);
  return Tensor(std::vector<float>(p, p + bi.size), std::move(shape));
}
Tensor to_tensor_flat(const farray& a) {
  py::buffer_info bi = a.request();
  const float* p = static_cast<const float*>(bi.ptr);
  return Tensor(std::vector<float>(p, p + bi.size), {size_t(bi.size)});
}
py::array_t<float> to_array(const std::vector<float>& v) {
  py::array_t<float> a(py::ssize_t(v.size()));
  if (!v.empty()) std::memcpy(a.mutable_data(), v.data(), v.size() * 4);
  return a;
}
py::bytes to_bytes(const std::vector<uint8_t>& v) {
  return py::bytes(reinterpret_cast<const char*>(v.data()), v.size());
}
std::vector<uint8_t> from_bytes(const py::bytes& b) {
  std::string s = b;
  return std::vector<uint8_t>(s.begin(), s.end());
}

struct PySyncMode {
  int mode;
};

CompressorType ctype_from_py(const py::object& o) {
  if (py::isinstance<CompressorType>(o)) return o.cast<CompressorType>();
  int v = o.cast<int>();
  if (v < 0 || v > 2) throw py::value_error("Invalid compressor_type " + std::to_string(v));
  return static_cast<CompressorType>(v);
}

py::dict telemetry_dict(const LayerTelemetry& t) {
  py::dict d;
  d["total_original_bytes"] = t.total_original_bytes;
  d["total_compressed_bytes"] = t.total_compressed_bytes;
  d["compression_count"] = t.compression_count;
  d["avg_compression_ratio"] = t.avg_compression_ratio;
  d["min_compression_ratio"] = t.min_compression_ratio;
  d["max_compression_ratio"] = t.max_compression_ratio;
  d["avg_prediction_error"] = t.avg_prediction_error;
  d["passenger_skip_count"] = t.passenger_skip_count;
  return d;
}

}  // namespace

PYBIND11_MODULE(_C, m) {
  m.doc() = "Nangila host-side core (C++): config, mask, packets, predictor, quantizer, compressors, "
            "Sculptor, hook state machine, Safe Mode, metrics, checkpoints.";
  m.attr("__version__") = "0.1.0";

  py::register_exception_translator([](std::exception_ptr p) {
    try {
      if (p) std::rethrow_exception(p);
    } catch (const NangilaError& e) {
      switch (e.kind()) {
        case ErrorKind::Config: PyErr_SetString(PyExc_ValueError, e.what()); break;
        case ErrorKind::Io: PyErr_SetString(PyExc_IOError, e.what()); break;
        default: PyErr_SetString(PyExc_RuntimeError, e.what()); break;
      }
    }
  });

  // --- SyncMode ------------------------------------------------------------------------------
  py::class_<PySyncMode>(m, "SyncMode")
      .def(py::init([](int mode) {
             if (mode < 0 || mode > 2)
               throw py::value_error("Invalid sync mode. Use SyncMode.ASYNC (0), ALWAYS (1), or PERIODIC (2)");
             return PySyncMode{mode};
           }),
           py::arg("mode"))
      .def_property_readonly("mode", [](const PySyncMode& s) { return s.mode; })
      .def("__int__", [](const PySyncMode& s) { return s.mode; })
      .def("__index__", [](const PySyncMode& s) { return s.mode; })
      .def("__eq__", [](const PySyncMode& s, const py::object& o) {
        if (py::isinstance<PySyncMode>(o)) return o.cast<PySyncMode>().mode == s.mode;
        if (py::isinstance<py::int_>(o)) return o.cast<int>() == s.mode;
        return false;
      })
      .def("__hash__", [](const PySyncMode& s) { return s.mode; })
      .def("__repr__", [](const PySyncMode& s) { return std::string(sync_mode_name(SyncMode(s.mode))); })
      .def_property_readonly_static("ASYNC", [](py::object) { return 0; })
      .def_property_readonly_static("ALWAYS", [](py::object) { return 1; })
      .def_property_readonly_static("PERIODIC", [](py::object) { return 2; });

  // --- CompressorType ------------------------------------------------------------------------
  py::enum_<CompressorType> ctype(m, "CompressorType", py::arithmetic());
  ctype.value("PredictionResidual", CompressorType::PredictionResidual)
      .value("DGC", CompressorType::DGC)
      .value("PowerSGD", CompressorType::PowerSGD);
  // Members compare equal to their integer values (0, 1, 2), like the reference's enum.
  ctype.attr("__eq__") = py::cpp_function(
      [](const CompressorType& a, const py::object& b) {
        if (py::isinstance<CompressorType>(b)) return b.cast<CompressorType>() == a;
        if (py::isinstance<py::int_>(b)) return b.cast<long>() == long(a);
        return false;
      },
      py::is_method(ctype));
  ctype.attr("__ne__") = py::cpp_function(
      [](const CompressorType& a, const py::object& b) {
        if (py::isinstance<CompressorType>(b)) return b.cast<CompressorType>() != a;
        if (py::isinstance<py::int_>(b)) return b.cast<long>() != long(a);
        return true;
      },
      py::is_method(ctype));

  // --- NangilaConfig -------------------------------------------------------------------------
  py::class_<NangilaConfig>(m, "NangilaConfig")
      .def(py::init([](float momentum, float threshold, size_t warmup_steps, size_t shadow_run_steps,
                       int quantize_bits, py::object compressor_type, float dgc_sparsity, size_t power_sgd_rank) {
             if (quantize_bits < 0 || quantize_bits > 255) throw py::value_error("Invalid quantize_bits");
             NangilaConfig c;
             c.momentum = momentum;
             c.sculptor_threshold = threshold;
             c.warmup_steps = warmup_steps;
             c.shadow_run_steps = shadow_run_steps;
             c.quantize_bits = uint8_t(quantize_bits);
             c.compressor_type = ctype_from_py(compressor_type);
             c.dgc_sparsity = dgc_sparsity;
             c.power_sgd_rank = power_sgd_rank;
             c.validate();
             return c;
           }),
           py::arg("momentum") = 0.9f, py::arg("threshold") = 0.95f, py::arg("warmup_steps") = 1000,
           py::arg("shadow_run_steps") = 100, py::arg("quantize_bits") = 4,
           py::arg("compressor_type") = CompressorType::PredictionResidual, py::arg("dgc_sparsity") = 0.999f,
           py::arg("power_sgd_rank") = 1)
      .def_static("conservative", &NangilaConfig::conservative)
      .def_static("aggressive", &NangilaConfig::aggressive)
      .def("validate", &NangilaConfig::validate)
      .def_readwrite("momentum", &NangilaConfig::momentum)
      .def_readwrite("threshold", &NangilaConfig::sculptor_threshold)
      .def_readwrite("sculptor_threshold", &NangilaConfig::sculptor_threshold)
      .def_readwrite("warmup_steps", &NangilaConfig::warmup_steps)
      .def_readwrite("shadow_run_steps", &NangilaConfig::shadow_run_steps)
      .def_property("quantize_bits", [](const NangilaConfig& c) { return int(c.quantize_bits); },
                    [](NangilaConfig& c, int b) { c.quantize_bits = uint8_t(b); })
      .def_readwrite("dynamic_gamma", &NangilaConfig::dynamic_gamma)
      .def_readwrite("monitor_interval", &NangilaConfig::monitor_interval)
      .def_readwrite("monitor_sample_fraction", &NangilaConfig::monitor_sample_fraction)
      .def_readwrite("promotion_threshold", &NangilaConfig::promotion_threshold)
      .def_readwrite("compressor_type", &NangilaConfig::compressor_type)
      .def_readwrite("dgc_sparsity", &NangilaConfig::dgc_sparsity)
      .def_readwrite("power_sgd_rank", &NangilaConfig::power_sgd_rank)
      .def("__repr__", [](const NangilaConfig& c) {
        return "NangilaConfig(momentum=" + std::to_string(c.momentum) + ", threshold=" +
               std::to_string(c.sculptor_threshold) + ", warmup_steps=" + std::to_string(c.warmup_steps) +
               ", shadow_run_steps=" + std::to_string(c.shadow_run_steps) + ", quantize_bits=" +
               std::to_string(int(c.quantize_bits)) + ", compressor_type=" + std::to_string(int(c.compressor_type)) +
               ", dgc_sparsity=" + std::to_string(c.dgc_sparsity) + ", power_sgd_rank=" +
               std::to_string(c.power_sgd_rank) + ")";
      });

  // --- fixed point / hashing / dtype helpers ---------------------------------------------------
  m.def("q8_23_from_f32", [](float f) { return Q8_23::from_f32(f).bits; });
  m.def("q8_23_to_f32", [](int32_t b) { return Q8_23{b}.to_f32(); });
  m.def("q8_23_add", [](int32_t a, int32_t b) { return (Q8_23{a} + Q8_23{b}).bits; });
  m.def("q8_23_sub", [](int32_t a, int32_t b) { return (Q8_23{a} - Q8_23{b}).bits; });
  m.def("q8_23_mul", [](int32_t a, int32_t b) { return (Q8_23{a} * Q8_23{b}).bits; });
  m.def("q8_23_fma", [](int32_t s, int32_t a, int32_t b) { return Q8_23{s}.fma(Q8_23{a}, Q8_23{b}).bits; });
  m.def("q8_23_saturation_count", [] { return q823_saturation_counter().load(); });
  m.def("fixed_buffer_hash", [](const farray& a) { return FixedPointBuffer::from_f32(to_tensor_flat(a).data).hash(); });
  m.def("fixed_buffer_roundtrip", [](const farray& a) { return to_array(FixedPointBuffer::from_f32(to_tensor_flat(a).data).to_f32()); });
  m.def("fixed_buffer_auto_clip", [](const farray& a) { return to_array(FixedPointBuffer::from_f32_auto_clip(to_tensor_flat(a).data).to_f32()); });
  m.def("siphash13", [](const py::bytes& b, uint64_t k0, uint64_t k1) {
    std::string s = b;
    SipHasher13 h(k0, k1);
    h.write(s.data(), s.size());
    return h.finish();
  }, py::arg("data"), py::arg("k0") = 0, py::arg("k1") = 0);
  m.def("siphash24", [](const py::bytes& b, uint64_t k0, uint64_t k1) {
    std::string s = b;
    SipHasher24 h(k0, k1);
    h.write(s.data(), s.size());
    return h.finish();
  }, py::arg("data"), py::arg("k0") = 0, py::arg("k1") = 0);
  m.def("crc32", [](const py::bytes& b) {
    std::string s = b;
    return compute_crc32(reinterpret_cast<const uint8_t*>(s.data()), s.size());
  });
  m.def("f32_to_f16_bytes", [](const farray& a) { auto t = to_tensor_flat(a); return to_bytes(f32_to_f16_bytes(t.data.data(), t.data.size())); });
  m.def("f32_to_bf16_bytes", [](const farray& a) { auto t = to_tensor_flat(a); return to_bytes(f32_to_bf16_bytes(t.data.data(), t.data.size())); });
  m.def("f16_bytes_to_f32", [](const py::bytes& b) { auto v = from_bytes(b); return to_array(f16_bytes_to_f32(v.data(), v.size())); });
  m.def("bf16_bytes_to_f32", [](const py::bytes& b) { auto v = from_bytes(b); return to_array(bf16_bytes_to_f32(v.data(), v.size())); });

  // --- packets ---------------------------------------------------------------------------------
  py::class_<PacketHeader>(m, "PacketHeader")
      .def(py::init<>())
      .def_static("new_driver", &PacketHeader::new_driver)
      .def_static("new_passenger", &PacketHeader::new_passenger)
      .def_static("new_force_sync", &PacketHeader::new_force_sync)
      .def_static("new_partial_retransmit", &PacketHeader::new_partial_retransmit)
      .def_readwrite("magic", &PacketHeader::magic)
      .def_readwrite("version", &PacketHeader::version)
      .def_readwrite("flags", &PacketHeader::flags)
      .def_readwrite("step", &PacketHeader::step)
      .def_readwrite("layer_id", &PacketHeader::layer_id)
      .def_readwrite("crc32", &PacketHeader::crc32)
      .def_readwrite("predictor_hash", &PacketHeader::predictor_hash)
      .def_readwrite("start_offset", &PacketHeader::start_offset)
      .def_readwrite("end_offset", &PacketHeader::end_offset)
      .def("is_valid", &PacketHeader::is_valid)
      .def("is_force_sync", &PacketHeader::is_force_sync)
      .def("is_driver", &PacketHeader::is_driver)
      .def("is_passenger", &PacketHeader::is_passenger)
      .def("is_desync_recovery", &PacketHeader::is_desync_recovery)
      .def("is_partial_retransmit", &PacketHeader::is_partial_retransmit)
      .def("to_bytes", [](const PacketHeader& h) {
        auto b = h.to_bytes();
        return py::bytes(reinterpret_cast<const char*>(b.data()), b.size());
      })
      .def_static("from_bytes", [](const py::bytes& b) -> py::object {
        auto v = from_bytes(b);
        auto h = PacketHeader::from_bytes(v.data(), v.size());
        if (!h) return py::none();
        return py::cast(*h);
      })
      .def("__eq__", &PacketHeader::operator==);
  m.attr("PACKET_HEADER_SIZE") = PacketHeader::SIZE;
  py::class_<Packet>(m, "Packet")
      .def(py::init([](PacketHeader h, const py::bytes& payload) { return Packet(h, from_bytes(payload)); }))
      .def_readwrite("header", &Packet::header)
      .def_property("payload", [](const Packet& p) { return to_bytes(p.payload); },
                    [](Packet& p, const py::bytes& b) { p.payload = from_bytes(b); })
      .def("verify", &Packet::verify)
      .def("to_bytes", [](const Packet& p) { return to_bytes(p.to_bytes()); })
      .def_static("from_bytes", [](const py::bytes& b) -> py::object {
        auto v = from_bytes(b);
        auto p = Packet::from_bytes(v.data(), v.size());
        if (!p) return py::none();
        return py::cast(*p);
      });
  py::module_ fl = m.def_submodule("flags");
  fl.attr("FORCE_SYNC") = flags::FORCE_SYNC;
  fl.attr("DRIVER") = flags::DRIVER;
  fl.attr("PASSENGER") = flags::PASSENGER;
  fl.attr("ACK_REQUEST") = flags::ACK_REQUEST;
  fl.attr("ACK_RESPONSE") = flags::ACK_RESPONSE;
  fl.attr("DESYNC_RECOVERY") = flags::DESYNC_RECOVERY;
  fl.attr("PARTIAL_RETRANSMIT") = flags::PARTIAL_RETRANSMIT;

  // --- mask ------------------------------------------------------------------------------------
  py::class_<TopologyMask>(m, "TopologyMask")
      .def(py::init<>())
      .def_static("all_drivers", &TopologyMask::all_drivers)
      .def_static("from_bytes", [](const py::bytes& b) {
        auto v = from_bytes(b);
        return TopologyMask::from_bytes(v.data(), v.size());
      })
      .def("to_bytes", [](const TopologyMask& mk) { return to_bytes(mk.to_bytes()); })
      .def("add_driver", &TopologyMask::add_driver)
      .def("add_passenger", &TopologyMask::add_passenger)
      .def("add_passenger_checked", &TopologyMask::add_passenger_checked)
      .def("is_driver", &TopologyMask::is_driver)
      .def("is_passenger", &TopologyMask::is_passenger)
      .def("get_role", [](const TopologyMask& mk, LayerId id) -> py::object {
        const LayerRole& r = mk.get_role(id);
        if (r.is_driver()) return py::make_tuple("driver");
        return py::make_tuple("passenger", r.source_id, r.alpha, r.beta);
      })
      .def("drivers", &TopologyMask::drivers)
      .def("passengers", [](const TopologyMask& mk) {
        py::list l;
        for (auto& p : mk.passengers()) l.append(py::make_tuple(p.id, p.source, p.alpha, p.beta));
        return l;
      })
      .def("num_drivers", &TopologyMask::num_drivers)
      .def("num_passengers", &TopologyMask::num_passengers)
      .def("num_layers", &TopologyMask::num_layers)
      .def("compression_ratio", &TopologyMask::compression_ratio)
      .def("fsdp_ordered_layers", &TopologyMask::fsdp_ordered_layers)
      .def("prefetch_hints", &TopologyMask::prefetch_hints)
      .def("dependencies_ready", [](const TopologyMask& mk, LayerId id, const std::set<LayerId>& ready) {
        return mk.dependencies_ready(id, ready);
      })
      .def("promote_to_driver", &TopologyMask::promote_to_driver)
      .def("validate", &TopologyMask::validate)
      .def("report_json", [](const TopologyMask& mk, bool pretty) { return TopologyReport::from_mask(mk).to_json(pretty); },
           py::arg("pretty") = true);

  // --- predictor ---------------------------------------------------------------------------------
  py::enum_<MemoryMode>(m, "MemoryMode")
      .value("Full", MemoryMode::Full)
      .value("DriversOnly", MemoryMode::DriversOnly)
      .value("Auto", MemoryMode::Auto);
  py::class_<Predictor>(m, "Predictor")
      .def(py::init<float, size_t>(), py::arg("momentum") = 0.9f, py::arg("warmup_steps") = 0)
      .def("update", [](Predictor& p, LayerId id, const farray& g) { p.update(id, to_tensor_flat(g)); })
      .def("predict", [](const Predictor& p, LayerId id) { return to_array(p.predict(id).data); })
      .def("predict_partial", [](const Predictor& p, LayerId id, size_t s, size_t e) { return to_array(p.predict_partial(id, s, e).data); })
      .def("can_predict", &Predictor::can_predict)
      .def("step", &Predictor::step)
      .def("is_ready", &Predictor::is_ready)
      .def("current_step", &Predictor::current_step)
      .def("momentum", &Predictor::momentum)
      .def("get_momentum", &Predictor::get_momentum)
      .def("record_error", &Predictor::record_error)
      .def("set_adaptive_config", &Predictor::set_adaptive_config)
      .def("set_memory_mode", &Predictor::set_memory_mode)
      .def("set_large_model_threshold", &Predictor::set_large_model_threshold)
      .def("set_driver_layers", &Predictor::set_driver_layers)
      .def("should_track_layer", &Predictor::should_track_layer)
      .def("memory_stats", [](const Predictor& p) {
        auto s = p.memory_stats();
        return py::make_tuple(s.mode, s.total_params, s.num_layers, s.estimated_mb);
      })
      .def("state_hash", &Predictor::state_hash)
      .def("reset", &Predictor::reset)
      .def("reset_layer", &Predictor::reset_layer)
      .def("num_tracked_layers", &Predictor::num_tracked_layers)
      .def("force_sync_layer", [](Predictor& p, LayerId id, const farray& g) { p.force_sync_layer(id, to_tensor_flat(g)); })
      .def("export_snapshots", [](const Predictor& p) {
        py::dict d;
        for (auto& kv : p.export_snapshots()) {
          py::object pr = kv.second.prev ? py::cast(*kv.second.prev) : py::none();
          py::object cu = kv.second.current ? py::cast(*kv.second.current) : py::none();
          d[py::int_(kv.first)] = py::make_tuple(pr, cu);
        }
        return d;
      })
      .def("restore_snapshots", [](Predictor& p, const py::dict& d) {
        std::map<LayerId, LayerHistorySnapshot> snaps;
        for (auto item : d) {
          py::tuple t = item.second.cast<py::tuple>();
          LayerHistorySnapshot s;
          if (!t[0].is_none()) s.prev = t[0].cast<std::vector<int32_t>>();
          if (!t[1].is_none()) s.current = t[1].cast<std::vector<int32_t>>();
          snaps[item.first.cast<LayerId>()] = std::move(s);
        }
        p.restore_snapshots(snaps);
      });

  // --- quantizer ---------------------------------------------------------------------------------
  py::class_<CompressedTensor>(m, "CompressedTensor")
      .def(py::init<>())
      .def_property("data", [](const CompressedTensor& c) { return to_bytes(c.data); },
                    [](CompressedTensor& c, const py::bytes& b) { c.data = from_bytes(b); })
      .def_readwrite("gamma", &CompressedTensor::gamma)
      .def_readwrite("shape", &CompressedTensor::shape)
      .def_readwrite("numel", &CompressedTensor::numel)
      .def("size_bytes", &CompressedTensor::size_bytes)
      .def("compression_ratio", &CompressedTensor::compression_ratio);
  py::class_<Quantizer>(m, "Quantizer")
      .def(py::init<uint8_t, bool, bool>(), py::arg("bits") = 4, py::arg("dynamic_gamma") = true,
           py::arg("reference_exact") = false)
      .def_static("int4", &Quantizer::int4)
      .def("compute_gamma", [](const Quantizer& q, const farray& a) { return q.compute_gamma(to_tensor_flat(a)); })
      .def("quantize", [](Quantizer& q, const farray& a, uint32_t layer, uint64_t step, size_t off) {
        return q.quantize_with_offset(to_tensor(a), layer, step, off);
      }, py::arg("tensor"), py::arg("layer_id") = 0, py::arg("step") = 0, py::arg("global_offset") = 0)
      .def("dequantize", [](const Quantizer& q, const CompressedTensor& c) { return to_array(q.dequantize(c).data); })
      .def("dequantize_partial", [](const Quantizer& q, const CompressedTensor& c, size_t s, size_t e) {
        return to_array(q.dequantize_partial(c, s, e).data);
      })
      .def("unpack", [](const Quantizer& q, const CompressedTensor& c) { return q.unpack(c); })
      .def("gamma", &Quantizer::gamma)
      .def("set_gamma", &Quantizer::set_gamma)
      .def("set_dynamic_gamma", &Quantizer::set_dynamic_gamma)
      .def("set_stochastic", &Quantizer::set_stochastic)
      .def("set_seed", &Quantizer::set_seed);
  m.def("pack_int4", [](const std::vector<int8_t>& v) { return to_bytes(pack_int4(v)); });
  m.def("unpack_int4", [](const py::bytes& b, size_t n) { return unpack_int4(from_bytes(b), n); });

  // --- compressors (host) --------------------------------------------------------------------------
  struct PyCompressor {
    std::unique_ptr<Compressor> c;
  };
  py::class_<PyCompressor>(m, "HostCompressor")
      .def(py::init([](const NangilaConfig& cfg, float dgc_momentum, bool error_feedback, bool reference_exact) {
             PyCompressor p;
             if (cfg.compressor_type == CompressorType::DGC) p.c = std::make_unique<DGCCompressor>(cfg, dgc_momentum);
             else if (cfg.compressor_type == CompressorType::PowerSGD) p.c = std::make_unique<PowerSGDCompressor>(cfg);
             else p.c = std::make_unique<PredictionResidualCompressor>(cfg, error_feedback, reference_exact);
             return p;
           }),
           py::arg("config"), py::arg("dgc_momentum") = 0.0f, py::arg("error_feedback") = true,
           py::arg("reference_exact") = false)
      .def("name", [](const PyCompressor& p) { return std::string(p.c->name()); })
      .def("compress", [](PyCompressor& p, const farray& g, LayerId id) { return to_bytes(p.c->compress(to_tensor(g), id).to_bytes()); })
      .def("decompress", [](PyCompressor& p, const py::bytes& b, LayerId id) {
        auto v = from_bytes(b);
        auto pk = Packet::from_bytes(v.data(), v.size());
        if (!pk || !pk->verify()) throw NangilaError::invalid_format("bad packet");
        return to_array(p.c->decompress(*pk, id).data);
      })
      .def("update", [](PyCompressor& p, LayerId id, const farray& g) { p.c->update(id, to_tensor_flat(g)); })
      .def("step", [](PyCompressor& p) { p.c->step(); })
      .def("state_hash", [](const PyCompressor& p) { return p.c->state_hash(); })
      .def("last_compression_ratio", [](const PyCompressor& p) { return p.c->last_compression_ratio(); })
      .def("last_prediction_error", [](const PyCompressor& p) { return p.c->last_prediction_error(); })
      .def("quantizer_gamma", [](const PyCompressor& p) { return p.c->quantizer_gamma(); });
  m.def("dgc_top_k", [](const farray& a, size_t k) { return DGCCompressor::top_k(to_tensor_flat(a).data, k); });
  m.def("dgc_keep_count", &DGCCompressor::keep_count);
  m.def("orthogonalize_columns", [](const farray& a) {
    py::buffer_info bi = a.request();
    if (bi.ndim != 2) throw py::value_error("expected a 2-D array");
    Mat mt(size_t(bi.shape[0]), size_t(bi.shape[1]));
    std::memcpy(mt.a.data(), bi.ptr, mt.a.size() * 4);
    orthogonalize_columns(mt);
    py::array_t<float> out({bi.shape[0], bi.shape[1]});
    std::memcpy(out.mutable_data(), mt.a.data(), mt.a.size() * 4);
    return out;
  });
  m.def("powersgd_initial_q", [](size_t n, size_t r) {
    Mat q = PowerSGDCompressor::initial_q(n, r);
    py::array_t<float> out({py::ssize_t(n), py::ssize_t(r)});
    std::memcpy(out.mutable_data(), q.a.data(), q.a.size() * 4);
    return out;
  });

  // --- Sculptor ------------------------------------------------------------------------------------
  py::class_<Sculptor>(m, "Sculptor")
      .def(py::init<float>(), py::arg("threshold") = 0.95f)
      .def_static("new_large_model", &Sculptor::new_large_model)
      .def("record", [](Sculptor& s, LayerId id, const farray& g) {
        py::buffer_info bi = g.request();
        s.record(id, static_cast<const float*>(bi.ptr), size_t(bi.size));
      })
      .def("record_norm", &Sculptor::record_norm)
      .def("end_step", &Sculptor::end_step)
      .def("note_step", &Sculptor::note_step)
      .def("set_pair_result", &Sculptor::set_pair_result)
      .def("scheduled_pairs", &Sculptor::scheduled_pairs)
      .def("set_sampling_strategy", [](Sculptor& s, const std::string& kind, size_t param) {
        SamplingStrategy st;
        if (kind == "full") st.kind = SamplingStrategy::Full;
        else if (kind == "knn") st.kind = SamplingStrategy::KNearestNeighbors;
        else if (kind == "random") st.kind = SamplingStrategy::RandomSampling;
        else if (kind == "hierarchical") st.kind = SamplingStrategy::Hierarchical;
        else throw py::value_error("unknown sampling strategy " + kind);
        st.param = param;
        s.set_sampling_strategy(st);
      }, py::arg("kind"), py::arg("param") = 0)
      .def("generate_mask", [](Sculptor& s) {
        if (s.has_open_step()) s.end_step();
        return to_bytes(s.generate_mask().to_bytes());
      })
      .def("correlation", [](const Sculptor& s, LayerId a, LayerId b) -> py::object {
        auto c = s.correlation(a, b);
        if (!c) return py::none();
        return py::float_(*c);
      })
      .def("coupling", [](const Sculptor& s, LayerId d, LayerId p) -> py::object {
        auto c = s.coupling(d, p);
        if (!c) return py::none();
        return py::make_tuple(c->first, c->second);
      })
      .def("correlation_matrix", [](const Sculptor& s) -> py::object {
        auto mtx = s.correlation_matrix();
        if (!mtx) return py::none();
        return py::cast(*mtx);
      })
      .def("report_json", [](Sculptor& s, bool pretty) {
        if (s.has_open_step()) s.end_step();
        TopologyMask mk = s.generate_mask();
        return TopologyReport::from_sculptor_and_mask(s, mk).to_json(pretty);
      }, py::arg("pretty") = true)
      .def("num_samples", &Sculptor::num_samples)
      .def("num_layers", &Sculptor::num_layers)
      .def("num_steps", &Sculptor::num_steps)
      .def("num_pairs", &Sculptor::num_pairs)
      .def("threshold", &Sculptor::threshold)
      .def("layer_ids", &Sculptor::layer_ids)
      .def("norm_std_dev", &Sculptor::norm_std_dev)
      .def("reset", &Sculptor::reset);

  // --- Safe Mode -------------------------------------------------------------------------------------
  py::class_<SafeModeConfig>(m, "SafeModeConfig")
      .def(py::init([](size_t check_interval, float divergence_threshold, uint32_t max_consecutive_failures,
                       size_t recovery_cooldown, float canary_fraction, size_t canary_steps, uint32_t canary_max_failures) {
             return SafeModeConfig{check_interval, divergence_threshold, max_consecutive_failures,
                                   recovery_cooldown, canary_fraction, canary_steps, canary_max_failures};
           }),
           py::arg("check_interval") = 100, py::arg("divergence_threshold") = 0.005f,
           py::arg("max_consecutive_failures") = 3, py::arg("recovery_cooldown") = 500,
           py::arg("canary_fraction") = 0.1f, py::arg("canary_steps") = 100, py::arg("canary_max_failures") = 2)
      .def_static("conservative", &SafeModeConfig::conservative)
      .def_static("relaxed", &SafeModeConfig::relaxed)
      .def_readwrite("check_interval", &SafeModeConfig::check_interval)
      .def_readwrite("divergence_threshold", &SafeModeConfig::divergence_threshold)
      .def_readwrite("max_consecutive_failures", &SafeModeConfig::max_consecutive_failures)
      .def_readwrite("recovery_cooldown", &SafeModeConfig::recovery_cooldown)
      .def_readwrite("canary_fraction", &SafeModeConfig::canary_fraction)
      .def_readwrite("canary_steps", &SafeModeConfig::canary_steps)
      .def_readwrite("canary_max_failures", &SafeModeConfig::canary_max_failures);
  py::enum_<SafeModeAction>(m, "SafeModeAction")
      .value("Continue", SafeModeAction::Continue)
      .value("TriggerFallback", SafeModeAction::TriggerFallback)
      .value("RecoveryComplete", SafeModeAction::RecoveryComplete)
      .value("NoCheck", SafeModeAction::NoCheck)
      .value("CanaryTest", SafeModeAction::CanaryTest);
  py::enum_<SafeModeState>(m, "SafeModeState")
      .value("Active", SafeModeState::Active)
      .value("Fallback", SafeModeState::Fallback)
      .value("Recovering", SafeModeState::Recovering)
      .value("Canary", SafeModeState::Canary);
  py::class_<SafeMode>(m, "SafeMode")
      .def(py::init<SafeModeConfig>(), py::arg("config") = SafeModeConfig{})
      .def("should_check", &SafeMode::should_check)
      .def("check", &SafeMode::check)
      .def("should_compress", &SafeMode::should_compress)
      .def("state", &SafeMode::state)
      .def("force_fallback", &SafeMode::force_fallback)
      .def("enter_canary", &SafeMode::enter_canary)
      .def("reset", &SafeMode::reset)
      .def("stats", [](const SafeMode& s) {
        SafeModeStats st = s.stats();
        py::dict d;
        auto opt = [](const std::optional<float>& o) -> py::object { return o ? py::object(py::float_(*o)) : py::none(); };
        d["state"] = st.state;
        d["baseline_loss"] = opt(st.baseline_loss);
        d["last_loss"] = opt(st.last_loss);
        d["ema_loss_short"] = opt(st.ema_loss_short);
        d["ema_loss_long"] = opt(st.ema_loss_long);
        d["failure_count"] = st.failure_count;
        d["cooldown_remaining"] = st.cooldown_remaining;
        d["total_fallbacks"] = st.total_fallbacks;
        return d;
      });

  // --- metrics ---------------------------------------------------------------------------------------
  py::class_<MetricsCollector>(m, "MetricsCollector")
      .def(py::init<>())
      .def("record_step", &MetricsCollector::record_step)
      .def("record_bytes", &MetricsCollector::record_bytes)
      .def("record_fallback", &MetricsCollector::record_fallback)
      .def("set_compression_ratio", &MetricsCollector::set_compression_ratio)
      .def("reset", &MetricsCollector::reset)
      .def("to_prometheus", [](const MetricsCollector& c) { return c.snapshot().to_prometheus(); })
      .def("to_json", [](const MetricsCollector& c) { return c.snapshot().to_json(); })
      .def("snapshot", [](const MetricsCollector& c) {
        NangilaMetrics s = c.snapshot();
        py::dict d;
        d["compression_ratio"] = s.compression_ratio;
        d["virtual_throughput_gbps"] = s.virtual_throughput_gbps;
        d["physical_throughput_gbps"] = s.physical_throughput_gbps;
        d["steps_total"] = s.steps_total;
        d["steps_compressed"] = s.steps_compressed;
        d["bytes_received"] = s.bytes_received;
        d["bytes_transmitted"] = s.bytes_transmitted;
        d["bytes_saved"] = s.bytes_saved;
        d["fallback_count"] = s.fallback_count;
        d["uptime_seconds"] = s.uptime_seconds;
        return d;
      });

  // --- checkpoint --------------------------------------------------------------------------------------
  py::class_<NangilaCheckpoint>(m, "NangilaCheckpoint")
      .def(py::init<>())
      .def_static("load", &NangilaCheckpoint::load)
      .def_static("from_bytes", [](const py::bytes& b) {
        auto v = from_bytes(b);
        return NangilaCheckpoint::from_bytes(v.data(), v.size());
      })
      .def("save", &NangilaCheckpoint::save)
      .def("to_bytes", [](const NangilaCheckpoint& c) { return to_bytes(c.to_bytes()); })
      .def("compute_hash", &NangilaCheckpoint::compute_hash)
      .def("verify_integrity", &NangilaCheckpoint::verify_integrity)
      .def("seal", &NangilaCheckpoint::seal)
      .def_readwrite("version", &NangilaCheckpoint::version)
      .def_readwrite("step", &NangilaCheckpoint::step)
      .def_readwrite("state_hash", &NangilaCheckpoint::state_hash)
      .def_readwrite("quantizer_gamma", &NangilaCheckpoint::quantizer_gamma)
      .def_readwrite("config", &NangilaCheckpoint::config)
      .def_property("predictor_step", [](const NangilaCheckpoint& c) { return c.predictor.current_step; },
                    [](NangilaCheckpoint& c, size_t s) { c.predictor.current_step = s; })
      .def_property("momentum", [](const NangilaCheckpoint& c) { return c.predictor.momentum; },
                    [](NangilaCheckpoint& c, float f) { c.predictor.momentum = f; })
      .def("layer_ids", [](const NangilaCheckpoint& c) {
        std::vector<LayerId> v;
        for (auto& kv : c.predictor.histories) v.push_back(kv.first);
        return v;
      })
      .def("get_layer", [](const NangilaCheckpoint& c, LayerId id) -> py::object {
        auto it = c.predictor.histories.find(id);
        if (it == c.predictor.histories.end()) return py::none();
        py::object pr = it->second.prev ? py::cast(*it->second.prev) : py::none();
        py::object cu = it->second.current ? py::cast(*it->second.current) : py::none();
        return py::make_tuple(pr, cu);
      })
      .def("set_layer", [](NangilaCheckpoint& c, LayerId id, py::object prev, py::object cur) {
        LayerHistorySnapshot s;
        if (!prev.is_none()) s.prev = prev.cast<std::vector<int32_t>>();
        if (!cur.is_none()) s.current = cur.cast<std::vector<int32_t>>();
        c.predictor.histories[id] = std::move(s);
      })
      .def("extra_sections", [](const NangilaCheckpoint& c) {
        py::list l;
        for (auto& s : c.extra) l.append(py::make_tuple(s.name, s.layer_id, to_array(s.data)));
        return l;
      })
      .def("add_extra", [](NangilaCheckpoint& c, const std::string& name, LayerId id, const farray& a) {
        c.extra.push_back({name, id, to_tensor_flat(a).data});
        c.version = NangilaCheckpoint::VERSION_EXT;
      });
  py::class_<GradientHistory>(m, "GradientHistory")
      .def(py::init<size_t>(), py::arg("max_depth") = 10)
      .def("push", [](GradientHistory& h, LayerId id, const farray& a) { h.push(id, FixedPointBuffer::from_f32(to_tensor_flat(a).data)); })
      .def("get", [](const GradientHistory& h, LayerId id, size_t ago) -> py::object {
        const FixedPointBuffer* b = h.get(id, ago);
        if (!b) return py::none();
        return to_array(b->to_f32());
      })
      .def("rewind", [](GradientHistory& h, LayerId id, size_t steps) -> py::object {
        auto b = h.rewind(id, steps);
        if (!b) return py::none();
        return to_array(b->to_f32());
      })
      .def("depth", &GradientHistory::depth)
      .def("clear", &GradientHistory::clear)
      .def("clear_layer", &GradientHistory::clear_layer);

  // --- NangilaHook -----------------------------------------------------------------------------------
  py::enum_<RecoveryMode>(m, "RecoveryMode")
      .value("Normal", RecoveryMode::Normal)
      .value("Pending", RecoveryMode::Pending)
      .value("Active", RecoveryMode::Active);
  py::class_<NangilaHook>(m, "NangilaHook", py::dynamic_attr())  // instances carry their device state (gpu_methods.py)
      .def(py::init([](const py::bytes& mask_bytes, py::object config) {
             auto v = from_bytes(mask_bytes);
             TopologyMask mk = TopologyMask::from_bytes(v.data(), v.size());
             NangilaConfig cfg = config.is_none() ? NangilaConfig{} : config.cast<NangilaConfig>();
             return NangilaHook(cfg, std::move(mk));
           }),
           py::arg("mask_bytes"), py::arg("config") = py::none())
      .def_static("from_mask_file", [](const std::string& path, py::object config) {
        return NangilaHook::from_mask_file(path, config.is_none() ? NangilaConfig{} : config.cast<NangilaConfig>());
      }, py::arg("path"), py::arg("config") = py::none())
      .def_static("all_drivers", [](size_t n, py::object config) {
        return NangilaHook::all_drivers(n, config.is_none() ? NangilaConfig{} : config.cast<NangilaConfig>());
      }, py::arg("num_layers"), py::arg("config") = py::none())
      // the array's own shape travels in the packet (matrix-shaped gradients matter to PowerSGD)
      .def("compress", [](NangilaHook& h, LayerId id, const farray& g) { return to_bytes(h.on_send(id, to_tensor(g))); })
      .def("decompress", [](NangilaHook& h, LayerId id, const py::bytes& b) {
        auto v = from_bytes(b);
        return to_array(h.on_receive(id, v.data(), v.size()).data);
      })
      .def("decompress_gathered", [](NangilaHook& h, LayerId id, const py::bytes& b) {
        auto v = from_bytes(b);
        return to_array(h.on_receive_gathered(id, v.data(), v.size()).data);
      })
      .def("update", [](NangilaHook& h, LayerId id, const farray& g) { h.on_complete(id, to_tensor_flat(g)); })
      .def("step", &NangilaHook::step)
      .def("is_compression_enabled", &NangilaHook::is_compression_enabled)
      .def("current_step", &NangilaHook::current_step)
      .def("get_stats", [](const NangilaHook& h) {
        CompressionStats s = h.get_stats();
        py::dict d;
        d["step"] = s.step;
        d["compression_enabled"] = s.compression_enabled;
        d["num_drivers"] = s.num_drivers;
        d["num_passengers"] = s.num_passengers;
        d["mask_compression_ratio"] = s.mask_compression_ratio;
        d["quantizer_gamma"] = s.quantizer_gamma;
        return d;
      })
      .def("predictor_hash", &NangilaHook::predictor_hash)
      .def("should_verify_hash", &NangilaHook::should_verify_hash)
      .def("verify_hash", &NangilaHook::verify_hash)
      .def("set_hash_verify_interval", &NangilaHook::set_hash_verify_interval)
      .def("hash_verify_interval", &NangilaHook::hash_verify_interval)
      .def("get_layer_telemetry", [](const NangilaHook& h, LayerId id) -> py::object {
        const LayerTelemetry* t = h.get_layer_telemetry(id);
        if (!t) return py::none();
        return telemetry_dict(*t);
      })
      .def("get_summary_telemetry", [](const NangilaHook& h) {
        SummaryTelemetry s = h.get_summary_telemetry();
        py::dict d;
        d["total_original_bytes"] = s.total_original_bytes;
        d["total_compressed_bytes"] = s.total_compressed_bytes;
        d["overall_compression_ratio"] = s.overall_compression_ratio;
        d["total_compressions"] = s.total_compressions;
        d["total_passenger_skips"] = s.total_passenger_skips;
        d["avg_prediction_error"] = s.avg_prediction_error;
        d["num_layers_tracked"] = s.num_layers_tracked;
        return d;
      })
      .def("record_external", [](NangilaHook& h, LayerId id, size_t orig, size_t comp, float err) {
        h.state().record_external(id, orig, comp, err);
      })
      .def("set_partial_retransmit", &NangilaHook::set_partial_retransmit)
      .def("set_gpu_mode", &NangilaHook::set_gpu_mode)
      .def("gpu_mode", &NangilaHook::gpu_mode)
      .def("trigger_recovery", &NangilaHook::trigger_recovery)
      .def("recovery_mode", &NangilaHook::recovery_mode)
      .def("crc_failure_count", &NangilaHook::crc_failure_count)
      .def("enable_safe_mode", &NangilaHook::enable_safe_mode, py::arg("config") = SafeModeConfig{})
      .def("report_validation_loss", &NangilaHook::report_validation_loss)
      .def("is_paused", &NangilaHook::is_paused)
      .def("config", [](const NangilaHook& h) { return h.config(); })
      .def("momentum", &NangilaHook::momentum)
      .def("gamma", &NangilaHook::gamma)
      .def("mask_bytes", [](const NangilaHook& h) { return to_bytes(h.state().mask().to_bytes()); })
      .def("promote_to_driver", [](NangilaHook& h, LayerId id) { h.state().mask_mut().promote_to_driver(id); })
      .def("save_checkpoint", &NangilaHook::save_checkpoint)
      .def("load_checkpoint", &NangilaHook::load_checkpoint)
      .def("make_checkpoint", &NangilaHook::make_checkpoint)
      .def("restore_checkpoint", &NangilaHook::restore_checkpoint);

  m.def("max_compressed_size", [](size_t count) { return 16 + 12 + 4 * count + 32; });
}
