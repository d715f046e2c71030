// NangilaState: owns the configuration, the topology mask, the selected compressor, the passenger
// reconstructor, the step counter / warm-up gate, Safe Mode and per-layer telemetry.
//
// Parity: nangila-core/src/state.rs:22-80 (LayerTelemetry with EMA 0.1), :118-146 (compressor
// chosen by compressor_type), :156-195 (compress: passthrough while disabled with a shadow
// predictor update once step >= warmup_steps; passengers send nothing; drivers compress),
// :201-330 (decompress / partial / all), :340-364 (update_state, step: enable at
// warmup + shadow_run, clear passenger cache), :399-461 (stats, telemetry), :466-523 (Safe Mode).
// Unlike the reference (state.rs:184 forces every payload through the INT4 struct), the Driver
// result carries the compressor's own payload bytes, so DGC and PowerSGD work through this path,
// and prediction error / gamma are real numbers instead of constants.
#pragma once
#include <limits>
#include <map>
#include <memory>
#include <optional>

#include "compressor.hpp"
#include "mask.hpp"
#include "reconstructor.hpp"
#include "safe_mode.hpp"

namespace nangila {

struct LayerTelemetry {
  uint64_t total_original_bytes = 0, total_compressed_bytes = 0, compression_count = 0;
  float avg_compression_ratio = 0.0f;
  float min_compression_ratio = std::numeric_limits<float>::max();
  float max_compression_ratio = 0.0f;
  float avg_prediction_error = 0.0f;
  uint64_t passenger_skip_count = 0;

  void record_compression(size_t original, size_t compressed, float pred_error) {
    total_original_bytes += original;
    total_compressed_bytes += compressed;
    ++compression_count;
    float ratio = float(original) / float(std::max<size_t>(compressed, 1));
    min_compression_ratio = std::min(min_compression_ratio, ratio);
    max_compression_ratio = std::max(max_compression_ratio, ratio);
    const float a = 0.1f;
    avg_compression_ratio = a * ratio + (1.0f - a) * avg_compression_ratio;
    avg_prediction_error = a * pred_error + (1.0f - a) * avg_prediction_error;
  }
};

struct SummaryTelemetry {
  uint64_t total_original_bytes = 0, total_compressed_bytes = 0;
  float overall_compression_ratio = 1.0f;
  uint64_t total_compressions = 0, total_passenger_skips = 0;
  float avg_prediction_error = 0.0f;
  size_t num_layers_tracked = 0;
};

struct CompressionStats {
  size_t step;
  bool compression_enabled;
  size_t num_drivers, num_passengers;
  float mask_compression_ratio;
  float quantizer_gamma;
};

struct CompressionResult {
  enum Kind { Driver, Passenger, Passthrough } kind = Passthrough;
  std::vector<uint8_t> payload;  // Driver: compressor payload
  uint8_t flags = 0;             // Driver: extra header flags chosen by the compressor
  Tensor tensor;                 // Passthrough: the gradient itself
};

class NangilaState {
 public:
  NangilaState(NangilaConfig cfg, TopologyMask mask)
      : config(cfg), mask_(std::move(mask)), compressor_(make_compressor(cfg)) {}

  CompressionResult compress(LayerId id, const Tensor& g) {
    CompressionResult r;
    if (!is_compression_enabled()) {
      if (step_ >= config.warmup_steps) compressor_->update(id, g);  // shadow run
      r.kind = CompressionResult::Passthrough;
      r.tensor = g;
      return r;
    }
    const LayerRole& role = mask_.get_role(id);
    if (role.is_passenger()) {
      ++telemetry_[id].passenger_skip_count;
      r.kind = CompressionResult::Passenger;
      return r;
    }
    Packet p = compressor_->compress(g, id);
    telemetry_[id].record_compression(g.numel() * 4, p.payload.size(), compressor_->last_prediction_error());
    r.kind = CompressionResult::Driver;
    r.flags = uint8_t(p.header.flags & ~flags::DRIVER);
    r.payload = std::move(p.payload);
    return r;
  }
  Tensor decompress(LayerId id, const std::vector<uint8_t>& payload, uint8_t header_flags = flags::DRIVER) {
    const LayerRole& role = mask_.get_role(id);
    if (role.is_driver()) {
      PacketHeader hd = PacketHeader::new_driver(uint32_t(step_), id);
      hd.flags = uint8_t(header_flags | flags::DRIVER);
      Packet p(hd, payload);
      Tensor g = compressor_->decompress(p, id);
      reconstructor_.cache_driver_gradient(id, g);
      return g;
    }
    return reconstructor_.synthesize_passenger(id, mask_);
  }
  Tensor decompress_partial(LayerId id, const std::vector<uint8_t>& payload, size_t start, size_t end,
                            uint8_t header_flags = flags::DRIVER) {
    const LayerRole& role = mask_.get_role(id);
    if (role.is_driver()) {
      PacketHeader hd = PacketHeader::new_driver(uint32_t(step_), id);
      hd.flags = uint8_t(header_flags | flags::DRIVER);
      Packet p(hd, payload);
      if (auto* pr = dynamic_cast<PredictionResidualCompressor*>(compressor_.get()))
        return pr->decompress_partial(p, id, start, end);
      Tensor full = compressor_->decompress(p, id);
      start = std::min(start, full.numel());
      end = std::min(end, full.numel());
      std::vector<float> d(full.data.begin() + start, full.data.begin() + std::max(start, end));
      size_t n = d.size();
      return Tensor(std::move(d), {n});
    }
    return reconstructor_.synthesize_passenger_partial(id, mask_, start, end);
  }
  std::map<LayerId, Tensor> decompress_all(const std::map<LayerId, std::vector<uint8_t>>& drivers) {
    std::map<LayerId, Tensor> out;
    for (auto& kv : drivers) out[kv.first] = decompress(kv.first, kv.second);
    for (auto& p : mask_.passengers()) out[p.id] = reconstructor_.synthesize_passenger(p.id, mask_);
    return out;
  }
  void update_state(LayerId id, const Tensor& g) { compressor_->update(id, g); }
  void step() {
    ++step_;
    compressor_->step();
    if (step_ >= config.warmup_steps + config.shadow_run_steps) compression_enabled_ = true;
    reconstructor_.clear_cache();
  }
  bool is_compression_enabled() const { return compression_enabled_ && !paused_; }
  size_t current_step() const { return step_; }
  const TopologyMask& mask() const { return mask_; }
  TopologyMask& mask_mut() { return mask_; }
  uint64_t predictor_hash() const { return compressor_->state_hash(); }
  void force_sync_layer(LayerId id, const Tensor& g) { compressor_->force_sync_layer(id, g); }
  Compressor& compressor() { return *compressor_; }

  CompressionStats stats() const {
    return {step_, is_compression_enabled(), mask_.num_drivers(), mask_.num_passengers(),
            mask_.compression_ratio(), compressor_->quantizer_gamma()};
  }
  const LayerTelemetry* layer_telemetry(LayerId id) const {
    auto it = telemetry_.find(id);
    return it == telemetry_.end() ? nullptr : &it->second;
  }
  const std::map<LayerId, LayerTelemetry>& all_layer_telemetry() const { return telemetry_; }
  SummaryTelemetry summary_telemetry() const {
    SummaryTelemetry s;
    float err = 0;
    size_t n = 0;
    for (auto& kv : telemetry_) {
      s.total_original_bytes += kv.second.total_original_bytes;
      s.total_compressed_bytes += kv.second.total_compressed_bytes;
      s.total_compressions += kv.second.compression_count;
      s.total_passenger_skips += kv.second.passenger_skip_count;
      if (kv.second.compression_count > 0) {
        err += kv.second.avg_prediction_error;
        ++n;
      }
    }
    if (s.total_compressed_bytes > 0)
      s.overall_compression_ratio = float(s.total_original_bytes) / float(s.total_compressed_bytes);
    s.avg_prediction_error = n ? err / float(n) : 0.0f;
    s.num_layers_tracked = telemetry_.size();
    return s;
  }
  // Telemetry fed by a device path that did the compression itself.
  void record_external(LayerId id, size_t original, size_t compressed, float pred_error) {
    telemetry_[id].record_compression(original, compressed, pred_error);
  }

  void enable_safe_mode(SafeModeConfig c) { safe_mode_ = SafeMode(c); }
  SafeModeAction report_validation_loss(float loss) {
    if (!safe_mode_) return SafeModeAction::NoCheck;
    if (!safe_mode_->should_check(step_)) return SafeModeAction::NoCheck;
    SafeModeAction a = safe_mode_->check(step_, loss);
    if (a == SafeModeAction::TriggerFallback) paused_ = true;
    if (a == SafeModeAction::RecoveryComplete) paused_ = false;
    return a;
  }
  bool is_paused() const { return paused_; }
  std::optional<SafeModeStats> safe_mode_stats() const {
    if (!safe_mode_) return std::nullopt;
    return safe_mode_->stats();
  }
  bool has_safe_mode() const { return safe_mode_.has_value(); }
  void set_step(size_t s) {
    step_ = s;
    compression_enabled_ = step_ >= config.warmup_steps + config.shadow_run_steps;
  }

  NangilaConfig config;

 private:
  TopologyMask mask_;
  std::unique_ptr<Compressor> compressor_;
  Reconstructor reconstructor_;
  size_t step_ = 0;
  bool compression_enabled_ = false;
  std::optional<SafeMode> safe_mode_;
  bool paused_ = false;
  std::map<LayerId, LayerTelemetry> telemetry_;
};

}  // namespace nangila
