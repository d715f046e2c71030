// Run-time configuration of the compression engine, its presets and validation.
//
// Parity: nangila-core/src/config.rs:30-38 (CompressorType), :41-99 (fields and defaults),
// :101-187 (validated constructor, conservative/aggressive presets, validate()).
// nangila-cuda/src/bindings.rs:61-77 (SyncMode).
#pragma once
#include <cstdint>
#include <string>

#include "types.hpp"

namespace nangila {

enum class CompressorType : int32_t { PredictionResidual = 0, DGC = 1, PowerSGD = 2 };

// When the device status word / stream is checked after a fused kernel was queued.
enum class SyncMode : int32_t { Async = 0, Always = 1, Periodic = 2 };

inline bool sync_mode_from_i32(int32_t v, SyncMode* out) {
  if (v < 0 || v > 2) return false;
  *out = static_cast<SyncMode>(v);
  return true;
}
inline const char* sync_mode_name(SyncMode m) {
  switch (m) {
    case SyncMode::Async: return "SyncMode.ASYNC";
    case SyncMode::Always: return "SyncMode.ALWAYS";
    default: return "SyncMode.PERIODIC";
  }
}

struct NangilaConfig {
  float momentum = 0.9f;
  float sculptor_threshold = 0.95f;
  size_t warmup_steps = 1000;
  size_t shadow_run_steps = 100;
  uint8_t quantize_bits = 4;
  bool dynamic_gamma = true;
  size_t monitor_interval = 1000;
  float monitor_sample_fraction = 0.10f;
  float promotion_threshold = 0.15f;
  CompressorType compressor_type = CompressorType::PredictionResidual;
  float dgc_sparsity = 0.999f;
  size_t power_sgd_rank = 1;

  // Throws NangilaError(Config) with a message naming the offending field.
  void validate() const {
    auto bad = [](const std::string& m) { throw NangilaError(ErrorKind::Config, m); };
    if (!(momentum >= 0.0f && momentum <= 1.0f))
      bad("Invalid momentum " + std::to_string(momentum) + ": must be in [0, 1]");
    if (!(sculptor_threshold >= 0.0f && sculptor_threshold <= 1.0f))
      bad("Invalid threshold " + std::to_string(sculptor_threshold) + ": must be in [0, 1]");
    if (quantize_bits < 1 || quantize_bits > 8)
      bad("Invalid quantize_bits " + std::to_string(int(quantize_bits)) + ": must be in [1, 8]");
    if (!(monitor_sample_fraction >= 0.0f && monitor_sample_fraction <= 1.0f))
      bad("Invalid monitor_sample_fraction " + std::to_string(monitor_sample_fraction));
    if (!(promotion_threshold > 0.0f))
      bad("Invalid promotion_threshold " + std::to_string(promotion_threshold));
    if (!(dgc_sparsity >= 0.0f && dgc_sparsity <= 1.0f))
      bad("Invalid dgc_sparsity " + std::to_string(dgc_sparsity) + ": must be in [0, 1]");
    if (power_sgd_rank == 0) bad("Invalid power_sgd_rank 0: must be >= 1");
  }

  static NangilaConfig make(float momentum, float threshold, size_t warmup, size_t shadow,
                            uint8_t bits) {
    NangilaConfig c;
    c.momentum = momentum;
    c.sculptor_threshold = threshold;
    c.warmup_steps = warmup;
    c.shadow_run_steps = shadow;
    c.quantize_bits = bits;
    c.validate();
    return c;
  }
  static NangilaConfig conservative() {
    NangilaConfig c;
    c.sculptor_threshold = 0.97f;
    c.monitor_interval = 500;
    c.dgc_sparsity = 0.99f;
    c.power_sgd_rank = 2;
    return c;
  }
  static NangilaConfig aggressive() {
    NangilaConfig c;
    c.sculptor_threshold = 0.90f;
    c.monitor_interval = 1000;
    c.dgc_sparsity = 0.999f;
    c.power_sgd_rank = 1;
    return c;
  }
};

}  // namespace nangila
