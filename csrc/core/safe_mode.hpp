// Safe Mode: watches reported validation losses with a fast and a slow exponential average and
// switches compression off when the fast one runs away from the slow one.
//
// Parity: nangila-core/src/safe_mode.rs:8-67 (config + conservative/relaxed presets), :70-95
// (actions and states), :126-349 (state machine: Active -> Fallback after N consecutive
// divergent checks; Fallback -> Recovering once stable; Recovering -> Active after the cool-down;
// Canary handled but only entered explicitly).
#pragma once
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <optional>

namespace nangila {

struct SafeModeConfig {
  size_t check_interval = 100;
  float divergence_threshold = 0.005f;
  uint32_t max_consecutive_failures = 3;
  size_t recovery_cooldown = 500;
  float canary_fraction = 0.1f;
  size_t canary_steps = 100;
  uint32_t canary_max_failures = 2;

  static SafeModeConfig conservative() { return {50, 0.003f, 2, 1000, 0.05f, 200, 1}; }
  static SafeModeConfig relaxed() { return {200, 0.01f, 5, 200, 0.2f, 50, 3}; }
};

enum class SafeModeAction : int { Continue = 0, TriggerFallback = 1, RecoveryComplete = 2, NoCheck = 3, CanaryTest = 4 };
enum class SafeModeState : int { Active = 0, Fallback = 1, Recovering = 2, Canary = 3 };

struct SafeModeStats {
  SafeModeState state;
  std::optional<float> baseline_loss, last_loss, ema_loss_short, ema_loss_long;
  uint32_t failure_count;
  size_t cooldown_remaining;
  uint32_t total_fallbacks;
};

class SafeMode {
 public:
  explicit SafeMode(SafeModeConfig c = {}) : cfg_(c) {}

  bool should_check(size_t step) const { return step > 0 && cfg_.check_interval > 0 && step % cfg_.check_interval == 0; }

  SafeModeAction check(size_t step, float loss) {
    ema_short_ = ema_short_ ? kAlphaShort * loss + (1.0f - kAlphaShort) * *ema_short_ : loss;
    ema_long_ = ema_long_ ? kAlphaLong * loss + (1.0f - kAlphaLong) * *ema_long_ : loss;
    last_loss_ = loss;
    last_check_step_ = step;
    switch (state_) {
      case SafeModeState::Active: return check_active(loss);
      case SafeModeState::Fallback: return check_fallback(loss);
      case SafeModeState::Recovering: return check_recovering();
      default: return check_canary(loss);
    }
  }
  bool should_compress() const { return state_ == SafeModeState::Active; }
  SafeModeState state() const { return state_; }
  SafeModeStats stats() const {
    return {state_, baseline_, last_loss_, ema_short_, ema_long_, failures_, cooldown_, total_fallbacks_};
  }
  void force_fallback() { trigger_fallback(); }
  // Start a canary period: compression on for a fraction of layers while being watched.
  void enter_canary() {
    state_ = SafeModeState::Canary;
    failures_ = 0;
    cooldown_ = cfg_.canary_steps;
  }
  void reset() {
    state_ = SafeModeState::Active;
    failures_ = 0;
    cooldown_ = 0;
  }
  const SafeModeConfig& config() const { return cfg_; }

 private:
  static constexpr float kAlphaShort = 0.3f, kAlphaLong = 0.05f;

  float delta(float loss) const {
    float l = ema_long_.value_or(loss), s = ema_short_.value_or(loss);
    return (s - l) / std::max(std::fabs(l), 1e-6f);
  }
  SafeModeAction check_active(float loss) {
    if (!baseline_) {
      if (ema_long_) baseline_ = *ema_long_;
      return SafeModeAction::Continue;
    }
    if (delta(loss) > cfg_.divergence_threshold) {
      if (++failures_ >= cfg_.max_consecutive_failures) {
        trigger_fallback();
        return SafeModeAction::TriggerFallback;
      }
    } else {
      failures_ = 0;
      if (ema_long_ && *ema_long_ < *baseline_) baseline_ = *ema_long_;
    }
    return SafeModeAction::Continue;
  }
  SafeModeAction check_fallback(float loss) {
    if (delta(loss) <= cfg_.divergence_threshold) {
      failures_ = 0;
      state_ = SafeModeState::Recovering;
      cooldown_ = cfg_.recovery_cooldown;
    }
    return SafeModeAction::Continue;
  }
  SafeModeAction check_recovering() {
    cooldown_ = cooldown_ > cfg_.check_interval ? cooldown_ - cfg_.check_interval : 0;
    if (cooldown_ == 0) {
      state_ = SafeModeState::Active;
      return SafeModeAction::RecoveryComplete;
    }
    return SafeModeAction::Continue;
  }
  SafeModeAction check_canary(float loss) {
    if (delta(loss) > cfg_.divergence_threshold) {
      if (++failures_ >= cfg_.canary_max_failures) {
        state_ = SafeModeState::Fallback;
        failures_ = 0;
        return SafeModeAction::TriggerFallback;
      }
    } else {
      failures_ = 0;
      cooldown_ = cooldown_ > cfg_.check_interval ? cooldown_ - cfg_.check_interval : 0;
      if (cooldown_ == 0) {
        state_ = SafeModeState::Active;
        return SafeModeAction::RecoveryComplete;
      }
    }
    return SafeModeAction::CanaryTest;
  }
  void trigger_fallback() {
    state_ = SafeModeState::Fallback;
    failures_ = 0;
    ++total_fallbacks_;
  }

  SafeModeConfig cfg_;
  SafeModeState state_ = SafeModeState::Active;
  std::optional<float> baseline_, last_loss_, ema_short_, ema_long_;
  uint32_t failures_ = 0;
  size_t cooldown_ = 0;
  size_t last_check_step_ = 0;
  uint32_t total_fallbacks_ = 0;
};

}  // namespace nangila
