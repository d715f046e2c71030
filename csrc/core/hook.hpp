// NangilaHook: the packet-level state machine around NangilaState. on_send turns a gradient into
// packet bytes, on_receive / on_receive_gathered validate a packet and reconstruct the gradient,
// on_complete feeds the averaged gradient back, step() advances. It also owns desync recovery
// (CRC failure counting, FORCE_SYNC, cached-packet reuse, history fallback), periodic predictor
// hash verification, Safe Mode pass-through and checkpoint export / import.
//
// Parity: nangila-hook/src/hook.rs:27-35 (RecoveryMode), :42-147 (construction, gpu mode, mask
// file, all_drivers), :152-185 (on_send), :190-266 (on_receive: parse, header, CRC with threshold
// 3, cached-packet recovery, stale-step check, FORCE_SYNC), :274-298 (gathered variant without
// step bookkeeping), :301-319 (on_complete, step), :352-396 (hash verification every 100 steps;
// a mismatch marks up to 10 driver layers for recovery), :399-439, :559-794 (packet builders and
// payload formats). The reference has no checkpoint wiring; save/load here write the NZCHK001
// format of checkpoint.hpp from the live predictor.
#pragma once
#include <fstream>
#include <map>

#include "checkpoint.hpp"
#include "state.hpp"

namespace nangila {

enum class RecoveryMode : int { Normal = 0, Pending = 1, Active = 2 };

class NangilaHook {
 public:
  NangilaHook(NangilaConfig cfg, TopologyMask mask) : state_(cfg, std::move(mask)) {}
  static NangilaHook from_mask_file(const std::string& path, NangilaConfig cfg = {}) {
    std::ifstream f(path, std::ios::binary);
    if (!f) throw NangilaError::io("cannot open " + path);
    std::vector<uint8_t> b((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
    return NangilaHook(cfg, TopologyMask::from_bytes(b.data(), b.size()));
  }
  static NangilaHook all_drivers(size_t n, NangilaConfig cfg = {}) {
    return NangilaHook(cfg, TopologyMask::all_drivers(n));
  }

  void set_partial_retransmit(bool on) {
    partial_retransmit_ = on;
    if (!on) packet_cache_.clear();
  }
  void set_gpu_mode(bool on) {
    gpu_mode_ = on;
    if (on) history_.clear();
  }
  bool gpu_mode() const { return gpu_mode_; }

  std::vector<uint8_t> on_send(LayerId id, const Tensor& g) {
    auto rm = recovery_.find(id);
    if (rm != recovery_.end() && rm->second == RecoveryMode::Pending) {
      rm->second = RecoveryMode::Active;
      return make_packet(PacketHeader::new_force_sync(uint32_t(step_counter_), id), wire::serialize_tensor(g));
    }
    if (!gpu_mode_) history_.push(id, FixedPointBuffer::from_f32(g.data));
    try {
      CompressionResult r = state_.compress(id, g);
      switch (r.kind) {
        case CompressionResult::Driver: {
          PacketHeader h = PacketHeader::new_driver(uint32_t(step_counter_), id);
          h.flags |= r.flags;
          return make_packet(h, std::move(r.payload));
        }
        case CompressionResult::Passenger:
          return make_packet(PacketHeader::new_passenger(uint32_t(step_counter_), id), {});
        default:
          return passthrough_packet(id, r.tensor);
      }
    } catch (const NangilaError&) {
      return passthrough_packet(id, g);
    }
  }

  Tensor on_receive(LayerId id, const uint8_t* data, size_t len) {
    auto pk = Packet::from_bytes(data, len);
    if (!pk) return Tensor::zeros({1});
    if (!pk->header.is_valid()) {
      trigger_recovery(id);
      return Tensor::zeros({1});
    }
    if (!pk->verify()) {
      uint32_t n = ++crc_failures_[id];
      if (partial_retransmit_ && packet_cache_.count(id)) {
        if (auto t = try_partial_recovery(id, *pk)) {
          crc_failures_[id] = 0;
          return *t;
        }
      }
      if (n >= crc_failure_threshold_) trigger_recovery(id);
      return recover_from_history(id);
    }
    crc_failures_[id] = 0;
    if (partial_retransmit_ && !pk->header.is_partial_retransmit()) packet_cache_[id].assign(data, data + len);
    uint64_t expected = expected_peer_step_.count(id) ? expected_peer_step_[id] : 0;
    if (uint64_t(pk->header.step) < expected) return recover_from_history(id);
    expected_peer_step_[id] = uint64_t(pk->header.step) + 1;
    if (pk->header.is_force_sync()) return handle_force_sync(id, *pk);
    return decode_payload(id, *pk);
  }
  // One packet per rank arrives for the same step in an all-gather transport, so the monotonic
  // peer-step rule of on_receive does not apply here.
  Tensor on_receive_gathered(LayerId id, const uint8_t* data, size_t len) {
    auto pk = Packet::from_bytes(data, len);
    if (!pk || !pk->header.is_valid()) return Tensor::zeros({1});
    if (!pk->verify()) {
      ++crc_failures_[id];
      return recover_from_history(id);
    }
    if (pk->header.is_force_sync()) return handle_force_sync(id, *pk);
    return decode_payload(id, *pk);
  }
  void on_complete(LayerId id, const Tensor& g) {
    state_.update_state(id, g);
    auto rm = recovery_.find(id);
    if (rm != recovery_.end() && rm->second == RecoveryMode::Active) rm->second = RecoveryMode::Normal;
  }
  void step() {
    ++step_counter_;
    state_.step();
  }

  bool is_compression_enabled() const { return state_.is_compression_enabled(); }
  size_t current_step() const { return state_.current_step(); }
  CompressionStats get_stats() const { return state_.stats(); }
  const LayerTelemetry* get_layer_telemetry(LayerId id) const { return state_.layer_telemetry(id); }
  SummaryTelemetry get_summary_telemetry() const { return state_.summary_telemetry(); }
  uint64_t predictor_hash() const { return state_.predictor_hash(); }
  bool should_verify_hash() const {
    return hash_verify_interval_ > 0 && step_counter_ > 0 && step_counter_ % hash_verify_interval_ == 0;
  }
  bool verify_hash(uint64_t peer) {
    uint64_t local = predictor_hash();
    if (local == peer) {
      last_verified_hash_ = local;
      return true;
    }
    std::vector<LayerId> d = state_.mask().drivers();
    for (size_t i = 0; i < d.size() && i < 10; ++i) trigger_recovery(d[i]);
    return false;
  }
  uint64_t hash_verify_interval() const { return hash_verify_interval_; }
  void set_hash_verify_interval(uint64_t n) { hash_verify_interval_ = n; }
  void enable_safe_mode(SafeModeConfig c) { state_.enable_safe_mode(c); }
  SafeModeAction report_validation_loss(float l) { return state_.report_validation_loss(l); }
  bool is_paused() const { return state_.is_paused(); }
  const NangilaConfig& config() const { return state_.config; }
  float momentum() const { return state_.config.momentum; }
  float gamma() const { return state_.stats().quantizer_gamma; }
  void trigger_recovery(LayerId id) {
    recovery_[id] = RecoveryMode::Pending;
    crc_failures_[id] = 0;
  }
  RecoveryMode recovery_mode(LayerId id) const {
    auto it = recovery_.find(id);
    return it == recovery_.end() ? RecoveryMode::Normal : it->second;
  }
  uint32_t crc_failure_count(LayerId id) const {
    auto it = crc_failures_.find(id);
    return it == crc_failures_.end() ? 0 : it->second;
  }
  NangilaState& state() { return state_; }
  const NangilaState& state() const { return state_; }
  uint64_t step_counter() const { return step_counter_; }

  // --- checkpoint ---------------------------------------------------------------------------
  NangilaCheckpoint make_checkpoint() {
    NangilaCheckpoint c;
    c.step = step_counter_;
    c.config = state_.config;
    c.quantizer_gamma = state_.stats().quantizer_gamma;
    c.predictor.momentum = state_.config.momentum;
    c.predictor.current_step = state_.current_step();
    Compressor* comp = &state_.compressor();
    if (auto* pr = dynamic_cast<PredictionResidualCompressor*>(comp)) {
      c.predictor.histories = pr->predictor().export_snapshots();
      for (auto& kv : pr->error_feedback()) c.extra.push_back({"predres.ef", kv.first, kv.second});
    } else if (auto* d = dynamic_cast<DGCCompressor*>(comp)) {
      for (auto& kv : d->residuals()) c.extra.push_back({"dgc.residual", kv.first, kv.second});
    } else if (auto* p = dynamic_cast<PowerSGDCompressor*>(comp)) {
      for (auto& kv : p->residuals()) c.extra.push_back({"powersgd.residual", kv.first, kv.second});
      for (auto& kv : p->q_memory()) c.extra.push_back({"powersgd.q", kv.first, kv.second.a});
    }
    c.version = c.extra.empty() ? NangilaCheckpoint::VERSION : NangilaCheckpoint::VERSION_EXT;
    c.seal();
    return c;
  }
  void restore_checkpoint(const NangilaCheckpoint& c) {
    if (!c.verify_integrity()) throw NangilaError::invalid_format("checkpoint state hash mismatch");
    step_counter_ = c.step;
    state_.set_step(c.predictor.current_step);
    Compressor* comp = &state_.compressor();
    if (auto* pr = dynamic_cast<PredictionResidualCompressor*>(comp)) {
      pr->predictor().restore_snapshots(c.predictor.histories);
      pr->predictor().set_step(c.predictor.current_step);
      pr->set_step(c.predictor.current_step);
      pr->quantizer().set_gamma(c.quantizer_gamma);
      pr->error_feedback().clear();
      for (auto& s : c.extra)
        if (s.name == "predres.ef") pr->error_feedback()[s.layer_id] = s.data;
    } else if (auto* d = dynamic_cast<DGCCompressor*>(comp)) {
      d->residuals().clear();
      for (auto& s : c.extra)
        if (s.name == "dgc.residual") d->residuals()[s.layer_id] = s.data;
    } else if (auto* p = dynamic_cast<PowerSGDCompressor*>(comp)) {
      p->residuals().clear();
      for (auto& s : c.extra)
        if (s.name == "powersgd.residual") p->residuals()[s.layer_id] = s.data;
      // Q memories are re-derived on first use when their shape is unknown here.
    }
  }
  void save_checkpoint(const std::string& path) { make_checkpoint().save(path); }
  void load_checkpoint(const std::string& path) { restore_checkpoint(NangilaCheckpoint::load(path)); }

 private:
  static std::vector<uint8_t> make_packet(PacketHeader h, std::vector<uint8_t> payload) {
    return Packet(h, std::move(payload)).to_bytes();
  }
  std::vector<uint8_t> passthrough_packet(LayerId id, const Tensor& t) {
    PacketHeader h = PacketHeader::new_driver(uint32_t(step_counter_), id);
    h.flags = 0;
    return make_packet(h, wire::serialize_tensor(t));
  }
  Tensor handle_force_sync(LayerId id, const Packet& p) {
    Tensor g = wire::deserialize_tensor(p.payload.data(), p.payload.size());
    state_.force_sync_layer(id, g);
    recovery_[id] = RecoveryMode::Normal;
    return g;
  }
  Tensor decode_payload(LayerId id, const Packet& p) {
    try {
      if (p.header.is_passenger()) return state_.decompress(id, {});
      if (!p.header.is_driver()) return wire::deserialize_tensor(p.payload.data(), p.payload.size());
      return state_.decompress(id, p.payload, p.header.flags);
    } catch (const NangilaError&) {
      return p.header.is_passenger() ? Tensor::zeros({1}) : recover_from_history(id);
    }
  }
  Tensor recover_from_history(LayerId id) const {
    if (const FixedPointBuffer* b = history_.get(id, 0)) {
      std::vector<float> d = b->to_f32();
      size_t n = d.size();
      return Tensor(std::move(d), {n});
    }
    return Tensor::zeros({1});
  }
  // A corrupted driver packet is replaced by the cached good packet of the same layer when that
  // one is at most one step old.
  std::optional<Tensor> try_partial_recovery(LayerId id, const Packet& bad) {
    auto& cached_bytes = packet_cache_[id];
    auto cached = Packet::from_bytes(cached_bytes.data(), cached_bytes.size());
    if (!cached) return std::nullopt;
    uint32_t diff = bad.header.step >= cached->header.step ? bad.header.step - cached->header.step : 0;
    if (diff > 1) return std::nullopt;
    try {
      if (cached->header.is_driver() && bad.header.is_driver())
        return state_.decompress(id, cached->payload, cached->header.flags);
      if (!cached->header.is_driver() && !cached->header.is_passenger())
        return wire::deserialize_tensor(cached->payload.data(), cached->payload.size());
    } catch (const NangilaError&) {
    }
    return std::nullopt;
  }

  NangilaState state_;
  uint64_t step_counter_ = 0;
  std::map<LayerId, uint64_t> expected_peer_step_;
  GradientHistory history_;
  std::map<LayerId, RecoveryMode> recovery_;
  uint32_t crc_failure_threshold_ = 3;
  std::map<LayerId, uint32_t> crc_failures_;
  bool gpu_mode_ = false;
  uint64_t hash_verify_interval_ = 100;
  uint64_t last_verified_hash_ = 0;
  std::map<LayerId, std::vector<uint8_t>> packet_cache_;
  bool partial_retransmit_ = true;
};

}  // namespace nangila
