// Checkpoint file "NZCHK001" with integrity hash, and the bounded gradient-history ring used for
// rewind / recovery.
//
// Parity: nangila-core/src/checkpoint.rs:13 (magic), :36-50 (fields), :57-90 (hash = SipHash-1-3
// over step(u64), then per ascending layer id: id(u32), every i32 of prev, every i32 of current;
// verify_integrity), :93-261 (file layout), :266-333 (history ring, depth 10).
// File layout, little-endian:
//   "NZCHK001", u32 version, u64 step, u64 state_hash, f32 quantizer_gamma, u64 predictor_step,
//   f32 momentum, u32 num_layers, num_layers x { u32 layer_id, opt_buf prev, opt_buf current },
//   u64 warmup_steps, u64 shadow_run_steps
//   opt_buf = u8 present; if 1: u32 len, i32 q8_23[len]
// version 2 appends, after the trailer above, an extension the reference format has no room for:
//   u32 num_sections, sections x { u32 name_len, bytes name, u32 layer_id, u64 len, f32 data[len] }
// (error-feedback, DGC and PowerSGD memories). Version-1 readers stop before it.
#pragma once
#include <cstdio>
#include <cstring>
#include <deque>
#include <fstream>
#include <map>
#include <string>

#include "config.hpp"
#include "packet.hpp"
#include "predictor.hpp"
#include "siphash.hpp"

namespace nangila {

struct PredictorSnapshot {
  std::map<LayerId, LayerHistorySnapshot> histories;
  size_t current_step = 0;
  float momentum = 0.9f;
};

struct ExtraSection {
  std::string name;
  LayerId layer_id = 0;
  std::vector<float> data;
};

struct NangilaCheckpoint {
  static constexpr uint32_t VERSION = 1;
  static constexpr uint32_t VERSION_EXT = 2;

  uint32_t version = VERSION;
  uint64_t step = 0;
  PredictorSnapshot predictor;
  float quantizer_gamma = 0.0f;
  uint64_t state_hash = 0;
  NangilaConfig config;
  std::vector<ExtraSection> extra;  // only written when version >= 2

  uint64_t compute_hash() const {
    SipHasher13 h;
    h.write_u64(step);
    for (auto& kv : predictor.histories) {
      h.write_u32(kv.first);
      if (kv.second.prev)
        for (int32_t v : *kv.second.prev) h.write_i32(v);
      if (kv.second.current)
        for (int32_t v : *kv.second.current) h.write_i32(v);
    }
    return h.finish();
  }
  bool verify_integrity() const { return compute_hash() == state_hash; }
  void seal() { state_hash = compute_hash(); }

  std::vector<uint8_t> to_bytes() const {
    std::vector<uint8_t> o;
    auto put = [&o](const void* p, size_t n) {
      const uint8_t* b = static_cast<const uint8_t*>(p);
      o.insert(o.end(), b, b + n);
    };
    auto u32 = [&](uint32_t v) { uint8_t b[4]; detail::put_le<uint32_t>(b, v); put(b, 4); };
    auto u64 = [&](uint64_t v) { uint8_t b[8]; detail::put_le<uint64_t>(b, v); put(b, 8); };
    auto f32 = [&](float f) { uint32_t u; std::memcpy(&u, &f, 4); u32(u); };
    auto opt = [&](const std::optional<std::vector<int32_t>>& b) {
      if (!b) { o.push_back(0); return; }
      o.push_back(1);
      u32(uint32_t(b->size()));
      for (int32_t v : *b) u32(uint32_t(v));
    };
    put("NZCHK001", 8);
    u32(version);
    u64(step);
    u64(state_hash);
    f32(quantizer_gamma);
    u64(uint64_t(predictor.current_step));
    f32(predictor.momentum);
    u32(uint32_t(predictor.histories.size()));
    for (auto& kv : predictor.histories) {
      u32(kv.first);
      opt(kv.second.prev);
      opt(kv.second.current);
    }
    u64(uint64_t(config.warmup_steps));
    u64(uint64_t(config.shadow_run_steps));
    if (version >= VERSION_EXT) {
      u32(uint32_t(extra.size()));
      for (auto& s : extra) {
        u32(uint32_t(s.name.size()));
        put(s.name.data(), s.name.size());
        u32(s.layer_id);
        u64(uint64_t(s.data.size()));
        put(s.data.data(), s.data.size() * 4);
      }
    }
    return o;
  }
  static NangilaCheckpoint from_bytes(const uint8_t* p, size_t len) {
    size_t off = 0;
    auto need = [&](size_t n) {
      if (off + n > len) throw NangilaError::io("failed to fill whole buffer (checkpoint truncated)");
    };
    auto u32 = [&]() { need(4); uint32_t v = detail::get_le<uint32_t>(p + off); off += 4; return v; };
    auto u64 = [&]() { need(8); uint64_t v = detail::get_le<uint64_t>(p + off); off += 8; return v; };
    auto f32 = [&]() { uint32_t u = u32(); float f; std::memcpy(&f, &u, 4); return f; };
    auto opt = [&]() -> std::optional<std::vector<int32_t>> {
      need(1);
      if (p[off++] == 0) return std::nullopt;
      uint32_t n = u32();
      need(size_t(n) * 4);
      std::vector<int32_t> v(n);
      for (uint32_t i = 0; i < n; ++i) v[i] = int32_t(u32());
      return v;
    };
    need(8);
    if (std::memcmp(p, "NZCHK001", 8) != 0) throw NangilaError::invalid_format("Invalid checkpoint magic");
    off = 8;
    NangilaCheckpoint c;
    c.version = u32();
    c.step = u64();
    c.state_hash = u64();
    c.quantizer_gamma = f32();
    c.predictor.current_step = size_t(u64());
    c.predictor.momentum = f32();
    uint32_t n = u32();
    for (uint32_t i = 0; i < n; ++i) {
      LayerId id = u32();
      LayerHistorySnapshot s;
      s.prev = opt();
      s.current = opt();
      c.predictor.histories[id] = std::move(s);
    }
    c.config.warmup_steps = size_t(u64());
    c.config.shadow_run_steps = size_t(u64());
    if (c.version >= VERSION_EXT && off < len) {
      uint32_t ns = u32();
      for (uint32_t i = 0; i < ns; ++i) {
        ExtraSection s;
        uint32_t nl = u32();
        need(nl);
        s.name.assign(reinterpret_cast<const char*>(p + off), nl);
        off += nl;
        s.layer_id = u32();
        uint64_t dl = u64();
        need(size_t(dl) * 4);
        s.data.resize(size_t(dl));
        if (dl) std::memcpy(s.data.data(), p + off, size_t(dl) * 4);
        off += size_t(dl) * 4;
        c.extra.push_back(std::move(s));
      }
    }
    return c;
  }
  void save(const std::string& path) const {
    std::vector<uint8_t> b = to_bytes();
    std::ofstream f(path, std::ios::binary | std::ios::trunc);
    if (!f) throw NangilaError::io("cannot create " + path);
    f.write(reinterpret_cast<const char*>(b.data()), std::streamsize(b.size()));
    if (!f) throw NangilaError::io("short write to " + path);
  }
  static NangilaCheckpoint load(const std::string& path) {
    std::ifstream f(path, std::ios::binary);
    if (!f) throw NangilaError::io("cannot open " + path);
    std::vector<uint8_t> b((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
    return from_bytes(b.data(), b.size());
  }
};

// Last `max_depth` gradients per layer, newest last.
class GradientHistory {
 public:
  explicit GradientHistory(size_t max_depth = 10) : max_depth_(max_depth) {}
  void push(LayerId id, FixedPointBuffer g) {
    auto& q = buf_[id];
    if (q.size() >= max_depth_) q.pop_front();
    q.push_back(std::move(g));
  }
  // steps_ago = 0 is the most recent entry.
  const FixedPointBuffer* get(LayerId id, size_t steps_ago) const {
    auto it = buf_.find(id);
    if (it == buf_.end() || steps_ago >= it->second.size()) return nullptr;
    return &it->second[it->second.size() - 1 - steps_ago];
  }
  // Drop the newest `steps` entries; returns the entry that is newest afterwards (if any).
  std::optional<FixedPointBuffer> rewind(LayerId id, size_t steps) {
    auto it = buf_.find(id);
    if (it == buf_.end()) return std::nullopt;
    for (size_t i = 0, n = std::min(steps, it->second.size()); i < n; ++i) it->second.pop_back();
    if (it->second.empty()) return std::nullopt;
    return it->second.back();
  }
  void clear_layer(LayerId id) { buf_.erase(id); }
  void clear() { buf_.clear(); }
  size_t depth(LayerId id) const {
    auto it = buf_.find(id);
    return it == buf_.end() ? 0 : it->second.size();
  }

 private:
  std::map<LayerId, std::deque<FixedPointBuffer>> buf_;
  size_t max_depth_;
};

}  // namespace nangila
