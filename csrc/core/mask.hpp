// Topology mask: which layers are Drivers (transmitted) and which are Passengers (synthesised
// locally as alpha * driver + beta), plus the byte format produced by the Sculptor.
//
// Parity: nangila-core/src/mask.rs:12-37 (roles), :58-140 (add/get/counts/ratio), :144-188 (FSDP
// ordering, prefetch hints, dependency check), :191-202 (promote), :208-284 (validate, checked
// add), :287-342 (byte format). Byte format, little-endian:
//   u32 num_layers; per layer: u32 layer_id, u8 tag (0 Driver, 1 Passenger),
//   and for tag 1: u32 source_id, f32 alpha, f32 beta.
// Entries are accepted in any order and written sorted by layer id, so output is deterministic.
// An unknown tag is an InvalidFormat error (the reference aborts there).
#pragma once
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <map>
#include <set>
#include <utility>
#include <vector>

#include "packet.hpp"
#include "types.hpp"

namespace nangila {

struct LayerRole {
  bool passenger = false;
  LayerId source_id = 0;
  float alpha = 1.0f;
  float beta = 0.0f;
  bool is_driver() const { return !passenger; }
  bool is_passenger() const { return passenger; }
};

class TopologyMask {
 public:
  void add_driver(LayerId id) {
    erase_counts(id);
    layers_[id] = LayerRole{};
    ++num_drivers_;
  }
  void add_passenger(LayerId id, LayerId source, float alpha, float beta) {
    erase_counts(id);
    layers_[id] = LayerRole{true, source, alpha, beta};
    ++num_passengers_;
  }
  void add_passenger_checked(LayerId id, LayerId source, float alpha, float beta) {
    if (!is_driver(source)) {
      if (layers_.count(source))
        throw NangilaError::invalid_format("Cannot add passenger " + std::to_string(id) + ": source " +
                                           std::to_string(source) + " is not a driver");
      throw NangilaError::invalid_format("Cannot add passenger " + std::to_string(id) + ": source driver " +
                                         std::to_string(source) + " does not exist");
    }
    if (id == source)
      throw NangilaError::invalid_format("Passenger " + std::to_string(id) + " cannot reference itself");
    add_passenger(id, source, alpha, beta);
  }

  const LayerRole& get_role(LayerId id) const {
    auto it = layers_.find(id);
    if (it == layers_.end()) throw NangilaError::layer_not_found(id);
    return it->second;
  }
  bool contains(LayerId id) const { return layers_.count(id) != 0; }
  bool is_driver(LayerId id) const {
    auto it = layers_.find(id);
    return it != layers_.end() && it->second.is_driver();
  }
  bool is_passenger(LayerId id) const {
    auto it = layers_.find(id);
    return it != layers_.end() && it->second.is_passenger();
  }
  std::vector<LayerId> drivers() const {
    std::vector<LayerId> v;
    for (auto& kv : layers_)
      if (kv.second.is_driver()) v.push_back(kv.first);
    return v;
  }
  // (passenger id, source id, alpha)
  struct PassengerInfo { LayerId id, source; float alpha, beta; };
  std::vector<PassengerInfo> passengers() const {
    std::vector<PassengerInfo> v;
    for (auto& kv : layers_)
      if (kv.second.is_passenger())
        v.push_back({kv.first, kv.second.source_id, kv.second.alpha, kv.second.beta});
    return v;
  }
  size_t num_drivers() const { return num_drivers_; }
  size_t num_passengers() const { return num_passengers_; }
  size_t num_layers() const { return layers_.size(); }
  std::vector<LayerId> all_layer_ids() const {
    std::vector<LayerId> v;
    for (auto& kv : layers_) v.push_back(kv.first);
    return v;
  }
  float compression_ratio() const {
    if (layers_.empty()) return 1.0f;
    return float(layers_.size()) / float(std::max<size_t>(num_drivers_, 1));
  }

  // Drivers (sorted) first, then passengers (sorted): the order in which an FSDP shard consumer
  // must reconstruct layers so every passenger finds its driver.
  std::vector<LayerId> fsdp_ordered_layers() const {
    std::vector<LayerId> d = drivers();
    for (auto& p : passengers()) d.push_back(p.id);
    return d;
  }
  std::vector<std::pair<LayerId, uint32_t>> prefetch_hints() const {
    std::vector<std::pair<LayerId, uint32_t>> h;
    for (LayerId d : drivers()) h.emplace_back(d, 0u);
    for (auto& p : passengers()) h.emplace_back(p.id, 1u);
    return h;
  }
  bool dependencies_ready(LayerId id, const std::set<LayerId>& ready) const {
    auto it = layers_.find(id);
    if (it == layers_.end()) return false;
    if (it->second.is_driver()) return true;
    return ready.count(it->second.source_id) != 0;
  }
  void promote_to_driver(LayerId id) {
    auto it = layers_.find(id);
    if (it == layers_.end()) throw NangilaError::layer_not_found(id);
    if (it->second.is_passenger()) {
      it->second = LayerRole{};
      --num_passengers_;
      ++num_drivers_;
    }
  }
  void validate() const {
    for (auto& kv : layers_) {
      if (!kv.second.is_passenger()) continue;
      LayerId src = kv.second.source_id;
      if (!is_driver(src)) {
        if (layers_.count(src))
          throw NangilaError::invalid_format("Passenger " + std::to_string(kv.first) +
                                             " depends on non-driver layer " + std::to_string(src) +
                                             ". Passengers can only depend on drivers.");
        throw NangilaError::invalid_format("Passenger " + std::to_string(kv.first) +
                                           " references non-existent driver " + std::to_string(src));
      }
      if (kv.first == src)
        throw NangilaError::invalid_format("Passenger " + std::to_string(kv.first) +
                                           " references itself as source");
    }
  }

  std::vector<uint8_t> to_bytes() const {
    std::vector<uint8_t> out;
    out.reserve(4 + layers_.size() * 17);
    auto put32 = [&out](uint32_t v) {
      uint8_t b[4];
      detail::put_le<uint32_t>(b, v);
      out.insert(out.end(), b, b + 4);
    };
    auto putf = [&](float f) {
      uint32_t u;
      std::memcpy(&u, &f, 4);
      put32(u);
    };
    put32(uint32_t(layers_.size()));
    for (auto& kv : layers_) {
      put32(kv.first);
      if (kv.second.is_driver()) {
        out.push_back(0);
      } else {
        out.push_back(1);
        put32(kv.second.source_id);
        putf(kv.second.alpha);
        putf(kv.second.beta);
      }
    }
    return out;
  }
  static TopologyMask from_bytes(const uint8_t* p, size_t len) {
    size_t off = 0;
    auto need = [&](size_t n) {
      if (off + n > len) throw NangilaError::io("failed to fill whole buffer (mask truncated)");
    };
    auto get32 = [&]() {
      need(4);
      uint32_t v = detail::get_le<uint32_t>(p + off);
      off += 4;
      return v;
    };
    auto getf = [&]() {
      uint32_t u = get32();
      float f;
      std::memcpy(&f, &u, 4);
      return f;
    };
    TopologyMask m;
    uint32_t n = get32();
    for (uint32_t i = 0; i < n; ++i) {
      LayerId id = get32();
      need(1);
      uint8_t tag = p[off++];
      if (tag == 0) {
        m.add_driver(id);
      } else if (tag == 1) {
        LayerId src = get32();
        float a = getf();
        float b = getf();
        m.add_passenger(id, src, a, b);
      } else {
        throw NangilaError::invalid_format("Invalid layer role tag " + std::to_string(int(tag)));
      }
    }
    return m;
  }
  static TopologyMask all_drivers(size_t n) {
    TopologyMask m;
    for (size_t i = 0; i < n; ++i) m.add_driver(LayerId(i));
    return m;
  }

 private:
  void erase_counts(LayerId id) {
    auto it = layers_.find(id);
    if (it == layers_.end()) return;
    if (it->second.is_driver()) --num_drivers_; else --num_passengers_;
  }
  std::map<LayerId, LayerRole> layers_;  // ordered: deterministic iteration and serialisation
  size_t num_drivers_ = 0;
  size_t num_passengers_ = 0;
};

}  // namespace nangila
