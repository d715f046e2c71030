// JSON report of a topology mask (and optionally of the Sculptor statistics behind it): summary,
// per-layer role with its coupling, optional correlation matrix, and the driver -> passenger edges.
//
// Parity: nangila-core/src/topology_report.rs:11-56 (schema: summary{num_layers, num_drivers,
// num_passengers, compression_ratio, threshold}, layers[{layer_id, role, source_id, alpha, beta}],
// correlation_matrix{layer_ids, values} | null, dependency_graph[{from_layer, to_layer, alpha,
// relationship:"drives"}]), :58-143 (builders and JSON output).
#pragma once
#include <cstdio>
#include <sstream>
#include <string>
#include <vector>

#include "mask.hpp"
#include "sculptor.hpp"

namespace nangila {

struct TopologyReport {
  struct LayerInfo { LayerId layer_id; bool passenger; LayerId source_id; float alpha, beta; };
  struct Edge { LayerId from_layer, to_layer; float alpha; };

  size_t num_layers = 0, num_drivers = 0, num_passengers = 0;
  float compression_ratio = 1.0f, threshold = 0.95f;
  std::vector<LayerInfo> layers;
  bool has_matrix = false;
  std::vector<LayerId> matrix_ids;
  std::vector<std::vector<float>> matrix;
  std::vector<Edge> dependency_graph;

  static TopologyReport from_mask(const TopologyMask& mask) {
    TopologyReport r;
    for (LayerId id : mask.all_layer_ids()) {
      const LayerRole& role = mask.get_role(id);
      r.layers.push_back({id, role.is_passenger(), role.source_id, role.alpha, role.beta});
      if (role.is_passenger()) r.dependency_graph.push_back({role.source_id, id, role.alpha});
    }
    r.num_drivers = mask.num_drivers();
    r.num_passengers = mask.num_passengers();
    r.num_layers = r.num_drivers + r.num_passengers;
    r.compression_ratio = mask.compression_ratio();
    return r;
  }
  static TopologyReport from_sculptor_and_mask(const Sculptor& s, const TopologyMask& mask) {
    TopologyReport r = from_mask(mask);
    if (s.num_layers() > 0 && s.num_samples() > 1) {
      if (auto m = s.correlation_matrix()) {
        r.has_matrix = true;
        r.matrix_ids = s.layer_ids();
        r.matrix = *m;
      }
    }
    r.threshold = s.threshold();
    return r;
  }

  static std::string num(float f) {
    char b[48];
    std::snprintf(b, sizeof b, "%.9g", double(f));
    return b;
  }
  std::string to_json(bool pretty = true) const {
    const char* nl = pretty ? "\n" : "";
    auto ind = [&](int n) { return pretty ? std::string(size_t(n) * 2, ' ') : std::string(); };
    const char* sp = pretty ? " " : "";
    std::ostringstream o;
    o << "{" << nl << ind(1) << "\"summary\":" << sp << "{" << nl;
    o << ind(2) << "\"num_layers\":" << sp << num_layers << "," << nl;
    o << ind(2) << "\"num_drivers\":" << sp << num_drivers << "," << nl;
    o << ind(2) << "\"num_passengers\":" << sp << num_passengers << "," << nl;
    o << ind(2) << "\"compression_ratio\":" << sp << num(compression_ratio) << "," << nl;
    o << ind(2) << "\"threshold\":" << sp << num(threshold) << nl << ind(1) << "}," << nl;
    o << ind(1) << "\"layers\":" << sp << "[" << nl;
    for (size_t i = 0; i < layers.size(); ++i) {
      const LayerInfo& l = layers[i];
      o << ind(2) << "{\"layer_id\":" << sp << l.layer_id << "," << sp << "\"role\":" << sp
        << (l.passenger ? "\"passenger\"" : "\"driver\"") << "," << sp << "\"source_id\":" << sp;
      if (l.passenger) o << l.source_id; else o << "null";
      o << "," << sp << "\"alpha\":" << sp << (l.passenger ? num(l.alpha) : std::string("null"));
      o << "," << sp << "\"beta\":" << sp << (l.passenger ? num(l.beta) : std::string("null")) << "}";
      o << (i + 1 < layers.size() ? "," : "") << nl;
    }
    o << ind(1) << "]," << nl << ind(1) << "\"correlation_matrix\":" << sp;
    if (!has_matrix) {
      o << "null";
    } else {
      o << "{" << nl << ind(2) << "\"layer_ids\":" << sp << "[";
      for (size_t i = 0; i < matrix_ids.size(); ++i) o << (i ? "," : "") << matrix_ids[i];
      o << "]," << nl << ind(2) << "\"values\":" << sp << "[" << nl;
      for (size_t i = 0; i < matrix.size(); ++i) {
        o << ind(3) << "[";
        for (size_t j = 0; j < matrix[i].size(); ++j) o << (j ? "," : "") << num(matrix[i][j]);
        o << "]" << (i + 1 < matrix.size() ? "," : "") << nl;
      }
      o << ind(2) << "]" << nl << ind(1) << "}";
    }
    o << "," << nl << ind(1) << "\"dependency_graph\":" << sp << "[" << nl;
    for (size_t i = 0; i < dependency_graph.size(); ++i) {
      const Edge& e = dependency_graph[i];
      o << ind(2) << "{\"from_layer\":" << sp << e.from_layer << "," << sp << "\"to_layer\":" << sp << e.to_layer
        << "," << sp << "\"alpha\":" << sp << num(e.alpha) << "," << sp << "\"relationship\":" << sp
        << "\"drives\"}" << (i + 1 < dependency_graph.size() ? "," : "") << nl;
    }
    o << ind(1) << "]" << nl << "}";
    return o.str();
  }
  std::string to_json_compact() const { return to_json(false); }
};

}  // namespace nangila
