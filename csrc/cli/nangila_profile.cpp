// nangila-profile: offline Sculptor calibration from recorded gradients.
//   nangila-profile calibrate -g grads.jsonl [-s 500] [-t 0.95] -o mask.bin [--report report.json]
//   nangila-profile report    -m mask.bin -o report.json
//   nangila-profile info      -m mask.bin
// Input: JSON lines {"step": int, "layer_id": int, "data": [float...], "shape": [int...]}.
// Sub-commands and options follow the reference tool (nangila-profile/src/main.rs:25-206). Unlike the
// reference (which never closes a calibration step, so its masks are always all-Driver), a change of
// "step" between lines closes the step and updates the pair statistics.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <iostream>
#include <string>

#include "sculptor.hpp"
#include "topology_report.hpp"

using namespace nangila;

static const char* opt(int argc, char** argv, const char* s, const char* l) {
  for (int i = 2; i + 1 < argc; ++i)
    if ((s && !std::strcmp(argv[i], s)) || !std::strcmp(argv[i], l)) return argv[i + 1];
  return nullptr;
}
static int usage() {
  std::fprintf(stderr, "usage: nangila-profile calibrate -g FILE [-s N] [-t T] -o MASK [--report JSON] | "
                       "report -m MASK -o JSON | info -m MASK\n");
  return 1;
}
// Minimal scanner for the fixed line schema.
static bool find_key(const std::string& line, const char* key, size_t* pos) {
  std::string k = std::string("\"") + key + "\"";
  size_t p = line.find(k);
  if (p == std::string::npos) return false;
  p = line.find(':', p + k.size());
  if (p == std::string::npos) return false;
  *pos = p + 1;
  return true;
}
static bool parse_line(const std::string& line, long* step, long* layer, std::vector<float>* data) {
  size_t p;
  if (!find_key(line, "step", &p)) return false;
  *step = std::strtol(line.c_str() + p, nullptr, 10);
  if (!find_key(line, "layer_id", &p)) return false;
  *layer = std::strtol(line.c_str() + p, nullptr, 10);
  if (!find_key(line, "data", &p)) return false;
  p = line.find('[', p);
  if (p == std::string::npos) return false;
  data->clear();
  const char* c = line.c_str() + p + 1;
  while (*c && *c != ']') {
    char* end;
    float v = std::strtof(c, &end);
    if (end == c) { ++c; continue; }
    data->push_back(v);
    c = end;
  }
  return true;
}
static TopologyMask load_mask(const char* path) {
  std::ifstream f(path, std::ios::binary);
  if (!f) throw NangilaError::io(std::string("cannot open ") + path);
  std::vector<uint8_t> b((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
  return TopologyMask::from_bytes(b.data(), b.size());
}

int main(int argc, char** argv) {
  if (argc < 2) return usage();
  const std::string cmd = argv[1];
  try {
    if (cmd == "calibrate") {
      const char* g = opt(argc, argv, "-g", "--gradients");
      const char* o = opt(argc, argv, "-o", "--output");
      const char* s = opt(argc, argv, "-s", "--steps");
      const char* t = opt(argc, argv, "-t", "--threshold");
      const char* rep = opt(argc, argv, nullptr, "--report");
      if (!g || !o) return usage();
      const long max_steps = s ? std::strtol(s, nullptr, 10) : 500;
      Sculptor sc(t ? std::strtof(t, nullptr) : 0.95f);
      sc.set_auto_end_step(false);
      std::ifstream f(g);
      if (!f) throw NangilaError::io(std::string("cannot open ") + g);
      std::string line;
      std::vector<float> data;
      long cur_step = -1, steps_seen = 0, samples = 0;
      while (std::getline(f, line)) {
        long step, layer;
        if (line.empty() || !parse_line(line, &step, &layer, &data)) continue;
        if (step != cur_step) {
          if (cur_step >= 0) sc.end_step();
          if (steps_seen >= max_steps) { cur_step = -1; break; }
          cur_step = step;
          ++steps_seen;
        }
        sc.record(LayerId(layer), data.data(), data.size());
        ++samples;
      }
      if (cur_step >= 0 && sc.has_open_step()) sc.end_step();
      std::printf("Loaded %ld gradient samples over %ld steps, %zu layers\n", samples, steps_seen, sc.num_layers());
      TopologyMask mask = sc.generate_mask();
      std::vector<uint8_t> bytes = mask.to_bytes();
      std::ofstream out(o, std::ios::binary);
      out.write(reinterpret_cast<const char*>(bytes.data()), std::streamsize(bytes.size()));
      std::printf("Mask: %zu drivers, %zu passengers, %.2fx layer compression -> %s\n", mask.num_drivers(),
                  mask.num_passengers(), mask.compression_ratio(), o);
      if (rep) {
        std::ofstream r(rep);
        r << TopologyReport::from_sculptor_and_mask(sc, mask).to_json() << "\n";
        std::printf("Report written to %s\n", rep);
      }
      return 0;
    }
    if (cmd == "report") {
      const char* m = opt(argc, argv, "-m", "--mask");
      const char* o = opt(argc, argv, "-o", "--output");
      if (!m || !o) return usage();
      std::ofstream r(o);
      r << TopologyReport::from_mask(load_mask(m)).to_json() << "\n";
      std::printf("Report written to %s\n", o);
      return 0;
    }
    if (cmd == "info") {
      const char* m = opt(argc, argv, "-m", "--mask");
      if (!m) return usage();
      TopologyMask mask = load_mask(m);
      mask.validate();
      std::printf("Topology mask: %s\n  Layers:      %zu\n  Drivers:     %zu\n  Passengers:  %zu\n  Compression: %.2fx\n", m,
                  mask.num_layers(), mask.num_drivers(), mask.num_passengers(), mask.compression_ratio());
      for (auto& p : mask.passengers())
        std::printf("  layer %u <- %.4f * layer %u + %.4f\n", p.id, p.alpha, p.source, p.beta);
      return 0;
    }
  } catch (const std::exception& e) {
    std::fprintf(stderr, "Error: %s\n", e.what());
    return 1;
  }
  return usage();
}
