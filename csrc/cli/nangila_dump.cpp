// nangila-dump: inspect and compare NZCHK001 checkpoints.
//   nangila-dump verify  -c FILE          exit 2 when the stored state hash does not match
//   nangila-dump diff    -a FILE -b FILE  JSON result; exit 3 when the two states differ
//   nangila-dump inspect -c FILE [-o OUT] JSON with per-layer sizes and hashes
//   nangila-dump info    -c FILE          human-readable summary
// Sub-commands, options and exit codes follow the reference tool (nangila-dump/src/main.rs:23-58,
// :116-295).
#include <cstdio>
#include <cstring>
#include <fstream>
#include <iostream>
#include <sstream>
#include <string>

#include "checkpoint.hpp"

using namespace nangila;

static std::string hex16(uint64_t v) {
  char b[32];
  std::snprintf(b, sizeof b, "%016llx", static_cast<unsigned long long>(v));
  return b;
}
static uint64_t hash_bits(const std::vector<int32_t>& v) {
  SipHasher13 h;
  for (int32_t x : v) h.write_i32(x);
  return h.finish();
}
static const char* opt(int argc, char** argv, const char* s, const char* l) {
  for (int i = 2; i + 1 < argc; ++i)
    if (!std::strcmp(argv[i], s) || !std::strcmp(argv[i], l)) return argv[i + 1];
  return nullptr;
}
static int usage() {
  std::fprintf(stderr,
               "usage: nangila-dump verify -c FILE | diff -a FILE -b FILE | inspect -c FILE [-o OUT] | info -c FILE\n");
  return 1;
}

int main(int argc, char** argv) {
  if (argc < 2) return usage();
  const std::string cmd = argv[1];
  try {
    if (cmd == "verify") {
      const char* p = opt(argc, argv, "-c", "--checkpoint");
      if (!p) return usage();
      NangilaCheckpoint c = NangilaCheckpoint::load(p);
      const uint64_t computed = c.compute_hash();
      if (computed == c.state_hash) {
        std::printf("VALID: Checkpoint integrity verified\n  Step: %llu\n  Hash: %s\n  Layers: %zu\n",
                    (unsigned long long)c.step, hex16(c.state_hash).c_str(), c.predictor.histories.size());
        return 0;
      }
      std::printf("INVALID: Checkpoint integrity check failed\n  Stored hash:   %s\n  Computed hash: %s\n",
                  hex16(c.state_hash).c_str(), hex16(computed).c_str());
      return 2;
    }
    if (cmd == "diff") {
      const char* pa = opt(argc, argv, "-a", "--checkpoint-a");
      const char* pb = opt(argc, argv, "-b", "--checkpoint-b");
      if (!pa || !pb) return usage();
      NangilaCheckpoint a = NangilaCheckpoint::load(pa), b = NangilaCheckpoint::load(pb);
      std::vector<LayerId> divergent;
      for (auto& kv : a.predictor.histories) {
        auto it = b.predictor.histories.find(kv.first);
        if (it == b.predictor.histories.end() || it->second.prev != kv.second.prev || it->second.current != kv.second.current)
          divergent.push_back(kv.first);
      }
      for (auto& kv : b.predictor.histories)
        if (!a.predictor.histories.count(kv.first)) divergent.push_back(kv.first);
      const bool same = divergent.empty() && a.step == b.step && a.compute_hash() == b.compute_hash();
      std::printf("{\n  \"match_status\": \"%s\",\n  \"step_a\": %llu,\n  \"step_b\": %llu,\n  \"hash_a\": \"%s\",\n"
                  "  \"hash_b\": \"%s\",\n  \"divergent_layers\": [",
                  same ? "MATCH" : "DIVERGED", (unsigned long long)a.step, (unsigned long long)b.step,
                  hex16(a.compute_hash()).c_str(), hex16(b.compute_hash()).c_str());
      for (size_t i = 0; i < divergent.size(); ++i) std::printf("%s%u", i ? ", " : "", divergent[i]);
      std::printf("]\n}\n");
      return same ? 0 : 3;
    }
    if (cmd == "inspect") {
      const char* p = opt(argc, argv, "-c", "--checkpoint");
      const char* o = opt(argc, argv, "-o", "--output");
      if (!p) return usage();
      NangilaCheckpoint c = NangilaCheckpoint::load(p);
      std::ostringstream js;
      js << "{\n  \"info\": {\n    \"version\": " << c.version << ",\n    \"step\": " << c.step << ",\n    \"state_hash\": \""
         << hex16(c.state_hash) << "\",\n    \"integrity_valid\": " << (c.verify_integrity() ? "true" : "false")
         << ",\n    \"num_layers\": " << c.predictor.histories.size() << ",\n    \"quantizer_gamma\": " << c.quantizer_gamma
         << ",\n    \"warmup_steps\": " << c.config.warmup_steps << ",\n    \"predictor_step\": " << c.predictor.current_step
         << ",\n    \"predictor_momentum\": " << c.predictor.momentum << ",\n    \"extra_sections\": " << c.extra.size()
         << "\n  },\n  \"layers\": [";
      bool first = true;
      for (auto& kv : c.predictor.histories) {
        js << (first ? "\n" : ",\n") << "    {\"layer_id\": " << kv.first << ", \"has_prev\": " << (kv.second.prev ? "true" : "false")
           << ", \"has_current\": " << (kv.second.current ? "true" : "false") << ", \"prev_size\": "
           << (kv.second.prev ? kv.second.prev->size() : 0) << ", \"current_size\": "
           << (kv.second.current ? kv.second.current->size() : 0) << ", \"prev_hash\": ";
        if (kv.second.prev) js << "\"" << hex16(hash_bits(*kv.second.prev)) << "\""; else js << "null";
        js << ", \"current_hash\": ";
        if (kv.second.current) js << "\"" << hex16(hash_bits(*kv.second.current)) << "\""; else js << "null";
        js << "}";
        first = false;
      }
      js << "\n  ]\n}\n";
      if (o) {
        std::ofstream f(o);
        f << js.str();
        std::printf("Written to: %s\n", o);
      } else {
        std::cout << js.str();
      }
      return 0;
    }
    if (cmd == "info") {
      const char* p = opt(argc, argv, "-c", "--checkpoint");
      if (!p) return usage();
      NangilaCheckpoint c = NangilaCheckpoint::load(p);
      size_t elems = 0;
      for (auto& kv : c.predictor.histories) {
        if (kv.second.prev) elems += kv.second.prev->size();
        if (kv.second.current) elems += kv.second.current->size();
      }
      std::printf("Nangila Checkpoint: %s\n-------------------------------------\n", p);
      std::printf("  Version:          %u\n  Step:             %llu\n  State Hash:       %s\n  Integrity:        %s\n",
                  c.version, (unsigned long long)c.step, hex16(c.state_hash).c_str(), c.verify_integrity() ? "valid" : "INVALID");
      std::printf("  Layers:           %zu (%zu Q8.23 values, %.2f MB)\n", c.predictor.histories.size(), elems, elems * 4.0 / 1e6);
      std::printf("  Quantizer Gamma:  %.6f\n  Predictor Step:   %zu\n  Predictor mu:     %g\n  Warmup Steps:     %zu\n",
                  c.quantizer_gamma, c.predictor.current_step, c.predictor.momentum, c.config.warmup_steps);
      std::printf("  Extra sections:   %zu\n", c.extra.size());
      return 0;
    }
  } catch (const std::exception& e) {
    std::fprintf(stderr, "Error: %s\n", e.what());
    return 1;
  }
  return usage();
}
