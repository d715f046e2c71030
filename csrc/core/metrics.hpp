// Thread-safe counters with Prometheus text and JSON export.
//
// Parity: nangila-core/src/metrics.rs:12-122 (collector: steps, bytes, fallbacks, ratio; snapshot
// derives compression ratio = received / transmitted, virtual / physical throughput in Gbit/s and
// bytes saved), :126-232 (metric names and number formats of the Prometheus text, JSON keys).
#pragma once
#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <string>

namespace nangila {

struct NangilaMetrics {
  float compression_ratio = 1.0f;
  double virtual_throughput_gbps = 0, physical_throughput_gbps = 0;
  uint64_t steps_total = 0, steps_compressed = 0;
  uint64_t bytes_received = 0, bytes_transmitted = 0, bytes_saved = 0;
  uint32_t fallback_count = 0;
  double uptime_seconds = 0;

  std::string to_prometheus() const {
    std::string o;
    char buf[256];
    auto gauge = [&](const char* name, const char* help, const char* type, const char* fmt, double v, bool last = false) {
      std::snprintf(buf, sizeof buf, "# HELP %s %s\n# TYPE %s %s\n", name, help, name, type);
      o += buf;
      std::snprintf(buf, sizeof buf, fmt, v);
      o += std::string(name) + " " + buf + (last ? "\n" : "\n\n");
    };
    auto counter = [&](const char* name, const char* help, uint64_t v) {
      std::snprintf(buf, sizeof buf, "# HELP %s %s\n# TYPE %s counter\n%s %llu\n\n", name, help, name, name,
                    static_cast<unsigned long long>(v));
      o += buf;
    };
    gauge("nangila_compression_ratio", "Current compression ratio", "gauge", "%.3f", compression_ratio);
    gauge("nangila_virtual_throughput_gbps", "Effective bandwidth in Gbps", "gauge", "%.6f", virtual_throughput_gbps);
    gauge("nangila_physical_throughput_gbps", "Actual bandwidth in Gbps", "gauge", "%.6f", physical_throughput_gbps);
    counter("nangila_steps_total", "Total training steps", steps_total);
    counter("nangila_steps_compressed", "Steps with compression enabled", steps_compressed);
    counter("nangila_bytes_received", "Total bytes received (uncompressed)", bytes_received);
    counter("nangila_bytes_transmitted", "Total bytes transmitted (compressed)", bytes_transmitted);
    counter("nangila_bytes_saved", "Total bytes saved by compression", bytes_saved);
    counter("nangila_fallback_total", "Safe Mode fallback events", fallback_count);
    gauge("nangila_uptime_seconds", "Time since start", "gauge", "%.3f", uptime_seconds, true);
    return o;
  }
  std::string to_json() const {
    char buf[768];
    std::snprintf(buf, sizeof buf,
                  "{\n  \"compression_ratio\": %.6g,\n  \"virtual_throughput_gbps\": %.9g,\n"
                  "  \"physical_throughput_gbps\": %.9g,\n  \"steps_total\": %llu,\n  \"steps_compressed\": %llu,\n"
                  "  \"bytes_received\": %llu,\n  \"bytes_transmitted\": %llu,\n  \"bytes_saved\": %llu,\n"
                  "  \"fallback_count\": %u,\n  \"uptime_seconds\": %.6f\n}",
                  compression_ratio, virtual_throughput_gbps, physical_throughput_gbps,
                  (unsigned long long)steps_total, (unsigned long long)steps_compressed,
                  (unsigned long long)bytes_received, (unsigned long long)bytes_transmitted,
                  (unsigned long long)bytes_saved, fallback_count, uptime_seconds);
    return buf;
  }
};

class MetricsCollector {
 public:
  MetricsCollector() : start_(std::chrono::steady_clock::now()) {}
  void record_step(bool compressed) {
    steps_total_.fetch_add(1, std::memory_order_relaxed);
    if (compressed) steps_compressed_.fetch_add(1, std::memory_order_relaxed);
  }
  // received = bytes the step would have moved uncompressed; transmitted = bytes actually moved.
  void record_bytes(uint64_t received, uint64_t transmitted) {
    bytes_received_.fetch_add(received, std::memory_order_relaxed);
    bytes_transmitted_.fetch_add(transmitted, std::memory_order_relaxed);
  }
  void record_fallback() { fallbacks_.fetch_add(1, std::memory_order_relaxed); }
  void set_compression_ratio(float r) { ratio_x1000_.store(uint64_t(r * 1000.0f), std::memory_order_relaxed); }
  NangilaMetrics snapshot() const {
    NangilaMetrics m;
    double el = std::chrono::duration<double>(std::chrono::steady_clock::now() - start_).count();
    m.bytes_received = bytes_received_.load();
    m.bytes_transmitted = bytes_transmitted_.load();
    m.compression_ratio = m.bytes_transmitted > 0 ? float(double(m.bytes_received) / double(m.bytes_transmitted))
                                                  : float(double(ratio_x1000_.load()) / 1000.0);
    if (el > 0) {
      m.virtual_throughput_gbps = double(m.bytes_received) * 8.0 / (el * 1e9);
      m.physical_throughput_gbps = double(m.bytes_transmitted) * 8.0 / (el * 1e9);
    }
    m.steps_total = steps_total_.load();
    m.steps_compressed = steps_compressed_.load();
    m.bytes_saved = m.bytes_received > m.bytes_transmitted ? m.bytes_received - m.bytes_transmitted : 0;
    m.fallback_count = uint32_t(fallbacks_.load());
    m.uptime_seconds = el;
    return m;
  }
  void reset() {
    steps_total_ = 0;
    steps_compressed_ = 0;
    bytes_received_ = 0;
    bytes_transmitted_ = 0;
    fallbacks_ = 0;
  }

 private:
  std::chrono::steady_clock::time_point start_;
  std::atomic<uint64_t> steps_total_{0}, steps_compressed_{0}, bytes_received_{0}, bytes_transmitted_{0},
      fallbacks_{0}, ratio_x1000_{1000};
};

}  // namespace nangila
