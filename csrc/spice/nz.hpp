// `.nz` waveform container: error-bounded lossy compression of simulation waveforms.
//
// Container layout (little endian), shared with the reference's format
// (nangila-spice/nangila-node/src/nz.rs:344-417): "NZWF", u16 version, u32 nodes, u32 points,
// f64 t_start, f64 t_end, f64 error_bound, names (u16 length + bytes), times (f64 each), u32 block
// count, then blocks: 0x01 predicted {u32 node, u32 start, u32 count, f64 base, f64 gradient,
// f64 scale, i16 residuals[count]} or 0x02 raw {u32 node, u32 start, u32 count, f64 values[count]}.
//
// Version 2 (written here) predicts every sample from the *reconstructed* previous two samples
// (linear extrapolation) and quantizes the residual with step 2 * error_bound, so the decoder sees
// exactly the predictor inputs the encoder used and |error| <= error_bound holds for every sample.
// Version 1 files (the reference's: damped-curvature prediction around a per-block line) are read
// with that rule.
#pragma once
#include <cmath>
#include <cstdint>
#include <cstring>
#include <fstream>
#include <stdexcept>
#include <string>
#include <vector>

namespace nspice {

struct NzBlock {
    bool predicted = true;
    uint32_t node = 0, start = 0, count = 0;
    double base = 0, gradient = 0, scale = 1;
    std::vector<int16_t> residuals;
    std::vector<double> raw;
};

struct NzFile {
    uint16_t version = 2;
    double t_start = 0, t_end = 0, error_bound = 0;
    std::vector<std::string> names;
    std::vector<double> time;
    std::vector<NzBlock> blocks;
};

struct NzStats {
    uint64_t total_points = 0, predicted_points = 0, raw_points = 0, predicted_blocks = 0, raw_blocks = 0, raw_bytes = 0, compressed_bytes = 0;
    double compression_ratio() const { return compressed_bytes ? double(raw_bytes) / double(compressed_bytes) : 1.0; }
    double prediction_rate() const { return total_points ? double(predicted_points) / double(total_points) : 0.0; }
};

namespace nz_detail {
template <class T> void put(std::string& b, T v) { char tmp[sizeof(T)]; std::memcpy(tmp, &v, sizeof(T)); b.append(tmp, sizeof(T)); }
template <class T> T get(const std::string& b, size_t& pos) {
    if (pos + sizeof(T) > b.size()) throw std::runtime_error("nz: truncated file");
    T v;
    std::memcpy(&v, b.data() + pos, sizeof(T));
    pos += sizeof(T);
    return v;
}
// prediction of sample i of a block from already reconstructed samples r[0..i)
inline double predict_v2(const NzBlock& b, const double* t, const double* r, uint32_t i) {
    if (i == 0) return b.base;
    if (i == 1) return b.base + b.gradient * (t[1] - t[0]);
    return 2.0 * r[i - 1] - r[i - 2];
}
inline double predict_v1(const NzBlock& b, const double* t, const double* r, uint32_t i) {
    double lin = b.base + b.gradient * (t[i] - t[0]);
    if (i >= 2) lin += 0.25 * (r[i - 2] - 2.0 * r[i - 1] + lin);
    return lin;
}
}  // namespace nz_detail

class NzWriter {
public:
    double error_bound;
    size_t block_size = 256;
    NzStats stats;
    explicit NzWriter(double eb = 1e-6) : error_bound(eb > 0 ? eb : 1e-12) {}

    NzFile compress(const std::vector<std::string>& names, const std::vector<double>& time, const std::vector<std::vector<double>>& signals) {
        NzFile f;
        f.names = names;
        f.time = time;
        f.error_bound = error_bound;
        f.t_start = time.empty() ? 0.0 : time.front();
        f.t_end = time.empty() ? 0.0 : time.back();
        for (size_t n = 0; n < signals.size(); ++n) {
            if (signals[n].size() != time.size()) throw std::invalid_argument("nz: signal length differs from the time axis");
            for (size_t pos = 0; pos < time.size(); pos += block_size) {
                size_t cnt = std::min(block_size, time.size() - pos);
                NzBlock b;
                b.node = uint32_t(n); b.start = uint32_t(pos); b.count = uint32_t(cnt);
                if (!encode_block(b, time.data() + pos, signals[n].data() + pos)) {
                    b.predicted = false;
                    b.residuals.clear();
                    b.raw.assign(signals[n].begin() + long(pos), signals[n].begin() + long(pos + cnt));
                    stats.raw_points += cnt; ++stats.raw_blocks;
                    stats.compressed_bytes += 13 + 8 * cnt;
                } else {
                    stats.predicted_points += cnt; ++stats.predicted_blocks;
                    stats.compressed_bytes += 37 + 2 * cnt;
                }
                stats.total_points += cnt;
                f.blocks.push_back(std::move(b));
            }
        }
        stats.raw_bytes += uint64_t(signals.size()) * time.size() * 8;
        stats.compressed_bytes += 38;
        return f;
    }

    static std::string to_bytes(const NzFile& f) {
        using nz_detail::put;
        std::string b("NZWF");
        put<uint16_t>(b, f.version);
        put<uint32_t>(b, uint32_t(f.names.size()));
        put<uint32_t>(b, uint32_t(f.time.size()));
        put<double>(b, f.t_start); put<double>(b, f.t_end); put<double>(b, f.error_bound);
        for (auto& n : f.names) { put<uint16_t>(b, uint16_t(n.size())); b.append(n); }
        for (double t : f.time) put<double>(b, t);
        put<uint32_t>(b, uint32_t(f.blocks.size()));
        for (auto& k : f.blocks) {
            b.push_back(k.predicted ? char(1) : char(2));
            put<uint32_t>(b, k.node); put<uint32_t>(b, k.start); put<uint32_t>(b, k.count);
            if (k.predicted) {
                put<double>(b, k.base); put<double>(b, k.gradient); put<double>(b, k.scale);
                for (int16_t r : k.residuals) put<int16_t>(b, r);
            } else {
                for (double v : k.raw) put<double>(b, v);
            }
        }
        return b;
    }

    void write_file(const std::string& path, const std::vector<std::string>& names, const std::vector<double>& time,
                    const std::vector<std::vector<double>>& signals) {
        std::string bytes = to_bytes(compress(names, time, signals));
        std::ofstream f(path, std::ios::binary);
        if (!f) throw std::runtime_error("cannot write '" + path + "'");
        f.write(bytes.data(), long(bytes.size()));
    }

private:
    bool encode_block(NzBlock& b, const double* t, const double* v) const {
        if (b.count < 2) return false;
        b.base = v[0];
        double dt = t[1] - t[0];
        b.gradient = std::fabs(dt) > 1e-30 ? (v[1] - v[0]) / dt : 0.0;
        b.scale = 2.0 * error_bound;
        b.residuals.resize(b.count);
        std::vector<double> r(b.count);
        for (uint32_t i = 0; i < b.count; ++i) {
            double p = nz_detail::predict_v2(b, t, r.data(), i);
            double q = std::nearbyint((v[i] - p) / b.scale);
            if (!(std::fabs(q) <= 32767.0)) return false;
            b.residuals[i] = int16_t(q);
            r[i] = p + q * b.scale;
            if (!(std::fabs(r[i] - v[i]) <= error_bound * (1.0 + 1e-9))) return false;
        }
        return true;
    }
};

class NzReader {
public:
    static NzFile from_bytes(const std::string& b) {
        using nz_detail::get;
        if (b.size() < 4 || b.compare(0, 4, "NZWF") != 0) throw std::runtime_error("nz: bad magic");
        size_t pos = 4;
        NzFile f;
        f.version = get<uint16_t>(b, pos);
        if (f.version != 1 && f.version != 2) throw std::runtime_error("nz: unsupported version");
        uint32_t nodes = get<uint32_t>(b, pos), points = get<uint32_t>(b, pos);
        f.t_start = get<double>(b, pos); f.t_end = get<double>(b, pos); f.error_bound = get<double>(b, pos);
        for (uint32_t i = 0; i < nodes; ++i) {
            uint16_t len = get<uint16_t>(b, pos);
            if (pos + len > b.size()) throw std::runtime_error("nz: truncated file");
            f.names.emplace_back(b.substr(pos, len));
            pos += len;
        }
        if (uint64_t(points) * 8 > b.size() - pos) throw std::runtime_error("nz: truncated file");
        for (uint32_t i = 0; i < points; ++i) f.time.push_back(get<double>(b, pos));
        uint32_t nb = get<uint32_t>(b, pos);
        for (uint32_t k = 0; k < nb; ++k) {
            NzBlock blk;
            uint8_t kind = get<uint8_t>(b, pos);
            blk.node = get<uint32_t>(b, pos); blk.start = get<uint32_t>(b, pos); blk.count = get<uint32_t>(b, pos);
            if (blk.node >= nodes || uint64_t(blk.start) + blk.count > points) throw std::runtime_error("nz: block outside the waveform");
            if (kind == 1) {
                blk.base = get<double>(b, pos); blk.gradient = get<double>(b, pos); blk.scale = get<double>(b, pos);
                if (uint64_t(blk.count) * 2 > b.size() - pos) throw std::runtime_error("nz: truncated file");
                for (uint32_t i = 0; i < blk.count; ++i) blk.residuals.push_back(get<int16_t>(b, pos));
            } else if (kind == 2) {
                blk.predicted = false;
                if (uint64_t(blk.count) * 8 > b.size() - pos) throw std::runtime_error("nz: truncated file");
                for (uint32_t i = 0; i < blk.count; ++i) blk.raw.push_back(get<double>(b, pos));
            } else {
                throw std::runtime_error("nz: unknown block type");
            }
            f.blocks.push_back(std::move(blk));
        }
        return f;
    }
    static NzFile read_file(const std::string& path) {
        std::ifstream f(path, std::ios::binary);
        if (!f) throw std::runtime_error("cannot open '" + path + "'");
        std::string bytes((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
        return from_bytes(bytes);
    }
    // One vector per node, in header order.
    static std::vector<std::vector<double>> decompress(const NzFile& f) {
        std::vector<std::vector<double>> out(f.names.size(), std::vector<double>(f.time.size(), 0.0));
        for (auto& b : f.blocks) {
            double* r = out[b.node].data() + b.start;
            const double* t = f.time.data() + b.start;
            if (!b.predicted) { for (uint32_t i = 0; i < b.count; ++i) r[i] = b.raw[i]; continue; }
            for (uint32_t i = 0; i < b.count; ++i) {
                double p = f.version >= 2 ? nz_detail::predict_v2(b, t, r, i) : nz_detail::predict_v1(b, t, r, i);
                r[i] = p + double(b.residuals[i]) * b.scale;
            }
        }
        return out;
    }
};

}  // namespace nspice
