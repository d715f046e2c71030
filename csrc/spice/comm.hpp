// Messages between partitions, the residual codec, the per-node mailbox, a thread-safe full-mesh
// fabric and the speculative-depth controller.
// Behavioural reference: nangila-spice/nangila-node/src/comm.rs:14-134, codec.rs:19-205,
// fabric.rs:23-357. The reference's fabric is tokio mpsc channels between async tasks; this one is
// plain mutex + condition-variable queues shared by std::thread workers (one per partition).
#pragma once
#include <algorithm>
#include <chrono>
#include <cmath>
#include <condition_variable>
#include <cstdint>
#include <deque>
#include <memory>
#include <mutex>
#include <string>
#include <utility>
#include <vector>

#include "json.hpp"

namespace nspice {

struct ResidualMessage {
    uint32_t from = 0, to = 0;
    double time = 0;
    std::vector<std::pair<uint64_t, double>> updates;  // (net id, true voltage)
};
struct RollbackRequest { uint32_t from = 0; double rollback_to_time = 0; };
struct NodeStatus { uint32_t partition = 0; double time = 0; uint64_t steps = 0, hits = 0, misses = 0, rollbacks = 0; };

struct CompressedResidual {
    uint32_t from = 0, to = 0;
    double time = 0;
    std::vector<std::pair<uint64_t, int32_t>> deltas;
    double scale = 1.0;
    std::vector<std::pair<uint64_t, double>> base_values;

    Json to_json() const {
        Json j = Json::object();
        j.set("from_partition", uint64_t(from)).set("to_partition", uint64_t(to)).set("time", time);
        Json d = Json::array();
        for (auto& p : deltas) { Json t = Json::array(); t.push(p.first).push(int64_t(p.second)); d.push(t); }
        Json b = Json::array();
        for (auto& p : base_values) { Json t = Json::array(); t.push(p.first).push(p.second); b.push(t); }
        j.set("deltas", d).set("scale", scale).set("base_values", b);
        return j;
    }
    static CompressedResidual from_json(const Json& j) {
        CompressedResidual c;
        c.from = uint32_t(j.number("from_partition", 0));
        c.to = uint32_t(j.number("to_partition", 0));
        c.time = j.number("time", 0);
        c.scale = j.number("scale", 1.0);
        for (auto& t : j.at("deltas").arr) c.deltas.emplace_back(uint64_t(t.arr.at(0).as_num()), int32_t(t.arr.at(1).as_num()));
        for (auto& t : j.at("base_values").arr) c.base_values.emplace_back(uint64_t(t.arr.at(0).as_num()), t.arr.at(1).as_num());
        return c;
    }
};

struct CodecStats {
    uint64_t encoded = 0, decoded = 0, updates = 0, skipped = 0, raw_bytes = 0, compressed_bytes = 0;
    double compression_ratio() const { return compressed_bytes ? double(raw_bytes) / double(compressed_bytes) : 1.0; }
};

// Sends (true - predicted) per net, quantized to `quant_bits` signed levels with one scale per
// message; deltas under `min_delta` are dropped (the receiver keeps its prediction).
class ResidualCodec {
public:
    int quant_bits = 16;
    double min_delta = 1e-15;
    CodecStats stats;

    CompressedResidual encode(const ResidualMessage& msg, const std::vector<std::pair<uint64_t, double>>& predicted) {
        const int32_t max_q = (int32_t(1) << (quant_bits - 1)) - 1;
        CompressedResidual out;
        out.from = msg.from; out.to = msg.to; out.time = msg.time;
        std::vector<std::pair<uint64_t, double>> raw;
        double max_delta = 0.0;
        // the caller usually lists predictions in the order of the updates: look there first, else search from
        // where the last match was found
        size_t at = 0;
        for (auto& u : msg.updates) {
            double pred = 0.0;
            for (size_t tries = 0; tries < predicted.size(); ++tries) {
                const size_t i = (at + tries) % predicted.size();
                if (predicted[i].first == u.first) { pred = predicted[i].second; at = i + 1; break; }
            }
            double d = u.second - pred;
            if (std::fabs(d) < min_delta) { ++stats.skipped; continue; }
            max_delta = std::max(max_delta, std::fabs(d));
            raw.emplace_back(u.first, d);
            out.base_values.emplace_back(u.first, pred);
        }
        out.scale = max_delta > 0.0 ? max_delta / double(max_q) : 1.0;
        for (auto& r : raw) {
            long q = std::lround(r.second / out.scale);
            out.deltas.emplace_back(r.first, int32_t(std::min<long>(max_q, std::max<long>(-max_q, q))));
        }
        ++stats.encoded;
        stats.updates += msg.updates.size();
        stats.raw_bytes += msg.updates.size() * 16;
        stats.compressed_bytes += out.deltas.size() * 12;
        return out;
    }
    ResidualMessage decode(const CompressedResidual& c) {
        ResidualMessage m;
        m.from = c.from; m.to = c.to; m.time = c.time;
        for (size_t k = 0; k < c.deltas.size(); ++k) {
            auto& d = c.deltas[k];
            double base = 0.0;
            if (k < c.base_values.size() && c.base_values[k].first == d.first) base = c.base_values[k].second;  // the encoder writes both in step
            else
                for (auto& b : c.base_values) if (b.first == d.first) { base = b.second; break; }
            m.updates.emplace_back(d.first, base + double(d.second) * c.scale);
        }
        ++stats.decoded;
        return m;
    }
    std::string encode_to_bytes(const ResidualMessage& msg, const std::vector<std::pair<uint64_t, double>>& predicted) {
        return encode(msg, predicted).to_json().dump();
    }
    bool decode_from_bytes(const std::string& bytes, ResidualMessage& out) {
        try { out = decode(CompressedResidual::from_json(Json::parse(bytes))); return true; }
        catch (const std::exception&) { return false; }
    }
};

// Mailbox of one solver node. Single-process runs use inject_* from tests or from the fabric pump.
class CommLayer {
public:
    uint32_t node_id, total_partitions;
    CommLayer(uint32_t id = 0, uint32_t total = 1) : node_id(id), total_partitions(total) {}
    void send_residual(ResidualMessage m) { outbox_.push_back(std::move(m)); }
    void inject_message(ResidualMessage m) { inbox_.push_back(std::move(m)); }
    void inject_rollback(RollbackRequest r) { rollbacks_.push_back(r); }
    std::vector<ResidualMessage> drain_outbox() { std::vector<ResidualMessage> v(outbox_.begin(), outbox_.end()); outbox_.clear(); return v; }
    std::vector<ResidualMessage> poll_residuals() { std::vector<ResidualMessage> v(inbox_.begin(), inbox_.end()); inbox_.clear(); return v; }
    bool poll_rollback(RollbackRequest& out) {
        if (rollbacks_.empty()) return false;
        out = rollbacks_.front();
        rollbacks_.pop_front();
        return true;
    }
    ResidualMessage build_residual(uint32_t to, double time, std::vector<std::pair<uint64_t, double>> updates) const {
        ResidualMessage m; m.from = node_id; m.to = to; m.time = time; m.updates = std::move(updates); return m;
    }
    NodeStatus build_status(double time, uint64_t steps, uint64_t hits, uint64_t misses, uint64_t rollbacks) const {
        return {node_id, time, steps, hits, misses, rollbacks};
    }
private:
    std::deque<ResidualMessage> inbox_, outbox_;
    std::deque<RollbackRequest> rollbacks_;
};

struct FabricMessage {
    enum Kind { Residual, Rollback, Done, Shutdown } kind = Shutdown;
    CompressedResidual residual;
    RollbackRequest rollback;
    uint32_t done_partition = 0;
};

struct FabricConfig { size_t channel_capacity = 1024; bool compress = true; int quant_bits = 16; };
struct FabricNodeStats { uint64_t sent = 0, received = 0, dropped = 0, bytes_sent = 0; };

class FabricQueue {
public:
    explicit FabricQueue(size_t cap) : cap_(cap) {}
    bool push(FabricMessage m) {
        std::lock_guard<std::mutex> lk(mu_);
        if (q_.size() >= cap_) return false;
        q_.push_back(std::move(m));
        cv_.notify_one();
        return true;
    }
    bool try_pop(FabricMessage& out) {
        std::lock_guard<std::mutex> lk(mu_);
        if (q_.empty()) return false;
        out = std::move(q_.front());
        q_.pop_front();
        return true;
    }
    bool pop_wait(FabricMessage& out, int timeout_ms) {
        std::unique_lock<std::mutex> lk(mu_);
        if (!cv_.wait_for(lk, std::chrono::milliseconds(timeout_ms), [&] { return !q_.empty(); })) return false;
        out = std::move(q_.front());
        q_.pop_front();
        return true;
    }
private:
    size_t cap_;
    std::mutex mu_;
    std::condition_variable cv_;
    std::deque<FabricMessage> q_;
};

// One endpoint of the mesh: its own inbox plus handles to every peer's inbox.
class FabricNode {
public:
    uint32_t id = 0;
    FabricNodeStats stats;
    ResidualCodec codec;
    FabricNode(uint32_t id_, std::vector<std::shared_ptr<FabricQueue>> all, FabricConfig cfg)
        : id(id_), queues_(std::move(all)), cfg_(cfg) { codec.quant_bits = cfg.quant_bits; }
    uint32_t num_partitions() const { return uint32_t(queues_.size()); }
    bool send_residual(const ResidualMessage& m, const std::vector<std::pair<uint64_t, double>>& predicted) {
        FabricMessage f;
        f.kind = FabricMessage::Residual;
        f.residual = codec.encode(m, cfg_.compress ? predicted : std::vector<std::pair<uint64_t, double>>{});
        return send(m.to, std::move(f), f.residual.deltas.size() * 12 + 32);
    }
    bool send_rollback(uint32_t to, double t) {
        FabricMessage f;
        f.kind = FabricMessage::Rollback;
        f.rollback = {id, t};
        return send(to, std::move(f), 16);
    }
    void broadcast_done() {
        for (uint32_t p = 0; p < queues_.size(); ++p)
            if (p != id) { FabricMessage f; f.kind = FabricMessage::Done; f.done_partition = id; send(p, std::move(f), 4); }
    }
    bool try_recv(FabricMessage& out) {
        if (!queues_[id]->try_pop(out)) return false;
        ++stats.received;
        return true;
    }
    bool recv_wait(FabricMessage& out, int timeout_ms) {
        if (!queues_[id]->pop_wait(out, timeout_ms)) return false;
        ++stats.received;
        return true;
    }
    std::vector<FabricMessage> drain_inbox() {
        std::vector<FabricMessage> v;
        FabricMessage m;
        while (try_recv(m)) v.push_back(std::move(m));
        return v;
    }
    ResidualMessage decode_residual(const CompressedResidual& c) { return codec.decode(c); }
private:
    std::vector<std::shared_ptr<FabricQueue>> queues_;
    FabricConfig cfg_;
    bool send(uint32_t to, FabricMessage f, size_t bytes) {
        if (to >= queues_.size() || to == id) { ++stats.dropped; return false; }
        if (!queues_[to]->push(std::move(f))) { ++stats.dropped; return false; }
        ++stats.sent;
        stats.bytes_sent += bytes;
        return true;
    }
};

inline std::vector<std::unique_ptr<FabricNode>> create_mesh(uint32_t n, FabricConfig cfg = {}) {
    std::vector<std::shared_ptr<FabricQueue>> qs;
    for (uint32_t i = 0; i < n; ++i) qs.push_back(std::make_shared<FabricQueue>(cfg.channel_capacity));
    std::vector<std::unique_ptr<FabricNode>> nodes;
    for (uint32_t i = 0; i < n; ++i) nodes.push_back(std::make_unique<FabricNode>(i, qs, cfg));
    return nodes;
}

// Window of the last 32 prediction outcomes: above 98 % hits and no rollback -> one step deeper;
// under 90 % or any rollback -> one step shallower; a rollback also cuts the depth to 3/4 at once.
class SpeculativeDepthController {
public:
    uint32_t current, min_depth, max_depth;
    SpeculativeDepthController(uint32_t initial, uint32_t mn, uint32_t mx) : current(initial), min_depth(mn), max_depth(mx) {}
    void record_prediction(bool accurate) {
        window_.push_back(accurate);
        if (window_.size() > kWindow) window_.pop_front();
        if (window_.size() >= kWindow / 4) adjust();
    }
    void record_rollback() {
        ++rollbacks_;
        if (current > min_depth) current = std::max(min_depth, current * 3 / 4);
    }
    uint32_t depth() const { return current; }
private:
    static constexpr size_t kWindow = 32;
    std::deque<bool> window_;
    uint32_t rollbacks_ = 0;
    void adjust() {
        size_t hits = size_t(std::count(window_.begin(), window_.end(), true));
        double rate = double(hits) / double(window_.size());
        if (rate > 0.98 && rollbacks_ == 0) current = std::min(max_depth, current + 1);
        else if (rate < 0.90 || rollbacks_ > 0) current = std::max(min_depth, current > 0 ? current - 1 : 0);
        if (window_.size() >= kWindow) rollbacks_ = 0;
    }
};

}  // namespace nspice
