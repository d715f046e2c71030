// Circuit description of one partition: source waveforms, elements, device models and the netlist
// record with its JSON form.
//
// The JSON layout is the one the reference's partition files use (externally tagged variants:
// {"Resistor": {"a": 1, "b": 2, "r": 1000.0}}, {"Dc": 1.8}; ghost_map entries are
// [net_id, local_node, owner]); reference: nangila-spice/nangila-node/src/mna.rs:30-106 (Element,
// SourceWaveform), ngspice_ffi.rs:35-48 (PartitionNetlist), device_model.rs:24-225 (models).
// Node 0 is ground; node k > 0 is unknown k-1 of the system.
#pragma once
#include <algorithm>
#include <cmath>
#include <limits>
#include <cstdint>
#include <string>
#include <tuple>
#include <vector>

#include "json.hpp"

namespace nspice {

struct SourceWaveform {
    // Dc and Pulse as in the reference (nangila-spice/nangila-node/src/mna.rs, which holds a SIN source at a constant);
    // Sin, Exp and Pwl follow the usual SPICE definitions.
    enum Kind { Dc, Pulse, Sin, Exp, Pwl } kind = Dc;
    double dc = 0.0;
    double v1 = 0, v2 = 0, td = 0, tr = 0, tf = 0, pw = 0, per = 0;
    // Sin: v1 = offset, v2 = amplitude, per = frequency (Hz), td = delay, tr = damping (1/s), tf = phase (degrees)
    // Exp: v1, v2, td = rise delay, tr = rise time constant, tf = fall delay, pw = fall time constant
    std::vector<double> pts;  // Pwl: t0, v0, t1, v1, ... with increasing times

    static SourceWaveform make_dc(double v) { SourceWaveform s; s.kind = Dc; s.dc = v; return s; }
    static SourceWaveform make_pulse(double v1, double v2, double td, double tr, double tf, double pw, double per) {
        SourceWaveform s; s.kind = Pulse; s.v1 = v1; s.v2 = v2; s.td = td; s.tr = tr; s.tf = tf; s.pw = pw; s.per = per;
        return s;
    }
    static SourceWaveform make_sin(double offset, double amplitude, double freq, double delay = 0.0, double damping = 0.0, double phase_deg = 0.0) {
        SourceWaveform s; s.kind = Sin; s.v1 = offset; s.v2 = amplitude; s.per = freq; s.td = delay; s.tr = damping; s.tf = phase_deg;
        return s;
    }
    static SourceWaveform make_exp(double v1, double v2, double td1, double tau1, double td2, double tau2) {
        SourceWaveform s; s.kind = Exp; s.v1 = v1; s.v2 = v2; s.td = td1; s.tr = tau1; s.tf = td2; s.pw = tau2;
        return s;
    }
    // Points whose time does not increase are dropped, so that interpolation never divides by zero.
    static SourceWaveform make_pwl(const std::vector<double>& time_value_pairs) {
        SourceWaveform s; s.kind = Pwl;
        for (size_t i = 0; i + 1 < time_value_pairs.size(); i += 2) {
            double t = time_value_pairs[i], v = time_value_pairs[i + 1];
            if (!std::isfinite(t) || !std::isfinite(v)) continue;
            if (!s.pts.empty() && t <= s.pts[s.pts.size() - 2]) continue;
            s.pts.push_back(t); s.pts.push_back(v);
        }
        if (s.pts.empty()) return make_dc(0.0);
        return s;
    }
    double value_at(double t) const {
        switch (kind) {
            case Dc: return dc;
            case Pulse: {
                if (per <= 0.0 || t < td) return v1;
                double local = std::fmod(t - td, per);
                if (local < tr) return tr <= 0.0 ? v2 : v1 + (v2 - v1) * (local / tr);
                if (local < tr + pw) return v2;
                if (local < tr + pw + tf) return tf <= 0.0 ? v1 : v2 + (v1 - v2) * ((local - tr - pw) / tf);
                return v1;
            }
            case Sin: {
                const double two_pi = 6.283185307179586, ph = tf * (two_pi / 360.0);
                if (t < td) return v1 + v2 * std::sin(ph);
                return v1 + v2 * std::sin(two_pi * per * (t - td) + ph) * std::exp(-(t - td) * tr);
            }
            case Exp: {
                double v = v1;
                if (t > td) v += (v2 - v1) * (1.0 - std::exp(-(t - td) / std::max(tr, 1e-30)));
                if (t > tf) v += (v1 - v2) * (1.0 - std::exp(-(t - tf) / std::max(pw, 1e-30)));
                return v;
            }
            case Pwl: {
                size_t n = pts.size() / 2;
                if (t <= pts[0]) return pts[1];
                if (t >= pts[2 * (n - 1)]) return pts[2 * (n - 1) + 1];
                size_t lo = 0, hi = n - 1;  // pts[2 lo] <= t < pts[2 hi]
                while (hi - lo > 1) {
                    size_t mid = (lo + hi) / 2;
                    (pts[2 * mid] <= t ? lo : hi) = mid;
                }
                double t0 = pts[2 * lo], t1 = pts[2 * hi];
                return pts[2 * lo + 1] + (pts[2 * hi + 1] - pts[2 * lo + 1]) * ((t - t0) / (t1 - t0));
            }
        }
        return dc;
    }
    // The first time strictly after t at which the waveform has a corner (infinity when it has none left); the
    // adaptive transient loop lands a step on it.
    double next_corner_after(double t) const {
        const double inf = std::numeric_limits<double>::infinity();
        switch (kind) {
            case Pulse: {
                if (per <= 0.0) return inf;
                const double offs[4] = {0.0, tr, tr + pw, tr + pw + tf};
                const double eps = 1e-9 * per;
                double base = td + std::floor(std::max(0.0, t - td) / per) * per;
                for (int cyc = 0; cyc < 3; ++cyc)
                    for (double o : offs) {
                        double c = base + cyc * per + o;
                        if (c > t + eps) return c;
                    }
                return inf;
            }
            case Sin: return t < td ? td : inf;
            case Exp: return t < td ? td : (t < tf ? tf : inf);
            case Pwl: {
                for (size_t i = 0; i < pts.size(); i += 2)
                    if (pts[i] > t * (1.0 + 1e-12) + 1e-300) return pts[i];
                return inf;
            }
            default: return inf;
        }
    }
    // Whether a corner lies in (t0, t1].
    bool has_corner_in(double t0, double t1) const { return next_corner_after(t0) <= t1; }
    Json to_json() const {
        Json j = Json::object();
        Json p = Json::object();
        switch (kind) {
            case Dc: j.set("Dc", dc); return j;
            case Pulse:
                p.set("v1", v1).set("v2", v2).set("td", td).set("tr", tr).set("tf", tf).set("pw", pw).set("per", per);
                j.set("Pulse", p);
                return j;
            case Sin:
                p.set("offset", v1).set("amplitude", v2).set("freq", per).set("delay", td).set("damping", tr).set("phase", tf);
                j.set("Sin", p);
                return j;
            case Exp:
                p.set("v1", v1).set("v2", v2).set("td1", td).set("tau1", tr).set("td2", tf).set("tau2", pw);
                j.set("Exp", p);
                return j;
            case Pwl: {
                Json a = Json::array();
                for (double x : pts) a.push(Json(x));
                p.set("points", a);
                j.set("Pwl", p);
                return j;
            }
        }
        return j;
    }
    static SourceWaveform from_json(const Json& j) {
        if (j.is_num()) return make_dc(j.num);
        if (const Json* d = j.find("Dc")) return make_dc(d->as_num());
        if (const Json* q = j.find("Sin"))
            return make_sin(q->number("offset", 0), q->number("amplitude", 0), q->number("freq", 0), q->number("delay", 0),
                            q->number("damping", 0), q->number("phase", 0));
        if (const Json* q = j.find("Exp"))
            return make_exp(q->number("v1", 0), q->number("v2", 0), q->number("td1", 0), q->number("tau1", 0), q->number("td2", 0), q->number("tau2", 0));
        if (const Json* q = j.find("Pwl")) {
            std::vector<double> flat;
            if (const Json* a = q->find("points"))
                for (const Json& x : a->arr) flat.push_back(x.as_num());
            return make_pwl(flat);
        }
        const Json& p = j.at("Pulse");
        return make_pulse(p.number("v1", 0), p.number("v2", 0), p.number("td", 0), p.number("tr", 0),
                          p.number("tf", 0), p.number("pw", 0), p.number("per", 0));
    }
};

struct DiodeModel {
    double is = 1e-14, vt = 0.02585, n = 1.0;
    // Current and conductance at junction voltage vd; the exponent is capped at 40 and the
    // conductance floored at 1e-12 S so the matrix pattern never loses the entry.
    void eval(double vd, double& current, double& g) const {
        double nvt = n * vt;
        double e = std::exp(std::min(vd / nvt, 40.0));
        current = is * (e - 1.0);
        g = std::max(is * e / nvt, 1e-12);
    }
    // Norton companion: i = g * vd + ieq
    void companion(double vd, double& g, double& ieq) const {
        double cur;
        eval(vd, cur, g);
        ieq = cur - g * vd;
    }
};

enum class MosType { Nmos, Pmos };
enum class MosRegion { Cutoff, Linear, Saturation };

struct MosfetLevel1 {
    MosType kind = MosType::Nmos;
    double vth = 0.5, beta = 1e-3, lambda = 0.1;

    // Drain current (into the drain for NMOS) and its derivatives w.r.t. vgs and vds. The device is
    // symmetric: with vds < 0 drain and source trade places, so the current is the forward expression of
    // (vgd, -vds), negated. Channel-length modulation multiplies the linear region too, which keeps the
    // current continuous across the linear / saturation boundary (a jump there makes Newton oscillate
    // whenever the solution sits on the boundary).
    void evaluate(double vgs, double vds, double& id, double& gm, double& gds, MosRegion& region) const {
        const double sign = kind == MosType::Nmos ? 1.0 : -1.0;
        const double vc = sign * vgs, vo = sign * vds;
        double i, fc, fo;
        if (vo >= 0.0) {
            forward(vc, vo, i, fc, fo, region);
            id = sign * i; gm = fc; gds = fo;
        } else {
            forward(vc - vo, -vo, i, fc, fo, region);
            id = -sign * i; gm = -fc; gds = fc + fo;
        }
        gds = std::max(gds, 1e-12);
    }
    // Linearisation around (vgs, vds): id ~ gm*vgs + gds*vds + ieq
    void companion(double vgs, double vds, double& gm, double& gds, double& ieq) const {
        double id;
        MosRegion r;
        evaluate(vgs, vds, id, gm, gds, r);
        ieq = id - gm * vgs - gds * vds;
    }

private:
    // I(vc, vo) for vo >= 0 with its partial derivatives.
    void forward(double vc, double vo, double& i, double& d_vc, double& d_vo, MosRegion& region) const {
        const double vov = vc - std::fabs(vth);
        if (vov <= 0.0) { i = d_vc = d_vo = 0.0; region = MosRegion::Cutoff; return; }
        const double clm = 1.0 + lambda * vo;
        if (vo < vov) {
            const double core = vov * vo - 0.5 * vo * vo;
            i = beta * core * clm;
            d_vc = beta * vo * clm;
            d_vo = beta * ((vov - vo) * clm + core * lambda);
            region = MosRegion::Linear;
        } else {
            i = 0.5 * beta * vov * vov * clm;
            d_vc = beta * vov * clm;
            d_vo = 0.5 * beta * vov * vov * lambda;
            region = MosRegion::Saturation;
        }
    }
};

struct Element {
    enum Kind { Resistor, Capacitor, Inductor, VSource, ISource, Ghost, Diode, Mosfet } kind = Resistor;
    // two-terminal parts use (a, b); sources (a = pos, b = neg); ghost uses a; diode (a = anode,
    // b = cathode); MOSFET uses (d, g, s, bulk)
    int a = 0, b = 0, d = 0, g = 0, s = 0, bulk = 0;
    double value = 0.0;  // ohms / farads / henries / ghost voltage
    SourceWaveform source;
    DiodeModel diode;
    MosfetLevel1 mos;

    static Element resistor(int a, int b, double r) { Element e; e.kind = Resistor; e.a = a; e.b = b; e.value = r; return e; }
    static Element capacitor(int a, int b, double c) { Element e; e.kind = Capacitor; e.a = a; e.b = b; e.value = c; return e; }
    static Element inductor(int a, int b, double l) { Element e; e.kind = Inductor; e.a = a; e.b = b; e.value = l; return e; }
    static Element vsource(int p, int n, SourceWaveform w) { Element e; e.kind = VSource; e.a = p; e.b = n; e.source = w; return e; }
    static Element isource(int p, int n, SourceWaveform w) { Element e; e.kind = ISource; e.a = p; e.b = n; e.source = w; return e; }
    static Element ghost(int node, double v) { Element e; e.kind = Ghost; e.a = node; e.value = v; return e; }
    static Element make_diode(int p, int n, DiodeModel m) { Element e; e.kind = Diode; e.a = p; e.b = n; e.diode = m; return e; }
    static Element mosfet(int d, int g, int s, int b, MosfetLevel1 m) {
        Element e; e.kind = Mosfet; e.d = d; e.g = g; e.s = s; e.bulk = b; e.mos = m; return e;
    }

    Json to_json() const {
        Json body = Json::object(), j = Json::object();
        switch (kind) {
            case Resistor: body.set("a", a).set("b", b).set("r", value); j.set("Resistor", body); break;
            case Capacitor: body.set("a", a).set("b", b).set("c", value); j.set("Capacitor", body); break;
            case Inductor: body.set("a", a).set("b", b).set("l", value); j.set("Inductor", body); break;
            case VSource: body.set("pos", a).set("neg", b).set("source", source.to_json()); j.set("VoltageSource", body); break;
            case ISource: body.set("pos", a).set("neg", b).set("source", source.to_json()); j.set("CurrentSource", body); break;
            case Ghost: body.set("node", a).set("voltage", value); j.set("GhostSource", body); break;
            case Diode: {
                Json m = Json::object();
                m.set("is", diode.is).set("vt", diode.vt).set("n", diode.n).set("node_p", a).set("node_n", b);
                body.set("p", a).set("n", b).set("model", m);
                j.set("Diode", body);
                break;
            }
            case Mosfet: {
                Json m = Json::object();
                m.set("kind", mos.kind == MosType::Nmos ? "Nmos" : "Pmos").set("vth", mos.vth).set("beta", mos.beta)
                    .set("lambda", mos.lambda).set("node_g", g).set("node_d", d).set("node_s", s);
                body.set("d", d).set("g", g).set("s", s).set("b", bulk).set("model", m);
                j.set("Mosfet", body);
                break;
            }
        }
        return j;
    }
    static Element from_json(const Json& j) {
        if (!j.is_obj() || j.obj.size() != 1) throw std::runtime_error("element: expected a single-key object");
        const std::string& tag = j.obj[0].first;
        const Json& o = j.obj[0].second;
        // a node index outside the int range would be undefined behaviour in the cast; Netlist::validate() rejects the
        // -1 this maps it to (and every other index outside the netlist)
        auto I = [&](const char* k) {
            const double v = o.number(k, 0);
            return (v >= 0.0 && v <= 2147483647.0) ? int(v) : -1;
        };
        if (tag == "Resistor") return resistor(I("a"), I("b"), o.number("r", 1.0));
        if (tag == "Capacitor") return capacitor(I("a"), I("b"), o.number("c", 0.0));
        if (tag == "Inductor") return inductor(I("a"), I("b"), o.number("l", 0.0));
        if (tag == "VoltageSource") return vsource(I("pos"), I("neg"), SourceWaveform::from_json(o.at("source")));
        if (tag == "CurrentSource") return isource(I("pos"), I("neg"), SourceWaveform::from_json(o.at("source")));
        if (tag == "GhostSource") return ghost(I("node"), o.number("voltage", 0.0));
        if (tag == "Diode") {
            DiodeModel m;
            if (const Json* mj = o.find("model")) { m.is = mj->number("is", m.is); m.vt = mj->number("vt", m.vt); m.n = mj->number("n", m.n); }
            return make_diode(I("p"), I("n"), m);
        }
        if (tag == "Mosfet") {
            MosfetLevel1 m;
            if (const Json* mj = o.find("model")) {
                if (const Json* k = mj->find("kind")) m.kind = (k->is_str() && k->str == "Pmos") ? MosType::Pmos : MosType::Nmos;
                m.vth = mj->number("vth", m.vth); m.beta = mj->number("beta", m.beta); m.lambda = mj->number("lambda", m.lambda);
            }
            return mosfet(I("d"), I("g"), I("s"), I("b"), m);
        }
        throw std::runtime_error("element: unknown kind '" + tag + "'");
    }
};

struct GhostLink { uint64_t net_id = 0; int local_node = 0; uint32_t owner = 0; };

struct Netlist {
    std::string name;
    int num_nodes = 0;
    std::vector<Element> elements;
    std::vector<GhostLink> ghost_map;
    std::vector<std::string> node_names;
    std::vector<std::pair<int, double>> initial_conditions;

    std::vector<std::string> names_or_default() const {
        if (!node_names.empty()) return node_names;
        std::vector<std::string> out;
        for (int i = 1; i <= num_nodes; ++i) out.push_back("node_" + std::to_string(i));
        return out;
    }
    Json to_json() const {
        Json j = Json::object();
        j.set("name", name).set("num_nodes", num_nodes);
        Json els = Json::array();
        for (auto& e : elements) els.push(e.to_json());
        j.set("elements", els);
        Json gm = Json::array();
        for (auto& g : ghost_map) { Json t = Json::array(); t.push(g.net_id).push(g.local_node).push(uint64_t(g.owner)); gm.push(t); }
        j.set("ghost_map", gm);
        Json nn = Json::array();
        for (auto& n : node_names) nn.push(n);
        j.set("node_names", nn);
        Json ic = Json::array();
        for (auto& p : initial_conditions) { Json t = Json::array(); t.push(p.first).push(p.second); ic.push(t); }
        j.set("initial_conditions", ic);
        return j;
    }
    static Netlist from_json(const Json& j) {
        Netlist n;
        if (const Json* p = j.find("name")) n.name = p->is_str() ? p->str : "";
        {
            const double nodes = j.number("num_nodes", 0);
            if (!(nodes >= 0.0 && nodes <= 100000000.0)) throw std::runtime_error("netlist: num_nodes out of range");
            n.num_nodes = int(nodes);
        }
        for (auto& e : j.at("elements").arr) n.elements.push_back(Element::from_json(e));
        if (const Json* gm = j.find("ghost_map"))
            for (auto& t : gm->arr)
                if (t.arr.size() >= 3) {
                    const double id = t.arr[0].as_num(), node = t.arr[1].as_num(), owner = t.arr[2].as_num();
                    if (!(id >= 0.0 && id < 18446744073709551616.0) || !(node >= 0.0 && node <= 2147483647.0) || !(owner >= 0.0 && owner <= 4294967295.0))
                        throw std::runtime_error("netlist: ghost link with a number out of range");
                    n.ghost_map.push_back({uint64_t(id), int(node), uint32_t(owner)});
                }
        if (const Json* nn = j.find("node_names"))
            for (auto& s : nn->arr) n.node_names.push_back(s.as_str());
        if (const Json* ic = j.find("initial_conditions"))
            for (auto& t : ic->arr)
                if (t.arr.size() >= 2) {
                    const double node = t.arr[0].as_num();
                    n.initial_conditions.emplace_back((node >= 0.0 && node <= 2147483647.0) ? int(node) : -1, t.arr[1].as_num());
                }
        n.validate();
        return n;
    }
    // Throws when an element, a ghost link or an initial condition names a node outside 0 .. num_nodes, or a part has a
    // value no solver can use. Files come from the partitioner, but also from users and over the network.
    void validate() const {
        auto bad = [&](int node) { return node < 0 || node > num_nodes; };
        if (num_nodes < 0 || num_nodes > 100000000) throw std::runtime_error("netlist: num_nodes out of range");
        for (size_t k = 0; k < elements.size(); ++k) {
            const Element& e = elements[k];
            const bool mos = e.kind == Element::Mosfet;
            if (mos ? (bad(e.d) || bad(e.g) || bad(e.s) || bad(e.bulk)) : (bad(e.a) || (e.kind != Element::Ghost && bad(e.b))))
                throw std::runtime_error("netlist: element " + std::to_string(k) + " names a node outside 0.." + std::to_string(num_nodes));
            if ((e.kind == Element::Resistor && !(std::fabs(e.value) > 0.0)) || !std::isfinite(e.value))
                throw std::runtime_error("netlist: element " + std::to_string(k) + " has an unusable value");
        }
        for (auto& g : ghost_map)
            if (g.local_node <= 0 || g.local_node > num_nodes) throw std::runtime_error("netlist: ghost link names a node outside 1.." + std::to_string(num_nodes));
        for (auto& ic : initial_conditions)
            if (ic.first <= 0 || ic.first > num_nodes || !std::isfinite(ic.second)) throw std::runtime_error("netlist: initial condition on a node outside 1.." + std::to_string(num_nodes));
        if (!node_names.empty() && node_names.size() < size_t(num_nodes)) throw std::runtime_error("netlist: fewer node names than nodes");
    }
};

}  // namespace nspice
