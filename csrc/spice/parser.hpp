// SPICE-subset reader: R, C, L, V, I, D, M and X lines, `.subckt` flattening (hierarchical names
// `inst.node`), `.param` (with + - * / expressions in quotes or braces), `.global`, `.model`, `.ic`, DC / PULSE / SIN / EXP / PWL sources, engineering suffixes, `+`
// continuation lines, and the partition directives `.ghost <net> <local node> <owner>` and
// `.nodemap <name> <index>`. MOSFET cards are reduced to Level-1 parameters with process corner,
// supply and temperature scaling applied at parse time.
// Behavioural reference: nangila-spice/nangila-node/src/parser.rs:13-738.
#pragma once
#include <algorithm>
#include <cctype>
#include <fstream>
#include <map>
#include <set>
#include <sstream>
#include <unordered_map>

#include "circuit.hpp"

namespace nspice {

inline std::string lower(std::string s) { for (auto& c : s) c = char(std::tolower((unsigned char)c)); return s; }
inline std::string upper(std::string s) { for (auto& c : s) c = char(std::toupper((unsigned char)c)); return s; }

// "10k" -> 1e4, "2.5meg" -> 2.5e6, "1e-9" -> 1e-9, "10pF" -> 1e-11. Returns false on a non-number.
inline bool parse_scaled(const std::string& raw, double& out) {
    std::string s = lower(raw);
    while (!s.empty() && std::string("(),;'{}").find(s.front()) != std::string::npos) s.erase(s.begin());
    while (!s.empty() && std::string("(),;'{}").find(s.back()) != std::string::npos) s.pop_back();
    if (s.empty()) return false;
    const char* b = s.c_str();
    char* e = nullptr;
    double v = std::strtod(b, &e);
    if (e == b) return false;
    std::string suf(e);
    double mul = 1.0;
    if (suf.rfind("meg", 0) == 0) mul = 1e6;
    else if (suf.rfind("mil", 0) == 0) mul = 25.4e-6;
    else if (!suf.empty()) {
        switch (suf[0]) {
            case 'f': mul = 1e-15; break;
            case 'p': mul = 1e-12; break;
            case 'n': mul = 1e-9; break;
            case 'u': mul = 1e-6; break;
            case 'm': mul = 1e-3; break;
            case 'k': mul = 1e3; break;
            case 'g': mul = 1e9; break;
            case 't': mul = 1e12; break;
            default: mul = 1.0;
        }
    }
    out = v * mul;
    return true;
}

// FNV-1a over the lower-cased name, folded to 53 bits so the id survives JSON readers that keep
// numbers as doubles.
inline uint64_t net_name_hash(const std::string& name) {
    uint64_t h = 1469598103934665603ull;
    for (char c : lower(name)) { h ^= uint64_t((unsigned char)c); h *= 1099511628211ull; }
    return (h ^ (h >> 53)) & ((uint64_t(1) << 53) - 1);
}

struct ModelCard { std::string name, type; std::map<std::string, double> params; };

struct Corner {
    std::string process = "TT";
    double vdd = 1.8, temp_c = 27.0;
};

class SpiceParser {
public:
    std::map<std::string, ModelCard> models;
    mutable std::vector<std::string> warnings;
    double tran_step = 0.0, tran_stop = 0.0;  // `.tran <step> <stop>` of the deck (0 when it has none): defaults for a run

    explicit SpiceParser(Corner c = {}) : corner_(std::move(c)) {
        corner_.process = upper(corner_.process);
        node_map_["0"] = 0;
        node_map_["gnd"] = 0;
    }

    static Netlist parse_file(const std::string& path, const Corner& c = {}) {
        std::ifstream f(path);
        if (!f) throw std::runtime_error("cannot open netlist '" + path + "'");
        std::stringstream ss;
        ss << f.rdbuf();
        std::string name = path;
        size_t slash = name.find_last_of('/');
        if (slash != std::string::npos) name = name.substr(slash + 1);
        SpiceParser p(c);
        p.follow_includes_from(directory_of(path), path);
        return p.parse_text(ss.str(), name);
    }

    // Directory part of a path, with its trailing slash ("" for a bare file name).
    static std::string directory_of(const std::string& path) {
        size_t slash = path.find_last_of('/');
        return slash != std::string::npos ? path.substr(0, slash + 1) : std::string();
    }
    // From now on `parse_text` follows `.include` / `.lib`, resolving relative paths against `dir`.
    void follow_includes_from(const std::string& dir, const std::string& deck_path = std::string()) {
        if (!deck_path.empty()) include_stack_.assign(1, deck_path);  // so that a deck cannot include itself
        base_dir_ = dir;
        if (!base_dir_.empty() && base_dir_.back() != '/') base_dir_ += '/';
        follow_includes_ = true;
    }
    // The deck text with every readable `.include` / `.lib` replaced by what it names.
    static std::string expand(const std::string& text, const std::string& dir, const std::string& deck_path = std::string()) {
        SpiceParser p;
        p.follow_includes_from(dir, deck_path);
        return p.expand_includes(text, p.base_dir_, 0);
    }

    Netlist parse_text(const std::string& raw_text, const std::string& name = "netlist") {
        // `.include` / `.lib` are followed for decks read from a file (paths relative to the deck); text handed over
        // directly has no directory to resolve them against and only gets a warning
        const std::string text = follow_includes_ ? expand_includes(raw_text, base_dir_, 0) : raw_text;
        std::vector<std::string> stmts = statements(text);
        // pass 1: definitions (.subckt bodies, .param, .model), which may follow their first use
        {
            Subckt* cur = nullptr;
            int depth = 0;
            for (auto& st : stmts) {
                auto tok = split(st);
                if (tok.empty()) continue;
                std::string first = upper(tok[0]);
                if (first == ".SUBCKT") {
                    if (depth++ == 0 && tok.size() >= 2) {
                        cur = &subckts_[upper(tok[1])];
                        cur->ports.clear();
                        cur->defaults.clear();
                        for (size_t i = 2; i < tok.size(); ++i) {
                            size_t eq = tok[i].find('=');
                            if (eq != std::string::npos) { cur->defaults.emplace_back(lower(tok[i].substr(0, eq)), tok[i].substr(eq + 1)); continue; }
                            if (upper(tok[i]) == "PARAMS:") continue;
                            if (cur->defaults.empty()) cur->ports.push_back(lower(tok[i]));
                        }
                        continue;
                    }
                } else if (first == ".ENDS") {
                    if (--depth <= 0) { depth = 0; cur = nullptr; continue; }
                }
                if (cur) { cur->lines.push_back(st); continue; }
                if (first == ".GLOBAL") {
                    for (size_t i = 1; i < tok.size(); ++i) globals_.insert(lower(tok[i]));
                } else if (first == ".PARAM") {
                    for (size_t i = 1; i < tok.size(); ++i) {
                        size_t eq = tok[i].find('=');
                        double v;
                        if (eq != std::string::npos && try_value(tok[i].substr(eq + 1), v)) params_[lower(tok[i].substr(0, eq))] = v;  // may use earlier ones
                    }
                } else if (first == ".MODEL" && tok.size() >= 3) {
                    ModelCard mc;
                    mc.name = upper(tok[1]);
                    std::string type = upper(tok[2]);
                    size_t paren = type.find('(');
                    std::vector<std::string> rest(tok.begin() + 3, tok.end());
                    if (paren != std::string::npos) { rest.insert(rest.begin(), tok[2].substr(paren + 1)); type = type.substr(0, paren); }
                    mc.type = type;
                    for (auto& t : rest) {
                        size_t eq = t.find('=');
                        double v;
                        if (eq != std::string::npos && try_value(t.substr(eq + 1), v)) {
                            std::string k = lower(t.substr(0, eq));
                            while (!k.empty() && k.front() == '(') k.erase(k.begin());
                            mc.params[k] = v;
                        }
                    }
                    models[mc.name] = mc;
                }
            }
        }
        // pass 2: top-level elements
        {
            int depth = 0;
            for (auto& st : stmts) {
                auto tok = split(st);
                if (tok.empty()) continue;
                std::string first = upper(tok[0]);
                if (first == ".SUBCKT") { ++depth; continue; }
                if (first == ".ENDS") { if (depth > 0) --depth; continue; }
                if (depth > 0) continue;
                if (first == ".END") break;
                element_line(tok, "", {});
            }
        }
        Netlist nl;
        nl.name = name;
        nl.num_nodes = next_node_ - 1;
        nl.elements = std::move(elements_);
        nl.ghost_map = std::move(ghosts_);
        nl.node_names.assign(size_t(nl.num_nodes), "");
        for (auto& kv : node_map_)
            if (kv.second > 0 && kv.second <= nl.num_nodes) {
                std::string& slot = nl.node_names[size_t(kv.second - 1)];
                if (slot.empty() || kv.first < slot) slot = kv.first;
            }
        for (int i = 0; i < nl.num_nodes; ++i)
            if (nl.node_names[size_t(i)].empty()) nl.node_names[size_t(i)] = "node_" + std::to_string(i + 1);
        for (auto& ic : ic_raw_) {
            auto it = node_map_.find(ic.first);
            if (it != node_map_.end() && it->second > 0) nl.initial_conditions.emplace_back(it->second, ic.second);
            else warnings.push_back(".ic names unknown node '" + ic.first + "'");
        }
        return nl;
    }

private:
    struct Subckt { std::vector<std::string> ports, lines; std::vector<std::pair<std::string, std::string>> defaults; };  // defaults: name, value text
    Corner corner_;
    std::unordered_map<std::string, int> node_map_;
    int next_node_ = 1;
    std::vector<Element> elements_;
    std::map<std::string, Subckt> subckts_;
    std::map<std::string, double> params_;
    std::set<std::string> globals_;  // nets named by `.global`
    int instance_depth_ = 0;
    std::string base_dir_;
    bool follow_includes_ = false;
    size_t included_bytes_ = 0;
    mutable std::vector<std::string> unread_;  // fields already reported as unreadable
    std::vector<std::string> include_stack_;
    std::vector<GhostLink> ghosts_;
    std::vector<std::pair<std::string, double>> ic_raw_;

    // Replaces `.include <file>`, `.lib <file>` (the whole file) and `.lib <file> <section>` (the lines between
    // `.lib <section>` and `.endl` of that file) by the text they name, up to 16 levels deep and 64 MB in total. A file that cannot be
    // read leaves the line in place, which earns the usual warning. The first line (the title) is never a directive.
    std::string expand_includes(const std::string& text, const std::string& dir, int depth) {
        std::istringstream in(text);
        std::string line, out;
        bool first = depth == 0;
        while (std::getline(in, line)) {
            bool title = first;
            first = false;
            size_t b = line.find_first_not_of(" \t");
            if (title || b == std::string::npos || line[b] != '.') { out += line + "\n"; continue; }
            std::istringstream ls(line.substr(b));
            std::string kw, file, section;
            ls >> kw >> file >> section;
            kw = upper(kw);
            if (kw == ".ENDL" || (kw == ".END" && depth > 0)) continue;  // the `.end` of an included file does not end the deck
            if ((kw != ".INCLUDE" && kw != ".INC" && kw != ".LIB") || file.empty()) { out += line + "\n"; continue; }
            auto unquote = [](std::string v) {
                while (!v.empty() && (v.front() == '"' || v.front() == '\'')) v.erase(v.begin());
                while (!v.empty() && (v.back() == '"' || v.back() == '\'')) v.pop_back();
                return v;
            };
            file = unquote(file);
            section = upper(unquote(section));
            std::string path = (!file.empty() && file[0] == '/') ? file : dir + file;
            std::ifstream f(path);
            bool cycle = std::find(include_stack_.begin(), include_stack_.end(), path) != include_stack_.end();
            if (cycle) { warnings.push_back(kw + " of a file that is being included already: " + file); continue; }
            if (!f || depth >= 16 || included_bytes_ > (size_t(64) << 20)) {
                if (kw == ".LIB" && section.empty()) continue;  // `.lib <section>` inside a library: a marker, not a request
                out += line + "\n";
                continue;
            }
            std::stringstream body;
            body << f.rdbuf();
            std::string inner = body.str();
            included_bytes_ += inner.size();
            if (kw == ".LIB" && !section.empty()) {
                std::istringstream lib(inner);
                std::string l, picked;
                bool on = false;
                while (std::getline(lib, l)) {
                    std::istringstream t(l);
                    std::string a, c;
                    t >> a >> c;
                    a = upper(a);
                    if (a == ".LIB" && upper(unquote(c)) == section) { on = true; continue; }
                    if (a == ".ENDL") { on = false; continue; }
                    if (on) picked += l + "\n";
                }
                inner = picked;
            }
            include_stack_.push_back(path);
            out += expand_includes(inner, directory_of(path), depth + 1);
            include_stack_.pop_back();
            if (out.empty() || out.back() != '\n') out += "\n";
        }
        return out;
    }

    // Decks written by tools often start with an element instead of a title. A first line counts as an element when it
    // starts with an element letter and has the shape of that card: a two-terminal element or source has nothing but values
    // (numbers, expressions in quotes or braces, source keywords, `name=value`) after its nodes, a diode four fields, a
    // MOSFET six, a sub-circuit call three, and the model / sub-circuit they name is defined in the deck.
    // "inverter with a 10 fF load" is a title, "I1 0 n1 1m" is not.
    static bool first_line_is_card(char letter, const std::vector<std::string>& tok, const std::string& deck) {
        if (tok.size() < 3 || tok[0].size() < 2 || !std::isalnum((unsigned char)tok[0][1])) return false;
        // whether the deck has a `.model <name>` / `.subckt <name>` card
        auto defines = [&deck](const char* directive, const std::string& name) {
            std::istringstream in(deck);
            std::string line, want = upper(name);
            while (std::getline(in, line)) {
                std::istringstream ls(line);
                std::string a, b;
                ls >> a >> b;
                if (upper(a) == directive && upper(b) == want) return true;
            }
            return false;
        };
        switch (letter) {
            // "Diode bridge rectifier circuit" and "Mixer with two local oscillator inputs" have the field count of a
            // card, so the model or sub-circuit the line would name has to exist in the deck
            case 'D': return tok.size() >= 4 && defines(".MODEL", tok[3]);
            case 'M': return tok.size() >= 6 && defines(".MODEL", tok[5]);
            case 'X': {
                size_t last = tok.size() - 1;
                while (last > 2 && tok[last].find('=') != std::string::npos) --last;
                return defines(".SUBCKT", tok[last]);
            }
            case 'R': case 'C': case 'L': case 'V': case 'I': {
                // everything after the two nodes is a value, a source keyword or a `name=value` parameter
                auto value_like = [](const std::string& t) {
                    size_t d = (t[0] == '+' || t[0] == '-') ? 1 : 0;
                    if (d < t.size() && (std::isdigit((unsigned char)t[d]) || (t[d] == '.' && d + 1 < t.size() && std::isdigit((unsigned char)t[d + 1])))) return true;
                    if (t[0] == '{' || t[0] == '\'' || t.find('=') != std::string::npos) return true;
                    std::string u = upper(t);
                    return u == "DC" || u == "AC" || u == "PULSE" || u == "SIN" || u == "PWL" || u == "EXP";
                };
                if (tok.size() < 4) return false;
                for (size_t i = 3; i < tok.size(); ++i)
                    if (!value_like(tok[i])) return false;
                return true;
            }
            default: return false;
        }
    }

    // Joins `+` continuations, drops comment lines and trailing `;` / `$` comments. The first line of
    // a deck is its title unless it already looks like an element or a directive.
    static std::vector<std::string> statements(const std::string& text) {
        std::vector<std::string> out;
        std::istringstream in(text);
        std::string line;
        bool first_line = true;
        while (std::getline(in, line)) {
            if (!line.empty() && line.back() == '\r') line.pop_back();
            size_t c = line.find_first_of(";$");
            if (c != std::string::npos) line = line.substr(0, c);
            size_t b = line.find_first_not_of(" \t");
            if (b == std::string::npos) { first_line = false; continue; }
            line = line.substr(b);
            if (line[0] == '*') { first_line = false; continue; }
            if (first_line) {
                first_line = false;
                char ch = char(std::toupper((unsigned char)line[0]));
                if (!(ch == '.' || first_line_is_card(ch, split(line), text))) continue;
            }
            if (line[0] == '+') {
                if (!out.empty()) out.back() += " " + line.substr(1);
                continue;
            }
            out.push_back(line);
        }
        return out;
    }
    static std::vector<std::string> split(const std::string& s) {
        // parentheses and commas become separators except that "PULSE(" keeps its name as a token
        // ... and an expression in quotes or braces stays one token, blanks removed: '(w + 1u) / 2' -> '(w+1u)/2'
        std::string t;
        char closing = 0;
        for (char c : s) {
            if (closing) {
                if (c == closing) closing = 0;
                if (!std::isspace((unsigned char)c)) t += c;
                continue;
            }
            if (c == '\'' || c == '{') { closing = c == '{' ? '}' : '\''; t += c; continue; }
            t += (c == '(' || c == ')' || c == ',') ? ' ' : c;
        }
        std::istringstream in(t);
        std::vector<std::string> out;
        std::string w;
        while (in >> w) out.push_back(w);
        // re-join "name = value" and "name= value"
        std::vector<std::string> merged;
        for (size_t i = 0; i < out.size(); ++i) {
            if (out[i] == "=" && !merged.empty() && i + 1 < out.size()) { merged.back() += "=" + out[++i]; continue; }
            if (!out[i].empty() && out[i].back() == '=' && i + 1 < out.size()) { merged.push_back(out[i] + out[i + 1]); ++i; continue; }
            if (!out[i].empty() && out[i].front() == '=' && !merged.empty()) { merged.back() += out[i]; continue; }
            merged.push_back(out[i]);
        }
        return merged;
    }
    // A number with an engineering suffix or the name of a parameter; false for anything else (a keyword, say).
    bool try_value(const std::string& raw, double& out) const {
        std::string s = lower(raw);
        while (!s.empty() && (s.front() == '\'' || s.front() == '{')) s.erase(s.begin());
        while (!s.empty() && (s.back() == '\'' || s.back() == '}')) s.pop_back();
        auto it = params_.find(s);
        if (it != params_.end()) { out = it->second; return true; }
        // arithmetic first where there is an operator: the number reader accepts trailing unit text, and "2*w" would read as 2
        const bool marked = !raw.empty() && (raw.front() == '\'' || raw.front() == '{');
        if (s.find_first_of("*/()^") != std::string::npos || (marked && s.find_first_of("+-", 1) != std::string::npos)) {
            size_t pos = 0;
            double v = 0.0;
            if (expr_sum(s, pos, v, 0) && pos == s.size() && std::isfinite(v)) { out = v; return true; }
            if (marked) return false;
        }
        return parse_scaled(s, out);
    }
    // The value of a field; what cannot be read counts as 0 and is reported once per text.
    double value(const std::string& raw) const {
        double v = 0.0;
        if (try_value(raw, v)) return v;
        if (!raw.empty() && std::find(unread_.begin(), unread_.end(), raw) == unread_.end()) {
            unread_.push_back(raw);
            warnings.push_back("cannot evaluate '" + raw + "': taken as 0");
        }
        return 0.0;
    }
    // Arithmetic in parameter values: + - * / ** (or ^), parentheses and sqrt abs exp ln log log10 pow min max over numbers
    // with engineering suffixes and parameter names, e.g. '(w + 1u) / 2' or 'sqrt(2*kp*i)'. Recursive descent, at most 64
    // levels of nesting.
    bool expr_sum(const std::string& s, size_t& pos, double& out, int depth) const {
        if (!expr_product(s, pos, out, depth)) return false;
        while (pos < s.size() && (s[pos] == '+' || s[pos] == '-')) {
            char op = s[pos++];
            double rhs;
            if (!expr_product(s, pos, rhs, depth)) return false;
            out = op == '+' ? out + rhs : out - rhs;
        }
        return true;
    }
    bool expr_product(const std::string& s, size_t& pos, double& out, int depth) const {
        if (!expr_factor(s, pos, out, depth)) return false;
        while (pos < s.size() && (s[pos] == '*' || s[pos] == '/') && !(s[pos] == '*' && pos + 1 < s.size() && s[pos + 1] == '*')) {
            char op = s[pos++];
            double rhs;
            if (!expr_factor(s, pos, rhs, depth)) return false;
            out = op == '*' ? out * rhs : out / rhs;
            if (!std::isfinite(out)) return false;
        }
        return true;
    }
    // A primary with an optional power: a ** b or a ^ b, right to left, binding tighter than a sign in front of it.
    bool expr_factor(const std::string& s, size_t& pos, double& out, int depth) const {
        if (!expr_primary(s, pos, out, depth)) return false;
        size_t len = pos + 1 < s.size() && s[pos] == '*' && s[pos + 1] == '*' ? 2 : (pos < s.size() && s[pos] == '^' ? 1 : 0);
        if (len) {
            pos += len;
            double e;
            if (depth > 64 || !expr_factor(s, pos, e, depth + 1)) return false;
            out = std::pow(out, e);
            if (!std::isfinite(out)) return false;  // 0 ** -1 and the like: refused here, before a later step hides it
        }
        return true;
    }
    bool expr_primary(const std::string& s, size_t& pos, double& out, int depth) const {
        if (pos >= s.size() || depth > 64) return false;
        if (s[pos] == '-' || s[pos] == '+') {
            bool neg = s[pos++] == '-';
            if (!expr_factor(s, pos, out, depth + 1)) return false;  // -2**2 is -(2**2)
            if (neg) out = -out;
            return true;
        }
        if (s[pos] == '(') {
            ++pos;
            if (!expr_sum(s, pos, out, depth + 1) || pos >= s.size() || s[pos] != ')') return false;
            ++pos;
            return true;
        }
        // a number (its exponent may carry a sign: 1e-9) or a name, up to the next operator
        size_t start = pos;
        while (pos < s.size()) {
            char c = s[pos];
            if (c == '*' || c == '/' || c == '(' || c == ')' || c == ',' || c == '^') break;
            if ((c == '+' || c == '-') && !(pos > start && (s[pos - 1] == 'e') && std::isdigit((unsigned char)s[start]) && pos + 1 < s.size() &&
                                            std::isdigit((unsigned char)s[pos + 1])))
                break;
            ++pos;
        }
        std::string atom = s.substr(start, pos - start);
        if (atom.empty()) return false;
        if (pos < s.size() && s[pos] == '(') {  // a function call: sqrt abs exp ln log log10 pow min max
            ++pos;
            std::vector<double> args;
            for (;;) {
                double a;
                if (!expr_sum(s, pos, a, depth + 1) || pos >= s.size()) return false;
                args.push_back(a);
                if (s[pos] == ',') { ++pos; continue; }
                if (s[pos] == ')') { ++pos; break; }
                return false;
            }
            const size_t n = args.size();
            if (atom == "sqrt" && n == 1) out = std::sqrt(args[0]);
            else if (atom == "abs" && n == 1) out = std::fabs(args[0]);
            else if (atom == "exp" && n == 1) out = std::exp(args[0]);
            else if ((atom == "ln" || atom == "log") && n == 1) out = std::log(args[0]);
            else if (atom == "log10" && n == 1) out = std::log10(args[0]);
            else if ((atom == "pow" || atom == "pwr") && n == 2) out = std::pow(args[0], args[1]);
            else if (atom == "min" && n >= 1) out = *std::min_element(args.begin(), args.end());
            else if (atom == "max" && n >= 1) out = *std::max_element(args.begin(), args.end());
            else return false;
            return std::isfinite(out);
        }
        auto it = params_.find(atom);
        if (it != params_.end()) { out = it->second; return true; }
        return parse_scaled(atom, out);
    }
    int node(const std::string& raw, const std::string& prefix, const std::map<std::string, std::string>& alias) {
        std::string n = lower(raw);
        if (n == "0" || n == "gnd" || n == "gnd!" || n == "vss!") return 0;
        std::string full;
        auto al = alias.find(n);
        if (al != alias.end()) full = al->second;
        else if (prefix.empty() || globals_.count(n)) full = n;  // a `.global` net is the same net inside every sub-circuit
        else full = prefix + "." + n;
        if (full == "0" || full == "gnd") return 0;
        auto it = node_map_.find(full);
        if (it != node_map_.end()) return it->second;
        node_map_[full] = next_node_;
        return next_node_++;
    }
    std::string resolved_name(const std::string& raw, const std::string& prefix, const std::map<std::string, std::string>& alias) const {
        std::string n = lower(raw);
        if (n == "0" || n == "gnd") return "0";
        auto al = alias.find(n);
        if (al != alias.end()) return al->second;
        return prefix.empty() || globals_.count(n) ? n : prefix + "." + n;
    }
    SourceWaveform source(const std::vector<std::string>& tok, size_t from, bool scale_supply) const {
        SourceWaveform w = SourceWaveform::make_dc(0.0);
        size_t i = from;
        bool have = false;
        while (i < tok.size()) {
            std::string u = upper(tok[i]);
            if (u == "DC" && i + 1 < tok.size()) { w = SourceWaveform::make_dc(value(tok[i + 1])); have = true; i += 2; continue; }
            if (u == "PULSE") {
                double p[7] = {0, 0, 0, 0, 0, 0, 0};
                size_t k = 0;
                for (size_t j = i + 1; j < tok.size() && k < 7; ++j, ++k) p[k] = value(tok[j]);
                if (k >= 7) return SourceWaveform::make_pulse(p[0], p[1], p[2], p[3], p[4], p[5], p[6]);
                if (k >= 2) return SourceWaveform::make_pulse(p[0], p[1], p[2], p[3], p[4], k > 5 ? p[5] : 1e30, 0.0);
                return w;
            }
            if (u == "SIN" || u == "EXP" || u == "PWL") {
                std::vector<double> p;
                double x;
                for (size_t j = i + 1; j < tok.size() && try_value(tok[j], x); ++j) p.push_back(x);
                auto arg = [&](size_t k, double dflt) { return k < p.size() ? p[k] : dflt; };
                if (u == "SIN") return SourceWaveform::make_sin(arg(0, 0), arg(1, 0), arg(2, 0), arg(3, 0), arg(4, 0), arg(5, 0));
                if (u == "EXP") {
                    double td1 = arg(2, 0), tau1 = arg(3, 0);
                    return SourceWaveform::make_exp(arg(0, 0), arg(1, 0), td1, tau1, arg(4, td1 + tau1), arg(5, tau1));
                }
                return SourceWaveform::make_pwl(p);
            }
            if (u == "AC") { i += 2; continue; }
            if (!have) { w = SourceWaveform::make_dc(value(tok[i])); have = true; }
            ++i;
        }
        // decks written for a 1.8 V (or 1.0 V) supply follow the requested supply voltage
        if (scale_supply && w.kind == SourceWaveform::Dc && (std::fabs(w.dc - 1.8) < 0.2 || std::fabs(w.dc - 1.0) < 0.2)) w.dc *= corner_.vdd / 1.8;
        return w;
    }
    MosfetLevel1 mos_model(const std::string& model_name, double w, double l) const {
        MosfetLevel1 m;
        m.kind = model_name.find('P') != std::string::npos ? MosType::Pmos : MosType::Nmos;
        double vth = 0.5, u0 = 0.04, tox = 2e-9, lambda = 0.0, kp = -1.0;
        auto it = models.find(model_name);
        if (it != models.end()) {
            if (it->second.type.find("PMOS") != std::string::npos) m.kind = MosType::Pmos;
            else if (it->second.type.find("NMOS") != std::string::npos) m.kind = MosType::Nmos;
            auto& p = it->second.params;
            if (p.count("vto")) vth = p.at("vto");
            if (p.count("kp")) kp = std::fabs(p.at("kp"));
            if (p.count("u0")) u0 = p.at("u0") * 1e-4;
            if (p.count("tox")) tox = p.at("tox");
            if (p.count("lambda")) lambda = std::max(0.0, p.at("lambda"));
        }
        double mob = std::pow(300.15 / (corner_.temp_c + 273.15), 1.5);
        vth -= 0.002 * (corner_.temp_c - 27.0);
        const bool is_n = m.kind == MosType::Nmos;
        double cm = 1.0, dv = 0.0;
        const std::string& pr = corner_.process;
        if (pr == "FF") { cm = 1.15; dv = -0.1; }
        else if (pr == "SS") { cm = 0.85; dv = 0.1; }
        else if (pr == "FS") { cm = is_n ? 1.10 : 0.90; dv = is_n ? -0.1 : 0.1; }
        else if (pr == "SF") { cm = is_n ? 0.90 : 1.10; dv = is_n ? 0.1 : -0.1; }
        mob *= cm;
        // thresholds are stored as magnitudes for both polarities
        m.vth = std::fabs(vth) + dv;
        const double cox = 3.9 * 8.854e-12 / tox;
        m.beta = (kp > 0 ? kp * mob : u0 * mob * cox) * (w / l);
        m.lambda = lambda;
        return m;
    }

    void element_line(const std::vector<std::string>& tok, const std::string& prefix, const std::map<std::string, std::string>& alias) {
        std::string kw = upper(tok[0]);
        char ch = kw[0];
        auto N = [&](size_t i) { return node(tok[i], prefix, alias); };
        switch (ch) {
            case 'R': if (tok.size() >= 4) { double r = value(tok[3]); elements_.push_back(Element::resistor(N(1), N(2), r != 0.0 ? r : 1e-3)); } return;
            case 'C': if (tok.size() >= 4) elements_.push_back(Element::capacitor(N(1), N(2), value(tok[3]))); return;
            case 'L': if (tok.size() >= 4) elements_.push_back(Element::inductor(N(1), N(2), value(tok[3]))); return;
            case 'V': if (tok.size() >= 4) { int p = N(1), n = N(2); elements_.push_back(Element::vsource(p, n, source(tok, 3, true))); } return;
            case 'I': if (tok.size() >= 4) { int p = N(1), n = N(2); elements_.push_back(Element::isource(p, n, source(tok, 3, false))); } return;
            case 'D':
                if (tok.size() >= 4) {
                    DiodeModel dm;
                    auto it = models.find(upper(tok[3]));
                    if (it != models.end()) {
                        if (it->second.params.count("is")) dm.is = it->second.params.at("is");
                        if (it->second.params.count("n")) dm.n = it->second.params.at("n");
                    }
                    dm.vt = 8.617333e-5 * (corner_.temp_c + 273.15);
                    int a = N(1), c = N(2);
                    elements_.push_back(Element::make_diode(a, c, dm));
                }
                return;
            case 'M':
                if (tok.size() >= 6) {
                    int d = N(1), g = N(2), s = N(3), b = N(4);
                    double w = 1e-6, l = 100e-9, mult = 1.0;
                    for (size_t i = 6; i < tok.size(); ++i) {
                        size_t eq = tok[i].find('=');
                        if (eq == std::string::npos) continue;
                        std::string k = lower(tok[i].substr(0, eq));
                        if (k == "w") w = value(tok[i].substr(eq + 1));
                        else if (k == "l") l = value(tok[i].substr(eq + 1));
                        else if (k == "m") mult = value(tok[i].substr(eq + 1));
                    }
                    if (mult > 0.0) w *= mult;  // m devices in parallel are one device of m times the width (current and width-scaled capacitances)
                    elements_.push_back(Element::mosfet(d, g, s, b, mos_model(upper(tok[5]), w, l)));
                    // Constant device capacitances, where the model card gives them (SPICE level-1 names): gate overlap
                    // cgso / cgdo in F per metre of width, zero-bias junction cbd / cbs in F. Their bias dependence and the
                    // channel charge are not modelled.
                    auto mit = models.find(upper(tok[5]));
                    if (mit != models.end()) {
                        auto& mp = mit->second.params;
                        auto cap = [&](const char* key, double scale, int a, int c) {
                            auto f = mp.find(key);
                            if (f != mp.end() && f->second * scale > 0.0 && a != c) elements_.push_back(Element::capacitor(a, c, f->second * scale));
                        };
                        cap("cgso", w, g, s);
                        cap("cgdo", w, g, d);
                        cap("cbd", 1.0, d, b);
                        cap("cbs", 1.0, s, b);
                    }
                }
                return;
            case 'X': {
                if (tok.size() < 3) return;
                size_t last = tok.size() - 1;
                while (last > 1 && tok[last].find('=') != std::string::npos) --last;  // instance parameters
                auto it = subckts_.find(upper(tok[last]));
                if (it == subckts_.end()) { warnings.push_back("unknown subcircuit '" + tok[last] + "'"); return; }
                const Subckt& def = it->second;
                if (def.ports.size() != last - 1) { warnings.push_back("port count mismatch on '" + tok[0] + "'"); return; }
                std::map<std::string, std::string> inner;
                for (size_t i = 0; i < def.ports.size(); ++i) {
                    node(tok[i + 1], prefix, alias);
                    inner[def.ports[i]] = resolved_name(tok[i + 1], prefix, alias);
                }
                std::string np = prefix.empty() ? lower(tok[0]) : prefix + "." + lower(tok[0]);
                // parameters of the instance: the sub-circuit's defaults, then what the X line gives, each evaluated in the
                // caller's scope; they shadow outer parameters of the same name while the body is expanded
                std::vector<std::pair<std::string, double>> scope;
                for (auto& d : def.defaults) { double v; if (try_value(d.second, v)) scope.emplace_back(d.first, v); }
                for (size_t i = last + 1; i < tok.size(); ++i) {
                    size_t eq = tok[i].find('=');
                    double v;
                    if (eq == std::string::npos || !try_value(tok[i].substr(eq + 1), v)) continue;
                    std::string k = lower(tok[i].substr(0, eq));
                    bool found = false;
                    for (auto& kv : scope) if (kv.first == k) { kv.second = v; found = true; }
                    if (!found) scope.emplace_back(k, v);
                }
                std::vector<std::pair<std::string, std::pair<bool, double>>> saved;
                for (auto& kv : scope) {
                    auto old = params_.find(kv.first);
                    saved.push_back({kv.first, {old != params_.end(), old != params_.end() ? old->second : 0.0}});
                    params_[kv.first] = kv.second;
                }
                if (++instance_depth_ <= 64)
                    for (auto& ln : def.lines) {
                        auto t = split(ln);
                        if (!t.empty()) element_line(t, np, inner);
                    }
                else warnings.push_back("sub-circuits nested more than 64 deep at '" + tok[0] + "'");
                --instance_depth_;
                for (auto& sv : saved) {
                    if (sv.second.first) params_[sv.first] = sv.second.second;
                    else params_.erase(sv.first);
                }
                return;
            }
            default: break;
        }
        if (kw == ".IC") {
            for (size_t i = 1; i < tok.size(); ++i) {
                // after splitting, "V(out)=0.5" arrives as "V", "out", "=0.5" or "out=0.5"
                std::string t = tok[i];
                if (upper(t) == "V") continue;
                size_t eq = t.find('=');
                if (eq == std::string::npos || eq == 0) continue;
                ic_raw_.emplace_back(resolved_name(t.substr(0, eq), prefix, alias), value(t.substr(eq + 1)));
            }
        } else if (kw == ".TRAN" && tok.size() >= 3) {
            tran_step = value(tok[1]);
            tran_stop = value(tok[2]);
        } else if (kw == ".GHOST" && tok.size() >= 4) {
            ghosts_.push_back({net_name_hash(tok[1]), std::atoi(tok[2].c_str()), uint32_t(std::atoi(tok[3].c_str()))});
        } else if (kw == ".NODEMAP" && tok.size() >= 3) {
            int idx = std::atoi(tok[2].c_str());
            node_map_[lower(tok[1])] = idx;
            if (idx >= next_node_) next_node_ = idx + 1;
        } else if (kw == ".INCLUDE" || kw == ".LIB") {
            warnings.push_back(kw + " is not followed: " + (tok.size() > 1 ? tok[1] : std::string("?")));
        }
    }
};

}  // namespace nspice
