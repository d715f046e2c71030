// Minimal JSON value (parse + serialise) for the circuit simulator: partition files, waveform files,
// codec payloads. Numbers are doubles (integers up to 2^53 survive), objects keep insertion order.
#pragma once
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace nspice {

class Json {
public:
    enum Kind { Null, Bool, Num, Str, Arr, Obj };
    Kind kind = Null;
    bool b = false;
    double num = 0.0;
    std::string str;
    std::vector<Json> arr;
    std::vector<std::pair<std::string, Json>> obj;

    Json() = default;
    Json(bool v) : kind(Bool), b(v) {}
    Json(double v) : kind(Num), num(v) {}
    Json(int v) : kind(Num), num(v) {}
    Json(int64_t v) : kind(Num), num(double(v)) {}
    Json(uint64_t v) : kind(Num), num(double(v)) {}
    Json(const char* s) : kind(Str), str(s) {}
    Json(std::string s) : kind(Str), str(std::move(s)) {}
    static Json array() { Json j; j.kind = Arr; return j; }
    static Json object() { Json j; j.kind = Obj; return j; }

    bool is_null() const { return kind == Null; }
    bool is_obj() const { return kind == Obj; }
    bool is_arr() const { return kind == Arr; }
    bool is_num() const { return kind == Num; }
    bool is_str() const { return kind == Str; }

    Json& push(Json v) { kind = Arr; arr.push_back(std::move(v)); return *this; }
    Json& set(const std::string& k, Json v) {
        kind = Obj;
        for (auto& kv : obj) if (kv.first == k) { kv.second = std::move(v); return *this; }
        obj.emplace_back(k, std::move(v));
        return *this;
    }
    const Json* find(const std::string& k) const {
        if (kind != Obj) return nullptr;
        for (auto& kv : obj) if (kv.first == k) return &kv.second;
        return nullptr;
    }
    const Json& at(const std::string& k) const {
        const Json* p = find(k);
        if (!p) throw std::runtime_error("json: missing key '" + k + "'");
        return *p;
    }
    double number(const std::string& k, double dflt) const {
        const Json* p = find(k);
        return (p && p->kind == Num) ? p->num : dflt;
    }
    double as_num() const {
        if (kind != Num) throw std::runtime_error("json: expected a number");
        return num;
    }
    const std::string& as_str() const {
        if (kind != Str) throw std::runtime_error("json: expected a string");
        return str;
    }

    static Json parse(const std::string& text) {
        size_t i = 0;
        Json v = parse_value(text, i);
        skip_ws(text, i);
        if (i != text.size()) throw std::runtime_error("json: trailing characters");
        return v;
    }

    std::string dump(int indent = -1) const {
        std::string out;
        write(out, indent, 0);
        return out;
    }

private:
    static void skip_ws(const std::string& s, size_t& i) {
        while (i < s.size() && (s[i] == ' ' || s[i] == '\n' || s[i] == '\t' || s[i] == '\r')) ++i;
    }
    static Json parse_value(const std::string& s, size_t& i) {
        skip_ws(s, i);
        if (i >= s.size()) throw std::runtime_error("json: unexpected end");
        char c = s[i];
        if (c == '{') {
            Json j = object();
            ++i;
            skip_ws(s, i);
            if (i < s.size() && s[i] == '}') { ++i; return j; }
            while (true) {
                skip_ws(s, i);
                std::string key = parse_string(s, i);
                skip_ws(s, i);
                if (i >= s.size() || s[i] != ':') throw std::runtime_error("json: expected ':'");
                ++i;
                j.obj.emplace_back(std::move(key), parse_value(s, i));
                skip_ws(s, i);
                if (i < s.size() && s[i] == ',') { ++i; continue; }
                if (i < s.size() && s[i] == '}') { ++i; return j; }
                throw std::runtime_error("json: expected ',' or '}'");
            }
        }
        if (c == '[') {
            Json j = array();
            ++i;
            skip_ws(s, i);
            if (i < s.size() && s[i] == ']') { ++i; return j; }
            while (true) {
                j.arr.push_back(parse_value(s, i));
                skip_ws(s, i);
                if (i < s.size() && s[i] == ',') { ++i; continue; }
                if (i < s.size() && s[i] == ']') { ++i; return j; }
                throw std::runtime_error("json: expected ',' or ']'");
            }
        }
        if (c == '"') return Json(parse_string(s, i));
        if (s.compare(i, 4, "true") == 0) { i += 4; return Json(true); }
        if (s.compare(i, 5, "false") == 0) { i += 5; return Json(false); }
        if (s.compare(i, 4, "null") == 0) { i += 4; return Json(); }
        const char* start = s.c_str() + i;
        char* end = nullptr;
        double v = std::strtod(start, &end);
        if (end == start) throw std::runtime_error("json: bad token");
        i += size_t(end - start);
        return Json(v);
    }
    static std::string parse_string(const std::string& s, size_t& i) {
        if (i >= s.size() || s[i] != '"') throw std::runtime_error("json: expected string");
        ++i;
        std::string out;
        while (i < s.size() && s[i] != '"') {
            char c = s[i++];
            if (c == '\\' && i < s.size()) {
                char e = s[i++];
                switch (e) {
                    case 'n': out += '\n'; break;
                    case 't': out += '\t'; break;
                    case 'r': out += '\r'; break;
                    case 'b': out += '\b'; break;
                    case 'f': out += '\f'; break;
                    case 'u': {
                        unsigned cp = unsigned(std::strtoul(s.substr(i, 4).c_str(), nullptr, 16));
                        i += 4;
                        if (cp < 0x80) out += char(cp);
                        else if (cp < 0x800) { out += char(0xC0 | (cp >> 6)); out += char(0x80 | (cp & 0x3F)); }
                        else { out += char(0xE0 | (cp >> 12)); out += char(0x80 | ((cp >> 6) & 0x3F)); out += char(0x80 | (cp & 0x3F)); }
                        break;
                    }
                    default: out += e;
                }
            } else {
                out += c;
            }
        }
        if (i >= s.size()) throw std::runtime_error("json: unterminated string");
        ++i;
        return out;
    }
    static void write_str(std::string& out, const std::string& s) {
        out += '"';
        for (char c : s) {
            switch (c) {
                case '"': out += "\\\""; break;
                case '\\': out += "\\\\"; break;
                case '\n': out += "\\n"; break;
                case '\t': out += "\\t"; break;
                case '\r': out += "\\r"; break;
                default:
                    if ((unsigned char)c < 0x20) { char buf[8]; std::snprintf(buf, sizeof buf, "\\u%04x", c); out += buf; }
                    else out += c;
            }
        }
        out += '"';
    }
    void write(std::string& out, int indent, int depth) const {
        auto nl = [&](int d) {
            if (indent >= 0) { out += '\n'; out.append(size_t(indent * d), ' '); }
        };
        switch (kind) {
            case Null: out += "null"; break;
            case Bool: out += b ? "true" : "false"; break;
            case Num: {
                if (!std::isfinite(num)) { out += "null"; break; }
                char buf[40];
                if (num == std::floor(num) && std::fabs(num) < 9.0e15) std::snprintf(buf, sizeof buf, "%.0f", num);
                else std::snprintf(buf, sizeof buf, "%.17g", num);
                out += buf;
                break;
            }
            case Str: write_str(out, str); break;
            case Arr:
                out += '[';
                for (size_t k = 0; k < arr.size(); ++k) {
                    if (k) out += ',';
                    nl(depth + 1);
                    arr[k].write(out, indent, depth + 1);
                }
                if (!arr.empty()) nl(depth);
                out += ']';
                break;
            case Obj:
                out += '{';
                for (size_t k = 0; k < obj.size(); ++k) {
                    if (k) out += ',';
                    nl(depth + 1);
                    write_str(out, obj[k].first);
                    out += indent >= 0 ? ": " : ":";
                    obj[k].second.write(out, indent, depth + 1);
                }
                if (!obj.empty()) nl(depth);
                out += '}';
                break;
        }
    }
};

}  // namespace nspice
