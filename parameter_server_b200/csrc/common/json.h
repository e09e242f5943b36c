// Minimal JSON value (object / array / string / number / bool / null) with parse and dump.
//
// Parity: plays the role of prpc's PicoJsonNode (context blobs published to the master,
// pico-ps/service/TableDescriptor.cpp:132-157; model objects, pico-ps/model/Model.cpp:28-44) and of
// its YAML Configure for operator configs (pico-ps/service/Context.cpp:14-25): configs here are JSON,
// which every YAML parser also reads.
#pragma once
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <memory>
#include <sstream>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace psb {

class Json {
public:
    enum Type { NUL, BOOL, NUM, STR, ARR, OBJ };

    Json() : type_(NUL) {}
    Json(std::nullptr_t) : type_(NUL) {}
    Json(bool b) : type_(BOOL), num_(b ? 1 : 0) {}
    Json(int v) : type_(NUM), num_(v), is_int_(true) {}
    Json(int64_t v) : type_(NUM), num_((double)v), int_(v), is_int_(true) { }
    Json(uint64_t v) : type_(NUM), num_((double)v), int_((int64_t)v), is_int_(true) {}
    Json(double v) : type_(NUM), num_(v) {}
    Json(const char* s) : type_(STR), str_(s) {}
    Json(std::string s) : type_(STR), str_(std::move(s)) {}

    static Json array() { Json j; j.type_ = ARR; return j; }
    static Json object() { Json j; j.type_ = OBJ; return j; }

    Type type() const { return type_; }
    bool is_null() const { return type_ == NUL; }
    bool is_object() const { return type_ == OBJ; }
    bool is_array() const { return type_ == ARR; }
    bool is_string() const { return type_ == STR; }
    bool is_number() const { return type_ == NUM; }

    bool as_bool(bool d = false) const { return type_ == BOOL || type_ == NUM ? num_ != 0 : d; }
    int64_t as_int(int64_t d = 0) const {
        if (type_ == NUM) return is_int_ && int_ != 0 ? int_ : (int64_t)num_;
        if (type_ == BOOL) return (int64_t)num_;
        if (type_ == STR) return std::strtoll(str_.c_str(), nullptr, 10);
        return d;
    }
    double as_double(double d = 0) const {
        if (type_ == NUM || type_ == BOOL) return num_;
        if (type_ == STR) return std::strtod(str_.c_str(), nullptr);
        return d;
    }
    const std::string& as_string() const {
        static const std::string empty;
        return type_ == STR ? str_ : empty;
    }

    // object access
    bool has(const std::string& k) const { return type_ == OBJ && obj_.count(k); }
    Json& operator[](const std::string& k) {
        if (type_ == NUL) type_ = OBJ;
        if (type_ != OBJ) throw std::runtime_error("Json: not an object");
        return obj_[k];
    }
    const Json& at(const std::string& k) const {
        static const Json null_json;
        if (type_ != OBJ) return null_json;
        auto it = obj_.find(k);
        return it == obj_.end() ? null_json : it->second;
    }
    const std::map<std::string, Json>& items() const { return obj_; }
    void erase(const std::string& k) { obj_.erase(k); }

    // array access
    void push_back(Json v) {
        if (type_ == NUL) type_ = ARR;
        if (type_ != ARR) throw std::runtime_error("Json: not an array");
        arr_.push_back(std::move(v));
    }
    size_t size() const { return type_ == ARR ? arr_.size() : type_ == OBJ ? obj_.size() : 0; }
    const Json& at(size_t i) const { return arr_.at(i); }
    Json& at(size_t i) { return arr_.at(i); }
    const std::vector<Json>& elements() const { return arr_; }

    // ---------------------------------------------------------------------------------------
    std::string dump() const {
        std::string out;
        dump_to(out);
        return out;
    }

    static bool parse(const std::string& text, Json* out, std::string* err = nullptr) {
        size_t pos = 0;
        try {
            *out = parse_value(text, pos);
            skip_ws(text, pos);
            if (pos != text.size()) throw std::runtime_error("trailing characters");
            return true;
        } catch (const std::exception& e) {
            if (err) *err = std::string(e.what()) + " at offset " + std::to_string(pos);
            return false;
        }
    }
    static Json parse_or_throw(const std::string& text) {
        Json j;
        std::string err;
        if (!parse(text, &j, &err)) throw std::runtime_error("Json parse error: " + err);
        return j;
    }

private:
    static void skip_ws(const std::string& s, size_t& p) {
        while (p < s.size() && (s[p] == ' ' || s[p] == '\n' || s[p] == '\t' || s[p] == '\r')) ++p;
    }
    // Nesting is bounded: configs and contexts are a few levels deep, and a recursive parser must not be walked off
    // the stack by a hostile or damaged input.
    static constexpr int kMaxDepth = 128;
    static Json parse_value(const std::string& s, size_t& p, int depth = 0) {
        if (depth > kMaxDepth) throw std::runtime_error("nested too deeply");
        skip_ws(s, p);
        if (p >= s.size()) throw std::runtime_error("unexpected end");
        char c = s[p];
        if (c == '{') {
            Json j = object();
            ++p;
            skip_ws(s, p);
            if (p < s.size() && s[p] == '}') { ++p; return j; }
            for (;;) {
                skip_ws(s, p);
                std::string k = parse_string(s, p);
                skip_ws(s, p);
                if (p >= s.size() || s[p] != ':') throw std::runtime_error("expected ':'");
                ++p;
                j.obj_[k] = parse_value(s, p, depth + 1);
                skip_ws(s, p);
                if (p < s.size() && s[p] == ',') { ++p; continue; }
                if (p < s.size() && s[p] == '}') { ++p; return j; }
                throw std::runtime_error("expected ',' or '}'");
            }
        }
        if (c == '[') {
            Json j = array();
            ++p;
            skip_ws(s, p);
            if (p < s.size() && s[p] == ']') { ++p; return j; }
            for (;;) {
                j.arr_.push_back(parse_value(s, p, depth + 1));
                skip_ws(s, p);
                if (p < s.size() && s[p] == ',') { ++p; continue; }
                if (p < s.size() && s[p] == ']') { ++p; return j; }
                throw std::runtime_error("expected ',' or ']'");
            }
        }
        if (c == '"') return Json(parse_string(s, p));
        if (s.compare(p, 4, "true") == 0) { p += 4; return Json(true); }
        if (s.compare(p, 5, "false") == 0) { p += 5; return Json(false); }
        if (s.compare(p, 4, "null") == 0) { p += 4; return Json(); }
        // number
        size_t start = p;
        bool is_float = false;
        if (s[p] == '-' || s[p] == '+') ++p;
        while (p < s.size() && (isdigit((unsigned char)s[p]) || s[p] == '.' || s[p] == 'e' || s[p] == 'E' || s[p] == '-' || s[p] == '+')) {
            if (s[p] == '.' || s[p] == 'e' || s[p] == 'E') is_float = true;
            ++p;
        }
        if (p == start) throw std::runtime_error("unexpected character");
        std::string tok = s.substr(start, p - start);
        if (is_float) return Json(std::strtod(tok.c_str(), nullptr));
        return Json((int64_t)std::strtoll(tok.c_str(), nullptr, 10));
    }
    static std::string parse_string(const std::string& s, size_t& p) {
        if (p >= s.size() || s[p] != '"') throw std::runtime_error("expected string");
        ++p;
        std::string out;
        while (p < s.size() && s[p] != '"') {
            if (s[p] == '\\' && p + 1 < s.size()) {
                ++p;
                switch (s[p]) {
                    case 'n': out += '\n'; break;
                    case 't': out += '\t'; break;
                    case 'r': out += '\r'; break;
                    case 'b': out += '\b'; break;
                    case 'f': out += '\f'; break;
                    case 'u': {
                        if (p + 4 >= s.size()) throw std::runtime_error("bad \\u escape");
                        unsigned code = (unsigned)std::strtoul(s.substr(p + 1, 4).c_str(), nullptr, 16);
                        p += 4;
                        if (code < 0x80) out += (char)code;
                        else if (code < 0x800) { out += (char)(0xC0 | (code >> 6)); out += (char)(0x80 | (code & 0x3F)); }
                        else { out += (char)(0xE0 | (code >> 12)); out += (char)(0x80 | ((code >> 6) & 0x3F)); out += (char)(0x80 | (code & 0x3F)); }
                        break;
                    }
                    default: out += s[p];
                }
                ++p;
            } else {
                out += s[p++];
            }
        }
        if (p >= s.size()) throw std::runtime_error("unterminated string");
        ++p;
        return out;
    }
    static void dump_string(const std::string& s, std::string& out) {
        out += '"';
        for (unsigned char c : s) {
            switch (c) {
                case '"': out += "\\\""; break;
                case '\\': out += "\\\\"; break;
                case '\n': out += "\\n"; break;
                case '\t': out += "\\t"; break;
                case '\r': out += "\\r"; break;
                default:
                    if (c < 0x20) { char buf[8]; std::snprintf(buf, sizeof buf, "\\u%04x", c); out += buf; }
                    else out += (char)c;
            }
        }
        out += '"';
    }
    void dump_to(std::string& out) const {
        switch (type_) {
            case NUL: out += "null"; break;
            case BOOL: out += num_ != 0 ? "true" : "false"; break;
            case NUM: {
                char buf[40];
                if (is_int_) std::snprintf(buf, sizeof buf, "%lld", (long long)(int_ != 0 ? int_ : (int64_t)num_));
                else std::snprintf(buf, sizeof buf, "%.17g", num_);
                out += buf;
                break;
            }
            case STR: dump_string(str_, out); break;
            case ARR: {
                out += '[';
                for (size_t i = 0; i < arr_.size(); ++i) {
                    if (i) out += ',';
                    arr_[i].dump_to(out);
                }
                out += ']';
                break;
            }
            case OBJ: {
                out += '{';
                bool first = true;
                for (auto& kv : obj_) {
                    if (!first) out += ',';
                    first = false;
                    dump_string(kv.first, out);
                    out += ':';
                    kv.second.dump_to(out);
                }
                out += '}';
                break;
            }
        }
    }

    Type type_;
    double num_ = 0;
    int64_t int_ = 0;
    bool is_int_ = false;
    std::string str_;
    std::vector<Json> arr_;
    std::map<std::string, Json> obj_;
};

}  // namespace psb
