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
#include <cerrno>
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
    // Operator and storage configs may be written as JSON or as YAML (the reference reads its configs with a YAML
    // reader, pico-ps/service/Context.cpp:14-25). The YAML accepted here is the subset such configs use: block
    // mappings and block sequences by indentation (spaces), flow sequences `[a, b]`, scalars (numbers, true / false /
    // yes / no, null / ~, plain and quoted strings) and `#` comments; no anchors, tags or multi-line scalars. A text
    // that starts with `{` or `[` is JSON.
    static bool parse_config(const std::string& text, Json* out, std::string* err = nullptr) {
        size_t p = 0;
        skip_ws(text, p);
        if (p >= text.size()) {
            *out = object();
            return true;
        }
        if (text[p] == '{' || text[p] == '[') return parse(text, out, err);
        try {
            std::vector<YamlLine> lines = yaml_lines(text);
            if (lines.empty()) {
                *out = object();
                return true;
            }
            size_t i = 0;
            *out = yaml_node(lines, i, lines[0].indent, 0);
            if (i != lines.size()) throw std::runtime_error("bad indentation in line " + std::to_string(lines[i].number));
            return true;
        } catch (const std::exception& e) {
            if (err) *err = std::string("YAML: ") + e.what();
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
    // ---- YAML subset ------------------------------------------------------------------------------
    struct YamlLine {
        int indent;
        std::string text;
        int number;
    };
    static std::string trim(const std::string& s) {
        size_t a = 0, b = s.size();
        while (a < b && (s[a] == ' ' || s[a] == '\t' || s[a] == '\r')) ++a;
        while (b > a && (s[b - 1] == ' ' || s[b - 1] == '\t' || s[b - 1] == '\r')) --b;
        return s.substr(a, b - a);
    }
    static std::vector<YamlLine> yaml_lines(const std::string& text) {
        std::vector<YamlLine> out;
        size_t pos = 0;
        int number = 0;
        while (pos <= text.size()) {
            size_t nl = text.find('\n', pos);
            if (nl == std::string::npos) nl = text.size();
            std::string line = text.substr(pos, nl - pos);
            pos = nl + 1;
            ++number;
            // strip a comment: '#' at the start or after a space, outside quotes
            char quote = 0;
            for (size_t k = 0; k < line.size(); ++k) {
                const char c = line[k];
                if (quote) {
                    if (c == quote) quote = 0;
                } else if (c == '"' || c == '\'') {
                    quote = c;
                } else if (c == '#' && (k == 0 || line[k - 1] == ' ' || line[k - 1] == '\t')) {
                    line.resize(k);
                    break;
                }
            }
            int indent = 0;
            while ((size_t)indent < line.size() && line[indent] == ' ') ++indent;
            if ((size_t)indent < line.size() && line[indent] == '\t') throw std::runtime_error("tab in the indentation of line " + std::to_string(number));
            const std::string t = trim(line);
            if (t.empty() || t == "---") continue;
            out.push_back({indent, t, number});
        }
        return out;
    }
    static bool yaml_is_dash(const std::string& t) { return t == "-" || (t.size() > 1 && t[0] == '-' && t[1] == ' '); }
    // position of the ':' that ends a mapping key (followed by a space or the end of the line, outside quotes), or npos
    static size_t yaml_key_end(const std::string& t) {
        char quote = 0;
        for (size_t k = 0; k < t.size(); ++k) {
            const char c = t[k];
            if (quote) {
                if (c == quote) quote = 0;
            } else if (c == '"' || c == '\'') {
                quote = c;
            } else if (c == '[' || c == '{') {
                return std::string::npos;
            } else if (c == ':' && (k + 1 == t.size() || t[k + 1] == ' ')) {
                return k;
            }
        }
        return std::string::npos;
    }
    static Json yaml_scalar(const std::string& raw) {
        const std::string t = trim(raw);
        if (t.empty() || t == "~" || t == "null" || t == "Null" || t == "NULL") return Json();
        if (t.size() >= 2 && ((t.front() == '"' && t.back() == '"') || (t.front() == '\'' && t.back() == '\''))) {
            if (t.front() == '"') {   // the JSON string rules are the double-quoted YAML rules for what configs contain
                Json j;
                if (parse(t, &j)) return j;
            }
            return Json(t.substr(1, t.size() - 2));
        }
        if (t.front() == '[' || t.front() == '{') {
            // flow collection: items separated by commas at depth 1, each a scalar or a nested flow collection
            const bool map = t.front() == '{';
            if (t.back() != (map ? '}' : ']')) throw std::runtime_error("unterminated flow collection: " + t);
            Json out = map ? object() : array();
            std::vector<std::string> items;
            int depth = 0;
            char quote = 0;
            std::string cur;
            for (size_t k = 1; k + 1 < t.size(); ++k) {
                const char c = t[k];
                if (quote) {
                    if (c == quote) quote = 0;
                } else if (c == '"' || c == '\'') {
                    quote = c;
                } else if (c == '[' || c == '{') {
                    ++depth;
                } else if (c == ']' || c == '}') {
                    --depth;
                } else if (c == ',' && depth == 0) {
                    items.push_back(cur);
                    cur.clear();
                    continue;
                }
                cur.push_back(c);
            }
            if (!trim(cur).empty()) items.push_back(cur);
            for (const std::string& it : items) {
                if (!map) {
                    out.push_back(yaml_scalar(it));
                    continue;
                }
                const std::string e = trim(it);
                const size_t ke = yaml_key_end(e + " ");
                if (ke == std::string::npos) throw std::runtime_error("flow mapping entry without a key: " + e);
                out[yaml_scalar(e.substr(0, ke)).scalar_text()] = yaml_scalar(e.substr(ke + 1));
            }
            return out;
        }
        if (t == "true" || t == "True" || t == "yes" || t == "Yes" || t == "on") return Json(true);
        if (t == "false" || t == "False" || t == "no" || t == "No" || t == "off") return Json(false);
        char* end = nullptr;
        errno = 0;
        const long long iv = std::strtoll(t.c_str(), &end, 10);
        if (errno == 0 && end != t.c_str() && *end == 0) return Json((int64_t)iv);
        const double dv = std::strtod(t.c_str(), &end);
        if (end != t.c_str() && *end == 0) return Json(dv);
        return Json(t);
    }
    // text of a scalar used as a mapping key
    std::string scalar_text() const {
        if (type_ == STR) return str_;
        if (type_ == NUL) return "null";
        if (type_ == BOOL) return num_ != 0 ? "true" : "false";
        return dump();
    }
    static Json yaml_node(std::vector<YamlLine>& lines, size_t& i, int indent, int depth) {
        if (depth > kMaxDepth) throw std::runtime_error("nested too deeply");
        if (yaml_is_dash(lines[i].text)) {
            Json arr = array();
            while (i < lines.size() && lines[i].indent == indent && yaml_is_dash(lines[i].text)) {
                const std::string rest = trim(lines[i].text.substr(1));
                if (rest.empty()) {
                    ++i;
                    if (i < lines.size() && lines[i].indent > indent) arr.push_back(yaml_node(lines, i, lines[i].indent, depth + 1));
                    else arr.push_back(Json());
                } else if (yaml_is_dash(rest) || yaml_key_end(rest) != std::string::npos) {
                    // "- key: value" (or "- - item"): a mapping (sequence) whose first entry sits on the dash line, two
                    // columns further in
                    lines[i].indent = indent + 2;
                    lines[i].text = rest;
                    arr.push_back(yaml_node(lines, i, indent + 2, depth + 1));
                } else {
                    arr.push_back(yaml_scalar(rest));
                    ++i;
                }
            }
            return arr;
        }
        Json obj = object();
        while (i < lines.size() && lines[i].indent == indent && !yaml_is_dash(lines[i].text)) {
            const std::string& t = lines[i].text;
            const size_t ke = yaml_key_end(t);
            if (ke == std::string::npos) throw std::runtime_error("expected 'key: value' in line " + std::to_string(lines[i].number));
            const std::string key = yaml_scalar(t.substr(0, ke)).scalar_text();
            const std::string val = trim(t.substr(ke + 1));
            ++i;
            if (!val.empty()) {
                obj[key] = yaml_scalar(val);
            } else if (i < lines.size() && lines[i].indent > indent) {
                obj[key] = yaml_node(lines, i, lines[i].indent, depth + 1);
            } else if (i < lines.size() && lines[i].indent == indent && yaml_is_dash(lines[i].text)) {
                obj[key] = yaml_node(lines, i, indent, depth + 1);   // a sequence may sit at its key's indentation
            } else {
                obj[key] = Json();
            }
        }
        return obj;
    }

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
