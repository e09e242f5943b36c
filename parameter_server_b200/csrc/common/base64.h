// Binary values inside configs: a blob is compressed, base64-encoded and stored as a string value of the config
// tree, and read back the same way (add_base64_config / get_base64_config of the reference,
// pico-ps/common/common.h:22-41, which uses snappy + base64 inside YAML; here the fast codec the image has - lz4 -
// inside JSON). byte2str prints bytes as hex (pico-ps/common/common.cpp:31-37).
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "compress.h"
#include "json.h"
#include "status.h"

namespace psb {

inline std::string base64_encode(const uint8_t* data, size_t n) {
    static const char* tab = "ABCDEFGHIJKLMNOPQRSTUVWXYZabcdefghijklmnopqrstuvwxyz0123456789+/";
    std::string out;
    out.reserve((n + 2) / 3 * 4);
    for (size_t i = 0; i < n; i += 3) {
        const uint32_t b0 = data[i], b1 = i + 1 < n ? data[i + 1] : 0, b2 = i + 2 < n ? data[i + 2] : 0;
        const uint32_t v = (b0 << 16) | (b1 << 8) | b2;
        out += tab[(v >> 18) & 63];
        out += tab[(v >> 12) & 63];
        out += i + 1 < n ? tab[(v >> 6) & 63] : '=';
        out += i + 2 < n ? tab[v & 63] : '=';
    }
    return out;
}

// False when the text is not valid base64 (length, alphabet, padding).
inline bool base64_decode(const std::string& text, std::vector<uint8_t>* out) {
    out->clear();
    if (text.size() % 4) return false;
    auto val = [](char c) -> int {
        if (c >= 'A' && c <= 'Z') return c - 'A';
        if (c >= 'a' && c <= 'z') return c - 'a' + 26;
        if (c >= '0' && c <= '9') return c - '0' + 52;
        if (c == '+') return 62;
        if (c == '/') return 63;
        return -1;
    };
    for (size_t i = 0; i < text.size(); i += 4) {
        int v[4];
        int pad = 0;
        for (int k = 0; k < 4; ++k) {
            const char c = text[i + k];
            if (c == '=') {
                if (i + 4 != text.size() || k < 2) return false;   // padding only at the very end, at most two
                v[k] = 0;
                ++pad;
            } else {
                if (pad) return false;                              // data after padding
                v[k] = val(c);
                if (v[k] < 0) return false;
            }
        }
        const uint32_t w = ((uint32_t)v[0] << 18) | ((uint32_t)v[1] << 12) | ((uint32_t)v[2] << 6) | (uint32_t)v[3];
        out->push_back((uint8_t)(w >> 16));
        if (pad < 2) out->push_back((uint8_t)(w >> 8));
        if (pad < 1) out->push_back((uint8_t)w);
    }
    return true;
}

inline Status add_base64_config(Json& conf, const std::string& key, const uint8_t* data, size_t n) {
    Compressor c;
    PSB_RETURN_IF_ERROR(Compressor::create("lz4", &c));
    std::vector<uint8_t> packed;
    PSB_RETURN_IF_ERROR(c.compress(data, n, &packed));
    conf[key] = Json(base64_encode(packed.data(), packed.size()));
    return Status::Ok();
}

inline Status get_base64_config(const Json& conf, const std::string& key, std::vector<uint8_t>* out) {
    if (!conf.has(key) || !conf.at(key).is_string()) return Status::InvalidConfig("no base64 value under \"" + key + "\"");
    std::vector<uint8_t> packed;
    if (!base64_decode(conf.at(key).as_string(), &packed)) return Status::InvalidConfig("\"" + key + "\" is not base64");
    Compressor c;
    PSB_RETURN_IF_ERROR(Compressor::create("lz4", &c));
    return c.decompress(packed.data(), packed.size(), out);
}

inline std::string byte2str(const uint8_t* data, size_t n) {
    static const char* hex = "0123456789abcdef";
    std::string out;
    out.reserve(n * 2);
    for (size_t i = 0; i < n; ++i) {
        out += hex[data[i] >> 4];
        out += hex[data[i] & 15];
    }
    return out;
}

}  // namespace psb
