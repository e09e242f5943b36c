// Optional whole-block compression of dump files, sync blocks and RPC payloads.
//
// Parity: CompressInfo / initialize_compress_info (pico-ps/common/common.h:10-41,
// pico-ps/common/common.cpp:14-37): the operator config key `compress_algorithm` selects a codec
// ("" = off). The reference offers prpc's snappy / zstd / lz4; this build loads libzstd / liblz4 at run
// time when present (no headers are installed, so the few entry points used are declared here) and
// maps "snappy" to lz4, the closest codec available on this image.
#pragma once
#include <dlfcn.h>

#include <cstdint>
#include <cstring>
#include <string>
#include <vector>

#include "status.h"

namespace psb {

class Compressor {
public:
    static Status create(const std::string& algo, Compressor* out) {
        out->algo_ = algo;
        if (algo.empty() || algo == "none") {
            out->kind_ = 0;
            return Status::Ok();
        }
        if (algo == "zstd") {
            void* h = dlopen("libzstd.so.1", RTLD_NOW | RTLD_GLOBAL);
            if (!h) return Status::InvalidConfig("compress_algorithm zstd: libzstd.so.1 not found");
            out->z_bound_ = (size_t(*)(size_t))dlsym(h, "ZSTD_compressBound");
            out->z_comp_ = (size_t(*)(void*, size_t, const void*, size_t, int))dlsym(h, "ZSTD_compress");
            out->z_decomp_ = (size_t(*)(void*, size_t, const void*, size_t))dlsym(h, "ZSTD_decompress");
            out->z_err_ = (unsigned (*)(size_t))dlsym(h, "ZSTD_isError");
            if (!out->z_bound_ || !out->z_comp_ || !out->z_decomp_ || !out->z_err_)
                return Status::InvalidConfig("libzstd lacks the expected symbols");
            out->kind_ = 1;
            return Status::Ok();
        }
        if (algo == "lz4" || algo == "snappy") {
            void* h = dlopen("liblz4.so.1", RTLD_NOW | RTLD_GLOBAL);
            if (!h) return Status::InvalidConfig("compress_algorithm " + algo + ": liblz4.so.1 not found");
            out->l_bound_ = (int (*)(int))dlsym(h, "LZ4_compressBound");
            out->l_comp_ = (int (*)(const char*, char*, int, int))dlsym(h, "LZ4_compress_default");
            out->l_decomp_ = (int (*)(const char*, char*, int, int))dlsym(h, "LZ4_decompress_safe");
            if (!out->l_bound_ || !out->l_comp_ || !out->l_decomp_)
                return Status::InvalidConfig("liblz4 lacks the expected symbols");
            out->kind_ = 2;
            return Status::Ok();
        }
        return Status::InvalidConfig("unknown compress_algorithm: " + algo);
    }

    bool enabled() const { return kind_ != 0; }
    const std::string& algorithm() const { return algo_; }

    // Block format: u64 raw_size, compressed bytes.
    Status compress(const uint8_t* src, size_t n, std::vector<uint8_t>* out) const {
        if (kind_ == 0) {
            out->assign(src, src + n);
            return Status::Ok();
        }
        uint64_t raw = n;
        if (kind_ == 1) {
            size_t bound = z_bound_(n);
            out->resize(8 + bound);
            size_t c = z_comp_(out->data() + 8, bound, src, n, 3);
            if (z_err_(c)) return Status::Error("zstd compress failed");
            out->resize(8 + c);
        } else {
            int bound = l_bound_((int)n);
            out->resize(8 + (size_t)bound);
            int c = l_comp_((const char*)src, (char*)out->data() + 8, (int)n, bound);
            if (c <= 0 && n > 0) return Status::Error("lz4 compress failed");
            out->resize(8 + (size_t)c);
        }
        std::memcpy(out->data(), &raw, 8);
        return Status::Ok();
    }
    Status decompress(const uint8_t* src, size_t n, std::vector<uint8_t>* out) const {
        if (kind_ == 0) {
            out->assign(src, src + n);
            return Status::Ok();
        }
        if (n < 8) return Status::Error("compressed block too short");
        uint64_t raw;
        std::memcpy(&raw, src, 8);
        // the announced size comes from a file or from the wire: refuse what no compressor could have produced from
        // n bytes before sizing a buffer by it
        if (raw > (1ull << 40) || raw > (uint64_t)(n - 8) * (1u << 20) + (1u << 20) || (kind_ != 1 && raw > 0x7FFFFFFFull))
            return Status::Error("compressed block announces an implausible size");
        try {
            out->resize(raw);
        } catch (const std::exception&) {
            return Status::OOM("cannot allocate the decompressed block");
        }
        if (kind_ == 1) {
            size_t d = z_decomp_(out->data(), raw, src + 8, n - 8);
            if (z_err_(d) || d != raw) return Status::Error("zstd decompress failed");
        } else {
            int d = l_decomp_((const char*)src + 8, (char*)out->data(), (int)(n - 8), (int)raw);
            if (d < 0 || (uint64_t)d != raw) return Status::Error("lz4 decompress failed");
        }
        return Status::Ok();
    }

private:
    std::string algo_;
    int kind_ = 0;
    size_t (*z_bound_)(size_t) = nullptr;
    size_t (*z_comp_)(void*, size_t, const void*, size_t, int) = nullptr;
    size_t (*z_decomp_)(void*, size_t, const void*, size_t) = nullptr;
    unsigned (*z_err_)(size_t) = nullptr;
    int (*l_bound_)(int) = nullptr;
    int (*l_comp_)(const char*, char*, int, int) = nullptr;
    int (*l_decomp_)(const char*, char*, int, int) = nullptr;
};

}  // namespace psb
