// Byte archive used for control-plane messages, dump records and context blobs.
//
// Parity: plays the role of prpc's BinaryArchive as used through pico-ps/common/message.h:165-236
// (trivially copyable values are raw memcpy, pairs likewise; strings and vectors carry a 64-bit
// length; the message meta is appended at the tail and popped with read_back). The prpc source is
// not part of the reference tree, so the layout below is this build's own and is documented here:
//   scalar / POD          : sizeof(T) raw little-endian bytes
//   std::string           : u64 length, bytes
//   std::vector<POD>      : u64 count, count*sizeof(T) raw bytes
//   std::vector<string>   : u64 count, then each string
#pragma once
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>
#include <type_traits>
#include <utility>
#include <vector>

namespace psb {

class Archive {
public:
    Archive() = default;
    explicit Archive(std::vector<uint8_t> bytes) : buf_(std::move(bytes)) {}
    Archive(const void* p, size_t n) : buf_((const uint8_t*)p, (const uint8_t*)p + n) {}

    // --- writing -------------------------------------------------------------------------
    void write_raw(const void* p, size_t n) {
        const uint8_t* b = (const uint8_t*)p;
        buf_.insert(buf_.end(), b, b + n);
    }
    template <class T>
    typename std::enable_if<std::is_trivially_copyable<T>::value, Archive&>::type operator<<(const T& v) {
        write_raw(&v, sizeof(T));
        return *this;
    }
    Archive& operator<<(const std::string& s) {
        uint64_t n = s.size();
        write_raw(&n, 8);
        write_raw(s.data(), s.size());
        return *this;
    }
    template <class T>
    typename std::enable_if<std::is_trivially_copyable<T>::value, Archive&>::type operator<<(
        const std::vector<T>& v) {
        uint64_t n = v.size();
        write_raw(&n, 8);
        if (n) write_raw(v.data(), n * sizeof(T));
        return *this;
    }
    Archive& operator<<(const std::vector<std::string>& v) {
        uint64_t n = v.size();
        write_raw(&n, 8);
        for (auto& s : v) *this << s;
        return *this;
    }

    // --- reading -------------------------------------------------------------------------
    void read_raw(void* p, size_t n) {
        if (n > buf_.size() - cur_) throw std::out_of_range("Archive::read_raw past end");  // no overflow: cur_ <= size
        if (n == 0) return;   // an empty block may come with a null destination (an empty vector's data())
        std::memcpy(p, buf_.data() + cur_, n);
        cur_ += n;
    }
    template <class T>
    typename std::enable_if<std::is_trivially_copyable<T>::value, Archive&>::type operator>>(T& v) {
        read_raw(&v, sizeof(T));
        return *this;
    }
    Archive& operator>>(std::string& s) {
        uint64_t n = 0;
        read_raw(&n, 8);
        if (n > buf_.size() - cur_) throw std::out_of_range("Archive: string past end");
        s.assign((const char*)buf_.data() + cur_, n);
        cur_ += n;
        return *this;
    }
    template <class T>
    typename std::enable_if<std::is_trivially_copyable<T>::value, Archive&>::type operator>>(std::vector<T>& v) {
        uint64_t n = 0;
        read_raw(&n, 8);
        if (n > (buf_.size() - cur_) / sizeof(T)) throw std::out_of_range("Archive: vector past end");
        v.resize(n);
        if (n) read_raw(v.data(), n * sizeof(T));
        return *this;
    }
    Archive& operator>>(std::vector<std::string>& v) {
        uint64_t n = 0;
        read_raw(&n, 8);
        if (n > (buf_.size() - cur_) / 8) throw std::out_of_range("Archive: string vector past end");  // each entry has an 8-byte length
        v.resize(n);
        for (auto& s : v) *this >> s;
        return *this;
    }
    // Pop a POD from the tail (message meta travels last).
    template <class T>
    void read_back(T& v) {
        static_assert(std::is_trivially_copyable<T>::value, "POD only");
        if (buf_.size() < cur_ + sizeof(T)) throw std::out_of_range("Archive::read_back underflow");
        std::memcpy(&v, buf_.data() + buf_.size() - sizeof(T), sizeof(T));
        buf_.resize(buf_.size() - sizeof(T));
    }

    bool is_exhausted() const { return cur_ == buf_.size(); }
    size_t remaining() const { return buf_.size() - cur_; }
    // A count read from the wire may claim at most what is left: `n` records of `record_bytes` each.
    bool can_hold(int64_t n, size_t record_bytes) const { return n >= 0 && (uint64_t)n <= remaining() / (record_bytes ? record_bytes : 1); }
    size_t size() const { return buf_.size(); }
    size_t cursor() const { return cur_; }
    const uint8_t* data() const { return buf_.data(); }
    const uint8_t* cursor_ptr() const { return buf_.data() + cur_; }
    void skip(size_t n) {
        if (n > buf_.size() - cur_) throw std::out_of_range("Archive::skip past end");
        cur_ += n;
    }
    void rewind() { cur_ = 0; }
    void clear() { buf_.clear(); cur_ = 0; }
    std::vector<uint8_t>& bytes() { return buf_; }
    const std::vector<uint8_t>& bytes() const { return buf_; }
    std::vector<uint8_t> release() { cur_ = 0; return std::move(buf_); }

private:
    std::vector<uint8_t> buf_;
    size_t cur_ = 0;
};

}  // namespace psb
