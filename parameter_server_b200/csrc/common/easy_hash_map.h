// Small host-side open-addressing map used for key dedup / gradient pre-aggregation on the CPU path
// and inside the host storage shards.
//
// Parity: same contract as pico-ps/common/EasyHashMap.h:18-247 - power-of-two bucket count, load
// factor kept at or below 1/2 (the default; set_max_load changes it, the `grow_ratio` of the reference's storage
// configs, pico-ps/storage/KVShardStorage.h:444-452,881-897), triangular probing (step grows by one each probe), one reserved
// "empty" key, try_emplace / force_emplace / find / at / clear / reserve. Erase (not in the
// reference's map) is added with backward-shift-free tombstones because the host storage needs it.
#pragma once
#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <utility>
#include <vector>

#include "hash.h"

namespace psb {

template <class K, class V>
class EasyHashMap {
public:
    struct Entry {
        K first;
        V second;
    };

    explicit EasyHashMap(K empty_key, size_t expected = 0) : empty_(empty_key), tomb_(empty_key + 1) { rehash(buckets_for(expected)); }

    size_t size() const { return size_; }
    bool empty() const { return size_ == 0; }
    size_t bucket_count() const { return table_.size(); }

    void reserve(size_t n) {
        size_t b = buckets_for(n);
        if (b > table_.size()) rehash(b);
    }

    // Highest load (live entries + tombstones over buckets) before the table doubles. Kept inside [0.25, 0.85]:
    // triangular probing over a power-of-two table reaches every bucket, so any load below 1 ends, but probes get
    // long near it.
    void set_max_load(double f) {
        max_load_ = f < 0.25 ? 0.25 : (f > 0.85 ? 0.85 : f);
        if ((double)used_ > max_load_ * (double)table_.size()) rehash(buckets_for(size_));
    }
    double max_load() const { return max_load_; }
    // Memory of the bucket array, and how much it grows by when the next new key is inserted (0 when there is room).
    size_t bytes() const { return table_.size() * sizeof(Entry); }
    size_t next_insert_growth_bytes() const {
        if ((double)(used_ + 1) <= max_load_ * (double)table_.size()) return 0;
        return used_ > size_ * 2 + 8 ? 0 : table_.size() * sizeof(Entry);   // tombstone-heavy: rebuilt at the same size
    }
    // Counts the rebuilds of the bucket array: a bucket cursor taken under one value is meaningless under another.
    uint64_t generation() const { return generation_; }

    // Rebuild into the smallest table that holds the live entries when they fill less than `min_load` of the buckets
    // (also drops the tombstones). Invalidates bucket cursors, like growth does. Returns whether it rebuilt.
    bool shrink_if_below(double min_load) {
        if (min_load <= 0.0 || table_.size() <= 8) return false;
        if ((double)size_ >= min_load * (double)table_.size()) return false;
        const size_t want = buckets_for(size_);
        if (want >= table_.size()) return false;
        rehash(want);
        return true;
    }

    void clear() {
        // shrink when the table is much larger than what it held (keeps clear() cheap for small batches)
        size_t want = buckets_for(size_);
        if (table_.size() > 4 * want) {
            table_.assign(want, Entry{empty_, V()});
            ++generation_;
        } else {
            for (auto& e : table_) e.first = empty_;
        }
        size_ = 0;
        used_ = 0;
    }

    // Returns (entry*, inserted)
    // The two reserved keys (the empty marker and the one after it, the tombstone) cannot be stored: find never
    // matches them and try_emplace refuses them, so a caller that lets one through reads "absent" instead of the
    // contents of an empty bucket.
    bool reserved(const K& key) const { return key == empty_ || key == tomb_; }

    std::pair<Entry*, bool> try_emplace(const K& key, const V& value = V()) {
        if (reserved(key)) throw std::invalid_argument("EasyHashMap: reserved key");
        if ((double)(used_ + 1) > max_load_ * (double)table_.size()) rehash(used_ > size_ * 2 + 8 ? table_.size() : table_.size() * 2);
        size_t mask = table_.size() - 1;
        size_t p = (size_t)slot_hash((int64_t)key) & mask;
        Entry* first_tomb = nullptr;
        for (size_t np = 1;; ++np) {
            Entry& e = table_[p];
            if (e.first == key) return {&e, false};
            if (e.first == empty_) {
                Entry* dst = first_tomb ? first_tomb : &e;
                if (!first_tomb) ++used_;
                dst->first = key;
                dst->second = value;
                ++size_;
                return {dst, true};
            }
            if (e.first == tomb_ && !first_tomb) first_tomb = &e;
            p = (p + np) & mask;
        }
    }
    // Insert a key that is known to be absent.
    Entry* force_emplace(const K& key, const V& value = V()) { return try_emplace(key, value).first; }

    Entry* find(const K& key) {
        if (reserved(key)) return nullptr;
        size_t mask = table_.size() - 1;
        size_t p = (size_t)slot_hash((int64_t)key) & mask;
        for (size_t np = 1;; ++np) {
            Entry& e = table_[p];
            if (e.first == key) return &e;
            if (e.first == empty_) return nullptr;
            p = (p + np) & mask;
        }
    }
    const Entry* find(const K& key) const { return const_cast<EasyHashMap*>(this)->find(key); }
    size_t count(const K& key) const { return find(key) ? 1 : 0; }
    V& at(const K& key) {
        Entry* e = find(key);
        if (!e) throw std::out_of_range("EasyHashMap::at");
        return e->second;
    }
    bool erase(const K& key) {
        Entry* e = find(key);
        if (!e) return false;
        e->first = tomb_;
        --size_;
        return true;
    }

    template <class F>
    void for_each(F&& f) {
        for (auto& e : table_)
            if (e.first != empty_ && e.first != tomb_) f(e.first, e.second);
    }
    // Resumable iteration by bucket index (ShardIterator support).
    const std::vector<Entry>& buckets() const { return table_; }
    bool live(const Entry& e) const { return e.first != empty_ && e.first != tomb_; }

private:
    size_t buckets_for(size_t n) const {
        size_t b = 8;
        while ((double)n > max_load_ * (double)b) b <<= 1;
        return b;
    }
    void rehash(size_t nb) {
        std::vector<Entry> old;
        old.swap(table_);
        ++generation_;
        table_.assign(nb, Entry{empty_, V()});
        size_ = 0;
        used_ = 0;
        for (auto& e : old)
            if (e.first != empty_ && e.first != tomb_) try_emplace(e.first, e.second);
    }

    K empty_, tomb_;
    double max_load_ = 0.5;
    std::vector<Entry> table_;
    size_t size_ = 0;  // live entries
    size_t used_ = 0;  // live + tombstones (drives growth)
    uint64_t generation_ = 0;
};

}  // namespace psb
