// KVStorage: what the operators see of one table on one server - a set of local shards holding
// key -> row records - independent of where the rows live (host DRAM or GPU HBM).
//
// Parity: the ShardStorage contract of pico-ps/storage/Storage.h:129-138,261-289 (create_shard /
// erase_shard / shard_size / shard_memory_usage / get_shard_iterator / clear / healthy) plus the typed
// access the operators do through boost::any casts; here the value type is fixed to
// fp32 rows [embedding | optimizer slots | optional sync delta] so that one interface serves both
// back-ends.
#pragma once
#include <functional>
#include <memory>
#include <vector>

#include "../common/status.h"
#include "../kernels/optim.cuh"
#include "host_table.h"

namespace psb {

// Built-in scan predicates and reductions that a storage may evaluate where its rows live (a GPU table scans its
// slot array in a kernel; nothing but counters crosses PCIe). A storage that does not implement a hook returns
// false and the operator scans through export_shard on the host.
struct ScanPredicate {
    enum Type : int { KEY_MOD = 0, L2_BELOW = 1, SLOT0_BELOW = 2, ALL = 3 };
    int type = ALL;
    int64_t mod = 2, rem = 1;   // KEY_MOD: ((key % mod) + mod) % mod == rem
    double threshold = 0;       // L2_BELOW: ||emb||_2 < t;  SLOT0_BELOW: mean(slot 0) < t
};
struct ScanStats {
    uint64_t count = 0;
    double sum = 0, sum_sq = 0, max_abs = 0;
};

class KVStorage {
public:
    virtual ~KVStorage() = default;
    // Erase the entries of shard s that satisfy a built-in predicate, in place. Returns false when the storage has
    // no in-place scan (the caller falls back to the host scan); *st carries the outcome otherwise.
    virtual bool erase_if_builtin(int /*s*/, const ScanPredicate& /*p*/, uint64_t* /*erased*/, Status* /*st*/) { return false; }
    // count / sum / sum of squares / max |x| over row section `section` of every entry of shard s, in place.
    virtual bool reduce_builtin(int /*s*/, uint32_t /*section*/, ScanStats* /*out*/, Status* /*st*/) { return false; }
    virtual uint32_t dim() const = 0;
    virtual uint32_t stride() const = 0;
    virtual int32_t n_shards() const = 0;
    virtual void set_n_shards(int32_t n) = 0;
    virtual int shard_of(int64_t key) const = 0;
    virtual const char* backend() const = 0;

    virtual Status create_shard(int s) = 0;
    virtual Status erase_shard(int s) = 0;
    virtual bool has_shard(int s) const = 0;
    virtual std::vector<int> shard_list() const = 0;

    // keys all belong to shard s. out: n*dim.
    virtual Status pull(int s, const int64_t* keys, size_t n, float* out, bool insert) = 0;
    // pre-aggregated items of shard s. grads: n*dim.
    virtual Status push(int s, const int64_t* keys, const float* grads, size_t n, const OptConfig& opt, bool sync) = 0;
    virtual Status store(const OptConfig& opt) = 0;
    // rows: n*stride (or n*dim with emb_only); keys of shards that are not local are skipped.
    virtual Status set_rows(const int64_t* keys, const float* rows, size_t n, bool emb_only) = 0;
    // Resumable scan of one shard; appends to keys/rows (rows: stride floats per key).
    virtual Status export_shard(int s, uint64_t cursor, uint64_t window, bool dirty_only, std::vector<int64_t>* keys,
                                std::vector<float>* rows, uint64_t* next_cursor, bool* finished) = 0;
    virtual Status erase_keys(const int64_t* keys, size_t n, uint64_t* erased) = 0;
    // A number that changes whenever cursors of export_shard lose their meaning for shard s (the index was rebuilt).
    // A resumable scan that spans several requests compares it between windows and starts over when it moved.
    virtual uint64_t layout_epoch(int /*s*/) { return 0; }
    // Scan of a whole shard, entries handed to `fn` in windows (rows: stride floats per key). `fn` must not call into
    // this storage. A host shard is read as one snapshot under its lock. This default walks export_shard windows: when
    // the index is rebuilt between two of them, the scan starts over after `restart()` (the consumer forgets what it
    // got) - or fails with an error when the consumer cannot forget (`restart` empty), so the caller runs it again.
    using ScanFn = std::function<Status(const std::vector<int64_t>& keys, const std::vector<float>& rows)>;
    virtual Status scan_shard(int s, uint64_t window, bool dirty_only, const ScanFn& fn, const std::function<void()>& restart = nullptr) {
        std::vector<int64_t> keys;
        std::vector<float> rows;
        for (int attempt = 0; attempt < 8; ++attempt) {
            const uint64_t epoch = layout_epoch(s);
            uint64_t cursor = 0;
            bool finished = false, moved = false;
            while (!finished && !moved) {
                keys.clear();
                rows.clear();
                PSB_RETURN_IF_ERROR(export_shard(s, cursor, window, dirty_only, &keys, &rows, &cursor, &finished));
                moved = layout_epoch(s) != epoch;
                if (!moved && !keys.empty()) PSB_RETURN_IF_ERROR(fn(keys, rows));
            }
            if (!moved) return Status::Ok();
            if (!restart) break;
            restart();
        }
        return Status::Error("the index of shard " + std::to_string(s) + " was rebuilt during the scan: run it again");
    }

    // Writing scan of a whole shard: `fn(key, row)` may change the row (stride floats) and says whether it did. A host
    // shard is updated in place under its write lock. This default reads windows through export_shard and writes the
    // changed rows back with set_rows after each window: pushes of other clients that land in between are overwritten,
    // and a rebuild of the index in mid-scan ends it with an error (rows of the windows before it stay updated).
    using UpdateFn = std::function<bool(int64_t key, float* row)>;
    virtual Status update_shard(int s, uint64_t window, const UpdateFn& fn, uint64_t* changed) {
        if (changed) *changed = 0;
        const uint32_t w = stride();
        const uint64_t epoch = layout_epoch(s);
        std::vector<int64_t> keys, ckeys;
        std::vector<float> rows, crows;
        uint64_t cursor = 0;
        bool finished = false;
        while (!finished) {
            keys.clear();
            rows.clear();
            ckeys.clear();
            crows.clear();
            PSB_RETURN_IF_ERROR(export_shard(s, cursor, window, false, &keys, &rows, &cursor, &finished));
            if (layout_epoch(s) != epoch)
                return Status::Error("the index of shard " + std::to_string(s) + " was rebuilt during the writing scan");
            for (size_t i = 0; i < keys.size(); ++i) {
                if (!fn(keys[i], rows.data() + i * w)) continue;
                ckeys.push_back(keys[i]);
                crows.insert(crows.end(), rows.begin() + i * w, rows.begin() + (i + 1) * w);
            }
            if (!ckeys.empty()) PSB_RETURN_IF_ERROR(set_rows(ckeys.data(), crows.data(), ckeys.size(), false));
            if (changed) *changed += ckeys.size();
        }
        return Status::Ok();
    }

    virtual uint64_t shard_size(int s) = 0;
    virtual uint64_t size() = 0;
    virtual uint64_t memory_usage() = 0;
    virtual bool healthy() = 0;
    virtual void set_healthy(bool h) = 0;
    virtual bool check_healthy() = 0;   // re-evaluate the flag against the limits (the server's monitor calls it)
    // Pushed items that found no room and wait for memory (host storage only; a GPU table refuses the whole launch).
    virtual uint64_t overflow_size() { return 0; }
    virtual uint64_t drain_overflow() { return 0; }
    virtual void overflow_rows(int /*shard*/, std::vector<int64_t>* /*keys*/, std::vector<float>* /*rows*/) {}
    virtual void set_limits(uint64_t soft, uint64_t hard) = 0;
    virtual void enable_dirty_tracking() = 0;
    virtual void clear_dirty() = 0;
    virtual Status clear() = 0;
};

class HostKVStorage : public KVStorage {
public:
    explicit HostKVStorage(const HostTableConfig& cfg) : t_(cfg) {}
    HostTable& table() { return t_; }
    uint32_t dim() const override { return t_.dim(); }
    uint32_t stride() const override { return t_.stride(); }
    int32_t n_shards() const override { return t_.n_shards(); }
    void set_n_shards(int32_t n) override { t_.set_n_shards(n); }
    int shard_of(int64_t key) const override { return t_.shard_of(key); }
    const char* backend() const override { return "host"; }
    Status create_shard(int s) override { t_.create_shard(s); return Status::Ok(); }
    Status erase_shard(int s) override { t_.erase_shard(s); return Status::Ok(); }
    bool has_shard(int s) const override { return t_.has_shard(s); }
    std::vector<int> shard_list() const override { return t_.shard_list(); }
    Status pull(int s, const int64_t* keys, size_t n, float* out, bool insert) override {
        return t_.pull_shard(s, keys, n, out, insert);
    }
    Status push(int s, const int64_t* keys, const float* grads, size_t n, const OptConfig& opt, bool sync) override {
        return t_.push_shard(s, keys, grads, n, opt, sync);
    }
    Status store(const OptConfig& opt) override { return t_.store(opt); }
    Status set_rows(const int64_t* keys, const float* rows, size_t n, bool emb_only) override {
        return t_.set_rows(keys, rows, n, emb_only);
    }
    Status export_shard(int s, uint64_t cursor, uint64_t window, bool dirty_only, std::vector<int64_t>* keys,
                        std::vector<float>* rows, uint64_t* next_cursor, bool* finished) override {
        *next_cursor = t_.export_shard(s, cursor, window, dirty_only, keys, rows, finished);
        return Status::Ok();
    }
    Status erase_keys(const int64_t* keys, size_t n, uint64_t* erased) override {
        *erased = t_.erase_keys(keys, n);
        return Status::Ok();
    }
    uint64_t layout_epoch(int s) override { return t_.layout_epoch(s); }
    Status scan_shard(int s, uint64_t window, bool dirty_only, const ScanFn& fn, const std::function<void()>& = nullptr) override {
        return t_.scan_shard(s, (size_t)window, dirty_only, fn);
    }
    Status update_shard(int s, uint64_t, const UpdateFn& fn, uint64_t* changed) override { return t_.update_shard(s, fn, changed); }
    uint64_t shard_size(int s) override { return t_.shard_size(s); }
    uint64_t size() override { return t_.size(); }
    uint64_t memory_usage() override { return t_.memory_usage(); }
    bool healthy() override { return t_.healthy(); }
    void set_healthy(bool h) override { t_.set_healthy(h); }
    bool check_healthy() override { return t_.check_healthy(); }
    uint64_t overflow_size() override { return t_.overflow_size(); }
    uint64_t drain_overflow() override { return t_.drain_overflow(); }
    void overflow_rows(int s, std::vector<int64_t>* keys, std::vector<float>* rows) override { t_.overflow_rows(s, keys, rows); }
    void set_limits(uint64_t soft, uint64_t hard) override { t_.set_limits(soft, hard); }
    void enable_dirty_tracking() override { t_.enable_dirty_tracking(); }
    void clear_dirty() override { t_.clear_dirty(); }
    Status clear() override { t_.clear(); return Status::Ok(); }

private:
    HostTable t_;
};

// Factory of the GPU back-end (defined in gpu_kv_storage.cu; fails with a Status when no device is present).
struct GpuKVStorageConfig {
    int device = 0;
    HostTableConfig base;         // dim, optimizer, init, limits, n_shards
    uint64_t capacity = 1 << 20;  // expected keys on this server
    uint32_t max_batch = 1 << 18; // largest request (keys) served in one kernel call
    uint64_t max_rows = 0;        // row ceiling; 0 = follows the index, which then grows with the table
};
// Default visibility: operator plug-ins that subclass a built-in operator reference it through the inline code of
// the storage operator and bind to the host's definition.
__attribute__((visibility("default"))) Status make_gpu_kv_storage(const GpuKVStorageConfig& cfg, std::unique_ptr<KVStorage>* out);

}  // namespace psb
