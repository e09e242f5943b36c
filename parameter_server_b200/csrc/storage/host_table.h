// HostTable: the CPU storage back-end (sharded, locked, in host DRAM).
//
// Three jobs: (1) the numerical oracle that the GPU kernels are tested against; (2) the storage of
// servers that run without a GPU (control-plane tests, serving on CPU); (3) the timed "CPU
// restatement" of the reference algorithm. It follows the reference's structure directly: one
// hash map per shard guarded by a reader/writer lock, pull that inserts missing keys unless
// read_only (pico-ps/operator/SparsePullOperator.h:200-229), push that applies the update rule per
// item under the exclusive lock (pico-ps/operator/SparsePushOperator.h:245-268), sync push into a
// delta buffer folded by store (pico-ps/operator/SparsePushOperator.h:278-416), resumable shard
// iteration (pico-ps/storage/KVShardStorage.h:52-92) and a byte budget that turns into
// OUT_OF_MEMORY (pico-ps/storage/Storage.cpp:114-136).
#pragma once
#include <algorithm>
#include <atomic>
#include <cstdint>
#include <map>
#include <memory>
#include <mutex>
#include <set>
#include <shared_mutex>
#include <vector>

#include "../common/easy_hash_map.h"
#include "../common/hash.h"
#include "../common/status.h"
#include "../kernels/optim.cuh"

namespace psb {

struct HostTableConfig {
    uint32_t dim = 16;
    int32_t opt_type = OPT_SGD;
    bool sync_delta = false;
    int32_t n_shards = 1;  // global shard count
    int32_t partition = 0; // 0: sparse keys, jump_consistent_hash(murmur(key)); 1: dense slices, key = (id << 24) | slice,
                           //    shard = hash(id, slice) % n_shards (pico-ps/common/dense_common.h:58-65);
                           // 2: key mod n_shards
    uint64_t init_seed = 0;
    float init_range = 0.01f;
    float slot_init0 = 0.f;
    float slot_init1 = 0.f;
    uint64_t soft_limit_bytes = 0;
    uint64_t hard_limit_bytes = 0;
    // Expected number of items of the whole table: every new shard sizes its index for its share up front, so that
    // the index is not rebuilt again and again while the table fills (`pool_hash_map.expected_max_items` of the
    // reference's default storage, pico-ps/storage/KVShardStorage.h:881-897).
    uint64_t expected_max_items = 0;
    // Load of a shard's index before it doubles (0 = the default 1/2), and the load under which the index is rebuilt
    // smaller after keys were erased (0 = never): `grow_ratio` / `shrink_ratio` of the reference's storage configs
    // (pico-ps/storage/KVShardStorage.h:425-429,444-449,863-866).
    double index_grow_ratio = 0.0;
    double index_shrink_ratio = 0.0;
};

constexpr int64_t kHostEmptyKey = (int64_t)0x8000000000000000ull;

class HostTable {
public:
    struct Shard {
        explicit Shard() : map(kHostEmptyKey) {}
        uint64_t born = 0;                   // which creation of a shard of this table this is (see layout_epoch)
        uint64_t index_bytes = 0;            // what of map.bytes() is counted in the table's memory usage
        EasyHashMap<int64_t, uint32_t> map;
        std::vector<float> rows;
        std::vector<uint32_t> free_rows;
        std::vector<uint32_t> touched;       // rows with a pending sync delta
        std::vector<uint8_t> touched_flag;   // per row
        std::vector<uint8_t> dirty;          // per row (incremental sync)
        // Pushed items whose key could not get a row (memory limit). The request they came with was accepted as a
        // whole, so they are kept here and applied once there is room again (ShardData::data_vector of the
        // reference: pico-ps/operator/SparsePushOperator.h:257-259, re-inserted by the purge,
        // pico-ps/operator/UpdateContextOperator.h:165-187). While the list is not empty pulls of the shard answer
        // OUT_OF_MEMORY (pico-ps/operator/SparsePullOperator.h:195-199).
        struct Parked {
            int64_t key;
            std::vector<float> grad;
            OptConfig opt;
            bool sync;
        };
        std::vector<Parked> overflow;
        mutable std::shared_mutex mu;
    };

    explicit HostTable(const HostTableConfig& cfg) : cfg_(cfg) {
        n_slots_ = (uint32_t)opt_num_slots(cfg_.opt_type);
        stride_ = cfg_.dim * (1 + n_slots_ + (cfg_.sync_delta ? 1 : 0));
    }

    uint32_t dim() const { return cfg_.dim; }
    uint32_t stride() const { return stride_; }
    int32_t n_shards() const { return cfg_.n_shards; }
    const HostTableConfig& config() const { return cfg_; }

    // --- shard lifecycle (create_shard / erase_shard of ShardStorage) --------------------------
    void create_shard(int s) {
        std::unique_lock<std::shared_mutex> g(mu_);
        if (!shards_.count(s)) {
            shards_[s].reset(new Shard());
            shards_[s]->born = ++shards_born_;
            if (cfg_.index_grow_ratio > 0.0) shards_[s]->map.set_max_load(cfg_.index_grow_ratio);
            if (cfg_.expected_max_items) {
                const uint64_t share = cfg_.expected_max_items / (uint64_t)std::max<int32_t>(1, cfg_.n_shards);
                shards_[s]->map.reserve((size_t)(share + share / 8 + 16));   // shards are not perfectly even
            }
            account_index(*shards_[s]);
        }
    }
    void erase_shard(int s) {
        std::unique_lock<std::shared_mutex> g(mu_);
        auto it = shards_.find(s);
        if (it != shards_.end()) {
            bytes_ -= it->second->rows.capacity() * sizeof(float) + it->second->index_bytes;
            n_items_ -= it->second->map.size();
            n_parked_ -= it->second->overflow.size();
            shards_.erase(it);
        }
    }
    bool has_shard(int s) const {
        std::shared_lock<std::shared_mutex> g(mu_);
        return shards_.count(s) != 0;
    }
    std::vector<int> shard_list() const {
        std::shared_lock<std::shared_mutex> g(mu_);
        std::vector<int> v;
        for (auto& kv : shards_) v.push_back(kv.first);
        return v;
    }

    int shard_of(int64_t key) const {
        if (cfg_.partition == 1) return dense_shard_of(key >> 24, (int32_t)(key & 0xFFFFFF), cfg_.n_shards);
        if (cfg_.partition == 2) return modulo_shard_of(key, cfg_.n_shards);
        return sparse_shard_of(key, cfg_.n_shards);
    }
    // Change the global shard count (reshard): existing shards keep their ids, the caller migrates keys.
    void set_n_shards(int32_t n) { cfg_.n_shards = n; }

    void init_row(float* row, int64_t key) const {
        for (uint32_t d = 0; d < cfg_.dim; ++d) row[d] = init_uniform(key, d, cfg_.init_seed, cfg_.init_range);
        for (uint32_t s = 0; s < n_slots_; ++s) {
            float iv = s == 0 ? cfg_.slot_init0 : cfg_.slot_init1;
            for (uint32_t d = 0; d < cfg_.dim; ++d) row[(s + 1) * cfg_.dim + d] = iv;
        }
        if (cfg_.sync_delta)
            for (uint32_t d = 0; d < cfg_.dim; ++d) row[(n_slots_ + 1) * cfg_.dim + d] = 0.f;
    }

    // Pull one shard's keys (keys must all map to shard `s`). out: n*dim floats.
    Status pull_shard(int s, const int64_t* keys, size_t n, float* out, bool insert) {
        Shard* sh = get(s);
        if (!sh) return Status::InvalidID("shard " + std::to_string(s) + " is not local");
        if (insert && !healthy_) return Status::OOM("storage is unhealthy");
        {
            // fast path: shared lock, no inserts needed
            std::shared_lock<std::shared_mutex> g(sh->mu);
            if (!sh->overflow.empty()) return Status::OOM("shard holds pushed items that are waiting for memory");
            size_t i = 0;
            for (; i < n; ++i) {
                auto* e = sh->map.find(keys[i]);
                if (!e) break;
                std::copy_n(sh->rows.data() + (size_t)e->second * stride_, cfg_.dim, out + i * cfg_.dim);
            }
            if (i == n) return Status::Ok();
            if (!insert) {
                for (; i < n; ++i) {
                    auto* e = sh->map.find(keys[i]);
                    if (e) std::copy_n(sh->rows.data() + (size_t)e->second * stride_, cfg_.dim, out + i * cfg_.dim);
                    else for (uint32_t d = 0; d < cfg_.dim; ++d)
                        out[i * cfg_.dim + d] = init_uniform(keys[i], d, cfg_.init_seed, cfg_.init_range);
                }
                return Status::Ok();
            }
        }
        // upgrade: exclusive lock for the inserts (the reference upgrades on the first miss)
        std::unique_lock<std::shared_mutex> g(sh->mu);
        for (size_t i = 0; i < n; ++i) {
            uint32_t row;
            Status st = find_or_insert(*sh, keys[i], &row);
            if (!st.ok()) return st;
            std::copy_n(sh->rows.data() + (size_t)row * stride_, cfg_.dim, out + i * cfg_.dim);
        }
        return Status::Ok();
    }

    // Push one shard's pre-aggregated items. grads: n*dim floats.
    Status push_shard(int s, const int64_t* keys, const float* grads, size_t n, const OptConfig& opt, bool sync) {
        Shard* sh = get(s);
        if (!sh) return Status::InvalidID("shard " + std::to_string(s) + " is not local");
        if (sync && !cfg_.sync_delta) return Status::InvalidConfig("table was created without sync_delta");
        std::unique_lock<std::shared_mutex> g(sh->mu);
        for (size_t i = 0; i < n; ++i) {
            uint32_t row;
            const float* gr = grads + i * cfg_.dim;
            Status st = find_or_insert(*sh, keys[i], &row);
            if (st.is(StatusCode::OUT_OF_MEMORY)) {
                // A request is applied as a whole or not at all (a client that is told OUT_OF_MEMORY sends it again,
                // and what had been applied would then count twice): items that find no room are parked, the
                // request succeeds, and the table - unhealthy from now on - refuses the NEXT requests up front.
                sh->overflow.push_back(typename Shard::Parked{keys[i], std::vector<float>(gr, gr + cfg_.dim), opt, sync});
                ++n_parked_;
                continue;
            }
            if (!st.ok()) return st;
            float* w = sh->rows.data() + (size_t)row * stride_;
            if (sync) {
                float* delta = w + (size_t)(n_slots_ + 1) * cfg_.dim;
                for (uint32_t d = 0; d < cfg_.dim; ++d) delta[d] += gr[d];
                if (!sh->touched_flag[row]) { sh->touched_flag[row] = 1; sh->touched.push_back(row); }
            } else {
                apply(opt, w, gr);
                if (track_dirty_) sh->dirty[row] = 1;
            }
        }
        return Status::Ok();
    }

    // OP_STORE: fold pending deltas of every local shard.
    Status store(const OptConfig& opt) {
        for (int s : shard_list()) {
            Shard* sh = get(s);
            std::unique_lock<std::shared_mutex> g(sh->mu);
            for (uint32_t row : sh->touched) {
                float* w = sh->rows.data() + (size_t)row * stride_;
                float* delta = w + (size_t)(n_slots_ + 1) * cfg_.dim;
                apply(opt, w, delta);
                for (uint32_t d = 0; d < cfg_.dim; ++d) delta[d] = 0.f;
                sh->touched_flag[row] = 0;
                if (track_dirty_) sh->dirty[row] = 1;
            }
            sh->touched.clear();
        }
        return Status::Ok();
    }

    // DirectPush: overwrite / insert full rows (n*stride floats) or embeddings only (n*dim).
    Status set_rows(const int64_t* keys, const float* rows, size_t n, bool emb_only) {
        for (size_t i = 0; i < n; ++i) {
            Shard* sh = get(shard_of(keys[i]));
            if (!sh) continue;  // not local: the caller routes, foreign keys are skipped (restore semantics)
            std::unique_lock<std::shared_mutex> g(sh->mu);
            uint32_t row;
            Status st = find_or_insert(*sh, keys[i], &row);
            if (!st.ok()) return st;
            float* w = sh->rows.data() + (size_t)row * stride_;
            if (emb_only) std::copy_n(rows + i * cfg_.dim, cfg_.dim, w);
            else std::copy_n(rows + i * stride_, stride_, w);
            if (!emb_only && cfg_.sync_delta && !sh->touched_flag[row]) {
                // a full row may carry a pending sync delta (a restore from a replica that buffered sync pushes): it
                // must be folded by the next store here as it will be there
                const float* delta = w + (size_t)(n_slots_ + 1) * cfg_.dim;
                bool pending = false;
                for (uint32_t d = 0; d < cfg_.dim && !pending; ++d) pending = delta[d] != 0.f;
                if (pending) { sh->touched_flag[row] = 1; sh->touched.push_back(row); }
            }
            if (track_dirty_) sh->dirty[row] = 1;
        }
        return Status::Ok();
    }

    // Read existing rows; found[i] = 0/1. Missing rows are zero-filled.
    void get_rows(const int64_t* keys, size_t n, float* out, int32_t* found, bool emb_only) const {
        const uint32_t width = emb_only ? cfg_.dim : stride_;
        for (size_t i = 0; i < n; ++i) {
            Shard* sh = get(shard_of(keys[i]));
            bool ok = false;
            if (sh) {
                std::shared_lock<std::shared_mutex> g(sh->mu);
                auto* e = sh->map.find(keys[i]);
                if (e) {
                    std::copy_n(sh->rows.data() + (size_t)e->second * stride_, width, out + i * width);
                    ok = true;
                }
            }
            if (!ok) std::fill_n(out + i * width, width, 0.f);
            if (found) found[i] = ok ? 1 : 0;
        }
    }

    uint64_t erase_keys(const int64_t* keys, size_t n) {
        uint64_t erased = 0;
        std::set<Shard*> thinned;
        for (size_t i = 0; i < n; ++i) {
            Shard* sh = get(shard_of(keys[i]));
            if (!sh) continue;
            std::unique_lock<std::shared_mutex> g(sh->mu);
            auto* e = sh->map.find(keys[i]);
            if (!e) continue;
            if (cfg_.index_shrink_ratio > 0.0) thinned.insert(sh);
            uint32_t row = e->second;
            sh->map.erase(keys[i]);
            sh->free_rows.push_back(row);
            sh->dirty[row] = 0;
            if (sh->touched_flag[row]) {
                sh->touched_flag[row] = 0;
                for (auto& t : sh->touched) if (t == row) { t = sh->touched.back(); sh->touched.pop_back(); break; }
            }
            ++erased;
        }
        n_items_ -= erased;
        for (Shard* sh : thinned) {   // safe_shrink of the reference (pico-ps/storage/KVShardStorage.h:786-834)
            std::unique_lock<std::shared_mutex> g(sh->mu);
            if (sh->map.shrink_if_below(std::min(cfg_.index_shrink_ratio, 0.5 * sh->map.max_load()))) account_index(*sh);
        }
        return erased;
    }

    // Resumable export of shard `s`: examines buckets [cursor, cursor+window) and appends live
    // entries (optionally only dirty ones). Returns the next cursor; == bucket_count when done.
    size_t export_shard(int s, size_t cursor, size_t window, bool dirty_only, std::vector<int64_t>* keys,
                        std::vector<float>* rows, bool* finished) const {
        Shard* sh = get(s);
        *finished = true;
        if (!sh) return 0;
        std::shared_lock<std::shared_mutex> g(sh->mu);
        const auto& b = sh->map.buckets();
        cursor = std::min(cursor, b.size());
        size_t end = std::min(b.size(), cursor + std::max<size_t>(window, 1));   // a window of 0 still moves on
        for (size_t i = cursor; i < end; ++i) {
            if (!sh->map.live(b[i])) continue;
            if (dirty_only && !sh->dirty[b[i].second]) continue;
            keys->push_back(b[i].first);
            const float* w = sh->rows.data() + (size_t)b[i].second * stride_;
            rows->insert(rows->end(), w, w + stride_);
        }
        *finished = end >= b.size();
        return end;
    }

    // Scan of a whole shard as one snapshot: the shard's read lock is held from the first window to the last, so
    // pushes and inserting pulls of that shard wait until the scan is over, while reads go on - what the reference
    // gets by iterating a shard under its lock (pico-ps/operator/DumpOperator.h:170-190,
    // pico-ps/operator/ForEachOperator.h:182-191). `fn(keys, rows)` sees at most `window` buckets' entries per call
    // and must not touch this table.
    template <class F>
    Status scan_shard(int s, size_t window, bool dirty_only, F&& fn) const {
        Shard* sh = get(s);
        if (!sh) return Status::Ok();
        std::shared_lock<std::shared_mutex> g(sh->mu);
        const auto& b = sh->map.buckets();
        std::vector<int64_t> keys;
        std::vector<float> rows;
        window = std::max<size_t>(window, 1);
        for (size_t cursor = 0; cursor < b.size(); cursor += window) {
            keys.clear();
            rows.clear();
            const size_t end = std::min(b.size(), cursor + window);
            for (size_t i = cursor; i < end; ++i) {
                if (!sh->map.live(b[i])) continue;
                if (dirty_only && !sh->dirty[b[i].second]) continue;
                keys.push_back(b[i].first);
                const float* w = sh->rows.data() + (size_t)b[i].second * stride_;
                rows.insert(rows.end(), w, w + stride_);
            }
            if (!keys.empty()) PSB_RETURN_IF_ERROR(fn(keys, rows));
        }
        return Status::Ok();
    }
    // Writing scan of a whole shard: `fn(key, row)` may change the row (stride floats) in place and says whether it
    // did. The shard's write lock is held for the scan, as in the reference's writing for_each
    // (pico-ps/operator/ForEachOperator.h:303-313 write_shard): no push lands between reading a row and writing it.
    template <class F>
    Status update_shard(int s, F&& fn, uint64_t* changed) {
        if (changed) *changed = 0;
        Shard* sh = get(s);
        if (!sh) return Status::Ok();
        std::unique_lock<std::shared_mutex> g(sh->mu);
        for (const auto& b : sh->map.buckets()) {
            if (!sh->map.live(b)) continue;
            if (!fn(b.first, sh->rows.data() + (size_t)b.second * stride_)) continue;
            if (track_dirty_) sh->dirty[b.second] = 1;
            if (changed) ++*changed;
        }
        return Status::Ok();
    }
    // Changes whenever the bucket cursors of export_shard lose their meaning for shard `s`: the index was rebuilt
    // (growth, shrink, clear) or the shard was dropped and created again.
    uint64_t layout_epoch(int s) const {
        Shard* sh = get(s);
        if (!sh) return 0;
        std::shared_lock<std::shared_mutex> g(sh->mu);
        return (sh->born << 32) + sh->map.generation();
    }

    uint64_t shard_size(int s) const {
        Shard* sh = get(s);
        if (!sh) return 0;
        std::shared_lock<std::shared_mutex> g(sh->mu);
        return sh->map.size();
    }
    uint64_t size() const { return n_items_; }
    uint64_t memory_usage() const { return bytes_; }
    bool healthy() const { return healthy_; }
    void set_healthy(bool h) { healthy_ = h; }
    void set_limits(uint64_t soft, uint64_t hard) { cfg_.soft_limit_bytes = soft; cfg_.hard_limit_bytes = hard; }
    // Re-evaluation of the health flag, called periodically by the server's monitor
    // (ShardStorageMemory::check_healthy, pico-ps/storage/Storage.cpp:114-136): over a limit means unhealthy; a table
    // that went unhealthy because a row pool could not grow is healthy again once there is room - rows were erased
    // (their slots are on the free lists), memory was given back (a shard dropped, a clear) or the limits were
    // raised far enough for the growth that failed.
    bool check_healthy() {
        const uint64_t b = bytes_;
        const uint64_t soft = cfg_.soft_limit_bytes, hard = cfg_.hard_limit_bytes;
        if ((hard && b > hard) || (soft && b > soft)) {
            healthy_ = false;
            return false;
        }
        if (!healthy_) {
            // parked items first: they take the rows that an erase freed in their shard, or memory that came back.
            // While some of them still find no room the table stays as it is - it does not turn healthy for a
            // moment only to refuse the next insert.
            if (n_parked_) drain_overflow(true);
            const uint64_t now = bytes_;
            const uint64_t extra = failed_extra_;
            const bool fits = (!hard || now + extra <= hard) && (!soft || now + extra <= soft);
            bool free_rows = false;
            for (int s : shard_list()) {
                Shard* sh = get(s);
                if (!sh) continue;
                std::shared_lock<std::shared_mutex> g(sh->mu);
                free_rows = free_rows || !sh->free_rows.empty();
            }
            if (n_parked_ == 0 && (fits || free_rows || now < failed_at_bytes_)) healthy_ = true;
        }
        if (healthy_ && n_parked_) drain_overflow();
        return healthy_;
    }
    // Fault injection for tests of the out-of-memory paths: every `period`-th insert of a NEW key fails as if the
    // row pool could not grow (0 switches it off). The role of the reference's TestBadAllocator, which throws
    // bad_alloc on every other large allocation (pico-ps/test/TestOps.h:437-476).
    void inject_insert_failures(uint32_t period) { fail_period_ = period; }
    // Items parked by pushes that found no room.
    uint64_t overflow_size() const { return n_parked_; }
    // The parked items of shard `s` as full rows - initial value with the parked gradients applied in their order: a
    // reshard sends them to the shard's new owners together with its stored rows. The list itself stays (it goes
    // with the old storage when the reshard commits, and is still needed when the reshard is abandoned).
    void overflow_rows(int s, std::vector<int64_t>* keys, std::vector<float>* rows) const {
        Shard* sh = get(s);
        if (!sh) return;
        std::shared_lock<std::shared_mutex> g(sh->mu);
        EasyHashMap<int64_t, uint32_t> at(kHostEmptyKey, sh->overflow.size());
        for (auto& it : sh->overflow) {
            auto r = at.try_emplace(it.key, (uint32_t)keys->size());
            if (r.second) {
                keys->push_back(it.key);
                rows->resize(rows->size() + stride_);
                float* fresh = rows->data() + (size_t)r.first->second * stride_;
                // the key may have got a row since (a push after the table had recovered, before the list was
                // drained): the parked gradients then go on top of that row, which this record will overwrite
                if (auto* have = sh->map.find(it.key)) std::copy_n(sh->rows.data() + (size_t)have->second * stride_, stride_, fresh);
                else init_row(fresh, it.key);
            }
            float* w = rows->data() + (size_t)r.first->second * stride_;
            if (it.sync) {
                float* delta = w + (size_t)(n_slots_ + 1) * cfg_.dim;
                for (uint32_t d = 0; d < cfg_.dim; ++d) delta[d] += it.grad[d];
            } else {
                apply(it.opt, w, it.grad.data());
            }
        }
    }
    // Apply the parked items now (after memory came back: the monitor, a purge, raised limits). Items that still find
    // no room stay parked. Returns how many are left.
    uint64_t drain_overflow(bool while_unhealthy = false) {
        for (int s : shard_list()) {
            Shard* sh = get(s);
            if (!sh) continue;
            std::unique_lock<std::shared_mutex> g(sh->mu);
            std::vector<typename Shard::Parked> still;
            for (auto& it : sh->overflow) {
                uint32_t row;
                if (!still.empty() || !find_or_insert(*sh, it.key, &row, while_unhealthy).ok()) {   // keep the order of what is left
                    still.push_back(std::move(it));
                    continue;
                }
                float* w = sh->rows.data() + (size_t)row * stride_;
                if (it.sync) {
                    float* delta = w + (size_t)(n_slots_ + 1) * cfg_.dim;
                    for (uint32_t d = 0; d < cfg_.dim; ++d) delta[d] += it.grad[d];
                    if (!sh->touched_flag[row]) { sh->touched_flag[row] = 1; sh->touched.push_back(row); }
                } else {
                    apply(it.opt, w, it.grad.data());
                    if (track_dirty_) sh->dirty[row] = 1;
                }
                --n_parked_;
            }
            sh->overflow.swap(still);
        }
        return n_parked_;
    }
    void enable_dirty_tracking() { track_dirty_ = true; }
    void clear_dirty() {
        for (int s : shard_list()) {
            Shard* sh = get(s);
            std::unique_lock<std::shared_mutex> g(sh->mu);
            std::fill(sh->dirty.begin(), sh->dirty.end(), 0);
        }
    }
    void clear() {
        for (int s : shard_list()) {
            Shard* sh = get(s);
            std::unique_lock<std::shared_mutex> g(sh->mu);
            bytes_ -= sh->rows.capacity() * sizeof(float);
            sh->map.clear();
            account_index(*sh);
            std::vector<float>().swap(sh->rows);
            sh->free_rows.clear(); sh->touched.clear(); sh->touched_flag.clear(); sh->dirty.clear();
            sh->overflow.clear();
        }
        n_items_ = 0;
        n_parked_ = 0;
        healthy_ = true;
    }

private:
    Shard* get(int s) const {
        std::shared_lock<std::shared_mutex> g(mu_);
        auto it = shards_.find(s);
        return it == shards_.end() ? nullptr : it->second.get();
    }

    // `draining`: the caller re-applies parked items of an unhealthy table (check_healthy); the limits still hold.
    Status find_or_insert(Shard& sh, int64_t key, uint32_t* row, bool draining = false) {
        auto* e = sh.map.find(key);
        if (e) { *row = e->second; return Status::Ok(); }
        if (sh.map.reserved(key)) return Status::InvalidConfig("key " + std::to_string(key) + " is reserved (the two smallest int64 values mark empty and erased slots)");
        if (!healthy_ && !draining) return Status::OOM("storage is unhealthy");
        if (fail_period_ && ++fail_counter_ % fail_period_ == 0) {   // fault injection, see inject_insert_failures
            failed_extra_ = 0;
            failed_at_bytes_ = bytes_.load();
            healthy_ = false;
            return Status::OOM("injected allocation failure");
        }
        // What this insert makes the table grow by: the row pool when it is full (it doubles) and the index when it
        // is at its load limit (it doubles too; the old bucket array beside the new one during the rebuild is not
        // counted). Both are refused together when they would cross a limit (the governor of the reference counts
        // its maps the same way, pico-ps/storage/KVShardStorage.h:875-877, pico-ps/storage/Storage.cpp:154-204).
        const bool reuse = !sh.free_rows.empty();
        const size_t old_cap = sh.rows.capacity();
        const size_t need = sh.rows.size() + stride_;
        size_t new_cap = old_cap;
        if (!reuse && need > old_cap) new_cap = std::max<size_t>(old_cap * 2, (size_t)stride_ * 64);
        const uint64_t extra = (new_cap - old_cap) * sizeof(float) + sh.map.next_insert_growth_bytes();
        if (extra) {
            const uint64_t b = bytes_;
            if ((cfg_.hard_limit_bytes && b + extra > cfg_.hard_limit_bytes) ||
                (cfg_.soft_limit_bytes && b + extra > cfg_.soft_limit_bytes)) {
                failed_extra_ = extra;
                failed_at_bytes_ = b;
                healthy_ = false;
                return Status::OOM("host table would exceed the memory limit");
            }
        }
        uint32_t r;
        if (reuse) {
            r = sh.free_rows.back();
            sh.free_rows.pop_back();
        } else {
            if (new_cap != old_cap) {
                sh.rows.reserve(new_cap);
                bytes_ += (sh.rows.capacity() - old_cap) * sizeof(float);
            }
            r = (uint32_t)(sh.rows.size() / stride_);
            sh.rows.resize(need);
            sh.touched_flag.push_back(0);
            sh.dirty.push_back(0);
        }
        init_row(sh.rows.data() + (size_t)r * stride_, key);
        sh.map.force_emplace(key, r);
        if (sh.map.bytes() != sh.index_bytes) account_index(sh);
        if (track_dirty_) sh.dirty[r] = 1;
        ++n_items_;
        *row = r;
        return Status::Ok();
    }

    // Keep the table's byte count in step with the shard's bucket array (called with the shard locked for writing).
    void account_index(Shard& sh) {
        const uint64_t now = sh.map.bytes();
        if (now >= sh.index_bytes) bytes_ += now - sh.index_bytes;
        else bytes_ -= sh.index_bytes - now;
        sh.index_bytes = now;
    }

    void apply(const OptConfig& opt, float* w, const float* g) const {
        const uint32_t dim = cfg_.dim;
        float dummy0 = 0.f, dummy1 = 0.f;
        for (uint32_t d = 0; d < dim; ++d) {
            float& s0 = n_slots_ > 0 ? w[dim + d] : dummy0;
            float& s1 = n_slots_ > 1 ? w[2 * dim + d] : dummy1;
            opt_update(opt, w[d], s0, s1, g[d]);
        }
    }

    HostTableConfig cfg_;
    uint32_t stride_ = 0, n_slots_ = 0;
    mutable std::shared_mutex mu_;
    std::map<int, std::unique_ptr<Shard>> shards_;
    std::atomic<uint64_t> n_items_{0};
    std::atomic<uint64_t> bytes_{0};
    std::atomic<bool> healthy_{true};
    std::atomic<uint64_t> n_parked_{0};
    std::atomic<uint32_t> fail_period_{0}, fail_counter_{0};
    uint64_t shards_born_ = 0;   // under mu_
    std::atomic<uint64_t> failed_extra_{0}, failed_at_bytes_{0};   // the growth that made the table unhealthy
    std::atomic<bool> track_dirty_{false};   // may be switched on while pushes run (a follower table appears)
};

}  // namespace psb
