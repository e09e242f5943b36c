// GpuKVShardStorage: the sparse table of one GPU.
//
// Parity: fills the role of the reference's KV shard storages (pico-ps/storage/KVShardStorage.h:97-952;
// pool_hash_map is its default, :958) and of the memory governor ShardStorageMemory
// (pico-ps/storage/Storage.h:141-258). Design for HBM3e instead of a CPU heap:
//   * ONE open-addressing index per GPU (16-byte slots, linear probing, 64-bit CAS) holds the keys
//     of every local shard; a shard is a logical subset (shard = jump_hash(murmur(key), G)) that
//     scans filter on, so resharding never rebuilds per-shard maps;
//   * rows ([embedding | optimizer slots | optional sync delta]) live in a slab pool that grows by
//     whole slabs without moving rows or rehashing: no 2x memory spike;
//   * a soft/hard byte budget makes allocation fail with OUT_OF_MEMORY and flips `healthy`, which
//     the service layer turns into the reference's back-pressure (pico-ps/storage/Storage.cpp:114-136).
#pragma once
#include <atomic>
#include <cstdint>
#include <string>
#include <vector>

#include "../common/status.h"
#include "../kernels/common.cuh"
#include "../kernels/optim.cuh"

namespace psb {

struct GpuTableConfig {
    int device = 0;
    uint32_t dim = 16;
    int32_t opt_type = OPT_SGD;
    bool sync_delta = false;         // rows carry a delta section for sync_push / store
    uint64_t index_capacity = 1u << 20;  // slots, rounded up to a power of two
    uint32_t slab_shift = 16;        // rows per slab = 2^slab_shift
    uint64_t init_seed = 0;
    float init_range = 0.01f;
    float slot_init0 = 0.f;
    float slot_init1 = 0.f;
    uint64_t soft_limit_bytes = 0;   // 0 = unlimited
    uint64_t hard_limit_bytes = 0;
    uint32_t max_probe = 4096;
    uint64_t max_rows = 0;           // row-pool ceiling (0 = 3/4 of the index capacity)
};

struct ShardFilter {
    // mode 0: every live entry; 1: entries of shard `shard`; 2: entries whose shard is NOT owned by
    // `rank` under `shard_owner` (foreign keys, purge); 3: entries whose shard is owned by `rank`
    // under `shard_owner` (what must move to `rank` during a reshard / restore)
    // 4: entries with the dirty bit set (incremental sync)
    int mode = 0;
    int shard = -1;
    int rank = -1;
    int n_shards = 1;
    const int* shard_owner = nullptr;  // device pointer, [n_shards]
};

class GpuTable {
public:
    explicit GpuTable(const GpuTableConfig& cfg);
    ~GpuTable();
    GpuTable(const GpuTable&) = delete;
    GpuTable& operator=(const GpuTable&) = delete;

    const GpuTableConfig& config() const { return cfg_; }
    uint32_t dim() const { return cfg_.dim; }
    uint32_t stride() const { return stride_; }
    uint32_t n_opt_slots() const { return n_slots_; }

    // Make sure `n` more rows can be attached without running out; grows the pool by slabs.
    Status reserve_rows(uint64_t n);
    // Room for exactly n_new more rows than are in use now (synchronous; for explicit pre-allocation).
    Status reserve_exact(uint64_t n_new);
    // Enqueue a copy of the allocation counters into pinned host memory (read by reserve_rows).
    void refresh_usage_async(void* stream);
    TableView view() const;
    // The same view in device memory, kept current by the table. Kernels whose launch is captured in a CUDA graph
    // read the table through this pointer, so that what the host changes between replays (a grown index, a larger
    // row ceiling, dirty tracking switched on) reaches them.
    const TableView* view_dev() const { return view_dev_; }
    // Grow the index (and the row ceiling with it) when `n_new` more keys would push its load above one half:
    // the reference's maps rehash on their own (pico-ps/storage/KVShardStorage.h:861-877 grow_ratio); here the
    // host calls this between launches (it synchronises the device when it has to grow, which is rare).
    // `auto_grow` off (the default for tables with an explicit max_rows) makes it a no-op.
    Status maybe_grow(uint64_t n_new);
    void set_auto_grow(bool on) { auto_grow_ = on; }
    uint64_t grow_count() const { return grows_; }

    uint64_t size();       // live keys (synchronises)
    uint64_t rows_used();  // rows handed out minus rows on the free stack (synchronises)
    uint64_t memory_usage() const { return bytes_; }
    bool healthy() const { return healthy_; }
    void set_limits(uint64_t soft, uint64_t hard) { cfg_.soft_limit_bytes = soft; cfg_.hard_limit_bytes = hard; }
    void set_healthy(bool h) { healthy_ = h; }
    // Periodic re-evaluation by the server's monitor: over a limit means unhealthy. The way back is explicit here
    // (clear, a purge after a reshard, set_healthy): slabs are never returned to the driver while the table lives.
    bool check_healthy() {
        if ((cfg_.hard_limit_bytes && bytes_ > cfg_.hard_limit_bytes) || (cfg_.soft_limit_bytes && bytes_ > cfg_.soft_limit_bytes))
            healthy_ = false;
        return healthy_;
    }

    // Resumable scan (the reference's ShardIterator, pico-ps/storage/Storage.h:49-77): examines at
    // most `window` slots starting at `cursor`, appends matching (key, full row) records to the
    // device buffers (capacity >= window) and returns the number written; *next_cursor == slot
    // capacity when the scan is finished.
    Status export_window(uint64_t cursor, uint64_t window, const ShardFilter& f, long long* out_keys,
                         float* out_rows, uint64_t* n_out, uint64_t* next_cursor, void* stream);
    // Overwrite / insert full rows (DirectPush semantics). `rows` holds n*stride floats, or n*dim
    // when `emb_only` (slots then take their initial values on insert and are kept on overwrite).
    Status set_rows(const long long* keys, const float* rows, uint64_t n, bool emb_only, void* stream);
    // Read rows of existing keys into out (n*stride floats, or n*dim when emb_only); found[i] = 0/1.
    Status get_rows(const long long* keys, uint64_t n, float* out, int* found, bool emb_only, void* stream);
    Status erase_keys(const long long* keys, uint64_t n, uint64_t* n_erased, void* stream);
    Status erase_filter(const ShardFilter& f, uint64_t* n_erased, void* stream);
    // In-place predicate erase over the entries matched by `f` (pico-ps/operator/EraseIfOperator.h:39-48 iterates a
    // shard under its lock and erases in place). pred_type: 0 key_mod (mod, rem), 1 ||emb||_2 < threshold,
    // 2 mean(slot 0) < threshold, 3 all. One kernel over the slot array; only the count returns to the host.
    Status erase_if(const ShardFilter& f, int pred_type, long long mod, long long rem, double threshold, uint64_t* n_erased,
                    void* stream);
    // count / sum / sum of squares / max |x| over row section `section` of the entries matched by `f`
    // (the reduction of pico-ps/operator/ForEachOperator.h:182-191 done where the rows live).
    Status reduce_section(const ShardFilter& f, uint32_t section, uint64_t* count, double* sum, double* sum_sq, double* max_abs,
                          void* stream);
    Status shard_counts(int n_shards, std::vector<uint64_t>* counts, void* stream);
    // Fold the sync-push delta sections into the weights (OP_STORE).
    Status store_delta(const OptConfig& opt, void* stream);
    Status clear(void* stream);
    // Reset the per-slot election word used by the fused push (only needed after a push that did not finish).
    Status clear_aux(void* stream);
    // Rebuild the index with `new_capacity` slots (drops tombstones; rows do not move).
    Status rebuild_index(uint64_t new_capacity, void* stream);
    uint64_t index_capacity() const { return capacity_; }
    uint64_t tombstones() const { return tombstones_; }
    // Dirty tracking for incremental sync: rows updated since the last clear_dirty().
    void enable_dirty_tracking();
    Status clear_dirty(void* stream);

    int device() const { return cfg_.device; }

private:
    Status add_slab();
    Status check_budget(uint64_t extra) ;
    Status publish_view();
    Status grow_row_ceiling(uint64_t new_max_rows);

    GpuTableConfig cfg_;
    uint32_t stride_ = 0, n_slots_ = 0;
    uint64_t capacity_ = 0;
    Slot* slots_ = nullptr;
    float** slabs_dev_ = nullptr;
    std::vector<float*> slabs_;
    uint32_t max_slabs_ = 0;
    uint32_t rows_avail_ = 0;
    volatile unsigned long long* host_mirror_ = nullptr;  // pinned copy of {row_bump, free_count}
    unsigned* row_bump_ = nullptr;
    unsigned* free_rows_ = nullptr;
    int* free_count_ = nullptr;
    uint64_t free_cap_ = 0;
    unsigned long long* n_items_ = nullptr;
    unsigned* touched_bits_ = nullptr;
    unsigned* touched_list_ = nullptr;
    unsigned* touched_count_ = nullptr;
    uint32_t touched_cap_ = 0;
    unsigned* dirty_bits_ = nullptr;
    uint64_t max_rows_ = 0;
    unsigned long long* scratch_ = nullptr;  // small device scratch for counters
    uint64_t bytes_ = 0;
    uint64_t tombstones_ = 0;
    std::atomic<bool> healthy_{true};   // read by request threads, re-evaluated by the server's monitor
    TableView* view_dev_ = nullptr;
    bool auto_grow_ = true;
    uint64_t grows_ = 0;
};

}  // namespace psb
