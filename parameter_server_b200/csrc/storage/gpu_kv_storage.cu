// GPU back-end of KVStorage: the table of one server lives in HBM (GpuTable); requests that arrive
// over the host RPC path carry host buffers, which are staged through pinned memory and served by the
// same fused kernels as the collective path (a private single-rank SparseEngine). Shards are logical:
// the set of local shard ids is kept on the host and scans filter on shard_of(key).
#include <cuda_runtime.h>

#include <algorithm>
#include <mutex>
#include <set>

#include "../operator/sparse_engine.h"
#include "gpu_table.h"
#include "kv_storage.h"

namespace psb {

namespace {

class GpuKVStorage : public KVStorage {
public:
    explicit GpuKVStorage(const GpuKVStorageConfig& cfg) : cfg_(cfg) {
        GpuTableConfig tc;
        tc.device = cfg.device;
        tc.dim = cfg.base.dim;
        tc.opt_type = cfg.base.opt_type;
        tc.sync_delta = cfg.base.sync_delta;
        tc.index_capacity = std::max<uint64_t>(2 * cfg.capacity, 4096);
        tc.max_rows = cfg.max_rows;
        tc.init_seed = cfg.base.init_seed;
        tc.init_range = cfg.base.init_range;
        tc.slot_init0 = cfg.base.slot_init0;
        tc.slot_init1 = cfg.base.slot_init1;
        tc.soft_limit_bytes = cfg.base.soft_limit_bytes;
        tc.hard_limit_bytes = cfg.base.hard_limit_bytes;
        const uint64_t stride_bytes = 4ull * cfg.base.dim * (1 + opt_num_slots(cfg.base.opt_type) + (cfg.base.sync_delta ? 1 : 0));
        uint32_t shift = 12;
        while (shift < 22 && ((stride_bytes << (shift + 1)) <= (256ull << 20))) ++shift;
        tc.slab_shift = shift;
        table_.reset(new GpuTable(tc));
        SparseEngineConfig ec;
        ec.world = 1;
        ec.rank = 0;
        ec.max_keys = cfg.max_batch;
        ec.n_shards = 1;  // the private engine never partitions: every key is local
        engine_.reset(new SparseEngine(table_.get(), ec));
        n_shards_ = cfg.base.n_shards;
        cudaSetDevice(cfg.device);
        cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking);
        const size_t B = cfg.max_batch;
        cudaMalloc(&d_keys_, B * 8);
        cudaMalloc(&d_rows_, B * table_->stride() * 4);
        cudaMalloc(&d_found_, B * 4);
        cudaHostAlloc((void**)&h_keys_, B * 8, cudaHostAllocDefault);
        cudaHostAlloc((void**)&h_rows_, B * table_->stride() * 4, cudaHostAllocDefault);
    }
    ~GpuKVStorage() override {
        cudaSetDevice(cfg_.device);
        cudaStreamSynchronize(stream_);
        engine_.reset();
        cudaFree(d_keys_);
        cudaFree(d_rows_);
        cudaFree(d_found_);
        cudaFreeHost(h_keys_);
        cudaFreeHost(h_rows_);
        cudaStreamDestroy(stream_);
    }

    uint32_t dim() const override { return table_->dim(); }
    uint32_t stride() const override { return table_->stride(); }
    int32_t n_shards() const override { return n_shards_; }
    void set_n_shards(int32_t n) override { n_shards_ = n; }
    int shard_of(int64_t key) const override { return sparse_shard_of(key, n_shards_); }
    const char* backend() const override { return "gpu"; }

    Status create_shard(int s) override {
        std::lock_guard<std::mutex> g(mu_);
        local_.insert(s);
        return Status::Ok();
    }
    Status erase_shard(int s) override {
        std::lock_guard<std::mutex> g(mu_);
        if (!local_.erase(s)) return Status::Ok();
        ShardFilter f;
        f.mode = 1;
        f.shard = s;
        f.n_shards = n_shards_;
        uint64_t erased = 0;
        return table_->erase_filter(f, &erased, stream_);
    }
    bool has_shard(int s) const override {
        std::lock_guard<std::mutex> g(mu_);
        return local_.count(s) != 0;
    }
    std::vector<int> shard_list() const override {
        std::lock_guard<std::mutex> g(mu_);
        return std::vector<int>(local_.begin(), local_.end());
    }

    // Keys arrive from the network: the two values the index reserves for "empty" and "erased" are refused
    // before anything is launched.
    static Status screen_keys(const int64_t* keys, size_t n) {
        for (size_t i = 0; i < n; ++i)
            if (keys[i] <= (int64_t)kTombstoneKey)
                return Status::InvalidConfig("key " + std::to_string(keys[i]) + " is reserved by the GPU table (INT64_MIN, INT64_MIN + 1)");
        return Status::Ok();
    }
    // After a fatal device status (time-out, scratch inconsistency) the private engine is re-armed at once, so
    // that the failed request does not poison the requests after it.
    Status checked(Status st) {
        if (!st.ok() && st.code() != StatusCode::OUT_OF_MEMORY && st.code() != StatusCode::INVALID_CONFIG &&
            st.code() != StatusCode::INVALID_ID)
            engine_->reset(stream_);
        return st;
    }

    Status pull(int s, const int64_t* keys, size_t n, float* out, bool insert) override {
        std::lock_guard<std::mutex> g(mu_);
        if (!local_.count(s)) return Status::InvalidID("shard " + std::to_string(s) + " is not local");
        if (insert && !table_->healthy()) return Status::OOM("storage is unhealthy");
        PSB_RETURN_IF_ERROR(screen_keys(keys, n));
        cudaSetDevice(cfg_.device);
        const uint32_t dim = table_->dim();
        for (size_t off = 0; off < n; off += cfg_.max_batch) {
            const size_t m = std::min<size_t>(cfg_.max_batch, n - off);
            std::copy_n(keys + off, m, h_keys_);
            cudaMemcpyAsync(d_keys_, h_keys_, m * 8, cudaMemcpyHostToDevice, stream_);
            unsigned flags = FUSED_COPY_ROWS | (insert ? FUSED_INSERT : 0);
            PSB_RETURN_IF_ERROR(checked(engine_->pull(d_keys_, (uint32_t)m, 1, d_rows_, flags, stream_)));
            cudaMemcpyAsync(h_rows_, d_rows_, m * dim * 4, cudaMemcpyDeviceToHost, stream_);
            PSB_RETURN_IF_ERROR(checked(engine_->check(stream_)));
            std::copy_n(h_rows_, m * dim, out + off * dim);
        }
        return Status::Ok();
    }

    // All or nothing on memory pressure, as the client's retry after OUT_OF_MEMORY expects
    // (pico-ps/handler/Handler.cpp:65-103): rows are attached by the plan step (a pull without output); only
    // when every key of the request has a row is the first gradient applied. A request larger than one batch
    // plans all its batches before it applies any.
    Status push(int s, const int64_t* keys, const float* grads, size_t n, const OptConfig& opt, bool sync) override {
        std::lock_guard<std::mutex> g(mu_);
        if (!local_.count(s)) return Status::InvalidID("shard " + std::to_string(s) + " is not local");
        if (!table_->healthy()) return Status::OOM("storage is unhealthy");
        PSB_RETURN_IF_ERROR(screen_keys(keys, n));
        cudaSetDevice(cfg_.device);
        const uint32_t dim = table_->dim();
        const bool one_batch = n <= cfg_.max_batch;
        for (int pass = one_batch ? 1 : 0; pass < 2; ++pass) {
            for (size_t off = 0; off < n; off += cfg_.max_batch) {
                const size_t m = std::min<size_t>(cfg_.max_batch, n - off);
                std::copy_n(keys + off, m, h_keys_);
                cudaMemcpyAsync(d_keys_, h_keys_, m * 8, cudaMemcpyHostToDevice, stream_);
                PSB_RETURN_IF_ERROR(checked(engine_->pull(d_keys_, (uint32_t)m, 1, nullptr, FUSED_INSERT | FUSED_PREPARE_PUSH, stream_)));
                PSB_RETURN_IF_ERROR(checked(engine_->check(stream_)));  // OUT_OF_MEMORY here: nothing was applied
                if (pass == 0) continue;
                std::copy_n(grads + off * dim, m * dim, h_rows_);
                cudaMemcpyAsync(d_rows_, h_rows_, m * dim * 4, cudaMemcpyHostToDevice, stream_);
                PSB_RETURN_IF_ERROR(checked(engine_->push(d_rows_, (uint32_t)m, opt, sync ? FUSED_SYNC_PUSH : 0, stream_)));
                PSB_RETURN_IF_ERROR(checked(engine_->check(stream_)));
            }
        }
        return Status::Ok();
    }

    Status store(const OptConfig& opt) override {
        std::lock_guard<std::mutex> g(mu_);
        PSB_RETURN_IF_ERROR(table_->store_delta(opt, stream_));
        cudaStreamSynchronize(stream_);
        return Status::Ok();
    }

    Status set_rows(const int64_t* keys, const float* rows, size_t n, bool emb_only) override {
        std::lock_guard<std::mutex> g(mu_);
        PSB_RETURN_IF_ERROR(screen_keys(keys, n));
        cudaSetDevice(cfg_.device);
        const uint32_t w = emb_only ? table_->dim() : table_->stride();
        size_t m = 0;
        auto flush = [&]() -> Status {
            if (m == 0) return Status::Ok();
            cudaMemcpyAsync(d_keys_, h_keys_, m * 8, cudaMemcpyHostToDevice, stream_);
            cudaMemcpyAsync(d_rows_, h_rows_, m * w * 4, cudaMemcpyHostToDevice, stream_);
            Status st = table_->set_rows(d_keys_, d_rows_, m, emb_only, stream_);
            m = 0;
            return st;
        };
        for (size_t i = 0; i < n; ++i) {
            if (!local_.count(shard_of(keys[i]))) continue;
            h_keys_[m] = keys[i];
            std::copy_n(rows + i * w, w, h_rows_ + m * w);
            if (++m == cfg_.max_batch) PSB_RETURN_IF_ERROR(flush());
        }
        return flush();
    }

    Status export_shard(int s, uint64_t cursor, uint64_t window, bool dirty_only, std::vector<int64_t>* keys,
                        std::vector<float>* rows, uint64_t* next_cursor, bool* finished) override {
        std::lock_guard<std::mutex> g(mu_);
        cudaSetDevice(cfg_.device);
        *finished = true;
        *next_cursor = cursor;
        if (!local_.count(s)) return Status::Ok();
        window = std::min<uint64_t>(window, cfg_.max_batch);
        ShardFilter f;
        f.mode = 1;
        f.shard = s;
        f.n_shards = n_shards_;
        uint64_t n = 0, next = 0;
        // dirty_only: scan the shard and keep the dirty rows (two filters: scan dirty, then match the shard on the host)
        if (dirty_only) f.mode = 4;
        PSB_RETURN_IF_ERROR(table_->export_window(cursor, window, f, (long long*)d_keys_, d_rows_, &n, &next, stream_));
        if (n) {
            cudaMemcpyAsync(h_keys_, d_keys_, n * 8, cudaMemcpyDeviceToHost, stream_);
            cudaMemcpyAsync(h_rows_, d_rows_, n * table_->stride() * 4, cudaMemcpyDeviceToHost, stream_);
            cudaStreamSynchronize(stream_);
            for (uint64_t i = 0; i < n; ++i) {
                if (dirty_only && shard_of(h_keys_[i]) != s) continue;
                keys->push_back(h_keys_[i]);
                rows->insert(rows->end(), h_rows_ + i * table_->stride(), h_rows_ + (i + 1) * table_->stride());
            }
        }
        *next_cursor = next;
        *finished = next >= table_->index_capacity();
        return Status::Ok();
    }

    // slot cursors hold until the index is rebuilt larger
    uint64_t layout_epoch(int) override {
        std::lock_guard<std::mutex> g(mu_);
        return table_->grow_count();
    }

    Status erase_keys(const int64_t* keys, size_t n, uint64_t* erased) override {
        std::lock_guard<std::mutex> g(mu_);
        PSB_RETURN_IF_ERROR(screen_keys(keys, n));
        cudaSetDevice(cfg_.device);
        *erased = 0;
        for (size_t off = 0; off < n; off += cfg_.max_batch) {
            const size_t m = std::min<size_t>(cfg_.max_batch, n - off);
            std::copy_n(keys + off, m, h_keys_);
            cudaMemcpyAsync(d_keys_, h_keys_, m * 8, cudaMemcpyHostToDevice, stream_);
            uint64_t e = 0;
            PSB_RETURN_IF_ERROR(table_->erase_keys((const long long*)d_keys_, m, &e, stream_));
            *erased += e;
        }
        return Status::Ok();
    }

    bool erase_if_builtin(int s, const ScanPredicate& p, uint64_t* erased, Status* st) override {
        std::lock_guard<std::mutex> g(mu_);
        *erased = 0;
        if (!local_.count(s)) {
            *st = Status::Ok();
            return true;
        }
        ShardFilter f;
        f.mode = 1;
        f.shard = s;
        f.n_shards = n_shards_;
        *st = table_->erase_if(f, p.type, p.mod, p.rem, p.threshold, erased, stream_);
        return true;
    }
    bool reduce_builtin(int s, uint32_t section, ScanStats* out, Status* st) override {
        std::lock_guard<std::mutex> g(mu_);
        *out = ScanStats();
        if (!local_.count(s)) {
            *st = Status::Ok();
            return true;
        }
        ShardFilter f;
        f.mode = 1;
        f.shard = s;
        f.n_shards = n_shards_;
        *st = table_->reduce_section(f, section, &out->count, &out->sum, &out->sum_sq, &out->max_abs, stream_);
        return true;
    }

    uint64_t shard_size(int s) override {
        std::lock_guard<std::mutex> g(mu_);
        if (!local_.count(s)) return 0;
        std::vector<uint64_t> counts;
        if (!table_->shard_counts(n_shards_, &counts, stream_).ok()) return 0;
        return counts[s];
    }
    uint64_t size() override { return table_->size(); }
    uint64_t memory_usage() override { return table_->memory_usage(); }
    bool healthy() override { return table_->healthy(); }
    void set_healthy(bool h) override { table_->set_healthy(h); }
    bool check_healthy() override { return table_->check_healthy(); }
    void set_limits(uint64_t soft, uint64_t hard) override { table_->set_limits(soft, hard); }
    void enable_dirty_tracking() override { table_->enable_dirty_tracking(); }
    void clear_dirty() override {
        table_->clear_dirty(stream_);
        cudaStreamSynchronize(stream_);
    }
    Status clear() override {
        std::lock_guard<std::mutex> g(mu_);
        PSB_RETURN_IF_ERROR(table_->clear(stream_));
        return engine_->reset(stream_);
    }

private:
    GpuKVStorageConfig cfg_;
    std::unique_ptr<GpuTable> table_;
    std::unique_ptr<SparseEngine> engine_;
    int32_t n_shards_ = 1;
    mutable std::mutex mu_;
    std::set<int> local_;
    cudaStream_t stream_ = nullptr;
    long long* d_keys_ = nullptr;
    float* d_rows_ = nullptr;
    int* d_found_ = nullptr;
    int64_t* h_keys_ = nullptr;
    float* h_rows_ = nullptr;
};

}  // namespace

Status make_gpu_kv_storage(const GpuKVStorageConfig& cfg, std::unique_ptr<KVStorage>* out) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || cfg.device >= n) {
        cudaGetLastError();
        return Status::InvalidConfig("gpu storage requested but CUDA device " + std::to_string(cfg.device) + " is not available");
    }
    if (cfg.base.partition != 0) return Status::InvalidConfig("gpu storage holds sparse tables; dense RPC tables use the host back-end");
    try {
        out->reset(new GpuKVStorage(cfg));
    } catch (const std::exception& e) {
        return Status::OOM(std::string("gpu storage: ") + e.what());
    }
    return Status::Ok();
}

}  // namespace psb
