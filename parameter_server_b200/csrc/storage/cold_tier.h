// HostColdTier: a pinned-host-DRAM tier under a GpuTable, fed by cudaMemcpyAsync on a side stream.
//
// Parity: takes the place of the reference's persistent-memory tier (pico-ps/storage/DCPmemory.h:324-513,
// PmemHashMapShardStorage): capacity beyond the fast tier, and a persistent image that a restarted
// server can open locally instead of restoring over the network. Rows that are rarely touched are
// spilled from HBM to the host tier (the whole row: embedding + optimizer slots, so nothing is lost);
// rows that a batch is about to use are fetched back before the pull. `save` / `load` persist the tier
// with the table's version_uuid, checked on load like the reference's sanity_check
// (pico-ps/storage/DCPmemory.h:493-507).
#pragma once
#include <cstdint>
#include <future>
#include <string>
#include <vector>

#include "../common/easy_hash_map.h"
#include "gpu_table.h"

namespace psb {

class HostColdTier {
public:
    HostColdTier(GpuTable* table, uint64_t capacity_rows, uint32_t window = 1u << 16);
    ~HostColdTier();
    HostColdTier(const HostColdTier&) = delete;
    HostColdTier& operator=(const HostColdTier&) = delete;

    // Evict every row whose mean over row section `section` (0 = embedding, 1.. = optimizer slots) is below
    // `threshold` (e.g. section 1 of an Adagrad table: keys that received little gradient).
    Status spill_if(uint32_t section, float threshold, uint64_t* n_spilled);
    // Evict the given keys (host array) if they are in the table.
    Status spill_keys(const int64_t* keys, uint64_t n, uint64_t* n_spilled);
    // Bring back the rows of `keys` that live in the cold tier (call before pulling those keys).
    Status fetch(const int64_t* keys, uint64_t n, uint64_t* n_fetched);

    // Asynchronous fetch in two steps, so that the host-side gather and the PCIe copy of the NEXT batch's cold
    // rows overlap the current training step: stage_fetch_async returns at once (a worker thread looks the keys
    // up, packs at most `window` rows into pinned staging and starts their copy on the side stream);
    // commit_fetch joins the worker, makes `stream` wait for the copy and inserts the rows with a kernel on
    // `stream` (call it between two steps, before the pull that needs the rows).
    void stage_fetch_async(const int64_t* keys, uint64_t n);
    Status commit_fetch(void* stream, uint64_t* n_fetched);

    uint64_t size() const { return map_.size(); }
    uint64_t capacity() const { return capacity_; }
    uint64_t bytes() const { return capacity_ * (uint64_t)stride_ * 4; }
    Status save(const std::string& path, const std::string& version_uuid) const;
    Status load(const std::string& path, const std::string& expected_uuid);

private:
    Status store_row(int64_t key, const float* row);

    GpuTable* table_;
    uint64_t capacity_;
    uint32_t window_, stride_;
    float* pool_ = nullptr;  // pinned: capacity * stride floats
    EasyHashMap<int64_t, uint32_t> map_;
    std::vector<uint32_t> free_;
    uint32_t next_ = 0;
    void* stream_ = nullptr;          // side stream
    long long* d_keys_ = nullptr;     // device staging
    float* d_rows_ = nullptr;
    std::future<uint64_t> staging_;   // rows staged by the worker thread
    bool staging_active_ = false;
    void* copied_ = nullptr;          // event: staged rows are on the device
    int64_t* h_keys_ = nullptr;       // pinned staging
    float* h_rows_ = nullptr;
};

}  // namespace psb
