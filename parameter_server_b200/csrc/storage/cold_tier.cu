#include "cold_tier.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <cstring>
#include <fstream>
#include <stdexcept>

namespace psb {

HostColdTier::HostColdTier(GpuTable* table, uint64_t capacity_rows, uint32_t window)
    : table_(table), capacity_(capacity_rows), window_(window), stride_(table->stride()), map_((int64_t)0x8000000000000000ull) {
    cudaSetDevice(table_->device());
    auto must = [](cudaError_t e, const char* what) {
        if (e != cudaSuccess) throw std::runtime_error(std::string("HostColdTier: ") + what + ": " + cudaGetErrorString(e));
    };
    must(cudaHostAlloc((void**)&pool_, capacity_ * (size_t)stride_ * 4, cudaHostAllocDefault), "pinned pool");
    cudaStream_t s;
    must(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking), "side stream");
    stream_ = s;
    cudaEvent_t ev;
    must(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming), "event");
    copied_ = ev;
    must(cudaMalloc(&d_keys_, (size_t)window_ * 8), "staging");
    must(cudaMalloc(&d_rows_, (size_t)window_ * stride_ * 4), "staging");
    must(cudaHostAlloc((void**)&h_keys_, (size_t)window_ * 8, cudaHostAllocDefault), "staging");
    must(cudaHostAlloc((void**)&h_rows_, (size_t)window_ * stride_ * 4, cudaHostAllocDefault), "staging");
}

HostColdTier::~HostColdTier() {
    cudaSetDevice(table_->device());
    if (staging_active_) staging_.wait();
    cudaStreamSynchronize((cudaStream_t)stream_);
    cudaEventDestroy((cudaEvent_t)copied_);
    cudaFree(d_keys_);
    cudaFree(d_rows_);
    cudaFreeHost(h_keys_);
    cudaFreeHost(h_rows_);
    cudaFreeHost(pool_);
    cudaStreamDestroy((cudaStream_t)stream_);
}

Status HostColdTier::store_row(int64_t key, const float* row) {
    auto* e = map_.find(key);
    uint32_t slot;
    if (e) {
        slot = e->second;
    } else {
        if (!free_.empty()) {
            slot = free_.back();
            free_.pop_back();
        } else if (next_ < capacity_) {
            slot = next_++;
        } else {
            return Status::OOM("cold tier is full");
        }
        map_.force_emplace(key, slot);
    }
    std::memcpy(pool_ + (size_t)slot * stride_, row, (size_t)stride_ * 4);
    return Status::Ok();
}

Status HostColdTier::spill_if(uint32_t section, float threshold, uint64_t* n_spilled) {
    // staged rows live only in the staging buffers until commit_fetch inserts them
    if (staging_active_) return Status::Error("cold tier: a staged prefetch is pending, call commit_fetch first");
    cudaSetDevice(table_->device());
    cudaStream_t s = (cudaStream_t)stream_;
    *n_spilled = 0;
    const uint32_t dim = table_->dim();
    if ((section + 1) * dim > stride_) return Status::InvalidConfig("spill_if: no such row section");
    ShardFilter all;
    all.mode = 0;
    uint64_t cursor = 0;
    std::vector<int64_t> victims;
    while (cursor < table_->index_capacity()) {
        uint64_t n = 0, next = 0;
        PSB_RETURN_IF_ERROR(table_->export_window(cursor, window_, all, d_keys_, d_rows_, &n, &next, s));
        cursor = next;
        if (n == 0) continue;
        cudaMemcpyAsync(h_keys_, d_keys_, n * 8, cudaMemcpyDeviceToHost, s);
        cudaMemcpyAsync(h_rows_, d_rows_, n * (size_t)stride_ * 4, cudaMemcpyDeviceToHost, s);
        if (cudaStreamSynchronize(s) != cudaSuccess) return Status::Error("cold tier: device to host copy failed");
        victims.clear();
        for (uint64_t i = 0; i < n; ++i) {
            const float* v = h_rows_ + i * stride_ + section * dim;
            double sum = 0;
            for (uint32_t k = 0; k < dim; ++k) sum += v[k];
            if (sum / dim < threshold) {
                PSB_RETURN_IF_ERROR(store_row(h_keys_[i], h_rows_ + i * stride_));
                victims.push_back(h_keys_[i]);
            }
        }
        if (!victims.empty()) {
            std::copy(victims.begin(), victims.end(), h_keys_);
            cudaMemcpyAsync(d_keys_, h_keys_, victims.size() * 8, cudaMemcpyHostToDevice, s);
            uint64_t erased = 0;
            PSB_RETURN_IF_ERROR(table_->erase_keys(d_keys_, victims.size(), &erased, s));
            *n_spilled += erased;
        }
    }
    return Status::Ok();
}

Status HostColdTier::spill_keys(const int64_t* keys, uint64_t n, uint64_t* n_spilled) {
    // staged rows live only in the staging buffers until commit_fetch inserts them
    if (staging_active_) return Status::Error("cold tier: a staged prefetch is pending, call commit_fetch first");
    cudaSetDevice(table_->device());
    cudaStream_t s = (cudaStream_t)stream_;
    *n_spilled = 0;
    int* d_found = nullptr;
    if (cudaMalloc(&d_found, (size_t)window_ * 4) != cudaSuccess) return Status::Error("cold tier: cudaMalloc");
    std::vector<int> found(window_);
    Status result;
    for (uint64_t off = 0; off < n && result.ok(); off += window_) {
        const uint64_t m = std::min<uint64_t>(window_, n - off);
        std::copy_n(keys + off, m, h_keys_);
        cudaMemcpyAsync(d_keys_, h_keys_, m * 8, cudaMemcpyHostToDevice, s);
        result = table_->get_rows(d_keys_, m, d_rows_, d_found, false, s);
        if (!result.ok()) break;
        cudaMemcpyAsync(h_rows_, d_rows_, m * (size_t)stride_ * 4, cudaMemcpyDeviceToHost, s);
        cudaMemcpyAsync(found.data(), d_found, m * 4, cudaMemcpyDeviceToHost, s);
        cudaStreamSynchronize(s);
        uint64_t v = 0;
        for (uint64_t i = 0; i < m && result.ok(); ++i)
            if (found[i]) {
                result = store_row(keys[off + i], h_rows_ + i * stride_);
                h_keys_[v++] = keys[off + i];
            }
        if (v && result.ok()) {
            cudaMemcpyAsync(d_keys_, h_keys_, v * 8, cudaMemcpyHostToDevice, s);
            uint64_t erased = 0;
            result = table_->erase_keys(d_keys_, v, &erased, s);
            *n_spilled += erased;
        }
    }
    cudaFree(d_found);
    return result;
}

Status HostColdTier::fetch(const int64_t* keys, uint64_t n, uint64_t* n_fetched) {
    // staged rows live only in the staging buffers until commit_fetch inserts them
    if (staging_active_) return Status::Error("cold tier: a staged prefetch is pending, call commit_fetch first");
    cudaSetDevice(table_->device());
    cudaStream_t s = (cudaStream_t)stream_;
    *n_fetched = 0;
    uint64_t m = 0;
    auto flush = [&]() -> Status {
        if (m == 0) return Status::Ok();
        cudaMemcpyAsync(d_keys_, h_keys_, m * 8, cudaMemcpyHostToDevice, s);
        cudaMemcpyAsync(d_rows_, h_rows_, m * (size_t)stride_ * 4, cudaMemcpyHostToDevice, s);
        Status st = table_->set_rows(d_keys_, d_rows_, m, false, s);  // synchronises the side stream
        *n_fetched += m;
        m = 0;
        return st;
    };
    for (uint64_t i = 0; i < n; ++i) {
        auto* e = map_.find(keys[i]);
        if (!e) continue;
        h_keys_[m] = keys[i];
        std::memcpy(h_rows_ + m * stride_, pool_ + (size_t)e->second * stride_, (size_t)stride_ * 4);
        free_.push_back(e->second);
        map_.erase(keys[i]);
        if (++m == window_) PSB_RETURN_IF_ERROR(flush());
    }
    return flush();
}

void HostColdTier::stage_fetch_async(const int64_t* keys, uint64_t n) {
    if (staging_active_) return;  // one staged batch at a time: commit_fetch first
    std::vector<int64_t> copy(keys, keys + n);  // the caller's buffer may go away
    staging_active_ = true;
    staging_ = std::async(std::launch::async, [this, copy = std::move(copy)]() -> uint64_t {
        cudaSetDevice(table_->device());
        cudaStream_t s = (cudaStream_t)stream_;
        uint64_t m = 0;
        for (uint64_t i = 0; i < copy.size() && m < window_; ++i) {
            auto* e = map_.find(copy[i]);
            if (!e) continue;
            h_keys_[m] = copy[i];
            std::memcpy(h_rows_ + m * stride_, pool_ + (size_t)e->second * stride_, (size_t)stride_ * 4);
            free_.push_back(e->second);
            map_.erase(copy[i]);
            ++m;
        }
        if (m) {
            cudaMemcpyAsync(d_keys_, h_keys_, m * 8, cudaMemcpyHostToDevice, s);
            cudaMemcpyAsync(d_rows_, h_rows_, m * (size_t)stride_ * 4, cudaMemcpyHostToDevice, s);
        }
        cudaEventRecord((cudaEvent_t)copied_, s);
        return m;
    });
}

Status HostColdTier::commit_fetch(void* stream, uint64_t* n_fetched) {
    *n_fetched = 0;
    if (!staging_active_) return Status::Ok();
    const uint64_t m = staging_.get();
    staging_active_ = false;
    if (m == 0) return Status::Ok();
    cudaSetDevice(table_->device());
    if (cudaStreamWaitEvent((cudaStream_t)stream, (cudaEvent_t)copied_, 0) != cudaSuccess)
        return Status::Error("cold tier: cudaStreamWaitEvent failed");
    PSB_RETURN_IF_ERROR(table_->set_rows(d_keys_, d_rows_, m, false, stream));
    *n_fetched = m;
    return Status::Ok();
}

Status HostColdTier::save(const std::string& path, const std::string& version_uuid) const {
    std::ofstream f(path, std::ios::binary | std::ios::trunc);
    if (!f) return Status::Error("cold tier: cannot open " + path);
    const char magic[8] = {'P', 'S', 'B', 'C', 'O', 'L', 'D', '1'};
    uint64_t n = map_.size(), ulen = version_uuid.size();
    f.write(magic, 8);
    f.write((const char*)&stride_, 4);
    f.write((const char*)&ulen, 8);
    f.write(version_uuid.data(), (std::streamsize)ulen);
    f.write((const char*)&n, 8);
    for (auto& e : map_.buckets()) {
        if (!map_.live(e)) continue;
        f.write((const char*)&e.first, 8);
        f.write((const char*)(pool_ + (size_t)e.second * stride_), (std::streamsize)stride_ * 4);
    }
    return f.good() ? Status::Ok() : Status::Error("cold tier: write failed");
}

Status HostColdTier::load(const std::string& path, const std::string& expected_uuid) {
    std::ifstream f(path, std::ios::binary);
    if (!f) return Status::Error("cold tier: cannot open " + path);
    char magic[8];
    uint32_t stride = 0;
    uint64_t ulen = 0, n = 0;
    f.read(magic, 8);
    f.read((char*)&stride, 4);
    f.read((char*)&ulen, 8);
    if (!f || std::memcmp(magic, "PSBCOLD1", 8) != 0 || stride != stride_ || ulen > 4096) return Status::Error("cold tier: bad image");
    std::string uuid(ulen, '\0');
    f.read(&uuid[0], (std::streamsize)ulen);
    // a tier image written for another data layout must not be opened (need_remote_restore instead)
    if (uuid != expected_uuid) return Status::InvalidID("cold tier: version_uuid mismatch, restore remotely");
    f.read((char*)&n, 8);
    std::vector<float> row(stride_);
    for (uint64_t i = 0; i < n; ++i) {
        int64_t key;
        f.read((char*)&key, 8);
        f.read((char*)row.data(), (std::streamsize)stride_ * 4);
        if (!f) return Status::Error("cold tier: truncated image");
        PSB_RETURN_IF_ERROR(store_row(key, row.data()));
    }
    return Status::Ok();
}

}  // namespace psb
