// CPU restatement of the reference's client-side sparse operators on top of HostTable:
//   pull = dedup keys -> partition by shard -> per-shard server pull -> scatter back per position
//          (pico-ps/operator/SparsePullOperator.h:81-110, :156-254, :278-304)
//   push = pre-aggregate duplicate keys (sum, in position order) -> partition -> per-shard apply
//          (pico-ps/operator/SparsePushOperator.h:109-154, :197-276)
// This is the numerical oracle of the fused kernels and the timed CPU baseline.
#pragma once
#include <vector>

#include "../common/easy_hash_map.h"
#include "../storage/host_table.h"

namespace psb {

// out: n_bags*dim with sum/mean pooling of `bag_size` consecutive keys (bag_size 1 = one row per key).
inline Status cpu_pull(HostTable& t, const int64_t* keys, size_t n, size_t bag_size, bool mean, float* out,
                       bool insert) {
    const uint32_t dim = t.dim();
    EasyHashMap<int64_t, uint32_t> whole(kHostEmptyKey, n);
    std::vector<std::vector<int64_t>> shard_keys(t.n_shards());
    std::vector<std::vector<uint32_t>> shard_uid(t.n_shards());
    uint32_t n_uniq = 0;
    std::vector<uint32_t> inverse(n);
    for (size_t i = 0; i < n; ++i) {
        if (whole.reserved(keys[i])) return Status::InvalidConfig("key " + std::to_string(keys[i]) + " is reserved");
        auto r = whole.try_emplace(keys[i], n_uniq);
        if (r.second) {
            int s = t.shard_of(keys[i]);
            shard_keys[s].push_back(keys[i]);
            shard_uid[s].push_back(n_uniq);
            ++n_uniq;
        }
        inverse[i] = r.first->second;
    }
    std::vector<float> uniq_rows((size_t)n_uniq * dim);
    std::vector<float> tmp;
    for (int s = 0; s < t.n_shards(); ++s) {
        if (shard_keys[s].empty()) continue;
        tmp.resize(shard_keys[s].size() * dim);
        PSB_RETURN_IF_ERROR(t.pull_shard(s, shard_keys[s].data(), shard_keys[s].size(), tmp.data(), insert));
        for (size_t j = 0; j < shard_keys[s].size(); ++j)
            std::copy_n(tmp.data() + j * dim, dim, uniq_rows.data() + (size_t)shard_uid[s][j] * dim);
    }
    const size_t n_bags = n / bag_size;
    const float scale = mean ? 1.0f / (float)bag_size : 1.0f;
    for (size_t b = 0; b < n_bags; ++b) {
        float* o = out + b * dim;
        for (uint32_t d = 0; d < dim; ++d) o[d] = 0.f;
        for (size_t j = 0; j < bag_size; ++j) {
            const float* r = uniq_rows.data() + (size_t)inverse[b * bag_size + j] * dim;
            for (uint32_t d = 0; d < dim; ++d) o[d] += r[d];
        }
        if (bag_size > 1)
            for (uint32_t d = 0; d < dim; ++d) o[d] *= scale;
    }
    return Status::Ok();
}

// grads: n_bags*dim (gradient w.r.t. the pooled output).
inline Status cpu_push(HostTable& t, const int64_t* keys, const float* grads, size_t n, size_t bag_size, bool mean,
                       const OptConfig& opt, bool sync) {
    // an unhealthy table refuses a push before anything of it is applied (what a push that was let in cannot place is
    // parked by the table, so a request is never half applied)
    if (!t.healthy()) return Status::OOM("storage is unhealthy");
    const uint32_t dim = t.dim();
    EasyHashMap<int64_t, uint32_t> whole(kHostEmptyKey, n);
    std::vector<int64_t> uniq_keys;
    std::vector<float> agg;
    const float scale = mean ? 1.0f / (float)bag_size : 1.0f;
    for (size_t i = 0; i < n; ++i) {
        if (whole.reserved(keys[i])) return Status::InvalidConfig("key " + std::to_string(keys[i]) + " is reserved");
        auto r = whole.try_emplace(keys[i], (uint32_t)uniq_keys.size());
        if (r.second) {
            uniq_keys.push_back(keys[i]);
            agg.resize(agg.size() + dim, 0.f);
        }
        float* a = agg.data() + (size_t)r.first->second * dim;
        const float* g = grads + (i / bag_size) * dim;
        if (bag_size > 1 && mean) for (uint32_t d = 0; d < dim; ++d) a[d] += g[d] * scale;
        else for (uint32_t d = 0; d < dim; ++d) a[d] += g[d];
    }
    std::vector<std::vector<int64_t>> shard_keys(t.n_shards());
    std::vector<std::vector<float>> shard_grads(t.n_shards());
    for (size_t u = 0; u < uniq_keys.size(); ++u) {
        int s = t.shard_of(uniq_keys[u]);
        shard_keys[s].push_back(uniq_keys[u]);
        shard_grads[s].insert(shard_grads[s].end(), agg.data() + u * dim, agg.data() + (u + 1) * dim);
    }
    for (int s = 0; s < t.n_shards(); ++s) {
        if (shard_keys[s].empty()) continue;
        PSB_RETURN_IF_ERROR(t.push_shard(s, shard_keys[s].data(), shard_grads[s].data(), shard_keys[s].size(), opt, sync));
    }
    return Status::Ok();
}

}  // namespace psb
