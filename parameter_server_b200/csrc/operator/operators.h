// Built-in operators: each class carries the CLIENT half (build requests, digest responses) and the
// SERVER half (apply a request to the table entry) of one operation, as in the reference.
//
//   SparseTableStorageOperator   pico-ps/operator/StorageOperator.h:48-158
//   SparseTablePullOperator      pico-ps/operator/SparsePullOperator.h:48-346
//   SparseTablePushOperator      pico-ps/operator/SparsePushOperator.h:60-464   (async, sync, store)
//   DirectPushOperator           pico-ps/operator/SparsePushOperator.h:479-654  (overwrite; load / reshard / restore)
//   DenseTablePull/PushOperator  pico-ps/operator/DensePullOperator.h, DensePushOperator.h (slice keys)
//   ForEachOperator / EraseIfOperator   pico-ps/operator/ForEachOperator.h, EraseIfOperator.h
//   DumpOperator / LoadOperator / RestoreOperator   pico-ps/operator/{Dump,Load,Restore}Operator.h
//   ShardUpdateContextOperator   pico-ps/operator/UpdateContextOperator.h
//   KVSyncOperator               pico-ps/operator/SyncOperator.h
//   UDFOperator                  pico-ps/operator/UDFOperator.h
//
// Request / response bodies keep the content of the reference's messages (Appendix: sparse pull =
// {i32 shards_num, i32 merge_num, {i32 shard_id, {i32 n_keys, KEY[n]}}}, response = {i32 shards_num,
// shard ids, values}); the encoding is this build's Archive. The user hooks of the reference
// (init_store_value, store_push_value, ...) are the configured optimizer / initialiser functors.
#pragma once
#include <dirent.h>
#include <sys/stat.h>

#include <cmath>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <functional>
#include <map>
#include <set>
#include <string>
#include <vector>

#include "../common/archive.h"
#include "../common/compress.h"
#include "../common/easy_hash_map.h"
#include "../common/filesystem.h"
#include "../common/message.h"
#include "../service/context.h"
#include "operator.h"

namespace psb {

// ---------------------------------------------------------------------------------------------------
inline int opt_type_from_name(const std::string& n) {
    if (n == "sgd") return OPT_SGD;
    if (n == "adagrad") return OPT_ADAGRAD;
    if (n == "ftrl") return OPT_FTRL;
    if (n == "adam" || n == "adamw") return OPT_ADAM;
    if (n == "sum") return OPT_SUM;
    if (n == "set") return OPT_SET;
    return -1;
}

inline Status parse_opt_config(const Json& c, OptConfig* o) {
    std::string name = c.has("optimizer") ? c.at("optimizer").as_string() : "sgd";
    int t = opt_type_from_name(name);
    if (t < 0) return Status::InvalidConfig("unknown optimizer " + name);
    o->type = t;
    if (t == OPT_ADAGRAD) o->eps = 1e-10f;
    auto f = [&](const char* k, float& dst) { if (c.has(k)) dst = (float)c.at(k).as_double(); };
    f("lr", o->lr); f("eps", o->eps); f("l1", o->l1); f("l2", o->l2); f("alpha", o->alpha); f("beta", o->beta);
    f("beta1", o->beta1); f("beta2", o->beta2); f("weight_decay", o->weight_decay);
    f("slot_init0", o->slot_init0); f("slot_init1", o->slot_init1); f("init_accumulator", o->slot_init0);
    return Status::Ok();
}

// ---------------------------------------------------------------------------------------------------
class SparseTableStorageOperator : public Operator {
public:
    explicit SparseTableStorageOperator(const Json& c) : Operator(c) {
        Status st = parse_opt_config(c, &opt_);
        if (!st.ok()) throw std::runtime_error(st.msg());
        const int64_t dim = c.at("dim").as_int(16);
        if (dim < 1 || dim > 65536) throw std::runtime_error("dim must be between 1 and 65536, not " + std::to_string(dim));
        dim_ = (uint32_t)dim;
        // key -> shard: "hash" (the default: jump-consistent hash of the mixed key), "dense" (slices of dense values,
        // hash % N) or "modulo" (key mod N, for tables whose keys are laid out by their producer - the custom
        // partitioner of the reference's predictor test family, pico-ps/test/TestPredictorOps.h:52-64)
        const std::string part = c.at("partition").as_string();
        if (!part.empty() && part != "hash" && part != "dense" && part != "modulo") throw std::runtime_error("unknown partition '" + part + "'");
        partition_ = part == "dense" ? 1 : (part == "modulo" ? 2 : 0);
        if (partition_ == 1 && !c.has("init_range")) init_range_ = 0.f;
        else init_range_ = c.has("init_range") ? (float)c.at("init_range").as_double() : 0.01f;
    }
    const char* kind() const override { return "storage"; }
    uint32_t dim() const { return dim_; }
    const OptConfig& opt() const { return opt_; }
    int partition() const { return partition_; }
    int shard_of(int64_t key, int32_t n_shards) const {
        if (partition_ == 1) return dense_shard_of(key >> 24, (int32_t)(key & 0xFFFFFF), n_shards);
        if (partition_ == 2) return modulo_shard_of(key, n_shards);
        return sparse_shard_of(key, n_shards);
    }
    HostTableConfig table_config(int32_t n_shards) const {
        HostTableConfig h;
        h.dim = dim_;
        h.opt_type = opt_.type;
        h.sync_delta = config_.at("sync").as_bool(false);
        h.n_shards = n_shards;
        h.partition = partition_;
        h.init_seed = (uint64_t)config_.at("seed").as_int(0);
        h.init_range = init_range_;
        h.slot_init0 = opt_.slot_init0;
        h.slot_init1 = opt_.slot_init1;
        h.soft_limit_bytes = h.hard_limit_bytes = (uint64_t)config_.at("memory_limit").as_int(0);
        // Index sizing, under the plain names or under the reference's sections `pool_hash_map` (its default
        // storage) and `google_dense_hash_map` (pico-ps/storage/KVShardStorage.h:439-456,880-897); the pool section
        // wins where both are given, as it does there.
        const Json& pool = config_.at("pool_hash_map");
        const Json& gdh = config_.at("google_dense_hash_map");
        h.expected_max_items = (uint64_t)std::max<int64_t>(0, config_.at("expected_max_items").as_int(
            pool.at("expected_max_items").as_int(gdh.at("expected_max_items").as_int(0))));
        h.index_grow_ratio = config_.at("grow_ratio").as_double(pool.at("grow_ratio").as_double(gdh.at("grow_ratio").as_double(0.0)));
        h.index_shrink_ratio = config_.at("shrink_ratio").as_double(gdh.at("shrink_ratio").as_double(0.0));
        return h;
    }
    // Whether this node's saved image of the table outlives the table's deletion. The reference's persistent-memory
    // storage keeps or removes its pool when it is destroyed by `pmem_create_storage.retain_dcpmm_data_after_deconstruction`
    // (pico-ps/storage/DCPmemory.h:355-365,378-385); the `storage_id` of that section is filled in by the server there
    // and here alike, so a value given by the user is ignored.
    bool retain_local_image() const {
        return config_.at("retain_local_image").as_bool(
            config_.at("pmem_create_storage").at("retain_dcpmm_data_after_deconstruction").as_int(0) != 0);
    }
    // Server side: build the storage and create the local shards.
    Status create_storage(int32_t n_shards, const std::set<int32_t>& local_shards, std::unique_ptr<KVStorage>* out) const {
        const std::string backend = config_.has("backend") ? config_.at("backend").as_string() : "host";
        if (backend == "gpu") {
            GpuKVStorageConfig g;
            g.device = (int)config_.at("device").as_int(0);
            g.base = table_config(n_shards);
            g.capacity = (uint64_t)config_.at("capacity").as_int(1 << 20);
            g.max_batch = (uint32_t)config_.at("max_batch").as_int(1 << 18);
            g.max_rows = (uint64_t)std::max<int64_t>(0, config_.at("max_rows").as_int(0));   // fixed size: no index growth
            PSB_RETURN_IF_ERROR(make_gpu_kv_storage(g, out));
        } else if (backend == "host") {
            out->reset(new HostKVStorage(table_config(n_shards)));
        } else {
            return Status::InvalidConfig("unknown storage backend " + backend);
        }
        for (int32_t s : local_shards) PSB_RETURN_IF_ERROR((*out)->create_shard(s));
        return Status::Ok();
    }

private:
    OptConfig opt_;
    uint32_t dim_ = 16;
    int partition_ = 0;
    float init_range_ = 0.01f;
};

inline const SparseTableStorageOperator* storage_op_of(const TableEntry& e) {
    return static_cast<const SparseTableStorageOperator*>(e.storage_op.get());
}

// ---------------------------------------------------------------------------------------------------
struct NodeRequests {
    std::map<int, Archive> body;              // node id -> request body
    std::map<int, std::vector<int32_t>> shards;  // node id -> shard ids in the order they were written
};

struct PullRequestData {
    size_t n = 0;
    uint32_t n_uniq = 0;
    std::vector<uint32_t> inverse;                 // position -> unique id
    std::map<int32_t, std::vector<int64_t>> shard_keys;
    std::map<int32_t, std::vector<uint32_t>> shard_uid;
    std::vector<float> uniq_rows;                  // n_uniq * dim
    int32_t global_shard_num = 0;                  // the partitioning these lists were built under
};

class SparseTablePullOperator : public Operator {
public:
    explicit SparseTablePullOperator(const Json& c) : Operator(c) {
        read_only_ = c.at("read_only").as_bool(false);
        // how a replica is picked for a shard: uniformly at random per request, the only policy there is
        // (`node_selection`, pico-ps/service/Context.cpp:176-192)
        if (c.has("node_selection") && c.at("node_selection").as_string() != "random")
            throw std::runtime_error("node_selection: only \"random\" is supported");
        max_merge_ = (int)std::max<int64_t>(1, c.at("max_request_merge_num").as_int(32));
    }
    const char* kind() const override { return "pull"; }
    bool read_only() const { return read_only_; }
    // how many requests of sibling threads one message may carry (`max_request_merge_num`,
    // pico-ps/operator/SparsePullOperator.h:71-73); 1 switches merging off
    int max_request_merge_num() const { return max_merge_; }

    // ---- client ----
    // dedup + partition (HOT LOOP A of the reference)
    void generate_request_data(const TableEntry& e, const int64_t* keys, size_t n, PullRequestData* d) const {
        const auto* sop = storage_op_of(e);
        const int32_t G = e.rt.global_shard_num();
        EasyHashMap<int64_t, uint32_t> whole(kHostEmptyKey, n);
        d->n = n;
        d->n_uniq = 0;
        d->global_shard_num = G;
        d->inverse.resize(n);
        d->shard_keys.clear();
        d->shard_uid.clear();
        for (size_t i = 0; i < n; ++i) {
            auto r = whole.try_emplace(keys[i], d->n_uniq);
            if (r.second) {
                int32_t s = sop->shard_of(keys[i], G);
                d->shard_keys[s].push_back(keys[i]);
                d->shard_uid[s].push_back(d->n_uniq);
                ++d->n_uniq;
            }
            d->inverse[i] = r.first->second;
        }
        d->uniq_rows.assign((size_t)d->n_uniq * sop->dim(), 0.f);
    }
    // one request per node, one random live replica per shard
    Status generate_requests(const TableEntry& e, const PullRequestData& d, NodeRequests* out) const {
        std::map<int, std::vector<int32_t>> by_node;
        for (auto& kv : d.shard_keys) {
            int node = e.rt.pick_one_replica(kv.first);
            if (node < 0) return Status::NoReplica("no live replica of shard " + std::to_string(kv.first));
            by_node[node].push_back(kv.first);
        }
        for (auto& kv : by_node) {
            Archive& ar = out->body[kv.first];
            ar << (int32_t)kv.second.size() << (int32_t)1;
            for (int32_t s : kv.second) {
                const auto& ks = d.shard_keys.at(s);
                ar << s << (int32_t)ks.size();
                ar.write_raw(ks.data(), ks.size() * 8);
            }
            out->shards[kv.first] = kv.second;
        }
        return Status::Ok();
    }
    // Several threads' requests in one message per node (request coalescing): the node's shard list is the
    // union over the merged requests, every shard carries one key list per merged request (possibly empty).
    Status generate_merged_requests(const TableEntry& e, const std::vector<PullRequestData*>& ds, NodeRequests* out) const {
        std::map<int32_t, int> shard_node;
        for (auto* d : ds) {
            if (d->global_shard_num != e.rt.global_shard_num())
                return Status::ServerTooNewCtx("the context changed while pull requests were being merged");
            for (auto& kv : d->shard_keys) shard_node.emplace(kv.first, -1);
        }
        std::map<int, std::vector<int32_t>> by_node;
        for (auto& kv : shard_node) {
            int node = e.rt.pick_one_replica(kv.first);
            if (node < 0) return Status::NoReplica("no live replica of shard " + std::to_string(kv.first));
            by_node[node].push_back(kv.first);
        }
        static const std::vector<int64_t> none;
        for (auto& kv : by_node) {
            Archive& ar = out->body[kv.first];
            ar << (int32_t)kv.second.size() << (int32_t)ds.size();
            for (int32_t s : kv.second) {
                ar << s;
                for (auto* d : ds) {
                    auto it = d->shard_keys.find(s);
                    const auto& ks = it == d->shard_keys.end() ? none : it->second;
                    ar << (int32_t)ks.size();
                    ar.write_raw(ks.data(), ks.size() * 8);
                }
            }
            out->shards[kv.first] = kv.second;
        }
        return Status::Ok();
    }
    Status apply_merged_response(const TableEntry& e, const std::vector<PullRequestData*>& ds, Archive& resp) const {
        const uint32_t dim = storage_op_of(e)->dim();
        int32_t shards_num = 0;
        resp >> shards_num;
        std::vector<int32_t> ids(shards_num);
        for (auto& s : ids) resp >> s;
        std::vector<float> tmp;
        for (int32_t s : ids)
            for (auto* d : ds) {
                auto it = d->shard_uid.find(s);
                if (it == d->shard_uid.end()) continue;
                tmp.resize(it->second.size() * dim);
                resp.read_raw(tmp.data(), tmp.size() * 4);
                for (size_t j = 0; j < it->second.size(); ++j)
                    std::copy_n(tmp.data() + j * dim, dim, d->uniq_rows.data() + (size_t)it->second[j] * dim);
            }
        return Status::Ok();
    }
    Status apply_response(const TableEntry& e, PullRequestData* d, Archive& resp) const {
        const uint32_t dim = storage_op_of(e)->dim();
        int32_t shards_num = 0;
        resp >> shards_num;
        std::vector<int32_t> ids(shards_num);
        for (auto& s : ids) resp >> s;
        std::vector<float> tmp;
        for (int32_t s : ids) {
            auto it = d->shard_uid.find(s);
            if (it == d->shard_uid.end()) return Status::Error("pull response for a shard that was not requested");
            tmp.resize(it->second.size() * dim);
            resp.read_raw(tmp.data(), tmp.size() * 4);
            for (size_t j = 0; j < it->second.size(); ++j)
                std::copy_n(tmp.data() + j * dim, dim, d->uniq_rows.data() + (size_t)it->second[j] * dim);
        }
        return Status::Ok();
    }
    // un-dedup (HOT LOOP C): one row per original key position
    void fill_pull_items(const TableEntry& e, const PullRequestData& d, float* out) const {
        const uint32_t dim = storage_op_of(e)->dim();
        for (size_t i = 0; i < d.n; ++i) std::copy_n(d.uniq_rows.data() + (size_t)d.inverse[i] * dim, dim, out + i * dim);
    }

    // ---- server (HOT LOOP B) ----
    Status apply_request(TableEntry& e, Archive& req, Archive* resp) const {
        KVStorage* st = e.storage.get();
        if (!read_only_ && !st->healthy()) return Status::OOM("storage unhealthy");
        const uint32_t dim = st->dim();
        int32_t shards_num = 0, merge_num = 0;
        req >> shards_num >> merge_num;
        // counts come from the wire: each shard carries at least an id and merge_num list lengths
        if (merge_num < 0 || !req.can_hold(shards_num, 4 + (size_t)merge_num * 4)) return Status::Error("pull: malformed request");
        std::vector<int32_t> ids;
        std::vector<std::vector<float>> vals;
        for (int32_t i = 0; i < shards_num; ++i) {
            int32_t s = 0;
            req >> s;
            ids.push_back(s);
            vals.emplace_back();
            for (int32_t m = 0; m < merge_num; ++m) {
                int32_t n = 0;
                req >> n;
                if (!req.can_hold(n, 8)) return Status::Error("pull: malformed request");
                const int64_t* keys = (const int64_t*)req.cursor_ptr();
                std::vector<int64_t> aligned(keys, keys + n);  // archive bytes may be unaligned
                req.skip((size_t)n * 8);
                size_t off = vals.back().size();
                vals.back().resize(off + (size_t)n * dim);
                PSB_RETURN_IF_ERROR(st->pull(s, aligned.data(), (size_t)n, vals.back().data() + off, !read_only_));
            }
        }
        *resp << shards_num;
        for (int32_t s : ids) *resp << s;
        for (auto& v : vals) resp->write_raw(v.data(), v.size() * 4);
        return Status::Ok();
    }

private:
    bool read_only_ = false;
    int max_merge_ = 32;
};

// ---------------------------------------------------------------------------------------------------
// What a push has achieved so far, kept across the retries of ONE push call so that a retry resends only what
// no server applied. A push fans out to several nodes; when some of them apply it and another refuses (it
// already switched to a newer context, or it blocks writes during a reshard) the reference resends the whole
// request and the first nodes apply it twice. Here a (shard, node) pair that answered OK is never sent again, a
// node that was a target and did not answer OK is retried while it still holds the shard, and a node that
// received the shard through a reshard in between is skipped: the rows it was given already contain the update.
struct PushAckState {
    int32_t G = -1;
    std::map<int32_t, std::set<int>> targeted, acked;
    void reset(int32_t g) {
        G = g;
        targeted.clear();
        acked.clear();
    }
    bool wants(int32_t shard, int node) const {
        auto a = acked.find(shard);
        if (a == acked.end() || a->second.empty()) return true;
        if (a->second.count(node)) return false;
        auto t = targeted.find(shard);
        return t != targeted.end() && t->second.count(node) > 0;
    }
    void record(int32_t shard, int node, bool ok) {
        targeted[shard].insert(node);
        if (ok) acked[shard].insert(node);
    }
};

struct PushRequestData {
    std::map<int32_t, std::vector<int64_t>> shard_keys;
    std::map<int32_t, std::vector<float>> shard_grads;
    int32_t global_shard_num = 0;  // the partitioning these lists were built under
};

class SparseTablePushOperator : public Operator {
public:
    explicit SparseTablePushOperator(const Json& c) : Operator(c) {
        has_opt_ = c.has("optimizer");
        if (has_opt_) {
            Status st = parse_opt_config(c, &opt_);
            if (!st.ok()) throw std::runtime_error(st.msg());
        }
        // tables (of this or of another cluster) that follow this one: what pushes change here is shipped to them
        // by the server's sync thread (pico-ps/operator/PushOperator.h:45-55)
        if (c.has("sync_table"))
            for (auto& t : c.at("sync_table").elements())
                sync_tables_.push_back({t.at("model_name").as_string(), t.at("table_name").as_string(), t.at("op_key").as_string()});
        max_merge_ = (int)std::max<int64_t>(1, c.at("max_request_merge_num").as_int(32));
    }
    int max_request_merge_num() const { return max_merge_; }   // see SparseTablePullOperator
    struct SyncTarget {
        std::string model_name, table_name, op_key;
    };
    const std::vector<SyncTarget>& sync_tables() const { return sync_tables_; }
    const char* kind() const override { return "push"; }
    OptConfig opt_for(const TableEntry& e) const { return has_opt_ ? opt_ : storage_op_of(e)->opt(); }

    // ---- client: pre-aggregate duplicates, partition (HOT LOOP D) ----
    void generate_request_data(const TableEntry& e, const int64_t* keys, const float* grads, size_t n,
                               PushRequestData* d) const {
        const auto* sop = storage_op_of(e);
        const uint32_t dim = sop->dim();
        const int32_t G = e.rt.global_shard_num();
        EasyHashMap<int64_t, uint32_t> whole(kHostEmptyKey, n);
        std::vector<int64_t> uk;
        std::vector<float> agg;
        for (size_t i = 0; i < n; ++i) {
            auto r = whole.try_emplace(keys[i], (uint32_t)uk.size());
            if (r.second) {
                uk.push_back(keys[i]);
                agg.resize(agg.size() + dim, 0.f);
            }
            float* a = agg.data() + (size_t)r.first->second * dim;
            for (uint32_t k = 0; k < dim; ++k) a[k] += grads[i * dim + k];
        }
        d->shard_keys.clear();
        d->shard_grads.clear();
        d->global_shard_num = G;
        for (size_t u = 0; u < uk.size(); ++u) {
            int32_t s = sop->shard_of(uk[u], G);
            d->shard_keys[s].push_back(uk[u]);
            auto& g = d->shard_grads[s];
            g.insert(g.end(), agg.data() + u * dim, agg.data() + (u + 1) * dim);
        }
    }
    // every node that hosts a touched shard gets that shard's items (all replicas are updated)
    Status generate_requests(const TableEntry& e, const PushRequestData& d, NodeRequests* out,
                             const PushAckState* ack = nullptr) const {
        std::map<int, std::vector<int32_t>> by_node;
        for (auto& kv : d.shard_keys) {
            auto it = e.rt.shards().find(kv.first);
            if (it == e.rt.shards().end() || it->second.empty())
                return Status::NoReplica("no live holder of shard " + std::to_string(kv.first));
            for (int node : it->second)
                if (ack == nullptr || ack->wants(kv.first, node)) by_node[node].push_back(kv.first);
        }
        for (auto& kv : by_node) {
            Archive& ar = out->body[kv.first];
            ar << (int32_t)kv.second.size() << (int32_t)1;
            for (int32_t s : kv.second) {
                const auto& ks = d.shard_keys.at(s);
                const auto& gs = d.shard_grads.at(s);
                ar << s << (int32_t)ks.size();
                ar.write_raw(ks.data(), ks.size() * 8);
                ar.write_raw(gs.data(), gs.size() * 4);
            }
            out->shards[kv.first] = kv.second;
        }
        return Status::Ok();
    }

    // Several threads' pushes in one message per node: the node's shard list is the union over the merged
    // requests, every shard carries one item list per merged request (possibly empty).
    // `acks[i]` (may be null) filters what member i still has to send; `sent[i]` receives the (node, shard) pairs
    // that carry member i's items in this message set.
    Status generate_merged_requests(const TableEntry& e, const std::vector<PushRequestData*>& ds,
                                    const std::vector<PushAckState*>& acks, NodeRequests* out,
                                    std::vector<std::vector<std::pair<int, int32_t>>>* sent) const {
        std::map<int, std::set<int32_t>> by_node;
        sent->assign(ds.size(), {});
        for (size_t i = 0; i < ds.size(); ++i) {
            if (ds[i]->global_shard_num != e.rt.global_shard_num())
                return Status::ServerTooNewCtx("the context changed while push requests were being merged");
            for (auto& kv : ds[i]->shard_keys) {
                auto it = e.rt.shards().find(kv.first);
                if (it == e.rt.shards().end() || it->second.empty())
                    return Status::NoReplica("no live holder of shard " + std::to_string(kv.first));
                for (int node : it->second)
                    if (acks[i] == nullptr || acks[i]->wants(kv.first, node)) {
                        by_node[node].insert(kv.first);
                        (*sent)[i].push_back({node, kv.first});
                    }
            }
        }
        for (auto& kv : by_node) {
            const int node = kv.first;
            Archive& ar = out->body[node];
            ar << (int32_t)kv.second.size() << (int32_t)ds.size();
            for (int32_t s : kv.second) {
                ar << s;
                for (size_t i = 0; i < ds.size(); ++i) {
                    auto it = ds[i]->shard_keys.find(s);
                    const bool include = it != ds[i]->shard_keys.end() && (acks[i] == nullptr || acks[i]->wants(s, node));
                    if (!include) {
                        ar << (int32_t)0;
                        continue;
                    }
                    const auto& gs = ds[i]->shard_grads.at(s);
                    ar << (int32_t)it->second.size();
                    ar.write_raw(it->second.data(), it->second.size() * 8);
                    ar.write_raw(gs.data(), gs.size() * 4);
                }
            }
            out->shards[node] = std::vector<int32_t>(kv.second.begin(), kv.second.end());
        }
        return Status::Ok();
    }

    // ---- server (HOT LOOP E / the queueing half of F) ----
    Status apply_request(TableEntry& e, Archive& req, bool sync) const {
        KVStorage* st = e.storage.get();
        if (!st->healthy()) return Status::OOM("storage unhealthy");
        const uint32_t dim = st->dim();
        const OptConfig opt = opt_for(e);
        int32_t shards_num = 0, merge_num = 0;
        req >> shards_num >> merge_num;
        if (merge_num < 0 || !req.can_hold(shards_num, 4 + (size_t)merge_num * 4)) return Status::Error("push: malformed request");
        std::shared_lock<std::shared_mutex> ig(e.incr.mu);
        for (int32_t i = 0; i < shards_num; ++i) {
            int32_t s = 0;
            req >> s;
            for (int32_t m = 0; m < merge_num; ++m) {
                int32_t n = 0;
                req >> n;
                if (!req.can_hold(n, 8 + (size_t)dim * 4)) return Status::Error("push: malformed request");
                std::vector<int64_t> keys((size_t)n);
                std::vector<float> grads((size_t)n * dim);
                req.read_raw(keys.data(), (size_t)n * 8);
                req.read_raw(grads.data(), grads.size() * 4);
                PSB_RETURN_IF_ERROR(st->push(s, keys.data(), grads.data(), (size_t)n, opt, sync));
            }
        }
        e.incr.updated = true;
        return Status::Ok();
    }
    // OP_STORE: fold what sync pushes buffered (the merging half of HOT LOOP F)
    Status apply_store(TableEntry& e) const {
        std::shared_lock<std::shared_mutex> ig(e.incr.mu);
        e.incr.updated = true;
        return e.storage->store(opt_for(e));
    }

private:
    bool has_opt_ = false;
    OptConfig opt_;
    std::vector<SyncTarget> sync_tables_;
    int max_merge_ = 32;
};

// ---------------------------------------------------------------------------------------------------
// DirectPush: records {key, full row} overwrite / insert. Used by load (rehash), reshard shuffle, sync.
class DirectPushOperator : public Operator {
public:
    explicit DirectPushOperator(const Json& c) : Operator(c) {}
    const char* kind() const override { return "direct_push"; }

    // Partition records by the owners under runtime info `rt` (all holders of a shard receive it).
    static Status generate_requests(const SparseTableStorageOperator* sop, const RuntimeInfo& rt, const int64_t* keys,
                                    const float* rows, size_t n, uint32_t stride, std::map<int, Archive>* out) {
        const int32_t G = rt.global_shard_num();
        std::map<int, std::pair<std::vector<int64_t>, std::vector<float>>> per_node;
        for (size_t i = 0; i < n; ++i) {
            int32_t s = sop->shard_of(keys[i], G);
            auto it = rt.shards().find(s);
            if (it == rt.shards().end() || it->second.empty())
                return Status::NoReplica("direct push: no holder of shard " + std::to_string(s));
            for (int node : it->second) {
                auto& p = per_node[node];
                p.first.push_back(keys[i]);
                p.second.insert(p.second.end(), rows + i * stride, rows + (i + 1) * stride);
            }
        }
        for (auto& kv : per_node) {
            Archive& ar = (*out)[kv.first];
            ar << (int32_t)kv.second.first.size() << (int32_t)stride;
            ar.write_raw(kv.second.first.data(), kv.second.first.size() * 8);
            ar.write_raw(kv.second.second.data(), kv.second.second.size() * 4);
        }
        return Status::Ok();
    }
    // Server: write into `dst` (the serving storage, or the update storage during a reshard).
    static Status apply_request(KVStorage* dst, Archive& req) {
        int32_t n = 0, stride = 0;
        req >> n >> stride;
        if ((uint32_t)stride != dst->stride() && (uint32_t)stride != dst->dim())
            return Status::Error("direct push: record width does not match the table");
        if (!req.can_hold(n, 8 + (size_t)stride * 4)) return Status::Error("direct push: malformed request");
        std::vector<int64_t> keys((size_t)n);
        std::vector<float> rows((size_t)n * stride);
        req.read_raw(keys.data(), (size_t)n * 8);
        req.read_raw(rows.data(), rows.size() * 4);
        return dst->set_rows(keys.data(), rows.data(), (size_t)n, (uint32_t)stride == dst->dim() && dst->dim() != dst->stride());
    }
};

// ---------------------------------------------------------------------------------------------------
// Dense tables: a dense value (tensor `id` of `numel` floats) is cut into slices of `dim` floats
// (DenseValuePartitioner), slice j has key (id << 24) | j and lives on shard hash(id, j) % G; pull
// reassembles (DenseValueMerger). The sparse machinery above does the rest.
struct DenseSlice {
    int64_t key;     // (id << 24) | slice index
    size_t offset;   // first element of the dense value held by this slice
    uint32_t len;    // elements of the value in this slice (<= the table's slice width)
};
// The default cut: consecutive slices of `slice_len` elements.
// A dense key is (id << 24) | slice: 2^24 slices per value and ids of 39 bits and a sign. What does not fit would land
// on another value's keys (or on a reserved key), so it is refused before anything is sent.
inline Status dense_check_id(int64_t id, size_t numel, uint32_t slice_len) {
    constexpr int64_t kIdLimit = 1LL << 39;
    if (id <= -kIdLimit || id >= kIdLimit) return Status::InvalidConfig("dense id " + std::to_string(id) + " does not fit 40 bits");
    if (slice_len == 0 || (numel + slice_len - 1) / slice_len > (size_t)(1 << 24))
        return Status::InvalidConfig("a dense value of " + std::to_string(numel) + " elements needs more than 2^24 slices of " + std::to_string(slice_len));
    return Status::Ok();
}
inline void dense_default_partition(int64_t id, size_t numel, uint32_t slice_len, std::vector<DenseSlice>* out) {
    const size_t ns = (numel + slice_len - 1) / slice_len;
    out->resize(ns);
    for (size_t j = 0; j < ns; ++j)
        (*out)[j] = DenseSlice{(id << 24) | (int64_t)j, j * slice_len, (uint32_t)std::min<size_t>(slice_len, numel - j * slice_len)};
}
inline void dense_slice_keys(int64_t id, size_t numel, uint32_t slice_len, std::vector<int64_t>* keys) {
    std::vector<DenseSlice> sl;
    dense_default_partition(id, numel, slice_len, &sl);
    keys->resize(sl.size());
    for (size_t j = 0; j < sl.size(); ++j) (*keys)[j] = sl[j].key;
}

// The two customisation points of dense tables (pico-ps/common/dense_common.h:135-171): a subclass registered by a
// plug-in may cut a value differently (DenseValuePartitioner::partition) and reassemble it differently
// (DenseValueMerger::merge), e.g. to keep rows of a matrix together or to interleave for balance. Pull and push
// operators of one table must agree on the cut.
class DenseTablePullOperator : public SparseTablePullOperator {
public:
    explicit DenseTablePullOperator(const Json& c) : SparseTablePullOperator(c) {}
    virtual void partition(int64_t id, size_t numel, uint32_t slice_len, std::vector<DenseSlice>* out) const {
        dense_default_partition(id, numel, slice_len, out);
    }
    // Place one pulled slice (slice_len floats, the first `len` meaningful) into the reassembled value.
    virtual void merge(const DenseSlice& s, const float* slice_values, float* value) const {
        std::copy_n(slice_values, s.len, value + s.offset);
    }
};
class DenseTablePushOperator : public SparseTablePushOperator {
public:
    explicit DenseTablePushOperator(const Json& c) : SparseTablePushOperator(c) {}
    virtual void partition(int64_t id, size_t numel, uint32_t slice_len, std::vector<DenseSlice>* out) const {
        dense_default_partition(id, numel, slice_len, out);
    }
    // Fill one slice to push (slice_len floats, zero padded) from the dense gradient.
    virtual void extract(const DenseSlice& s, const float* value, float* slice_values) const {
        std::copy_n(value + s.offset, s.len, slice_values);
    }
};

// ---------------------------------------------------------------------------------------------------
// for_each: a per-shard scan that folds every entry into a result; results merge associatively on the client.
// The three hooks are the extension points of the reference (init_result / for_each / merge_result,
// pico-ps/operator/ForEachOperator.h:214-232, :340-358): a plug-in library registers a subclass under its own
// (lib, class) name and the server runs it. A result travels as bytes whose layout only the operator knows.
class ForEachOperatorBase : public Operator {
public:
    explicit ForEachOperatorBase(const Json& c) : Operator(c) {}
    const char* kind() const override { return "for_each"; }
    // The empty result (the neutral element of merge_result).
    virtual std::string init_result(const Json& carried) const = 0;
    // Fold one entry (key, full row of `stride` floats whose first `dim` are the embedding) into *result.
    virtual void for_each(int64_t key, const float* row, uint32_t dim, uint32_t stride, const Json& carried,
                          std::string* result) const = 0;
    // *out = merge(*out, in); must be associative and commutative (shards answer in any order).
    virtual void merge_result(const std::string& in, std::string* out) const = 0;
    // Whether the scan changes rows (ForEachWriteOperatorBase): the client then sends it to every holder of a shard,
    // so that replicas stay alike, and counts the answer of one of them.
    virtual bool writes() const { return false; }

    // Server half: the scan of one shard. The default walks the shard in windows and calls for_each per entry.
    virtual Status apply_request(TableEntry& e, int32_t shard, const Json& carried, std::string* result) const {
        KVStorage* st = e.storage.get();
        const uint32_t dim = st->dim(), stride = st->stride();
        *result = init_result(carried);
        return st->scan_shard(
            shard, 1 << 16, false,
            [&](const std::vector<int64_t>& keys, const std::vector<float>& rows) {
                for (size_t i = 0; i < keys.size(); ++i) for_each(keys[i], rows.data() + i * stride, dim, stride, carried, result);
                return Status::Ok();
            },
            [&] { *result = init_result(carried); });
    }
};

// The built-in reducer: count, sum, sum of squares and max |x| over one row section (`carried` may hold
// {"section": 0|1|2}: 0 = embedding, 1 / 2 = optimizer slots).
struct ForEachResult {
    uint64_t count = 0;
    double sum = 0, sum_sq = 0, max_abs = 0;
    void merge(const ForEachResult& o) {
        count += o.count;
        sum += o.sum;
        sum_sq += o.sum_sq;
        max_abs = std::max(max_abs, o.max_abs);
    }
    std::string pack() const { return std::string((const char*)this, sizeof(*this)); }
    static bool unpack(const std::string& s, ForEachResult* r) {
        if (s.size() != sizeof(ForEachResult)) return false;
        std::memcpy(r, s.data(), sizeof(ForEachResult));
        return true;
    }
};

class ForEachOperator : public ForEachOperatorBase {
public:
    explicit ForEachOperator(const Json& c) : ForEachOperatorBase(c) {}
    std::string init_result(const Json&) const override { return ForEachResult().pack(); }
    void for_each(int64_t, const float* row, uint32_t dim, uint32_t stride, const Json& carried, std::string* result) const override {
        const uint32_t section = (uint32_t)carried.at("section").as_int(0);
        if ((section + 1) * dim > stride) return;
        ForEachResult* r = (ForEachResult*)&(*result)[0];
        ++r->count;
        const float* v = row + section * dim;
        for (uint32_t k = 0; k < dim; ++k) {
            r->sum += v[k];
            r->sum_sq += (double)v[k] * v[k];
            r->max_abs = std::max(r->max_abs, (double)std::fabs(v[k]));
        }
    }
    void merge_result(const std::string& in, std::string* out) const override {
        ForEachResult a, b;
        if (!ForEachResult::unpack(in, &a) || !ForEachResult::unpack(*out, &b)) return;
        b.merge(a);
        *out = b.pack();
    }
    // The built-in reduction runs where the rows are when the storage can do that (GPU tables: one kernel over the
    // slot array, four numbers come back); otherwise the generic host scan.
    Status apply_request(TableEntry& e, int32_t shard, const Json& carried, std::string* result) const override {
        KVStorage* st = e.storage.get();
        const uint32_t section = (uint32_t)carried.at("section").as_int(0);
        if ((section + 1) * st->dim() > st->stride()) return Status::InvalidConfig("for_each: no such row section");
        ScanStats s;
        Status status;
        if (st->reduce_builtin(shard, section, &s, &status)) {
            PSB_RETURN_IF_ERROR(status);
            ForEachResult r;
            r.count = s.count; r.sum = s.sum; r.sum_sq = s.sum_sq; r.max_abs = s.max_abs;
            *result = r.pack();
            return Status::Ok();
        }
        return ForEachOperatorBase::apply_request(e, shard, carried, result);
    }
};

// The writing scan (SparseTableForEachWriteOperator, pico-ps/operator/ForEachOperator.h:277-359): for_each_write may
// change the row it is shown and folds something into the result as the reading scan does. A host shard is updated in
// place under its write lock; rows marked for the incremental sync are marked by it as well.
class ForEachWriteOperatorBase : public ForEachOperatorBase {
public:
    explicit ForEachWriteOperatorBase(const Json& c) : ForEachOperatorBase(c) {}
    bool writes() const final { return true; }
    // Returns whether it changed `row` (stride floats: embedding, optimizer slots, pending delta).
    virtual bool for_each_write(int64_t key, float* row, uint32_t dim, uint32_t stride, const Json& carried,
                                std::string* result) const = 0;
    void for_each(int64_t, const float*, uint32_t, uint32_t, const Json&, std::string*) const final {}
    // Checked once per request before the scan.
    virtual Status check_carried(const KVStorage&, const Json&) const { return Status::Ok(); }
    Status apply_request(TableEntry& e, int32_t shard, const Json& carried, std::string* result) const override {
        KVStorage* st = e.storage.get();
        PSB_RETURN_IF_ERROR(check_carried(*st, carried));
        const uint32_t dim = st->dim(), stride = st->stride();
        *result = init_result(carried);
        std::shared_lock<std::shared_mutex> ig(e.incr.mu);   // like a push: not while the increment is collected
        uint64_t changed = 0;
        Status status = st->update_shard(
            shard, 1 << 16, [&](int64_t key, float* row) { return for_each_write(key, row, dim, stride, carried, result); }, &changed);
        if (changed) e.incr.updated = true;
        return status;
    }
};

// The built-in writing scans, chosen by the carried item; `section` 0 = embedding, 1 / 2 = optimizer slots:
//   {"type":"scale","factor":f} | {"type":"clip","limit":c} (to [-c, c]) | {"type":"fill","value":v}
// The result is the statistics record of the reading scan over the section AFTER the write, counted over the rows
// that changed.
class ForEachWriteOperator : public ForEachWriteOperatorBase {
public:
    explicit ForEachWriteOperator(const Json& c) : ForEachWriteOperatorBase(c) {}
    std::string init_result(const Json&) const override { return ForEachResult().pack(); }
    Status check_carried(const KVStorage& st, const Json& carried) const override {
        const std::string type = carried.at("type").as_string();
        if (type != "scale" && type != "clip" && type != "fill") return Status::InvalidConfig("for_each (write): unknown type '" + type + "'");
        const int64_t section = carried.at("section").as_int(0);
        if (section < 0 || (uint64_t)(section + 1) * st.dim() > st.stride()) return Status::InvalidConfig("for_each (write): no such row section");
        if (type == "clip" && carried.at("limit").as_double(-1) < 0) return Status::InvalidConfig("for_each (write): clip needs a limit >= 0");
        return Status::Ok();
    }
    bool for_each_write(int64_t, float* row, uint32_t dim, uint32_t, const Json& carried, std::string* result) const override {
        const std::string type = carried.at("type").as_string();
        float* v = row + (size_t)carried.at("section").as_int(0) * dim;
        bool changed = false;
        auto put = [&](uint32_t k, float x) {
            if (std::memcmp(&v[k], &x, sizeof(float)) != 0) changed = true;
            v[k] = x;
        };
        if (type == "scale") {
            const float f = (float)carried.at("factor").as_double(1.0);
            for (uint32_t k = 0; k < dim; ++k) put(k, v[k] * f);
        } else if (type == "clip") {
            const float c = (float)carried.at("limit").as_double(0.0);
            for (uint32_t k = 0; k < dim; ++k) put(k, std::min(c, std::max(-c, v[k])));
        } else {
            const float x = (float)carried.at("value").as_double(0.0);
            for (uint32_t k = 0; k < dim; ++k) put(k, x);
        }
        if (changed) {
            ForEachResult* r = (ForEachResult*)&(*result)[0];
            ++r->count;
            for (uint32_t k = 0; k < dim; ++k) {
                r->sum += v[k];
                r->sum_sq += (double)v[k] * v[k];
                r->max_abs = std::max(r->max_abs, (double)std::fabs(v[k]));
            }
        }
        return changed;
    }
    void merge_result(const std::string& in, std::string* out) const override {
        ForEachResult a, b;
        if (!ForEachResult::unpack(in, &a) || !ForEachResult::unpack(*out, &b)) return;
        b.merge(a);
        *out = b.pack();
    }
};

// erase_if: exclusive per-shard scan; entries for which the predicate holds are erased
// (pico-ps/operator/EraseIfOperator.h:39-58: `virtual bool erase_if(key, value) = 0`). A plug-in subclass supplies
// its own predicate; it is evaluated on the host over the exported rows of the shard.
class EraseIfOperatorBase : public Operator {
public:
    explicit EraseIfOperatorBase(const Json& c) : Operator(c) {}
    const char* kind() const override { return "erase_if"; }
    virtual bool erase_if(int64_t key, const float* row, uint32_t dim, uint32_t stride, const Json& carried) const = 0;
    // Checked once per request before the scan (bad carried items are refused, not ignored).
    virtual Status check_carried(const KVStorage&, const Json&) const { return Status::Ok(); }
    virtual Status apply_request(TableEntry& e, int32_t shard, const Json& carried, uint64_t* erased) const {
        KVStorage* st = e.storage.get();
        PSB_RETURN_IF_ERROR(check_carried(*st, carried));
        const uint32_t dim = st->dim(), stride = st->stride();
        // the doomed keys are collected during the scan and erased after it: the scan holds the shard for reading
        std::vector<int64_t> doomed;
        PSB_RETURN_IF_ERROR(st->scan_shard(
            shard, 1 << 16, false,
            [&](const std::vector<int64_t>& keys, const std::vector<float>& rows) {
                for (size_t i = 0; i < keys.size(); ++i)
                    if (erase_if(keys[i], rows.data() + i * stride, dim, stride, carried)) doomed.push_back(keys[i]);
                return Status::Ok();
            },
            [&] { doomed.clear(); }));
        *erased = 0;
        if (!doomed.empty()) PSB_RETURN_IF_ERROR(st->erase_keys(doomed.data(), doomed.size(), erased));
        return Status::Ok();
    }
};

// The built-in predicates, chosen by the carried item:
//   {"type":"key_mod","mod":m,"rem":r} | {"type":"l2_below","threshold":t} | {"type":"slot0_below","threshold":t}
//   | {"type":"all"}
class EraseIfOperator : public EraseIfOperatorBase {
public:
    explicit EraseIfOperator(const Json& c) : EraseIfOperatorBase(c) {}
    static bool parse(const Json& carried, ScanPredicate* p) {
        const std::string type = carried.at("type").as_string();
        if (type == "key_mod") p->type = ScanPredicate::KEY_MOD;
        else if (type == "l2_below") p->type = ScanPredicate::L2_BELOW;
        else if (type == "slot0_below") p->type = ScanPredicate::SLOT0_BELOW;
        else if (type == "all") p->type = ScanPredicate::ALL;
        else return false;
        p->mod = carried.at("mod").as_int(2);
        p->rem = carried.at("rem").as_int(1);
        p->threshold = carried.at("threshold").as_double(0);
        return true;
    }
    Status check_carried(const KVStorage& st, const Json& carried) const override {
        ScanPredicate p;
        if (!parse(carried, &p)) return Status::InvalidConfig("erase_if: unknown predicate " + carried.at("type").as_string());
        if (p.type == ScanPredicate::KEY_MOD && p.mod == 0) return Status::InvalidConfig("erase_if key_mod: mod must not be 0");
        if (p.type == ScanPredicate::SLOT0_BELOW && st.stride() < 2 * st.dim())
            return Status::InvalidConfig("erase_if slot0_below: table has no optimizer slot");
        return Status::Ok();
    }
    bool erase_if(int64_t key, const float* v, uint32_t dim, uint32_t, const Json& carried) const override {
        ScanPredicate p;
        if (!parse(carried, &p)) return false;
        switch (p.type) {
            case ScanPredicate::KEY_MOD: return ((key % p.mod) + p.mod) % p.mod == p.rem;
            case ScanPredicate::ALL: return true;
            case ScanPredicate::L2_BELOW: {
                double s = 0;
                for (uint32_t k = 0; k < dim; ++k) s += (double)v[k] * v[k];
                return std::sqrt(s) < p.threshold;
            }
            case ScanPredicate::SLOT0_BELOW: {
                double s = 0;
                for (uint32_t k = 0; k < dim; ++k) s += v[dim + k];
                return s / dim < p.threshold;
            }
        }
        return false;
    }
    // Built-in predicates are evaluated where the rows are when the storage can do that.
    Status apply_request(TableEntry& e, int32_t shard, const Json& carried, uint64_t* erased) const override {
        KVStorage* st = e.storage.get();
        PSB_RETURN_IF_ERROR(check_carried(*st, carried));
        ScanPredicate p;
        parse(carried, &p);
        Status status;
        *erased = 0;
        if (st->erase_if_builtin(shard, p, erased, &status)) return status;
        return EraseIfOperatorBase::apply_request(e, shard, carried, erased);
    }
};

// ---------------------------------------------------------------------------------------------------
// Dump / load file codec. Layout rules are the reference's (pico-ps/operator/DumpOperator.h:72-83,156):
// directory <uri>, files model_<node_id>_<file_id>, shard -> file by shard_id % file_number, one record
// per entry {key, value}. Record encodings ("?format=" option of the uri):
//   binary      : header "PSB1" u32 stride | records: i64 key, stride * fp32         (default)
//   archiveline : one text line per record: key \t v0 v1 ... (%.9g round-trips fp32 bit for bit)
// With a compress_algorithm the whole file body is one compressed block.
struct DumpArgs {
    std::string uri;
    int32_t file_number = 1;
    static void split_uri(const std::string& uri, std::string* path, std::string* format) {
        auto q = uri.find('?');
        *path = uri.substr(0, q);
        *format = "binary";
        if (q != std::string::npos) {
            auto f = uri.find("format=", q);
            if (f != std::string::npos) {
                auto end = uri.find('&', f);
                *format = uri.substr(f + 7, end == std::string::npos ? std::string::npos : end - f - 7);
            }
        }
    }
};

// Local paths or a Hadoop file system behind the `hadoop fs` command: common/filesystem.h.
inline Status mkdir_p(const std::string& path) { return fs::mkdir_p(path); }

inline std::vector<std::string> list_model_files(const std::string& dir) { return fs::list(dir, "model_"); }

class DsWriter {
public:
    DsWriter(std::string path, std::string format, uint32_t stride, const Compressor* comp)
        : path_(std::move(path)), format_(std::move(format)), stride_(stride), comp_(comp) {
        if (format_ == "binary") {
            body_.insert(body_.end(), {'P', 'S', 'B', '1'});
            const uint8_t* p = (const uint8_t*)&stride_;
            body_.insert(body_.end(), p, p + 4);
        }
    }
    void write(int64_t key, const float* row) {
        if (format_ == "binary") {
            const uint8_t* k = (const uint8_t*)&key;
            body_.insert(body_.end(), k, k + 8);
            const uint8_t* r = (const uint8_t*)row;
            body_.insert(body_.end(), r, r + (size_t)stride_ * 4);
        } else {
            char buf[32];
            int m = std::snprintf(buf, sizeof buf, "%lld\t", (long long)key);
            body_.insert(body_.end(), buf, buf + m);
            for (uint32_t i = 0; i < stride_; ++i) {
                m = std::snprintf(buf, sizeof buf, i + 1 == stride_ ? "%.9g\n" : "%.9g ", row[i]);
                body_.insert(body_.end(), buf, buf + m);
            }
        }
    }
    Status close() {
        std::vector<uint8_t> out;
        if (comp_ && comp_->enabled()) PSB_RETURN_IF_ERROR(comp_->compress(body_.data(), body_.size(), &out));
        else out.swap(body_);
        return fs::write_file(path_, out);
    }

private:
    std::string path_, format_;
    uint32_t stride_;
    const Compressor* comp_;
    std::vector<uint8_t> body_;
};

// Reads a whole file and hands out records in blocks.
class DsReader {
public:
    Status open(const std::string& path, const std::string& format, uint32_t stride, const Compressor* comp) {
        std::vector<uint8_t> raw;
        PSB_RETURN_IF_ERROR(fs::read_file(path, &raw));
        if (comp && comp->enabled()) PSB_RETURN_IF_ERROR(comp->decompress(raw.data(), raw.size(), &body_));
        else body_.swap(raw);
        format_ = format;
        stride_ = stride;
        pos_ = 0;
        size_ = body_.size();
        bad_ = false;
        body_.push_back(0);  // the text parser (strtoll / strtof) needs a terminator behind the last byte
        if (format_ == "binary") {
            if (size_ < 8 || std::memcmp(body_.data(), "PSB1", 4) != 0) return Status::Error(path + ": not a PSB1 dump file");
            uint32_t s;
            std::memcpy(&s, body_.data() + 4, 4);
            if (s != stride) return Status::Error(path + ": record width differs from the table");
            pos_ = 8;
        }
        return Status::Ok();
    }
    // Up to `block` records; returns false when the file is exhausted (or damaged: see ok()).
    bool next_block(size_t block, std::vector<int64_t>* keys, std::vector<float>* rows) {
        keys->clear();
        rows->clear();
        while (keys->size() < block && pos_ < size_) {
            if (format_ == "binary") {
                if (8 + (size_t)stride_ * 4 > size_ - pos_) {  // a record cut short: the file was truncated
                    bad_ = true;
                    pos_ = size_;
                    break;
                }
                int64_t k;
                std::memcpy(&k, body_.data() + pos_, 8);
                keys->push_back(k);
                size_t off = rows->size();
                rows->resize(off + stride_);
                std::memcpy(rows->data() + off, body_.data() + pos_ + 8, (size_t)stride_ * 4);
                pos_ += 8 + (size_t)stride_ * 4;
            } else {
                const char* base = (const char*)body_.data();
                const char* p = base + pos_;
                char* end = nullptr;
                long long k = std::strtoll(p, &end, 10);
                bool good = end != p;
                std::vector<float> row(stride_);
                for (uint32_t i = 0; good && i < stride_; ++i) {
                    const char* q = end;
                    row[i] = std::strtof(q, &end);
                    good = end != q && (size_t)(end - base) <= size_;
                }
                if (!good) {  // not a record: stop instead of looping on the same bytes
                    bad_ = true;
                    pos_ = size_;
                    break;
                }
                keys->push_back(k);
                rows->insert(rows->end(), row.begin(), row.end());
                while ((size_t)(end - base) < size_ && (*end == '\n' || *end == '\r')) ++end;
                pos_ = (size_t)(end - base);
            }
        }
        return !keys->empty();
    }
    // False once a truncated or unparsable record was met; what was returned before it is valid.
    bool ok() const { return !bad_; }

private:
    std::vector<uint8_t> body_;
    std::string format_;
    uint32_t stride_ = 0;
    size_t pos_ = 0, size_ = 0;
    bool bad_ = false;
};

class DumpOperator : public Operator {
public:
    explicit DumpOperator(const Json& c) : Operator(c) {
        Status st = Compressor::create(c.at("compress_algorithm").as_string(), &comp_);
        if (!st.ok()) throw std::runtime_error(st.msg());
    }
    const char* kind() const override { return "dump"; }
    // Server: write the local shards that map to file `file_id` into <uri>/model_<node>_<file_id>.
    Status apply_request(TableEntry& e, int node_id, const DumpArgs& args, int32_t file_id, const std::vector<int32_t>& shards,
                         uint64_t* n_records) const {
        std::string dir, format;
        DumpArgs::split_uri(args.uri, &dir, &format);
        if (dir.empty()) return Status::InvalidConfig("dump: the uri names no directory");   // never "/model_..." by accident
        PSB_RETURN_IF_ERROR(mkdir_p(dir));
        KVStorage* st = e.storage.get();
        DsWriter w(dir + "/model_" + std::to_string(node_id) + "_" + std::to_string(file_id), format, st->stride(), &comp_);
        *n_records = 0;
        // every shard is written as one snapshot: its writers wait while it is read, as under the write lock that
        // the reference holds per shard (pico-ps/operator/DumpOperator.h:170-190)
        for (int32_t s : shards) {
            PSB_RETURN_IF_ERROR(st->scan_shard(s, 1 << 16, false, [&](const std::vector<int64_t>& keys, const std::vector<float>& rows) {
                for (size_t i = 0; i < keys.size(); ++i) w.write(keys[i], rows.data() + i * st->stride());
                *n_records += keys.size();
                return Status::Ok();
            }));
        }
        return w.close();
    }
    const Compressor& compressor() const { return comp_; }

private:
    Compressor comp_;
};

class LoadOperator : public Operator {
public:
    explicit LoadOperator(const Json& c) : Operator(c) {
        Status st = Compressor::create(c.at("compress_algorithm").as_string(), &comp_);
        if (!st.ok()) throw std::runtime_error(st.msg());
        block_size_ = (size_t)c.at("block_size").as_int(1000);
    }
    const char* kind() const override { return "load"; }
    size_t block_size() const { return block_size_; }
    const Compressor& compressor() const { return comp_; }
    // restore (no rehash): read `file`, keep the records whose shard is local.
    Status restore_file(TableEntry& e, const std::string& file, const std::string& format, uint64_t* kept) const {
        KVStorage* st = e.storage.get();
        DsReader r;
        PSB_RETURN_IF_ERROR(r.open(file, format, st->stride(), &comp_));
        std::vector<int64_t> keys;
        std::vector<float> rows;
        while (r.next_block(block_size_, &keys, &rows)) {
            PSB_RETURN_IF_ERROR(st->set_rows(keys.data(), rows.data(), keys.size(), false));  // foreign keys are skipped
            for (int64_t k : keys) *kept += st->has_shard(st->shard_of(k)) ? 1 : 0;
        }
        return r.ok() ? Status::Ok() : Status::Error(file + ": damaged dump file (a record is cut short or does not parse)");
    }

private:
    Compressor comp_;
    size_t block_size_ = 1000;
};

class RestoreOperator : public LoadOperator {
public:
    explicit RestoreOperator(const Json& c) : LoadOperator(c) {}
    const char* kind() const override { return "restore"; }
};

// Reshard codec (pico-ps/operator/UpdateContextOperator.h:59-309): the server half of the update-context
// transaction is owned by this operator, so a table may replace it with a subclass registered by a plug-in:
//   create_new_shards        the storage that receives shuffled items on a node of the NEW placement (:136-141)
//   generate_shuffle_requests which items of an old shard travel, in blocks of at most block_serialized_size bytes,
//                            addressed to their owners under the new placement (PushItemsGenerator, :215-304)
//   apply_purge_request      after the commit: drop what no longer belongs here, re-apply what waited for memory
//                            (:143-193)
class ShardUpdateContextOperator : public Operator {
public:
    // Sends one block of per-node DirectPush bodies over s2s and waits for the owners' answers.
    using SendBlock = std::function<Status(const std::map<int, Archive>&)>;

    explicit ShardUpdateContextOperator(const Json& c) : Operator(c) {
        block_bytes_ = (size_t)c.at("block_serialized_size").as_int(1000000);
    }
    const char* kind() const override { return "update_ctx"; }
    size_t block_bytes() const { return block_bytes_; }

    virtual Status create_new_shards(TableEntry& e) const {
        if (e.update_rt.local_shards().empty()) return Status::Ok();  // this node leaves the table
        PSB_RETURN_IF_ERROR(storage_op_of(e)->create_storage(e.update_rt.global_shard_num(), e.update_rt.local_shards(),
                                                             &e.update_storage));
        // a followed table keeps recording changes across the reshard: rows that move are marked on arrival, so what
        // was still waiting to be shipped on their old owner is not lost (some rows are shipped twice instead)
        if (e.sync_enabled) e.update_storage->enable_dirty_tracking();
        return Status::Ok();
    }

    virtual Status generate_shuffle_requests(TableEntry& e, int32_t old_shard, const SendBlock& send) const {
        if (!e.storage || !e.storage->has_shard(old_shard)) return Status::InvalidID("shuffle: shard is not on this node");
        const uint32_t stride = e.storage->stride();
        const uint64_t window = std::max<uint64_t>(64, block_bytes_ / (8 + (size_t)stride * 4));
        const auto* sop = storage_op_of(e);
        uint64_t cursor = 0;
        bool finished = false;
        std::vector<int64_t> keys;
        std::vector<float> rows;
        auto ship = [&]() -> Status {
            if (keys.empty()) return Status::Ok();
            std::map<int, Archive> bodies;
            PSB_RETURN_IF_ERROR(DirectPushOperator::generate_requests(sop, e.update_rt, keys.data(), rows.data(), keys.size(),
                                                                      stride, &bodies));
            return send(bodies);
        };
        while (!finished) {
            keys.clear();
            rows.clear();
            PSB_RETURN_IF_ERROR(e.storage->export_shard(old_shard, cursor, window, false, &keys, &rows, &cursor, &finished));
            PSB_RETURN_IF_ERROR(ship());
        }
        // pushed items that were waiting for memory on this node travel as rows too: the new owners may have room
        keys.clear();
        rows.clear();
        e.storage->overflow_rows(old_shard, &keys, &rows);
        return ship();
    }

    virtual Status apply_purge_request(TableEntry& e) const {
        e.update_storage.reset();
        if (e.storage) {
            for (int s : e.storage->shard_list())
                if (!e.rt.local_shards().count(s)) e.storage->erase_shard(s);
            e.storage->set_healthy(true);
            e.storage->drain_overflow();   // what waited for memory is applied now that shards have left
        }
        return Status::Ok();
    }

private:
    size_t block_bytes_;
};

class KVSyncOperator : public Operator {
public:
    explicit KVSyncOperator(const Json& c) : Operator(c) {
        block_size_ = (size_t)c.at("block_size").as_int(1000);
        Status st = Compressor::create(c.at("compress_algorithm").as_string(), &comp_);
        if (!st.ok()) throw std::runtime_error(st.msg());
    }
    const char* kind() const override { return "sync"; }
    size_t block_size() const { return block_size_; }
    const Compressor& compressor() const { return comp_; }

private:
    size_t block_size_;
    Compressor comp_;
};

// UDF: named server-side functions. apply(entry, param bytes) -> result bytes. Functions are registered
// in a process-wide table (C++ or, through the bindings, Python callables).
class UDFRegistry {
public:
    using Fn = std::function<Status(TableEntry&, const std::string& param, std::string* result)>;
    static UDFRegistry& instance() {
        static UDFRegistry r;
        return r;
    }
    void add(const std::string& name, Fn f) {
        std::lock_guard<std::mutex> g(mu_);
        fns_[name] = std::move(f);
    }
    bool get(const std::string& name, Fn* f) {
        std::lock_guard<std::mutex> g(mu_);
        auto it = fns_.find(name);
        if (it == fns_.end()) return false;
        *f = it->second;
        return true;
    }

private:
    std::mutex mu_;
    std::map<std::string, Fn> fns_;
};

class UDFOperator : public Operator {
public:
    explicit UDFOperator(const Json& c) : Operator(c) {
        fn_ = c.at("function").as_string();
        read_only_ = c.at("read_only").as_bool(true);
    }
    const char* kind() const override { return "udf"; }
    bool read_only() const { return read_only_; }
    Status apply_request(TableEntry& e, const std::string& param, std::string* result) const {
        UDFRegistry::Fn f;
        if (!UDFRegistry::instance().get(fn_, &f)) return Status::InvalidConfig("udf: no function named " + fn_);
        return f(e, param, result);
    }

private:
    std::string fn_;
    bool read_only_ = true;
};

// Registers every built-in operator under lib name "psb" (idempotent).
void register_builtin_operators();

}  // namespace psb
