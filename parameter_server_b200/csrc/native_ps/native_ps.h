// NativePS: an in-process, single-node parameter server for serving (no RPC, no master): the same
// operators applied directly to local storages.
//
// Parity: pico-ps/native_ps/NativePS.{h,cpp} (local context, local storage ids),
// NativePullHandler (generate -> apply -> response -> fill in the calling thread,
// pico-ps/native_ps/NativePullHandler.cpp:20-36) and NativeLoadHandler (threaded file load through the
// push operator, pico-ps/native_ps/NativeLoadHandler.cpp:22-76).
#pragma once
#include <thread>

#include "../operator/operators.h"

namespace psb {

class NativePS {
public:
    NativePS() { register_builtin_operators(); }
    // All `shard_num` shards are local. op_config as for SparseTableStorageOperator.
    Status create_storage(const std::string& lib, const std::string& op, const std::string& op_config_json, int shard_num,
                          int32_t* sid) {
        Json cfg = Json::object(), opc;
        if (!Json::parse_config(op_config_json.empty() ? "{}" : op_config_json, &opc)) return Status::InvalidConfig("op_config parses neither as JSON nor as YAML");
        Json node = Json::object();
        node["g_rank"] = 0;
        Json sl = Json::array();
        for (int s = 0; s < shard_num; ++s) sl.push_back(Json(s));
        node["shard_list"] = sl;
        Json nodes = Json::array();
        nodes.push_back(node);
        cfg["nodes"] = nodes;
        cfg["op_config"] = opc;
        std::shared_ptr<TableEntry> e;
        *sid = next_sid_++;
        PSB_RETURN_IF_ERROR(ctx_.create_storage(*sid, lib, op, cfg, 0, &e));
        auto* sop = static_cast<SparseTableStorageOperator*>(e->storage_op.get());
        return sop->create_storage(e->rt.global_shard_num(), e->rt.local_shards(), &e->storage);
    }
    Status register_handler(int32_t sid, const std::string& key, const std::string& lib, const std::string& op,
                            const std::string& cfg, int32_t* hid) {
        auto e = ctx_.get(sid);
        if (!e) return Status::InvalidID("unknown storage");
        *hid = next_hid_++;
        e->td.handlers[*hid] = OperatorDescriptor{key, lib, op, cfg};
        e->td.refresh_info();
        return e->update_handlers();
    }
    std::shared_ptr<TableEntry> entry(int32_t sid) { return ctx_.get(sid); }

private:
    Context ctx_;
    int32_t next_sid_ = 0, next_hid_ = 0;
};

class NativePullHandler {
public:
    NativePullHandler(NativePS* ps, int32_t sid, int32_t hid) : ps_(ps), sid_(sid), hid_(hid) {}
    // Width of a pulled row (0 when the storage is unknown): `out` of pull() holds n * dim() floats.
    uint32_t dim() const {
        auto e = ps_->entry(sid_);
        return e && e->storage_op ? storage_op_of(*e)->dim() : 0;
    }
    Status pull(const int64_t* keys, size_t n, float* out) {
        auto e = ps_->entry(sid_);
        if (!e) return Status::InvalidID("unknown storage");
        auto it = e->ops.find(hid_);
        auto p = it == e->ops.end() ? nullptr : std::dynamic_pointer_cast<SparseTablePullOperator>(it->second);
        if (!p) return Status::InvalidID("handler is not a pull operator");
        PullRequestData data;
        NodeRequests reqs;
        p->generate_request_data(*e, keys, n, &data);
        PSB_RETURN_IF_ERROR(p->generate_requests(*e, data, &reqs));
        for (auto& kv : reqs.body) {  // still (de)serialises, like the reference, but never leaves the thread
            Archive req = kv.second, resp;
            PSB_RETURN_IF_ERROR(p->apply_request(*e, req, &resp));
            PSB_RETURN_IF_ERROR(p->apply_response(*e, &data, resp));
        }
        p->fill_pull_items(*e, data, out);
        return Status::Ok();
    }

private:
    NativePS* ps_;
    int32_t sid_, hid_;
};

class NativeLoadHandler {
public:
    NativeLoadHandler(NativePS* ps, int32_t sid, int32_t hid) : ps_(ps), sid_(sid), hid_(hid) {}
    // Loads every model_* file under `uri` with `threads` workers.
    Status load(const std::string& uri, int threads, uint64_t* n_records) {
        auto e = ps_->entry(sid_);
        if (!e) return Status::InvalidID("unknown storage");
        auto it = e->ops.find(hid_);
        auto p = it == e->ops.end() ? nullptr : std::dynamic_pointer_cast<LoadOperator>(it->second);
        if (!p) return Status::InvalidID("handler is not a load operator");
        std::string dir, format;
        DumpArgs::split_uri(uri, &dir, &format);
        std::vector<std::string> files = list_model_files(dir);
        std::atomic<size_t> next{0};
        std::atomic<uint64_t> total{0};
        std::mutex mu;
        Status first;
        std::vector<std::thread> pool;
        for (int t = 0; t < std::max(1, threads); ++t)
            pool.emplace_back([&] {
                for (;;) {
                    size_t i = next++;
                    if (i >= files.size()) return;
                    uint64_t n = 0;
                    Status st = p->restore_file(*e, files[i], format, &n);
                    total += n;
                    if (!st.ok()) {
                        std::lock_guard<std::mutex> g(mu);
                        if (first.ok()) first = st;
                    }
                }
            });
        for (auto& t : pool) t.join();
        *n_records = total;
        return first;
    }

private:
    NativePS* ps_;
    int32_t sid_, hid_;
};

}  // namespace psb
