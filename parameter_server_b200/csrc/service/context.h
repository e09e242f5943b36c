// Context: storage id -> table entry (descriptor, runtime view, storages, operators), each behind
// its own reader/writer lock.
//
// Parity: pico-ps/service/Context.{h,cpp} (CreateStorage, reader / writer guards, update_runtime_info,
// update_handlers) and the per-table members of TableDescriptor that are not metadata
// (storage / update_storage / incr_storage / handlers, pico-ps/service/TableDescriptor.h:103-130).
// The same class serves the client (no storages, node id -1) and the server.
#pragma once
#include <atomic>
#include <map>
#include <memory>
#include <mutex>
#include <shared_mutex>
#include <string>

#include "../operator/operator.h"
#include "../storage/kv_storage.h"
#include "table_descriptor.h"

namespace psb {

// Double-buffered record of what changed since the last incremental sync
// (pico-ps/service/IncrementStorage.h:11-43): writers mark under a shared lock, the reader flips.
// With both back-ends the dirty marks live next to the rows (one bit / byte per row); this object
// serialises "collect + clear" against concurrent pushes.
struct IncrementStorage {
    std::shared_mutex mu;
    std::atomic<bool> updated{false};  // set by concurrent pushes under the shared lock
};

struct RestoreIterator {
    int shard = -1;
    uint64_t cursor = 0;
    uint64_t epoch = 0;   // KVStorage::layout_epoch of the shard when the cursor was taken
};

struct TableEntry {
    int32_t sid = -1;
    TableDescriptor td;
    RuntimeInfo rt, update_rt;
    std::shared_ptr<Operator> storage_op;
    std::unique_ptr<KVStorage> storage;         // serving data
    std::unique_ptr<KVStorage> update_storage;  // receives shuffled items during a reshard
    IncrementStorage incr;
    std::atomic<bool> sync_enabled{false};      // changed rows are being recorded for follower tables
    std::mutex sync_mu;                         // serialises switching the recording on
    std::map<int32_t, std::shared_ptr<Operator>> ops;  // handler id -> operator
    std::map<int32_t, RestoreIterator> restore_iters;
    int32_t next_iter_id = 0;
    std::mutex iter_mu;
    mutable std::shared_mutex mu;  // table-descriptor lock (reader: data ops, writer: metadata changes)

    Status update_handlers() {
        // instantiate operators for descriptors that have none yet, drop the ones that disappeared
        for (auto it = ops.begin(); it != ops.end();)
            it = td.handlers.count(it->first) ? std::next(it) : ops.erase(it);
        for (auto& kv : td.handlers) {
            if (ops.count(kv.first)) continue;
            std::shared_ptr<Operator> op;
            PSB_RETURN_IF_ERROR(OperatorFactory::instance().create(kv.second.lib_name, kv.second.op_name,
                                                                   kv.second.config_str, &op));
            ops[kv.first] = op;
        }
        return Status::Ok();
    }
};

class Context {
public:
    std::shared_ptr<TableEntry> get(int32_t sid) const {
        std::shared_lock<std::shared_mutex> g(mu_);
        auto it = tables_.find(sid);
        return it == tables_.end() ? nullptr : it->second;
    }
    // Build an entry from a storage config {nodes:[...], op_config:{...}}.
    Status create_storage(int32_t sid, const std::string& lib, const std::string& op_name, const Json& cfg, int my_node_id,
                          std::shared_ptr<TableEntry>* out) {
        auto e = std::make_shared<TableEntry>();
        e->sid = sid;
        PSB_RETURN_IF_ERROR(TableDescriptor::parse_nodes(cfg.at("nodes"), &e->td.nodes));
        e->td.storage_op = OperatorDescriptor{"storage", lib, op_name, cfg.at("op_config").dump()};
        e->td.table_name = cfg.at("table_name").as_string();
        // the creator's identity of the data layout travels in the config, so that every process holds the same one
        if (cfg.has("version_uuid") && !cfg.at("version_uuid").as_string().empty()) e->td.version_uuid = cfg.at("version_uuid").as_string();
        else e->td.gen_new_version_uuid();
        e->td.refresh_info();
        PSB_RETURN_IF_ERROR(OperatorFactory::instance().create(lib, op_name, e->td.storage_op.config_str, &e->storage_op));
        e->rt.build(e->td, my_node_id);
        std::unique_lock<std::shared_mutex> g(mu_);
        tables_[sid] = e;
        *out = e;
        return Status::Ok();
    }
    // Install / refresh an entry from the JSON published on the master.
    Status set_table_descriptor(int32_t sid, const std::string& json, int my_node_id, std::shared_ptr<TableEntry>* out) {
        std::shared_ptr<TableEntry> e = get(sid);
        bool fresh = false;
        if (!e) {
            e = std::make_shared<TableEntry>();
            e->sid = sid;
            fresh = true;
        }
        {
            std::unique_lock<std::shared_mutex> tg(e->mu);
            Json j;
            if (!Json::parse(json, &j)) return Status::Error("context JSON does not parse");
            e->td.from_json(j, !fresh);
            e->rt.build(e->td, my_node_id);
            e->update_rt.build(e->td, my_node_id, true);
            if (!e->storage_op)
                PSB_RETURN_IF_ERROR(OperatorFactory::instance().create(e->td.storage_op.lib_name, e->td.storage_op.op_name,
                                                                       e->td.storage_op.config_str, &e->storage_op));
            PSB_RETURN_IF_ERROR(e->update_handlers());
        }
        if (fresh) {
            std::unique_lock<std::shared_mutex> g(mu_);
            tables_[sid] = e;
        }
        if (out) *out = e;
        return Status::Ok();
    }
    void erase(int32_t sid) {
        std::unique_lock<std::shared_mutex> g(mu_);
        tables_.erase(sid);
    }
    std::vector<int32_t> ids() const {
        std::shared_lock<std::shared_mutex> g(mu_);
        std::vector<int32_t> v;
        for (auto& kv : tables_) v.push_back(kv.first);
        return v;
    }

private:
    mutable std::shared_mutex mu_;
    std::map<int32_t, std::shared_ptr<TableEntry>> tables_;
};

}  // namespace psb
