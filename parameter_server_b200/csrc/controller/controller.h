// Controller: the single-threaded operations tool - placement, table life cycle, rebalancing, shard and
// replica resizing, node expansion and shutdown, introspection as JSON.
//
// Parity: pico-ps/controller/Controller.{h,cpp}: load_nodes from the RPC registry (:56-68), placement
// = least shard count with a random tie-break, `replica_num` distinct lowest-loaded nodes per shard
// (:188-199, :294-301), create_table (:280-350), delete_table (:368-405), balance_table (:407-441),
// update_table_shard / update_table_replica (:443-478), update_table through the handler registered
// under key "update_ctx" (:486-522), expand_nodes / expand_storage_nodes (append `local_shard_num`
// shards per new node; single-replica tables only, :545-596), clean_unused_storage (:524-543),
// shutdown_node, show_node(s) / gen_table_json (:643-733).
#pragma once
#include <random>

#include "../handler/handlers.h"
#include "../model/model.h"

namespace psb {

struct OpSpec {
    std::string key, lib, op, config;
};

class Controller {
public:
    explicit Controller(const std::string& master_addr) : client_(master_addr), rng_(std::random_device{}()) {}
    Client& client() { return client_; }

    // The usual operator set of a sparse table, under the keys that the tools look handlers up by.
    static std::vector<OpSpec> standard_ops(const std::string& compress = "", int block_size = 1000) {
        const std::string c = "{\"compress_algorithm\":\"" + compress + "\",\"block_size\":" + std::to_string(block_size) + "}";
        return {{"pull", "psb", "SparseTablePullOperator", "{}"},
                {"pull_ro", "psb", "SparseTablePullOperator", "{\"read_only\":true}"},
                {"push", "psb", "SparseTablePushOperator", "{}"},
                {"for_each", "psb", "ForEachOperator", "{}"},
                {"erase_if", "psb", "EraseIfOperator", "{}"},
                {"dump", "psb", "DumpOperator", c},
                {"load", "psb", "LoadOperator", c},
                {"update_ctx", "psb", "ShardUpdateContextOperator", "{}"},
                {"sync", "psb", "KVSyncOperator", c}};
    }

    Status load_nodes(std::vector<int>* nodes) {
        std::map<int32_t, std::string> m;
        PSB_RETURN_IF_ERROR(client_.get_pserver_list(&m));
        nodes->clear();
        for (auto& kv : m) nodes->push_back(kv.first);
        return Status::Ok();
    }

    // Least-loaded placement: returns [{g_rank, shard_list}] JSON for `shard_num` shards x `replica_num`.
    Status place(int shard_num, int replica_num, const std::vector<int>& nodes, std::map<int, double> load, Json* out) {
        if (nodes.empty()) return Status::Error("no pserver is registered");
        if (replica_num > (int)nodes.size()) return Status::InvalidConfig("replica_num exceeds the number of nodes");
        std::uniform_real_distribution<double> tie(0.0, 1.0);
        for (int n : nodes) load[n] += tie(rng_);  // init_weight = shard_num + U(0,1)
        std::map<int, std::vector<int>> assign;
        for (int s = 0; s < shard_num; ++s) {
            std::vector<int> order(nodes);
            std::sort(order.begin(), order.end(), [&](int a, int b) { return load[a] < load[b]; });
            for (int r = 0; r < replica_num; ++r) {
                assign[order[r]].push_back(s);
                load[order[r]] += 1.0;
            }
        }
        *out = nodes_json(assign);
        return Status::Ok();
    }

    Status create_table(const std::string& table_name, const std::string& lib, const std::string& storage_op,
                        const std::string& op_config_json, int shard_num, int replica_num, const std::vector<OpSpec>& ops,
                        const std::string& table_uri, int32_t* sid) {
        std::vector<int> nodes;
        PSB_RETURN_IF_ERROR(load_nodes(&nodes));
        Json placement;
        PSB_RETURN_IF_ERROR(place(shard_num, replica_num, nodes, current_load(), &placement));
        Json op_cfg;
        if (!Json::parse_config(op_config_json.empty() ? "{}" : op_config_json, &op_cfg)) return Status::InvalidConfig("op_config parses neither as JSON nor as YAML");
        Json cfg = Json::object();
        cfg["nodes"] = placement;
        cfg["op_config"] = op_cfg;
        cfg["table_name"] = table_name;
        PSB_RETURN_IF_ERROR(client_.create_storage(lib, storage_op, cfg.dump(), sid));
        TableObject tobj;
        tobj.table_name = table_name; tobj.table_uri = table_uri; tobj.lib_name = lib; tobj.shard_num = shard_num;
        tobj.replica_num = replica_num; tobj.storage_id = *sid;
        tobj.storage_op = OperatorObject{"storage", lib, storage_op, op_cfg.dump(), -1};
        for (auto& o : ops) {
            int32_t hid = -1;
            PSB_RETURN_IF_ERROR(client_.register_handler(o.key, o.lib, o.op, o.config, *sid, &hid));
            tobj.ops.push_back(OperatorObject{o.key, o.lib, o.op, o.config, hid});
        }
        if (!table_uri.empty()) PSB_RETURN_IF_ERROR(client_.set_table_uri(*sid, table_uri));
        return client_.master().tree_node_set("table/" + std::to_string(*sid), tobj.to_json().dump());
    }
    Status delete_table(int32_t sid) {
        client_.master().tree_node_del("table/" + std::to_string(sid));
        return client_.delete_storage(sid);
    }

    // Re-place the table evenly over the live nodes (same shard / replica numbers).
    Status balance_table(int32_t sid) {
        int shards = 0, replicas = 1;
        PSB_RETURN_IF_ERROR(table_shape(sid, &shards, &replicas));
        return replace_table(sid, shards, replicas);
    }
    Status update_table_shard(int32_t sid, int shard_num) {
        int shards = 0, replicas = 1;
        PSB_RETURN_IF_ERROR(table_shape(sid, &shards, &replicas));
        return replace_table(sid, shard_num, replicas);
    }
    Status update_table_replica(int32_t sid, int replica_num) {
        int shards = 0, replicas = 1;
        PSB_RETURN_IF_ERROR(table_shape(sid, &shards, &replicas));
        return replace_table(sid, shards, replica_num);
    }
    // Run the reshard transaction with an explicit placement.
    Status update_table(int32_t sid, const std::string& nodes_json) {
        PSB_RETURN_IF_ERROR(client_.initialize_storage(sid));
        int32_t hid = -1;
        PSB_RETURN_IF_ERROR(client_.handler_by_key(sid, "update_ctx", &hid));
        UpdateContextHandler h(&client_, sid, hid);
        return h.update_context(nodes_json);
    }
    // The abort path of update_table for an operator: a table that a dead client left in the middle of a reshard (status
    // RESHARD: writes are refused) - or closed by a restore that never finished - goes back to its last published
    // placement, the half-built shards are dropped, writes resume (UpdateContextHandler::purge,
    // pico-ps/handler/UpdateContextHandler.cpp:279-298).
    Status purge_table(int32_t sid) {
        PSB_RETURN_IF_ERROR(client_.initialize_storage(sid));
        int32_t hid = -1;
        PSB_RETURN_IF_ERROR(client_.handler_by_key(sid, "update_ctx", &hid));
        UpdateContextHandler h(&client_, sid, hid);
        return h.purge();
    }
    // Data operations of a table created with the standard operator set, for the command line: the handlers are found
    // by their keys ("dump", "load", "for_each", "erase_if").
    Status dump_table(int32_t sid, const std::string& uri, int file_number, uint64_t* n_records) {
        PSB_RETURN_IF_ERROR(client_.initialize_storage(sid));
        int32_t hid = -1;
        PSB_RETURN_IF_ERROR(client_.handler_by_key(sid, "dump", &hid));
        DumpArgs args;
        args.uri = uri;
        args.file_number = file_number;
        return DumpHandler(&client_, sid, hid).dump(args, n_records);
    }
    Status load_table(int32_t sid, const std::string& uri, uint64_t* n_records) {
        PSB_RETURN_IF_ERROR(client_.initialize_storage(sid));
        int32_t hid = -1;
        PSB_RETURN_IF_ERROR(client_.handler_by_key(sid, "load", &hid));
        return LoadHandler(&client_, sid, hid).load(uri, n_records);
    }
    // count / sum / sum of squares / max |x| over a row section (0 = embedding, 1 / 2 = optimizer slots)
    Status table_stats(int32_t sid, int section, Json* out) {
        PSB_RETURN_IF_ERROR(client_.initialize_storage(sid));
        int32_t hid = -1;
        PSB_RETURN_IF_ERROR(client_.handler_by_key(sid, "for_each", &hid));
        ForEachResult r;
        PSB_RETURN_IF_ERROR(ForEachHandler(&client_, sid, hid).for_each("{\"section\":" + std::to_string(section) + "}", &r));
        *out = Json::object();
        (*out)["count"] = (int64_t)r.count;
        (*out)["sum"] = r.sum;
        (*out)["sum_sq"] = r.sum_sq;
        (*out)["max_abs"] = r.max_abs;
        return Status::Ok();
    }
    // `carried_json`: a built-in predicate, e.g. {"type":"slot0_below","threshold":0.2}
    Status erase_from_table(int32_t sid, const std::string& carried_json, uint64_t* erased) {
        PSB_RETURN_IF_ERROR(client_.initialize_storage(sid));
        int32_t hid = -1;
        PSB_RETURN_IF_ERROR(client_.handler_by_key(sid, "erase_if", &hid));
        return EraseIfHandler(&client_, sid, hid).erase_if(carried_json, erased);
    }
    // Scale out: every new node gets `local_shard_num` NEW shards appended (single-replica tables only).
    Status expand_storage_nodes(int32_t sid, const std::vector<int>& new_nodes, int local_shard_num) {
        PSB_RETURN_IF_ERROR(client_.initialize_storage(sid));
        auto e = client_.context().get(sid);
        std::map<int, std::vector<int>> assign;
        int next_shard = 0;
        {
            std::shared_lock<std::shared_mutex> g(e->mu);
            for (auto& kv : e->td.shards)
                if (kv.second.size() > 1) return Status::InvalidConfig("expand_storage_nodes refuses replicated tables");
            for (auto& n : e->td.nodes) {
                if (n.status == NodeStatus::DEAD) continue;
                for (int s : n.shard_list) {
                    assign[n.node_id].push_back(s);
                    next_shard = std::max(next_shard, s + 1);
                }
            }
        }
        for (int n : new_nodes) {
            if (assign.count(n)) return Status::InvalidConfig("node " + std::to_string(n) + " already serves the table");
            for (int k = 0; k < local_shard_num; ++k) assign[n].push_back(next_shard++);
        }
        return update_table(sid, nodes_json(assign).dump());
    }
    Status expand_nodes(const std::vector<int>& new_nodes, int local_shard_num) {
        std::vector<std::string> keys;
        PSB_RETURN_IF_ERROR(client_.master().list_contexts(&keys));
        for (auto& k : keys)
            if (k.compare(0, 8, "storage/") == 0) PSB_RETURN_IF_ERROR(expand_storage_nodes(std::stoi(k.substr(8)), new_nodes, local_shard_num));
        return Status::Ok();
    }
    // Contexts whose table object is gone are storages nobody owns any more.
    Status clean_unused_storage(int* removed) {
        *removed = 0;
        std::vector<std::string> keys;
        PSB_RETURN_IF_ERROR(client_.master().list_contexts(&keys));
        for (auto& k : keys) {
            if (k.compare(0, 8, "storage/") != 0) continue;
            int32_t sid = std::stoi(k.substr(8));
            std::string s;
            if (client_.master().tree_node_get("table/" + std::to_string(sid), &s).ok()) continue;
            if (client_.delete_storage(sid).ok()) ++*removed;
        }
        return Status::Ok();
    }
    Status shutdown_node(int node) { return client_.close_pserver(node); }

    Status show_node(int node, Json* out) {
        *out = Json::object();
        (*out)["node_id"] = node;
        NodeMemoryInfo mi;
        Status st = client_.query_memory_info(node, &mi, 2000);
        (*out)["alive"] = st.ok();
        if (st.ok()) {
            (*out)["healthy"] = mi.healthy;
            (*out)["used_bytes"] = (int64_t)mi.used;
        }
        Json tables = Json::array();
        std::vector<std::string> keys;
        PSB_RETURN_IF_ERROR(client_.master().list_contexts(&keys));
        for (auto& k : keys) {
            if (k.compare(0, 8, "storage/") != 0) continue;
            std::string json;
            if (!client_.master().get_context(k, &json).ok()) continue;
            TableDescriptor td;
            td.from_json_str(json);
            for (auto& n : td.nodes)
                if (n.node_id == node) {
                    Json t = Json::object();
                    t["storage_id"] = std::stoi(k.substr(8));
                    t["shard_num"] = (int)n.shard_list.size();
                    t["status"] = (int)n.status;
                    tables.push_back(t);
                }
        }
        (*out)["tables"] = tables;
        return Status::Ok();
    }
    Status show_nodes(Json* out) {
        *out = Json::array();
        std::vector<int> nodes;
        PSB_RETURN_IF_ERROR(load_nodes(&nodes));
        for (int n : nodes) {
            Json j;
            PSB_RETURN_IF_ERROR(show_node(n, &j));
            out->push_back(j);
        }
        return Status::Ok();
    }
    Status gen_table_json(int32_t sid, Json* out) {
        std::string json;
        PSB_RETURN_IF_ERROR(client_.master().get_context(ctx_key(sid), &json));
        Json ctx;
        Json::parse(json, &ctx);
        *out = Json::object();
        (*out)["storage_id"] = sid;
        (*out)["context"] = ctx;
        PSB_RETURN_IF_ERROR(client_.initialize_storage(sid));
        std::vector<StorageStatisticInfo> info;
        if (client_.query_storage_info(sid, &info, 5000).ok()) {
            Json arr = Json::array();
            for (auto& s : info) {
                Json j = Json::object();
                j["node_id"] = s.node_id; j["shard_id"] = s.shard_id; j["item_number"] = (int64_t)s.item_number;
                j["memory_usage"] = (int64_t)s.memory_usage;
                arr.push_back(j);
            }
            (*out)["shards"] = arr;
        }
        return Status::Ok();
    }

private:
    static Json nodes_json(const std::map<int, std::vector<int>>& assign) {
        Json arr = Json::array();
        for (auto& kv : assign) {
            Json n = Json::object();
            n["g_rank"] = kv.first;
            Json sl = Json::array();
            for (int s : kv.second) sl.push_back(Json(s));
            n["shard_list"] = sl;
            arr.push_back(n);
        }
        return arr;
    }
    std::map<int, double> current_load() {
        std::map<int, double> load;
        std::vector<std::string> keys;
        if (!client_.master().list_contexts(&keys).ok()) return load;
        for (auto& k : keys) {
            std::string json;
            if (k.compare(0, 8, "storage/") != 0 || !client_.master().get_context(k, &json).ok()) continue;
            TableDescriptor td;
            td.from_json_str(json);
            for (auto& n : td.nodes) load[n.node_id] += (double)n.shard_list.size();
        }
        return load;
    }
    Status table_shape(int32_t sid, int* shards, int* replicas) {
        PSB_RETURN_IF_ERROR(client_.initialize_storage(sid));
        auto e = client_.context().get(sid);
        std::shared_lock<std::shared_mutex> g(e->mu);
        *shards = e->td.global_shard_num();
        size_t r = 1;
        for (auto& n : e->td.nodes) (void)n;
        std::map<int, int> holders;
        for (auto& n : e->td.nodes)
            for (int s : n.shard_list) ++holders[s];
        for (auto& kv : holders) r = std::max<size_t>(r, (size_t)kv.second);
        *replicas = (int)r;
        return Status::Ok();
    }
    Status replace_table(int32_t sid, int shards, int replicas) {
        std::vector<int> nodes;
        PSB_RETURN_IF_ERROR(load_nodes(&nodes));
        std::map<int, double> load = current_load();
        // the table's own shards do not count against its new placement
        auto e = client_.context().get(sid);
        {
            std::shared_lock<std::shared_mutex> g(e->mu);
            for (auto& n : e->td.nodes) load[n.node_id] -= (double)n.shard_list.size();
        }
        Json placement;
        PSB_RETURN_IF_ERROR(place(shards, replicas, nodes, load, &placement));
        return update_table(sid, placement.dump());
    }

    Client client_;
    std::mt19937 rng_;
};

}  // namespace psb
