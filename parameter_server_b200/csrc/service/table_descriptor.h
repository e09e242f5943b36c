// Versioned per-table metadata ("context") shared by clients, servers and the controller through the
// master, and the runtime view derived from it.
//
// Parity: OperatorDescriptor / NodeStatus / StorageStatus / NodeDescriptor / TableDescriptor /
// RuntimeInfo of pico-ps/service/TableDescriptor.h:24-228 with the JSON layout of
// pico-ps/service/TableDescriptor.cpp:132-157:
//   {version, update_version, version_uuid, table_uri, table_name, status,
//    storage_op:{key,lib_name,op_name,config_str}, handlers:{"<hid>":{...}},
//    nodes:[{g_rank,shard_list,status}], update_nodes:[...]}
// and the transitions of :165-355 (dead-node marking, dead-node replacement by a restoring server
// that takes over the descriptor under a NEW node id, update-info create / apply / drop). Replica
// choice is uniformly random among RUNNING holders (:425-439).
#pragma once
#include <algorithm>
#include <climits>
#include <cstdint>
#include <map>
#include <random>
#include <set>
#include <string>
#include <vector>

#include "../common/json.h"
#include "../common/status.h"

namespace psb {

struct OperatorDescriptor {
    std::string key, lib_name, op_name, config_str;
    Json to_json() const {
        Json j = Json::object();
        j["key"] = key; j["lib_name"] = lib_name; j["op_name"] = op_name; j["config_str"] = config_str;
        return j;
    }
    static OperatorDescriptor from_json(const Json& j) {
        OperatorDescriptor d;
        d.key = j.at("key").as_string(); d.lib_name = j.at("lib_name").as_string();
        d.op_name = j.at("op_name").as_string(); d.config_str = j.at("config_str").as_string();
        return d;
    }
};

enum class NodeStatus : int { RUNNING = 0, DEAD = 1, LOADING = 2, UNAVAILABLE = 3 };
enum class StorageStatus : int { NORMAL = 0, RESHARD = 1, LOADING = 2 };

struct NodeDescriptor {
    int node_id = -1;  // g_rank: id of the server process that currently serves these shards
    std::vector<int32_t> shard_list;
    NodeStatus status = NodeStatus::RUNNING;
    Json to_json() const {
        Json j = Json::object();
        j["g_rank"] = node_id;
        Json sl = Json::array();
        for (int s : shard_list) sl.push_back(Json(s));
        j["shard_list"] = sl;
        j["status"] = (int)status;
        return j;
    }
    static NodeDescriptor from_json(const Json& j) {
        NodeDescriptor n;
        n.node_id = (int)j.at("g_rank").as_int(-1);
        for (auto& s : j.at("shard_list").elements()) n.shard_list.push_back((int32_t)s.as_int());
        n.status = (NodeStatus)j.at("status").as_int(0);
        return n;
    }
};

struct TableDescriptor {
    int32_t version = 0;         // bumped on every committed change of placement / status / handlers
    int32_t update_version = 0;  // bumped when a reshard transaction starts and when it commits
    std::string version_uuid;    // identity of the data layout (checked by persistent tiers on restore)
    std::string table_uri;       // where the last dump lives: file-system fallback of HA restore
    std::string table_name;
    StorageStatus status = StorageStatus::NORMAL;
    OperatorDescriptor storage_op;
    std::map<int32_t, OperatorDescriptor> handlers;
    std::vector<NodeDescriptor> nodes, update_nodes;

    // ---- derived (refresh_info) ----
    std::map<int32_t, std::vector<int>> shards, update_shards;  // shard -> non-DEAD holders
    std::map<std::string, int32_t> key_to_hdl;

    void refresh_info() {
        shards.clear();
        update_shards.clear();
        key_to_hdl.clear();
        for (auto& n : nodes)
            for (int s : n.shard_list) {
                auto& v = shards[s];
                if (n.status != NodeStatus::DEAD) v.push_back(n.node_id);
            }
        for (auto& n : update_nodes)
            for (int s : n.shard_list) {
                auto& v = update_shards[s];
                if (n.status != NodeStatus::DEAD) v.push_back(n.node_id);
            }
        for (auto& kv : handlers) key_to_hdl[kv.second.key] = kv.first;
    }

    int32_t global_shard_num() const { return (int32_t)shards.size(); }
    int32_t update_global_shard_num() const { return (int32_t)update_shards.size(); }

    Json to_json() const {
        Json j = Json::object();
        j["version"] = version;
        j["update_version"] = update_version;
        j["version_uuid"] = version_uuid;
        j["table_uri"] = table_uri;
        j["table_name"] = table_name;
        j["status"] = (int)status;
        j["storage_op"] = storage_op.to_json();
        Json h = Json::object();
        for (auto& kv : handlers) h[std::to_string(kv.first)] = kv.second.to_json();
        j["handlers"] = h;
        Json n = Json::array(), un = Json::array();
        for (auto& d : nodes) n.push_back(d.to_json());
        for (auto& d : update_nodes) un.push_back(d.to_json());
        j["nodes"] = n;
        j["update_nodes"] = un;
        return j;
    }
    std::string to_json_str() const { return to_json().dump(); }

    // Replace the content from JSON. With `only_if_newer` the descriptor is left alone (returns
    // false) unless the incoming version or update_version is larger.
    bool from_json(const Json& j, bool only_if_newer = false) {
        // anything that is not a context object leaves the descriptor alone
        if (!j.has("version") || !j.has("update_version") || !j.has("nodes") || !j.has("storage_op")) return false;
        int32_t v = (int32_t)j.at("version").as_int(), uv = (int32_t)j.at("update_version").as_int();
        if (only_if_newer && v <= version && uv <= update_version) return false;
        version = v;
        update_version = uv;
        version_uuid = j.at("version_uuid").as_string();
        table_uri = j.at("table_uri").as_string();
        table_name = j.at("table_name").as_string();
        status = (StorageStatus)j.at("status").as_int();
        storage_op = OperatorDescriptor::from_json(j.at("storage_op"));
        handlers.clear();
        for (auto& kv : j.at("handlers").items())
            handlers[(int32_t)std::stol(kv.first)] = OperatorDescriptor::from_json(kv.second);
        nodes.clear();
        update_nodes.clear();
        for (auto& n : j.at("nodes").elements()) nodes.push_back(NodeDescriptor::from_json(n));
        for (auto& n : j.at("update_nodes").elements()) update_nodes.push_back(NodeDescriptor::from_json(n));
        refresh_info();
        return true;
    }
    bool from_json_str(const std::string& s, bool only_if_newer = false) {
        Json j;
        if (!Json::parse(s, &j)) return false;
        return from_json(j, only_if_newer);
    }

    // Parse the "nodes" list of a storage config: [{g_rank, shard_list:[...]}, ...]
    static Status parse_nodes(const Json& cfg, std::vector<NodeDescriptor>* out) {
        if (!cfg.is_array()) return Status::InvalidConfig("nodes must be a list");
        std::set<int> seen;
        for (auto& n : cfg.elements()) {
            NodeDescriptor d;
            d.node_id = (int)n.at("g_rank").as_int(-1);
            if (d.node_id < 0) return Status::InvalidConfig("node without g_rank");
            if (!seen.insert(d.node_id).second) return Status::InvalidConfig("duplicate g_rank in nodes");
            std::set<int32_t> mine;
            for (auto& s : n.at("shard_list").elements()) {
                const int64_t id = s.as_int(-1);
                if (id < 0 || id > INT32_MAX) return Status::InvalidConfig("shard ids are non-negative integers");
                if (!mine.insert((int32_t)id).second) return Status::InvalidConfig("shard " + std::to_string(id) + " is listed twice for node " + std::to_string(d.node_id));
                d.shard_list.push_back((int32_t)id);
            }
            out->push_back(d);
        }
        // Keys map to shards 0 .. G-1, so a placement must name exactly those: a gap would be a shard that nobody
        // holds (every key of it unreachable), an empty placement a table without data.
        std::set<int32_t> all;
        for (auto& d : *out) all.insert(d.shard_list.begin(), d.shard_list.end());
        if (all.empty()) return Status::InvalidConfig("the placement holds no shard");
        if ((size_t)*all.rbegin() + 1 != all.size()) {
            int32_t missing = 0;
            while (all.count(missing)) ++missing;
            return Status::InvalidConfig("shard ids must be 0 .. G-1 without gaps: nobody holds shard " + std::to_string(missing));
        }
        return Status::Ok();
    }

    // ---- liveness ---------------------------------------------------------------------------
    // Nodes that are not in `live` turn DEAD (a LOADING node is a restoring server: left alone).
    bool update_node_status(const std::set<int>& live) {
        bool changed = false;
        for (auto* list : {&nodes, &update_nodes})
            for (auto& n : *list)
                if (n.status != NodeStatus::DEAD && n.status != NodeStatus::LOADING && !live.count(n.node_id)) {
                    n.status = NodeStatus::DEAD;
                    changed = true;
                }
        if (changed) refresh_info();
        return changed;
    }
    bool mark_node(int node_id, NodeStatus st) {
        bool changed = false;
        for (auto* list : {&nodes, &update_nodes})
            for (auto& n : *list)
                if (n.node_id == node_id && n.status != st) {
                    n.status = st;
                    changed = true;
                }
        if (changed) refresh_info();
        return changed;
    }
    // A restoring server adopts the first DEAD descriptor under its own (new) id. Node ids are never
    // reused (pico-ps/service/TableDescriptor.cpp:261-273).
    bool try_to_replace_one_dead_node(int my_id, int* replaced_id = nullptr) {
        for (auto& n : nodes)
            if (n.status == NodeStatus::DEAD) {
                if (replaced_id) *replaced_id = n.node_id;
                int old = n.node_id;
                n.node_id = my_id;
                n.status = NodeStatus::LOADING;
                for (auto& u : update_nodes)
                    if (u.node_id == old) { u.node_id = my_id; u.status = NodeStatus::LOADING; }
                ++version;
                refresh_info();
                return true;
            }
        return false;
    }
    bool set_node_status_to_running(int my_id) {
        bool changed = mark_node(my_id, NodeStatus::RUNNING);
        if (changed) ++version;
        return changed;
    }

    // ---- reshard transaction ---------------------------------------------------------------------
    void create_update_info(const std::vector<NodeDescriptor>& new_nodes) {
        update_nodes = new_nodes;
        ++update_version;
        status = StorageStatus::RESHARD;
        refresh_info();
    }
    void apply_update() {
        nodes = update_nodes;
        update_nodes.clear();
        ++version;
        ++update_version;
        gen_new_version_uuid();
        refresh_info();
    }
    void drop_update() {
        update_nodes.clear();
        status = StorageStatus::NORMAL;
        ++version;
        refresh_info();
    }
    void gen_new_version_uuid() {
        static thread_local std::mt19937_64 rng{std::random_device{}()};
        char buf[40];
        unsigned long long a = rng(), b = rng();
        std::snprintf(buf, sizeof buf, "%08llx-%04llx-%04llx-%04llx-%012llx", a >> 32, (a >> 16) & 0xffff, a & 0xffff,
                      b >> 48, b & 0xffffffffffffull);
        version_uuid = buf;
    }
};

// What one process needs at run time: who owns what, and which shards are mine.
class RuntimeInfo {
public:
    RuntimeInfo() = default;
    RuntimeInfo(const TableDescriptor& td, int my_node_id, bool use_update = false) { build(td, my_node_id, use_update); }

    void build(const TableDescriptor& td, int my_node_id, bool use_update = false) {
        my_id_ = my_node_id;
        const auto& list = use_update ? td.update_nodes : td.nodes;
        shards_.clear();
        nodes_.clear();
        local_.clear();
        running_.clear();
        for (auto& n : list) {
            if (n.status == NodeStatus::DEAD) {
                for (int s : n.shard_list) shards_[s];  // shard exists even when a holder is dead
                continue;
            }
            nodes_[n.node_id] = n.shard_list;
            if (n.status == NodeStatus::RUNNING) running_.insert(n.node_id);
            for (int s : n.shard_list) shards_[s].push_back(n.node_id);
            if (n.node_id == my_node_id) local_.insert(n.shard_list.begin(), n.shard_list.end());
        }
    }

    int32_t global_shard_num() const { return (int32_t)shards_.size(); }
    const std::set<int32_t>& local_shards() const { return local_; }
    const std::map<int32_t, std::vector<int>>& shards() const { return shards_; }
    const std::map<int, std::vector<int32_t>>& nodes() const { return nodes_; }
    int node_id() const { return my_id_; }
    bool is_running(int node) const { return running_.count(node) != 0; }

    // Uniformly random RUNNING holder of `shard`, -1 when none (-> Status::NoReplica).
    int pick_one_replica(int32_t shard, const std::set<int>* exclude = nullptr) const {
        auto it = shards_.find(shard);
        if (it == shards_.end()) return -1;
        std::vector<int> cand;
        for (int n : it->second)
            if (running_.count(n) && !(exclude && exclude->count(n))) cand.push_back(n);
        if (cand.empty()) return -1;
        static thread_local std::mt19937 rng{std::random_device{}()};
        return cand[rng() % cand.size()];
    }

private:
    int my_id_ = -1;
    std::map<int32_t, std::vector<int>> shards_;
    std::map<int, std::vector<int32_t>> nodes_;
    std::set<int32_t> local_;
    std::set<int> running_;
};

}  // namespace psb
