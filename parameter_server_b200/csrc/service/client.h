// Client: the process-side library of learners, predictors and the controller. Manages storages and
// handlers (ids from the master, context JSON published under the global lock), sends requests to
// servers, and reacts to failures.
//
// Parity: pico-ps/service/Client.h:25-140 and pico-ps/service/Client.cpp (create_storage :68-106,
// initialize_storage :116-129, delete / clear / query :131-172, register_handler :174-218,
// set_table_uri :220-231, failure handling handle_timeout / detect_deadnode :239-246,359-399,
// handle_server_too_new_ctx :248-275, handle_out_of_memory with 100 ms x 1.1^n back-off :277-327,
// context push / pull and update broadcasts :412-498), plus the scatter / gather primitive of
// pico-ps/common/DistributedAsyncReturn.{h,cpp} (send to several servers, wait with a timeout, map
// transport failures to Status::Timeout).
#pragma once
#include <chrono>
#include <thread>

#include "../operator/operators.h"
#include "context.h"
#include "master.h"
#include "../common/log.h"
#include "server.h"

namespace psb {

struct NodeResponse {
    int node = -1;
    Status status;
    Archive body;
};

class Client {
public:
    explicit Client(const std::string& master_addr) : master_(master_addr) { register_builtin_operators(); }

    MasterClient& master() { return master_; }
    Context& context() { return ctx_; }

    Status get_pserver_list(std::map<int32_t, std::string>* nodes) { return master_.get_nodes(PSERVER_C2S_RPC_NAME, nodes); }
    // Servers that are registered AND answer a health check within `timeout_ms`
    // (Client::get_available_pserver_list of pico-ps/service/Client.h:36-116).
    Status get_available_pserver_list(std::vector<int32_t>* nodes, int timeout_ms = 2000) {
        std::map<int32_t, std::string> all;
        PSB_RETURN_IF_ERROR(get_pserver_list(&all));
        nodes->clear();
        for (auto& kv : all)
            if (health_check(kv.first, timeout_ms).ok()) nodes->push_back(kv.first);
        return Status::Ok();
    }

    // ---- scatter / gather -------------------------------------------------------------------
    // Sends one request per node and waits for all. The result is the first non-OK status (transport
    // failures are Timeout); per-node outcomes are in `out`.
    Status send_and_wait(int32_t sid, int32_t hid, RequestType type, const std::map<int, Archive>& bodies, int timeout_ms,
                         std::vector<NodeResponse>* out, int32_t ctx_ver = -2, int32_t ctx_u_ver = -1) {
        // the addresses come from a short-lived copy of the registry (a request does not cost a round trip to the
        // master, and the data path outlives a master that is away for a moment); a node that the copy does not
        // know, or any failure below, makes the next look-up go to the master again
        std::map<int32_t, std::string> nodes;
        bool need_fresh = false;
        {
            std::lock_guard<std::mutex> g(nodes_mu_);
            const auto age = std::chrono::steady_clock::now() - nodes_at_;
            need_fresh = nodes_cache_.empty() || age > std::chrono::milliseconds(kNodeCacheMs);
            if (!need_fresh) {
                nodes = nodes_cache_;
                for (auto& kv : bodies)
                    if (!nodes.count(kv.first)) need_fresh = true;
            }
        }
        if (need_fresh) {
            Status ls = get_pserver_list(&nodes);
            std::lock_guard<std::mutex> g(nodes_mu_);
            if (ls.ok()) {
                nodes_cache_ = nodes;
                nodes_at_ = std::chrono::steady_clock::now();
            } else if (nodes_cache_.empty()) {
                return ls;
            } else {
                nodes = nodes_cache_;   // the master is away: go on with what was known
            }
        }
        PSMessageMeta meta;
        meta.sid = sid;
        meta.hid = hid;
        meta.req_type = type;
        meta.ctx_u_ver = ctx_u_ver;
        if (ctx_ver == -2) {
            auto e = ctx_.get(sid);
            meta.ctx_ver = -1;
            if (e) {
                std::shared_lock<std::shared_mutex> g(e->mu);
                meta.ctx_ver = e->td.version;
            }
        } else {
            meta.ctx_ver = ctx_ver;
        }
        struct Flight { int node; RpcClient::Ticket t; bool missing; };
        std::vector<Flight> flights;
        for (auto& kv : bodies) {
            auto it = nodes.find(kv.first);
            if (it == nodes.end()) {
                flights.push_back({kv.first, nullptr, true});
                continue;
            }
            PSMessage m;
            m.ar = kv.second;
            m.meta = meta;
            flights.push_back({kv.first, rpc_.send(it->second, m.seal()), false});
        }
        Status result;
        for (auto& f : flights) {
            NodeResponse r;
            r.node = f.node;
            if (f.missing) {
                r.status = Status::Timeout("node " + std::to_string(f.node) + " is not registered (no such server)");
            } else {
                Bytes b;
                r.status = rpc_.wait(f.t, timeout_ms, &b);
                if (r.status.ok()) {
                    PSMessage resp = PSMessage::open(std::move(b));
                    if (resp.meta.sid != sid || resp.meta.hid != hid || resp.meta.req_type != type) {
                        r.status = Status::Error("response meta does not match the request");
                    } else {
                        resp.ar >> r.status;
                        r.body = std::move(resp.ar);
                    }
                }
            }
            if (!r.status.ok() && result.ok()) result = r.status;
            if (out) out->push_back(std::move(r));
        }
        if (!result.ok()) {
            std::lock_guard<std::mutex> g(nodes_mu_);
            nodes_at_ = std::chrono::steady_clock::time_point();   // look the registry up again next time
        }
        return result;
    }
    Status broadcast(int32_t sid, RequestType type, const std::set<int>& nodes, const Archive& body, int timeout_ms,
                     int32_t ctx_ver = -2, int32_t ctx_u_ver = -1, std::vector<NodeResponse>* out = nullptr) {
        std::map<int, Archive> bodies;
        for (int n : nodes) bodies[n] = body;
        return send_and_wait(sid, -1, type, bodies, timeout_ms, out, ctx_ver, ctx_u_ver);
    }

    // ---- storages ----------------------------------------------------------------------------
    // cfg: {"nodes":[{"g_rank":..,"shard_list":[..]}], "op_config":{..}, "table_name": ".."}
    Status create_storage(const std::string& lib, const std::string& op, const std::string& cfg_json, int32_t* sid,
                          int timeout_ms = 30000) {
        Json cfg;
        if (!Json::parse_config(cfg_json, &cfg)) return Status::InvalidConfig("storage config is neither valid JSON nor YAML");
        PSB_RETURN_IF_ERROR(master_.generate_id(STORAGE_ID_KEY, sid));
        std::shared_ptr<TableEntry> e;
        PSB_RETURN_IF_ERROR(ctx_.create_storage(*sid, lib, op, cfg, -1, &e));
        Archive body;
        cfg["version_uuid"] = Json(e->td.version_uuid);
        body << lib << op << cfg.dump();
        std::set<int> nodes;
        for (auto& n : e->td.nodes) nodes.insert(n.node_id);
        Status st = broadcast(*sid, RequestType::STORAGE_CREATE, nodes, body, timeout_ms, -1);
        if (!st.ok()) {
            broadcast(*sid, RequestType::STORAGE_DELETE, nodes, Archive(), timeout_ms, -1);
            ctx_.erase(*sid);
            return st;
        }
        PSB_RETURN_IF_ERROR(master_.acquire_lock(PSERVER_LOCK_NAME));
        st = master_.add_context(ctx_key(*sid), e->td.to_json_str());
        master_.release_lock(PSERVER_LOCK_NAME);
        return st;
    }
    // Predictor-side alias of create_storage (pico-ps/service/Client.cpp:108-114).
    Status pred_create_storage(const std::string& lib, const std::string& op, const std::string& cfg_json, int32_t* sid,
                               int timeout_ms = 30000) {
        return create_storage(lib, op, cfg_json, sid, timeout_ms);
    }
    Status initialize_storage(int32_t sid) { return pull_context(sid); }
    Status delete_storage(int32_t sid, int timeout_ms = 30000) {
        PSB_RETURN_IF_ERROR(pull_context(sid));
        auto e = ctx_.get(sid);
        // servers that are gone have nothing left to delete
        std::map<int32_t, std::string> live;
        PSB_RETURN_IF_ERROR(get_pserver_list(&live));
        std::set<int> nodes;
        for (int n : all_nodes(*e))
            if (live.count(n)) nodes.insert(n);
        Status st = broadcast(sid, RequestType::STORAGE_DELETE, nodes, Archive(), timeout_ms, -1);
        master_.acquire_lock(PSERVER_LOCK_NAME);
        master_.delete_context(ctx_key(sid));
        master_.release_lock(PSERVER_LOCK_NAME);
        ctx_.erase(sid);
        return st;
    }
    Status clear_storage(int32_t sid, int timeout_ms = 30000) {
        auto e = ctx_.get(sid);
        if (!e) return Status::InvalidID("unknown storage");
        return broadcast(sid, RequestType::STORAGE_CLEAR, all_nodes(*e), Archive(), timeout_ms);
    }
    Status query_storage_info(int32_t sid, std::vector<StorageStatisticInfo>* info, int timeout_ms = 30000) {
        auto e = ctx_.get(sid);
        if (!e) return Status::InvalidID("unknown storage");
        std::vector<NodeResponse> rs;
        PSB_RETURN_IF_ERROR(broadcast(sid, RequestType::STORAGE_STATISTIC, all_nodes(*e), Archive(), timeout_ms, -2, -1, &rs));
        for (auto& r : rs) {
            int32_t n = 0;
            r.body >> n;
            for (int32_t i = 0; i < n; ++i) {
                StorageStatisticInfo s;
                r.body >> s.item_number >> s.memory_usage >> s.node_id >> s.shard_id;
                info->push_back(s);
            }
        }
        return Status::Ok();
    }
    Status query_memory_info(int node, NodeMemoryInfo* mi, int timeout_ms = 10000) {
        std::vector<NodeResponse> rs;
        PSB_RETURN_IF_ERROR(broadcast(-1, RequestType::MEMORY_INFO, {node}, Archive(), timeout_ms, -1, -1, &rs));
        int32_t h = 1;
        rs[0].body >> h >> mi->used >> mi->managed;
        mi->healthy = h != 0;
        return Status::Ok();
    }
    Status health_check(int node, int timeout_ms = 2000) {
        return broadcast(-1, RequestType::HEALTH_CHECK, {node}, Archive(), timeout_ms, -1);
    }
    Status close_pserver(int node, int timeout_ms = 5000) {
        Status st = broadcast(-1, RequestType::EXIT, {node}, Archive(), timeout_ms, -1);
        std::lock_guard<std::mutex> g(nodes_mu_);
        nodes_at_ = std::chrono::steady_clock::time_point();   // the registry has just changed
        return st;
    }
    Status load_operator_library(const std::string& path, int timeout_ms = 30000) {
        PSB_RETURN_IF_ERROR(OperatorFactory::instance().load_library(path));
        std::map<int32_t, std::string> nodes;
        PSB_RETURN_IF_ERROR(get_pserver_list(&nodes));
        std::set<int> ids;
        for (auto& kv : nodes) ids.insert(kv.first);
        Archive body;
        body << path;
        return broadcast(-1, RequestType::OP_LOAD_LIBRARY, ids, body, timeout_ms, -1);
    }

    // ---- handlers ----------------------------------------------------------------------------
    Status register_handler(const std::string& key, const std::string& lib, const std::string& op, const std::string& cfg,
                            int32_t sid, int32_t* hid, int timeout_ms = 30000) {
        if (!OperatorFactory::instance().has(lib, op)) return Status::InvalidConfig("no operator (" + lib + ", " + op + ")");
        PSB_RETURN_IF_ERROR(master_.acquire_lock(PSERVER_LOCK_NAME));
        Status st = [&]() -> Status {
            PSB_RETURN_IF_ERROR(pull_context_nolock(sid));
            auto e = ctx_.get(sid);
            PSB_RETURN_IF_ERROR(master_.generate_id(HANDLER_ID_KEY, hid));
            Archive body;
            body << *hid << key << lib << op << cfg;
            PSB_RETURN_IF_ERROR(broadcast(sid, RequestType::HANDLER_REGISTER, all_nodes(*e), body, timeout_ms, -1));
            {
                std::unique_lock<std::shared_mutex> g(e->mu);
                e->td.handlers[*hid] = OperatorDescriptor{key, lib, op, cfg};
                e->td.refresh_info();
                PSB_RETURN_IF_ERROR(e->update_handlers());
            }
            return master_.set_context(ctx_key(sid), e->td.to_json_str());
        }();
        master_.release_lock(PSERVER_LOCK_NAME);
        return st;
    }
    Status deregister_handler(int32_t sid, int32_t hid, int timeout_ms = 30000) {
        PSB_RETURN_IF_ERROR(master_.acquire_lock(PSERVER_LOCK_NAME));
        Status st = [&]() -> Status {
            PSB_RETURN_IF_ERROR(pull_context_nolock(sid));
            auto e = ctx_.get(sid);
            Archive body;
            body << hid;
            PSB_RETURN_IF_ERROR(broadcast(sid, RequestType::HANDLER_DEREGISTER, all_nodes(*e), body, timeout_ms, -1));
            {
                std::unique_lock<std::shared_mutex> g(e->mu);
                e->td.handlers.erase(hid);
                e->td.refresh_info();
                e->update_handlers();
            }
            return master_.set_context(ctx_key(sid), e->td.to_json_str());
        }();
        master_.release_lock(PSERVER_LOCK_NAME);
        return st;
    }
    // Handler id of the operator registered under `key` (other clients attach by key).
    Status handler_by_key(int32_t sid, const std::string& key, int32_t* hid) {
        auto e = ctx_.get(sid);
        if (!e) return Status::InvalidID("unknown storage");
        std::shared_lock<std::shared_mutex> g(e->mu);
        auto it = e->td.key_to_hdl.find(key);
        if (it == e->td.key_to_hdl.end()) return Status::InvalidID("no handler with key " + key);
        *hid = it->second;
        return Status::Ok();
    }
    Status set_table_uri(int32_t sid, const std::string& uri) {
        PSB_RETURN_IF_ERROR(master_.acquire_lock(PSERVER_LOCK_NAME));
        Status st = [&]() -> Status {
            PSB_RETURN_IF_ERROR(pull_context_nolock(sid));
            auto e = ctx_.get(sid);
            {
                std::unique_lock<std::shared_mutex> g(e->mu);
                e->td.table_uri = uri;
                ++e->td.version;
            }
            PSB_RETURN_IF_ERROR(master_.set_context(ctx_key(sid), e->td.to_json_str()));
            return require_update_ctx_nolock(sid, all_nodes(*e));
        }();
        master_.release_lock(PSERVER_LOCK_NAME);
        return st;
    }
    Status get_current_ctx(int32_t sid, std::string* json) {
        auto e = ctx_.get(sid);
        if (!e) return Status::InvalidID("unknown storage");
        std::shared_lock<std::shared_mutex> g(e->mu);
        *json = e->td.to_json_str();
        return Status::Ok();
    }
    // Overwrite the placement of a table with a saved context (the reference's set_ctx, used to go back
    // to an earlier sharding before a restore).
    Status set_ctx(int32_t sid, const std::string& json) {
        PSB_RETURN_IF_ERROR(master_.acquire_lock(PSERVER_LOCK_NAME));
        Status st = [&]() -> Status {
            PSB_RETURN_IF_ERROR(pull_context_nolock(sid));
            auto e = ctx_.get(sid);
            TableDescriptor saved;
            if (!saved.from_json_str(json)) return Status::InvalidConfig("set_ctx: JSON does not parse");
            std::set<int> nodes = all_nodes(*e);
            {
                std::unique_lock<std::shared_mutex> g(e->mu);
                e->td.nodes = saved.nodes;
                e->td.update_nodes.clear();
                ++e->td.version;
                e->td.refresh_info();
                e->rt.build(e->td, -1);
            }
            for (int n : all_nodes(*e)) nodes.insert(n);
            PSB_RETURN_IF_ERROR(master_.set_context(ctx_key(sid), e->td.to_json_str()));
            return require_update_ctx_nolock(sid, nodes);
        }();
        master_.release_lock(PSERVER_LOCK_NAME);
        return st;
    }

    // ---- context sync and failure handling -----------------------------------------------------
    Status pull_context(int32_t sid) { return pull_context_nolock(sid); }
    Status pull_context_nolock(int32_t sid) {
        std::string json;
        PSB_RETURN_IF_ERROR(master_.get_context(ctx_key(sid), &json));
        return ctx_.set_table_descriptor(sid, json, -1, nullptr);
    }
    Status push_context_nolock(int32_t sid) {
        auto e = ctx_.get(sid);
        if (!e) return Status::InvalidID("unknown storage");
        return master_.set_context(ctx_key(sid), e->td.to_json_str());
    }
    Status require_update_ctx_nolock(int32_t sid, const std::set<int>& nodes, int timeout_ms = 30000) {
        // servers that are gone cannot be told; that is fine, they re-read the context when they return
        std::map<int32_t, std::string> live;
        PSB_RETURN_IF_ERROR(get_pserver_list(&live));
        std::set<int> targets;
        for (int n : nodes)
            if (live.count(n)) targets.insert(n);
        return broadcast(sid, RequestType::CTX_UPDATE, targets, Archive(), timeout_ms, -1);
    }
    // Fire-and-forget form (pico-ps/service/Client.cpp:233-237): every live node of the table is told to re-read its
    // context; nobody waits for the answers, which the connection's reader drops when they arrive.
    void require_update_ctx_async(int32_t sid) {
        auto e = ctx_.get(sid);
        std::map<int32_t, std::string> live;
        if (!e || !get_pserver_list(&live).ok()) return;
        std::set<int> targets;
        {
            std::shared_lock<std::shared_mutex> g(e->mu);
            for (auto& kv : e->rt.nodes())
                if (live.count(kv.first)) targets.insert(kv.first);
        }
        PSMessageMeta meta;
        meta.sid = sid;
        meta.hid = -1;
        meta.ctx_ver = -1;
        meta.ctx_u_ver = -1;
        meta.req_type = RequestType::CTX_UPDATE;
        for (int n : targets) {
            PSMessage m;
            m.meta = meta;
            rpc_.send(live[n], m.seal());
        }
    }
    // Timeout / NoReplica: find out who died. A node that is no longer registered at the master is DEAD
    // for everybody (published); a registered node that does not answer is UNAVAILABLE for this client.
    Status handle_timeout(int32_t sid) {
        PSB_RETURN_IF_ERROR(master_.acquire_lock(PSERVER_LOCK_NAME));
        Status st = [&]() -> Status {
            PSB_RETURN_IF_ERROR(pull_context_nolock(sid));
            auto e = ctx_.get(sid);
            std::map<int32_t, std::string> live;
            PSB_RETURN_IF_ERROR(get_pserver_list(&live));
            std::set<int> live_ids;
            for (auto& kv : live) live_ids.insert(kv.first);
            bool changed = false;
            std::set<int> nodes = all_nodes(*e);
            {
                std::unique_lock<std::shared_mutex> g(e->mu);
                changed = e->td.update_node_status(live_ids);
                if (changed) ++e->td.version;
                e->rt.build(e->td, -1);
            }
            if (changed) {
                PSB_LOG(WARNING) << "storage " << sid << ": nodes that left the registry are marked DEAD, context version " << e->td.version;
                PSB_RETURN_IF_ERROR(master_.set_context(ctx_key(sid), e->td.to_json_str()));
                require_update_ctx_nolock(sid, nodes);
            }
            for (auto& kv : live) {
                if (!nodes.count(kv.first)) continue;
                if (!health_check(kv.first, 1000).ok()) {
                    PSB_LOG(WARNING) << "storage " << sid << ": node " << kv.first << " is registered but does not answer, avoiding it";
                    std::unique_lock<std::shared_mutex> g(e->mu);
                    e->td.mark_node(kv.first, NodeStatus::UNAVAILABLE);
                    e->rt.build(e->td, -1);
                }
            }
            return Status::Ok();
        }();
        master_.release_lock(PSERVER_LOCK_NAME);
        return st;
    }
    Status handle_server_too_new_ctx(int32_t sid) { return pull_context(sid); }
    // OUT_OF_MEMORY: somebody has to rescale (or a reshard is running); wait for a context change.
    Status handle_out_of_memory(int32_t sid, int timeout_ms) {
        auto e = ctx_.get(sid);
        if (!e) return Status::InvalidID("unknown storage");
        auto snapshot = [&](int32_t* ver, StorageStatus* status) {
            std::shared_lock<std::shared_mutex> g(e->mu);
            *ver = e->td.version;
            *status = e->td.status;
        };
        int32_t v0 = 0, v = 0;
        StorageStatus status;
        snapshot(&v0, &status);
        PSB_LOG(INFO) << "storage " << sid << ": out of memory or resharding, waiting for a context newer than " << v0;
        double wait_ms = 100;
        auto t0 = std::chrono::steady_clock::now();
        for (;;) {
            PSB_RETURN_IF_ERROR(pull_context(sid));
            snapshot(&v, &status);
            if (v != v0 && status == StorageStatus::NORMAL) return Status::Ok();
            auto el = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
            if (timeout_ms >= 0 && el + (long)wait_ms > timeout_ms) return Status::Timeout("still out of memory / resharding");
            std::this_thread::sleep_for(std::chrono::milliseconds((long)wait_ms));
            wait_ms = std::min(wait_ms * 1.1, 2000.0);
        }
    }

    static std::set<int> all_nodes(const TableEntry& e) {
        std::set<int> s;
        for (auto& n : e.td.nodes)
            if (n.status != NodeStatus::DEAD) s.insert(n.node_id);
        for (auto& n : e.td.update_nodes)
            if (n.status != NodeStatus::DEAD) s.insert(n.node_id);
        return s;
    }

private:
    static constexpr int kNodeCacheMs = 500;
    std::mutex nodes_mu_;
    std::map<int32_t, std::string> nodes_cache_;
    std::chrono::steady_clock::time_point nodes_at_{};
    MasterClient master_;
    RpcClient rpc_;
    Context ctx_;
};

}  // namespace psb
