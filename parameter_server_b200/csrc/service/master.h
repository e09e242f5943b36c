// The master: one small process-wide coordination service (context store, id generator, global lock,
// barrier, node registry with liveness, tree nodes for broadcast and model objects).
//
// Parity: the subset of prpc's Master / MasterClient API that pico-ps calls (listed in
// pico-ps/common/core.h:128-131 and used in pico-ps/service/Client.cpp:68-106,174-201,359-399 and
// pico-ps/service/Service.cpp:150-191): acquire_lock / release_lock (PSERVER_LOCK), generate_id
// ("storage_id", "handler"), add/set/get/delete_context, get_storage_list, the RPC service registry
// whose membership IS the liveness signal (a node whose session connection closes is unregistered),
// barrier, tree_node_add / get, get_model / set_model. The in-process TCP master of the reference's
// tests (pico-ps/test/TestUtils.h:16-92) corresponds to constructing Master directly.
#pragma once
#include <algorithm>
#include <chrono>
#include <cstdio>
#include <fstream>
#include <iterator>
#include <map>
#include <set>
#include <string>
#include <vector>

#include "../common/archive.h"
#include "../common/message.h"
#include "rpc.h"

namespace psb {

enum class MasterOp : int32_t {
    GEN_ID = 1, LOCK = 2, UNLOCK = 3, CTX_SET = 4, CTX_GET = 5, CTX_DEL = 6, CTX_LIST = 7, REGISTER = 8,
    DEREGISTER = 9, NODES = 10, BARRIER = 11, TREE_SET = 12, TREE_GET = 13, TREE_DEL = 14, TREE_LIST = 15, PING = 16,
};

class Master {
public:
    // `state_file`: the durable part of the master's state (id counters, contexts, tree nodes, the next node id) is
    // written there after every change (temp file + rename) and read back at start, so a master that is restarted
    // on the same `port` carries on: servers notice that their registration is gone and register again under their
    // node ids, clients reconnect on their next call. For `recover_ms` after a start from a state file the node
    // list is not served (TIMEOUT "recovering"): nobody must take the not-yet-re-registered servers for dead.
    // Locks and barriers are not durable: a holder that outlives the master simply fails to release.
    explicit Master(int n_threads = 4, int port = 0, std::string state_file = "", int recover_ms = 3000)
        : state_file_(std::move(state_file)),
          server_((load_state(recover_ms), [this](Bytes&& b, RpcServer::Responder r) { handle(std::move(b), r); }), n_threads,
                  [this](uint64_t conn) { on_disconnect(conn); }, port) {}
    std::string address() const { return server_.address(); }
    void stop() { server_.stop(); }

private:
    static Bytes ok_reply(Archive&& ar = Archive()) {
        Archive out;
        out << Status::Ok();
        out.write_raw(ar.data(), ar.size());
        return out.release();
    }
    static Bytes err_reply(const Status& st) {
        Archive out;
        out << st;
        return out.release();
    }

    void handle(Bytes&& bytes, RpcServer::Responder resp) {
        Archive ar(std::move(bytes));
        int32_t op = 0;
        ar >> op;
        std::unique_lock<std::mutex> g(mu_);
        switch ((MasterOp)op) {
            case MasterOp::GEN_ID: {
                std::string key;
                ar >> key;
                Archive out;
                out << (int32_t)(ids_[key]++);
                save_state_locked();
                resp.send(ok_reply(std::move(out)));
                break;
            }
            case MasterOp::LOCK: {
                std::string name;
                ar >> name;
                auto& l = locks_[name];
                if (!l.held) {
                    l.held = true;
                    l.owner_conn = resp.conn_id();
                    resp.send(ok_reply());
                } else {
                    l.waiters.push_back(resp);  // answered when the lock is handed over
                }
                break;
            }
            case MasterOp::UNLOCK: {
                std::string name;
                ar >> name;
                // only the holder releases: a client whose connection broke lost the lock with it (on_disconnect), and
                // its late release over a new connection must not take the lock away from whoever holds it now
                auto& l = locks_[name];
                if (l.held && l.owner_conn == resp.conn_id()) release_lock_locked(name);
                resp.send(ok_reply());
                break;
            }
            case MasterOp::CTX_SET: {
                std::string key, value;
                int32_t only_if_absent = 0;
                ar >> key >> value >> only_if_absent;
                if (fenced_off(key, resp.conn_id())) {
                    resp.send(err_reply(Status::Error("context " + key + " is written under the global lock, which another session holds")));
                } else if (only_if_absent && ctx_.count(key)) {
                    resp.send(err_reply(Status::Error("context " + key + " already exists")));
                } else {
                    ctx_[key] = value;
                    save_state_locked();
                    resp.send(ok_reply());
                }
                break;
            }
            case MasterOp::CTX_GET: {
                std::string key;
                ar >> key;
                auto it = ctx_.find(key);
                if (it == ctx_.end()) {
                    resp.send(err_reply(Status::InvalidID("no context " + key)));
                } else {
                    Archive out;
                    out << it->second;
                    resp.send(ok_reply(std::move(out)));
                }
                break;
            }
            case MasterOp::CTX_DEL: {
                std::string key;
                ar >> key;
                if (fenced_off(key, resp.conn_id())) {
                    resp.send(err_reply(Status::Error("context " + key + " is written under the global lock, which another session holds")));
                    break;
                }
                ctx_.erase(key);
                save_state_locked();
                resp.send(ok_reply());
                break;
            }
            case MasterOp::CTX_LIST: {
                std::vector<std::string> keys;
                for (auto& kv : ctx_) keys.push_back(kv.first);
                Archive out;
                out << keys;
                resp.send(ok_reply(std::move(out)));
                break;
            }
            case MasterOp::REGISTER: {
                // the connection that registers is the node's session: when it closes the node is dead
                std::string service, addr;
                int32_t want_id = -1;
                ar >> service >> addr >> want_id;
                int32_t id = want_id >= 0 ? want_id : next_node_id_++;
                if (want_id >= next_node_id_) next_node_id_ = want_id + 1;
                if (want_id < 0) save_state_locked();   // ids are never handed out twice, also across a restart
                registry_[service][id] = addr;
                // the entry now belongs to THIS connection: a node that lost its session and registers again over a
                // new one must not be wiped when the close of the old connection is noticed afterwards
                auto& owner = owner_[{service, id}];
                if (owner != 0 && owner != resp.conn_id()) {
                    auto old = sessions_.find(owner);
                    if (old != sessions_.end()) old->second.erase({service, id});
                }
                owner = resp.conn_id();
                sessions_[resp.conn_id()].insert({service, id});
                Archive out;
                out << id;
                resp.send(ok_reply(std::move(out)));
                break;
            }
            case MasterOp::DEREGISTER: {
                std::string service;
                int32_t id = -1;
                ar >> service >> id;
                registry_[service].erase(id);
                owner_.erase({service, id});
                resp.send(ok_reply());
                break;
            }
            case MasterOp::NODES: {
                std::string service;
                ar >> service;
                if (std::chrono::steady_clock::now() < recovering_until_) {
                    resp.send(err_reply(Status::Timeout("master is recovering: the servers are registering again")));
                    break;
                }
                std::vector<int32_t> ids;
                std::vector<std::string> addrs;
                for (auto& kv : registry_[service]) {
                    ids.push_back(kv.first);
                    addrs.push_back(kv.second);
                }
                Archive out;
                out << ids << addrs;
                resp.send(ok_reply(std::move(out)));
                break;
            }
            case MasterOp::BARRIER: {
                std::string name;
                int32_t n = 0;
                ar >> name >> n;
                auto& b = barriers_[name];
                b.push_back(resp);
                if ((int32_t)b.size() >= n) {
                    for (auto& r : b) r.send(ok_reply());
                    barriers_.erase(name);
                }
                break;
            }
            case MasterOp::TREE_SET: {
                std::string path, value;
                ar >> path >> value;
                tree_[path] = value;
                save_state_locked();
                resp.send(ok_reply());
                break;
            }
            case MasterOp::TREE_GET: {
                std::string path;
                ar >> path;
                auto it = tree_.find(path);
                if (it == tree_.end()) {
                    resp.send(err_reply(Status::Empty("no tree node " + path)));
                } else {
                    Archive out;
                    out << it->second;
                    resp.send(ok_reply(std::move(out)));
                }
                break;
            }
            case MasterOp::TREE_DEL: {
                std::string path;
                ar >> path;
                tree_.erase(path);
                save_state_locked();
                resp.send(ok_reply());
                break;
            }
            case MasterOp::TREE_LIST: {
                std::string prefix;
                ar >> prefix;
                std::vector<std::string> keys;
                for (auto it = tree_.lower_bound(prefix); it != tree_.end() && it->first.compare(0, prefix.size(), prefix) == 0; ++it)
                    keys.push_back(it->first);
                Archive out;
                out << keys;
                resp.send(ok_reply(std::move(out)));
                break;
            }
            case MasterOp::PING: resp.send(ok_reply()); break;
            default: resp.send(err_reply(Status::Error("master: unknown op")));
        }
    }

    // ---- durable state: {"PSBM1", next_node_id, ids, ctx, tree} as one archive ----
    void save_state_locked() {
        if (state_file_.empty()) return;
        Archive ar;
        ar << std::string("PSBM1") << next_node_id_;
        ar << (uint64_t)ids_.size();
        for (auto& kv : ids_) ar << kv.first << kv.second;
        ar << (uint64_t)ctx_.size();
        for (auto& kv : ctx_) ar << kv.first << kv.second;
        ar << (uint64_t)tree_.size();
        for (auto& kv : tree_) ar << kv.first << kv.second;
        const std::string tmp = state_file_ + ".tmp";
        {
            std::ofstream f(tmp, std::ios::binary | std::ios::trunc);
            f.write((const char*)ar.data(), (std::streamsize)ar.size());
            if (!f.good()) return;   // the old file stays
        }
        ::rename(tmp.c_str(), state_file_.c_str());
    }
    // Returns 0 so that it can run inside the member initialiser list before the server starts its threads.
    int load_state(int recover_ms) {
        if (state_file_.empty()) return 0;
        std::ifstream f(state_file_, std::ios::binary);
        if (!f) return 0;   // first start
        std::vector<uint8_t> raw((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
        try {
            Archive ar(std::move(raw));
            std::string magic;
            ar >> magic;
            if (magic != "PSBM1") throw std::runtime_error("not a master state file");
            uint64_t n = 0;
            ar >> next_node_id_;
            ar >> n;
            for (uint64_t i = 0; i < n; ++i) { std::string k; int32_t v = 0; ar >> k >> v; ids_[k] = v; }
            ar >> n;
            for (uint64_t i = 0; i < n; ++i) { std::string k, v; ar >> k >> v; ctx_[k] = v; }
            ar >> n;
            for (uint64_t i = 0; i < n; ++i) { std::string k, v; ar >> k >> v; tree_[k] = v; }
        } catch (const std::exception& e) {
            throw std::runtime_error("master: cannot read " + state_file_ + ": " + e.what());
        }
        recovering_until_ = std::chrono::steady_clock::now() + std::chrono::milliseconds(recover_ms);
        return 0;
    }

    // Table contexts ("storage/<sid>") change only under the global lock. A writer that does not hold it while somebody
    // else does is a client that lost the lock with its connection and has not noticed: it is turned away instead of
    // writing over the holder's work. (Writes while nobody holds the lock pass: tools and tests edit contexts that way.)
    bool fenced_off(const std::string& key, uint64_t conn) {
        if (key.compare(0, 8, "storage/") != 0) return false;
        auto it = locks_.find(PSERVER_LOCK_NAME);
        return it != locks_.end() && it->second.held && it->second.owner_conn != conn;
    }
    void release_lock_locked(const std::string& name) {
        auto& l = locks_[name];
        while (!l.waiters.empty()) {
            RpcServer::Responder next = l.waiters.front();
            l.waiters.erase(l.waiters.begin());
            l.owner_conn = next.conn_id();
            if (next.send(ok_reply())) return;  // handed over (skips waiters that went away)
        }
        l.held = false;
        l.owner_conn = 0;
    }

    void on_disconnect(uint64_t conn) {
        std::lock_guard<std::mutex> g(mu_);
        auto it = sessions_.find(conn);
        if (it != sessions_.end()) {
            for (auto& sn : it->second) {
                auto o = owner_.find(sn);
                if (o == owner_.end() || o->second != conn) continue;   // registered again over another connection
                registry_[sn.first].erase(sn.second);
                owner_.erase(o);
            }
            sessions_.erase(it);
        }
        // a participant that went away no longer stands at its barriers: the next arrival must not complete one with it
        for (auto it = barriers_.begin(); it != barriers_.end();) {
            auto& v = it->second;
            v.erase(std::remove_if(v.begin(), v.end(), [&](const RpcServer::Responder& r) { return r.conn_id() == conn; }), v.end());
            if (v.empty()) it = barriers_.erase(it);
            else ++it;
        }
        // a client that died while holding a lock must not wedge everyone else
        for (auto& kv : locks_)
            if (kv.second.held && kv.second.owner_conn == conn) release_lock_locked(kv.first);
    }

    struct LockState {
        bool held = false;
        uint64_t owner_conn = 0;
        std::vector<RpcServer::Responder> waiters;
    };
    std::mutex mu_;
    std::map<std::string, int32_t> ids_;
    std::map<std::string, LockState> locks_;
    std::map<std::string, std::string> ctx_;
    std::map<std::string, std::map<int32_t, std::string>> registry_;
    std::map<uint64_t, std::set<std::pair<std::string, int32_t>>> sessions_;
    std::map<std::pair<std::string, int32_t>, uint64_t> owner_;   // which connection a registry entry belongs to
    std::map<std::string, std::vector<RpcServer::Responder>> barriers_;
    std::map<std::string, std::string> tree_;
    int32_t next_node_id_ = 0;
    std::string state_file_;
    std::chrono::steady_clock::time_point recovering_until_{};
    RpcServer server_;  // last member: its threads start using the state above at once
};

class MasterClient {
public:
    explicit MasterClient(std::string master_address, int timeout_ms = 30000)
        : addr_(std::move(master_address)), timeout_ms_(timeout_ms) {}

    Status generate_id(const std::string& key, int32_t* id) {
        Archive req, rep;
        req << (int32_t)MasterOp::GEN_ID << key;
        PSB_RETURN_IF_ERROR(call(req, &rep));
        rep >> *id;
        return Status::Ok();
    }
    Status acquire_lock(const std::string& name) {
        Archive req, rep;
        req << (int32_t)MasterOp::LOCK << name;
        return call(req, &rep, -1);
    }
    Status release_lock(const std::string& name) {
        Archive req, rep;
        req << (int32_t)MasterOp::UNLOCK << name;
        return call(req, &rep);
    }
    Status set_context(const std::string& key, const std::string& value, bool only_if_absent = false) {
        Archive req, rep;
        req << (int32_t)MasterOp::CTX_SET << key << value << (int32_t)(only_if_absent ? 1 : 0);
        return call(req, &rep);
    }
    Status add_context(const std::string& key, const std::string& value) { return set_context(key, value, true); }
    Status get_context(const std::string& key, std::string* value) {
        Archive req, rep;
        req << (int32_t)MasterOp::CTX_GET << key;
        PSB_RETURN_IF_ERROR(call(req, &rep));
        rep >> *value;
        return Status::Ok();
    }
    Status delete_context(const std::string& key) {
        Archive req, rep;
        req << (int32_t)MasterOp::CTX_DEL << key;
        return call(req, &rep);
    }
    Status list_contexts(std::vector<std::string>* keys) {
        Archive req, rep;
        req << (int32_t)MasterOp::CTX_LIST;
        PSB_RETURN_IF_ERROR(call(req, &rep));
        rep >> *keys;
        return Status::Ok();
    }
    // Registers on THIS client's connection: keep the MasterClient alive as long as the node lives.
    Status register_node(const std::string& service, const std::string& address, int32_t* node_id, int32_t want_id = -1) {
        Archive req, rep;
        req << (int32_t)MasterOp::REGISTER << service << address << want_id;
        PSB_RETURN_IF_ERROR(call(req, &rep));
        rep >> *node_id;
        return Status::Ok();
    }
    Status deregister_node(const std::string& service, int32_t node_id) {
        Archive req, rep;
        req << (int32_t)MasterOp::DEREGISTER << service << node_id;
        return call(req, &rep);
    }
    Status get_nodes(const std::string& service, std::map<int32_t, std::string>* nodes) {
        Archive req, rep;
        req << (int32_t)MasterOp::NODES << service;
        PSB_RETURN_IF_ERROR(call(req, &rep));
        std::vector<int32_t> ids;
        std::vector<std::string> addrs;
        rep >> ids >> addrs;
        nodes->clear();
        for (size_t i = 0; i < ids.size(); ++i) (*nodes)[ids[i]] = addrs[i];
        return Status::Ok();
    }
    Status barrier(const std::string& name, int32_t n) {
        Archive req, rep;
        req << (int32_t)MasterOp::BARRIER << name << n;
        return call(req, &rep, -1);
    }
    Status tree_node_set(const std::string& path, const std::string& value) {
        Archive req, rep;
        req << (int32_t)MasterOp::TREE_SET << path << value;
        return call(req, &rep);
    }
    Status tree_node_get(const std::string& path, std::string* value) {
        Archive req, rep;
        req << (int32_t)MasterOp::TREE_GET << path;
        PSB_RETURN_IF_ERROR(call(req, &rep));
        rep >> *value;
        return Status::Ok();
    }
    Status tree_node_del(const std::string& path) {
        Archive req, rep;
        req << (int32_t)MasterOp::TREE_DEL << path;
        return call(req, &rep);
    }
    Status tree_node_list(const std::string& prefix, std::vector<std::string>* keys) {
        Archive req, rep;
        req << (int32_t)MasterOp::TREE_LIST << prefix;
        PSB_RETURN_IF_ERROR(call(req, &rep));
        rep >> *keys;
        return Status::Ok();
    }
    Status ping() {
        Archive req, rep;
        req << (int32_t)MasterOp::PING;
        return call(req, &rep, 2000);
    }
    const std::string& address() const { return addr_; }
    void close() { rpc_.close_all(); }

private:
    Status call(Archive& req, Archive* rep, int timeout_ms = 0) {
        Bytes out;
        Status st = rpc_.call(addr_, req.bytes(), timeout_ms == 0 ? timeout_ms_ : timeout_ms, &out);
        if (!st.ok()) return Status::Fatal("master unreachable: " + st.msg());
        *rep = Archive(std::move(out));
        Status remote;
        *rep >> remote;
        return remote;
    }
    std::string addr_;
    int timeout_ms_;
    RpcClient rpc_;
};

}  // namespace psb
