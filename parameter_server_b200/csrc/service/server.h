// Server: one parameter-server process (one per GPU on a B200 box, or CPU-only). Owns the storages of
// the shards placed on it and answers two RPC services: c2s (clients) and s2s (other servers).
//
// Parity: pico-ps/service/Server.h:23-243 + pico-ps/service/Service.cpp: the request dispatch table
// (:377-541), the context version gates (:1316-1400; writes are refused with OUT_OF_MEMORY "write
// when update context" while the table is in RESHARD), storage / handler life cycle (:543-699), the
// data operations (:700-991), the reshard steps (:1052-1272), incremental sync apply (:1274-1301),
// HA restore (:150-366: take over a dead node's descriptor under a NEW node id, restore every table
// from a live replica over s2s in resumable batches, fall back to the dump at table_uri), and the
// memory self-monitor. A request is {body, PSMessageMeta tail}; a response is {Status, payload}.
#pragma once
#include <dirent.h>
#include <unistd.h>

#include <cstdio>
#include <cstring>
#include <fstream>
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <thread>

#include "../common/log.h"
#include "../operator/operators.h"
#include "context.h"
#include "master.h"

namespace psb {

struct ServerConfig {
    int c2s_thread_num = 4;
    int s2s_thread_num = 4;
    int load_thread_num = 4;
    int load_block_size = 1000;
    int report_interval_s = -1;
    int restore_wait_timeout_s = -1;
    int restore_batch_size = 1000;
    // A server in restore mode pauses the writes of a table while it copies the table's shards from the live
    // replicas (the table's status is LOADING for that time: pushes and inserting pulls answer OUT_OF_MEMORY, their
    // clients wait and send them again afterwards; reads go on). The restored replica is then exactly equal to its
    // source. Off: writes go on, and a push that meets a row between its export and its arrival can be missing on
    // the restored replica (the reference sends no writes at all to a node that is LOADING).
    bool restore_pauses_writes = false;
    int restore_thread_num = 4;
    int s2s_timeout_ms = 60000;
    // Directory of this host's persistent table images (empty: none). A server in restore mode that finds the image
    // of the node it replaces, with the table's version_uuid, opens it instead of the table's dump.
    std::string local_image_dir;
    int session_check_ms = 1000;  // how often the server checks that the master still lists it (0 = never); a master that
                                  // was restarted has lost the registrations, and the server registers again under its id
    std::string hadoop_bin;       // command behind hdfs:// dump paths ("" = $PSB_HADOOP_BIN, else "hadoop"); process-wide
};

struct StorageStatisticInfo {
    uint64_t item_number = 0, memory_usage = 0;
    int32_t node_id = -1, shard_id = -1;
};
struct NodeMemoryInfo {
    bool healthy = true;
    uint64_t used = 0, managed = 0;
};

inline std::string ctx_key(int32_t sid) { return "storage/" + std::to_string(sid); }

constexpr int kDurationBuckets = 10;
constexpr double kDurationBoundsMs[kDurationBuckets] = {0.05, 0.1, 0.25, 0.5, 1, 2.5, 5, 10, 50, 250};

class Server {
public:
    Server(const std::string& master_addr, const ServerConfig& cfg = ServerConfig())
        : cfg_(cfg), master_(master_addr), session_(master_addr) {
        register_builtin_operators();
        if (!cfg_.hadoop_bin.empty()) fs::set_hadoop_bin(cfg_.hadoop_bin);
        s2s_.reset(new RpcServer([this](Bytes&& b, RpcServer::Responder r) { dispatch(std::move(b), r, true); },
                                 cfg_.s2s_thread_num));
        Status st = session_.register_node(PSERVER_S2S_RPC_NAME, s2s_->address(), &node_id_);
        if (!st.ok()) throw std::runtime_error("server: cannot register at the master: " + st.to_string());
        c2s_.reset(new RpcServer([this](Bytes&& b, RpcServer::Responder r) { dispatch(std::move(b), r, false); },
                                 cfg_.c2s_thread_num));
        int32_t same = -1;
        st = session_.register_node(PSERVER_C2S_RPC_NAME, c2s_->address(), &same, node_id_);
        if (!st.ok()) throw std::runtime_error("server: cannot register c2s: " + st.to_string());
        PSB_LOG(INFO) << "pserver node " << node_id_ << " serves c2s " << c2s_->address() << ", s2s " << s2s_->address();
        if (cfg_.session_check_ms > 0)
            keeper_ = std::thread([this] {
                std::unique_lock<std::mutex> g(keeper_mu_);
                while (!keeper_cv_.wait_for(g, std::chrono::milliseconds(cfg_.session_check_ms), [this] { return stopped_.load(); })) {
                    g.unlock();
                    ensure_registered();
                    g.lock();
                }
            });
        if (cfg_.report_interval_s > 0)
            reporter_ = std::thread([this] {
                // one line per interval on stderr (ServerConfig::report_interval of the reference)
                std::unique_lock<std::mutex> g(report_mu_);
                while (!report_cv_.wait_for(g, std::chrono::seconds(cfg_.report_interval_s), [this] { return stopped_.load(); })) {
                    // the memory monitor rides on the same interval (Server::self_monitor of the reference,
                    // pico-ps/service/Service.cpp:368-375): tables over a limit stop taking new rows, tables with
                    // room again take them again
                    for (int32_t sid : ctx_.ids()) {
                        auto e = ctx_.get(sid);
                        if (!e) continue;
                        std::shared_lock<std::shared_mutex> tg(e->mu);
                        if (!e->storage) continue;
                        const bool was = e->storage->healthy();
                        const bool now = e->storage->check_healthy();
                        if (was && !now) PSB_LOG(WARNING) << "storage " << sid << " on node " << node_id_ << " is over its memory limit: " << e->storage->memory_usage() << " bytes, new rows are refused";
                        if (!was && now) PSB_LOG(INFO) << "storage " << sid << " on node " << node_id_ << " has room again";
                    }
                    last_report_ = report_line();
                    std::fprintf(stderr, "%s\n", last_report_.c_str());
                }
            });
    }
    ~Server() {
        stop();
        // the thread an EXIT request started may still be inside stop() (or about to enter it): wait for it
        std::lock_guard<std::mutex> g(exit_mu_);
        if (exit_thread_.joinable()) exit_thread_.join();
    }

    // The master's registry is the liveness record: if it no longer lists this node although the node is alive (the
    // master was restarted from its state file, or the session's connection broke), both services are registered
    // again under the same node id. A master that cannot be reached is simply asked again at the next check.
    void ensure_registered() {
        if (leaving_) return;
        std::map<int32_t, std::string> nodes;
        if (!session_.get_nodes(PSERVER_S2S_RPC_NAME, &nodes).ok()) {
            // "recovering" is answered to everybody; registering is what the master waits for
            if (!session_.ping().ok()) return;
        } else if (nodes.count(node_id_)) {
            return;
        }
        if (stopped_ || leaving_) return;
        // A node that the tables' contexts already call DEAD has been (or is about to be) replaced under a new id: it
        // must stay out of the registry, or clients with an old context would find it again and read stale rows.
        for (int32_t sid : ctx_.ids()) {
            std::string json;
            TableDescriptor td;
            if (!session_.get_context(ctx_key(sid), &json).ok() || !td.from_json_str(json)) continue;
            for (auto& n : td.nodes)
                if (n.node_id == node_id_ && n.status == NodeStatus::DEAD) {
                    if (!declared_dead_.exchange(true))
                        PSB_LOG(ERROR) << "pserver node " << node_id_ << " lost its registration and storage " << sid
                                       << " already counts it as dead: it stays out of the registry (start a server in restore mode)";
                    return;
                }
        }
        int32_t same = -1;
        Status a = session_.register_node(PSERVER_S2S_RPC_NAME, s2s_->address(), &same, node_id_);
        Status b = session_.register_node(PSERVER_C2S_RPC_NAME, c2s_->address(), &same, node_id_);
        if (a.ok() && b.ok()) PSB_LOG(WARNING) << "pserver node " << node_id_ << " was missing from the master's registry and registered again";
    }

    // Fault injection on the host: the connection to the master that carries this node's registration is closed, as
    // a network fault between server and master would close it. The master forgets the node until ensure_registered
    // puts it back.
    void drop_master_session() { session_.close(); }

    // "node=.. requests=.. errors=.. storages=[sid:items:bytes ...]"
    std::string report_line() {
        uint64_t requests = 0, errors = 0;
        {
            std::lock_guard<std::mutex> g(metric_mu_);
            for (auto& kv : series_) {
                requests += kv.second.requests;
                errors += kv.second.errors;
            }
        }
        std::string out = "pserver node=" + std::to_string(node_id_) + " requests=" + std::to_string(requests) +
                          " errors=" + std::to_string(errors) + " storages=[";
        bool first = true;
        for (int32_t sid : ctx_.ids()) {
            auto e = ctx_.get(sid);
            if (!e || !e->storage) continue;
            out += std::string(first ? "" : " ") + std::to_string(sid) + ":" + std::to_string(e->storage->size()) + ":" +
                   std::to_string(e->storage->memory_usage());
            first = false;
        }
        return out + "]";
    }
    // Where the data of each table restored by restore_storages came from: "replica", "image" or "dump".
    std::map<int32_t, std::string> restore_sources() {
        std::lock_guard<std::mutex> g(report_mu_);
        return restore_source_;
    }
    std::string last_report() {
        std::lock_guard<std::mutex> g(report_mu_);
        return last_report_;
    }

    int32_t node_id() const { return node_id_; }
    std::string c2s_address() const { return c2s_->address(); }
    std::string s2s_address() const { return s2s_->address(); }
    bool exited() const { return exited_; }
    Context& context() { return ctx_; }

    // Safe to call from several threads: the callers after the first wait until the first one is done, so that
    // nobody destroys the server while its thread pools are still being joined.
    void stop() {
        std::lock_guard<std::mutex> sg(stop_mu_);
        if (stopped_.exchange(true)) return;
        // taking each mutex once orders the flag before the waiter's next look at it: no wake-up is lost
        { std::lock_guard<std::mutex> g(report_mu_); }
        report_cv_.notify_all();
        if (reporter_.joinable()) reporter_.join();
        { std::lock_guard<std::mutex> g(keeper_mu_); }
        keeper_cv_.notify_all();
        if (keeper_.joinable()) keeper_.join();   // before the session closes: it must not register us again
        session_.close();  // the master drops our registrations: we are gone
        if (c2s_) c2s_->stop();
        if (s2s_) s2s_->stop();
    }

    // Counters in the spirit of ps_requests_total / ps_errors_total (pico-ps/service/Service.cpp:23-33).
    // Prometheus text exposition of the per-request series.
    std::string metrics_text() {
        std::lock_guard<std::mutex> g(metric_mu_);
        std::string out;
        auto labels = [&](const std::pair<std::string, int32_t>& k) {
            return "{node_id=\"" + std::to_string(node_id_) + "\",request_type=\"" + k.first + "\",storage_id=\"" + std::to_string(k.second) + "\"";
        };
        out += "# TYPE ps_requests_total counter\n";
        for (auto& kv : series_) out += "ps_requests_total" + labels(kv.first) + "} " + std::to_string(kv.second.requests) + "\n";
        out += "# TYPE ps_errors_total counter\n";
        for (auto& kv : series_) out += "ps_errors_total" + labels(kv.first) + "} " + std::to_string(kv.second.errors) + "\n";
        out += "# TYPE ps_requests_size_bytes counter\n";
        for (auto& kv : series_) out += "ps_requests_size_bytes" + labels(kv.first) + "} " + std::to_string(kv.second.req_bytes) + "\n";
        out += "# TYPE ps_response_size_bytes counter\n";
        for (auto& kv : series_) out += "ps_response_size_bytes" + labels(kv.first) + "} " + std::to_string(kv.second.resp_bytes) + "\n";
        out += "# TYPE ps_request_duration_ms histogram\n";
        for (auto& kv : series_) {
            uint64_t cum = 0;
            for (int b = 0; b <= kDurationBuckets; ++b) {
                cum += kv.second.buckets[b];
                const std::string le = b < kDurationBuckets ? std::to_string(kDurationBoundsMs[b]) : "+Inf";
                out += "ps_request_duration_ms_bucket" + labels(kv.first) + ",le=\"" + le + "\"} " + std::to_string(cum) + "\n";
            }
            out += "ps_request_duration_ms_sum" + labels(kv.first) + "} " + std::to_string(kv.second.sum_ms) + "\n";
            out += "ps_request_duration_ms_count" + labels(kv.first) + "} " + std::to_string(kv.second.requests) + "\n";
        }
        return out;
    }
    std::map<std::string, uint64_t> metrics() {
        std::lock_guard<std::mutex> g(metric_mu_);
        return metrics_;
    }

    // ---------------------------------------------------------------------------------------
    // HA: adopt the descriptors of a dead node in every table and refill the storages.
    Status restore_storages(int* restored_tables = nullptr) {
        std::vector<int32_t> mine;
        Status st;
        // a server started in restore mode may be faster than the detection of the node it is meant to replace:
        // with restore_wait_timeout_s > 0 it keeps looking for a dead node for that long
        const auto t0 = std::chrono::steady_clock::now();
        for (;;) {
            PSB_RETURN_IF_ERROR(master_.acquire_lock(PSERVER_LOCK_NAME));
            st = find_dead_node_and_replace(&mine);
            master_.release_lock(PSERVER_LOCK_NAME);
            PSB_RETURN_IF_ERROR(st);
            const double waited = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
            if (!mine.empty() || cfg_.restore_wait_timeout_s <= 0 || waited >= cfg_.restore_wait_timeout_s) break;
            std::this_thread::sleep_for(std::chrono::milliseconds(100));
        }
        for (int32_t sid : mine) {
            std::shared_ptr<TableEntry> e = ctx_.get(sid);
            {
                std::unique_lock<std::shared_mutex> g(e->mu);
                PSB_RETURN_IF_ERROR(ensure_storage(*e));
            }
            bool paused = false;
            if (cfg_.restore_pauses_writes) PSB_RETURN_IF_ERROR(pause_writes_for_restore(*e, true, &paused));
            // a live replica has the current data; without one, this host's own image of the dead node (if its
            // layout identity matches); then the table's dump
            Status rs = restore_storage_coordinated(*e);
            const char* source = "replica";
            if (!rs.ok()) {
                Status li = restore_storage_from_local_image(*e);
                source = "image";
                if (li.ok()) rs = li;
                else {
                    Status fs = restore_storage_from_fs(*e);
                    source = "dump";
                    rs = fs.ok() ? fs : Status(fs.code(), fs.msg() + " (replica: " + rs.msg() + "; local image: " + li.msg() + ")");
                }
            }
            if (!rs.ok()) {
                PSB_LOG(ERROR) << "storage " << sid << ": restore failed: " << rs.to_string();
                if (paused) pause_writes_for_restore(*e, false, nullptr);   // the table must not stay closed to writes
            }
            PSB_RETURN_IF_ERROR(rs);
            PSB_LOG(INFO) << "storage " << sid << ": restored from " << source << ", " << e->storage->size() << " items on node " << node_id_;
            {
                std::lock_guard<std::mutex> g(report_mu_);
                restore_source_[sid] = source;
            }
            // LOADING -> RUNNING, publish, tell the peers
            PSB_RETURN_IF_ERROR(master_.acquire_lock(PSERVER_LOCK_NAME));
            std::string json;
            st = master_.get_context(ctx_key(sid), &json);
            if (st.ok()) {
                std::unique_lock<std::shared_mutex> g(e->mu);
                e->td.from_json_str(json);
                e->td.set_node_status_to_running(node_id_);
                // writes resume - unless another server is still copying this table: the last one to finish opens it
                if (paused && e->td.status == StorageStatus::LOADING && !others_loading(e->td)) e->td.status = StorageStatus::NORMAL;
                e->rt.build(e->td, node_id_);
                st = master_.set_context(ctx_key(sid), e->td.to_json_str());
            }
            master_.release_lock(PSERVER_LOCK_NAME);
            PSB_RETURN_IF_ERROR(st);
            broadcast_ctx_update(*e);
        }
        if (restored_tables) *restored_tables = (int)mine.size();
        // the images that the replaced node left on this host are used up (this server writes its own, under its own
        // node id), and images of tables that no longer exist are of no use to anybody
        if (!cfg_.local_image_dir.empty() && !mine.empty()) clean_local_images(nullptr);
        return Status::Ok();
    }

    // Housekeeping of `local_image_dir` (DCPmemory::remove_storage / remove_storage_exclude in the reference's restore,
    // pico-ps/service/Service.cpp:284-303; scripts/clear_lvs.sh for whole volumes): removes the images of nodes that
    // this server replaced, of storages that the master no longer knows, and of another layout identity
    // (`version_uuid`) than the table has now. Images of other live nodes' current tables stay.
    Status clean_local_images(int* removed) {
        if (removed) *removed = 0;
        if (cfg_.local_image_dir.empty()) return Status::InvalidConfig("local_image_dir is not set");
        std::set<int> replaced;
        for (auto& kv : replaced_node_) replaced.insert(kv.second);
        std::map<int32_t, std::string> uuid_of;   // storage id -> current version_uuid ("" = unknown to the master)
        for (const std::string& node_dir : list_dir(cfg_.local_image_dir)) {
            if (node_dir.compare(0, 5, "node_") != 0) continue;
            const int node = std::atoi(node_dir.c_str() + 5);
            const std::string dir = cfg_.local_image_dir + "/" + node_dir;
            size_t left = 0;
            for (const std::string& name : list_dir(dir)) {
                const bool is_image = name.compare(0, 8, "storage_") == 0 && name.size() > 12 && name.compare(name.size() - 4, 4, ".img") == 0;
                if (!is_image) {
                    if (name.size() > 4 && name.compare(name.size() - 4, 4, ".tmp") == 0 && node != node_id_) ::unlink((dir + "/" + name).c_str());
                    else ++left;
                    continue;
                }
                const int32_t sid = (int32_t)std::atoi(name.c_str() + 8);
                if (!uuid_of.count(sid)) {
                    std::string json;
                    TableDescriptor td;
                    uuid_of[sid] = master_.get_context(ctx_key(sid), &json).ok() && td.from_json_str(json) ? td.version_uuid : "";
                }
                bool drop = replaced.count(node) || uuid_of[sid].empty();
                if (!drop) drop = image_uuid(dir + "/" + name) != uuid_of[sid];
                if (drop && ::unlink((dir + "/" + name).c_str()) == 0) {
                    if (removed) ++*removed;
                } else {
                    ++left;
                }
            }
            if (left == 0 && node != node_id_) ::rmdir(dir.c_str());
        }
        return Status::Ok();
    }

    // Write the persistent image of every local table under `local_image_dir` (atomically: temp file + rename).
    // Call it at checkpoints or before a planned shutdown; see restore_storage_from_local_image.
    Status save_local_images(int* n_tables = nullptr) {
        if (cfg_.local_image_dir.empty()) return Status::InvalidConfig("local_image_dir is not set");
        int saved = 0;
        for (int32_t sid : ctx_.ids()) {
            auto e = ctx_.get(sid);
            if (!e || !e->storage) continue;
            std::shared_lock<std::shared_mutex> g(e->mu);
            const std::string path = image_path(cfg_.local_image_dir, node_id_, sid);
            PSB_RETURN_IF_ERROR(mkdir_p(path.substr(0, path.rfind('/'))));
            const std::string tmp = path + ".tmp";
            {
                std::ofstream f(tmp, std::ios::binary | std::ios::trunc);
                if (!f) return Status::Error("cannot write " + tmp);
                const char magic[8] = {'P', 'S', 'B', 'I', 'M', 'G', '1', 0};
                const uint64_t ulen = e->td.version_uuid.size();
                const uint32_t stride = e->storage->stride();
                uint64_t n = 0;
                f.write(magic, 8);
                f.write((const char*)&ulen, 8);
                f.write(e->td.version_uuid.data(), (std::streamsize)ulen);
                f.write((const char*)&stride, 4);
                const auto n_pos = f.tellp();
                f.write((const char*)&n, 8);
                for (int s : e->storage->shard_list()) {
                    PSB_RETURN_IF_ERROR(e->storage->scan_shard(s, 1 << 14, false, [&](const std::vector<int64_t>& keys, const std::vector<float>& rows) {
                        for (size_t i = 0; i < keys.size(); ++i) {
                            f.write((const char*)&keys[i], 8);
                            f.write((const char*)(rows.data() + i * stride), (std::streamsize)stride * 4);
                        }
                        n += keys.size();
                        return Status::Ok();
                    }));
                }
                f.seekp(n_pos);
                f.write((const char*)&n, 8);
                if (!f.good()) return Status::Error("write to " + tmp + " failed");
            }
            if (std::rename(tmp.c_str(), path.c_str()) != 0) return Status::Error("cannot move " + tmp + " into place");
            ++saved;
        }
        if (n_tables) *n_tables = saved;
        return Status::Ok();
    }

    // ---------------------------------------------------------------------------------------
    // Incremental sync (trainer -> predictor, pico-ps/service/Service.cpp:1467-1540): start recording
    // which rows change, then stream the changed rows of the local shards through `send_block` in
    // blocks; the marks are cleared only when every block went through, so a failed round is simply
    // repeated (the reference rewinds its iterator clone).
    Status enable_sync(int32_t sid) {
        auto e = ctx_.get(sid);
        if (!e || !e->storage) return Status::InvalidID("no storage " + std::to_string(sid));
        std::shared_lock<std::shared_mutex> g(e->mu);
        ensure_tracking(*e);
        return Status::Ok();
    }

    // ---------------------------------------------------------------------------------------
    // Hook of the sync thread (pico-ps/service/Service.cpp:1467-1540; the thread itself lives in
    // service/table_syncer.h because it drives handlers, which sit above this header). The listener is called with
    // (storage id, deleted) after every applied async push or store on a table whose push operator names follower
    // tables (`sync_table` in its config), and once more when such a table is deleted. It must only take a note and
    // return: it runs on a request thread.
    using SyncListener = std::function<void(int32_t, bool)>;
    void set_sync_listener(SyncListener fn) {
        std::lock_guard<std::mutex> g(listener_mu_);
        sync_listener_ = fn ? std::make_shared<SyncListener>(std::move(fn)) : nullptr;
    }
    // The follower tables named by the push operators of table `sid`.
    std::vector<SparseTablePushOperator::SyncTarget> sync_targets(int32_t sid) {
        std::vector<SparseTablePushOperator::SyncTarget> out;
        auto e = ctx_.get(sid);
        if (!e) return out;
        std::shared_lock<std::shared_mutex> g(e->mu);
        for (auto& kv : e->ops)
            if (auto p = std::dynamic_pointer_cast<SparseTablePushOperator>(kv.second))
                out.insert(out.end(), p->sync_tables().begin(), p->sync_tables().end());
        return out;
    }
    Status push_sync_table(int32_t sid, size_t block,
                           const std::function<Status(const int64_t*, const float*, size_t, uint32_t)>& send_block,
                           uint64_t* n_synced, bool clear_marks = true) {
        auto e = ctx_.get(sid);
        if (!e || !e->storage) return Status::InvalidID("no storage " + std::to_string(sid));
        *n_synced = 0;
        std::unique_lock<std::shared_mutex> flip(e->incr.mu);  // pushes wait while the increment is collected
        if (!e->incr.updated) return Status::Ok();
        std::vector<int64_t> keys;
        std::vector<float> rows;
        for (int s : e->storage->shard_list()) {
            uint64_t cursor = 0;
            bool finished = false;
            while (!finished) {
                keys.clear();
                rows.clear();
                PSB_RETURN_IF_ERROR(e->storage->export_shard(s, cursor, std::max<size_t>(block, 64) * 4, true, &keys, &rows, &cursor, &finished));
                for (size_t off = 0; off < keys.size(); off += block) {
                    const size_t m = std::min(block, keys.size() - off);
                    PSB_RETURN_IF_ERROR(send_block(keys.data() + off, rows.data() + off * e->storage->stride(), m, e->storage->stride()));
                    *n_synced += m;
                }
            }
        }
        if (clear_marks) {   // with several followers only the pass for the last one clears
            e->storage->clear_dirty();
            e->incr.updated = false;
        }
        return Status::Ok();
    }

private:
    // ------------------------------------------------------------------------- plumbing
    static Bytes reply(const Status& st, const Archive* payload, const PSMessageMeta& meta) {
        Archive out;
        out << st;
        if (payload) out.write_raw(payload->data(), payload->size());
        out << meta;
        return out.release();
    }
    void count(const std::string& name) {
        std::lock_guard<std::mutex> g(metric_mu_);
        ++metrics_[name];
    }
    // Per (request type, storage) series in the spirit of ps_requests_total / ps_requests_size_bytes /
    // ps_response_size_bytes / ps_errors_total / ps_request_duration_ms_bucket
    // (pico-ps/service/Service.cpp:23-33).
    struct Series {
        uint64_t requests = 0, errors = 0, req_bytes = 0, resp_bytes = 0;
        double sum_ms = 0;
        uint64_t buckets[kDurationBuckets + 1] = {};
    };
    void observe(const std::string& type, int32_t sid, size_t req_bytes, size_t resp_bytes, bool error, double ms) {
        std::lock_guard<std::mutex> g(metric_mu_);
        Series& x = series_[{type, sid}];
        ++x.requests;
        x.errors += error ? 1 : 0;
        x.req_bytes += req_bytes;
        x.resp_bytes += resp_bytes;
        x.sum_ms += ms;
        int b = 0;
        while (b < kDurationBuckets && ms > kDurationBoundsMs[b]) ++b;
        ++x.buckets[b];
    }

    void dispatch(Bytes&& bytes, RpcServer::Responder resp, bool s2s) {
        PSMessage msg = PSMessage::open(std::move(bytes));
        const PSMessageMeta meta = msg.meta;
        Archive out;
        Status st;
        const std::string label = std::string(s2s ? "s2s_" : "c2s_") + request_type_label(meta.req_type);
        count(label);
        const size_t req_bytes = msg.ar.size();
        const auto t0 = std::chrono::steady_clock::now();
        try {
            // A node that the tables count as dead (see ensure_registered) answers data requests of clients from
            // TIMEOUT, the status that makes a client look at the registry and the published context again; requests
            // of other servers (a replacement fetching shards) and the admin's EXIT are still served.
            const bool data_op = meta.req_type == RequestType::OP_PULL || meta.req_type == RequestType::OP_PUSH_ASYNC ||
                                 meta.req_type == RequestType::OP_PUSH_SYNC || meta.req_type == RequestType::OP_STORE;
            if (meta.req_type == RequestType::EXIT) {
                // leave the registry before the answer goes out: whoever asked this node to leave must not find it
                // listed any more once the call has returned
                leaving_ = true;
                session_.deregister_node(PSERVER_C2S_RPC_NAME, node_id_);
                session_.deregister_node(PSERVER_S2S_RPC_NAME, node_id_);
            }
            if (!s2s && data_op && declared_dead_.load()) st = Status::Timeout("node " + std::to_string(node_id_) + " has been replaced");
            else st = process(msg, &out, s2s);
        } catch (const std::exception& ex) {
            st = Status::Error(std::string("server exception: ") + ex.what());
        }
        if (!st.ok()) count("errors_total");
        observe(label, meta.sid, req_bytes, out.size(), !st.ok(),
                std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count());
        resp.send(reply(st, &out, meta));
        if (meta.req_type == RequestType::EXIT && !exited_.exchange(true)) {
            PSB_LOG(INFO) << "pserver node " << node_id_ << " was asked to leave";
            // stop() joins the worker pools, this thread among them: it runs on a thread of its own, which the
            // destructor joins
            std::lock_guard<std::mutex> g(exit_mu_);
            exit_thread_ = std::thread([this] { stop(); });
        }
    }

    // Self-healing of a server that is behind: when a request carries a context version (or update version)
    // that this server has not seen, the context is fetched from the master and installed under the table's
    // exclusive lock BEFORE the request takes its shared lock. The version gates below only compare.
    void refresh_if_behind(TableEntry& e, const PSMessageMeta& meta) {
        bool behind = false;
        {
            std::shared_lock<std::shared_mutex> g(e.mu);
            behind = meta.ctx_ver > e.td.version || (meta.ctx_u_ver >= 0 && meta.ctx_u_ver != e.td.update_version);
        }
        if (!behind) return;
        std::string json;
        if (!master_.get_context(ctx_key(e.sid), &json).ok()) return;
        std::unique_lock<std::shared_mutex> g(e.mu);
        if (meta.ctx_ver > e.td.version || (meta.ctx_u_ver >= 0 && meta.ctx_u_ver != e.td.update_version)) apply_ctx_json(e, json);
    }
    // Context version gates (callers hold the table's lock).
    Status check_ctx_version(TableEntry& e, const PSMessageMeta& meta) {
        if (meta.ctx_ver > e.td.version) return Status::ServerTooOldCtx("server context older than the client's");
        if (meta.ctx_ver < e.td.version) return Status::ServerTooNewCtx("server context newer than the client's");
        return Status::Ok();
    }
    Status check_write_ctx_version(TableEntry& e, const PSMessageMeta& meta) {
        PSB_RETURN_IF_ERROR(check_ctx_version(e, meta));
        if (e.td.status == StorageStatus::RESHARD) return Status::OOM("write when update context");
        if (e.td.status == StorageStatus::LOADING) return Status::OOM("write while a replica of the table is being restored");
        return Status::Ok();
    }
    Status check_table_version(TableEntry& e, const PSMessageMeta& meta) {
        if (meta.ctx_ver != e.td.version) return meta.ctx_ver > e.td.version ? Status::ServerTooOldCtx("ctx") : Status::ServerTooNewCtx("ctx");
        if (meta.ctx_u_ver != e.td.update_version)
            return meta.ctx_u_ver > e.td.update_version ? Status::ServerTooOldCtxU("update ctx") : Status::ServerTooNewCtxU("update ctx");
        return Status::Ok();
    }

    Status ensure_storage(TableEntry& e) {
        if (e.storage) return Status::Ok();
        auto* sop = static_cast<SparseTableStorageOperator*>(e.storage_op.get());
        return sop->create_storage(e.rt.global_shard_num(), e.rt.local_shards(), &e.storage);
    }

    // Install a context JSON on an existing entry: refresh runtime info, match local shards, and swap
    // in the reshard result when the new placement has been committed.
    void apply_ctx_json(TableEntry& e, const std::string& json) {
        Json j;
        if (!Json::parse(json, &j)) return;
        const int32_t old_uv = e.td.update_version;
        const bool had_update = !e.td.update_nodes.empty();
        if (!e.td.from_json(j, true)) return;
        e.rt.build(e.td, node_id_);
        e.update_rt.build(e.td, node_id_, true);
        e.update_handlers();
        const bool committed = had_update && e.td.update_nodes.empty() && e.td.update_version > old_uv;
        if (committed && e.update_storage) {
            e.storage = std::move(e.update_storage);  // the reshuffled data becomes the serving data
            PSB_LOG(INFO) << "storage " << e.sid << ": reshard committed on node " << node_id_ << ", update version " << e.td.update_version << ", " << e.storage->size() << " items";
            // the rows arrived marked (see process_new_ctx_create_shard): the next sync round re-ships them
            if (e.sync_enabled) e.incr.updated = true;
        } else if (e.storage) {
            // plain placement change (e.g. a dead node replaced): create / drop local shards to match
            if (e.storage->n_shards() == e.rt.global_shard_num()) {
                for (int s : e.storage->shard_list())
                    if (!e.rt.local_shards().count(s)) e.storage->erase_shard(s);
                for (int s : e.rt.local_shards())
                    if (!e.storage->has_shard(s)) e.storage->create_shard(s);
            }
        }
    }

    Status refresh_from_master(int32_t sid, std::shared_ptr<TableEntry>* out) {
        std::string json;
        PSB_RETURN_IF_ERROR(master_.get_context(ctx_key(sid), &json));
        std::shared_ptr<TableEntry> e = ctx_.get(sid);
        if (!e) {
            PSB_RETURN_IF_ERROR(ctx_.set_table_descriptor(sid, json, node_id_, &e));
            std::unique_lock<std::shared_mutex> g(e->mu);
            PSB_RETURN_IF_ERROR(ensure_storage(*e));
        } else {
            std::unique_lock<std::shared_mutex> g(e->mu);
            apply_ctx_json(*e, json);
        }
        if (out) *out = e;
        return Status::Ok();
    }

    Status peers(const char* service, std::map<int32_t, std::string>* nodes) { return master_.get_nodes(service, nodes); }

    // Fan a request out to servers over s2s and collect the statuses.
    Status s2s_call(const std::map<int, Archive>& bodies, PSMessageMeta meta, RequestType type) {
        std::map<int32_t, std::string> nodes;
        PSB_RETURN_IF_ERROR(peers(PSERVER_S2S_RPC_NAME, &nodes));
        meta.req_type = type;
        std::vector<RpcClient::Ticket> tickets;
        for (auto& kv : bodies) {
            auto it = nodes.find(kv.first);
            if (it == nodes.end()) return Status::NoReplica("s2s: node " + std::to_string(kv.first) + " is not registered");
            PSMessage m;
            m.ar = kv.second;
            m.meta = meta;
            tickets.push_back(s2s_client_.send(it->second, m.seal()));
        }
        Status result;
        for (auto& t : tickets) {
            Bytes b;
            Status st = s2s_client_.wait(t, cfg_.s2s_timeout_ms, &b);
            if (st.ok()) {
                PSMessage r = PSMessage::open(std::move(b));
                r.ar >> st;
            }
            if (!st.ok() && result.ok()) result = st;
        }
        return result;
    }

    void broadcast_ctx_update(TableEntry& e) {
        std::map<int32_t, std::string> nodes;
        if (!peers(PSERVER_C2S_RPC_NAME, &nodes).ok()) return;
        PSMessage m;
        m.meta.sid = e.sid;
        m.meta.req_type = RequestType::CTX_UPDATE;
        std::vector<RpcClient::Ticket> tickets;
        for (auto& kv : nodes)
            if (kv.first != node_id_) tickets.push_back(s2s_client_.send(kv.second, m.seal()));
        for (auto& t : tickets) {
            Bytes b;
            s2s_client_.wait(t, 5000, &b);
        }
    }

    // ------------------------------------------------------------------------- dispatch
    Status process(PSMessage& msg, Archive* out, bool s2s) {
        const PSMessageMeta& meta = msg.meta;
        Archive& in = msg.ar;
        switch (meta.req_type) {
            case RequestType::HEALTH_CHECK: *out << node_id_; return Status::Ok();
            case RequestType::EXIT: return Status::Ok();
            case RequestType::OP_LOAD_LIBRARY: {
                std::string path;
                in >> path;
                return OperatorFactory::instance().load_library(path);
            }
            case RequestType::MEMORY_INFO: {
                NodeMemoryInfo mi;
                for (int32_t sid : ctx_.ids()) {
                    auto e = ctx_.get(sid);
                    if (!e || !e->storage) continue;
                    mi.healthy = mi.healthy && e->storage->healthy();
                    mi.used += e->storage->memory_usage();
                    mi.managed += e->storage->memory_usage();
                }
                *out << (int32_t)(mi.healthy ? 1 : 0) << mi.used << mi.managed;
                return Status::Ok();
            }
            case RequestType::STORAGE_CREATE: return process_create_storage(meta, in);
            case RequestType::CTX_UPDATE: return refresh_from_master(meta.sid, nullptr);
            default: break;
        }
        std::shared_ptr<TableEntry> e = ctx_.get(meta.sid);
        if (!e) {
            // a server that joined later (new node of a reshard, restored node) learns tables lazily
            Status st = refresh_from_master(meta.sid, &e);
            if (!st.ok() || !e) return Status::InvalidID("no storage " + std::to_string(meta.sid) + " on node " + std::to_string(node_id_));
        }
        if (meta.ctx_ver >= 0) refresh_if_behind(*e, meta);
        switch (meta.req_type) {
            case RequestType::STORAGE_DELETE: {
                auto gone = ctx_.get(meta.sid);
                const bool followed = gone && gone->sync_enabled;
                // the table's saved image goes with it, unless its storage config asks to keep it
                if (gone && gone->storage_op && !cfg_.local_image_dir.empty() && !storage_op_of(*gone)->retain_local_image())
                    ::unlink(image_path(cfg_.local_image_dir, node_id_, meta.sid).c_str());
                ctx_.erase(meta.sid);
                PSB_LOG(INFO) << "storage " << meta.sid << " deleted on node " << node_id_;
                if (followed) notify_sync(meta.sid, true);
                return Status::Ok();
            }
            case RequestType::STORAGE_CLEAR: {
                std::shared_lock<std::shared_mutex> g(e->mu);
                PSB_RETURN_IF_ERROR(check_write_ctx_version(*e, meta));
                PSB_RETURN_IF_ERROR(e->storage->clear());
                for (int s : e->rt.local_shards()) e->storage->create_shard(s);
                return Status::Ok();
            }
            case RequestType::STORAGE_STATISTIC: {
                std::shared_lock<std::shared_mutex> g(e->mu);
                std::vector<int> shards = e->storage->shard_list();
                *out << (int32_t)shards.size();
                for (int s : shards)
                    *out << (uint64_t)e->storage->shard_size(s) << (uint64_t)(e->storage->memory_usage() / std::max<size_t>(1, shards.size()))
                         << node_id_ << (int32_t)s;
                return Status::Ok();
            }
            case RequestType::HANDLER_REGISTER: {
                std::unique_lock<std::shared_mutex> g(e->mu);
                int32_t hid = 0;
                OperatorDescriptor d;
                in >> hid >> d.key >> d.lib_name >> d.op_name >> d.config_str;
                // nothing is touched unless the operator exists and can be built; a failed registration leaves the
                // table's handlers as they were
                if (hid < 0 || !OperatorFactory::instance().has(d.lib_name, d.op_name))
                    return Status::InvalidConfig("register handler: no operator (" + d.lib_name + ", " + d.op_name + ")");
                const auto before = e->td.handlers;
                e->td.handlers[hid] = d;
                e->td.refresh_info();
                Status st = e->update_handlers();
                if (!st.ok()) {
                    e->td.handlers = before;
                    e->td.refresh_info();
                    e->update_handlers();
                }
                return st;
            }
            case RequestType::HANDLER_DEREGISTER: {
                std::unique_lock<std::shared_mutex> g(e->mu);
                int32_t hid = 0;
                in >> hid;
                e->td.handlers.erase(hid);
                e->td.refresh_info();
                return e->update_handlers();
            }
            case RequestType::OP_PULL: return process_pull(*e, meta, in, out);
            case RequestType::OP_PUSH_ASYNC:
                if (s2s) return process_direct_push(*e, in, false);
                return process_push(*e, meta, in, false);
            case RequestType::OP_PUSH_SYNC: return process_push(*e, meta, in, true);
            case RequestType::OP_STORE: {
                std::shared_lock<std::shared_mutex> g(e->mu);
                PSB_RETURN_IF_ERROR(check_write_ctx_version(*e, meta));
                auto op = find_op<SparseTablePushOperator>(*e, meta.hid);
                if (!op) return Status::InvalidID("store: handler is not a push operator");
                Status st = op->apply_store(*e);
                if (st.ok() && !op->sync_tables().empty()) notify_sync(meta.sid, false);
                return st;
            }
            case RequestType::OP_FOREACH:
            case RequestType::OP_ERASEIF:
            case RequestType::OP_DUMP: return process_for_each(*e, meta, in, out);
            case RequestType::OP_LOAD: return process_load(*e, meta, in, out);
            case RequestType::OP_SYNC: {
                std::shared_lock<std::shared_mutex> g(e->mu);
                PSB_RETURN_IF_ERROR(check_write_ctx_version(*e, meta));
                auto op = find_op<KVSyncOperator>(*e, meta.hid);
                if (!op) return Status::InvalidID("sync: handler is not a sync operator");
                Bytes raw;
                in >> raw;
                std::vector<uint8_t> plain;
                PSB_RETURN_IF_ERROR(op->compressor().decompress(raw.data(), raw.size(), &plain));
                Archive body(std::move(plain));
                if (!e->storage->healthy()) return Status::OOM("storage unhealthy");
                return DirectPushOperator::apply_request(e->storage.get(), body);
            }
            case RequestType::OP_UDF: {
                std::shared_lock<std::shared_mutex> g(e->mu);
                auto op = find_op<UDFOperator>(*e, meta.hid);
                if (!op) return Status::InvalidID("udf: handler is not a udf operator");
                PSB_RETURN_IF_ERROR(op->read_only() ? check_ctx_version(*e, meta) : check_write_ctx_version(*e, meta));
                std::string param, result;
                in >> param;
                PSB_RETURN_IF_ERROR(op->apply_request(*e, param, &result));
                *out << result;
                return Status::Ok();
            }
            case RequestType::OP_COORDINATED_RESTORE_ITERATE: return process_restore_iterate(*e, in, out);
            case RequestType::NEW_CTX_CREATE_SHARD: return process_new_ctx_create_shard(*e, meta);
            case RequestType::NEW_CTX_SHUFFLE:
                if (s2s) return process_direct_push(*e, in, true);
                return process_new_ctx_shuffle(*e, meta, in);
            case RequestType::NEW_CTX_STORE: {
                std::shared_lock<std::shared_mutex> g(e->mu);
                PSB_RETURN_IF_ERROR(check_table_version(*e, meta));
                if (e->update_rt.local_shards().empty()) return Status::Ok();
                return e->update_storage ? Status::Ok() : Status::Error("new ctx store: no update storage on this node");
            }
            case RequestType::NEW_CTX_PURGE: {
                std::unique_lock<std::shared_mutex> g(e->mu);
                return update_ctx_op(*e)->apply_purge_request(*e);
            }
            default: return Status::Error(std::string("unhandled request type ") + request_type_name(meta.req_type));
        }
    }

    template <class OP>
    std::shared_ptr<OP> find_op(TableEntry& e, int32_t hid) {
        auto it = e.ops.find(hid);
        if (it == e.ops.end()) return nullptr;
        return std::dynamic_pointer_cast<OP>(it->second);
    }

    // ------------------------------------------------------------------------- storage life cycle
    Status process_create_storage(const PSMessageMeta& meta, Archive& in) {
        std::string lib, op, cfg_str;
        in >> lib >> op >> cfg_str;
        Json cfg;
        if (!Json::parse_config(cfg_str, &cfg)) return Status::InvalidConfig("storage config is neither valid JSON nor YAML");
        std::shared_ptr<TableEntry> e;
        PSB_RETURN_IF_ERROR(ctx_.create_storage(meta.sid, lib, op, cfg, node_id_, &e));
        if (std::string(e->storage_op->kind()) != "storage") return Status::InvalidConfig(op + " is not a storage operator");
        std::unique_lock<std::shared_mutex> g(e->mu);
        Status st = ensure_storage(*e);
        if (!st.ok()) ctx_.erase(meta.sid);
        else PSB_LOG(INFO) << "storage " << meta.sid << " created on node " << node_id_ << " with " << e->rt.local_shards().size() << " local shards";
        return st;
    }

    // ------------------------------------------------------------------------- data path
    Status process_pull(TableEntry& e, const PSMessageMeta& meta, Archive& in, Archive* out) {
        std::shared_lock<std::shared_mutex> g(e.mu);
        auto op = find_op<SparseTablePullOperator>(e, meta.hid);
        if (!op) return Status::InvalidID("pull: handler " + std::to_string(meta.hid) + " is not a pull operator");
        // read-only pulls keep working during a reshard; pulls that may insert are writes
        PSB_RETURN_IF_ERROR(op->read_only() ? check_ctx_version(e, meta) : check_write_ctx_version(e, meta));
        if (!e.storage) return Status::InvalidID("no storage");
        return op->apply_request(e, in, out);
    }
    Status process_push(TableEntry& e, const PSMessageMeta& meta, Archive& in, bool sync) {
        std::shared_lock<std::shared_mutex> g(e.mu);
        auto op = find_op<SparseTablePushOperator>(e, meta.hid);
        if (!op) return Status::InvalidID("push: handler " + std::to_string(meta.hid) + " is not a push operator");
        PSB_RETURN_IF_ERROR(check_write_ctx_version(e, meta));
        const bool followed = !op->sync_tables().empty() && has_sync_listener();
        // rows must be marked from the first push on, so the marks are switched on before it is applied
        if (followed) ensure_tracking(e);
        Status st = op->apply_request(e, in, sync);
        if (st.ok() && followed && !sync) notify_sync(meta.sid, false);   // a sync push changes nothing before its store
        return st;
    }
    // The flag is raised only after the storage records changes, so a push that sees it set is recorded.
    static void ensure_tracking(TableEntry& e) {
        if (e.sync_enabled.load(std::memory_order_acquire)) return;
        std::lock_guard<std::mutex> g(e.sync_mu);
        if (!e.sync_enabled.load(std::memory_order_relaxed)) {
            e.storage->enable_dirty_tracking();
            e.sync_enabled.store(true, std::memory_order_release);
        }
    }
    bool has_sync_listener() {
        std::lock_guard<std::mutex> g(listener_mu_);
        return sync_listener_ != nullptr;
    }
    void notify_sync(int32_t sid, bool deleted) {
        std::shared_ptr<SyncListener> fn;
        {
            std::lock_guard<std::mutex> g(listener_mu_);
            fn = sync_listener_;
        }
        if (fn) (*fn)(sid, deleted);
    }
    Status process_direct_push(TableEntry& e, Archive& in, bool into_update) {
        std::shared_lock<std::shared_mutex> g(e.mu);
        KVStorage* dst = into_update ? e.update_storage.get() : e.storage.get();
        if (!dst) return Status::Error(into_update ? "shuffle target has no update storage" : "no storage");
        if (!dst->healthy()) return Status::OOM("storage unhealthy");
        return DirectPushOperator::apply_request(dst, in);
    }

    Status process_for_each(TableEntry& e, const PSMessageMeta& meta, Archive& in, Archive* out) {
        std::shared_lock<std::shared_mutex> g(e.mu);
        PSB_RETURN_IF_ERROR(check_write_ctx_version(e, meta));
        if (meta.req_type == RequestType::OP_DUMP) {
            auto op = find_op<DumpOperator>(e, meta.hid);
            if (!op) return Status::InvalidID("dump: handler is not a dump operator");
            DumpArgs args;
            int32_t file_id = 0;
            std::vector<int32_t> shards;
            in >> args.uri >> args.file_number >> file_id >> shards;
            uint64_t n = 0;
            PSB_RETURN_IF_ERROR(op->apply_request(e, node_id_, args, file_id, shards, &n));
            *out << n;
            return Status::Ok();
        }
        int32_t shard = 0;
        std::string carried_str;
        in >> shard >> carried_str;
        Json carried = Json::object();
        if (!carried_str.empty() && !Json::parse(carried_str, &carried)) return Status::InvalidConfig("carried item is not JSON");
        if (meta.req_type == RequestType::OP_ERASEIF) {
            auto op = find_op<EraseIfOperatorBase>(e, meta.hid);
            if (!op) return Status::InvalidID("erase_if: handler is not an erase_if operator");
            uint64_t erased = 0;
            PSB_RETURN_IF_ERROR(op->apply_request(e, shard, carried, &erased));
            *out << erased;
            return Status::Ok();
        }
        auto op = find_op<ForEachOperatorBase>(e, meta.hid);
        if (!op) return Status::InvalidID("for_each: handler is not a for_each operator");
        std::string result;
        PSB_RETURN_IF_ERROR(op->apply_request(e, shard, carried, &result));
        *out << result;   // bytes whose layout the operator defines
        if (op->writes() && e.sync_enabled.load(std::memory_order_acquire)) notify_sync(meta.sid, false);   // followers get the changed rows
        return Status::Ok();
    }

    // load: {uri, need_rehash, files}. need_rehash: stream the files and DirectPush every block to the
    // owners over s2s (works across different shardings); else keep only the local keys.
    Status process_load(TableEntry& e, const PSMessageMeta& meta, Archive& in, Archive* out) {
        std::shared_lock<std::shared_mutex> g(e.mu);
        auto op = find_op<LoadOperator>(e, meta.hid);
        if (!op) return Status::InvalidID("load: handler is not a load operator");
        std::string uri;
        int32_t need_rehash = 0;
        std::vector<std::string> files;
        in >> uri >> need_rehash >> files;
        std::string dir, format;
        DumpArgs::split_uri(uri, &dir, &format);
        if (files.empty()) files = list_model_files(dir);
        const auto* sop = storage_op_of(e);
        const size_t block = op->block_size() ? op->block_size() : (size_t)cfg_.load_block_size;
        // the files of one request are read by up to load_thread_num threads (ServerConfig of the reference:
        // load_thread_num = 4, load_block_size = 1000)
        auto load_one = [&](const std::string& f, uint64_t* count) -> Status {
            if (!need_rehash) return op->restore_file(e, f, format, count);
            DsReader r;
            PSB_RETURN_IF_ERROR(r.open(f, format, e.storage->stride(), &op->compressor()));
            std::vector<int64_t> keys;
            std::vector<float> rows;
            while (r.next_block(block, &keys, &rows)) {
                std::map<int, Archive> bodies;
                PSB_RETURN_IF_ERROR(DirectPushOperator::generate_requests(sop, e.rt, keys.data(), rows.data(), keys.size(),
                                                                          e.storage->stride(), &bodies));
                PSMessageMeta m = meta;
                PSB_RETURN_IF_ERROR(s2s_call(bodies, m, RequestType::OP_PUSH_ASYNC));
                *count += keys.size();
            }
            if (!r.ok()) return Status::Error(f + ": damaged dump file (a record is cut short or does not parse)");
            return Status::Ok();
        };
        std::atomic<size_t> next{0};
        std::atomic<uint64_t> total{0};
        std::mutex first_mu;
        Status first;
        auto worker = [&] {
            for (;;) {
                const size_t i = next++;
                if (i >= files.size()) return;
                uint64_t c = 0;
                Status st = load_one(files[i], &c);
                total += c;
                if (!st.ok()) {
                    std::lock_guard<std::mutex> lg(first_mu);
                    if (first.ok()) first = st;
                }
            }
        };
        const int nthreads = (int)std::min<size_t>(std::max(1, cfg_.load_thread_num), files.size());
        std::vector<std::thread> pool;
        for (int t = 1; t < nthreads; ++t) pool.emplace_back(worker);
        worker();
        for (auto& t : pool) t.join();
        PSB_RETURN_IF_ERROR(first);
        const uint64_t n = total;
        *out << n;
        return Status::Ok();
    }

    // ------------------------------------------------------------------------- reshard
    // The table's reshard codec: the update_ctx operator registered for it (a plug-in may have replaced it), else the
    // built-in one with default settings.
    std::shared_ptr<ShardUpdateContextOperator> update_ctx_op(TableEntry& e) {
        for (auto& kv : e.ops)
            if (auto u = std::dynamic_pointer_cast<ShardUpdateContextOperator>(kv.second)) return u;
        return std::make_shared<ShardUpdateContextOperator>(Json::object());
    }
    Status process_new_ctx_create_shard(TableEntry& e, const PSMessageMeta& meta) {
        std::unique_lock<std::shared_mutex> g(e.mu);
        PSB_RETURN_IF_ERROR(check_table_version(e, meta));
        return update_ctx_op(e)->create_new_shards(e);
    }
    // One old shard: stream its items in blocks to the owners under the NEW placement.
    Status process_new_ctx_shuffle(TableEntry& e, const PSMessageMeta& meta, Archive& in) {
        std::shared_lock<std::shared_mutex> g(e.mu);
        PSB_RETURN_IF_ERROR(check_table_version(e, meta));
        int32_t old_shard = 0;
        in >> old_shard;
        return update_ctx_op(e)->generate_shuffle_requests(e, old_shard, [&](const std::map<int, Archive>& bodies) {
            return s2s_call(bodies, meta, RequestType::NEW_CTX_SHUFFLE);
        });
    }

    // ------------------------------------------------------------------------- HA restore
    // Replica side of coordinated restore: {iterator_id, offset, batch_size, shard_id} -> one batch.
    Status process_restore_iterate(TableEntry& e, Archive& in, Archive* out) {
        std::shared_lock<std::shared_mutex> g(e.mu);
        int32_t iterator_id = -1, shard = -1;
        uint64_t offset = 0, batch = 0;
        in >> iterator_id >> offset >> batch >> shard;
        if (!e.storage || !e.storage->has_shard(shard)) return Status::InvalidID("restore: shard is not on this node");
        // The iterator remembers under which layout of the index its cursor was taken. Pushes go on between two
        // batches and may make the index rebuild itself; the cursor then means nothing, and the iteration starts over
        // from the first bucket (the restoring side overwrites, so rows that it gets twice do no harm). A cursor that
        // comes without a known iterator (this server was restarted in between) starts over as well.
        uint64_t epoch = 0;
        bool known = false;
        {
            std::lock_guard<std::mutex> ig(e.iter_mu);
            auto it = iterator_id < 0 ? e.restore_iters.end() : e.restore_iters.find(iterator_id);
            if (it != e.restore_iters.end() && it->second.shard == shard) {
                epoch = it->second.epoch;
                known = true;
            } else {
                iterator_id = e.next_iter_id++;
                e.restore_iters[iterator_id] = RestoreIterator{shard, 0, 0};
            }
        }
        std::vector<int64_t> keys;
        std::vector<float> rows;
        uint64_t next = offset;
        bool finished = false;
        for (int attempt = 0;; ++attempt) {
            const uint64_t now = e.storage->layout_epoch(shard);
            if (!known || now != epoch) offset = 0;
            keys.clear();
            rows.clear();
            PSB_RETURN_IF_ERROR(e.storage->export_shard(shard, offset, std::max<uint64_t>(batch, 1), false, &keys, &rows, &next, &finished));
            epoch = now;
            known = true;
            if (e.storage->layout_epoch(shard) == now) break;   // nothing moved under the export
            known = false;
            if (attempt == 8) return Status::Error("restore: the index of shard " + std::to_string(shard) + " keeps being rebuilt");
        }
        {
            std::lock_guard<std::mutex> ig(e.iter_mu);
            if (finished) e.restore_iters.erase(iterator_id);
            else e.restore_iters[iterator_id] = RestoreIterator{shard, next, epoch};
        }
        *out << e.sid << shard << (int32_t)(finished ? 1 : 0) << iterator_id << next << (uint64_t)keys.size() << (int32_t)e.storage->stride();
        out->write_raw(keys.data(), keys.size() * 8);
        out->write_raw(rows.data(), rows.size() * 4);
        return Status::Ok();
    }

    // Close (or open again) a table to writes around a restore: the status LOADING is published under the global lock
    // and handed to every reachable server before the first row is copied, so no push is applied anywhere between a
    // row's export and the end of the restore. A table in the middle of a reshard is left alone (*paused stays false).
    // Whether another server is still copying this table. A LOADING entry whose server is no longer registered (its
    // restore failed and the process went away) does not count: it must not keep the table closed.
    bool others_loading(const TableDescriptor& td) {
        std::map<int32_t, std::string> live;
        if (!master_.get_nodes(PSERVER_S2S_RPC_NAME, &live).ok()) return false;
        for (auto& n : td.nodes)
            if (n.status == NodeStatus::LOADING && n.node_id != node_id_ && live.count(n.node_id)) return true;
        return false;
    }
    Status pause_writes_for_restore(TableEntry& e, bool on, bool* paused) {
        if (paused) *paused = false;
        PSB_RETURN_IF_ERROR(master_.acquire_lock(PSERVER_LOCK_NAME));
        std::string json;
        Status st = master_.get_context(ctx_key(e.sid), &json);
        bool changed = false, notify = false;
        if (st.ok()) {
            std::unique_lock<std::shared_mutex> g(e.mu);
            e.td.from_json_str(json);
            if (on && e.td.status == StorageStatus::NORMAL) {
                e.td.status = StorageStatus::LOADING;
                changed = true;
            } else if (on && e.td.status == StorageStatus::LOADING) {
                // another restoring server closed the table already (the last one to finish opens it). Its notice to
                // the other servers may still be on its way: this server sends its own before it copies anything.
                if (paused) *paused = true;
                notify = true;
            } else if (!on && e.td.status == StorageStatus::LOADING && !others_loading(e.td)) {
                e.td.status = StorageStatus::NORMAL;
                changed = true;
            }
            if (changed) {
                ++e.td.version;
                e.rt.build(e.td, node_id_);
                st = master_.set_context(ctx_key(e.sid), e.td.to_json_str());
            }
        }
        master_.release_lock(PSERVER_LOCK_NAME);
        PSB_RETURN_IF_ERROR(st);
        if (changed || notify) broadcast_ctx_update(e);   // waits for the peers' answers: they hold the status when it returns
        if (changed) {
            if (paused) *paused = on;
            PSB_LOG(INFO) << "storage " << e.sid << ": writes " << (on ? "paused for the restore" : "resumed");
        }
        return Status::Ok();
    }

    Status find_dead_node_and_replace(std::vector<int32_t>* mine) {
        std::map<int32_t, std::string> live;
        PSB_RETURN_IF_ERROR(master_.get_nodes(PSERVER_S2S_RPC_NAME, &live));
        std::set<int> live_ids;
        for (auto& kv : live) live_ids.insert(kv.first);
        std::vector<std::string> keys;
        PSB_RETURN_IF_ERROR(master_.list_contexts(&keys));
        for (auto& k : keys) {
            if (k.compare(0, 8, "storage/") != 0) continue;
            const int32_t sid = std::stoi(k.substr(8));
            std::string json;
            if (!master_.get_context(k, &json).ok()) continue;
            TableDescriptor td;
            if (!td.from_json_str(json)) continue;
            td.update_node_status(live_ids);
            int replaced = -1;
            if (!td.try_to_replace_one_dead_node(node_id_, &replaced)) continue;
            replaced_node_[sid] = replaced;
            PSB_LOG(INFO) << "storage " << sid << ": node " << node_id_ << " takes the place of dead node " << replaced;
            PSB_RETURN_IF_ERROR(master_.set_context(k, td.to_json_str()));
            std::shared_ptr<TableEntry> e;
            PSB_RETURN_IF_ERROR(ctx_.set_table_descriptor(sid, td.to_json_str(), node_id_, &e));
            mine->push_back(sid);
        }
        return Status::Ok();
    }

    // Pull every local shard from one live replica in resumable batches over s2s.
    Status restore_storage_coordinated(TableEntry& e) {
        std::map<int32_t, std::string> nodes;
        PSB_RETURN_IF_ERROR(peers(PSERVER_S2S_RPC_NAME, &nodes));
        // one live replica per shard, chosen up front: without one for every shard nothing is fetched at all
        // (CoordinatedRestoreProgress: queue of local shards, `no_replica` abort flag)
        std::vector<std::pair<int32_t, int>> plan;
        for (int32_t shard : e.rt.local_shards()) {
            std::set<int> exclude{node_id_};
            int replica = -1;
            {
                std::shared_lock<std::shared_mutex> g(e.mu);
                replica = e.rt.pick_one_replica(shard, &exclude);
            }
            if (replica < 0 || !nodes.count(replica)) return Status::NoReplica("restore: no live replica of shard " + std::to_string(shard));
            plan.push_back({shard, replica});
        }
        // the shards are fetched by restore_thread_num workers (CoordinatedRestoreController spawns thread_num workers)
        std::atomic<size_t> next{0};
        std::atomic<bool> failed{false};
        std::mutex first_mu;
        Status first;
        auto worker = [&] {
            RpcClient rpc;  // a connection of its own: the batches of different shards travel side by side
            for (;;) {
                const size_t i = next++;
                if (i >= plan.size() || failed.load()) return;
                Status st = restore_one_shard(e, plan[i].first, plan[i].second, nodes[plan[i].second], rpc);
                if (!st.ok()) {
                    failed = true;
                    std::lock_guard<std::mutex> g(first_mu);
                    if (first.ok()) first = st;
                }
            }
        };
        const int nthreads = (int)std::min<size_t>(std::max(1, cfg_.restore_thread_num), plan.size());
        std::vector<std::thread> pool;
        for (int t = 1; t < nthreads; ++t) pool.emplace_back(worker);
        worker();
        for (auto& t : pool) t.join();
        return first;
    }
    // One shard from one replica in resumable batches (CoordinatedRestoreWorker: loop RestoreBatch(iterator_id,
    // offset, batch_size) over s2s until finished).
    Status restore_one_shard(TableEntry& e, int32_t shard, int replica, const std::string& address, RpcClient& rpc) {
        int32_t iterator_id = -1;
        uint64_t offset = 0;
        for (;;) {
            PSMessage m;
            m.meta.sid = e.sid;
            m.meta.req_type = RequestType::OP_COORDINATED_RESTORE_ITERATE;
            m.ar << iterator_id << offset << (uint64_t)cfg_.restore_batch_size << shard;
            Bytes b;
            PSB_RETURN_IF_ERROR(rpc.call(address, m.seal(), cfg_.s2s_timeout_ms, &b));
            PSMessage r = PSMessage::open(std::move(b));
            Status st;
            r.ar >> st;
            PSB_RETURN_IF_ERROR(st);
            int32_t sid = 0, sh = 0, fin = 0, stride = 0;
            uint64_t num = 0;
            r.ar >> sid >> sh >> fin >> iterator_id >> offset >> num >> stride;
            if (stride < 0 || num > (1ull << 40) || !r.ar.can_hold((int64_t)num, 8 + (size_t)stride * 4))
                return Status::Error("restore: malformed batch from node " + std::to_string(replica));
            std::vector<int64_t> keys(num);
            std::vector<float> rows((size_t)num * stride);
            r.ar.read_raw(keys.data(), num * 8);
            r.ar.read_raw(rows.data(), rows.size() * 4);
            if (num) PSB_RETURN_IF_ERROR(e.storage->set_rows(keys.data(), rows.data(), num, false));
            if (fin) break;
        }
        return Status::Ok();
    }

    // Persistent image of one table on this host: <dir>/node_<id>/storage_<sid>.img = "PSBIMG1\0", version_uuid,
    // stride, then {key, row} records. The role of the reference's persistent-memory pool per storage, which a
    // restarted server opens locally when its version_uuid matches and otherwise discards in favour of a remote
    // restore (pico-ps/storage/DCPmemory.h:493-507, pico-ps/service/Service.cpp:275-294).
    static std::string image_path(const std::string& dir, int node, int32_t sid) {
        return dir + "/node_" + std::to_string(node) + "/storage_" + std::to_string(sid) + ".img";
    }
    static std::vector<std::string> list_dir(const std::string& dir) {
        std::vector<std::string> out;
        if (DIR* d = ::opendir(dir.c_str())) {
            while (dirent* ent = ::readdir(d)) {
                const std::string name = ent->d_name;
                if (name != "." && name != "..") out.push_back(name);
            }
            ::closedir(d);
        }
        return out;
    }
    // version_uuid recorded in an image file ("" when the file is not an image)
    static std::string image_uuid(const std::string& path) {
        std::ifstream f(path, std::ios::binary);
        char magic[8];
        uint64_t ulen = 0;
        f.read(magic, 8);
        f.read((char*)&ulen, 8);
        if (!f || std::memcmp(magic, "PSBIMG1", 8) != 0 || ulen > 4096) return "";
        std::string uuid(ulen, '\0');
        f.read(&uuid[0], (std::streamsize)ulen);
        return f ? uuid : "";
    }
    Status restore_storage_from_local_image(TableEntry& e) {
        if (cfg_.local_image_dir.empty()) return Status::Error("no local image directory");
        auto it = replaced_node_.find(e.sid);
        if (it == replaced_node_.end()) return Status::Error("no replaced node recorded");
        const std::string path = image_path(cfg_.local_image_dir, it->second, e.sid);
        std::ifstream f(path, std::ios::binary);
        if (!f) return Status::Error("no image " + path);
        char magic[8];
        uint64_t ulen = 0, n = 0;
        uint32_t stride = 0;
        f.read(magic, 8);
        f.read((char*)&ulen, 8);
        if (!f || std::memcmp(magic, "PSBIMG1", 8) != 0 || ulen > 4096) return Status::Error(path + ": not a table image");
        std::string uuid(ulen, '\0');
        f.read(&uuid[0], (std::streamsize)ulen);
        f.read((char*)&stride, 4);
        f.read((char*)&n, 8);
        if (!f) return Status::Error(path + ": truncated image");
        if (uuid != e.td.version_uuid) return Status::InvalidID(path + ": version_uuid differs, restore remotely");
        if (stride != e.storage->stride()) return Status::Error(path + ": record width differs from the table");
        const size_t block = 4096;
        std::vector<int64_t> keys;
        std::vector<float> rows;
        for (uint64_t done = 0; done < n;) {
            const size_t m = (size_t)std::min<uint64_t>(block, n - done);
            keys.resize(m);
            rows.resize(m * stride);
            for (size_t i = 0; i < m; ++i) {
                f.read((char*)&keys[i], 8);
                f.read((char*)(rows.data() + i * stride), (std::streamsize)stride * 4);
            }
            if (!f) return Status::Error(path + ": truncated image");
            PSB_RETURN_IF_ERROR(e.storage->set_rows(keys.data(), rows.data(), m, false));  // rows of shards that moved away are skipped
            done += m;
        }
        return Status::Ok();
    }

    // Fallback: the dump at table_uri, keeping local keys only.
    Status restore_storage_from_fs(TableEntry& e) {
        if (e.td.table_uri.empty()) return Status::Error("restore: no replica and no table_uri");
        std::string dir, format;
        DumpArgs::split_uri(e.td.table_uri, &dir, &format);
        Json cfg = Json::object();
        for (auto& kv : e.td.handlers)
            if (kv.second.op_name == "DumpOperator" || kv.second.op_name == "LoadOperator") Json::parse(kv.second.config_str, &cfg);
        LoadOperator op(cfg);
        uint64_t n = 0;
        for (auto& f : list_model_files(dir)) PSB_RETURN_IF_ERROR(op.restore_file(e, f, format, &n));
        return Status::Ok();
    }

    ServerConfig cfg_;
    MasterClient master_;   // request / response traffic with the master
    MasterClient session_;  // holds the registrations: its connection is this node's liveness
    int32_t node_id_ = -1;
    Context ctx_;
    std::unique_ptr<RpcServer> c2s_, s2s_;
    RpcClient s2s_client_;
    std::atomic<bool> declared_dead_{false}, leaving_{false};
    std::thread reporter_, keeper_;
    std::mutex keeper_mu_;
    std::condition_variable keeper_cv_;
    std::mutex report_mu_;
    std::condition_variable report_cv_;
    std::string last_report_;
    std::map<int32_t, std::string> restore_source_;
    std::map<int32_t, int> replaced_node_;  // storage id -> the dead node this server took over
    std::atomic<bool> stopped_{false}, exited_{false};
    std::mutex stop_mu_, exit_mu_, listener_mu_;
    std::shared_ptr<SyncListener> sync_listener_;
    std::thread exit_thread_;
    std::mutex metric_mu_;
    std::map<std::string, uint64_t> metrics_;
    std::map<std::pair<std::string, int32_t>, Series> series_;
};

}  // namespace psb
