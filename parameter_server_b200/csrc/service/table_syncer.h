// TableSyncer: the sync thread of a parameter server. Tables whose push operator lists follower tables
// (`"sync_table": [{"model_name", "table_name", "op_key"}, ...]` in the operator config) have the rows that pushes
// change shipped to those followers in the background: a trainer cluster keeps predictor tables fresh without the
// training job doing anything.
//
// Parity: Server::set_sync_env / add_sync_table / notify_sync_table / del_sync_table / push_sync_tables
// (pico-ps/service/Service.cpp:1467-1540): the server holds a client of the cluster where the followers live, a push
// or store notes the storage id and wakes the thread, the thread collects the increment of every noted table and
// runs SyncHandler::sync_pred against every follower (found through the model registry on the followers' master:
// model -> table -> storage id, operator key -> handler id). A deleted table is dropped from the thread's books
// after one last round. Rows are recorded as dirty marks in the table itself, so a round that fails keeps its marks
// and the next notification (or the next retry) ships them again.
#pragma once
#include <condition_variable>
#include <set>
#include <thread>

#include "../handler/handlers.h"
#include "../model/model.h"

namespace psb {

class TableSyncer {
public:
    struct Stats {
        uint64_t rounds = 0, rows = 0, errors = 0;
        std::string last_error;
    };

    // `server`: the server whose tables are followed. `follower_master`: master of the cluster that holds the
    // follower tables (the server's own master when both live in one cluster).
    TableSyncer(Server* server, const std::string& follower_master, int max_attempts = 5, double backoff_scale = 1.0)
        : server_(server), client_(follower_master), max_attempts_(max_attempts), backoff_scale_(backoff_scale) {
        thread_ = std::thread([this] { loop(); });
        server_->set_sync_listener([this](int32_t sid, bool deleted) { note(sid, deleted); });
    }
    ~TableSyncer() { stop(); }
    TableSyncer(const TableSyncer&) = delete;
    TableSyncer& operator=(const TableSyncer&) = delete;

    void stop() {
        {
            std::lock_guard<std::mutex> g(mu_);
            if (exit_) return;
            exit_ = true;
        }
        server_->set_sync_listener(nullptr);
        cv_.notify_all();
        if (thread_.joinable()) thread_.join();
    }
    Stats stats() {
        std::lock_guard<std::mutex> g(mu_);
        return stats_;
    }
    // Blocks until nothing is noted and no round is running (tests, orderly shutdown). False on timeout.
    bool wait_idle(int timeout_ms) {
        std::unique_lock<std::mutex> g(mu_);
        return idle_cv_.wait_for(g, std::chrono::milliseconds(timeout_ms), [this] { return noted_.empty() && !busy_; });
    }

private:
    struct Follower {
        SparseTablePushOperator::SyncTarget target;
        std::unique_ptr<SyncHandler> handler;
    };

    void note(int32_t sid, bool deleted) {
        {
            std::lock_guard<std::mutex> g(mu_);
            noted_.insert(sid);
            if (deleted) deleted_.insert(sid);
        }
        cv_.notify_one();
    }

    // model -> table -> (storage id, handler id of the operator keyed `op_key`) on the followers' cluster
    Status resolve(const SparseTablePushOperator::SyncTarget& t, std::unique_ptr<SyncHandler>* out) {
        ModelObject model;
        PSB_RETURN_IF_ERROR(get_model(client_.master(), t.model_name, &model));
        const TableObject* table = model.find_table(t.table_name);
        if (!table) return Status::InvalidID("sync: model " + t.model_name + " has no table " + t.table_name);
        const OperatorObject* op = table->find_op(t.op_key);
        if (!op || op->handler_id < 0) return Status::InvalidID("sync: table " + t.table_name + " has no operator " + t.op_key);
        PSB_RETURN_IF_ERROR(client_.initialize_storage(table->storage_id));
        out->reset(new SyncHandler(&client_, table->storage_id, op->handler_id));
        return Status::Ok();
    }

    Status sync_one(int32_t sid, uint64_t* rows) {
        auto& followers = followers_[sid];
        if (followers.empty())
            for (auto& t : server_->sync_targets(sid)) followers.push_back(Follower{t, nullptr});
        Status first;
        // The increment is collected once per follower, and the marks go only with the pass for the last follower, and
        // only if every follower before it got the rows: a follower that is down keeps the marks in place, so the
        // others receive those rows again next round (overwrites of equal rows) and the one that was down misses
        // nothing. One follower is the common case.
        for (size_t i = 0; i < followers.size(); ++i) {
            auto& f = followers[i];
            if (!f.handler) {
                Status st = resolve(f.target, &f.handler);
                if (!st.ok()) {
                    if (first.ok()) first = st;
                    continue;
                }
            }
            uint64_t n = 0;
            const bool last = i + 1 == followers.size() && first.ok();
            Status st = last ? f.handler->sync_pred(*server_, sid, &n, max_attempts_, backoff_scale_)
                             : f.handler->sync_pred_keep_marks(*server_, sid, &n, max_attempts_, backoff_scale_);
            *rows += n;
            if (!st.ok()) {
                if (st.is(StatusCode::INVALID_ID)) f.handler.reset();   // the follower was re-created: resolve it again
                if (first.ok()) first = st;
            }
        }
        return first;
    }

    void loop() {
        for (;;) {
            std::set<int32_t> todo, gone;
            {
                std::unique_lock<std::mutex> g(mu_);
                busy_ = false;
                idle_cv_.notify_all();
                cv_.wait(g, [this] { return !noted_.empty() || exit_; });
                if (exit_ && noted_.empty()) return;
                todo.swap(noted_);
                gone = deleted_;
                busy_ = true;
            }
            for (int32_t sid : todo) {
                uint64_t rows = 0;
                Status st = gone.count(sid) ? Status::Ok() : sync_one(sid, &rows);
                std::lock_guard<std::mutex> g(mu_);
                ++stats_.rounds;
                stats_.rows += rows;
                if (!st.ok()) {
                    ++stats_.errors;
                    stats_.last_error = st.to_string();
                    PSB_LOG(WARNING) << "sync of storage " << sid << " failed, the marks stay for the next round: " << stats_.last_error;
                }
                if (gone.count(sid)) {
                    followers_.erase(sid);
                    deleted_.erase(sid);
                }
            }
            std::lock_guard<std::mutex> g(mu_);
            if (exit_) {
                busy_ = false;
                idle_cv_.notify_all();
                return;
            }
        }
    }

    Server* server_;
    Client client_;
    int max_attempts_;
    double backoff_scale_;
    std::mutex mu_;
    std::condition_variable cv_, idle_cv_;
    std::set<int32_t> noted_, deleted_;
    std::map<int32_t, std::vector<Follower>> followers_;   // touched by the sync thread only
    Stats stats_;
    bool exit_ = false, busy_ = false;
    std::thread thread_;
};

}  // namespace psb
