// Handlers: the client-side façade of each operator, with the automatic retry policy.
//
// Parity: pico-ps/handler/Handler.{h,cpp} (wait() = wait_no_release + retry loop: Timeout / NoReplica
// -> dead-node detection then retry (NoReplica only once); ServerTooNewCtx -> refresh the context then
// retry; OutOfMemory -> wait for a context change then retry; anything else goes to the caller;
// remaining-time bookkeeping), PullHandler / PushHandler / ForEachHandler / EraseIfHandler /
// DumpHandler / LoadHandler / UpdateContextHandler / SyncHandler / UDFHandler of pico-ps/handler/*.
// UpdateContextHandler and SyncHandler never auto-retry (pico-ps/handler/UpdateContextHandler.cpp:
// 275-277, pico-ps/handler/SyncHandler.h:32-34). Counters mirror ps_wait_request_count /
// ps_pull_send_request_count (pico-ps/handler/Handler.cpp:14-18, pico-ps/handler/PullHandler.cpp:11-15).
#pragma once
#include <atomic>
#include <chrono>
#include <functional>
#include <thread>

#include "../common/thread_sync.h"
#include "../service/client.h"

namespace psb {

struct HandlerMetrics {
    std::atomic<uint64_t> requests{0}, retries{0}, errors{0};
    std::atomic<uint64_t> wait_us{0};
    // pulls only: requests built (dedup, partition, serialisation) and the time that took - the send side of a pull,
    // ps_pull_send_request_count / ps_pull_send_duration_ms of the reference (pico-ps/handler/PullHandler.cpp:11-15)
    std::atomic<uint64_t> sends{0}, send_us{0};
};

// Every request carries the context version it was BUILT under (read under the same lock as the placement it was
// routed by). The client's copy can move on between building and sending when another thread refreshes it; a
// request stamped with the newer version but routed by the older placement would pass the server's version gate
// and reach a node that no longer holds the shard.
// The two smallest int64 values are the "empty" and "erased" markers of every key map in this build (the client's
// dedup map, the host table, the GPU index): a request that carries one is refused where it enters.
inline Status check_request_keys(const int64_t* keys, size_t n) {
    for (size_t i = 0; i < n; ++i)
        if (keys[i] <= kHostEmptyKey + 1)
            return Status::InvalidConfig("key " + std::to_string(keys[i]) + " is reserved (INT64_MIN and INT64_MIN + 1 cannot be stored)");
    return Status::Ok();
}

class Handler {
public:
    Handler(Client* client, int32_t sid, int32_t hid) : client_(client), sid_(sid), hid_(hid) {}
    virtual ~Handler() = default;
    int32_t storage_id() const { return sid_; }
    int32_t handler_id() const { return hid_; }
    HandlerMetrics& metrics() { return metrics_; }

protected:
    std::shared_ptr<TableEntry> entry() { return client_->context().get(sid_); }

    template <class OP>
    Status op(std::shared_ptr<OP>* out) {
        auto e = entry();
        if (!e) return Status::InvalidID("storage " + std::to_string(sid_) + " is not initialised on this client");
        std::shared_lock<std::shared_mutex> g(e->mu);
        auto it = e->ops.find(hid_);
        if (it == e->ops.end()) return Status::InvalidID("handler " + std::to_string(hid_) + " is not registered");
        *out = std::dynamic_pointer_cast<OP>(it->second);
        if (!*out) return Status::InvalidID("handler " + std::to_string(hid_) + " has another operator type");
        return Status::Ok();
    }

    // Runs `attempt` (which builds the requests against the CURRENT context and waits for them) under
    // the retry policy. `timeout_ms` < 0 means no limit.
    Status with_retry(const std::function<Status(int remaining_ms)>& attempt, int timeout_ms, bool auto_retry = true) {
        auto t0 = std::chrono::steady_clock::now();
        auto remaining = [&]() -> int {
            if (timeout_ms < 0) return -1;
            long el = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
            return (int)std::max<long>(0, timeout_ms - el);
        };
        bool no_replica_retried = false;
        Status st;
        for (int round = 0;; ++round) {
            ++metrics_.requests;
            st = attempt(remaining());
            if (st.ok() || !auto_retry) break;
            const int left = remaining();
            if (timeout_ms >= 0 && left == 0) break;
            if (st.is(StatusCode::TIMEOUT) || st.is(StatusCode::NO_REPLICA)) {
                if (st.is(StatusCode::NO_REPLICA)) {
                    if (no_replica_retried) break;
                    no_replica_retried = true;
                }
                Status h = client_->handle_timeout(sid_);
                if (!h.ok()) break;
            } else if (st.is(StatusCode::SERVER_TOO_NEW_CTX) || st.is(StatusCode::SERVER_TOO_NEW_CTX_U)) {
                if (!client_->handle_server_too_new_ctx(sid_).ok()) break;
            } else if (st.is(StatusCode::OUT_OF_MEMORY)) {
                if (!client_->handle_out_of_memory(sid_, left).ok()) break;
            } else if (st.is(StatusCode::SERVER_TOO_OLD_CTX) || st.is(StatusCode::SERVER_TOO_OLD_CTX_U)) {
                // The server has not seen a context that this client already uses (the publisher updates its own
                // copy a moment before the master's). The server refreshes from the master on every such
                // request, so a short pause and a retry are enough.
                std::this_thread::sleep_for(std::chrono::milliseconds(20));
            } else {
                break;
            }
            ++metrics_.retries;
            if (round > 64) break;
        }
        if (!st.ok()) ++metrics_.errors;
        metrics_.wait_us += (uint64_t)std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now() - t0).count();
        return st;
    }

    Client* client_;
    int32_t sid_, hid_;
    HandlerMetrics metrics_;
};

// ---------------------------------------------------------------------------------------------------
// Request-merge group of pull handlers that live on different threads of one client
// (PullRequestDataGroup of pico-ps/handler/PullHandler.h:22-29): small requests of two threads travel as
// one message per node.
struct PullGroup {
    ThreadReduce reduce;
    ThreadBcast bcast;
    PullRequestData data[kThreadGroupSize];
    Status status[kThreadGroupSize];
    std::atomic<int> next_tid{0};
    std::atomic<uint64_t> merged_sends{0}, merged_requests{0};
};

class PullHandler : public Handler {
public:
    using Handler::Handler;
    static constexpr size_t kMergeBelowBytesPerNode = 128 << 10;  // pico-ps/handler/PullHandler.cpp:121-126

    // Join a merge group (at most 32 handlers, one per thread). Returns the slot, or -1 when it is full.
    int join_group(std::shared_ptr<PullGroup> g) {
        int t = g->next_tid.fetch_add(1);
        if (t >= kThreadGroupSize) return -1;
        group_ = std::move(g);
        tid_ = t;
        return t;
    }
    PullGroup* group() const { return group_.get(); }

    // out: n * dim floats, one row per key position.
    Status pull(const int64_t* keys, size_t n, float* out, int timeout_ms = -1, bool auto_retry = true) {
        PSB_RETURN_IF_ERROR(check_request_keys(keys, n));
        std::shared_ptr<SparseTablePullOperator> p;
        PSB_RETURN_IF_ERROR(op(&p));
        if (group_) return with_retry([&](int left) { return merged_attempt(*p, keys, n, out, left); }, timeout_ms, auto_retry);
        return with_retry([&](int left) -> Status {
            auto e = entry();
            PullRequestData data;
            NodeRequests reqs;
            int32_t built_under = -1;
            const auto b0 = std::chrono::steady_clock::now();
            {
                std::shared_lock<std::shared_mutex> g(e->mu);
                built_under = e->td.version;
                p->generate_request_data(*e, keys, n, &data);
                PSB_RETURN_IF_ERROR(p->generate_requests(*e, data, &reqs));
            }
            ++metrics_.sends;
            metrics_.send_us += (uint64_t)std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now() - b0).count();
            std::vector<NodeResponse> rs;
            PSB_RETURN_IF_ERROR(client_->send_and_wait(sid_, hid_, RequestType::OP_PULL, reqs.body, left, &rs, built_under));
            for (auto& r : rs) PSB_RETURN_IF_ERROR(p->apply_response(*e, &data, r.body));
            p->fill_pull_items(*e, data, out);
            return Status::Ok();
        }, timeout_ms, auto_retry);
    }
    // Dense pull: tensor `id` of `numel` floats, reassembled from its slices. A DenseTablePullOperator decides the cut
    // and the reassembly; a plain sparse pull operator gets the default (consecutive slices).
    Status pull_dense(int64_t id, size_t numel, float* out, int timeout_ms = -1) {
        auto e = entry();
        if (!e) return Status::InvalidID("storage is not initialised on this client");
        const uint32_t slice = storage_op_of(*e)->dim();
        PSB_RETURN_IF_ERROR(dense_check_id(id, numel, slice));
        std::shared_ptr<SparseTablePullOperator> p;
        PSB_RETURN_IF_ERROR(op(&p));
        const auto* dp = dynamic_cast<const DenseTablePullOperator*>(p.get());
        std::vector<DenseSlice> slices;
        if (dp) dp->partition(id, numel, slice, &slices);
        else dense_default_partition(id, numel, slice, &slices);
        std::vector<int64_t> keys(slices.size());
        for (size_t j = 0; j < slices.size(); ++j) keys[j] = slices[j].key;
        std::vector<float> tmp(keys.size() * slice);
        PSB_RETURN_IF_ERROR(pull(keys.data(), keys.size(), tmp.data(), timeout_ms));
        for (size_t j = 0; j < slices.size(); ++j) {
            if (slices[j].offset + slices[j].len > numel || slices[j].len > slice) return Status::Error("dense pull: the partitioner left the value");
            if (dp) dp->merge(slices[j], tmp.data() + j * slice, out);
            else std::copy_n(tmp.data() + j * slice, slices[j].len, out + slices[j].offset);
        }
        return Status::Ok();
    }
    uint32_t dim() {
        auto e = entry();
        return e ? storage_op_of(*e)->dim() : 0;
    }

private:
    // One attempt inside a merge group. Nothing between add() and reduce() can fail, so a thread that
    // announced itself always reaches reduce() and nobody waits for it in vain.
    Status merged_attempt(SparseTablePullOperator& p, const int64_t* keys, size_t n, float* out, int left) {
        PullGroup& g = *group_;
        auto e = entry();
        g.reduce.add(tid_);
        PullRequestData& mine = g.data[tid_];
        size_t nodes = 1;
        {
            std::shared_lock<std::shared_mutex> lk(e->mu);
            p.generate_request_data(*e, keys, n, &mine);
            nodes = std::max<size_t>(1, e->rt.nodes().size());
        }
        const int sync_num = (size_t)mine.n_uniq * 8 / nodes < kMergeBelowBytesPerNode ? 2 : 1;
        const uint32_t tids = g.reduce.reduce(tid_, sync_num);
        Status st;
        if (tids == 0) {
            g.bcast.wait(tid_);  // the owner of the merged request fills our rows and status
            st = g.status[tid_];
        } else {
            std::vector<PullRequestData*> all;
            for (int t = 0; t < kThreadGroupSize; ++t)
                if ((tids >> t) & 1u) all.push_back(&g.data[t]);
            // one message carries at most max_request_merge_num requests; what was claimed beyond that goes out in
            // further messages of the same size
            const size_t cap = (size_t)p.max_request_merge_num();
            for (size_t lo = 0; lo < all.size() && st.ok(); lo += cap) {
                std::vector<PullRequestData*> ds(all.begin() + lo, all.begin() + std::min(all.size(), lo + cap));
                st = [&]() -> Status {
                    NodeRequests reqs;
                    int32_t built_under = -1;
                    {
                        std::shared_lock<std::shared_mutex> lk(e->mu);
                        built_under = e->td.version;
                        PSB_RETURN_IF_ERROR(p.generate_merged_requests(*e, ds, &reqs));
                    }
                    std::vector<NodeResponse> rs;
                    PSB_RETURN_IF_ERROR(client_->send_and_wait(sid_, hid_, RequestType::OP_PULL, reqs.body, left, &rs, built_under));
                    for (auto& r : rs) PSB_RETURN_IF_ERROR(p.apply_merged_response(*e, ds, r.body));
                    return Status::Ok();
                }();
                ++g.merged_sends;
                g.merged_requests += ds.size();
            }
            for (int t = 0; t < kThreadGroupSize; ++t)
                if ((tids >> t) & 1u) g.status[t] = st;
            g.bcast.notify(tids, tid_);
        }
        if (st.ok()) p.fill_pull_items(*e, mine, out);
        return st;
    }

    std::shared_ptr<PullGroup> group_;
    int tid_ = -1;
};

// Request-merge group of push handlers on different threads of one client (PushRequestDataGroup of
// pico-ps/handler/PushHandler.h:20-27).
struct PushGroup {
    ThreadReduce reduce;
    ThreadBcast bcast;
    PushRequestData data[kThreadGroupSize];
    RequestType type[kThreadGroupSize];  // async or sync push, per slot
    PushAckState* ack[kThreadGroupSize] = {};  // progress of each member's push across its retries
    Status status[kThreadGroupSize];
    std::atomic<int> next_tid{0};
    std::atomic<uint64_t> merged_sends{0}, merged_requests{0};
};

class PushHandler : public Handler {
public:
    using Handler::Handler;
    // Join a merge group (at most 32 handlers, one per thread). Returns the slot, or -1 when it is full.
    int join_group(std::shared_ptr<PushGroup> g) {
        int t = g->next_tid.fetch_add(1);
        if (t >= kThreadGroupSize) return -1;
        group_ = std::move(g);
        tid_ = t;
        return t;
    }
    uint32_t dim() {
        auto e = entry();
        return e ? storage_op_of(*e)->dim() : 0;
    }
    Status async_push(const int64_t* keys, const float* grads, size_t n, int timeout_ms = -1) {
        return push(keys, grads, n, RequestType::OP_PUSH_ASYNC, timeout_ms);
    }
    Status sync_push(const int64_t* keys, const float* grads, size_t n, int timeout_ms = -1) {
        return push(keys, grads, n, RequestType::OP_PUSH_SYNC, timeout_ms);
    }
    // Fold everything sync_push buffered; one request per (node, shard) as in the reference.
    Status store(int timeout_ms = -1) {
        return with_retry([&](int left) -> Status {
            auto e = entry();
            std::map<int, Archive> bodies;
            int32_t built_under = -1;
            {
                std::shared_lock<std::shared_mutex> g(e->mu);
                built_under = e->td.version;
                for (auto& kv : e->rt.nodes()) bodies[kv.first] << (int32_t)(kv.second.empty() ? -1 : kv.second.front());
            }
            return client_->send_and_wait(sid_, hid_, RequestType::OP_STORE, bodies, left, nullptr, built_under);
        }, timeout_ms);
    }
    Status push_dense(int64_t id, const float* grad, size_t numel, bool sync, int timeout_ms = -1) {
        auto e = entry();
        if (!e) return Status::InvalidID("storage is not initialised on this client");
        const uint32_t slice = storage_op_of(*e)->dim();
        PSB_RETURN_IF_ERROR(dense_check_id(id, numel, slice));
        std::shared_ptr<SparseTablePushOperator> p;
        PSB_RETURN_IF_ERROR(op(&p));
        const auto* dp = dynamic_cast<const DenseTablePushOperator*>(p.get());
        std::vector<DenseSlice> slices;
        if (dp) dp->partition(id, numel, slice, &slices);
        else dense_default_partition(id, numel, slice, &slices);
        std::vector<int64_t> keys(slices.size());
        std::vector<float> tmp(slices.size() * slice, 0.f);
        for (size_t j = 0; j < slices.size(); ++j) {
            if (slices[j].offset + slices[j].len > numel || slices[j].len > slice) return Status::Error("dense push: the partitioner left the value");
            keys[j] = slices[j].key;
            if (dp) dp->extract(slices[j], grad, tmp.data() + j * slice);
            else std::copy_n(grad + slices[j].offset, slices[j].len, tmp.data() + j * slice);
        }
        return push(keys.data(), tmp.data(), keys.size(), sync ? RequestType::OP_PUSH_SYNC : RequestType::OP_PUSH_ASYNC, timeout_ms);
    }

private:
    Status push(const int64_t* keys, const float* grads, size_t n, RequestType type, int timeout_ms) {
        PSB_RETURN_IF_ERROR(check_request_keys(keys, n));
        std::shared_ptr<SparseTablePushOperator> p;
        PSB_RETURN_IF_ERROR(op(&p));
        PushAckState ack;  // lives for this call: what the retries need not send again
        if (group_) return with_retry([&](int left) { return merged_attempt(*p, keys, grads, n, type, left, &ack); }, timeout_ms);
        return with_retry([&](int left) -> Status {
            auto e = entry();
            PushRequestData data;
            NodeRequests reqs;
            int32_t built_under = -1;
            {
                std::shared_lock<std::shared_mutex> g(e->mu);
                built_under = e->td.version;
                p->generate_request_data(*e, keys, grads, n, &data);  // regenerated against the fresh context on retry
                if (ack.G != data.global_shard_num) ack.reset(data.global_shard_num);  // other shard count: start over
                PSB_RETURN_IF_ERROR(p->generate_requests(*e, data, &reqs, &ack));
            }
            if (reqs.body.empty()) return Status::Ok();  // everything was applied by earlier attempts
            std::vector<NodeResponse> rs;
            Status st = client_->send_and_wait(sid_, hid_, type, reqs.body, left, &rs, built_under);
            for (auto& r : rs)
                for (int32_t sh : reqs.shards[r.node]) ack.record(sh, r.node, r.status.ok());
            return st;
        }, timeout_ms);
    }

    // One attempt inside a merge group; requests of different kinds (async / sync) are not merged: a thread
    // that finds another kind among the claimed slots sends one message per kind.
    Status merged_attempt(SparseTablePushOperator& p, const int64_t* keys, const float* grads, size_t n, RequestType type,
                          int left, PushAckState* ack) {
        PushGroup& g = *group_;
        auto e = entry();
        g.reduce.add(tid_);
        PushRequestData& mine = g.data[tid_];
        size_t nodes = 1, bytes = 0;
        {
            std::shared_lock<std::shared_mutex> lk(e->mu);
            p.generate_request_data(*e, keys, grads, n, &mine);
            nodes = std::max<size_t>(1, e->rt.nodes().size());
        }
        for (auto& kv : mine.shard_keys) bytes += kv.second.size() * 8 + mine.shard_grads[kv.first].size() * 4;
        g.type[tid_] = type;
        if (ack->G != mine.global_shard_num) ack->reset(mine.global_shard_num);
        g.ack[tid_] = ack;
        const int sync_num = bytes / nodes < PullHandler::kMergeBelowBytesPerNode ? 2 : 1;
        const uint32_t tids = g.reduce.reduce(tid_, sync_num);
        if (tids == 0) {
            g.bcast.wait(tid_);
            return g.status[tid_];
        }
        for (RequestType kind : {RequestType::OP_PUSH_ASYNC, RequestType::OP_PUSH_SYNC}) {
            std::vector<PushRequestData*> ds;
            std::vector<PushAckState*> acks;
            uint32_t members = 0;
            for (int t = 0; t < kThreadGroupSize; ++t)
                if (((tids >> t) & 1u) && g.type[t] == kind) {
                    ds.push_back(&g.data[t]);
                    acks.push_back(g.ack[t]);
                    members |= 1u << t;
                }
            if (ds.empty()) continue;
            const std::vector<PushRequestData*> all_ds = ds;
            const std::vector<PushAckState*> all_acks = acks;
            const size_t cap = (size_t)p.max_request_merge_num();
            Status st;
            for (size_t lo = 0; lo < all_ds.size(); lo += cap) {
            const size_t hi = std::min(all_ds.size(), lo + cap);
            ds.assign(all_ds.begin() + lo, all_ds.begin() + hi);
            acks.assign(all_acks.begin() + lo, all_acks.begin() + hi);
            Status part = [&]() -> Status {
                NodeRequests reqs;
                std::vector<std::vector<std::pair<int, int32_t>>> sent;
                int32_t built_under = -1;
                {
                    std::shared_lock<std::shared_mutex> lk(e->mu);
                    built_under = e->td.version;
                    PSB_RETURN_IF_ERROR(p.generate_merged_requests(*e, ds, acks, &reqs, &sent));
                }
                if (reqs.body.empty()) return Status::Ok();
                std::vector<NodeResponse> rs;
                Status sst = client_->send_and_wait(sid_, hid_, kind, reqs.body, left, &rs, built_under);
                std::map<int, bool> node_ok;
                for (auto& r : rs) node_ok[r.node] = r.status.ok();
                for (size_t i = 0; i < ds.size(); ++i)   // the members sleep until the broadcast: their state is ours to update
                    for (auto& ns : sent[i]) acks[i]->record(ns.second, ns.first, node_ok[ns.first]);
                return sst;
            }();
            ++g.merged_sends;
            g.merged_requests += ds.size();
            if (!part.ok() && st.ok()) st = part;   // every member retries; what its nodes acknowledged is not resent
            }
            for (int t = 0; t < kThreadGroupSize; ++t)
                if ((members >> t) & 1u) g.status[t] = st;
        }
        g.bcast.notify(tids, tid_);
        return g.status[tid_];
    }

    std::shared_ptr<PushGroup> group_;
    int tid_ = -1;
};

class ForEachHandler : public Handler {
public:
    using Handler::Handler;
    // One request per (node, shard); the operator's merge_result folds the answers on the client
    // (pico-ps/handler/ForEachHandler.cpp:16-46 wait_and_merge_result). *result holds the operator's bytes.
    Status for_each_raw(const std::string& carried_json, std::string* result, int timeout_ms = -1) {
        std::shared_ptr<ForEachOperatorBase> fop;
        PSB_RETURN_IF_ERROR(op(&fop));
        Json carried = Json::object();
        if (!carried_json.empty() && !Json::parse(carried_json, &carried)) return Status::InvalidConfig("carried item is not JSON");
        return with_retry([&](int left) -> Status {
            *result = fop->init_result(carried);
            auto e = entry();
            // a reading scan asks one replica of every shard; a writing scan goes to every holder, so that replicas
            // stay alike, and the answer of the first holder of a shard is the one that counts
            std::vector<std::pair<int, int32_t>> targets;
            std::map<int32_t, int> primary;
            int32_t built_under = -1;
            {
                std::shared_lock<std::shared_mutex> g(e->mu);
                built_under = e->td.version;
                for (auto& kv : e->rt.shards()) {
                    if (fop->writes()) {
                        for (int node : kv.second) {
                            targets.push_back({node, kv.first});
                            if (!primary.count(kv.first)) primary[kv.first] = node;
                        }
                        continue;
                    }
                    int node = e->rt.pick_one_replica(kv.first);
                    if (node < 0) return Status::NoReplica("for_each: no live replica of shard " + std::to_string(kv.first));
                    targets.push_back({node, kv.first});
                    primary[kv.first] = node;
                }
            }
            for (auto& t : targets) {
                std::map<int, Archive> body;
                body[t.first] << t.second << carried_json;
                std::vector<NodeResponse> rs;
                PSB_RETURN_IF_ERROR(client_->send_and_wait(sid_, hid_, RequestType::OP_FOREACH, body, left, &rs, built_under));
                std::string part;
                rs[0].body >> part;
                if (primary[t.second] == t.first) fop->merge_result(part, result);
            }
            return Status::Ok();
        }, timeout_ms);
    }
    // The built-in statistics operator, unpacked.
    Status for_each(const std::string& carried_json, ForEachResult* result, int timeout_ms = -1) {
        std::string raw;
        PSB_RETURN_IF_ERROR(for_each_raw(carried_json, &raw, timeout_ms));
        if (!ForEachResult::unpack(raw, result)) return Status::Error("for_each: the operator's result is not the built-in statistics record");
        return Status::Ok();
    }
};

class EraseIfHandler : public Handler {
public:
    using Handler::Handler;
    // Every holder of every shard applies the predicate (replicas stay identical).
    Status erase_if(const std::string& carried_json, uint64_t* erased, int timeout_ms = -1) {
        return with_retry([&](int left) -> Status {
            *erased = 0;
            auto e = entry();
            std::vector<std::pair<int, int32_t>> targets;
            std::map<int32_t, int> primary;
            int32_t built_under = -1;
            {
                std::shared_lock<std::shared_mutex> g(e->mu);
                built_under = e->td.version;
                for (auto& kv : e->rt.shards())
                    for (int node : kv.second) {
                        targets.push_back({node, kv.first});
                        if (!primary.count(kv.first)) primary[kv.first] = node;
                    }
            }
            for (auto& t : targets) {
                std::map<int, Archive> body;
                body[t.first] << t.second << carried_json;
                std::vector<NodeResponse> rs;
                PSB_RETURN_IF_ERROR(client_->send_and_wait(sid_, hid_, RequestType::OP_ERASEIF, body, left, &rs, built_under));
                uint64_t n = 0;
                rs[0].body >> n;
                if (primary[t.second] == t.first) *erased += n;
            }
            return Status::Ok();
        }, timeout_ms);
    }
};

class DumpHandler : public Handler {
public:
    using Handler::Handler;
    // One request per (node, file): shard -> file by shard_id % file_number.
    Status dump(const DumpArgs& args, uint64_t* n_records, int timeout_ms = -1) {
        std::string dir, format;
        DumpArgs::split_uri(args.uri, &dir, &format);
        *n_records = 0;
        if (dir.empty()) return Status::InvalidConfig("dump: the uri names no directory");
        if (args.file_number < 1) return Status::InvalidConfig("dump: file_number must be at least 1");
        PSB_RETURN_IF_ERROR(mkdir_p(dir));
        return with_retry([&](int left) -> Status {
            *n_records = 0;
            auto e = entry();
            std::map<int, std::map<int32_t, std::vector<int32_t>>> plan;  // node -> file -> shards
            int32_t built_under = -1;
            {
                std::shared_lock<std::shared_mutex> g(e->mu);
                built_under = e->td.version;
                // every shard is dumped once: by its first live holder
                for (auto& kv : e->rt.shards()) {
                    int node = -1;
                    for (int n : kv.second)
                        if (e->rt.is_running(n)) { node = n; break; }
                    if (node < 0) return Status::NoReplica("dump: no live replica of shard " + std::to_string(kv.first));
                    plan[node][kv.first % args.file_number].push_back(kv.first);
                }
            }
            for (auto& nk : plan)
                for (auto& fk : nk.second) {
                    std::map<int, Archive> body;
                    body[nk.first] << args.uri << args.file_number << fk.first << fk.second;
                    std::vector<NodeResponse> rs;
                    PSB_RETURN_IF_ERROR(client_->send_and_wait(sid_, hid_, RequestType::OP_DUMP, body, left, &rs, built_under));
                    uint64_t n = 0;
                    rs[0].body >> n;
                    *n_records += n;
                }
            return Status::Ok();
        }, timeout_ms);
    }
};

class LoadHandler : public Handler {
public:
    using Handler::Handler;
    // load: rehash through the push path (any old / new sharding). Files are dealt to the servers with at
    // most `server_concurrency` outstanding per server.
    Status load(const std::string& uri, uint64_t* n_records, int server_concurrency = 4, int timeout_ms = -1) {
        return run(uri, true, n_records, server_concurrency, timeout_ms);
    }
    // restore: same sharding as the dump; every server reads all files and keeps its local keys.
    Status restore(const std::string& uri, uint64_t* n_records, bool drop = false, int timeout_ms = -1) {
        Status st = run(uri, false, n_records, 1, timeout_ms);
        if (st.ok() && drop) {
            std::string dir, format;
            DumpArgs::split_uri(uri, &dir, &format);
            for (auto& f : list_model_files(dir)) fs::remove_file(f);
        }
        return st;
    }

private:
    Status run(const std::string& uri, bool rehash, uint64_t* n_records, int conc, int timeout_ms) {
        std::string dir, format;
        DumpArgs::split_uri(uri, &dir, &format);
        *n_records = 0;
        if (dir.empty()) return Status::InvalidConfig("load: the uri names no directory");
        std::vector<std::string> files = list_model_files(dir);
        if (files.empty()) return Status::Error("load: no model_* files under " + dir);
        return with_retry([&](int left) -> Status {
            *n_records = 0;
            auto e = entry();
            std::vector<int> nodes;
            int32_t built_under = -1;
            {
                std::shared_lock<std::shared_mutex> g(e->mu);
                built_under = e->td.version;
                for (auto& kv : e->rt.nodes())
                    if (e->rt.is_running(kv.first)) nodes.push_back(kv.first);
            }
            if (nodes.empty()) return Status::NoReplica("load: no live server");
            std::map<int, std::vector<std::string>> deal;
            if (rehash) {
                for (size_t i = 0; i < files.size(); ++i) deal[nodes[i % nodes.size()]].push_back(files[i]);
            } else {
                for (int n : nodes) deal[n] = files;
            }
            // waves of at most `conc` files per server
            for (size_t wave = 0;; ++wave) {
                std::map<int, Archive> bodies;
                for (auto& kv : deal) {
                    std::vector<std::string> part;
                    for (size_t i = wave * conc; i < std::min<size_t>(kv.second.size(), (wave + 1) * conc); ++i) part.push_back(kv.second[i]);
                    if (!part.empty()) bodies[kv.first] << uri << (int32_t)(rehash ? 1 : 0) << part;
                }
                if (bodies.empty()) break;
                std::vector<NodeResponse> rs;
                PSB_RETURN_IF_ERROR(client_->send_and_wait(sid_, hid_, RequestType::OP_LOAD, bodies, left, &rs, built_under));
                for (auto& r : rs) {
                    uint64_t n = 0;
                    r.body >> n;
                    *n_records += n;
                }
            }
            return Status::Ok();
        }, timeout_ms);
    }
};

// The reshard / rebalance / replica-change transaction (7 steps; reads are served throughout, writes are
// refused between step 1 and step 7).
class UpdateContextHandler : public Handler {
public:
    using Handler::Handler;
    // new_nodes_json: [{"g_rank":..,"shard_list":[..]}, ...]
    Status update_context(const std::string& new_nodes_json, int timeout_ms = 60000) {
        Json nodes_cfg;
        if (!Json::parse(new_nodes_json, &nodes_cfg)) return Status::InvalidConfig("update_context: nodes JSON does not parse");
        std::vector<NodeDescriptor> new_nodes;
        PSB_RETURN_IF_ERROR(TableDescriptor::parse_nodes(nodes_cfg, &new_nodes));
        MasterClient& m = client_->master();
        std::set<int> involved;
        int32_t ver = 0, uver = 0;
        // 1. prepare: publish the update info, status RESHARD (from now on writes get OUT_OF_MEMORY)
        PSB_RETURN_IF_ERROR(m.acquire_lock(PSERVER_LOCK_NAME));
        Status st = [&]() -> Status {
            PSB_RETURN_IF_ERROR(client_->pull_context_nolock(sid_));
            auto e = entry();
            {
                std::unique_lock<std::shared_mutex> g(e->mu);
                if (e->td.status != StorageStatus::NORMAL) return Status::Error("update_context: table is not in NORMAL state");
                e->td.create_update_info(new_nodes);
                e->update_rt.build(e->td, -1, true);
                ver = e->td.version;
                uver = e->td.update_version;
            }
            involved = Client::all_nodes(*e);
            PSB_RETURN_IF_ERROR(client_->push_context_nolock(sid_));
            return client_->require_update_ctx_nolock(sid_, involved, timeout_ms);
        }();
        m.release_lock(PSERVER_LOCK_NAME);
        PSB_RETURN_IF_ERROR(st);
        auto e = entry();
        std::set<int> new_set;
        for (auto& n : new_nodes) new_set.insert(n.node_id);
        // 2. create the shards of the new placement
        st = client_->broadcast(sid_, RequestType::NEW_CTX_CREATE_SHARD, new_set, Archive(), timeout_ms, ver, uver);
        // 3. shuffle: one request per old shard to one live replica
        if (st.ok()) {
            std::vector<std::pair<int, int32_t>> targets;
            {
                std::shared_lock<std::shared_mutex> g(e->mu);
                for (auto& kv : e->rt.shards()) {
                    int node = e->rt.pick_one_replica(kv.first);
                    if (node < 0) { st = Status::NoReplica("shuffle: no live replica of shard " + std::to_string(kv.first)); break; }
                    targets.push_back({node, kv.first});
                }
            }
            for (auto& t : targets) {
                if (!st.ok()) break;
                std::map<int, Archive> body;
                body[t.first] << t.second;
                st = client_->send_and_wait(sid_, hid_, RequestType::NEW_CTX_SHUFFLE, body, timeout_ms, nullptr, ver, uver);
            }
        }
        // 4. store
        if (st.ok()) st = client_->broadcast(sid_, RequestType::NEW_CTX_STORE, new_set, Archive(), timeout_ms, ver, uver);
        if (!st.ok()) {
            purge(timeout_ms);
            return st;
        }
        // 5. commit the new placement (readers switch)
        PSB_RETURN_IF_ERROR(m.acquire_lock(PSERVER_LOCK_NAME));
        st = [&]() -> Status {
            std::string json;
            PSB_RETURN_IF_ERROR(m.get_context(ctx_key(sid_), &json));
            TableDescriptor cur;
            cur.from_json_str(json);
            if (cur.version != ver || cur.update_version != uver) return Status::Error("update_context: context changed under the transaction");
            {
                std::unique_lock<std::shared_mutex> g(e->mu);
                e->td.apply_update();
                e->rt.build(e->td, -1);
                e->update_rt.build(e->td, -1, true);
            }
            PSB_RETURN_IF_ERROR(client_->push_context_nolock(sid_));
            return client_->require_update_ctx_nolock(sid_, involved, timeout_ms);
        }();
        m.release_lock(PSERVER_LOCK_NAME);
        if (!st.ok()) {
            purge(timeout_ms);
            return st;
        }
        // 6. purge what no longer belongs
        client_->broadcast(sid_, RequestType::NEW_CTX_PURGE, involved, Archive(), timeout_ms, -1);
        // 7. back to NORMAL (writes resume)
        PSB_RETURN_IF_ERROR(m.acquire_lock(PSERVER_LOCK_NAME));
        st = [&]() -> Status {
            {
                std::unique_lock<std::shared_mutex> g(e->mu);
                e->td.status = StorageStatus::NORMAL;
                ++e->td.version;
            }
            PSB_RETURN_IF_ERROR(client_->push_context_nolock(sid_));
            return client_->require_update_ctx_nolock(sid_, involved, timeout_ms);
        }();
        m.release_lock(PSERVER_LOCK_NAME);
        return st;
    }
    // Abort / clean-up path: drop the update info and the half-built shards.
    Status purge(int timeout_ms = 60000) {
        MasterClient& m = client_->master();
        PSB_RETURN_IF_ERROR(m.acquire_lock(PSERVER_LOCK_NAME));
        Status st = [&]() -> Status {
            PSB_RETURN_IF_ERROR(client_->pull_context_nolock(sid_));
            auto e = entry();
            std::set<int> involved = Client::all_nodes(*e);
            {
                std::unique_lock<std::shared_mutex> g(e->mu);
                e->td.drop_update();
                e->rt.build(e->td, -1);
            }
            PSB_RETURN_IF_ERROR(client_->push_context_nolock(sid_));
            PSB_RETURN_IF_ERROR(client_->require_update_ctx_nolock(sid_, involved, timeout_ms));
            return client_->broadcast(sid_, RequestType::NEW_CTX_PURGE, involved, Archive(), timeout_ms, -1);
        }();
        m.release_lock(PSERVER_LOCK_NAME);
        return st;
    }
};

// Incremental sync of (key, full row) blocks into another table (trainer -> predictor). No auto retry:
// the caller rewinds and backs off (pico-ps/handler/SyncHandler.h:36-74).
class SyncHandler : public Handler {
public:
    using Handler::Handler;
    Status sync_block(const int64_t* keys, const float* rows, size_t n, uint32_t stride, int timeout_ms = 30000) {
        std::shared_ptr<KVSyncOperator> p;
        PSB_RETURN_IF_ERROR(op(&p));
        auto e = entry();
        std::map<int, Archive> plain;
        int32_t built_under = -1;
        {
            std::shared_lock<std::shared_mutex> g(e->mu);
            built_under = e->td.version;
            PSB_RETURN_IF_ERROR(DirectPushOperator::generate_requests(storage_op_of(*e), e->rt, keys, rows, n, stride, &plain));
        }
        std::map<int, Archive> bodies;
        for (auto& kv : plain) {
            std::vector<uint8_t> packed;
            PSB_RETURN_IF_ERROR(p->compressor().compress(kv.second.data(), kv.second.size(), &packed));
            bodies[kv.first] << packed;
        }
        ++metrics_.requests;
        return client_->send_and_wait(sid_, hid_, RequestType::OP_SYNC, bodies, timeout_ms, nullptr, built_under);
    }
    size_t block_size() {
        std::shared_ptr<KVSyncOperator> p;
        return op(&p).ok() ? p->block_size() : 1000;
    }

    // One incremental sync of the trainer table `trainer_sid` (held by `trainer`) into the predictor table behind
    // this handler, with the retry policy of SyncHandler::sync_pred (pico-ps/handler/SyncHandler.h:36-138): a
    // failed pass leaves the dirty marks in place (the iterator is rewound), the handler backs off - NoReplica
    // 5 s, ServerTooNewCtx 1 s (after refreshing the context), Timeout 3 s, InvalidID re-initialises the storage
    // on this client - and tries again, at most `max_attempts` times. `backoff_scale` scales the pauses.
    Status sync_pred(Server& trainer, int32_t trainer_sid, uint64_t* n_synced, int max_attempts = 5, double backoff_scale = 1.0) {
        return sync_pred_impl(trainer, trainer_sid, n_synced, max_attempts, backoff_scale, true);
    }
    // The same pass, but the changed-row marks stay: for a table with several followers, every follower but the last.
    Status sync_pred_keep_marks(Server& trainer, int32_t trainer_sid, uint64_t* n_synced, int max_attempts = 5,
                                double backoff_scale = 1.0) {
        return sync_pred_impl(trainer, trainer_sid, n_synced, max_attempts, backoff_scale, false);
    }

private:
    Status sync_pred_impl(Server& trainer, int32_t trainer_sid, uint64_t* n_synced, int max_attempts, double backoff_scale,
                          bool clear_marks) {
        Status st;
        uint64_t total = 0;
        for (int attempt = 0; attempt < max_attempts; ++attempt) {
            uint64_t n = 0;
            st = trainer.push_sync_table(trainer_sid, block_size(),
                                         [&](const int64_t* k, const float* r, size_t m, uint32_t stride) { return sync_block(k, r, m, stride); }, &n,
                                         clear_marks);
            total += n;
            if (st.ok()) break;
            ++metrics_.retries;
            double pause_s = 0;
            bool refresh_after_pause = false;
            if (st.is(StatusCode::NO_REPLICA)) {
                pause_s = 5;  // somebody may restore the shard meanwhile: look at the published context again afterwards
                refresh_after_pause = true;
            }
            else if (st.is(StatusCode::SERVER_TOO_NEW_CTX) || st.is(StatusCode::SERVER_TOO_NEW_CTX_U)) {
                client_->handle_server_too_new_ctx(sid_);
                pause_s = 1;
            } else if (st.is(StatusCode::TIMEOUT)) {
                client_->handle_timeout(sid_);
                pause_s = 3;
            } else if (st.is(StatusCode::INVALID_ID)) {
                client_->initialize_storage(sid_);
                pause_s = 0.1;
            } else break;  // anything else goes to the caller
            std::this_thread::sleep_for(std::chrono::milliseconds((long)(pause_s * 1000 * backoff_scale)));
            if (refresh_after_pause) client_->pull_context(sid_);
        }
        if (!st.ok()) ++metrics_.errors;
        *n_synced = total;
        return st;
    }
};

class UDFHandler : public Handler {
public:
    using Handler::Handler;
    // Calls the function on every live node of the table; results in node order.
    Status call(const std::string& param, std::vector<std::pair<int, std::string>>* results, int timeout_ms = -1, bool retry = true) {
        return with_retry([&](int left) -> Status {
            results->clear();
            auto e = entry();
            std::map<int, Archive> bodies;
            int32_t built_under = -1;
            {
                std::shared_lock<std::shared_mutex> g(e->mu);
                built_under = e->td.version;
                for (auto& kv : e->rt.nodes())
                    if (e->rt.is_running(kv.first)) bodies[kv.first] << param;
            }
            std::vector<NodeResponse> rs;
            PSB_RETURN_IF_ERROR(client_->send_and_wait(sid_, hid_, RequestType::OP_UDF, bodies, left, &rs, built_under));
            for (auto& r : rs) {
                std::string s;
                r.body >> s;
                results->push_back({r.node, s});
            }
            return Status::Ok();
        }, timeout_ms, retry);
    }

    // Request building split from sending (pico-ps/handler/UDFHandler.cpp:26-36,59-84): a request can be
    // prepared on another thread; send_request refuses it when the table's context has changed since (the node
    // list it was built for may be stale) and the caller generates it again.
    struct Request {
        std::map<int, Archive> bodies;
        int32_t ctx_version = -1;
    };
    Status generate_request(const std::string& param, Request* req) {
        auto e = entry();
        if (!e) return Status::InvalidID("storage is not initialised on this client");
        req->bodies.clear();
        std::shared_lock<std::shared_mutex> g(e->mu);
        req->ctx_version = e->td.version;
        for (auto& kv : e->rt.nodes())
            if (e->rt.is_running(kv.first)) req->bodies[kv.first] << param;
        return Status::Ok();
    }
    Status send_request(const Request& req, std::vector<std::pair<int, std::string>>* results, int timeout_ms = -1) {
        auto e = entry();
        if (!e) return Status::InvalidID("storage is not initialised on this client");
        {
            std::shared_lock<std::shared_mutex> g(e->mu);
            if (e->td.version != req.ctx_version)
                return Status::ServerTooNewCtx("the context changed since the request was generated");
        }
        results->clear();
        std::vector<NodeResponse> rs;
        ++metrics_.requests;
        PSB_RETURN_IF_ERROR(client_->send_and_wait(sid_, hid_, RequestType::OP_UDF, req.bodies, timeout_ms, &rs, req.ctx_version));
        for (auto& r : rs) {
            std::string s;
            r.body >> s;
            results->push_back({r.node, s});
        }
        return Status::Ok();
    }
};

}  // namespace psb
