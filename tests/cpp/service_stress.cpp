// Race-detection stress of the host control plane, built with -fsanitize=thread by tests/test_tsan_service.py.
//
// One master, three servers and one client in this process (real sockets on localhost, as in the
// reference's integration tests, pico-ps/test/ps_service_test.cpp:77-145). Four worker threads push and pull
// through handlers that share merge groups (request coalescing) while the main thread moves shards between
// the servers four times (the reshard transaction with its context-version gates and client retries). The program
// checks that every gradient was applied exactly once. A second phase reads a table with two replicas per
// shard from four threads while one server is stopped, a fresh one restores the lost shards from the live
// replicas, and a second original server is stopped. A third phase mixes immediate and buffered (sync + store)
// pushes from four threads with statistics scans, writing scans and dumps. In a fourth the controller changes the shard count
// and the replica count of a table and rebalances it while four threads read it. In a fifth the rows that change
// on a trainer table are shipped to a predictor table again and again while four threads keep pushing, and the
// predictor must end up equal to the trainer. A sixth loads the trainer's dump into an in-process table with four
// threads and reads it from four. A seventh sends malformed requests. An eighth closes servers by request and destroys
// them the moment they report that they have left. In a ninth the sync thread of a server keeps a follower table equal
// to a table that four threads push to. In a tenth a table sits at its memory limit while four threads push new keys:
// items are parked, requests refused and sent again, the limit is raised under load, and every gradient counts once.
// The sanitizers check the rest.
#include <algorithm>
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <memory>
#include <string>
#include <thread>
#include <vector>

#include "controller/controller.h"
#include "handler/handlers.h"
#include "native_ps/native_ps.h"
#include "service/master.h"
#include "service/server.h"
#include "service/table_syncer.h"

namespace psb {
// this host-only binary has no CUDA objects: a table that asks for the GPU back-end is refused
Status make_gpu_kv_storage(const GpuKVStorageConfig&, std::unique_ptr<KVStorage>*) {
    return Status::Error("no GPU back-end in this build");
}
}  // namespace psb

using namespace psb;

static std::string nodes_json(const std::vector<std::pair<int, std::vector<int>>>& nodes) {
    std::string s = "[";
    for (size_t i = 0; i < nodes.size(); ++i) {
        s += std::string(i ? "," : "") + "{\"g_rank\":" + std::to_string(nodes[i].first) + ",\"shard_list\":[";
        for (size_t j = 0; j < nodes[i].second.size(); ++j) s += std::string(j ? "," : "") + std::to_string(nodes[i].second[j]);
        s += "]}";
    }
    return s + "]";
}

#define MUST(expr)                                                              \
    do {                                                                        \
        Status _st = (expr);                                                    \
        if (!_st.ok()) {                                                        \
            std::fprintf(stderr, "FAILED %s: %s\n", #expr, _st.msg().c_str()); \
            return 1;                                                           \
        }                                                                       \
    } while (0)

int main() {
    constexpr int kDim = 4, kIters = 120, kKeys = 2000, kBatch = 128;
    const char* env_threads = std::getenv("PSB_STRESS_THREADS");   // worker threads per phase (default 4, at most 32)
    const int kThreads = std::max(1, std::min(32, env_threads ? std::atoi(env_threads) : 4));
    Master master(4);
    std::vector<std::unique_ptr<Server>> servers;
    for (int i = 0; i < 3; ++i) servers.emplace_back(new Server(master.address()));
    Client client(master.address());
    const int n0 = servers[0]->node_id(), n1 = servers[1]->node_id(), n2 = servers[2]->node_id();
    const std::string cfg = "{\"nodes\":" + nodes_json({{n0, {0, 1}}, {n1, {2, 3}}, {n2, {4, 5}}}) +
                            ",\"op_config\":{\"dim\":4,\"optimizer\":\"sum\",\"init_range\":0.0},\"table_name\":\"t\"}";
    int32_t sid = -1, h_pull = -1, h_push = -1, h_ctx = -1;
    MUST(client.create_storage("psb", "SparseTableStorageOperator", cfg, &sid));
    MUST(client.register_handler("pull_ro", "psb", "SparseTablePullOperator", "{\"read_only\":true}", sid, &h_pull));
    MUST(client.register_handler("push", "psb", "SparseTablePushOperator", "{}", sid, &h_push));
    MUST(client.register_handler("update_ctx", "psb", "ShardUpdateContextOperator", "{}", sid, &h_ctx));

    auto pull_group = std::make_shared<PullGroup>();
    auto push_group = std::make_shared<PushGroup>();
    std::vector<std::unique_ptr<PullHandler>> pulls;
    std::vector<std::unique_ptr<PushHandler>> pushes;
    for (int t = 0; t < kThreads; ++t) {
        pulls.emplace_back(new PullHandler(&client, sid, h_pull));
        pushes.emplace_back(new PushHandler(&client, sid, h_push));
        pulls.back()->join_group(pull_group);
        pushes.back()->join_group(push_group);
    }
    std::vector<std::atomic<uint64_t>> pushed(kKeys);
    for (auto& p : pushed) p = 0;
    std::atomic<int> failures{0};
    std::vector<std::thread> workers;
    for (int t = 0; t < kThreads; ++t)
        workers.emplace_back([&, t] {
            uint64_t x = 88172645463325252ull + (uint64_t)t * 7919;
            std::vector<int64_t> keys(kBatch);
            std::vector<float> grads((size_t)kBatch * kDim, 1.0f), rows((size_t)kBatch * kDim);
            for (int it = 0; it < kIters; ++it) {
                for (auto& k : keys) {
                    x ^= x << 13; x ^= x >> 7; x ^= x << 17;
                    k = (int64_t)(x % kKeys);
                }
                Status st = pushes[t]->async_push(keys.data(), grads.data(), keys.size(), 20000);
                if (!st.ok()) { std::fprintf(stderr, "push: %s\n", st.msg().c_str()); ++failures; continue; }
                for (auto k : keys) ++pushed[(size_t)k];
                st = pulls[t]->pull(keys.data(), keys.size(), rows.data(), 20000);
                if (!st.ok()) { std::fprintf(stderr, "pull: %s\n", st.msg().c_str()); ++failures; continue; }
                for (size_t i = 0; i < keys.size(); ++i)
                    if (rows[i * kDim] < 1.0f) ++failures;   // at least this thread's own push is visible
            }
        });
    // two reshards while the load runs: rotate the shard placement, then spread it unevenly
    {
        UpdateContextHandler uc(&client, sid, h_ctx);
        const std::vector<std::vector<std::pair<int, std::vector<int>>>> plans = {
            {{n0, {4, 5}}, {n1, {0, 1}}, {n2, {2, 3}}},       // rotate the placement
            {{n0, {0}}, {n1, {1, 2}}, {n2, {3, 4, 5}}},       // uneven
            {{n0, {0, 1, 2, 3}}, {n1, {4}}, {n2, {5}}},       // pile up on one node
            {{n0, {0, 1}}, {n1, {2, 3}}, {n2, {4, 5}}},       // back to the start
        };
        for (size_t i = 0; i < plans.size(); ++i) {
            std::this_thread::sleep_for(std::chrono::milliseconds(15));
            Status st = uc.update_context(nodes_json(plans[i]));
            if (!st.ok()) { std::fprintf(stderr, "reshard %zu: %s\n", i, st.msg().c_str()); ++failures; }
        }
    }
    for (auto& w : workers) w.join();
    // every gradient exactly once
    std::vector<int64_t> all(kKeys);
    for (int k = 0; k < kKeys; ++k) all[k] = k;
    std::vector<float> rows((size_t)kKeys * kDim);
    MUST(pulls[0]->pull(all.data(), all.size(), rows.data(), 20000));
    int wrong = 0;
    for (int k = 0; k < kKeys; ++k)
        for (int d = 0; d < kDim; ++d)
            if (rows[(size_t)k * kDim + d] != (float)pushed[k].load()) ++wrong;
    std::printf("merged pull sends %llu of %llu, merged push sends %llu of %llu, failures %d, wrong %d\n",
                (unsigned long long)pull_group->merged_sends.load(), (unsigned long long)pull_group->merged_requests.load(),
                (unsigned long long)push_group->merged_sends.load(), (unsigned long long)push_group->merged_requests.load(),
                failures.load(), wrong);
    pulls.clear();
    pushes.clear();

    // ---- phase 2: a replicated table keeps serving reads while a node dies and a fresh server takes over ----
    int wrong2 = 0;
    MUST(client.delete_storage(sid));   // the unreplicated table could not survive the loss of a node
    {
        const std::string cfg2 = "{\"nodes\":" + nodes_json({{n0, {0, 1}}, {n1, {1, 2}}, {n2, {2, 0}}}) +
                                 ",\"op_config\":{\"dim\":4,\"optimizer\":\"sum\",\"init_range\":0.0},\"table_name\":\"r\"}";
        int32_t sid2 = -1, hp = -1, hq = -1;
        MUST(client.create_storage("psb", "SparseTableStorageOperator", cfg2, &sid2));
        MUST(client.register_handler("pull_ro", "psb", "SparseTablePullOperator", "{\"read_only\":true}", sid2, &hp));
        MUST(client.register_handler("push", "psb", "SparseTablePushOperator", "{}", sid2, &hq));
        std::vector<float> vals((size_t)kKeys * kDim);
        for (int k = 0; k < kKeys; ++k)
            for (int d = 0; d < kDim; ++d) vals[(size_t)k * kDim + d] = (float)(k % 13 + 1);
        {
            PushHandler seed(&client, sid2, hq);
            MUST(seed.async_push(all.data(), vals.data(), all.size(), 20000));   // every replica gets it
        }
        std::atomic<bool> stop_readers{false};
        std::atomic<int> bad_reads{0}, reads{0};
        std::vector<std::thread> readers;
        for (int t = 0; t < kThreads; ++t)
            readers.emplace_back([&, t] {
                PullHandler h(&client, sid2, hp);
                std::vector<int64_t> keys(kBatch);
                std::vector<float> got((size_t)kBatch * kDim);
                uint64_t x = 1234567 + (uint64_t)t;
                while (!stop_readers.load()) {
                    for (auto& k : keys) {
                        x ^= x << 13; x ^= x >> 7; x ^= x << 17;
                        k = (int64_t)(x % kKeys);
                    }
                    Status st = h.pull(keys.data(), keys.size(), got.data(), 20000);   // time-out -> dead-node detection -> other replica
                    if (!st.ok()) { std::fprintf(stderr, "read: %s\n", st.msg().c_str()); ++bad_reads; continue; }
                    for (size_t i = 0; i < keys.size(); ++i)
                        if (got[i * kDim] != (float)(keys[i] % 13 + 1)) ++bad_reads;
                    ++reads;
                }
            });
        // one writer as well: it adds zeros (the values that the readers check stay), so that the restore below, which
        // closes the table to writes while it copies, has pushes to hold back and to let through again
        std::atomic<int> writes{0};
        readers.emplace_back([&] {
            PushHandler h(&client, sid2, hq);
            std::vector<int64_t> keys(kBatch);
            std::vector<float> zeros((size_t)kBatch * kDim, 0.0f);
            uint64_t x = 424243;
            while (!stop_readers.load()) {
                for (auto& k : keys) {
                    x ^= x << 13; x ^= x >> 7; x ^= x << 17;
                    k = (int64_t)(x % kKeys);
                }
                Status st = h.async_push(keys.data(), zeros.data(), keys.size(), 30000);
                if (!st.ok()) { std::fprintf(stderr, "phase 2 write: %s\n", st.msg().c_str()); ++bad_reads; continue; }
                ++writes;
            }
        });
        std::this_thread::sleep_for(std::chrono::milliseconds(30));
        servers[1]->stop();                                        // host-side fault: this node is gone
        std::this_thread::sleep_for(std::chrono::milliseconds(200));
        ServerConfig restoring;
        restoring.restore_pauses_writes = true;
        servers.emplace_back(new Server(master.address(), restoring));   // a fresh server replaces it from the live replicas
        int restored = 0;
        Status st = servers.back()->restore_storages(&restored);
        if (!st.ok() || restored < 1) { std::fprintf(stderr, "restore: %s (%d tables)\n", st.msg().c_str(), restored); ++wrong2; }
        servers[0]->stop();                                        // now the restored copy has to serve
        std::this_thread::sleep_for(std::chrono::milliseconds(300));
        stop_readers = true;
        for (auto& r : readers) r.join();
        wrong2 += bad_reads.load();
        std::printf("phase 2: %d reads, %d writes, %d bad, %d tables restored\n", reads.load(), writes.load(), bad_reads.load(), restored);
    }
    wrong += wrong2;

    // ---- phase 3: scans (statistics, dump) and sync push + store run against concurrent async pushes ----------
    {
        std::map<int32_t, std::string> live;
        MUST(client.get_pserver_list(&live));
        std::vector<std::pair<int, std::vector<int>>> placement;
        int shard = 0;
        for (auto& kv : live) {
            placement.push_back({kv.first, {shard, shard + 1}});
            shard += 2;
        }
        const std::string cfg3 = "{\"nodes\":" + nodes_json(placement) +
                                 ",\"op_config\":{\"dim\":4,\"optimizer\":\"sum\",\"init_range\":0.0,\"sync\":true},\"table_name\":\"s\"}";
        int32_t sid3 = -1, hp = -1, hq = -1, hf = -1, hd = -1;
        MUST(client.create_storage("psb", "SparseTableStorageOperator", cfg3, &sid3));
        MUST(client.register_handler("pull_ro", "psb", "SparseTablePullOperator", "{\"read_only\":true}", sid3, &hp));
        MUST(client.register_handler("push", "psb", "SparseTablePushOperator", "{}", sid3, &hq));
        MUST(client.register_handler("for_each", "psb", "ForEachOperator", "{}", sid3, &hf));
        MUST(client.register_handler("dump", "psb", "DumpOperator", "{}", sid3, &hd));
        int32_t hw = -1;
        MUST(client.register_handler("for_each_write", "psb", "ForEachWriteOperator", "{}", sid3, &hw));
        std::vector<std::atomic<uint64_t>> sent(kKeys);
        for (auto& x : sent) x = 0;
        std::atomic<int> bad{0};
        std::vector<std::thread> ts;
        for (int t = 0; t < kThreads; ++t)
            ts.emplace_back([&, t] {
                PushHandler h(&client, sid3, hq);
                std::vector<int64_t> keys(kBatch);
                std::vector<float> grads((size_t)kBatch * kDim, 1.0f);
                uint64_t x = 99991 + (uint64_t)t * 31;
                for (int it = 0; it < 40; ++it) {
                    for (auto& k : keys) {
                        x ^= x << 13; x ^= x >> 7; x ^= x << 17;
                        k = (int64_t)(x % kKeys);
                    }
                    // even threads apply at once, odd threads buffer on the servers until the store below
                    Status st = (t % 2 == 0) ? h.async_push(keys.data(), grads.data(), keys.size(), 20000)
                                             : h.sync_push(keys.data(), grads.data(), keys.size(), 20000);
                    if (!st.ok()) { std::fprintf(stderr, "phase 3 push: %s\n", st.msg().c_str()); ++bad; continue; }
                    for (auto k : keys) ++sent[(size_t)k];
                }
            });
        {
            ForEachHandler fe(&client, sid3, hf);
            DumpHandler dh(&client, sid3, hd);
            char tmpl[] = "/tmp/psb_stress_dump_XXXXXX";
            const char* dir = ::mkdtemp(tmpl);
            for (int round = 0; round < 6 && dir != nullptr; ++round) {
                ForEachResult r;
                Status st = fe.for_each("{}", &r, 20000);
                if (!st.ok()) { std::fprintf(stderr, "for_each: %s\n", st.msg().c_str()); ++bad; }
                // the writing scan walks the rows in place under each shard's write lock, against the pushes; these two
                // leave every value as it is, so the sums checked below still count every gradient once
                ForEachHandler fw(&client, sid3, hw);
                for (const char* carried : {"{\"type\":\"scale\",\"factor\":1.0}", "{\"type\":\"clip\",\"limit\":1e30}"}) {
                    st = fw.for_each(carried, &r, 20000);
                    if (!st.ok()) { std::fprintf(stderr, "for_each (write): %s\n", st.msg().c_str()); ++bad; }
                }
                DumpArgs da;
                da.uri = std::string(dir) + "/d" + std::to_string(round);
                da.file_number = 2;
                uint64_t n = 0;
                st = dh.dump(da, &n, 20000);
                if (!st.ok() || n > (uint64_t)kKeys) { std::fprintf(stderr, "dump: %s (%llu records)\n", st.msg().c_str(), (unsigned long long)n); ++bad; }
            }
            if (dir != nullptr) {
                std::string cmd = std::string("rm -rf ") + dir;
                if (std::system(cmd.c_str()) != 0) ++bad;
            }
        }
        for (auto& t : ts) t.join();
        {
            PushHandler h(&client, sid3, hq);
            MUST(h.store(20000));   // fold what the sync pushes buffered
        }
        PullHandler ph(&client, sid3, hp);
        std::vector<float> got((size_t)kKeys * kDim);
        MUST(ph.pull(all.data(), all.size(), got.data(), 20000));
        int wrong3 = bad.load();
        for (int k = 0; k < kKeys; ++k)
            if (got[(size_t)k * kDim] != (float)sent[k].load()) ++wrong3;
        std::printf("phase 3: %d wrong\n", wrong3);
        wrong += wrong3;
    }
    // ---- phase 4: the controller (its own client) reshapes a table - more shards, two replicas, rebalance - while
    // four threads of the first client keep reading it -------------------------------------------------------------
    {
        Controller ctl(master.address());
        std::vector<OpSpec> ops = {{"pull_ro", "psb", "SparseTablePullOperator", "{\"read_only\":true}"},
                                   {"push", "psb", "SparseTablePushOperator", "{}"},
                                   {"update_ctx", "psb", "ShardUpdateContextOperator", "{}"}};
        int32_t sid4 = -1;
        MUST(ctl.create_table("ctl_table", "psb", "SparseTableStorageOperator",
                              "{\"dim\":4,\"optimizer\":\"sum\",\"init_range\":0.0}", 4, 1, ops, "", &sid4));
        MUST(client.initialize_storage(sid4));
        int32_t hp = -1, hq = -1;
        MUST(client.handler_by_key(sid4, "pull_ro", &hp));
        MUST(client.handler_by_key(sid4, "push", &hq));
        std::vector<float> vals((size_t)kKeys * kDim);
        for (int k = 0; k < kKeys; ++k)
            for (int d = 0; d < kDim; ++d) vals[(size_t)k * kDim + d] = (float)(k % 5 + 2);
        {
            PushHandler seed(&client, sid4, hq);
            MUST(seed.async_push(all.data(), vals.data(), all.size(), 20000));
        }
        std::atomic<bool> stop_readers{false};
        std::atomic<int> bad_reads{0}, reads{0};
        std::vector<std::thread> readers;
        for (int t = 0; t < kThreads; ++t)
            readers.emplace_back([&, t] {
                PullHandler h(&client, sid4, hp);
                std::vector<int64_t> keys(kBatch);
                std::vector<float> got((size_t)kBatch * kDim);
                uint64_t x = 424242 + (uint64_t)t;
                while (!stop_readers.load()) {
                    for (auto& k : keys) {
                        x ^= x << 13; x ^= x >> 7; x ^= x << 17;
                        k = (int64_t)(x % kKeys);
                    }
                    Status st = h.pull(keys.data(), keys.size(), got.data(), 20000);
                    if (!st.ok()) { std::fprintf(stderr, "phase 4 read: %s\n", st.msg().c_str()); ++bad_reads; continue; }
                    for (size_t i = 0; i < keys.size(); ++i)
                        if (got[i * kDim] != (float)(keys[i] % 5 + 2)) ++bad_reads;
                    ++reads;
                }
            });
        int ctl_bad = 0;
        Status st = ctl.update_table_shard(sid4, 6);
        if (!st.ok()) { std::fprintf(stderr, "update_table_shard: %s\n", st.msg().c_str()); ++ctl_bad; }
        st = ctl.update_table_replica(sid4, 2);
        if (!st.ok()) { std::fprintf(stderr, "update_table_replica: %s\n", st.msg().c_str()); ++ctl_bad; }
        st = ctl.balance_table(sid4);
        if (!st.ok()) { std::fprintf(stderr, "balance_table: %s\n", st.msg().c_str()); ++ctl_bad; }
        Json shown;
        st = ctl.show_nodes(&shown);
        if (!st.ok()) ++ctl_bad;
        std::this_thread::sleep_for(std::chrono::milliseconds(100));
        stop_readers = true;
        for (auto& r : readers) r.join();
        std::printf("phase 4: %d reads, %d bad, %d controller errors\n", reads.load(), bad_reads.load(), ctl_bad);
        wrong += bad_reads.load() + ctl_bad;
    }
    // ---- phase 5: incremental sync trainer -> predictor while the trainer is being pushed to ----------------------
    {
        std::map<int32_t, std::string> live;
        MUST(client.get_pserver_list(&live));
        std::vector<int> ids;
        for (auto& kv : live) ids.push_back(kv.first);
        std::vector<Server*> by_id;
        for (int id : ids)
            for (auto& sp : servers)
                if (sp->node_id() == id && !sp->exited()) by_id.push_back(sp.get());
        const std::string opc = ",\"op_config\":{\"dim\":4,\"optimizer\":\"sum\",\"init_range\":0.0},\"table_name\":\"";
        int32_t trainer = -1, predictor = -1, hq = -1, hs = -1, hp = -1;
        MUST(client.create_storage("psb", "SparseTableStorageOperator",
                                   "{\"nodes\":" + nodes_json({{ids[0], {0, 1}}}) + opc + "tr\"}", &trainer));
        MUST(client.create_storage("psb", "SparseTableStorageOperator",
                                   "{\"nodes\":" + nodes_json({{ids[1], {0, 1, 2}}}) + opc + "pr\"}", &predictor));
        MUST(client.register_handler("push", "psb", "SparseTablePushOperator", "{}", trainer, &hq));
        MUST(client.register_handler("sync", "psb", "KVSyncOperator", "{\"block_size\":64}", predictor, &hs));
        MUST(client.register_handler("pull_ro", "psb", "SparseTablePullOperator", "{\"read_only\":true}", predictor, &hp));
        Server* tsrv = by_id.empty() ? nullptr : by_id[0];
        if (tsrv == nullptr) { std::fprintf(stderr, "phase 5: trainer server not found\n"); return 1; }
        MUST(tsrv->enable_sync(trainer));
        std::vector<std::atomic<uint64_t>> sent(kKeys);
        for (auto& x : sent) x = 0;
        std::atomic<int> bad{0};
        std::atomic<bool> pushing{true};
        std::vector<std::thread> ts;
        for (int t = 0; t < kThreads; ++t)
            ts.emplace_back([&, t] {
                PushHandler h(&client, trainer, hq);
                std::vector<int64_t> keys(kBatch);
                std::vector<float> grads((size_t)kBatch * kDim, 1.0f);
                uint64_t x = 777 + (uint64_t)t * 13;
                for (int it = 0; it < 50; ++it) {
                    for (auto& k : keys) {
                        x ^= x << 13; x ^= x >> 7; x ^= x << 17;
                        k = (int64_t)(x % kKeys);
                    }
                    Status st = h.async_push(keys.data(), grads.data(), keys.size(), 20000);
                    if (!st.ok()) { std::fprintf(stderr, "phase 5 push: %s\n", st.msg().c_str()); ++bad; continue; }
                    for (auto k : keys) ++sent[(size_t)k];
                }
            });
        SyncHandler sync(&client, predictor, hs);
        uint64_t synced_total = 0;
        std::thread syncer([&] {
            while (pushing.load()) {
                uint64_t n = 0;
                Status st = sync.sync_pred(*tsrv, trainer, &n, 3, 0.01);
                if (!st.ok()) { std::fprintf(stderr, "phase 5 sync: %s\n", st.msg().c_str()); ++bad; }
                synced_total += n;
                std::this_thread::sleep_for(std::chrono::milliseconds(2));
            }
        });
        for (auto& t : ts) t.join();
        pushing = false;
        syncer.join();
        uint64_t n = 0;
        MUST(sync.sync_pred(*tsrv, trainer, &n, 3, 0.01));        // what the last round left
        synced_total += n;
        PullHandler ph(&client, predictor, hp);
        std::vector<float> got((size_t)kKeys * kDim);
        MUST(ph.pull(all.data(), all.size(), got.data(), 20000));
        int wrong5 = bad.load();
        for (int k = 0; k < kKeys; ++k)
            if (got[(size_t)k * kDim] != (float)sent[k].load()) ++wrong5;
        std::printf("phase 5: %llu rows synced, %d wrong\n", (unsigned long long)synced_total, wrong5);
        wrong += wrong5;

        // ---- phase 6: the trainer's dump is loaded into an in-process table by four threads and read by four ----
        int32_t hd = -1;
        MUST(client.register_handler("dump", "psb", "DumpOperator", "{}", trainer, &hd));
        char tmpl[] = "/tmp/psb_stress_native_XXXXXX";
        const char* dir = ::mkdtemp(tmpl);
        if (dir == nullptr) return 1;
        DumpArgs da;
        da.uri = dir;
        da.file_number = 4;
        uint64_t dumped = 0;
        MUST(DumpHandler(&client, trainer, hd).dump(da, &dumped, 20000));
        NativePS nps;
        int32_t nsid = -1, nl = -1, np_ = -1;
        MUST(nps.create_storage("psb", "SparseTableStorageOperator", "{\"dim\":4,\"optimizer\":\"sum\",\"init_range\":0.0}", 3, &nsid));
        MUST(nps.register_handler(nsid, "load", "psb", "LoadOperator", "{}", &nl));
        MUST(nps.register_handler(nsid, "pull", "psb", "SparseTablePullOperator", "{\"read_only\":true}", &np_));
        uint64_t loaded = 0;
        MUST(NativeLoadHandler(&nps, nsid, nl).load(dir, 4, &loaded));
        std::atomic<int> bad6{0};
        std::vector<std::thread> rs;
        for (int t = 0; t < kThreads; ++t)
            rs.emplace_back([&, t] {
                NativePullHandler h(&nps, nsid, np_);
                std::vector<float> rows((size_t)kKeys * kDim);
                for (int it = 0; it < 5; ++it) {
                    Status st = h.pull(all.data(), all.size(), rows.data());
                    if (!st.ok()) { ++bad6; continue; }
                    for (int k = 0; k < kKeys; ++k)
                        if (rows[(size_t)k * kDim] != (float)sent[k].load()) ++bad6;
                }
            });
        for (auto& t : rs) t.join();
        std::string cmd = std::string("rm -rf ") + dir;
        if (std::system(cmd.c_str()) != 0) ++bad6;
        std::printf("phase 6: dumped %llu, loaded %llu, %d wrong\n", (unsigned long long)dumped, (unsigned long long)loaded, bad6.load());
        wrong += bad6.load() + (dumped == loaded ? 0 : 1);
    }
    // ---- phase 7: malformed requests (random bodies behind a tail that passes every gate) must be answered with an
    // error or dropped, never read out of bounds (the address sanitizer build watches) --------------------------
    {
        std::map<int32_t, std::string> live;
        MUST(client.get_pserver_list(&live));
        const int node = live.begin()->first;
        int32_t fsid = -1;
        MUST(client.create_storage("psb", "SparseTableStorageOperator",
                                   "{\"nodes\":" + nodes_json({{node, {0, 1}}}) +
                                       ",\"op_config\":{\"dim\":4,\"optimizer\":\"sum\",\"init_range\":0.0},\"table_name\":\"fz\"}",
                                   &fsid));
        std::map<std::string, int32_t> h;
        const char* specs[][2] = {{"pull", "SparseTablePullOperator"}, {"push", "SparseTablePushOperator"}, {"for_each", "ForEachOperator"},
                                  {"erase_if", "EraseIfOperator"}, {"load", "LoadOperator"}, {"update_ctx", "ShardUpdateContextOperator"},
                                  {"sync", "KVSyncOperator"}};
        for (auto& sp : specs) MUST(client.register_handler(sp[0], "psb", sp[1], "{}", fsid, &h[sp[0]]));
        const std::pair<RequestType, const char*> kinds[] = {
            {RequestType::OP_FOREACH, "for_each"}, {RequestType::OP_ERASEIF, "erase_if"}, {RequestType::OP_LOAD, "load"},
            {RequestType::OP_PULL, "pull"}, {RequestType::OP_PUSH_ASYNC, "push"}, {RequestType::OP_PUSH_SYNC, "push"},
            {RequestType::OP_STORE, "push"}, {RequestType::NEW_CTX_CREATE_SHARD, "update_ctx"}, {RequestType::NEW_CTX_SHUFFLE, "update_ctx"},
            {RequestType::NEW_CTX_STORE, "update_ctx"}, {RequestType::OP_SYNC, "sync"}, {RequestType::OP_COORDINATED_RESTORE_ITERATE, "pull"}};
        uint64_t x = 0x9E3779B97F4A7C15ull;
        auto rnd = [&] { x ^= x << 13; x ^= x >> 7; x ^= x << 17; return x; };
        int answered = 0;
        for (auto& kd : kinds)
            for (int it = 0; it < 150; ++it) {
                Archive body;
                if (rnd() % 2) body << (int32_t)(rnd() % 4) << (int32_t)(rnd() % 3);          // plausible counts first
                if (rnd() % 4 == 0) body << (int32_t)(rnd() % 3) << (int32_t)0x7FFFFFF0;       // then a hostile one
                const size_t len = rnd() % 200;
                for (size_t i = 0; i < len; ++i) body << (uint8_t)rnd();
                std::map<int, Archive> bodies;
                bodies[node] = body;
                std::vector<NodeResponse> rs;
                client.send_and_wait(fsid, h[kd.second], kd.first, bodies, 2000, &rs);
                answered += rs.empty() ? 0 : 1;
            }
        // the server still works
        std::vector<float> one(kDim, 2.0f), got(kDim);
        int64_t k = 5;
        MUST(PushHandler(&client, fsid, h["push"]).async_push(&k, one.data(), 1, 20000));
        MUST(PullHandler(&client, fsid, h["pull"]).pull(&k, 1, got.data(), 20000));
        std::printf("phase 7: %d malformed requests answered\n", answered);
        if (got[0] < 2.0f) ++wrong;
    }
    // ---- phase 8: servers asked to leave (EXIT) are destroyed the moment they report exited(), while the thread that
    // the request started may still be joining their worker pools -----------------------------------------------------
    {
        int closed = 0;
        for (int round = 0; round < 8; ++round) {
            std::unique_ptr<Server> extra(new Server(master.address()));
            const int node = extra->node_id();
            MUST(client.close_pserver(node));
            while (!extra->exited()) std::this_thread::yield();
            extra.reset();
            ++closed;
        }
        std::printf("phase 8: %d servers closed by request\n", closed);
    }
    // ---- phase 9: the sync thread of a server ships what concurrent pushes change to a follower table -------------
    {
        std::unique_ptr<Server> tr(new Server(master.address())), pr(new Server(master.address()));
        Client c9(master.address());
        const std::string opc9 = ",\"op_config\":{\"dim\":4,\"optimizer\":\"sum\",\"init_range\":0.0},\"table_name\":\"";
        int32_t fsid = -1, fh_sync = -1, fh_pull = -1, tsid = -1, th_push = -1;
        MUST(c9.create_storage("psb", "SparseTableStorageOperator",
                               "{\"nodes\":" + nodes_json({{pr->node_id(), {0, 1, 2}}}) + opc9 + "followed\"}", &fsid));
        MUST(c9.register_handler("sync", "psb", "KVSyncOperator", "{\"block_size\":64}", fsid, &fh_sync));
        MUST(c9.register_handler("pull_ro", "psb", "SparseTablePullOperator", "{\"read_only\":true}", fsid, &fh_pull));
        ModelObject model;
        model.name = "stress_model";
        TableObject tobj;
        tobj.table_name = "followed";
        tobj.storage_id = fsid;
        tobj.ops.push_back(OperatorObject{"sync", "psb", "KVSyncOperator", "{}", fh_sync});
        model.tables.push_back(tobj);
        MUST(set_model(c9.master(), model));
        MUST(c9.create_storage("psb", "SparseTableStorageOperator",
                               "{\"nodes\":" + nodes_json({{tr->node_id(), {0, 1}}}) + opc9 + "leader\"}", &tsid));
        MUST(c9.register_handler("push", "psb", "SparseTablePushOperator",
                                 "{\"sync_table\":[{\"model_name\":\"stress_model\",\"table_name\":\"followed\",\"op_key\":\"sync\"}]}",
                                 tsid, &th_push));
        TableSyncer syncer(tr.get(), master.address(), 3, 0.01);
        std::vector<std::atomic<uint64_t>> sent9(kKeys);
        for (auto& x : sent9) x = 0;
        std::atomic<int> bad9{0};
        std::vector<std::thread> ts;
        for (int t = 0; t < kThreads; ++t)
            ts.emplace_back([&, t] {
                PushHandler h(&c9, tsid, th_push);
                std::vector<int64_t> keys(kBatch);
                std::vector<float> grads((size_t)kBatch * kDim, 1.0f);
                uint64_t x = 4242 + (uint64_t)t * 17;
                for (int it = 0; it < 50; ++it) {
                    for (auto& k : keys) {
                        x ^= x << 13; x ^= x >> 7; x ^= x << 17;
                        k = (int64_t)(x % kKeys);
                    }
                    Status st = h.async_push(keys.data(), grads.data(), keys.size(), 20000);
                    if (!st.ok()) { std::fprintf(stderr, "phase 9 push: %s\n", st.msg().c_str()); ++bad9; continue; }
                    for (auto k : keys) ++sent9[(size_t)k];
                }
            });
        for (auto& t : ts) t.join();
        if (!syncer.wait_idle(30000)) { std::fprintf(stderr, "phase 9: the sync thread did not settle\n"); ++bad9; }
        std::vector<int64_t> all9(kKeys);
        for (int k = 0; k < kKeys; ++k) all9[k] = k;
        std::vector<float> got9((size_t)kKeys * kDim);
        MUST(PullHandler(&c9, fsid, fh_pull).pull(all9.data(), all9.size(), got9.data(), 20000));
        int wrong9 = bad9.load();
        for (int k = 0; k < kKeys; ++k)
            if (got9[(size_t)k * kDim] != (float)sent9[k].load()) ++wrong9;
        const auto stats9 = syncer.stats();
        std::printf("phase 9: %llu rows in %llu rounds, %llu errors, %d wrong\n", (unsigned long long)stats9.rows,
                    (unsigned long long)stats9.rounds, (unsigned long long)stats9.errors, wrong9);
        wrong += wrong9 + (int)stats9.errors;
        MUST(c9.delete_storage(tsid));
        syncer.wait_idle(5000);
        syncer.stop();
        tr->stop();
        pr->stop();
    }
    // ---- phase 10: a table at its memory limit: pushes that hit it are parked, later ones refused and sent again, the
    // limit is raised under load and the monitor thread drains what was parked - every gradient counts exactly once ----
    {
        ServerConfig mcfg;
        mcfg.report_interval_s = 1;   // the monitor (and a status line on stderr per second)
        std::unique_ptr<Server> srv(new Server(master.address(), mcfg));
        Client c10(master.address());
        int32_t msid = -1, mh_push = -1, mh_pull = -1;
        MUST(c10.create_storage("psb", "SparseTableStorageOperator",
                                "{\"nodes\":" + nodes_json({{srv->node_id(), {0, 1}}}) +
                                    ",\"op_config\":{\"dim\":4,\"optimizer\":\"sum\",\"init_range\":0.0,\"memory_limit\":65536},\"table_name\":\"tight\"}",
                                &msid));
        MUST(c10.register_handler("push", "psb", "SparseTablePushOperator", "{}", msid, &mh_push));
        MUST(c10.register_handler("pull_ro", "psb", "SparseTablePullOperator", "{\"read_only\":true}", msid, &mh_pull));
        constexpr int kNew = 8000;   // about twice what fits under the first limit
        std::vector<std::atomic<uint64_t>> sent10(kNew);
        for (auto& x : sent10) x = 0;
        std::atomic<int> bad10{0}, refused{0};
        std::vector<std::thread> ts;
        for (int t = 0; t < kThreads; ++t)
            ts.emplace_back([&, t] {
                PushHandler h(&c10, msid, mh_push);
                std::vector<int64_t> keys(200);
                std::vector<float> grads(keys.size() * kDim, 1.0f);
                uint64_t x = 99 + (uint64_t)t * 31;
                for (int it = 0; it < 12; ++it) {
                    for (auto& k : keys) {
                        x ^= x << 13; x ^= x >> 7; x ^= x << 17;
                        k = (int64_t)(x % kNew);
                    }
                    Status st;
                    for (int attempt = 0; attempt < 100; ++attempt) {
                        st = h.async_push(keys.data(), grads.data(), keys.size(), 150);
                        if (st.ok()) break;
                        ++refused;
                        std::this_thread::sleep_for(std::chrono::milliseconds(20));
                    }
                    if (!st.ok()) { std::fprintf(stderr, "phase 10 push: %s\n", st.msg().c_str()); ++bad10; continue; }
                    for (auto k : keys) ++sent10[(size_t)k];
                }
            });
        std::this_thread::sleep_for(std::chrono::milliseconds(1200));
        {
            auto e = srv->context().get(msid);
            if (e && e->storage) e->storage->set_limits(1 << 24, 1 << 24);   // the operator gives the table more room
        }
        for (auto& t : ts) t.join();
        std::this_thread::sleep_for(std::chrono::milliseconds(1500));      // one more monitor round drains the rest
        std::vector<int64_t> all10(kNew);
        for (int k = 0; k < kNew; ++k) all10[k] = k;
        std::vector<float> got10((size_t)kNew * kDim);
        Status pst;
        for (int attempt = 0; attempt < 50; ++attempt) {
            pst = PullHandler(&c10, msid, mh_pull).pull(all10.data(), all10.size(), got10.data(), 2000);
            if (pst.ok()) break;
            std::this_thread::sleep_for(std::chrono::milliseconds(100));
        }
        MUST(pst);
        int wrong10 = bad10.load();
        for (int k = 0; k < kNew; ++k)
            if (got10[(size_t)k * kDim] != (float)sent10[k].load()) ++wrong10;
        std::printf("phase 10: %d refusals on the way, %d wrong\n", refused.load(), wrong10);
        wrong += wrong10;
        srv->stop();
    }
    for (auto& s : servers) s->stop();
    master.stop();
    if (failures.load() == 0 && wrong == 0) {
        std::printf("STRESS OK\n");
        return 0;
    }
    return 1;
}
