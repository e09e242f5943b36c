// psb_node: the parameter server's processes as one native executable (no Python in the serving path).
//
//   psb_node master [--threads N] [--port P] [--state-file FILE]
//       prints the master's address on the first line of stdout and serves until it is killed. With a state file
//       (and a fixed port) a restarted master carries on where the old one stopped: ids, contexts and the model
//       registry are read back, the servers register again, clients reconnect.
//   psb_node pserver --master HOST:PORT [--restore] [--image-dir DIR] [--c2s-threads N] [--s2s-threads N]
//       registers at the master, prints "pserver node_id=.. c2s=.. s2s=..", serves both ports and exits when a
//       client sends EXIT (Client::close_pserver / Controller::shutdown_node). With --restore it first takes
//       over the shards of a dead node from their live replicas or from the table's dump
//       (the restore mode of the reference's server process, pico-ps/service/Service.cpp:237-313). With --image-dir
//       it writes its tables' persistent images there on a planned shutdown (EXIT, SIGTERM) and, in restore mode,
//       opens the image of the node it replaces when no live replica has the shards; --image-interval-ms N also
//       refreshes the images every N ms while serving. With --sync-master it runs the
//       sync thread: rows changed by pushes on tables whose push operator names follower tables ("sync_table") are
//       shipped to those tables, found through the model registry of that master. With --metrics-port P it serves
//       the Prometheus text of its request series on GET /metrics (P = 0: any free port, printed as "metrics port=N").
//
//   psb_node ctl --master HOST:PORT VERB ...
//       the controller from the command line: show nodes / a table, create, delete, balance, change the shard or
//       replica count of a table, add nodes to it, clean up storages without a table, shut a node down.
//
// --host ADDR (or $PSB_HOST), for master and pserver: the address of this machine that the process publishes; its
// servers then listen on every interface instead of loopback only, so the roles may run on different machines.
//
// The same objects as the Python bindings: tables with "backend": "gpu" are served by the fused kernels.
#include <algorithm>
#include <chrono>
#include <csignal>
#include <cstdio>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "../controller/controller.h"
#include "../service/master.h"
#include "../service/metrics_http.h"
#include "../service/server.h"
#include "../service/local_images.h"
#include "../service/table_syncer.h"

using namespace psb;

namespace {
volatile std::sig_atomic_t g_stop = 0;
void on_signal(int) { g_stop = 1; }

// psb_node ctl --master HOST:PORT <verb> [args]: the controller from the command line. JSON answers go to stdout.
int ctl_usage() {
    std::fprintf(stderr,
                 "usage: psb_node ctl --master HOST:PORT VERB ...\n"
                 "  nodes | node ID | table SID | clean | shutdown NODE | delete SID | balance SID\n"
                 "  purge SID   (abort a reshard that its client left unfinished: writes resume)\n"
                 "  dump SID URI [FILES_PER_NODE] | load SID URI | stats SID [SECTION] | erase SID PREDICATE_JSON\n"
                 "  shards SID N | replicas SID N | expand SID SHARDS_PER_NODE NODE [NODE ...]\n"
                 "  create NAME SHARDS REPLICAS OP_CONFIG_JSON [TABLE_URI]   (prints storage_id=N)\n");
    return 2;
}
int ctl_main(int argc, char** argv) {
    std::string master;
    std::vector<std::string> a;
    for (int i = 2; i < argc; ++i) {
        if (std::string(argv[i]) == "--master" && i + 1 < argc) master = argv[++i];
        else a.push_back(argv[i]);
    }
    if (master.empty() || a.empty()) return ctl_usage();
    try {
        Controller ctl(master);
        const std::string& verb = a[0];
        auto num = [&](size_t i) {   // a number, all of it: "abc" or "12x" is a mistake, not a 0 or a 12
            const std::string& t = a.at(i);
            size_t used = 0;
            int v = 0;
            try { v = std::stoi(t, &used); } catch (const std::exception&) { used = 0; }
            if (used == 0 || used != t.size()) throw std::invalid_argument("'" + t + "' is not a number");
            return v;
        };
        Status st;
        Json out;
        bool has_out = false;
        if (verb == "nodes") { st = ctl.show_nodes(&out); has_out = true; }
        else if (verb == "node" && a.size() == 2) { st = ctl.show_node(num(1), &out); has_out = true; }
        else if (verb == "table" && a.size() == 2) { st = ctl.gen_table_json(num(1), &out); has_out = true; }
        else if (verb == "clean") {
            int removed = 0;
            st = ctl.clean_unused_storage(&removed);
            if (st.ok()) std::printf("removed=%d\n", removed);
        }
        else if (verb == "shutdown" && a.size() == 2) st = ctl.shutdown_node(num(1));
        else if (verb == "delete" && a.size() == 2) st = ctl.delete_table(num(1));
        else if (verb == "balance" && a.size() == 2) st = ctl.balance_table(num(1));
        else if (verb == "purge" && a.size() == 2) st = ctl.purge_table(num(1));
        else if (verb == "dump" && (a.size() == 3 || a.size() == 4)) {
            uint64_t n = 0;
            st = ctl.dump_table(num(1), a[2], a.size() == 4 ? num(3) : 1, &n);
            if (st.ok()) std::printf("records=%llu\n", (unsigned long long)n);
        }
        else if (verb == "load" && a.size() == 3) {
            uint64_t n = 0;
            st = ctl.load_table(num(1), a[2], &n);
            if (st.ok()) std::printf("records=%llu\n", (unsigned long long)n);
        }
        else if (verb == "stats" && (a.size() == 2 || a.size() == 3)) { st = ctl.table_stats(num(1), a.size() == 3 ? num(2) : 0, &out); has_out = true; }
        else if (verb == "erase" && a.size() == 3) {
            uint64_t n = 0;
            st = ctl.erase_from_table(num(1), a[2], &n);
            if (st.ok()) std::printf("erased=%llu\n", (unsigned long long)n);
        }
        else if (verb == "shards" && a.size() == 3) st = ctl.update_table_shard(num(1), num(2));
        else if (verb == "replicas" && a.size() == 3) st = ctl.update_table_replica(num(1), num(2));
        else if (verb == "expand" && a.size() >= 4) {
            std::vector<int> nodes;
            for (size_t i = 3; i < a.size(); ++i) nodes.push_back(num(i));
            st = ctl.expand_storage_nodes(num(1), nodes, num(2));
        }
        else if (verb == "create" && (a.size() == 5 || a.size() == 6)) {
            int32_t sid = -1;
            st = ctl.create_table(a[1], "psb", "SparseTableStorageOperator", a[4], num(2), num(3), Controller::standard_ops(),
                                  a.size() == 6 ? a[5] : "", &sid);
            if (st.ok()) std::printf("storage_id=%d\n", sid);
        }
        else return ctl_usage();
        if (!st.ok()) {
            std::fprintf(stderr, "psb_node ctl: %s\n", st.to_string().c_str());
            return 1;
        }
        if (has_out) std::printf("%s\n", out.dump().c_str());
    } catch (const std::exception& e) {
        std::fprintf(stderr, "psb_node ctl: %s\n", e.what());
        return 1;
    }
    return 0;
}

// psb_node images DIR [--master HOST:PORT] [--remove-unused [--dead-nodes-too]]: what lies under an image directory
// (JSON on stdout) and removal of what no node can use any more.
int images_main(int argc, char** argv) {
    std::string dir, master;
    bool remove = false, dead_too = false;
    for (int i = 2; i < argc; ++i) {
        const std::string a = argv[i];
        if (a == "--master" && i + 1 < argc) master = argv[++i];
        else if (a == "--remove-unused") remove = true;
        else if (a == "--dead-nodes-too") dead_too = true;
        else if (dir.empty() && a.compare(0, 2, "--") != 0) dir = a;
        else return 2;
    }
    if (dir.empty() || (remove && master.empty())) {
        std::fprintf(stderr, "usage: psb_node images DIR [--master HOST:PORT] [--remove-unused [--dead-nodes-too]]\n");
        return 2;
    }
    try {
        std::unique_ptr<MasterClient> mc;
        if (!master.empty()) mc.reset(new MasterClient(master));
        Status st;
        if (remove) {
            int removed = 0;
            st = remove_unused_local_images(dir, mc.get(), dead_too, &removed);
            if (st.ok()) std::fprintf(stderr, "removed=%d\n", removed);
        }
        std::vector<LocalImage> images;
        if (st.ok()) st = list_local_images(dir, mc.get(), &images);
        if (!st.ok()) {
            std::fprintf(stderr, "psb_node images: %s\n", st.to_string().c_str());
            return 1;
        }
        std::printf("%s\n", local_images_json(images).dump().c_str());
    } catch (const std::exception& e) {
        std::fprintf(stderr, "psb_node images: %s\n", e.what());
        return 1;
    }
    return 0;
}

int usage() {
    std::fprintf(stderr,
                 "usage: psb_node master [--threads N] [--port P] [--state-file FILE] [--host ADDR]\n"
                 "       psb_node ctl --master HOST:PORT VERB ...   (the controller; `psb_node ctl` lists the verbs)\n"
                 "       psb_node images DIR [--master HOST:PORT] [--remove-unused [--dead-nodes-too]]\n"
                 "       psb_node pserver --master HOST:PORT [--restore] [--restore-wait S] [--restore-pauses-writes] [--image-dir DIR] [--image-interval-ms N] [--report-interval S]\n"
                 "                        [--load-threads N] [--c2s-threads N] [--s2s-threads N] [--sync-master HOST:PORT] [--hadoop-bin PATH]\n"
                 "                        [--metrics-port P] [--log-level debug|info|warning|error|off] [--host ADDR]\n");
    return 2;
}
}  // namespace

int main(int argc, char** argv) {
    if (argc < 2) return usage();
    std::signal(SIGINT, on_signal);
    std::signal(SIGTERM, on_signal);
    const std::string role = argv[1];
    if (role == "ctl") return ctl_main(argc, argv);
    if (role == "images") return images_main(argc, argv);
    std::string master_addr, sync_master, state_file;
    int master_port = 0;
    bool restore = false;
    int threads = 4, image_interval_ms = 0, metrics_port = -1;
    ServerConfig cfg;
    for (int i = 2; i < argc; ++i) {
        const std::string a = argv[i];
        auto next = [&](int* out) {
            if (i + 1 >= argc) return false;
            *out = std::atoi(argv[++i]);
            return true;
        };
        if (a == "--master" && i + 1 < argc) master_addr = argv[++i];
        else if (a == "--sync-master" && i + 1 < argc) sync_master = argv[++i];
        else if (a == "--state-file" && i + 1 < argc) state_file = argv[++i];
        else if (a == "--host" && i + 1 < argc) ::setenv("PSB_HOST", argv[++i], 1);   // before any server is created
        else if (a == "--port") { if (!next(&master_port)) return usage(); }
        else if (a == "--restore") restore = true;
        else if (a == "--restore-pauses-writes") cfg.restore_pauses_writes = true;
        else if (a == "--image-dir" && i + 1 < argc) cfg.local_image_dir = argv[++i];
        else if (a == "--hadoop-bin" && i + 1 < argc) cfg.hadoop_bin = argv[++i];
        else if (a == "--log-level" && i + 1 < argc) set_log_level(log_detail::parse(argv[++i], LogLevel::WARNING));
        else if (a == "--metrics-port") { if (!next(&metrics_port)) return usage(); }
        else if (a == "--image-interval-ms") { if (!next(&image_interval_ms)) return usage(); }
        else if (a == "--report-interval") { if (!next(&cfg.report_interval_s)) return usage(); }
        else if (a == "--restore-wait") { if (!next(&cfg.restore_wait_timeout_s)) return usage(); }
        else if (a == "--load-threads") { if (!next(&cfg.load_thread_num)) return usage(); }
        else if (a == "--threads") { if (!next(&threads)) return usage(); }
        else if (a == "--c2s-threads") { if (!next(&cfg.c2s_thread_num)) return usage(); }
        else if (a == "--s2s-threads") { if (!next(&cfg.s2s_thread_num)) return usage(); }
        else return usage();
    }
    if (role == "master") {
        std::unique_ptr<Master> owned;
        try {
            owned.reset(new Master(threads, master_port, state_file));
        } catch (const std::exception& e) {
            std::fprintf(stderr, "psb_node: %s\n", e.what());
            return 1;
        }
        Master& master = *owned;
        std::printf("%s\n", master.address().c_str());
        std::fflush(stdout);
        while (!g_stop) std::this_thread::sleep_for(std::chrono::milliseconds(50));
        master.stop();
        return 0;
    }
    if (role != "pserver" || master_addr.empty()) return usage();
    try {
        Server server(master_addr, cfg);
        std::printf("pserver node_id=%d c2s=%s s2s=%s\n", server.node_id(), server.c2s_address().c_str(), server.s2s_address().c_str());
        std::fflush(stdout);
        // Prometheus endpoint of this server's request series (GET /metrics); port 0 = any free port, printed below
        std::unique_ptr<MetricsHttpServer> metrics;
        if (metrics_port >= 0) {
            metrics.reset(new MetricsHttpServer(metrics_port, [&server] { return server.metrics_text(); }));
            std::printf("metrics port=%d\n", metrics->port());
            std::fflush(stdout);
        }
        // tables whose push operator names follower tables are mirrored to them in the background; the followers
        // live in the cluster of `--sync-master` (which may be this server's own master)
        std::unique_ptr<TableSyncer> syncer;
        if (!sync_master.empty()) syncer.reset(new TableSyncer(&server, sync_master));
        if (restore) {
            int n = 0;
            Status st = server.restore_storages(&n);
            std::string from;
            for (auto& kv : server.restore_sources()) from += (from.empty() ? " from " : ", ") + kv.second;
            std::printf("restore: %s (%d tables)%s\n", st.ok() ? "OK" : st.msg().c_str(), n, from.c_str());
            std::fflush(stdout);
            if (!st.ok()) return 1;
        }
        // with --image-interval-ms the images are also refreshed while serving (checkpoints on the host: a process
        // that is killed leaves the last complete image, never a torn one - temp file + rename)
        auto last_image = std::chrono::steady_clock::now();
        while (!server.exited() && !g_stop) {
            std::this_thread::sleep_for(std::chrono::milliseconds(image_interval_ms > 0 ? std::min(image_interval_ms, 20) : 20));
            if (image_interval_ms > 0 && !cfg.local_image_dir.empty() &&
                std::chrono::steady_clock::now() - last_image >= std::chrono::milliseconds(image_interval_ms)) {
                Status st = server.save_local_images(nullptr);
                if (!st.ok()) std::fprintf(stderr, "psb_node: periodic image: %s\n", st.msg().c_str());
                last_image = std::chrono::steady_clock::now();
            }
        }
        if (metrics) metrics->stop();
        if (syncer) {
            syncer->wait_idle(5000);   // what the last pushes changed still goes out
            syncer->stop();
        }
        if (!cfg.local_image_dir.empty()) {  // a planned shutdown leaves this node's tables on the host
            int n = 0;
            Status st = server.save_local_images(&n);
            std::printf("images: %s (%d tables)\n", st.ok() ? "OK" : st.msg().c_str(), n);
            std::fflush(stdout);
        }
        server.stop();
    } catch (const std::exception& e) {
        std::fprintf(stderr, "psb_node: %s\n", e.what());
        return 1;
    }
    return 0;
}
