// Control-plane bindings: master, server, client, handlers, controller, model objects, native PS and
// the small common pieces (archive / message codec, thread coalescing, heap, compression).
#include <pybind11/functional.h>
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "common/base64.h"
#include "common/heap.h"
#include "common/thread_sync.h"
#include "controller/controller.h"
#include "handler/handlers.h"
#include "native_ps/native_ps.h"
#include "service/local_images.h"
#include "service/table_syncer.h"

namespace py = pybind11;
using namespace psb;

using KeyArray = py::array_t<int64_t, py::array::c_style | py::array::forcecast>;
using F32Array = py::array_t<float, py::array::c_style | py::array::forcecast>;
using nogil = py::call_guard<py::gil_scoped_release>;

namespace {
template <class H>
std::unique_ptr<H> make_handler(Client& c, int32_t sid, int32_t hid) { return std::unique_ptr<H>(new H(&c, sid, hid)); }

py::dict metrics_dict(Handler& h) {
    py::dict d;
    d["requests"] = (uint64_t)h.metrics().requests;
    d["retries"] = (uint64_t)h.metrics().retries;
    d["errors"] = (uint64_t)h.metrics().errors;
    d["wait_us"] = (uint64_t)h.metrics().wait_us;
    d["sends"] = (uint64_t)h.metrics().sends;
    d["send_us"] = (uint64_t)h.metrics().send_us;
    return d;
}
}  // namespace

void bind_service(py::module_& m) {
    register_builtin_operators();

    // ---- codec / common ----------------------------------------------------------------------
    m.def("message_round_trip", [](py::bytes body, int sid, int hid, int ver, int uver, int type) {
        PSMessage msg;
        std::string b = body;
        msg.ar.write_raw(b.data(), b.size());
        msg.meta.sid = sid; msg.meta.hid = hid; msg.meta.ctx_ver = ver; msg.meta.ctx_u_ver = uver;
        msg.meta.req_type = (RequestType)type;
        Bytes wire = msg.seal();
        PSMessage back = PSMessage::open(wire);
        return py::make_tuple(py::bytes((const char*)wire.data(), wire.size()),
                              py::bytes((const char*)back.ar.data(), back.ar.size()), back.meta.sid, back.meta.hid,
                              back.meta.ctx_ver, back.meta.ctx_u_ver, (int)back.meta.req_type);
    });
    m.def("request_type_name", [](int t) { return std::string(request_type_name((RequestType)t)); });
    m.def("archive_round_trip", [](int64_t i, double d, const std::string& s, const std::vector<int32_t>& v,
                                   const std::vector<std::string>& vs) {
        Archive ar;
        ar << i << d << s << v << vs << Status::OOM("full");
        int64_t i2; double d2; std::string s2; std::vector<int32_t> v2; std::vector<std::string> vs2; Status st;
        ar >> i2 >> d2 >> s2 >> v2 >> vs2 >> st;
        return py::make_tuple(i2, d2, s2, v2, vs2, (int)st.code(), st.msg(), ar.is_exhausted(), ar.size());
    });
    m.def("compress_round_trip", [](const std::string& algo, py::bytes data) {
        Compressor c;
        Status st = Compressor::create(algo, &c);
        if (!st.ok()) return py::make_tuple(st, py::bytes(), (size_t)0);
        std::string in = data;
        std::vector<uint8_t> packed, plain;
        st = c.compress((const uint8_t*)in.data(), in.size(), &packed);
        if (st.ok()) st = c.decompress(packed.data(), packed.size(), &plain);
        return py::make_tuple(st, py::bytes((const char*)plain.data(), plain.size()), packed.size());
    });
    m.def("compress_only", [](const std::string& algo, py::bytes data) {
        Compressor c;
        Status st = Compressor::create(algo, &c);
        std::vector<uint8_t> packed;
        std::string in = data;
        if (st.ok()) st = c.compress((const uint8_t*)in.data(), in.size(), &packed);
        return py::make_tuple(st, py::bytes((const char*)packed.data(), packed.size()));
    });
    m.def("decompress_only", [](const std::string& algo, py::bytes data) {
        Compressor c;
        Status st = Compressor::create(algo, &c);
        std::vector<uint8_t> plain;
        std::string in = data;
        if (st.ok()) st = c.decompress((const uint8_t*)in.data(), in.size(), &plain);
        return py::make_tuple(st, py::bytes((const char*)plain.data(), plain.size()));
    });
    m.def("heap_sort", [](std::vector<double> v) {
        Heap<double> h;
        for (double x : v) h.push(x);
        std::vector<double> out;
        while (!h.empty()) out.push_back(h.pop());
        return out;
    });
    py::class_<ThreadReduce>(m, "ThreadReduce").def(py::init<>()).def("add", &ThreadReduce::add).def("reduce", &ThreadReduce::reduce);
    py::class_<ThreadBcast>(m, "ThreadBcast")
        .def(py::init<>())
        .def("notify", &ThreadBcast::notify)
        .def("wait", &ThreadBcast::wait, nogil());

    // ---- table descriptor ----------------------------------------------------------------------
    py::class_<TableDescriptor>(m, "TableDescriptor")
        .def(py::init<>())
        .def_readwrite("version", &TableDescriptor::version)
        .def_readwrite("update_version", &TableDescriptor::update_version)
        .def_readwrite("version_uuid", &TableDescriptor::version_uuid)
        .def_readwrite("table_uri", &TableDescriptor::table_uri)
        .def("to_json_str", &TableDescriptor::to_json_str)
        .def("from_json_str", &TableDescriptor::from_json_str, py::arg("json"), py::arg("only_if_newer") = false)
        .def("status", [](TableDescriptor& t) { return (int)t.status; })
        .def("global_shard_num", &TableDescriptor::global_shard_num)
        .def("set_nodes", [](TableDescriptor& t, const std::string& nodes_json) {
            Json j;
            if (!Json::parse(nodes_json, &j)) return Status::InvalidConfig("nodes JSON does not parse");
            t.nodes.clear();
            Status st = TableDescriptor::parse_nodes(j, &t.nodes);
            t.refresh_info();
            return st;
        })
        .def("update_node_status", [](TableDescriptor& t, const std::set<int>& live) { return t.update_node_status(live); })
        .def("try_to_replace_one_dead_node", [](TableDescriptor& t, int my_id) { return t.try_to_replace_one_dead_node(my_id); })
        .def("set_node_status_to_running", &TableDescriptor::set_node_status_to_running)
        .def("create_update_info", [](TableDescriptor& t, const std::string& nodes_json) {
            Json j;
            std::vector<NodeDescriptor> nodes;
            if (!Json::parse(nodes_json, &j)) return Status::InvalidConfig("nodes JSON does not parse");
            Status st = TableDescriptor::parse_nodes(j, &nodes);
            if (st.ok()) t.create_update_info(nodes);
            return st;
        })
        .def("apply_update", &TableDescriptor::apply_update)
        .def("drop_update", &TableDescriptor::drop_update)
        .def("node_status", [](TableDescriptor& t) {
            std::map<int, int> out;
            for (auto& n : t.nodes) out[n.node_id] = (int)n.status;
            return out;
        })
        .def("shards", [](TableDescriptor& t) { return t.shards; })
        .def("pick_one_replica", [](TableDescriptor& t, int shard) { return RuntimeInfo(t, -1).pick_one_replica(shard); });

    // ---- master ----------------------------------------------------------------------------------
    py::class_<Master>(m, "Master").def(py::init<int, int, std::string, int>(), py::arg("n_threads") = 4, py::arg("port") = 0, py::arg("state_file") = "", py::arg("recover_ms") = 3000).def("address", &Master::address).def("stop", &Master::stop, nogil());
    py::class_<MasterClient>(m, "MasterClient")
        .def(py::init<std::string, int>(), py::arg("address"), py::arg("timeout_ms") = 30000)
        .def("generate_id", [](MasterClient& c, const std::string& k) { int32_t id = -1; Status st = c.generate_id(k, &id); return std::make_tuple(st, id); }, nogil())
        .def("acquire_lock", &MasterClient::acquire_lock, nogil())
        .def("release_lock", &MasterClient::release_lock, nogil())
        .def("set_context", &MasterClient::set_context, py::arg("key"), py::arg("value"), py::arg("only_if_absent") = false, nogil())
        .def("get_context", [](MasterClient& c, const std::string& k) { std::string v; Status st = c.get_context(k, &v); return std::make_tuple(st, v); }, nogil())
        .def("delete_context", &MasterClient::delete_context, nogil())
        .def("list_contexts", [](MasterClient& c) { std::vector<std::string> k; Status st = c.list_contexts(&k); return std::make_tuple(st, k); }, nogil())
        .def("register_node", [](MasterClient& c, const std::string& s, const std::string& a, int32_t want_id) {
            int32_t id = -1;
            Status st = c.register_node(s, a, &id, want_id);
            return std::make_tuple(st, id);
        }, py::arg("service"), py::arg("address"), py::arg("want_id") = -1, nogil())
        .def("get_nodes", [](MasterClient& c, const std::string& s) { std::map<int32_t, std::string> n; Status st = c.get_nodes(s, &n); return std::make_tuple(st, n); }, nogil())
        .def("barrier", &MasterClient::barrier, nogil())
        .def("tree_node_set", &MasterClient::tree_node_set, nogil())
        .def("tree_node_get", [](MasterClient& c, const std::string& p) { std::string v; Status st = c.tree_node_get(p, &v); return std::make_tuple(st, v); }, nogil())
        .def("tree_node_del", &MasterClient::tree_node_del, nogil())
        .def("close", &MasterClient::close, nogil());

    // ---- server ----------------------------------------------------------------------------------
    py::class_<ServerConfig>(m, "ServerConfig")
        .def(py::init<>())
        .def_readwrite("c2s_thread_num", &ServerConfig::c2s_thread_num)
        .def_readwrite("s2s_thread_num", &ServerConfig::s2s_thread_num)
        .def_readwrite("load_thread_num", &ServerConfig::load_thread_num)
        .def_readwrite("load_block_size", &ServerConfig::load_block_size)
        .def_readwrite("restore_batch_size", &ServerConfig::restore_batch_size)
        .def_readwrite("restore_pauses_writes", &ServerConfig::restore_pauses_writes)
        .def_readwrite("restore_thread_num", &ServerConfig::restore_thread_num)
        .def_readwrite("s2s_timeout_ms", &ServerConfig::s2s_timeout_ms)
        .def_readwrite("local_image_dir", &ServerConfig::local_image_dir)
        .def_readwrite("hadoop_bin", &ServerConfig::hadoop_bin)
        .def_readwrite("session_check_ms", &ServerConfig::session_check_ms)
        .def_readwrite("report_interval_s", &ServerConfig::report_interval_s)
        .def_readwrite("restore_wait_timeout_s", &ServerConfig::restore_wait_timeout_s);
    // the sync thread of a server: keeps the follower tables named by push operators ("sync_table") fresh
    py::class_<TableSyncer>(m, "TableSyncer")
        .def(py::init<Server*, const std::string&, int, double>(), py::arg("server"), py::arg("follower_master"),
             py::arg("max_attempts") = 5, py::arg("backoff_scale") = 1.0, py::keep_alive<1, 2>(), nogil())
        .def("stop", &TableSyncer::stop, nogil())
        .def("wait_idle", &TableSyncer::wait_idle, py::arg("timeout_ms") = 10000, nogil())
        .def("stats", [](TableSyncer& t) {
            auto s = t.stats();
            py::dict d;
            d["rounds"] = s.rounds;
            d["rows"] = s.rows;
            d["errors"] = s.errors;
            d["last_error"] = s.last_error;
            return d;
        });
    py::class_<Server>(m, "Server")
        .def(py::init<const std::string&, const ServerConfig&>(), py::arg("master"), py::arg("config") = ServerConfig(), nogil())
        .def("node_id", &Server::node_id)
        .def("c2s_address", &Server::c2s_address)
        .def("s2s_address", &Server::s2s_address)
        .def("exited", &Server::exited)
        .def("stop", &Server::stop, nogil())
        .def("metrics", &Server::metrics)
        .def("metrics_text", &Server::metrics_text)
        .def("report_line", &Server::report_line)
        .def("last_report", &Server::last_report)
        .def("save_local_images", [](Server& s) { int n = 0; Status st = s.save_local_images(&n); return std::make_tuple(st, n); }, nogil())
        .def("restore_storages", [](Server& s) { int n = 0; Status st = s.restore_storages(&n); return std::make_tuple(st, n); }, nogil())
        .def("drop_master_session", &Server::drop_master_session, nogil())
        .def("restore_sources", &Server::restore_sources)
        .def("clean_local_images", [](Server& s) {
            int n = 0;
            Status st = s.clean_local_images(&n);
            return std::make_tuple(st, n);
        }, nogil())
        .def("enable_sync", &Server::enable_sync)
        .def("push_sync_table", [](Server& s, int32_t sid, SyncHandler& h) {
            uint64_t n = 0;
            Status st = s.push_sync_table(sid, h.block_size(), [&](const int64_t* k, const float* r, size_t m, uint32_t stride) {
                return h.sync_block(k, r, m, stride);
            }, &n);
            return std::make_tuple(st, n);
        }, nogil())
        .def("storage_size", [](Server& s, int32_t sid) -> int64_t {
            auto e = s.context().get(sid);
            return e && e->storage ? (int64_t)e->storage->size() : -1;
        })
        .def("set_memory_limit", [](Server& s, int32_t sid, uint64_t limit) {
            auto e = s.context().get(sid);
            if (!e || !e->storage) return Status::InvalidID("no such storage");
            e->storage->set_limits(limit, limit);
            return Status::Ok();
        })
        .def("set_healthy", [](Server& s, int32_t sid, bool h) {
            auto e = s.context().get(sid);
            if (e && e->storage) e->storage->set_healthy(h);
        });

    // binary values inside configs (compressed + base64) and the hex printer
    m.def("base64_encode", [](py::bytes b) { std::string s = b; return base64_encode((const uint8_t*)s.data(), s.size()); });
    m.def("base64_decode", [](const std::string& text) -> py::object {
        std::vector<uint8_t> out;
        if (!base64_decode(text, &out)) return py::none();
        return py::bytes((const char*)out.data(), out.size());
    });
    m.def("add_base64_config", [](const std::string& conf_json, const std::string& key, py::bytes value) {
        Json j = Json::parse_or_throw(conf_json);
        std::string v = value;
        Status st = add_base64_config(j, key, (const uint8_t*)v.data(), v.size());
        if (!st.ok()) throw std::runtime_error(st.to_string());
        return j.dump();
    });
    m.def("get_base64_config", [](const std::string& conf_json, const std::string& key) {
        std::vector<uint8_t> out;
        Status st = get_base64_config(Json::parse_or_throw(conf_json), key, &out);
        return std::make_tuple(st, py::bytes((const char*)out.data(), out.size()));
    });
    m.def("byte2str", [](py::bytes b) { std::string s = b; return byte2str((const uint8_t*)s.data(), s.size()); });
    // a config text as the native layer reads it (JSON, or the YAML subset of Json::parse_config), as JSON
    m.def("config_to_json", [](const std::string& text) {
        Json j;
        std::string err;
        if (!Json::parse_config(text, &j, &err)) throw std::runtime_error("config does not parse: " + err);
        return j.dump();
    });
    // logging of the host runtime: level by name ("debug", "info", "warning", "error", "off"); lines go to stderr or,
    // with a sink, to a Python callable (level: int, message: str) - e.g. a forwarder into the `logging` module
    m.def("set_log_level", [](const std::string& name) { set_log_level(log_detail::parse(name.c_str(), LogLevel::WARNING)); });
    m.def("log_level", [] { return (int)log_level(); });
    m.def("set_log_sink", [](py::object fn) {
        if (fn.is_none()) {
            set_log_sink(nullptr);
            return;
        }
        // like the UDF registry: the sink is a process-wide static, the reference to the callable is never dropped
        std::shared_ptr<py::object> holder(new py::object(std::move(fn)), [](py::object*) {});
        set_log_sink([holder](LogLevel l, const std::string& msg) {
            if (!Py_IsInitialized()) return;
            py::gil_scoped_acquire gil;
            try {
                (*holder)((int)l, msg);
            } catch (const std::exception&) {
                // a failing sink must not take the serving thread along
            }
        });
    });
    // dump / load paths with a remote scheme (hdfs://...) go through this command (`<bin> fs -cat / -put / -ls ...`)
    // housekeeping of an image directory from outside a server (psb_node images): JSON list, removal of unused ones
    m.def("list_local_images", [](const std::string& dir, const std::string& master) {
        std::unique_ptr<MasterClient> mc;
        if (!master.empty()) mc.reset(new MasterClient(master));
        std::vector<LocalImage> images;
        Status st = list_local_images(dir, mc.get(), &images);
        return py::make_tuple(st, local_images_json(images).dump());
    }, py::arg("dir"), py::arg("master") = "");
    m.def("remove_unused_local_images", [](const std::string& dir, const std::string& master, bool dead_nodes_too) {
        std::unique_ptr<MasterClient> mc;
        if (!master.empty()) mc.reset(new MasterClient(master));
        int removed = 0;
        Status st = remove_unused_local_images(dir, mc.get(), dead_nodes_too, &removed);
        return py::make_tuple(st, removed);
    }, py::arg("dir"), py::arg("master"), py::arg("dead_nodes_too") = false);
    m.def("set_hadoop_bin", &fs::set_hadoop_bin);
    m.def("hadoop_bin", &fs::hadoop_bin);
    m.def("register_udf", [](const std::string& name, py::function fn) {
        // fn(storage_id: int, node_items: int, param: bytes) -> bytes
        // The registry is a process-wide static that outlives the interpreter, so the reference to the Python
        // function is deliberately never dropped: releasing it during static destruction, after the interpreter has
        // been finalised, crashes the process on its way out.
        std::shared_ptr<py::function> holder(new py::function(std::move(fn)), [](py::function*) {});
        UDFRegistry::instance().add(name, [holder](TableEntry& e, const std::string& param, std::string* result) {
            py::gil_scoped_acquire gil;
            try {
                py::object r = (*holder)(e.sid, e.storage ? (int64_t)e.storage->size() : (int64_t)-1, py::bytes(param));
                *result = (std::string)py::bytes(r);
            } catch (const std::exception& ex) {
                return Status::Error(std::string("udf raised: ") + ex.what());
            }
            return Status::Ok();
        });
    });

    // ---- client + handlers -----------------------------------------------------------------------
    py::class_<StorageStatisticInfo>(m, "StorageStatisticInfo")
        .def_readonly("item_number", &StorageStatisticInfo::item_number)
        .def_readonly("memory_usage", &StorageStatisticInfo::memory_usage)
        .def_readonly("node_id", &StorageStatisticInfo::node_id)
        .def_readonly("shard_id", &StorageStatisticInfo::shard_id);

    py::class_<Client>(m, "Client")
        .def(py::init<const std::string&>(), py::arg("master"))
        .def("get_pserver_list", [](Client& c) { std::map<int32_t, std::string> n; Status st = c.get_pserver_list(&n); return std::make_tuple(st, n); }, nogil())
        .def("get_available_pserver_list", [](Client& c, int timeout_ms) { std::vector<int32_t> n; Status st = c.get_available_pserver_list(&n, timeout_ms); return std::make_tuple(st, n); },
             py::arg("timeout_ms") = 2000, nogil())
        .def("create_storage", [](Client& c, const std::string& lib, const std::string& op, const std::string& cfg) {
            int32_t sid = -1;
            Status st = c.create_storage(lib, op, cfg, &sid);
            return std::make_tuple(st, sid);
        }, nogil())
        .def("pred_create_storage", [](Client& c, const std::string& lib, const std::string& op, const std::string& cfg) {
            int32_t sid = -1;
            Status st = c.pred_create_storage(lib, op, cfg, &sid);
            return std::make_tuple(st, sid);
        }, nogil())
        .def("require_update_ctx_async", &Client::require_update_ctx_async, nogil())
        .def("initialize_storage", &Client::initialize_storage, nogil())
        .def("delete_storage", &Client::delete_storage, py::arg("sid"), py::arg("timeout_ms") = 30000, nogil())
        .def("clear_storage", &Client::clear_storage, py::arg("sid"), py::arg("timeout_ms") = 30000, nogil())
        .def("query_storage_info", [](Client& c, int32_t sid) {
            std::vector<StorageStatisticInfo> info;
            Status st = c.query_storage_info(sid, &info);
            return std::make_tuple(st, info);
        }, nogil())
        .def("query_memory_info", [](Client& c, int node) {
            NodeMemoryInfo mi;
            Status st = c.query_memory_info(node, &mi);
            return std::make_tuple(st, mi.healthy, mi.used, mi.managed);
        }, nogil())
        .def("health_check", &Client::health_check, py::arg("node"), py::arg("timeout_ms") = 2000, nogil())
        .def("close_pserver", &Client::close_pserver, py::arg("node"), py::arg("timeout_ms") = 5000, nogil())
        .def("load_operator_library", &Client::load_operator_library, py::arg("path"), py::arg("timeout_ms") = 30000, nogil())
        .def("register_handler", [](Client& c, const std::string& key, const std::string& lib, const std::string& op,
                                    const std::string& cfg, int32_t sid) {
            int32_t hid = -1;
            Status st = c.register_handler(key, lib, op, cfg, sid, &hid);
            return std::make_tuple(st, hid);
        }, nogil())
        .def("deregister_handler", &Client::deregister_handler, py::arg("sid"), py::arg("hid"), py::arg("timeout_ms") = 30000, nogil())
        .def("handler_by_key", [](Client& c, int32_t sid, const std::string& key) { int32_t h = -1; Status st = c.handler_by_key(sid, key, &h); return py::make_tuple(st, h); })
        .def("set_table_uri", &Client::set_table_uri, nogil())
        .def("get_current_ctx", [](Client& c, int32_t sid) { std::string j; Status st = c.get_current_ctx(sid, &j); return py::make_tuple(st, j); })
        .def("set_ctx", &Client::set_ctx, nogil())
        .def("pull_context", &Client::pull_context, nogil())
        .def("notify_ctx_update", [](Client& c, int32_t sid) {
            auto e = c.context().get(sid);
            if (!e) return Status::InvalidID("unknown storage");
            return c.require_update_ctx_nolock(sid, Client::all_nodes(*e));
        }, nogil())
        .def("handle_timeout", &Client::handle_timeout, nogil())
        .def("handle_out_of_memory", &Client::handle_out_of_memory, nogil());

    py::class_<PullGroup, std::shared_ptr<PullGroup>>(m, "PullGroup")
        .def(py::init<>())
        .def("merged_sends", [](PullGroup& g) { return g.merged_sends.load(); })
        .def("merged_requests", [](PullGroup& g) { return g.merged_requests.load(); });
    py::class_<PullHandler>(m, "PullHandler")
        .def(py::init(&make_handler<PullHandler>), py::keep_alive<1, 2>())
        .def("join_group", &PullHandler::join_group)
        .def("dim", &PullHandler::dim)
        .def("metrics", [](PullHandler& h) { return metrics_dict(h); })
        .def("pull", [](PullHandler& h, KeyArray keys, int timeout_ms, bool auto_retry) {
            F32Array out({(py::ssize_t)keys.size(), (py::ssize_t)h.dim()});
            Status st;
            {
                py::gil_scoped_release g;
                st = h.pull(keys.data(), (size_t)keys.size(), out.mutable_data(), timeout_ms, auto_retry);
                if (!st.ok()) std::fill_n(out.mutable_data(), (size_t)out.size(), 0.f);   // never hand out memory that nobody wrote
            }
            return py::make_tuple(st, out);
        }, py::arg("keys"), py::arg("timeout_ms") = -1, py::arg("auto_retry") = true)
        .def("pull_dense", [](PullHandler& h, int64_t id, size_t numel, int timeout_ms) {
            F32Array out((py::ssize_t)numel);
            Status st;
            {
                py::gil_scoped_release g;
                st = h.pull_dense(id, numel, out.mutable_data(), timeout_ms);
                if (!st.ok()) std::fill_n(out.mutable_data(), numel, 0.f);   // never hand out memory that nobody wrote
            }
            return py::make_tuple(st, out);
        }, py::arg("id"), py::arg("numel"), py::arg("timeout_ms") = -1);

    py::class_<PushGroup, std::shared_ptr<PushGroup>>(m, "PushGroup")
        .def(py::init<>())
        .def("merged_sends", [](PushGroup& g) { return g.merged_sends.load(); })
        .def("merged_requests", [](PushGroup& g) { return g.merged_requests.load(); });
    py::class_<PushHandler>(m, "PushHandler")
        .def(py::init(&make_handler<PushHandler>), py::keep_alive<1, 2>())
        .def("join_group", &PushHandler::join_group)
        .def("metrics", [](PushHandler& h) { return metrics_dict(h); })
        .def("async_push", [](PushHandler& h, KeyArray keys, F32Array grads, int timeout_ms) {
            if ((size_t)grads.size() != (size_t)keys.size() * h.dim()) throw std::invalid_argument("grads must hold one row of dim floats per key");
            py::gil_scoped_release g;
            return h.async_push(keys.data(), grads.data(), (size_t)keys.size(), timeout_ms);
        }, py::arg("keys"), py::arg("grads"), py::arg("timeout_ms") = -1)
        .def("sync_push", [](PushHandler& h, KeyArray keys, F32Array grads, int timeout_ms) {
            if ((size_t)grads.size() != (size_t)keys.size() * h.dim()) throw std::invalid_argument("grads must hold one row of dim floats per key");
            py::gil_scoped_release g;
            return h.sync_push(keys.data(), grads.data(), (size_t)keys.size(), timeout_ms);
        }, py::arg("keys"), py::arg("grads"), py::arg("timeout_ms") = -1)
        .def("store", &PushHandler::store, py::arg("timeout_ms") = -1, nogil())
        .def("push_dense", [](PushHandler& h, int64_t id, F32Array grad, bool sync, int timeout_ms) {
            py::gil_scoped_release g;
            return h.push_dense(id, grad.data(), (size_t)grad.size(), sync, timeout_ms);
        }, py::arg("id"), py::arg("grad"), py::arg("sync") = false, py::arg("timeout_ms") = -1);

    py::class_<ForEachHandler>(m, "ForEachHandler")
        .def(py::init(&make_handler<ForEachHandler>), py::keep_alive<1, 2>())
        .def("for_each", [](ForEachHandler& h, const std::string& carried, int timeout_ms) {
            ForEachResult r;
            Status st;
            {
                py::gil_scoped_release g;
                st = h.for_each(carried, &r, timeout_ms);
            }
            py::dict d;
            d["count"] = r.count; d["sum"] = r.sum; d["sum_sq"] = r.sum_sq; d["max_abs"] = r.max_abs;
            return py::make_tuple(st, d);
        }, py::arg("carried") = "{}", py::arg("timeout_ms") = -1)
        .def("for_each_raw", [](ForEachHandler& h, const std::string& carried, int timeout_ms) {
            // the operator's own result bytes (a plug-in reducer defines the layout)
            std::string raw;
            Status st;
            {
                py::gil_scoped_release rel;
                st = h.for_each_raw(carried, &raw, timeout_ms);
            }
            return py::make_tuple(st, py::bytes(raw));
        }, py::arg("carried") = "{}", py::arg("timeout_ms") = -1);

    py::class_<EraseIfHandler>(m, "EraseIfHandler")
        .def(py::init(&make_handler<EraseIfHandler>), py::keep_alive<1, 2>())
        .def("erase_if", [](EraseIfHandler& h, const std::string& carried, int timeout_ms) {
            uint64_t n = 0;
            py::gil_scoped_release g;
            Status st = h.erase_if(carried, &n, timeout_ms);
            return std::make_pair(st, n);
        }, py::arg("carried"), py::arg("timeout_ms") = -1);

    py::class_<DumpHandler>(m, "DumpHandler")
        .def(py::init(&make_handler<DumpHandler>), py::keep_alive<1, 2>())
        .def("dump", [](DumpHandler& h, const std::string& uri, int file_number, int timeout_ms) {
            DumpArgs a;
            a.uri = uri;
            a.file_number = file_number;
            uint64_t n = 0;
            py::gil_scoped_release g;
            Status st = h.dump(a, &n, timeout_ms);
            return std::make_pair(st, n);
        }, py::arg("uri"), py::arg("file_number") = 1, py::arg("timeout_ms") = -1);

    py::class_<LoadHandler>(m, "LoadHandler")
        .def(py::init(&make_handler<LoadHandler>), py::keep_alive<1, 2>())
        .def("load", [](LoadHandler& h, const std::string& uri, int conc, int timeout_ms) {
            uint64_t n = 0;
            py::gil_scoped_release g;
            Status st = h.load(uri, &n, conc, timeout_ms);
            return std::make_pair(st, n);
        }, py::arg("uri"), py::arg("server_concurrency") = 4, py::arg("timeout_ms") = -1)
        .def("restore", [](LoadHandler& h, const std::string& uri, bool drop, int timeout_ms) {
            uint64_t n = 0;
            py::gil_scoped_release g;
            Status st = h.restore(uri, &n, drop, timeout_ms);
            return std::make_pair(st, n);
        }, py::arg("uri"), py::arg("drop") = false, py::arg("timeout_ms") = -1);

    py::class_<UpdateContextHandler>(m, "UpdateContextHandler")
        .def(py::init(&make_handler<UpdateContextHandler>), py::keep_alive<1, 2>())
        .def("update_context", &UpdateContextHandler::update_context, py::arg("nodes_json"), py::arg("timeout_ms") = 60000, nogil())
        .def("purge", &UpdateContextHandler::purge, py::arg("timeout_ms") = 60000, nogil());

    py::class_<SyncHandler>(m, "SyncHandler")
        .def(py::init(&make_handler<SyncHandler>), py::keep_alive<1, 2>())
        .def("metrics", [](SyncHandler& h) { return metrics_dict(h); })
        .def("sync_pred", [](SyncHandler& h, Server& trainer, int32_t trainer_sid, int max_attempts, double backoff_scale) {
            uint64_t n = 0;
            Status st = h.sync_pred(trainer, trainer_sid, &n, max_attempts, backoff_scale);
            return std::make_tuple(st, n);
        }, py::arg("trainer"), py::arg("trainer_sid"), py::arg("max_attempts") = 5, py::arg("backoff_scale") = 1.0, nogil())
        .def("block_size", &SyncHandler::block_size)
        .def("sync_block", [](SyncHandler& h, KeyArray keys, F32Array rows, int timeout_ms) {
            const uint32_t stride = (uint32_t)(rows.size() / std::max<py::ssize_t>(1, keys.size()));
            if ((size_t)stride * (size_t)keys.size() != (size_t)rows.size()) throw std::invalid_argument("rows must hold the same number of floats per key");
            py::gil_scoped_release g;
            return h.sync_block(keys.data(), rows.data(), (size_t)keys.size(), stride, timeout_ms);
        }, py::arg("keys"), py::arg("rows"), py::arg("timeout_ms") = 30000);

    py::class_<UDFHandler>(m, "UDFHandler")
        .def(py::init(&make_handler<UDFHandler>), py::keep_alive<1, 2>())
        .def("call", [](UDFHandler& h, py::bytes param, int timeout_ms, bool retry) {
            std::vector<std::pair<int, std::string>> rs;
            std::string p = param;
            Status st;
            {
                py::gil_scoped_release g;
                st = h.call(p, &rs, timeout_ms, retry);
            }
            py::list out;
            for (auto& r : rs) out.append(py::make_tuple(r.first, py::bytes(r.second)));
            return py::make_tuple(st, out);
        }, py::arg("param"), py::arg("timeout_ms") = -1, py::arg("retry") = true)
        .def("generate_request", [](UDFHandler& h, py::bytes param) {
            auto req = std::make_shared<UDFHandler::Request>();
            Status st = h.generate_request(std::string(param), req.get());
            return py::make_tuple(st, req);
        })
        .def("send_request", [](UDFHandler& h, std::shared_ptr<UDFHandler::Request> req, int timeout_ms) {
            std::vector<std::pair<int, std::string>> rs;
            Status st;
            {
                py::gil_scoped_release g;
                st = h.send_request(*req, &rs, timeout_ms);
            }
            py::list out;
            for (auto& r : rs) out.append(py::make_tuple(r.first, py::bytes(r.second)));
            return py::make_tuple(st, out);
        }, py::arg("request"), py::arg("timeout_ms") = -1);
    py::class_<UDFHandler::Request, std::shared_ptr<UDFHandler::Request>>(m, "UDFRequest")
        .def_readonly("ctx_version", &UDFHandler::Request::ctx_version)
        .def("nodes", [](UDFHandler::Request& r) { std::vector<int> n; for (auto& kv : r.bodies) n.push_back(kv.first); return n; });

    // ---- controller / model ------------------------------------------------------------------------
    py::class_<OpSpec>(m, "OpSpec")
        .def(py::init([](std::string key, std::string lib, std::string op, std::string cfg) { return OpSpec{key, lib, op, cfg}; }),
             py::arg("key"), py::arg("lib"), py::arg("op"), py::arg("config") = "{}");
    py::class_<Controller>(m, "Controller")
        .def(py::init<const std::string&>(), py::arg("master"))
        .def("client", &Controller::client, py::return_value_policy::reference_internal)
        .def("load_nodes", [](Controller& c) { std::vector<int> n; Status st = c.load_nodes(&n); return std::make_tuple(st, n); }, nogil())
        .def("create_table", [](Controller& c, const std::string& name, const std::string& lib, const std::string& sop,
                                const std::string& cfg, int shards, int replicas, const std::vector<OpSpec>& ops,
                                const std::string& uri) {
            int32_t sid = -1;
            Status st = c.create_table(name, lib, sop, cfg, shards, replicas, ops, uri, &sid);
            return std::make_tuple(st, sid);
        }, py::arg("table_name"), py::arg("lib"), py::arg("storage_op"), py::arg("op_config"), py::arg("shard_num"),
           py::arg("replica_num"), py::arg("ops"), py::arg("table_uri") = "", nogil())
        .def("delete_table", &Controller::delete_table, nogil())
        .def("balance_table", &Controller::balance_table, nogil())
        .def("purge_table", &Controller::purge_table, nogil())
        .def("dump_table", [](Controller& c, int32_t sid, const std::string& uri, int files) {
            uint64_t n = 0;
            Status st = c.dump_table(sid, uri, files, &n);
            return std::make_tuple(st, n);
        }, py::arg("sid"), py::arg("uri"), py::arg("file_number") = 1, nogil())
        .def("load_table", [](Controller& c, int32_t sid, const std::string& uri) {
            uint64_t n = 0;
            Status st = c.load_table(sid, uri, &n);
            return std::make_tuple(st, n);
        }, nogil())
        .def("table_stats", [](Controller& c, int32_t sid, int section) {
            Json out;
            Status st = c.table_stats(sid, section, &out);
            return std::make_tuple(st, out.dump());
        }, py::arg("sid"), py::arg("section") = 0, nogil())
        .def("erase_from_table", [](Controller& c, int32_t sid, const std::string& carried) {
            uint64_t n = 0;
            Status st = c.erase_from_table(sid, carried, &n);
            return std::make_tuple(st, n);
        }, nogil())
        .def("update_table_shard", &Controller::update_table_shard, nogil())
        .def("update_table_replica", &Controller::update_table_replica, nogil())
        .def("update_table", &Controller::update_table, nogil())
        .def("expand_storage_nodes", &Controller::expand_storage_nodes, nogil())
        .def("expand_nodes", &Controller::expand_nodes, nogil())
        .def("clean_unused_storage", [](Controller& c) { int n = 0; Status st = c.clean_unused_storage(&n); return std::make_tuple(st, n); }, nogil())
        .def("shutdown_node", &Controller::shutdown_node, nogil())
        .def("show_node", [](Controller& c, int node) { Json j; Status st = c.show_node(node, &j); return std::make_tuple(st, j.dump()); }, nogil())
        .def("show_nodes", [](Controller& c) { Json j; Status st = c.show_nodes(&j); return std::make_tuple(st, j.dump()); }, nogil())
        .def("gen_table_json", [](Controller& c, int32_t sid) { Json j; Status st = c.gen_table_json(sid, &j); return std::make_tuple(st, j.dump()); }, nogil());

    m.def("model_round_trip", [](const std::string& json) {
        Json j;
        if (!Json::parse(json, &j)) return std::string();
        ModelObject mo = ModelObject::from_json(j);
        std::vector<const TableObject*> ts;
        mo.all_tables(&ts);
        std::vector<const OperatorObject*> os;
        mo.all_operators(&os);
        Json out = mo.to_json();
        out["n_tables"] = (int)ts.size();
        out["n_operators"] = (int)os.size();
        return out.dump();
    });
    m.def("set_model", [](MasterClient& mc, const std::string& json) {
        Json j;
        if (!Json::parse(json, &j)) return Status::InvalidConfig("model JSON does not parse");
        return set_model(mc, ModelObject::from_json(j));
    });
    m.def("get_model", [](MasterClient& mc, const std::string& name) {
        ModelObject mo;
        Status st = get_model(mc, name, &mo);
        return py::make_tuple(st, st.ok() ? mo.to_json().dump() : std::string());
    });

    // ---- native PS -----------------------------------------------------------------------------------
    py::class_<NativePS>(m, "NativePS")
        .def(py::init<>())
        .def("create_storage", [](NativePS& p, const std::string& lib, const std::string& op, const std::string& cfg, int shards) {
            int32_t sid = -1;
            Status st = p.create_storage(lib, op, cfg, shards, &sid);
            return py::make_tuple(st, sid);
        })
        .def("register_handler", [](NativePS& p, int32_t sid, const std::string& key, const std::string& lib, const std::string& op,
                                    const std::string& cfg) {
            int32_t hid = -1;
            Status st = p.register_handler(sid, key, lib, op, cfg, &hid);
            return py::make_tuple(st, hid);
        })
        .def("size", [](NativePS& p, int32_t sid) -> int64_t {
            auto e = p.entry(sid);
            return e && e->storage ? (int64_t)e->storage->size() : -1;
        });
    py::class_<NativePullHandler>(m, "NativePullHandler")
        .def(py::init<NativePS*, int32_t, int32_t>(), py::keep_alive<1, 2>())
        .def("dim", &NativePullHandler::dim)
        .def("pull", [](NativePullHandler& h, KeyArray keys, int dim) {
            // the handler writes rows of the table's width: a caller that names another one would get a buffer of
            // the wrong size written to (dim <= 0: use the table's)
            const uint32_t have = h.dim();
            if (dim <= 0) dim = (int)have;
            F32Array out({(py::ssize_t)keys.size(), (py::ssize_t)std::max(dim, 0)});
            Status st = have != 0 && (uint32_t)dim != have
                            ? Status::InvalidConfig("the table's rows are " + std::to_string(have) + " wide, not " + std::to_string(dim))
                            : h.pull(keys.data(), (size_t)keys.size(), out.mutable_data());
            return py::make_tuple(st, out);
        }, py::arg("keys"), py::arg("dim") = 0);
    py::class_<NativeLoadHandler>(m, "NativeLoadHandler")
        .def(py::init<NativePS*, int32_t, int32_t>(), py::keep_alive<1, 2>())
        .def("load", [](NativeLoadHandler& h, const std::string& uri, int threads) {
            uint64_t n = 0;
            py::gil_scoped_release g;
            Status st = h.load(uri, threads, &n);
            return std::make_pair(st, n);
        }, py::arg("uri"), py::arg("threads") = 4);
}
