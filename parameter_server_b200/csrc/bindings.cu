// pybind11 surface of the native library. Device buffers cross the boundary as integer addresses
// (torch.Tensor.data_ptr()) and streams as integer cudaStream_t handles, so the library has no
// link-time dependency on libtorch.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "common/hash.h"
#include "common/message.h"
#include "common/status.h"
#include "operator/sparse_engine.h"
#include "storage/cold_tier.h"
#include "storage/gpu_table.h"

namespace py = pybind11;
using namespace psb;

void bind_host(py::module_& m);    // host runtime (defined in bindings_host.cpp)
void bind_dense(py::module_& m);   // dense / GEMM kernels (defined in bindings_dense.cu)

namespace {
template <class T>
T* ptr(uintptr_t p) { return reinterpret_cast<T*>(p); }
void* stream_of(uintptr_t s) { return reinterpret_cast<void*>(s); }
}  // namespace

PYBIND11_MODULE(_C, m) {
    m.doc() = "parameter_server_b200 native core (sm_100a)";

    py::enum_<StatusCode>(m, "StatusCode")
        .value("OK", StatusCode::OK)
        .value("INVALID_CONFIG", StatusCode::INVALID_CONFIG)
        .value("INVALID_ID", StatusCode::INVALID_ID)
        .value("OUT_OF_MEMORY", StatusCode::OUT_OF_MEMORY)
        .value("TIMEOUT", StatusCode::TIMEOUT)
        .value("SERVER_TOO_NEW_CTX", StatusCode::SERVER_TOO_NEW_CTX)
        .value("SERVER_TOO_OLD_CTX", StatusCode::SERVER_TOO_OLD_CTX)
        .value("SERVER_TOO_NEW_CTX_U", StatusCode::SERVER_TOO_NEW_CTX_U)
        .value("SERVER_TOO_OLD_CTX_U", StatusCode::SERVER_TOO_OLD_CTX_U)
        .value("NO_REPLICA", StatusCode::NO_REPLICA)
        .value("ERROR", StatusCode::ERROR)
        .value("FATAL", StatusCode::FATAL)
        .value("EMPTY", StatusCode::EMPTY);

    py::class_<Status>(m, "Status")
        .def(py::init<>())
        .def(py::init<StatusCode, std::string>())
        .def("ok", &Status::ok)
        .def("code", &Status::code)
        .def("msg", &Status::msg)
        .def("__bool__", &Status::ok)
        .def("__repr__", [](const Status& s) { return "Status(" + s.to_string() + ")"; })
        .def("__str__", &Status::to_string);

    m.def("fmix64", [](uint64_t k) { return fmix64(k); });
    m.def("jump_consistent_hash", [](uint64_t k, int n) { return jump_consistent_hash(k, n); });
    m.def("sparse_shard_of", [](int64_t k, int n) { return sparse_shard_of(k, n); });
    m.def("dense_shard_of", [](int64_t id, int slice, int n) { return dense_shard_of(id, slice, n); });
    m.def("string_shard_of", [](const std::string& s, int n) { return string_shard_of(s.data(), s.size(), n); });
    m.def("init_uniform", [](int64_t key, uint32_t d, uint64_t seed, float range) {
        return init_uniform(key, d, seed, range);
    });
    m.attr("EMPTY_KEY") = (int64_t)kEmptyKey;
    m.attr("TOMBSTONE_KEY") = (int64_t)kTombstoneKey;
    m.attr("MAX_WORLD") = kMaxWorld;

    py::class_<OptConfig>(m, "OptConfig")
        .def(py::init<>())
        .def_readwrite("type", &OptConfig::type)
        .def_readwrite("lr", &OptConfig::lr)
        .def_readwrite("eps", &OptConfig::eps)
        .def_readwrite("l1", &OptConfig::l1)
        .def_readwrite("l2", &OptConfig::l2)
        .def_readwrite("alpha", &OptConfig::alpha)
        .def_readwrite("beta", &OptConfig::beta)
        .def_readwrite("beta1", &OptConfig::beta1)
        .def_readwrite("beta2", &OptConfig::beta2)
        .def_readwrite("weight_decay", &OptConfig::weight_decay)
        .def_readwrite("bias_corr1", &OptConfig::bias_corr1)
        .def_readwrite("bias_corr2", &OptConfig::bias_corr2)
        .def_readwrite("slot_init0", &OptConfig::slot_init0)
        .def_readwrite("slot_init1", &OptConfig::slot_init1)
        .def_readwrite("step_from_epoch", &OptConfig::step_from_epoch);
    m.attr("OPT_SGD") = (int)OPT_SGD;
    m.attr("OPT_ADAGRAD") = (int)OPT_ADAGRAD;
    m.attr("OPT_FTRL") = (int)OPT_FTRL;
    m.attr("OPT_ADAM") = (int)OPT_ADAM;
    m.attr("OPT_SUM") = (int)OPT_SUM;
    m.attr("OPT_SET") = (int)OPT_SET;
    m.def("opt_num_slots", [](int t) { return opt_num_slots(t); });
    m.def("opt_update_scalar", [](const OptConfig& c, float w, float s0, float s1, float g) {
        opt_update(c, w, s0, s1, g);
        return py::make_tuple(w, s0, s1);
    });

    py::class_<GpuTableConfig>(m, "GpuTableConfig")
        .def(py::init<>())
        .def_readwrite("device", &GpuTableConfig::device)
        .def_readwrite("dim", &GpuTableConfig::dim)
        .def_readwrite("opt_type", &GpuTableConfig::opt_type)
        .def_readwrite("sync_delta", &GpuTableConfig::sync_delta)
        .def_readwrite("index_capacity", &GpuTableConfig::index_capacity)
        .def_readwrite("slab_shift", &GpuTableConfig::slab_shift)
        .def_readwrite("init_seed", &GpuTableConfig::init_seed)
        .def_readwrite("init_range", &GpuTableConfig::init_range)
        .def_readwrite("slot_init0", &GpuTableConfig::slot_init0)
        .def_readwrite("slot_init1", &GpuTableConfig::slot_init1)
        .def_readwrite("soft_limit_bytes", &GpuTableConfig::soft_limit_bytes)
        .def_readwrite("hard_limit_bytes", &GpuTableConfig::hard_limit_bytes)
        .def_readwrite("max_probe", &GpuTableConfig::max_probe)
        .def_readwrite("max_rows", &GpuTableConfig::max_rows);

    py::class_<GpuTable>(m, "GpuTable")
        .def(py::init<const GpuTableConfig&>())
        .def("dim", &GpuTable::dim)
        .def("stride", &GpuTable::stride)
        .def("n_opt_slots", &GpuTable::n_opt_slots)
        .def("size", &GpuTable::size)
        .def("rows_used", &GpuTable::rows_used)
        .def("memory_usage", &GpuTable::memory_usage)
        .def("healthy", &GpuTable::healthy)
        .def("set_healthy", &GpuTable::set_healthy)
        .def("check_healthy", &GpuTable::check_healthy)
        .def("set_limits", &GpuTable::set_limits)
        .def("index_capacity", &GpuTable::index_capacity)
        .def("tombstones", &GpuTable::tombstones)
        .def("reserve_rows", &GpuTable::reserve_rows)
        .def("reserve_exact", &GpuTable::reserve_exact)
        .def("maybe_grow", &GpuTable::maybe_grow)
        .def("set_auto_grow", &GpuTable::set_auto_grow)
        .def("grow_count", &GpuTable::grow_count)
        .def("enable_dirty_tracking", &GpuTable::enable_dirty_tracking)
        .def("clear_dirty", [](GpuTable& t, uintptr_t s) { return t.clear_dirty(stream_of(s)); })
        .def("export_window",
             [](GpuTable& t, uint64_t cursor, uint64_t window, int mode, int shard, int rank, int n_shards,
                uintptr_t shard_owner, uintptr_t out_keys, uintptr_t out_rows, uintptr_t s) {
                 ShardFilter f;
                 f.mode = mode; f.shard = shard; f.rank = rank; f.n_shards = n_shards;
                 f.shard_owner = ptr<const int>(shard_owner);
                 uint64_t n = 0, next = 0;
                 Status st = t.export_window(cursor, window, f, ptr<long long>(out_keys), ptr<float>(out_rows), &n,
                                             &next, stream_of(s));
                 return py::make_tuple(st, n, next);
             })
        .def("set_rows",
             [](GpuTable& t, uintptr_t keys, uintptr_t rows, uint64_t n, bool emb_only, uintptr_t s) {
                 return t.set_rows(ptr<const long long>(keys), ptr<const float>(rows), n, emb_only, stream_of(s));
             })
        .def("get_rows",
             [](GpuTable& t, uintptr_t keys, uint64_t n, uintptr_t out, uintptr_t found, bool emb_only, uintptr_t s) {
                 return t.get_rows(ptr<const long long>(keys), n, ptr<float>(out), ptr<int>(found), emb_only,
                                   stream_of(s));
             })
        .def("erase_keys",
             [](GpuTable& t, uintptr_t keys, uint64_t n, uintptr_t s) {
                 uint64_t c = 0;
                 Status st = t.erase_keys(ptr<const long long>(keys), n, &c, stream_of(s));
                 return py::make_tuple(st, c);
             })
        .def("erase_filter",
             [](GpuTable& t, int mode, int shard, int rank, int n_shards, uintptr_t shard_owner, uintptr_t s) {
                 ShardFilter f;
                 f.mode = mode; f.shard = shard; f.rank = rank; f.n_shards = n_shards;
                 f.shard_owner = ptr<const int>(shard_owner);
                 uint64_t c = 0;
                 Status st = t.erase_filter(f, &c, stream_of(s));
                 return py::make_tuple(st, c);
             })
        .def("shard_counts",
             [](GpuTable& t, int n_shards, uintptr_t s) {
                 std::vector<uint64_t> c;
                 Status st = t.shard_counts(n_shards, &c, stream_of(s));
                 return py::make_tuple(st, c);
             })
        .def("store_delta", [](GpuTable& t, const OptConfig& o, uintptr_t s) { return t.store_delta(o, stream_of(s)); })
        .def("clear", [](GpuTable& t, uintptr_t s) { return t.clear(stream_of(s)); })
        .def("rebuild_index", [](GpuTable& t, uint64_t cap, uintptr_t s) { return t.rebuild_index(cap, stream_of(s)); });

    py::class_<HostColdTier>(m, "HostColdTier")
        .def(py::init<GpuTable*, uint64_t, uint32_t>(), py::arg("table"), py::arg("capacity_rows"), py::arg("window") = 1u << 16,
             py::keep_alive<1, 2>())
        .def("spill_if", [](HostColdTier& c, uint32_t section, float thr) { uint64_t n = 0; Status st = c.spill_if(section, thr, &n); return py::make_tuple(st, n); })
        .def("spill_keys", [](HostColdTier& c, uintptr_t keys, uint64_t n) { uint64_t k = 0; Status st = c.spill_keys((const int64_t*)keys, n, &k); return py::make_tuple(st, k); })
        .def("fetch", [](HostColdTier& c, uintptr_t keys, uint64_t n) { uint64_t k = 0; Status st = c.fetch((const int64_t*)keys, n, &k); return py::make_tuple(st, k); })
        .def("stage_fetch_async", [](HostColdTier& c, uintptr_t keys, uint64_t n) { c.stage_fetch_async((const int64_t*)keys, n); })
        .def("commit_fetch", [](HostColdTier& c, uintptr_t stream) { uint64_t k = 0; Status st = c.commit_fetch(stream_of(stream), &k); return py::make_tuple(st, k); })
        .def("size", &HostColdTier::size)
        .def("capacity", &HostColdTier::capacity)
        .def("bytes", &HostColdTier::bytes)
        .def("save", &HostColdTier::save)
        .def("load", &HostColdTier::load);

    py::class_<SparseEngineConfig>(m, "SparseEngineConfig")
        .def(py::init<>())
        .def_readwrite("world", &SparseEngineConfig::world)
        .def_readwrite("rank", &SparseEngineConfig::rank)
        .def_readwrite("max_keys", &SparseEngineConfig::max_keys)
        .def_readwrite("pair_capacity", &SparseEngineConfig::pair_capacity)
        .def_readwrite("n_shards", &SparseEngineConfig::n_shards)
        .def_readwrite("wait_limit_s", &SparseEngineConfig::wait_limit_s)
        .def_readwrite("replicate", &SparseEngineConfig::replicate);

    m.attr("FUSED_INSERT") = (unsigned)FUSED_INSERT;
    m.attr("FUSED_COPY_ROWS") = (unsigned)FUSED_COPY_ROWS;
    m.attr("FUSED_PREPARE_PUSH") = (unsigned)FUSED_PREPARE_PUSH;
    m.attr("FUSED_MEAN") = (unsigned)FUSED_MEAN;
    m.attr("FUSED_SYNC_PUSH") = (unsigned)FUSED_SYNC_PUSH;
    m.attr("FUSED_OUT_BF16") = (unsigned)FUSED_OUT_BF16;

    py::class_<SparseEngine>(m, "SparseEngine")
        .def(py::init<GpuTable*, const SparseEngineConfig&>(), py::keep_alive<1, 2>())
        .def("ipc_handle", [](SparseEngine& e) { return py::bytes(e.ipc_handle()); })
        .def("connect",
             [](SparseEngine& e, const std::vector<py::bytes>& hs) {
                 std::vector<std::string> v;
                 for (auto& h : hs) v.push_back((std::string)h);
                 return e.connect(v);
             })
        .def("connect_local", &SparseEngine::connect_local)
        .def("set_shard_owner", &SparseEngine::set_shard_owner)
        .def("shard_owner", &SparseEngine::shard_owner)
        .def("pull",
             [](SparseEngine& e, uintptr_t keys, uint32_t n, uint32_t bag, uintptr_t out, unsigned flags, uintptr_t s) {
                 return e.pull(ptr<const long long>(keys), n, bag, ptr<void>(out), flags, stream_of(s));
             })
        .def("push",
             [](SparseEngine& e, uintptr_t grads, uint32_t n_rows, const OptConfig& o, unsigned flags, uintptr_t s) {
                 return e.push(ptr<const float>(grads), n_rows, o, flags, stream_of(s));
             })
        .def("check", [](SparseEngine& e, uintptr_t s) { return e.check(stream_of(s)); })
        .def("reset", [](SparseEngine& e, uintptr_t s) { return e.reset(stream_of(s)); })
        .def("last_unique", [](SparseEngine& e, uintptr_t s) { return e.last_unique(stream_of(s)); })
        .def("pair_capacity", &SparseEngine::pair_capacity)
        .def("scratch_bytes", &SparseEngine::scratch_bytes)
        .def("kernel_launches", &SparseEngine::kernel_launches)
        .def("set_wait_limit", &SparseEngine::set_wait_limit)
        .def("set_sm_budget", &SparseEngine::set_sm_budget)
        .def("set_deterministic", &SparseEngine::set_deterministic)
        .def("set_grad_wire_bf16", &SparseEngine::set_grad_wire_bf16)
        .def("set_mirror", &SparseEngine::set_mirror, py::keep_alive<1, 2>())
        .def("deterministic", &SparseEngine::deterministic)
        .def("pull_blocks", &SparseEngine::pull_blocks)
        .def("push_blocks", &SparseEngine::push_blocks)
        .def("set_profile", &SparseEngine::set_profile)
        .def("phase_stamps", [](SparseEngine& e, uintptr_t s) { return e.phase_stamps(stream_of(s)); })
        .def("cta_stamps", [](SparseEngine& e, int which, uintptr_t s) { return e.cta_stamps(which, stream_of(s)); });

    bind_host(m);
    bind_dense(m);
}
