// Host runtime bindings (CPU storage, oracle, codec). numpy arrays cross the boundary here.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "common/archive.h"
#include "common/message.h"
#include "operator/cpu_ops.h"
#include "storage/host_table.h"

namespace py = pybind11;
using namespace psb;

void bind_service(py::module_& m);  // control plane (bindings_service.cpp)

using KeyArray = py::array_t<int64_t, py::array::c_style | py::array::forcecast>;
using F32Array = py::array_t<float, py::array::c_style | py::array::forcecast>;

void bind_host(py::module_& m) {
    py::class_<HostTableConfig>(m, "HostTableConfig")
        .def(py::init<>())
        .def_readwrite("dim", &HostTableConfig::dim)
        .def_readwrite("opt_type", &HostTableConfig::opt_type)
        .def_readwrite("sync_delta", &HostTableConfig::sync_delta)
        .def_readwrite("n_shards", &HostTableConfig::n_shards)
        .def_readwrite("init_seed", &HostTableConfig::init_seed)
        .def_readwrite("init_range", &HostTableConfig::init_range)
        .def_readwrite("slot_init0", &HostTableConfig::slot_init0)
        .def_readwrite("slot_init1", &HostTableConfig::slot_init1)
        .def_readwrite("expected_max_items", &HostTableConfig::expected_max_items)
        .def_readwrite("index_grow_ratio", &HostTableConfig::index_grow_ratio)
        .def_readwrite("index_shrink_ratio", &HostTableConfig::index_shrink_ratio)
        .def_readwrite("soft_limit_bytes", &HostTableConfig::soft_limit_bytes)
        .def_readwrite("hard_limit_bytes", &HostTableConfig::hard_limit_bytes);

    // shard (or, with `owner`, the owning rank) of every key of an int64 array: the vector form of sparse_shard_of
    m.def("sparse_shards_of", [](KeyArray keys, int n_shards, std::vector<int> owner) {
        if (n_shards < 1 || (!owner.empty() && (int)owner.size() != n_shards)) throw std::invalid_argument("n_shards / owner map");
        py::array_t<int64_t> out((py::ssize_t)keys.size());
        const int64_t* k = keys.data();
        int64_t* o = out.mutable_data();
        for (py::ssize_t i = 0; i < keys.size(); ++i) {
            const int s = sparse_shard_of(k[i], n_shards);
            o[i] = owner.empty() ? s : owner[s];
        }
        return out;
    }, py::arg("keys"), py::arg("n_shards"), py::arg("owner") = std::vector<int>());

    py::class_<HostTable>(m, "HostTable")
        .def(py::init<const HostTableConfig&>())
        .def("dim", &HostTable::dim)
        .def("stride", &HostTable::stride)
        .def("n_shards", &HostTable::n_shards)
        .def("create_shard", &HostTable::create_shard)
        .def("erase_shard", &HostTable::erase_shard)
        .def("has_shard", &HostTable::has_shard)
        .def("shard_list", &HostTable::shard_list)
        .def("shard_of", &HostTable::shard_of)
        .def("shard_size", &HostTable::shard_size)
        .def("size", &HostTable::size)
        .def("memory_usage", &HostTable::memory_usage)
        .def("healthy", &HostTable::healthy)
        .def("set_healthy", &HostTable::set_healthy)
        .def("check_healthy", &HostTable::check_healthy)
        .def("inject_insert_failures", &HostTable::inject_insert_failures)
        .def("overflow_size", &HostTable::overflow_size)
        .def("drain_overflow", [](HostTable& t) { return t.drain_overflow(); })
        .def("set_limits", &HostTable::set_limits)
        .def("enable_dirty_tracking", &HostTable::enable_dirty_tracking)
        .def("clear_dirty", &HostTable::clear_dirty)
        .def("clear", &HostTable::clear)
        .def("store", [](HostTable& t, const OptConfig& o) {
            py::gil_scoped_release nogil;
            return t.store(o);
        })
        .def("pull",
             [](HostTable& t, KeyArray keys, size_t bag_size, bool mean, bool insert) {
                 const size_t n = (size_t)keys.size();
                 if (bag_size == 0 || n % bag_size) throw std::invalid_argument("n must be a multiple of bag_size");
                 F32Array out({(py::ssize_t)(n / bag_size), (py::ssize_t)t.dim()});
                 Status st;
                 {
                     py::gil_scoped_release nogil;
                     st = cpu_pull(t, keys.data(), n, bag_size, mean, out.mutable_data(), insert);
                 }
                 return py::make_tuple(st, out);
             },
             py::arg("keys"), py::arg("bag_size") = 1, py::arg("mean") = false, py::arg("insert") = true)
        .def("push",
             [](HostTable& t, KeyArray keys, F32Array grads, const OptConfig& o, size_t bag_size, bool mean, bool sync) {
                 const size_t n = (size_t)keys.size();
                 if (bag_size == 0 || n % bag_size) throw std::invalid_argument("n must be a multiple of bag_size");
                 if ((size_t)grads.size() != n / bag_size * t.dim()) throw std::invalid_argument("grads shape");
                 py::gil_scoped_release nogil;
                 return cpu_push(t, keys.data(), grads.data(), n, bag_size, mean, o, sync);
             },
             py::arg("keys"), py::arg("grads"), py::arg("opt"), py::arg("bag_size") = 1, py::arg("mean") = false,
             py::arg("sync") = false)
        .def("pull_shard",
             [](HostTable& t, int s, KeyArray keys, bool insert) {
                 F32Array out({(py::ssize_t)keys.size(), (py::ssize_t)t.dim()});
                 Status st = t.pull_shard(s, keys.data(), (size_t)keys.size(), out.mutable_data(), insert);
                 return py::make_tuple(st, out);
             })
        .def("push_shard",
             [](HostTable& t, int s, KeyArray keys, F32Array grads, const OptConfig& o, bool sync) {
                 if ((size_t)grads.size() != (size_t)keys.size() * t.dim()) throw std::invalid_argument("grads shape");
                 return t.push_shard(s, keys.data(), grads.data(), (size_t)keys.size(), o, sync);
             })
        .def("set_rows",
             [](HostTable& t, KeyArray keys, F32Array rows, bool emb_only) {
                 const size_t w = emb_only ? t.dim() : t.stride();
                 if ((size_t)rows.size() != (size_t)keys.size() * w) throw std::invalid_argument("rows shape");
                 return t.set_rows(keys.data(), rows.data(), (size_t)keys.size(), emb_only);
             })
        .def("get_rows",
             [](HostTable& t, KeyArray keys, bool emb_only) {
                 const size_t w = emb_only ? t.dim() : t.stride();
                 F32Array out({(py::ssize_t)keys.size(), (py::ssize_t)w});
                 py::array_t<int32_t> found((py::ssize_t)keys.size());
                 t.get_rows(keys.data(), (size_t)keys.size(), out.mutable_data(), found.mutable_data(), emb_only);
                 return py::make_tuple(out, found);
             })
        .def("erase_keys", [](HostTable& t, KeyArray keys) { return t.erase_keys(keys.data(), (size_t)keys.size()); })
        .def("layout_epoch", &HostTable::layout_epoch)
        .def("export_shard",
             [](HostTable& t, int s, size_t cursor, size_t window, bool dirty_only) {
                 std::vector<int64_t> keys;
                 std::vector<float> rows;
                 bool finished = true;
                 size_t next = t.export_shard(s, cursor, window, dirty_only, &keys, &rows, &finished);
                 py::array_t<int64_t> k((py::ssize_t)keys.size());
                 std::copy(keys.begin(), keys.end(), k.mutable_data());
                 F32Array r({(py::ssize_t)keys.size(), (py::ssize_t)t.stride()});
                 std::copy(rows.begin(), rows.end(), r.mutable_data());
                 return py::make_tuple(k, r, next, finished);
             });

    bind_service(m);
}
