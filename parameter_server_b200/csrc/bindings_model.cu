// Bindings of the non-GEMM model kernels.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <tuple>
#include <vector>

#include "kernels/dedup.h"
#include "kernels/model_kernels.h"

namespace py = pybind11;
using namespace psb;

void bind_model_kernels(py::module_& m) {
    // emb_bf16: the embedding rows are bf16 (a pull with bf16 output) instead of fp32
    m.def("interaction_fwd", [](uintptr_t bottom, int64_t ldb, uintptr_t emb, int F, int D, uintptr_t out, int64_t ldo,
                                int B, uintptr_t s, bool emb_bf16) {
        return interaction_fwd((const void*)bottom, ldb, (const void*)emb, emb_bf16 ? 1 : 0, F, D, (void*)out, ldo, B, (void*)s);
    }, py::arg("bottom"), py::arg("ldb"), py::arg("emb"), py::arg("F"), py::arg("D"), py::arg("out"), py::arg("ldo"),
       py::arg("B"), py::arg("stream"), py::arg("emb_bf16") = false);
    m.def("interaction_bwd", [](uintptr_t dout, int64_t ldo, uintptr_t bottom, int64_t ldb, uintptr_t emb, int F, int D,
                                uintptr_t dbottom, int64_t lddb, uintptr_t demb, int B, bool relu_mask, uintptr_t s,
                                bool emb_bf16) {
        return interaction_bwd((const void*)dout, ldo, (const void*)bottom, ldb, (const void*)emb, emb_bf16 ? 1 : 0, F, D,
                               (void*)dbottom, lddb, (float*)demb, B, relu_mask ? 1 : 0, (void*)s);
    }, py::arg("dout"), py::arg("ldo"), py::arg("bottom"), py::arg("ldb"), py::arg("emb"), py::arg("F"), py::arg("D"),
       py::arg("dbottom"), py::arg("lddb"), py::arg("demb"), py::arg("B"), py::arg("relu_mask"), py::arg("stream"),
       py::arg("emb_bf16") = false);
    m.def("timestamp", [](uintptr_t slot, uintptr_t s) { return timestamp((unsigned long long*)slot, (void*)s); });
    m.def("bce_head", [](uintptr_t h, int64_t ldh, uintptr_t w, uintptr_t bias, uintptr_t y, int B, int K, float inv_batch,
                         uintptr_t loss_sum, uintptr_t logits, uintptr_t dz_prev, int64_t lddz, uintptr_t dw, uintptr_t db,
                         uintptr_t s) {
        return bce_head((const void*)h, ldh, (const void*)w, (const void*)bias, (const float*)y, B, K, inv_batch,
                        (float*)loss_sum, (float*)logits, (void*)dz_prev, lddz, (float*)dw, (float*)db, (void*)s);
    });
    m.def("bias_grad", [](uintptr_t dz, int64_t ld, int M, int N, uintptr_t db, uintptr_t s) {
        return bias_grad((const void*)dz, ld, M, N, (float*)db, (void*)s);
    });
    m.def("shard_of_keys", [](uintptr_t keys, unsigned long long n, int n_shards, uintptr_t shard_owner, uintptr_t out, uintptr_t s) {
        return shard_of_keys((const long long*)keys, n, n_shards, (const int*)shard_owner, (int*)out, (void*)s);
    });
    m.def("dedup_fill_scratch", [](uintptr_t scratch, unsigned long long slots, uintptr_t s) {
        return dedup_fill_scratch((void*)scratch, slots, (void*)s);
    });
    m.def("dedup_partition", [](uintptr_t keys, unsigned n, uintptr_t scratch, unsigned long long slots, uintptr_t pos,
                                uintptr_t shard_owner, int n_shards, int world, uintptr_t uniq_keys, uintptr_t uniq_owner,
                                uintptr_t inverse, uintptr_t counts, uintptr_t s) {
        return dedup_partition((const long long*)keys, n, (void*)scratch, slots, (unsigned*)pos, (const int*)shard_owner,
                               n_shards, world, (long long*)uniq_keys, (int*)uniq_owner, (int*)inverse, (unsigned*)counts,
                               (void*)s);
    });
    // items: (dz, ld, N, db); all tensors have M rows
    m.def("bias_grad_multi", [](const std::vector<std::tuple<uintptr_t, int64_t, int, uintptr_t>>& items, int M, uintptr_t s) {
        BiasGradSet set;
        if (items.size() > 8) return -2;
        set.count = (int)items.size();
        set.M = M;
        for (int i = 0; i < set.count; ++i) {
            set.dz[i] = (const void*)std::get<0>(items[i]);
            set.ld[i] = std::get<1>(items[i]);
            set.N[i] = std::get<2>(items[i]);
            set.db[i] = (float*)std::get<3>(items[i]);
        }
        return bias_grad_multi(set, (void*)s);
    });
    m.def("cast_pad", [](uintptr_t x, int B, int Kin, uintptr_t out, int64_t ldo, uintptr_t s) {
        return cast_pad((const float*)x, B, Kin, (void*)out, ldo, (void*)s);
    });
}
