// Dense-table and GEMM kernel bindings.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "kernels/gemm_tcgen05.h"
#include "kernels/model_kernels.h"
#include "comm/symmetric.h"
#include "operator/dense_engine.h"

namespace py = pybind11;
using namespace psb;

namespace {
template <class T>
T* ptr(uintptr_t p) { return reinterpret_cast<T*>(p); }
}  // namespace

void bind_dense(py::module_& m) {
    py::class_<SymmetricBuffer>(m, "SymmetricBuffer")
        .def(py::init<int, size_t>(), py::arg("device"), py::arg("bytes"))
        .def("ipc_handle", [](SymmetricBuffer& b) { return py::bytes(b.ipc_handle()); })
        .def("connect", [](SymmetricBuffer& b, const std::vector<py::bytes>& hs, int rank) {
            std::vector<std::string> v;
            for (auto& h : hs) v.push_back((std::string)h);
            return b.connect(v, rank);
        })
        .def("local", [](SymmetricBuffer& b) { return (uintptr_t)b.local(); })
        .def("peer", [](SymmetricBuffer& b, int r) { return (uintptr_t)b.peer(r); })
        .def("bytes", &SymmetricBuffer::bytes)
        .def("world", &SymmetricBuffer::world);

    py::class_<DenseEngine>(m, "DenseEngine")
        .def(py::init<int, int, int, size_t, bool, int, double>(), py::arg("device"), py::arg("world"), py::arg("rank"),
             py::arg("numel"), py::arg("grad_bf16"), py::arg("opt_type"), py::arg("wait_limit_s") = 10.0)
        .def("ipc_handle", [](DenseEngine& e) { return py::bytes(e.ipc_handle()); })
        .def("connect",
             [](DenseEngine& e, const std::vector<py::bytes>& hs) {
                 std::vector<std::string> v;
                 for (auto& h : hs) v.push_back((std::string)h);
                 return e.connect(v);
             })
        .def("connect_local", &DenseEngine::connect_local)
        .def("numel", &DenseEngine::numel)
        .def("shard_lo", &DenseEngine::shard_lo)
        .def("shard_len", &DenseEngine::shard_len)
        .def("params_ptr", [](DenseEngine& e) { return (uintptr_t)e.params_ptr(); })
        .def("grads_ptr", [](DenseEngine& e) { return (uintptr_t)e.grads_ptr(); })
        .def("peer_params_ptr", [](DenseEngine& e, int r) { return (uintptr_t)e.peer_params_ptr(r); })
        .def("master_ptr", [](DenseEngine& e) { return (uintptr_t)e.master_ptr(); })
        .def("slot_ptr", [](DenseEngine& e, int s) { return (uintptr_t)e.slot_ptr(s); })
        .def("grad_bf16", &DenseEngine::grad_bf16)
        .def("load_full", [](DenseEngine& e, uintptr_t full, uintptr_t s) { return e.load_full(ptr<const float>(full), (void*)s); })
        .def("step", [](DenseEngine& e, const OptConfig& o, float scale, uintptr_t s) { return e.step(o, scale, (void*)s); })
        .def("check", [](DenseEngine& e, uintptr_t s) { return e.check((void*)s); })
        .def("reset", [](DenseEngine& e, uintptr_t s) { return e.reset((void*)s); })
        .def("kernel_launches", &DenseEngine::kernel_launches)
        .def("set_scatter_peers", &DenseEngine::set_scatter_peers)
        .def("set_sm_budget", &DenseEngine::set_sm_budget);

    m.def("gemm_bf16",
          [](uintptr_t a, int64_t lda, bool a_mn, uintptr_t b, int64_t ldb, bool b_mn, int M, int N, int K,
             uintptr_t out_bf16, uintptr_t out_f32, int64_t ldd, uintptr_t bias, bool relu, uintptr_t mask,
             int64_t ldmask, bool accumulate, uintptr_t bias_bf16, int split_k, uintptr_t err_flag, double wait_limit_s, uintptr_t stream,
             const std::vector<uintptr_t>& gather_peers, int gather_rank, int rows_per_rank, uintptr_t gather_ready,
             unsigned gather_epoch, int gather_ctas) {
              GemmOperand A{ptr<const void>(a), lda, a_mn}, B{ptr<const void>(b), ldb, b_mn};
              GemmEpilogue ep;
              ep.out_bf16 = ptr<__nv_bfloat16>(out_bf16);
              ep.out_f32 = ptr<float>(out_f32);
              ep.ldd = ldd;
              ep.bias = ptr<const float>(bias);
              ep.relu = relu ? 1 : 0;
              ep.mask = ptr<const __nv_bfloat16>(mask);
              ep.ldmask = ldmask;
              ep.accumulate = accumulate ? 1 : 0;
              ep.bias_bf16 = ptr<const __nv_bfloat16>(bias_bf16);
              ep.split_k = split_k;
              GemmGather ag;
              if (!gather_peers.empty()) {
                  ag.enabled = 1;
                  ag.world = (int)gather_peers.size();
                  ag.rank = gather_rank;
                  for (size_t r = 0; r < gather_peers.size() && r < 8; ++r) ag.peer_b[r] = ptr<const __nv_bfloat16>(gather_peers[r]);
                  ag.local_b = ptr<__nv_bfloat16>(b);
                  ag.rows_per_rank = rows_per_rank;
                  ag.ready = ptr<unsigned>(gather_ready);
                  ag.epoch = gather_epoch;
                  ag.gather_ctas = gather_ctas;
              }
              return gemm_bf16(A, B, ep, M, N, K, ptr<unsigned>(err_flag), wait_limit_s, (void*)stream, &ag);
          },
          py::arg("a"), py::arg("lda"), py::arg("a_mn"), py::arg("b"), py::arg("ldb"), py::arg("b_mn"), py::arg("M"),
          py::arg("N"), py::arg("K"), py::arg("out_bf16") = 0, py::arg("out_f32") = 0, py::arg("ldd") = 0,
          py::arg("bias") = 0, py::arg("relu") = false, py::arg("mask") = 0, py::arg("ldmask") = 0,
          py::arg("accumulate") = false, py::arg("bias_bf16") = 0, py::arg("split_k") = 1, py::arg("err_flag") = 0, py::arg("wait_limit_s") = 2.0, py::arg("stream") = 0,
          py::arg("gather_peers") = std::vector<uintptr_t>(), py::arg("gather_rank") = 0, py::arg("rows_per_rank") = 0,
          py::arg("gather_ready") = 0, py::arg("gather_epoch") = 0, py::arg("gather_ctas") = 8);

    // problems: (a, lda, b, ldb, M, N, K, out_bf16, out_f32, ldd, accumulate, split_k)
    m.def("gemm_bf16_grouped",
          [](const std::vector<std::tuple<uintptr_t, int64_t, uintptr_t, int64_t, int, int, int, uintptr_t, uintptr_t, int64_t, bool, int>>& probs,
             bool a_mn, bool b_mn, uintptr_t err_flag, double wait_limit_s, uintptr_t stream) {
              const int n = (int)probs.size();
              if (n > 8) return -2;
              GemmOperand A[8], B[8];
              GemmEpilogue ep[8];
              int M[8], N[8], K[8];
              for (int i = 0; i < n; ++i) {
                  const auto& t = probs[i];
                  A[i] = GemmOperand{ptr<const void>(std::get<0>(t)), std::get<1>(t), a_mn};
                  B[i] = GemmOperand{ptr<const void>(std::get<2>(t)), std::get<3>(t), b_mn};
                  M[i] = std::get<4>(t);
                  N[i] = std::get<5>(t);
                  K[i] = std::get<6>(t);
                  ep[i].out_bf16 = ptr<__nv_bfloat16>(std::get<7>(t));
                  ep[i].out_f32 = ptr<float>(std::get<8>(t));
                  ep[i].ldd = std::get<9>(t);
                  ep[i].accumulate = std::get<10>(t) ? 1 : 0;
                  ep[i].split_k = std::get<11>(t);
              }
              return gemm_bf16_grouped(A, B, ep, M, N, K, n, ptr<unsigned>(err_flag), wait_limit_s, (void*)stream);
          },
          py::arg("problems"), py::arg("a_mn"), py::arg("b_mn"), py::arg("err_flag") = 0, py::arg("wait_limit_s") = 2.0,
          py::arg("stream") = 0);

    // layers: (a, lda, b, ldb, M, N, K, out_bf16, ldd, bias_bf16, relu, mask, ldmask); layer i + 1 must read layer i's output
    m.def("gemm_bf16_chain",
          [](const std::vector<std::tuple<uintptr_t, int64_t, uintptr_t, int64_t, int, int, int, uintptr_t, int64_t, uintptr_t, bool,
                                          uintptr_t, int64_t>>& layers,
             bool b_mn, uintptr_t chain_done, uintptr_t err_flag, double wait_limit_s, uintptr_t stream) {
              const int n = (int)layers.size();
              if (n > 8 || chain_done == 0) return -2;
              GemmOperand A[8], B[8];
              GemmEpilogue ep[8];
              int M[8], N[8], K[8];
              for (int i = 0; i < n; ++i) {
                  const auto& t = layers[i];
                  A[i] = GemmOperand{ptr<const void>(std::get<0>(t)), std::get<1>(t), false};
                  B[i] = GemmOperand{ptr<const void>(std::get<2>(t)), std::get<3>(t), b_mn};
                  M[i] = std::get<4>(t);
                  N[i] = std::get<5>(t);
                  K[i] = std::get<6>(t);
                  ep[i].out_bf16 = ptr<__nv_bfloat16>(std::get<7>(t));
                  ep[i].ldd = std::get<8>(t);
                  ep[i].bias_bf16 = ptr<const __nv_bfloat16>(std::get<9>(t));
                  ep[i].relu = std::get<10>(t) ? 1 : 0;
                  ep[i].mask = ptr<const __nv_bfloat16>(std::get<11>(t));
                  ep[i].ldmask = std::get<12>(t);
              }
              return gemm_bf16_grouped(A, B, ep, M, N, K, n, ptr<unsigned>(err_flag), wait_limit_s, (void*)stream,
                                       ptr<unsigned>(chain_done));
          },
          py::arg("layers"), py::arg("b_mn"), py::arg("chain_done"), py::arg("err_flag") = 0, py::arg("wait_limit_s") = 2.0,
          py::arg("stream") = 0);
    m.def("gemm_chain_scratch_words", &gemm_chain_scratch_words);
    m.def("gemm_set_trace", [](uintptr_t p) { gemm_set_trace((void*)p); });
    m.def("gemm_set_cta_limit", &gemm_set_cta_limit);
    m.def("gemm_set_pair", &gemm_set_pair);

    bind_model_kernels(m);
}
