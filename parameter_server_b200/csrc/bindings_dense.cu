// Dense-table and GEMM kernel bindings.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>
namespace py = pybind11;
void bind_dense(py::module_& m) { (void)m; }
