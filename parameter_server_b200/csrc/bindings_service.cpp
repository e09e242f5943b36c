// Control-plane bindings (master, context, RPC server / client).
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>
namespace py = pybind11;
void bind_service(py::module_& m) { (void)m; }
