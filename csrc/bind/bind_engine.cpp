#include <pybind11/pybind11.h>
namespace py = pybind11;
namespace kvx {
void bind_engine(py::module_& m) { (void)m; }
}  // namespace kvx
