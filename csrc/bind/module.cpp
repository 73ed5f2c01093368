// Entry point of the `kvtransfer_ops` extension module.  The module keeps the symbol names
// of the reference binding (kvtransfer/kvtransfer_pybind.cpp:415-522) for the engine API and
// adds the kernel-level `kvt_*` functions.
#include <pybind11/pybind11.h>

#include "core/crash_trace.h"

namespace py = pybind11;

namespace kvx {
void bind_kernels(py::module_& m);
void bind_engine(py::module_& m);
void bind_store(py::module_& m);
}  // namespace kvx

PYBIND11_MODULE(kvtransfer_ops, m) {
  m.doc() = "B200-native KV transfer engine: C++ runtime and sm_100a kernels";
  kvx::bind_kernels(m);
  kvx::bind_engine(m);
  kvx::bind_store(m);
  kvx::install_crash_trace();      // only with BLLM_KVTRANS_CRASH_TRACE=1
  m.def("install_crash_trace", [] { return kvx::install_crash_trace(true); },
        "Write the native frames of a crashing engine thread to stderr before the process dies.");
}
