// Python entry point of the host-side C++ runtime (`eredu_b200.lib._eredu_host`).
#include <pybind11/pybind11.h>

namespace py = pybind11;

namespace eredu {
void bind_gguf(py::module_& m);
void bind_safetensors(py::module_& m);
void bind_quant(py::module_& m);
void bind_runtime(py::module_& m);
void bind_residency(py::module_& m);
}  // namespace eredu

PYBIND11_MODULE(_eredu_host, m) {
  m.doc() = "eredu_b200 host runtime: GGUF / SafeTensors codecs, quantisers, topology, KV block manager, scheduler, consensus, residency ledger, cache byte pool";
  eredu::bind_gguf(m);
  eredu::bind_safetensors(m);
  eredu::bind_quant(m);
  eredu::bind_runtime(m);
  eredu::bind_residency(m);
}
