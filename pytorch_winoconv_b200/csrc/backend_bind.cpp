// Module MakePytorchBackend: same names and argument lists as the reference's pybind/bind.cpp:11-24.
#include <torch/extension.h>

#include "backend_ops.h"

namespace py = pybind11;

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  py::class_<Foo>(m, "Foo")
      .def(py::init<>())
      .def("setKey", &Foo::setKey)
      .def("getKey", &Foo::getKey)
      .def("__repr__", [](const Foo &a) { return a.toString(); });
  m.def("AddGPU", &AddGPU);
  m.def("WinoSplit", &WinoSplit);
  m.def("WinoConcat", &WinoConcat);
  m.def("DWM", &DWM);
  m.def("set_dwm_output_block", &set_dwm_output_block);
  m.def("get_dwm_output_block", &get_dwm_output_block);
}
