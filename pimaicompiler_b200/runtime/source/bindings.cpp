// pybind11 module `NNCompiler` with class `PipelineManager(input_file, model_type="", gpu_num=1)` and method
// `inferenceModel(input_tensors)`: the module the reference builds from runtime/python/nn_runtime_py.cpp:18-25.
// Added for tests and tools: a profiling switch with the trace path, and the fall-back counter of the tensor-level ops.
#include <torch/extension.h>

#include "pipeline_manager.h"
#include "tensor_ops.h"

namespace py = pybind11;
using namespace NNRuntimeInterface;

PYBIND11_MODULE(NNCompiler, m) {
    py::class_<PipelineManager>(m, "PipelineManager")
        .def(py::init<const std::string&, std::string, int, bool>(), py::arg("input_file"), py::arg("model_type") = "",
             py::arg("gpu_num") = 1, py::arg("profiling") = false)
        .def("inferenceModel", &PipelineManager::inferenceModel, py::arg("input_tensors"),
             py::call_guard<py::gil_scoped_release>())
        .def("setProfilePath", &PipelineManager::setProfilePath);
    m.def("fallback_count", &nn_compiler::runtime::tensor_ops::fallbackCount);
    m.def("reset_fallback_count", &nn_compiler::runtime::tensor_ops::resetFallbackCount);
    m.def("grouped_launch_count", &nn_compiler::runtime::tensor_ops::groupedLaunchCount);
}
