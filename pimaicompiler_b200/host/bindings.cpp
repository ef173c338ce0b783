// pybind11 module `_pimb200_host`: lets tests and Python callers build a hot-path graph out of the minimal IR and
// run it through the C++ executor registry, the way the reference's pybind module exposes its runtime
// (runtime/python/nn_runtime_py.cpp:18-25).  The TorchScript importer that normally produces the graph is not part
// of this library; graphs are assembled node by node.
#include <torch/extension.h>

#include "stream_executor.h"

namespace py = pybind11;
using namespace nn_compiler;

namespace {

struct GraphBuilder {
    std::shared_ptr<ir::NNGraph> graph = std::make_shared<ir::NNGraph>();
    int64_t next_id = 0;
    int64_t fresh() { return next_id++; }

    int64_t addInput() {
        const int64_t id = fresh();
        graph->input_ids.push_back(id);
        return id;
    }
    void markOutput(int64_t id) { graph->output_ids.push_back(id); }
    int64_t presetBlob(at::Tensor t) {
        const int64_t id = fresh();
        graph->preset_blobs.emplace_back(id, std::move(t));
        return id;
    }
    template <typename L>
    int64_t add(std::shared_ptr<L> layer, std::vector<int64_t> in, int n_out = 1) {
        std::vector<int64_t> out;
        for (int i = 0; i < n_out; ++i) out.push_back(fresh());
        layer->setInSTensorID(std::move(in));
        layer->setOutSTensorID(out);
        graph->addLayer(layer);
        return out[0];
    }
    int64_t addList(std::vector<int64_t> ids) {
        return add(std::make_shared<ir::PrimListConstructLayer>("prim::ListConstruct"), std::move(ids));
    }
    std::shared_ptr<ir::AtenAddmmLayer> makeAddmm(const std::string& act) {
        auto l = std::make_shared<ir::AtenAddmmLayer>("aten::addmm");
        l->setActType(act);
        return l;
    }
    int64_t addAddmm(int64_t self, int64_t m1, int64_t m2, const std::string& act, double beta, double alpha) {
        auto l = makeAddmm(act);
        l->beta = beta;
        l->alpha = alpha;
        return add(l, {self, m1, m2});
    }
    int64_t addMatmul(int64_t a, int64_t b) { return add(std::make_shared<ir::AtenMatmulLayer>("aten::matmul"), {a, b}); }
    int64_t addLinear(int64_t x, at::Tensor W, c10::optional<at::Tensor> b) {
        auto l = std::make_shared<ir::AtenLinearLayer>("aten::linear");
        l->setWeights(std::move(W));
        if (b.has_value()) l->setBiases(*b);
        return add(l, {x});
    }
    int64_t addAdd(int64_t a, int64_t b, double alpha) {
        auto l = std::make_shared<ir::AtenAddLayer>("aten::add");
        l->alpha = alpha;
        return add(l, {a, b});
    }
    int64_t addBmm(int64_t a, int64_t b) { return add(std::make_shared<ir::AtenBmmLayer>("aten::bmm"), {a, b}); }
    int64_t addSoftmax(int64_t x, int64_t dim, bool log) {
        auto l = std::make_shared<ir::AtenSoftmaxLayer>(log ? "aten::log_softmax" : "aten::softmax", log);
        l->dim = dim;
        return add(l, {x});
    }
    int64_t addArgmax(int64_t x, int64_t dim, bool keepdim) {
        auto l = std::make_shared<ir::AtenArgmaxLayer>("aten::argmax");
        l->dim = dim;
        l->keepdim = keepdim ? 1 : 0;
        return add(l, {x});
    }
    int64_t addLayerNorm(int64_t x, std::vector<int64_t> shape, c10::optional<at::Tensor> w, c10::optional<at::Tensor> b,
                         double eps) {
        auto l = std::make_shared<ir::AtenLayerNormLayer>("aten::layer_norm");
        l->normalized_shape = std::move(shape);
        if (w.has_value()) l->weight = *w;
        if (b.has_value()) l->bias = *b;
        l->eps = eps;
        return add(l, {x});
    }
    int64_t addEmbedding(int64_t table, int64_t idx) {
        return add(std::make_shared<ir::AtenEmbeddingLayer>("aten::embedding"), {table, idx});
    }
    int64_t addTanh(int64_t x) { return add(std::make_shared<ir::AtenTanhLayer>("aten::tanh"), {x}); }
    int64_t addMaskedFill(int64_t x, int64_t mask, double value) {
        auto l = std::make_shared<ir::AtenMaskedFillLayer>("aten::masked_fill");
        l->value = value;
        return add(l, {x, mask});
    }
    int64_t addCat(int64_t list_id, int64_t dim, int64_t mem_layer_id) {
        auto l = std::make_shared<ir::AtenCatLayer>("aten::cat");
        l->setDim(dim);
        l->setMemLayerId(mem_layer_id);
        return add(l, {list_id});
    }
    int64_t addCopy(int64_t self, int64_t src) { return add(std::make_shared<ir::AtenCopyLayer>("aten::copy_"), {self, src}); }
    // returns the id of `output`; h_n and c_n are the next two ids
    int64_t addLstm(std::vector<int64_t> in, std::vector<at::Tensor> params, bool has_biases, int64_t num_layers,
                    bool bidirectional, bool batch_first, bool packed, std::vector<std::pair<int64_t, int64_t>> aliases) {
        std::shared_ptr<ir::AtenLSTM1Layer> l;
        if (packed) l = std::make_shared<ir::AtenLSTM2Layer>("aten::lstm2");
        else l = std::make_shared<ir::AtenLSTM1Layer>("aten::lstm1");
        l->setParamVector(std::move(params));
        l->setHasBiases(has_biases);
        l->setNumLayers(num_layers);
        l->setBidirectional(bidirectional);
        l->setBatchFirst(batch_first);
        for (size_t i = 0; i < aliases.size() && i < 3; ++i) {
            l->out_alias[i].blob_id = aliases[i].first;
            l->out_alias[i].elem_offset = aliases[i].second;
        }
        return add(l, std::move(in), 3);
    }
    // wraps addmm/matmul nodes already described as (kind, ids, act) into one MULTISTREAM node followed by their copies
    std::vector<int64_t> addMultiStream(std::vector<std::tuple<std::string, std::vector<int64_t>, std::string>> branches) {
        auto ms = std::make_shared<ir::MultiStreamLayer>("MultiStream");
        std::vector<std::shared_ptr<ir::NNLayer>> subs;
        std::vector<int64_t> outs;
        for (auto& br : branches) {
            std::shared_ptr<ir::NNLayer> l;
            if (std::get<0>(br) == "addmm") l = makeAddmm(std::get<2>(br));
            else l = std::make_shared<ir::AtenMatmulLayer>("aten::matmul");
            l->setInSTensorID(std::get<1>(br));
            const int64_t o = fresh();
            l->setOutSTensorID({o});
            outs.push_back(o);
            subs.push_back(l);
        }
        ms->setLayers(subs);
        ms->setInSTensorID({});
        ms->setOutSTensorID({});
        graph->addLayer(ms);
        for (auto& l : subs) graph->addLayer(l);  // kept in the flat list for id contiguity; the cursor skips them
        return outs;
    }
};

struct RuntimeHandle {
    std::unique_ptr<runtime::NNRuntime> rt;
    RuntimeHandle(GraphBuilder& g, const std::string& model_type)
        : rt(std::make_unique<runtime::NNRuntime>(g.graph, model_type)) {
        if (rt->lastResult() != RetVal::SUCCESS) throw std::runtime_error("NNRuntime: preProcess failed");
    }
    std::vector<at::Tensor> inferenceModel(std::vector<at::Tensor> inputs, bool profiling, const std::string& profile_path) {
        std::vector<at::Tensor> out;
        if (!profile_path.empty()) rt->setProfilePath(profile_path);
        rt->inferenceModel(inputs, out, profiling);
        if (rt->lastResult() != RetVal::SUCCESS) throw std::runtime_error("NNRuntime::inferenceModel returned FAILURE");
        return out;
    }
};

std::string gemmTypeName(std::vector<int64_t> a, std::vector<int64_t> b) {
    switch (runtime::getGemmType(a, b)) {
        case runtime::GEMM_TYPE::VV: return "VV";
        case runtime::GEMM_TYPE::VM: return "VM";
        case runtime::GEMM_TYPE::MV: return "MV";
        case runtime::GEMM_TYPE::MM: return "MM";
        default: return "UNKNOW";
    }
}

}  // namespace

PYBIND11_MODULE(_pimb200_host, m) {
    m.def("get_gemm_type", &gemmTypeName, "shape class of two rank-4 padded operand shapes");
    py::class_<GraphBuilder>(m, "Graph")
        .def(py::init<>())
        .def("add_input", &GraphBuilder::addInput)
        .def("mark_output", &GraphBuilder::markOutput)
        .def("preset_blob", &GraphBuilder::presetBlob)
        .def("add_list", &GraphBuilder::addList)
        .def("add_addmm", &GraphBuilder::addAddmm, py::arg("self"), py::arg("mat1"), py::arg("mat2"),
             py::arg("act") = "none", py::arg("beta") = 1.0, py::arg("alpha") = 1.0)
        .def("add_matmul", &GraphBuilder::addMatmul)
        .def("add_linear", &GraphBuilder::addLinear, py::arg("x"), py::arg("weight"), py::arg("bias") = py::none())
        .def("add_add", &GraphBuilder::addAdd, py::arg("a"), py::arg("b"), py::arg("alpha") = 1.0)
        .def("add_bmm", &GraphBuilder::addBmm)
        .def("add_softmax", &GraphBuilder::addSoftmax, py::arg("x"), py::arg("dim") = -1, py::arg("log") = false)
        .def("add_argmax", &GraphBuilder::addArgmax, py::arg("x"), py::arg("dim") = -1, py::arg("keepdim") = false)
        .def("add_layer_norm", &GraphBuilder::addLayerNorm, py::arg("x"), py::arg("normalized_shape"),
             py::arg("weight") = py::none(), py::arg("bias") = py::none(), py::arg("eps") = 1e-5)
        .def("add_tanh", &GraphBuilder::addTanh)
        .def("add_embedding", &GraphBuilder::addEmbedding)
        .def("add_masked_fill", &GraphBuilder::addMaskedFill)
        .def("add_cat", &GraphBuilder::addCat, py::arg("list_id"), py::arg("dim"), py::arg("mem_layer_id") = -1)
        .def("add_copy", &GraphBuilder::addCopy)
        .def("add_lstm", &GraphBuilder::addLstm, py::arg("inputs"), py::arg("params"), py::arg("has_biases") = true,
             py::arg("num_layers") = 1, py::arg("bidirectional") = false, py::arg("batch_first") = false,
             py::arg("packed") = false, py::arg("aliases") = std::vector<std::pair<int64_t, int64_t>>())
        .def("add_multistream", &GraphBuilder::addMultiStream);
    py::class_<RuntimeHandle>(m, "NNRuntime")
        .def(py::init<GraphBuilder&, const std::string&>(), py::arg("graph"), py::arg("model_type") = "")
        .def("inferenceModel", &RuntimeHandle::inferenceModel, py::arg("input_tensors"), py::arg("profiling") = false,
             py::arg("profile_path") = "");
    m.def("fallback_count", &runtime::tensor_ops::fallbackCount,
          "how often an operator took the libtorch call instead of a device kernel of this library since the last reset");
    m.def("reset_fallback_count", &runtime::tensor_ops::resetFallbackCount);
    m.def("grouped_launch_count", &runtime::tensor_ops::groupedLaunchCount,
          "MULTISTREAM nodes issued as one grouped launch since the process started");
}
