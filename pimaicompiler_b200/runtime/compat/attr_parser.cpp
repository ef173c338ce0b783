// Replacement unit for the reference's compiler/source/frontend/importer/utils/attr_parser.cpp, which no longer
// compiles against libtorch 2.x (c10::ivalue::Tuple::elements() returns TupleElements, :264-270).  It implements the
// interface declared in the reference's compiler/include/frontend/importer/utils/attr_parser.h with the behaviour the
// importer relies on: node attributes by kind, constant weights of linear / lstm nodes, and the conversion of a
// prim::Constant into an ir::DTensor byte blob (scalars as 8-byte values, strings with their terminator, tensors with
// shape and strides padded to rank 4, tuples and lists of int / float / bool as packed 8-byte elements).
#include "frontend/importer/utils/attr_parser.h"

#include <glog/logging.h>

namespace nn_compiler {
namespace frontend {

using nn_compiler::ir::DataType;
using nn_compiler::ir::DTensor;
using nn_compiler::ir::STensor;

int64_t AttrParser::getIntAttr(const torch::jit::Node* node, c10::Symbol symbol) { return node->i(symbol); }
std::vector<int64_t> AttrParser::getIntArrayAttr(const torch::jit::Node* node, c10::Symbol symbol) { return node->is(symbol); }
double AttrParser::getFP64Attr(const torch::jit::Node* node, c10::Symbol symbol) { return node->f(symbol); }
std::string AttrParser::getStrAttr(const torch::jit::Node* node, c10::Symbol symbol) { return node->s(symbol); }
at::Tensor AttrParser::getTensorAttr(const torch::jit::Node* node, c10::Symbol symbol) { return node->t(symbol); }

namespace {
// the tensor held by a prim::Constant producer, if the value comes from one
bool constantTensor(const torch::jit::Value* v, at::Tensor* out) {
    const torch::jit::Node* n = v->node();
    if (n->kind() != c10::prim::Constant || !n->hasAttribute(c10::attr::value)) return false;
    if (n->kindOf(c10::attr::value) != torch::jit::AttributeKind::t) return false;
    *out = n->t(c10::attr::value);
    return true;
}
}  // namespace

std::pair<std::vector<at::Tensor>, std::vector<at::Tensor>> AttrParser::getGeneralWeightAndBias(
    const torch::jit::Node* node, int weight_idx, int bias_idx) {
    std::vector<at::Tensor> weights, biases;
    at::Tensor t;
    if (constantTensor(node->inputs()[weight_idx], &t)) weights.push_back(t);
    if (constantTensor(node->inputs()[bias_idx], &t)) biases.push_back(t);
    return {weights, biases};
}

std::pair<std::vector<at::Tensor>, std::vector<at::Tensor>> AttrParser::getLstmWeightAndBias(const torch::jit::Node* node) {
    // aten::lstm takes its parameters as a Tensor[] built by a prim::ListConstruct of constants: input 3 of the
    // padded overload, input 2 of the packed one (whose input 3 is hx's list or a flag).  Matrices are weights,
    // vectors are biases.
    std::vector<at::Tensor> weights, biases;
    const torch::jit::Node* list = node->inputs()[3]->node();
    if (list->kind() != c10::prim::ListConstruct) list = node->inputs()[2]->node();
    auto take = [&](const at::Tensor& t) { (t.dim() == 1 ? biases : weights).push_back(t); };
    if (list->kind() == c10::prim::Constant && list->hasAttribute(c10::attr::value) &&
        list->kindOf(c10::attr::value) == torch::jit::AttributeKind::ival) {
        // libtorch 2.x freezing folds the parameter list into one constant of type Tensor[]
        const c10::IValue iv = list->ival(c10::attr::value);
        if (iv.isTensorList())
            for (const at::Tensor& t : iv.toTensorList()) take(t);
        return {weights, biases};
    }
    for (const torch::jit::Value* item : list->inputs()) {
        at::Tensor t;
        if (constantTensor(item, &t)) take(t);
    }
    return {weights, biases};
}

void ptTensor2DTensor(at::Tensor torch_tensor, std::shared_ptr<DTensor> d_tensor) {
    at::Tensor t = torch_tensor;
    const size_t n = (size_t)t.numel();
    switch (t.scalar_type()) {
        case c10::ScalarType::Float: d_tensor->setData(t.data_ptr(), n * 4); d_tensor->setDataType(DataType::FLOAT32); break;
        case c10::ScalarType::Half: d_tensor->setData(t.data_ptr(), n * 2); d_tensor->setDataType(DataType::FLOAT16); break;
        case c10::ScalarType::Long: d_tensor->setData(t.data_ptr(), n * 8); d_tensor->setDataType(DataType::INT64); break;
        case c10::ScalarType::Bool: d_tensor->setData(t.data_ptr(), n * 1); d_tensor->setDataType(DataType::BOOL); break;
        case c10::ScalarType::Int: d_tensor->setData(t.data_ptr(), n * 4); d_tensor->setDataType(DataType::INT32); break;
        default: LOG(FATAL) << "prim::Constant tensor of an unsupported dtype: " << t.scalar_type();
    }
    // shape and strides right-aligned in rank 4, zeros in front (rank <= 4 is what the runtime rebuilds tensors from)
    const int64_t rank = t.dim();
    if (rank >= 1 && rank <= 4) {
        std::vector<int32_t> shape(4, 0);
        std::vector<int64_t> stride(4, 0);
        for (int64_t d = 0; d < rank; ++d) {
            shape[4 - rank + d] = (int32_t)t.size(d);
            stride[4 - rank + d] = t.stride(d);
        }
        d_tensor->setStride(stride);
        d_tensor->setTensorShape(STensor(shape));
    }
}

namespace {
void setScalarShape(const std::shared_ptr<DTensor>& d, int32_t count) {
    d->setTensorShape(STensor(std::vector<int32_t>{0, 0, 0, count}));
}
template <typename T>
void setPacked(const std::shared_ptr<DTensor>& d, const std::vector<T>& v, DataType dt) {
    static_assert(sizeof(T) == 8, "8-byte elements");
    d->setData(v.data(), (uint32_t)(v.size() * 8));
    setScalarShape(d, (int32_t)v.size());
    d->setDataType(dt);
}
// int / bool elements as int64, float elements as double; false when the elements are of another kind
bool packElements(const std::shared_ptr<DTensor>& d, const std::vector<c10::IValue>& elems, const std::string& ntype) {
    if (ntype.find("int") != std::string::npos || ntype.find("bool") != std::string::npos) {
        std::vector<int64_t> v;
        for (const auto& e : elems) v.push_back(e.isBool() ? (int64_t)e.toBool() : e.toInt());
        setPacked(d, v, DataType::INT64);
        return true;
    }
    if (ntype.find("float") != std::string::npos) {
        std::vector<double> v;
        for (const auto& e : elems) v.push_back(e.toDouble());
        setPacked(d, v, DataType::FLOAT64);
        return true;
    }
    return false;
}
}  // namespace

std::shared_ptr<DTensor> getDTensorData(const torch::jit::Node* node_constant) {
    auto data = std::make_shared<DTensor>();
    data->setDataType(DataType::UNDEFINED);
    const std::string ntype = node_constant->output()->type()->str();
    auto first_attr = [&]() { return node_constant->attributeNames().at(0); };
    if (ntype == "str" || ntype == "Device") {
        const std::string value = node_constant->s(first_attr());
        data->setData(value.c_str(), (uint32_t)value.length() + 1);
        setScalarShape(data, (int32_t)value.length());
        data->setDataType(DataType::UINT8);
    } else if (ntype == "int" || ntype == "bool") {
        const int64_t value = node_constant->i(first_attr());
        data->setData(&value, 8);
        setScalarShape(data, 1);
        data->setDataType(DataType::INT64);
    } else if (ntype == "float") {
        const double value = node_constant->f(first_attr());
        data->setData(&value, 8);
        setScalarShape(data, 1);
        data->setDataType(DataType::FLOAT64);
    } else if (ntype == "Tensor") {
        ptTensor2DTensor(node_constant->t(first_attr()), data);
    } else if (ntype.find("None") != std::string::npos) {
        data->setDataType(DataType::UINT8);
    } else if (ntype.find('(') != std::string::npos && ntype.find(')') != std::string::npos) {
        const auto tuple = node_constant->ival(c10::attr::value).toTuple();
        std::vector<c10::IValue> elems;
        for (const auto& e : tuple->elements()) elems.push_back(e);
        if (!packElements(data, elems, ntype)) LOG(FATAL) << "tuple constant of an unsupported element type: " << ntype;
    } else if (ntype.find('[') != std::string::npos && ntype.find(']') != std::string::npos) {
        const auto list = node_constant->ival(c10::attr::value).toList();
        std::vector<c10::IValue> elems;
        for (size_t i = 0; i < list.size(); ++i) elems.push_back(list.get(i));
        if (!packElements(data, elems, ntype)) LOG(FATAL) << "list constant of an unsupported element type: " << ntype;
    } else {
        LOG(FATAL) << "prim::Constant of an unsupported type: " << ntype;
        return nullptr;
    }
    return data;
}

}  // namespace frontend
}  // namespace nn_compiler
