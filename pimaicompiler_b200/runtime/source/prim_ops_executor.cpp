// Prim-op executors: constants, containers and the control ops of the flat layer list.
//
// The compiler's TakeInBodyNet pass flattens prim::If / prim::Loop sub-graphs into one layer list with marker layers
// (compiler/source/frontend/optimizer/take_in_body_net.cpp), and ControlLayerExecution fills in their jump targets
// (compiler/source/middlend/optimizer/stream_execution/control_layer_execution.cpp:34-74).  The protocol these
// executors implement is the one the reference's interpreter follows
// (runtime/source/executor/op_executor/prim_ops_executor.cpp:208-328, 373-393, 744-922):
//   If(cond)              true: fall through into the then-net; false: jump to getElseNetStartLayer()
//   EndIf (then-net's)    jump to getGotoLayer() (behind the else-net)
//   EndIf (else-net's)    its inputs are (then outputs..., else outputs...): publish the taken half as its outputs
//   Loop(max, cond, x..)  at position p; LoopIndex at p+1, Block at p+2.  Loop copies x.. to its outputs, resets the
//                         index and enters Block
//   Block(i, x..)         if i >= max or !cond: copy EndLoop's inputs[1..] to EndLoop's outputs and jump behind it;
//                         else publish (i, x..) as the block's outputs and fall through into the body
//   EndLoop(cond', y..)   i += 1, cond = cond', copy y.. to Block's inputs[1..], jump back to Block
#include <glog/logging.h>

#include "executor/op_executor/ops_executor.h"
#include "ir/include/common/utils.hpp"

namespace nn_compiler {
namespace runtime {
namespace op_executor {

namespace {
using ir::DataType;
using torch::jit::IValue;

IValue& blob(StreamExecutor& ex, int64_t id) { return ex.findBlob(id).second; }
void copyBlob(StreamExecutor& ex, int64_t from, int64_t to) {
    auto& src = ex.findBlob(from);
    ex.updateBlob(to, src.first, src.second);
}
std::vector<uint32_t> uniqueOuts(Layer& layer) {
    std::vector<uint32_t> out;
    for (auto id : layer->getOutSTensorID())
        if (std::find(out.begin(), out.end(), id) == out.end()) out.push_back(id);
    return out;
}
int64_t truth(const IValue& iv) {
    if (iv.isBool()) return iv.toBool() ? 1 : 0;
    if (iv.isInt()) return iv.toInt() != 0;
    if (iv.isTensor()) return iv.toTensor().item<int64_t>() != 0;
    TORCH_CHECK(false, "a condition must be an int, a bool or a one-element tensor");
}

at::ScalarType scalarTypeOf(DataType dt) {
    switch (dt) {
        case DataType::INT8: return at::kChar;
        case DataType::UINT8: return at::kByte;
        case DataType::INT16: return at::kShort;
        case DataType::INT32: return at::kInt;
        case DataType::INT64: return at::kLong;
        case DataType::FLOAT16: return at::kHalf;
        case DataType::FLOAT32: return at::kFloat;
        case DataType::FLOAT64: return at::kDouble;
        case DataType::BOOL: return at::kBool;
        default: TORCH_CHECK(false, "constant tensor of an unsupported element type");
    }
}
// the tensor a DTensor byte blob describes (shape and strides with their leading zeros dropped), on the device
at::Tensor tensorOf(const std::shared_ptr<ir::DTensor>& d) {
    auto st = d->getTensorShape();
    std::vector<int64_t> shape, stride;
    const auto dims = st.getDims();
    const auto strides = d->getStride();
    for (size_t i = 0; i < dims.size(); ++i) {
        if (dims[i] == 0) continue;
        shape.push_back(dims[i]);
        stride.push_back(i < strides.size() ? strides[i] : 1);
    }
    auto bytes = d->getData<uint8_t>();
    at::Tensor host = at::from_blob(bytes->data(), shape, stride, at::TensorOptions().dtype(scalarTypeOf(d->getDataType())));
    return host.to(at::kCUDA);   // the copy ends the borrow of `bytes`
}
// scalar constants are stored as 8-byte values
IValue scalarOf(const uint8_t* p, DataType dt) {
    if (dt == DataType::FLOAT64) { double v; std::memcpy(&v, p, 8); return IValue(v); }
    if (dt == DataType::FLOAT32) { float v; std::memcpy(&v, p, 4); return IValue((double)v); }
    int64_t v = 0;
    std::memcpy(&v, p, 8);
    return IValue(v);
}
bool isTupleType(const std::string& t) { return t.find('(') != std::string::npos && t.find(')') != std::string::npos; }
bool isListType(const std::string& t) { return t.find('[') != std::string::npos && t.find(']') != std::string::npos; }
}  // namespace

void executePrimConstant(Layer& layer, StreamExecutor& ex) {
    auto c = std::static_pointer_cast<ir::PrimConstantLayer>(layer);
    const std::string ntype = c->getNType();
    auto d = c->getAttr();
    auto bytes = d->getData<uint8_t>();
    const uint8_t* p = bytes->data();
    IValue iv;
    DataType dt = DataType::NONE;
    if (ntype == "str" || ntype == "Device") {
        iv = IValue(std::string(reinterpret_cast<const char*>(p)));
        dt = ntype == "str" ? DataType::STRING : DataType::DEVICE;
    } else if (ntype == "int" || ntype == "bool") {
        iv = scalarOf(p, DataType::INT64);
        dt = DataType::INT64;
    } else if (ntype == "float") {
        iv = scalarOf(p, DataType::FLOAT64);
        dt = DataType::FLOAT64;
    } else if (ntype == "Tensor") {
        iv = IValue(tensorOf(d));
        dt = DataType::TENSOR;
    } else if (ntype.find("None") != std::string::npos) {
        dt = DataType::NONE;
    } else if (isTupleType(ntype) || isListType(ntype)) {
        const bool is_float = d->getDataType() == DataType::FLOAT64;
        const size_t n = bytes->size() / 8;
        if (isTupleType(ntype)) {
            std::vector<IValue> elems;
            for (size_t i = 0; i < n; ++i) elems.push_back(scalarOf(p + 8 * i, is_float ? DataType::FLOAT64 : DataType::INT64));
            iv = IValue(c10::ivalue::Tuple::create(std::move(elems)));
            dt = DataType::TUPLE;
        } else if (is_float) {
            c10::List<double> l;
            for (size_t i = 0; i < n; ++i) l.push_back(scalarOf(p + 8 * i, DataType::FLOAT64).toDouble());
            iv = IValue(l);
            dt = DataType::LIST;
        } else {
            c10::List<int64_t> l;
            for (size_t i = 0; i < n; ++i) l.push_back(scalarOf(p + 8 * i, DataType::INT64).toInt());
            iv = IValue(l);
            dt = DataType::LIST;
        }
    } else {
        TORCH_CHECK(false, "prim::Constant of an unsupported type: ", ntype);
    }
    ex.updateBlob(layer->getOutSTensorID()[0], dt, iv);
}

// prim::Variable: a value (scalar, tensor, or list of either) the compiler materialised out of constants
void executePrimVariable(Layer& layer, StreamExecutor& ex) {
    auto v = std::static_pointer_cast<ir::PrimVariableLayer>(layer);
    const std::string ntype = v->getNType();
    auto attrs = v->getAttr();
    TORCH_CHECK(!attrs.empty(), "prim::Variable without data");
    const int64_t out_id = layer->getOutSTensorID()[0];
    auto elementOf = [&](const std::shared_ptr<ir::DTensor>& d) -> IValue {
        int64_t count = 1;
        for (auto e : d->getTensorShape().getDims())
            if (e != 0) count *= e;
        if (count != 1 || d->getDataType() == DataType::FLOAT16) return IValue(tensorOf(d));
        auto bytes = d->getData<uint8_t>();
        return scalarOf(bytes->data(), d->getDataType());
    };
    if (ntype.find("List") != std::string::npos) {
        c10::impl::GenericList l(c10::AnyType::get());
        for (auto& d : attrs) l.push_back(elementOf(d));
        bool all_tensors = true;
        for (const IValue& e : l.vec()) all_tensors = all_tensors && e.isTensor();
        if (all_tensors) {
            c10::List<at::Tensor> tl;
            for (const IValue& e : l.vec()) tl.push_back(e.toTensor());
            ex.updateBlob(out_id, DataType::LIST, IValue(tl));
        } else {
            ex.updateBlob(out_id, DataType::LIST, IValue(l));
        }
    } else if (ntype.find("Tensor") != std::string::npos) {
        ex.updateBlob(out_id, DataType::TENSOR, IValue(tensorOf(attrs[0])));
    } else if (ntype.find("bool") != std::string::npos) {
        ex.updateBlob(out_id, DataType::BOOL, elementOf(attrs[0]));
    } else if (ntype.find("int") != std::string::npos) {
        ex.updateBlob(out_id, DataType::INT64, elementOf(attrs[0]));
    } else {
        TORCH_CHECK(false, "prim::Variable of an unsupported type: ", ntype);
    }
}

void executePrimListConstruct(Layer& layer, StreamExecutor& ex) {
    auto in = layer->getInSTensorID();
    bool all_tensors = !in.empty(), all_ints = !in.empty();
    for (auto id : in) {
        const IValue& e = blob(ex, id);
        all_tensors = all_tensors && e.isTensor();
        all_ints = all_ints && e.isInt();
    }
    IValue out;
    if (all_tensors) {
        c10::List<at::Tensor> l;
        for (auto id : in) l.push_back(blob(ex, id).toTensor());
        out = IValue(l);
    } else if (all_ints) {
        c10::List<int64_t> l;
        for (auto id : in) l.push_back(blob(ex, id).toInt());
        out = IValue(l);
    } else {
        c10::impl::GenericList l(c10::AnyType::get());
        for (auto id : in) l.push_back(blob(ex, id));
        out = IValue(l);
    }
    ex.updateBlob(layer->getOutSTensorID()[0], DataType::LIST, out);
}

void executePrimListUnpack(Layer& layer, StreamExecutor& ex) {
    const IValue& l = blob(ex, layer->getInSTensorID()[0]);
    auto outs = uniqueOuts(layer);
    auto elems = l.toListRef();
    TORCH_CHECK(elems.size() >= outs.size(), "prim::ListUnpack: list shorter than the outputs");
    for (size_t i = 0; i < outs.size(); ++i)
        ex.updateBlob(outs[i], elems[i].isTensor() ? DataType::TENSOR : DataType::IVALUE, elems[i]);
}

void executePrimTupleConstruct(Layer& layer, StreamExecutor& ex) {
    std::vector<IValue> elems;
    for (auto id : layer->getInSTensorID()) elems.push_back(blob(ex, id));
    ex.updateBlob(layer->getOutSTensorID()[0], DataType::TUPLE, IValue(c10::ivalue::Tuple::create(std::move(elems))));
}

void executePrimTupleUnpack(Layer& layer, StreamExecutor& ex) {
    const IValue& t = blob(ex, layer->getInSTensorID()[0]);
    auto outs = uniqueOuts(layer);
    const auto& elems = t.toTupleRef().elements();
    TORCH_CHECK(elems.size() >= outs.size(), "prim::TupleUnpack: tuple shorter than the outputs");
    for (size_t i = 0; i < outs.size(); ++i)
        ex.updateBlob(outs[i], elems[i].isTensor() ? DataType::TENSOR : DataType::IVALUE, elems[i]);
}

void executePrimTupleIndex(Layer& layer, StreamExecutor& ex) {
    auto ti = std::static_pointer_cast<ir::PrimTupleIndexLayer>(layer);
    auto in = layer->getInSTensorID();
    int64_t index = ti->getIndex();
    if (ir::isDefaultValue(index)) index = blob(ex, in[1]).toInt();
    const auto& elems = blob(ex, in[0]).toTupleRef().elements();
    if (index < 0) index += (int64_t)elems.size();
    const IValue e = elems.at((size_t)index);
    ex.updateBlob(layer->getOutSTensorID()[0], e.isTensor() ? DataType::TENSOR : DataType::IVALUE, e);
}

// ---------------------------------------------------------------------------------------------
// control ops
// ---------------------------------------------------------------------------------------------
void executePrimIf(Layer& layer, StreamExecutor& ex) {
    auto if_layer = std::static_pointer_cast<ir::PrimIfLayer>(layer);
    const int64_t cond = truth(blob(ex, layer->getInSTensorID().at(0)));
    ex.setCursor(cond ? (int64_t)layer->getID() + 1 : if_layer->getElseNetStartLayer());
}

void executePrimEndIf(Layer& layer, StreamExecutor& ex) {
    auto end_if = std::static_pointer_cast<ir::PrimEndIfLayer>(layer);
    if (!end_if->getIsElseNet()) {   // end of the then-net: skip the else-net
        ex.setCursor(end_if->getGotoLayer());
        return;
    }
    auto in = layer->getInSTensorID();
    if (!in.empty()) {
        auto if_layer = ex.getGraph()->getLayerByPosition(end_if->getIfLayerId());
        const int64_t cond = truth(blob(ex, if_layer->getInSTensorID().at(0)));
        const size_t half = in.size() / 2, first = cond ? 0 : half;
        auto outs = uniqueOuts(layer);
        for (size_t i = 0; i < half && i < outs.size(); ++i) copyBlob(ex, in[first + i], outs[i]);
    }
    ex.setCursor((int64_t)layer->getID() + 1);
}

void executePrimLoopIndex(Layer& layer, StreamExecutor& ex) {
    auto li = std::static_pointer_cast<ir::PrimLoopIndexLayer>(layer);
    int64_t index = li->getIndex();
    if (index < 0 || ir::isDefaultValue(index)) index = 0;
    ex.updateBlob(layer->getOutSTensorID()[0], DataType::INT64, IValue(index));
}

namespace {
struct LoopInfo {
    std::shared_ptr<ir::PrimLoopLayer> loop;
    int64_t max_trip, cond, index, behind_end;
    int extra_first;   // index of the first carried value among the loop layer's inputs
};
// the loop a Block layer at position `block_pos` belongs to: Loop at block_pos - 2, LoopIndex at block_pos - 1
LoopInfo loopOfBlock(int64_t block_pos, StreamExecutor& ex) {
    auto graph = ex.getGraph();
    LoopInfo li;
    li.loop = std::static_pointer_cast<ir::PrimLoopLayer>(graph->getLayerByPosition(block_pos - 2));
    auto in = li.loop->getInSTensorID();
    int in_id = 0;
    li.max_trip = li.loop->getTripCount();
    if (ir::isDefaultValue(li.max_trip)) li.max_trip = blob(ex, in[in_id++]).toInt();
    li.cond = li.loop->getCond();
    if (ir::isDefaultValue(li.cond)) li.cond = truth(blob(ex, in[in_id++]));
    li.extra_first = in_id;
    auto index_layer = graph->getLayerByPosition(block_pos - 1);
    li.index = blob(ex, index_layer->getOutSTensorID()[0]).toInt();
    li.behind_end = li.loop->getGotoLayer();
    return li;
}
}  // namespace

void executePrimBlock(Layer& layer, StreamExecutor& ex) {
    auto in = layer->getInSTensorID();
    LoopInfo li = loopOfBlock(layer->getID(), ex);
    if (li.index >= li.max_trip || li.cond == 0) {
        // leave: what the last iteration (or the loop's inputs, for zero iterations) carried becomes the loop's result
        auto end_loop = ex.getGraph()->getLayerByPosition(li.behind_end - 1);
        auto end_in = end_loop->getInSTensorID();
        auto end_out = end_loop->getOutSTensorID();
        // carried value i of the next iteration sits in the block's input i + 1 (put there by the Loop layer on entry
        // and by EndLoop after every iteration)
        for (size_t i = 0; i < end_out.size(); ++i) {
            if (i + 1 < in.size() && ex.checkValidBlobID(in[i + 1])) copyBlob(ex, in[i + 1], end_out[i]);
            else if (i + 1 < end_in.size()) copyBlob(ex, end_in[i + 1], end_out[i]);
        }
        // the condition the loop was entered with is restored for the next run of the graph
        li.loop->setCond(ex.getTopOfLoopConditionStack());
        ex.popOfLoopConditionStack();
        ex.setCursor(li.behind_end);
        return;
    }
    // enter the body: block outputs = (index, carried values...)
    auto outs = uniqueOuts(layer);
    ex.updateBlob(outs.at(0), DataType::INT64, IValue(li.index));
    for (size_t i = 1; i < in.size() && i < outs.size(); ++i)
        if (ex.checkValidBlobID(in[i])) copyBlob(ex, in[i], outs[i]);
    ex.setCursor((int64_t)layer->getID() + 1);
}

void executePrimLoop(Layer& layer, StreamExecutor& ex) {
    auto loop = std::static_pointer_cast<ir::PrimLoopLayer>(layer);
    auto graph = ex.getGraph();
    const int64_t pos = layer->getID();
    ex.pushInLoopConditionStack(loop->getCond());
    auto index_layer = graph->getLayerByPosition(pos + 1);
    executePrimLoopIndex(index_layer, ex);   // a loop entered anew starts from its initial index
    // the carried values x.. enter through the Block's inputs[1..]
    auto block = graph->getLayerByPosition(pos + 2);
    auto in = layer->getInSTensorID();
    int first = 0;
    int64_t trip = loop->getTripCount(), cond = loop->getCond();
    if (ir::isDefaultValue(trip)) ++first;
    if (ir::isDefaultValue(cond)) ++first;
    auto block_in = block->getInSTensorID();
    for (size_t i = 0; first + i < in.size() && i + 1 < block_in.size(); ++i)
        if (in[first + i] != block_in[i + 1]) copyBlob(ex, in[first + i], block_in[i + 1]);
    executePrimBlock(block, ex);
}

void executePrimEndLoop(Layer& layer, StreamExecutor& ex) {
    auto end_loop = std::static_pointer_cast<ir::PrimEndLoopLayer>(layer);
    auto graph = ex.getGraph();
    const int64_t loop_pos = end_loop->getGotoLayer();
    auto loop = std::static_pointer_cast<ir::PrimLoopLayer>(graph->getLayerByPosition(loop_pos));
    auto index_layer = graph->getLayerByPosition(loop_pos + 1);
    auto block = graph->getLayerByPosition(loop_pos + 2);
    const int64_t index_blob = index_layer->getOutSTensorID()[0];
    ex.updateBlob(index_blob, DataType::INT64, IValue(blob(ex, index_blob).toInt() + 1));
    auto in = layer->getInSTensorID();
    loop->setCond(truth(blob(ex, in.at(0))));
    auto block_in = block->getInSTensorID();
    for (size_t i = 1; i < in.size() && i < block_in.size(); ++i) copyBlob(ex, in[i], block_in[i]);
    ex.setCursor(loop_pos + 2);
}

}  // namespace op_executor
}  // namespace runtime
}  // namespace nn_compiler
