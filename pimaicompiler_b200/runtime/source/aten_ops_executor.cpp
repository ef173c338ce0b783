// Op executors for aten layers, written against the reference's IR classes.  Each keeps the contract of its namesake in
// the reference's runtime/source/executor/op_executor/aten_ops_executor.cpp: inputs are read from the blob store by
// in-STensor id, an attribute comes from the layer object unless it still holds its "default value" sentinel (then it
// is the next input blob), results are published with updateBlob.  The device work of the hot ops goes through the
// tensor-level functions of tensor_ops (pimb200 C ABI); the adapters at the end make one libtorch call each.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDACachingAllocator.h>
#include <c10/cuda/CUDAGuard.h>
#include <glog/logging.h>

#include "executor/op_executor/ops_executor.h"
#include "ir/include/common/utils.hpp"
#include "pimb200.h"
#include "tensor_ops.h"

namespace nn_compiler {
namespace runtime {
namespace op_executor {

namespace {
using ir::DataType;
using torch::jit::IValue;

IValue& blob(StreamExecutor& ex, int64_t id) { return ex.findBlob(id).second; }
at::Tensor blobTensor(StreamExecutor& ex, int64_t id) {
    IValue& iv = blob(ex, id);
    TORCH_CHECK(iv.isTensor(), "blob ", id, " is not a tensor");
    return iv.toTensor();
}
tensor_ops::OpContext context(StreamExecutor& ex) {
    tensor_ops::OpContext cx;
    cx.stream = ex.currentStream();
    return cx;
}
void publish(StreamExecutor& ex, tensor_ops::OpContext& cx, Layer& layer, const at::Tensor& out) {
    ex.setStatus(cx.status);
    ex.updateBlob(layer->getOutSTensorID()[0], DataType::TENSOR, IValue(out));
}
// attribute-or-input: the layer's value unless it is the sentinel, else the next input blob (an int)
int64_t attrOrInput(StreamExecutor& ex, int64_t attr, const std::vector<uint32_t>& in, int& in_id) {
    if (!ir::isDefaultValue(attr)) return attr;
    return blob(ex, in[in_id++]).toInt();
}
int attrOrInput(StreamExecutor& ex, int attr, const std::vector<uint32_t>& in, int& in_id) {
    if (!ir::isDefaultValue(attr)) return attr;
    return (int)blob(ex, in[in_id++]).toInt();
}
std::vector<uint32_t> uniqueOuts(Layer& layer) {
    auto out = layer->getOutSTensorID();
    out.erase(std::unique(out.begin(), out.end()), out.end());
    return out;
}
std::vector<at::Tensor> tensorList(const IValue& iv) {
    std::vector<at::Tensor> ts;
    if (iv.isTensorList()) {
        for (const at::Tensor& t : iv.toTensorList()) ts.push_back(t);
    } else if (iv.isList()) {
        for (const IValue& e : iv.toListRef()) ts.push_back(e.toTensor());
    } else {
        TORCH_CHECK(false, "a tensor list was expected");
    }
    return ts;
}
}  // namespace

// aten::add(self, other, alpha): int + int, tensor + scalar (libtorch), tensor + tensor (fp16 same-shape / row
// broadcast through the device kernel, as the reference's custom_add branch, aten_ops_executor.cpp:110-166)
void executeAtenAdd(Layer& layer, StreamExecutor& ex) {
    auto add_layer = std::static_pointer_cast<ir::AtenAddLayer>(layer);
    auto in = layer->getInSTensorID();
    IValue a = blob(ex, in[0]), b = blob(ex, in[1]);
    int64_t alpha = add_layer->getAlpha();
    if (ir::isDefaultValue(alpha)) alpha = (in.size() == 3 && ex.checkValidBlobID(in[2]) && blob(ex, in[2]).isInt()) ? blob(ex, in[2]).toInt() : 1;
    const int64_t out_id = layer->getOutSTensorID()[0];
    if (a.isInt() && b.isInt()) {
        ex.updateBlob(out_id, DataType::INT64, IValue(a.toInt() + alpha * b.toInt()));
        return;
    }
    at::Tensor self = a.toTensor();
    if (b.isTensor()) {
        auto cx = context(ex);
        publish(ex, cx, layer, tensor_ops::add(cx, self, b.toTensor(), (double)alpha));
    } else if (b.isScalar()) {
        ex.updateBlob(out_id, DataType::TENSOR, IValue(at::add(self, b.toScalar(), alpha)));
    } else {
        TORCH_CHECK(false, "aten::add: unsupported operand kinds");
    }
}

// aten::addmm(self, mat1, mat2, beta, alpha) with the activation FuseActivation folded in (act_type)
void executeAtenAddmm(Layer& layer, StreamExecutor& ex) {
    auto addmm_layer = std::static_pointer_cast<ir::AtenAddmmLayer>(layer);
    auto in = layer->getInSTensorID();
    int64_t beta = 1, alpha = 1;
    if (in.size() == 5) {
        beta = blob(ex, in[3]).toInt();
        alpha = blob(ex, in[4]).toInt();
    }
    const std::string act = addmm_layer->get_act_type();
    const bool relu = act == "aten::relu" || act == "aten::max";
    auto cx = context(ex);
    IValue self = blob(ex, in[0]);
    at::Tensor out;
    if (self.isNone()) {
        out = tensor_ops::matmul(cx, blobTensor(ex, in[1]), blobTensor(ex, in[2]));
        if (relu) out = at::relu(out);
    } else {
        out = tensor_ops::addmm(cx, self.toTensor(), blobTensor(ex, in[1]), blobTensor(ex, in[2]), (double)beta, (double)alpha, relu);
    }
    publish(ex, cx, layer, out);
}

void executeAtenMatmul(Layer& layer, StreamExecutor& ex) {
    auto in = layer->getInSTensorID();
    auto cx = context(ex);
    publish(ex, cx, layer, tensor_ops::matmul(cx, blobTensor(ex, in[0]), blobTensor(ex, in[1])));
}

void executeAtenBmm(Layer& layer, StreamExecutor& ex) {
    auto in = layer->getInSTensorID();
    auto cx = context(ex);
    publish(ex, cx, layer, tensor_ops::bmm(cx, blobTensor(ex, in[0]), blobTensor(ex, in[1])));
}

// aten::linear with the weight / bias blobs ModelBuilder preloaded (only reached when ConvertLinearToAddmm did not fire)
void executeAtenLinear(Layer& layer, StreamExecutor& ex) {
    auto lin = std::static_pointer_cast<ir::AtenLinearLayer>(layer);
    auto in = layer->getInSTensorID();
    auto w_ids = lin->getWeightIds(), b_ids = lin->getBiasIds();
    TORCH_CHECK(w_ids.size() == 1, "aten::linear: one preloaded weight expected");
    at::Tensor W = blobTensor(ex, w_ids[0]);
    at::Tensor b = b_ids.size() == 1 ? blobTensor(ex, b_ids[0]) : at::Tensor();
    auto cx = context(ex);
    publish(ex, cx, layer, tensor_ops::linear(cx, blobTensor(ex, in[0]), W, b));
}

// aten::cat(tensors, dim).  A layer labelled with a pre-allocated buffer (CatLabeling, GNMT) returns that buffer:
// its producers wrote into slices of it, nothing is copied.
void executeAtenCat(Layer& layer, StreamExecutor& ex) {
    auto cat_layer = std::static_pointer_cast<ir::AtenCatLayer>(layer);
    auto in = layer->getInSTensorID();
    const int64_t out_id = layer->getOutSTensorID()[0];
    const int64_t mem_id = cat_layer->getMemLayerId();
    if (ex.getModelType() == "GNMT" && mem_id != -1 && ex.checkValidBlobID(mem_id)) {
        ex.updateBlob(out_id, DataType::TENSOR, blob(ex, mem_id));
        return;
    }
    int in_id = 1;
    int dim = attrOrInput(ex, cat_layer->getDim(), in, in_id);
    auto cx = context(ex);
    publish(ex, cx, layer, tensor_ops::cat(cx, tensorList(blob(ex, in[0])), dim));
}

void executeAtenCopy(Layer& layer, StreamExecutor& ex) {
    auto copy_layer = std::static_pointer_cast<ir::AtenCopyLayer>(layer);
    auto in = layer->getInSTensorID();
    int in_id = 2;
    int nb = attrOrInput(ex, copy_layer->getNonBlocking(), in, in_id);
    auto cx = context(ex);
    publish(ex, cx, layer, tensor_ops::copy_(cx, blobTensor(ex, in[0]), blobTensor(ex, in[1]), nb != 0));
}

// aten::embedding(weight, indices): the table is an input blob or, for the RNN-T prediction net, the rows
// SetWeightsForEmbedding lifted onto the layer (set_weights_for_embedding.cpp:37-85); indices already on the device
// stay there
void executeAtenEmbedding(Layer& layer, StreamExecutor& ex) {
    auto emb = std::static_pointer_cast<ir::AtenEmbeddingLayer>(layer);
    auto in = layer->getInSTensorID();
    auto cx = context(ex);
    auto rows = emb->getWeights();
    if (!rows.empty()) {
        at::Tensor table = at::cat(rows, 0).to(at::kCUDA);
        table = table.view({(int64_t)rows.size(), -1});
        publish(ex, cx, layer, tensor_ops::embedding(cx, table, blobTensor(ex, in[0]).to(at::kCUDA)));
        return;
    }
    publish(ex, cx, layer, tensor_ops::embedding(cx, blobTensor(ex, in[0]), blobTensor(ex, in[1])));
}

void executeAtenSoftmax(Layer& layer, StreamExecutor& ex) {
    auto sm = std::static_pointer_cast<ir::AtenSoftmaxLayer>(layer);
    auto in = layer->getInSTensorID();
    int in_id = 1;
    int64_t dim = attrOrInput(ex, sm->getDim(), in, in_id);
    auto cx = context(ex);
    publish(ex, cx, layer, tensor_ops::softmax(cx, blobTensor(ex, in[0]), dim, false));
}

void executeAtenLogSoftmax(Layer& layer, StreamExecutor& ex) {
    auto sm = std::static_pointer_cast<ir::AtenLogSoftmaxLayer>(layer);
    auto in = layer->getInSTensorID();
    int in_id = 1;
    int64_t dim = attrOrInput(ex, sm->getDim(), in, in_id);
    auto cx = context(ex);
    publish(ex, cx, layer, tensor_ops::softmax(cx, blobTensor(ex, in[0]), dim, true));
}

void executeAtenArgmax(Layer& layer, StreamExecutor& ex) {
    auto am = std::static_pointer_cast<ir::AtenArgmaxLayer>(layer);
    auto in = layer->getInSTensorID();
    int in_id = 1;
    int64_t dim = attrOrInput(ex, am->getDim(), in, in_id);
    int64_t keep = am->getKeepDim();
    if (ir::isDefaultValue(keep)) keep = blob(ex, in[in_id++]).toInt();
    auto cx = context(ex);
    publish(ex, cx, layer, tensor_ops::argmax(cx, blobTensor(ex, in[0]), dim, keep != 0));
}

// aten::topk(self, k, dim, largest, sorted) -> (values, indices)
void executeAtenTopk(Layer& layer, StreamExecutor& ex) {
    auto tk = std::static_pointer_cast<ir::AtenTopkLayer>(layer);
    auto in = layer->getInSTensorID();
    auto outs = uniqueOuts(layer);
    TORCH_CHECK(outs.size() == 2, "aten::topk publishes values and indices");
    int in_id = 1;
    const int k = attrOrInput(ex, tk->getK(), in, in_id);
    const int dim = attrOrInput(ex, tk->getDim(), in, in_id);
    const int largest = attrOrInput(ex, tk->getLargest(), in, in_id);
    const int sorted = attrOrInput(ex, tk->getSorted(), in, in_id);
    auto cx = context(ex);
    auto r = tensor_ops::topk(cx, blobTensor(ex, in[0]), k, dim, largest != 0, sorted != 0);
    ex.setStatus(cx.status);
    ex.updateBlob(outs[0], DataType::TENSOR, IValue(std::get<0>(r)));
    ex.updateBlob(outs[1], DataType::TENSOR, IValue(std::get<1>(r)));
}

void executeAtenTanh(Layer& layer, StreamExecutor& ex) {
    auto cx = context(ex);
    publish(ex, cx, layer, tensor_ops::tanh(cx, blobTensor(ex, layer->getInSTensorID()[0])));
}

namespace {
struct LstmFlags {
    int has_biases, train, bidirectional, batch_first;
    int64_t num_layers;
    double dropout;
};
}  // namespace

// aten::lstm, padded input.  inputs = (input, hx list[, params list][, flags still held as inputs]).  The packed
// weights come from the handle ModelBuilder made for this layer.  GNMT graphs labelled by LstmLabeling / CatLabeling
// (match_custom_opt, custom_opt_number k = 0..3) get their results written in place, as the reference's MIOpen executor
// does (miopen_ops_executor.cpp:193-228): (h_n, c_n) into rows 2k and 2k+1 of the pre-allocated [8,1,H] state buffer,
// and for k = 0, 1 the output into the first H columns of the [1,1,2H] buffer of the cat layer two layers downstream.
void executeAtenLSTM1(Layer& layer, StreamExecutor& ex) {
    auto lstm = std::static_pointer_cast<ir::AtenLSTM1Layer>(layer);
    auto in = layer->getInSTensorID();
    auto outs = uniqueOuts(layer);
    TORCH_CHECK(outs.size() == 3, "aten::lstm publishes output, h_n, c_n");
    int in_id = 0;
    at::Tensor input = blobTensor(ex, in[in_id++]);
    auto hx = tensorList(blob(ex, in[in_id++]));
    TORCH_CHECK(hx.size() == 2, "aten::lstm expects hx = [h0, c0]");
    if ((int)in.size() > in_id && (blob(ex, in[in_id]).isTensorList())) ++in_id;   // params list: preloaded instead
    LstmFlags f;
    f.has_biases = attrOrInput(ex, lstm->getHasBiases(), in, in_id);
    f.num_layers = attrOrInput(ex, lstm->getNumLayers(), in, in_id);
    f.dropout = lstm->getDropout();
    if (ir::isDefaultValue(f.dropout)) f.dropout = blob(ex, in[in_id++]).toDouble();
    f.train = attrOrInput(ex, lstm->getTrain(), in, in_id);
    f.bidirectional = attrOrInput(ex, lstm->getBidirectional(), in, in_id);
    f.batch_first = attrOrInput(ex, lstm->getBatchFirst(), in, in_id);
    pimb200_lstm* handle = ex.lstmHandle(layer->getID());
    TORCH_CHECK(handle != nullptr, "aten::lstm layer ", layer->getName(), " has no packed weights");

    tensor_ops::LstmResult pre;
    int64_t cat_mem_id = -1;
    const int k = lstm->getCustomOptNumber();
    if (ex.getModelType() == "GNMT" && lstm->getMatchCustomOpt() && hx[0].size(0) == 1 && hx[0].size(1) == 1 && k >= 0 && k < 4) {
        at::Tensor state = blobTensor(ex, lstm->getCustomCatMemId());           // [8, 1, H]
        pre.hn = state.narrow(0, 2 * k, 1);
        pre.cn = state.narrow(0, 2 * k + 1, 1);
        if (k <= 1 && input.size(0) == 1 && input.size(1) == 1) {
            auto out_layer = ex.getGraph()->getLayerByPosition(layer->getNextLayerIDs()[k == 0 ? 3 : 0]);
            auto cat_layer = ex.getGraph()->getLayerByPosition(out_layer->getNextLayerIDs()[0]);
            cat_mem_id = std::static_pointer_cast<ir::AtenCatLayer>(cat_layer)->getMemLayerId();
            at::Tensor buf = blobTensor(ex, cat_mem_id);                         // [1, 1, 2H]
            pre.y = buf.view({-1}).narrow(0, 0, hx[0].size(2)).view({1, 1, hx[0].size(2)});
        }
    }
    auto cx = context(ex);
    auto r = tensor_ops::lstm(cx, handle, input, hx[0], hx[1], f.batch_first != 0, f.bidirectional != 0, pre);
    ex.setStatus(cx.status);
    ex.updateBlob(outs[0], DataType::TENSOR, IValue(r.y));
    ex.updateBlob(outs[1], DataType::TENSOR, IValue(r.hn));
    ex.updateBlob(outs[2], DataType::TENSOR, IValue(r.cn));
}

// aten::lstm, packed sequence: inputs = (data, batch_sizes, hx list[, params list][, flags])
void executeAtenLSTM2(Layer& layer, StreamExecutor& ex) {
    auto lstm = std::static_pointer_cast<ir::AtenLSTM2Layer>(layer);
    auto in = layer->getInSTensorID();
    auto outs = uniqueOuts(layer);
    TORCH_CHECK(outs.size() == 3, "aten::lstm publishes output, h_n, c_n");
    int in_id = 0;
    at::Tensor data = blobTensor(ex, in[in_id++]);
    at::Tensor batch_sizes = blobTensor(ex, in[in_id++]);
    auto hx = tensorList(blob(ex, in[in_id++]));
    if ((int)in.size() > in_id && blob(ex, in[in_id]).isTensorList()) ++in_id;
    attrOrInput(ex, lstm->getHasBiases(), in, in_id);
    attrOrInput(ex, lstm->getNumLayers(), in, in_id);
    double dropout = lstm->getDropout();
    if (ir::isDefaultValue(dropout)) ++in_id;
    attrOrInput(ex, lstm->getTrain(), in, in_id);
    const int bidirectional = attrOrInput(ex, lstm->getBidirectional(), in, in_id);
    pimb200_lstm* handle = ex.lstmHandle(layer->getID());
    TORCH_CHECK(handle != nullptr, "aten::lstm layer ", layer->getName(), " has no packed weights");
    auto cx = context(ex);
    auto r = tensor_ops::lstmPacked(cx, handle, data, batch_sizes, hx[0], hx[1], bidirectional != 0);
    ex.setStatus(cx.status);
    ex.updateBlob(outs[0], DataType::TENSOR, IValue(r.y));
    ex.updateBlob(outs[1], DataType::TENSOR, IValue(r.hn));
    ex.updateBlob(outs[2], DataType::TENSOR, IValue(r.cn));
}

// MULTISTREAM (runtime/source/executor/op_executor/stream_ops_executor.cpp:27-50): the node's addmm / matmul layers
// are independent; each runs with a side stream of libtorch's pool as the current stream (so its temporaries are
// made on that stream), after the work already queued on the main stream; the main stream waits for all of them.  When
// every branch is a matrix-class fp16 product the whole node is ONE grouped launch on the main stream instead.  The
// cursor then skips the copies of those layers that follow the node in the flat list.
// The branches as one grouped launch on the main stream when all of them are matrix-class fp16 products with alpha = beta
// = 1; false when they are not (nothing has been launched then).
static bool multiStreamGrouped(std::shared_ptr<ir::MultiStreamLayer>& ms, StreamExecutor& ex) {
    std::vector<tensor_ops::MatmulBranch> branches;
    for (auto sub : ms->getLayers()) {
        auto in = sub->getInSTensorID();
        tensor_ops::MatmulBranch br;
        if (sub->getType() == ir::LayerType::ATENADDMM) {
            auto addmm_layer = std::static_pointer_cast<ir::AtenAddmmLayer>(sub);
            if (in.size() == 5 && (blob(ex, in[3]).toInt() != 1 || blob(ex, in[4]).toInt() != 1)) return false;
            const std::string act = addmm_layer->get_act_type();
            br.relu = act == "aten::relu" || act == "aten::max";
            IValue self = blob(ex, in[0]);
            if (!self.isNone()) br.bias = self.toTensor();
            br.mat1 = blobTensor(ex, in[1]);
            br.mat2 = blobTensor(ex, in[2]);
        } else if (sub->getType() == ir::LayerType::ATENMATMUL) {
            br.mat1 = blobTensor(ex, in[0]);
            br.mat2 = blobTensor(ex, in[1]);
        } else {
            return false;
        }
        branches.push_back(br);
    }
    auto cx = context(ex);
    auto outs = tensor_ops::groupedMatmul(cx, branches);
    if (outs.empty()) {
        if (cx.status != 0) ex.setStatus(cx.status);
        return false;
    }
    size_t i = 0;
    for (auto sub : ms->getLayers()) publish(ex, cx, sub, outs[i++]);
    return true;
}

void executeMultiStream(Layer& layer, StreamExecutor& ex) {
    auto ms = std::static_pointer_cast<ir::MultiStreamLayer>(layer);
    if (multiStreamGrouped(ms, ex)) {
        ex.setCursor(layer->getID() + ms->getLayerNum() + 1);
        return;
    }
    const c10::cuda::CUDAStream main = c10::cuda::getCurrentCUDAStream();
    at::cuda::CUDAEvent& fork = ex.event(0);
    fork.record(main);
    size_t i = 0;
    for (auto sub : ms->getLayers()) {
        const c10::cuda::CUDAStream side = ex.sideStream(i);
        fork.block(side);
        {
            c10::cuda::CUDAStreamGuard guard(side);
            if (sub->getType() == ir::LayerType::ATENADDMM) executeAtenAddmm(sub, ex);
            else if (sub->getType() == ir::LayerType::ATENMATMUL) executeAtenMatmul(sub, ex);
            else ex.setStatus(PIMB200_ERR_UNSUPPORTED);
        }
        for (auto id : sub->getOutSTensorID()) {
            if (!ex.checkValidBlobID(id)) continue;
            IValue& iv = blob(ex, id);
            if (iv.isTensor() && iv.toTensor().is_cuda())
                c10::cuda::CUDACachingAllocator::recordStream(iv.toTensor().storage().data_ptr(), main);
        }
        at::cuda::CUDAEvent& join = ex.event(1 + i);
        join.record(side);
        join.block(main);
        ++i;
    }
    ex.setCursor(layer->getID() + ms->getLayerNum() + 1);
}

// ---------------------------------------------------------------------------------------------
// pass-through adapters
// ---------------------------------------------------------------------------------------------
void executeAtenItem(Layer& layer, StreamExecutor& ex) {
    at::Tensor t = blobTensor(ex, layer->getInSTensorID()[0]);
    const c10::Scalar s = t.item();
    const int64_t out_id = layer->getOutSTensorID()[0];
    if (s.isFloatingPoint()) ex.updateBlob(out_id, DataType::FLOAT64, IValue(s.toDouble()));
    else if (s.isBoolean()) ex.updateBlob(out_id, DataType::BOOL, IValue((int64_t)s.toBool()));
    else ex.updateBlob(out_id, DataType::INT64, IValue(s.toLong()));
}

void executeAtenCompare(Layer& layer, StreamExecutor& ex) {
    auto in = layer->getInSTensorID();
    IValue a = blob(ex, in[0]), b = blob(ex, in[1]);
    const int64_t out_id = layer->getOutSTensorID()[0];
    const ir::LayerType type = layer->getType();
    if (a.isTensor()) {
        at::Tensor t = a.toTensor(), out;
        auto cmp = [&](auto&& rhs) {
            switch (type) {
                case ir::LayerType::ATENGT: return at::gt(t, rhs);
                case ir::LayerType::ATENLT: return at::lt(t, rhs);
                case ir::LayerType::ATENGE: return at::ge(t, rhs);
                case ir::LayerType::ATENLE: return at::le(t, rhs);
                case ir::LayerType::ATENEQ: return at::eq(t, rhs);
                default: return at::ne(t, rhs);
            }
        };
        out = b.isTensor() ? cmp(b.toTensor()) : cmp(b.toScalar());
        ex.updateBlob(out_id, DataType::TENSOR, IValue(out));
        return;
    }
    const double x = a.toScalar().toDouble(), y = b.toScalar().toDouble();
    bool r = false;
    switch (type) {
        case ir::LayerType::ATENGT: r = x > y; break;
        case ir::LayerType::ATENLT: r = x < y; break;
        case ir::LayerType::ATENGE: r = x >= y; break;
        case ir::LayerType::ATENLE: r = x <= y; break;
        case ir::LayerType::ATENEQ: r = x == y; break;
        default: r = x != y; break;
    }
    ex.updateBlob(out_id, DataType::BOOL, IValue((int64_t)r));
}

void executeAtenTranspose(Layer& layer, StreamExecutor& ex) {
    auto tr = std::static_pointer_cast<ir::AtenTransposeLayer>(layer);
    auto in = layer->getInSTensorID();
    int in_id = 1;
    int64_t d0 = attrOrInput(ex, tr->getDim0(), in, in_id);
    int64_t d1 = attrOrInput(ex, tr->getDim1(), in, in_id);
    ex.updateBlob(layer->getOutSTensorID()[0], DataType::TENSOR, IValue(at::transpose(blobTensor(ex, in[0]), d0, d1)));
}

void executeAtenSelect(Layer& layer, StreamExecutor& ex) {
    auto sel = std::static_pointer_cast<ir::AtenSelectLayer>(layer);
    auto in = layer->getInSTensorID();
    int in_id = 1;
    int64_t dim = attrOrInput(ex, sel->getDim(), in, in_id);
    int64_t index = attrOrInput(ex, sel->getIndex(), in, in_id);
    ex.updateBlob(layer->getOutSTensorID()[0], DataType::TENSOR, IValue(at::select(blobTensor(ex, in[0]), dim, index)));
}

void executeAtenRelu(Layer& layer, StreamExecutor& ex) {
    ex.updateBlob(layer->getOutSTensorID()[0], DataType::TENSOR, IValue(at::relu(blobTensor(ex, layer->getInSTensorID()[0]))));
}

void executeAtenSize(Layer& layer, StreamExecutor& ex) {
    auto sz = std::static_pointer_cast<ir::AtenSizeLayer>(layer);
    auto in = layer->getInSTensorID();
    at::Tensor t = blobTensor(ex, in[0]);
    int64_t dim = sz->getDim();
    const int64_t out_id = layer->getOutSTensorID()[0];
    if (ir::isDefaultValue(dim) && in.size() > 1) dim = blob(ex, in[1]).toInt();
    if (ir::isDefaultValue(dim)) {
        ex.updateBlob(out_id, DataType::LIST, IValue(t.sizes().vec()));
    } else {
        ex.updateBlob(out_id, DataType::INT64, IValue(t.size(dim)));
    }
}

void executeAtenInt(Layer& layer, StreamExecutor& ex) {
    IValue v = blob(ex, layer->getInSTensorID()[0]);
    const int64_t r = v.isTensor() ? v.toTensor().item<int64_t>() : v.toScalar().toLong();
    ex.updateBlob(layer->getOutSTensorID()[0], DataType::INT64, IValue(r));
}

void executeAtenUnsqueeze(Layer& layer, StreamExecutor& ex) {
    auto us = std::static_pointer_cast<ir::AtenUnsqueezeLayer>(layer);
    auto in = layer->getInSTensorID();
    int in_id = 1;
    int64_t dim = attrOrInput(ex, us->getDim(), in, in_id);
    ex.updateBlob(layer->getOutSTensorID()[0], DataType::TENSOR, IValue(at::unsqueeze(blobTensor(ex, in[0]), dim)));
}

}  // namespace op_executor
}  // namespace runtime
}  // namespace nn_compiler
