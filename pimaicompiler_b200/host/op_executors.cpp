// Bodies of the hot-path op executors, written against the pimb200 C ABI.
//
// Each function keeps the contract of its namesake in the reference's
// runtime/source/executor/op_executor/aten_ops_executor.cpp (inputs are read from the blob store by in-STensor id,
// attributes from the layer object, results are published with updateBlob), but the device work goes through
// libpimb200.so instead of PIM / MIOpen / the HIP templates.  Shapes outside the hot path (general batched matmul,
// non-unit alpha/beta, mixed dtypes) are forwarded to the same at:: op the reference falls back to.
#include <ATen/cuda/CUDAContext.h>

#include <ATen/cuda/CUDAEvent.h>
#include <c10/cuda/CUDACachingAllocator.h>
#include <c10/cuda/CUDAGuard.h>

#include "pimb200.h"
#include "stream_executor.h"
#include "tensor_ops.h"

namespace nn_compiler {
namespace runtime {
namespace op_executor {

namespace {

at::Tensor blobTensor(StreamExecutor& ex, int64_t id) {
    auto& iv = ex.findBlob(id).second;
    TORCH_CHECK(iv.isTensor(), "blob ", id, " is not a tensor");
    return iv.toTensor();
}

tensor_ops::OpContext context(StreamExecutor& ex, cudaStream_t st) {
    tensor_ops::OpContext cx;
    cx.stream = st;
    return cx;
}
void publish(StreamExecutor& ex, tensor_ops::OpContext& cx, std::shared_ptr<ir::NNLayer>& layer, const at::Tensor& out) {
    ex.setStatus(cx.status);
    ex.updateBlob(layer->getOutSTensorID()[0], ir::DataType::TENSOR, torch::jit::IValue(out));
}

void runAddmm(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& ex, cudaStream_t st) {
    auto addmm = std::static_pointer_cast<ir::AtenAddmmLayer>(layer);
    const auto& in = layer->getInSTensorID();
    auto cx = context(ex, st);
    at::Tensor out = tensor_ops::addmm(cx, blobTensor(ex, in[0]), blobTensor(ex, in[1]), blobTensor(ex, in[2]), addmm->beta,
                                       addmm->alpha, addmm->getActType() == "aten::relu");
    publish(ex, cx, layer, out);
}

void runMatmul(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& ex, cudaStream_t st) {
    const auto& in = layer->getInSTensorID();
    auto cx = context(ex, st);
    at::Tensor out = tensor_ops::matmul(cx, blobTensor(ex, in[0]), blobTensor(ex, in[1]));
    publish(ex, cx, layer, out);
}

}  // namespace

void executeAtenAddmm(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& ex) { runAddmm(layer, ex, ex.currentStream()); }
void executeAtenAddmmWithStream(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& ex, void* stream) {
    runAddmm(layer, ex, static_cast<cudaStream_t>(stream));
}
void executeAtenMatmul(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& ex) { runMatmul(layer, ex, ex.currentStream()); }
void executeAtenMatmulWithStream(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& ex, void* stream) {
    runMatmul(layer, ex, static_cast<cudaStream_t>(stream));
}

// aten::linear(x, W, b) with W/b preloaded on the layer (only reached when the linear->addmm rewrite did not fire)
void executeAtenLinear(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& ex) {
    auto lin = std::static_pointer_cast<ir::AtenLinearLayer>(layer);
    auto cx = context(ex, ex.currentStream());
    at::Tensor out = tensor_ops::linear(cx, blobTensor(ex, layer->getInSTensorID()[0]), lin->getWeights(), lin->getBiases());
    publish(ex, cx, layer, out);
}

void executeAtenAdd(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& ex) {
    auto add = std::static_pointer_cast<ir::AtenAddLayer>(layer);
    const auto& in = layer->getInSTensorID();
    auto cx = context(ex, ex.currentStream());
    at::Tensor out = tensor_ops::add(cx, blobTensor(ex, in[0]), blobTensor(ex, in[1]), add->alpha);
    publish(ex, cx, layer, out);
}

void executeAtenSoftmax(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& ex) {
    auto sm = std::static_pointer_cast<ir::AtenSoftmaxLayer>(layer);
    auto cx = context(ex, ex.currentStream());
    at::Tensor out = tensor_ops::softmax(cx, blobTensor(ex, layer->getInSTensorID()[0]), sm->dim,
                                         layer->getType() == ir::LayerType::ATENLOGSOFTMAX);
    publish(ex, cx, layer, out);
}

void executeAtenArgmax(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& ex) {
    auto am = std::static_pointer_cast<ir::AtenArgmaxLayer>(layer);
    auto cx = context(ex, ex.currentStream());
    at::Tensor out = tensor_ops::argmax(cx, blobTensor(ex, layer->getInSTensorID()[0]), am->dim, am->keepdim != 0);
    publish(ex, cx, layer, out);
}

void executeAtenLayerNorm(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& ex) {
    auto ln = std::static_pointer_cast<ir::AtenLayerNormLayer>(layer);
    auto cx = context(ex, ex.currentStream());
    at::Tensor out = tensor_ops::layerNorm(cx, blobTensor(ex, layer->getInSTensorID()[0]), ln->normalized_shape, ln->weight,
                                           ln->bias, ln->eps);
    publish(ex, cx, layer, out);
}

void executeAtenTanh(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& ex) {
    auto cx = context(ex, ex.currentStream());
    at::Tensor out = tensor_ops::tanh(cx, blobTensor(ex, layer->getInSTensorID()[0]));
    publish(ex, cx, layer, out);
}

void executeAtenMaskedFill(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& ex) {
    auto mf = std::static_pointer_cast<ir::AtenMaskedFillLayer>(layer);
    const auto& in = layer->getInSTensorID();
    auto cx = context(ex, ex.currentStream());
    at::Tensor out = tensor_ops::maskedFill(cx, blobTensor(ex, in[0]), blobTensor(ex, in[1]), mf->value);
    publish(ex, cx, layer, out);
}

// aten::embedding: the table is an input blob or preloaded on the layer
void executeAtenEmbedding(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& ex) {
    auto emb = std::static_pointer_cast<ir::AtenEmbeddingLayer>(layer);
    const auto& in = layer->getInSTensorID();
    at::Tensor table = emb->weights.defined() ? emb->weights : blobTensor(ex, in[0]);
    at::Tensor idx = blobTensor(ex, in[emb->weights.defined() ? 0 : 1]);
    auto cx = context(ex, ex.currentStream());
    at::Tensor out = tensor_ops::embedding(cx, table, idx);
    publish(ex, cx, layer, out);
}

void executeAtenBmm(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& ex) {
    const auto& in = layer->getInSTensorID();
    auto cx = context(ex, ex.currentStream());
    at::Tensor out = tensor_ops::bmm(cx, blobTensor(ex, in[0]), blobTensor(ex, in[1]));
    publish(ex, cx, layer, out);
}

// aten::cat over a TensorList blob.  When the layer carries the id of a pre-filled buffer (the "custom cat" label of
// the GNMT graphs) that buffer is the result and nothing is copied.
void executeAtenCat(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& ex) {
    auto cat = std::static_pointer_cast<ir::AtenCatLayer>(layer);
    const int64_t out_id = layer->getOutSTensorID()[0];
    if (cat->getMemLayerId() >= 0 && ex.checkValidBlobID(cat->getMemLayerId())) {
        ex.updateBlob(out_id, ir::DataType::TENSOR, ex.findBlob(cat->getMemLayerId()).second);
        return;
    }
    auto& iv = ex.findBlob(layer->getInSTensorID()[0]).second;
    TORCH_CHECK(iv.isTensorList(), "aten::cat expects a tensor list");
    std::vector<at::Tensor> ts;
    for (const at::Tensor& t : iv.toTensorList()) ts.push_back(t);
    auto cx = context(ex, ex.currentStream());
    at::Tensor out = tensor_ops::cat(cx, ts, cat->getDim());
    publish(ex, cx, layer, out);
}

void executeAtenCopy(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& ex) {
    auto cp = std::static_pointer_cast<ir::AtenCopyLayer>(layer);
    const auto& in = layer->getInSTensorID();
    auto cx = context(ex, ex.currentStream());
    at::Tensor out = tensor_ops::copy_(cx, blobTensor(ex, in[0]), blobTensor(ex, in[1]), cp->non_blocking != 0);
    publish(ex, cx, layer, out);
}

namespace {
// a view of a pre-allocated blob (the in-place "custom cat"), or an undefined tensor (= allocate)
at::Tensor aliasOf(StreamExecutor& ex, const ir::OutputAlias& al, at::IntArrayRef sizes) {
    if (al.blob_id < 0 || !ex.checkValidBlobID(al.blob_id)) return {};
    at::Tensor buf = ex.findBlob(al.blob_id).second.toTensor();
    int64_t n = 1;
    for (auto s : sizes) n *= s;
    TORCH_CHECK(al.elem_offset + n <= buf.numel(), "aliased LSTM output does not fit its buffer");
    return buf.view({-1}).narrow(0, al.elem_offset, n).view(sizes);
}
}  // namespace

// aten::lstm, padded input: inputs = (input, hx TensorList [h0, c0]); params and flags live on the layer.
// Publishes (output, h_n, c_n).  Outputs may be slices of pre-allocated blobs (the in-place custom cat).
void executeAtenLSTM1(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& ex) {
    auto lstm = std::static_pointer_cast<ir::AtenLSTM1Layer>(layer);
    const auto& in = layer->getInSTensorID();
    const auto& outs = layer->getOutSTensorID();
    at::Tensor input = blobTensor(ex, in[0]);
    auto& hx_iv = ex.findBlob(in[1]).second;
    TORCH_CHECK(hx_iv.isTensorList(), "aten::lstm expects hx as a tensor list");
    auto hx = hx_iv.toTensorList();
    TORCH_CHECK(hx.size() == 2, "aten::lstm expects hx = [h0, c0]");
    at::Tensor h0 = hx.get(0), c0 = hx.get(1);
    TORCH_CHECK(input.dim() == 3 && h0.dim() == 3, "aten::lstm: rank-3 input and state expected");
    const bool bf = lstm->getBatchFirst() != 0;
    const int64_t T = bf ? input.size(1) : input.size(0), B = bf ? input.size(0) : input.size(1);
    const int64_t H = h0.size(2), D = lstm->getBidirectional() ? 2 : 1, LD = h0.size(0);
    tensor_ops::LstmResult pre;
    pre.y = aliasOf(ex, lstm->out_alias[0], bf ? std::vector<int64_t>{B, T, D * H} : std::vector<int64_t>{T, B, D * H});
    pre.hn = aliasOf(ex, lstm->out_alias[1], {LD, B, H});
    pre.cn = aliasOf(ex, lstm->out_alias[2], {LD, B, H});
    auto cx = context(ex, ex.currentStream());
    auto r = tensor_ops::lstm(cx, lstm->getPackedHandle(), input, h0, c0, bf, lstm->getBidirectional() != 0, pre);
    ex.setStatus(cx.status);
    ex.updateBlob(outs[0], ir::DataType::TENSOR, torch::jit::IValue(r.y));
    ex.updateBlob(outs[1], ir::DataType::TENSOR, torch::jit::IValue(r.hn));
    ex.updateBlob(outs[2], ir::DataType::TENSOR, torch::jit::IValue(r.cn));
}

// aten::lstm, packed sequence: inputs = (data, batch_sizes (CPU int64), hx TensorList)
void executeAtenLSTM2(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& ex) {
    auto lstm = std::static_pointer_cast<ir::AtenLSTM1Layer>(layer);
    const auto& in = layer->getInSTensorID();
    const auto& outs = layer->getOutSTensorID();
    auto hx = ex.findBlob(in[2]).second.toTensorList();
    auto cx = context(ex, ex.currentStream());
    auto r = tensor_ops::lstmPacked(cx, lstm->getPackedHandle(), blobTensor(ex, in[0]), blobTensor(ex, in[1]), hx.get(0),
                                    hx.get(1), lstm->getBidirectional() != 0);
    ex.setStatus(cx.status);
    ex.updateBlob(outs[0], ir::DataType::TENSOR, torch::jit::IValue(r.y));
    ex.updateBlob(outs[1], ir::DataType::TENSOR, torch::jit::IValue(r.hn));
    ex.updateBlob(outs[2], ir::DataType::TENSOR, torch::jit::IValue(r.cn));
}

// MULTISTREAM: the node's addmm/matmul layers are independent; each runs on a side stream of libtorch's pool, made
// the current stream for the duration of the sub-layer, so that every temporary the sub-layer makes (contiguous copies,
// transposes, the output) is allocated and written on that stream.  The side streams start after the work already
// queued on the main stream, the main stream waits for all of them, and the outputs are marked as used by the main
// stream for the caching allocator.  The cursor then skips the copies of those layers that follow the node in the
// flat list.  Events are kept by the executor and reused across calls.
// When every branch is a matrix-class fp16 product (alpha = beta = 1) the node is ONE grouped launch on the main stream.
static bool multiStreamGrouped(std::shared_ptr<ir::MultiStreamLayer>& ms, StreamExecutor& ex) {
    std::vector<tensor_ops::MatmulBranch> branches;
    for (auto sub : ms->getLayers()) {
        const auto& in = sub->getInSTensorID();
        tensor_ops::MatmulBranch br;
        if (sub->getType() == ir::LayerType::ATENADDMM) {
            auto addmm = std::static_pointer_cast<ir::AtenAddmmLayer>(sub);
            if (addmm->beta != 1.0 || addmm->alpha != 1.0) return false;
            br.relu = addmm->getActType() == "aten::relu";
            br.bias = blobTensor(ex, in[0]);
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
    auto cx = context(ex, ex.currentStream());
    auto outs = tensor_ops::groupedMatmul(cx, branches);
    if (outs.empty()) {
        if (cx.status != 0) ex.setStatus(cx.status);
        return false;
    }
    size_t i = 0;
    for (auto sub : ms->getLayers()) publish(ex, cx, sub, outs[i++]);
    return true;
}

void executeMultiStream(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& ex) {
    auto ms = std::static_pointer_cast<ir::MultiStreamLayer>(layer);
    if (multiStreamGrouped(ms, ex)) {
        ex.setCursor(ex.getCursor() + 1 + ms->getLayerNum());
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
            auto& iv = ex.findBlob(id).second;
            if (iv.isTensor() && iv.toTensor().is_cuda()) c10::cuda::CUDACachingAllocator::recordStream(iv.toTensor().storage().data_ptr(), main);
        }
        at::cuda::CUDAEvent& join = ex.event(1 + i);
        join.record(side);
        join.block(main);
        ++i;
    }
    ex.setCursor(ex.getCursor() + 1 + ms->getLayerNum());
}

}  // namespace op_executor
}  // namespace runtime
}  // namespace nn_compiler
