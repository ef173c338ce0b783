// Weight preload (see builder/model_builder.h).
#include "builder/model_builder.h"

#include <glog/logging.h>

#include "ir/include/common/utils.hpp"
#include "pimb200.h"
#include "tensor_ops.h"

namespace nn_compiler {
namespace runtime {

namespace {
// weights, biases and flags of the two aten::lstm layer classes behind one view
struct LstmView {
    std::vector<at::Tensor> weights, biases;
    std::vector<int64_t> weight_ids, bias_ids;
    int has_biases = 0, train = 0, bidirectional = 0, batch_first = 0;
    int64_t num_layers = 0;
    double dropout = 0.0;
    bool padded = true;
};
bool viewOf(const std::shared_ptr<ir::NNLayer>& layer, LstmView* v) {
    if (layer->getType() == ir::LayerType::ATENLSTM1) {
        auto l = std::dynamic_pointer_cast<ir::AtenLSTM1Layer>(layer);
        *v = {l->getWeights(), l->getBiases(), l->getWeightIds(), l->getBiasIds(), l->getHasBiases(), l->getTrain(),
              l->getBidirectional(), l->getBatchFirst(), l->getNumLayers(), l->getDropout(), true};
        return true;
    }
    if (layer->getType() == ir::LayerType::ATENLSTM2) {
        auto l = std::dynamic_pointer_cast<ir::AtenLSTM2Layer>(layer);
        *v = {l->getWeights(), l->getBiases(), l->getWeightIds(), l->getBiasIds(), l->getHasBiases(), l->getTrain(),
              l->getBidirectional(), 0, l->getNumLayers(), l->getDropout(), false};
        return true;
    }
    return false;
}
}  // namespace

ModelBuilder::~ModelBuilder() {
    for (auto& kv : lstm_handles_) pimb200_lstm_destroy(kv.second);
}

RetVal ModelBuilder::preProcess(std::unique_ptr<nn_compiler::ir::NNModel>& model) {
    // preloaded constants get blob ids above every STensor id of the graph
    auto graph = model->getGraphs()[0];
    for (auto layer : graph->getLayers())
        for (auto id : layer->getOutSTensorID()) next_preload_id_ = std::max<int64_t>(next_preload_id_, id);
    ++next_preload_id_;
    return RetVal::SUCCESS;
}

std::pair<std::vector<int64_t>, std::vector<int64_t>> ModelBuilder::loadWeightAndBias(const std::vector<at::Tensor>& weight_data,
                                                                                      const std::vector<at::Tensor>& bias_data) {
    auto load = [&](const std::vector<at::Tensor>& src) {
        std::vector<int64_t> ids;
        for (const auto& t : src) {
            const int64_t id = next_preload_id_++;
            preloaded_.insert({id, {DataType::TENSOR, torch::jit::IValue(t.cuda())}});
            ids.push_back(id);
        }
        return ids;
    };
    auto w = load(weight_data);
    auto b = load(bias_data);
    return {w, b};
}

RetVal ModelBuilder::preloadModel(std::unique_ptr<nn_compiler::ir::NNModel>& model) {
    auto graph = model->getGraphs()[0];
    for (auto layer : graph->getLayers()) {
        switch (layer->getType()) {
            case ir::LayerType::ATENLSTM1: {
                auto l = std::dynamic_pointer_cast<ir::AtenLSTM1Layer>(layer);
                auto ids = loadWeightAndBias(l->getWeights(), l->getBiases());
                l->setWeightIds(ids.first);
                l->setBiasIds(ids.second);
                break;
            }
            case ir::LayerType::ATENLSTM2: {
                auto l = std::dynamic_pointer_cast<ir::AtenLSTM2Layer>(layer);
                auto ids = loadWeightAndBias(l->getWeights(), l->getBiases());
                l->setWeightIds(ids.first);
                l->setBiasIds(ids.second);
                break;
            }
            case ir::LayerType::ATENCONV2D: {
                auto l = std::dynamic_pointer_cast<ir::AtenConv2dLayer>(layer);
                auto ids = loadWeightAndBias(l->getWeights(), l->getBiases());
                l->setWeightIds(ids.first);
                l->setBiasIds(ids.second);
                break;
            }
            case ir::LayerType::ATENBATCHNORM2D: {
                auto l = std::dynamic_pointer_cast<ir::AtenBatchNorm2dLayer>(layer);
                auto ids = loadWeightAndBias(l->getWeights(), l->getBiases());
                l->setWeightIds(ids.first);
                l->setBiasIds(ids.second);
                break;
            }
            case ir::LayerType::ATENLINEAR: {
                auto l = std::dynamic_pointer_cast<ir::AtenLinearLayer>(layer);
                auto ids = loadWeightAndBias(l->getWeights(), l->getBiases());
                l->setWeightIds(ids.first);
                l->setBiasIds(ids.second);
                break;
            }
            case ir::LayerType::ATENLAYERNORM: {
                auto l = std::dynamic_pointer_cast<ir::AtenLayerNormLayer>(layer);
                auto ids = loadWeightAndBias(l->getWeights(), l->getBiases());
                l->setWeightIds(ids.first);
                l->setBiasIds(ids.second);
                break;
            }
            default: continue;
        }
        if (layer->getType() == ir::LayerType::ATENLSTM1 || layer->getType() == ir::LayerType::ATENLSTM2) {
            if (!feasibleForLstmWeightProcess(layer)) {
                LOG(ERROR) << "aten::lstm layer " << layer->getName() << " keeps its flags as graph inputs: weights not packed";
                return RetVal::FAILURE;
            }
            if (buildLstmParameterVector(layer) != RetVal::SUCCESS || reArangeLstmWeights(layer) != RetVal::SUCCESS)
                return RetVal::FAILURE;
        }
    }
    return RetVal::SUCCESS;
}

// the flags of the layer must have been folded in by the SetAttribute pass (none may still hold its "default value"
// sentinel): the packed layout depends on them
bool ModelBuilder::feasibleForLstmWeightProcess(std::shared_ptr<nn_compiler::ir::NNLayer>& layer) {
    LstmView v;
    if (!viewOf(layer, &v)) return false;
    bool ok = !ir::isDefaultValue(v.has_biases) && !ir::isDefaultValue(v.num_layers) && !ir::isDefaultValue(v.dropout) &&
              !ir::isDefaultValue(v.train) && !ir::isDefaultValue(v.bidirectional);
    if (v.padded) ok = ok && !ir::isDefaultValue(v.batch_first);
    return ok;
}

// at::lstm's flat parameter order: (w_ih, w_hh, b_ih?, b_hh?) per direction per layer, from the preloaded blobs
RetVal ModelBuilder::buildLstmParameterVector(std::shared_ptr<nn_compiler::ir::NNLayer>& layer) {
    LstmView v;
    if (!viewOf(layer, &v)) return RetVal::FAILURE;
    const int64_t cells = v.num_layers * (v.bidirectional ? 2 : 1);
    if ((int64_t)v.weight_ids.size() < 2 * cells || (v.has_biases && (int64_t)v.bias_ids.size() < 2 * cells)) {
        LOG(ERROR) << "aten::lstm layer " << layer->getName() << ": " << v.weight_ids.size() << " weight and " << v.bias_ids.size()
                   << " bias constants for " << cells << " cells";
        return RetVal::FAILURE;
    }
    std::vector<at::Tensor> params;
    auto blob = [&](int64_t id) { return preloaded_.at(id).second.toTensor(); };
    for (int64_t i = 0; i < cells; ++i) {
        params.push_back(blob(v.weight_ids[2 * i]));
        params.push_back(blob(v.weight_ids[2 * i + 1]));
        if (v.has_biases) {
            params.push_back(blob(v.bias_ids[2 * i]));
            params.push_back(blob(v.bias_ids[2 * i + 1]));
        }
    }
    if (v.padded) std::dynamic_pointer_cast<ir::AtenLSTM1Layer>(layer)->setParamVector(params);
    else std::dynamic_pointer_cast<ir::AtenLSTM2Layer>(layer)->setParamVector(params);
    return RetVal::SUCCESS;
}

RetVal ModelBuilder::reArangeLstmWeights(std::shared_ptr<nn_compiler::ir::NNLayer>& layer) {
    LstmView v;
    if (!viewOf(layer, &v)) return RetVal::FAILURE;
    std::vector<at::Tensor> params = v.padded ? std::dynamic_pointer_cast<ir::AtenLSTM1Layer>(layer)->getParamVector()
                                              : std::dynamic_pointer_cast<ir::AtenLSTM2Layer>(layer)->getParamVector();
    for (auto& p : params) p = p.to(at::kHalf).contiguous();   // fp16 storage is what the device path computes on
    tensor_ops::OpContext cx;
    pimb200_lstm* h = tensor_ops::lstmPack(cx, params, v.num_layers, v.bidirectional != 0, v.has_biases != 0);
    if (!h || cx.status != PIMB200_OK) {
        LOG(ERROR) << "aten::lstm layer " << layer->getName() << ": packing failed: " << pimb200_status_string(cx.status);
        return RetVal::FAILURE;
    }
    lstm_handles_[layer->getID()] = h;
    // the layer's arranged-weight slot carries the key of the handle table
    at::Tensor key = at::full({1}, (int64_t)layer->getID(), at::TensorOptions().dtype(at::kLong));
    if (v.padded) std::dynamic_pointer_cast<ir::AtenLSTM1Layer>(layer)->setArrangedWeight(key);
    else std::dynamic_pointer_cast<ir::AtenLSTM2Layer>(layer)->setArrangedWeight(key);
    return RetVal::SUCCESS;
}

pimb200_lstm* ModelBuilder::getLstmHandle(uint32_t layer_id) const {
    auto it = lstm_handles_.find(layer_id);
    return it == lstm_handles_.end() ? nullptr : it->second;
}

}  // namespace runtime
}  // namespace nn_compiler
