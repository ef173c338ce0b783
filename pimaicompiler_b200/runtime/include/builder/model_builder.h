// Weight preload of the runtime, written against the reference's IR (compiled with the reference tree on the include
// path).  Same class and method names as the reference's runtime/include/builder/model_builder.h and the same
// protocol: constants of lstm / linear / conv / batch-norm / layer-norm nodes are moved to the device once and
// registered as blobs above the largest STensor id (runtime/source/builder/model_builder.cpp:18-120); LSTM layers
// get their ordered parameter vector (:158-224).  The MIOpen flat-weight repacking of the reference (:226-319) is
// replaced by the packing step of the pimb200 library: the handle is kept in a table of this builder keyed by layer
// id, and the layer's arranged-weight slot (an at::Tensor in the reference's class) receives a one-element int64
// tensor carrying that key, so the reference's layer classes stay untouched.
#pragma once
#include <torch/script.h>

#include <map>
#include <memory>
#include <unordered_map>
#include <vector>

#include "common/include/types.hpp"
#include "ir/include/layers/all_layers.h"
#include "ir/include/nn_model.h"
#include "ir/include/types.h"

struct pimb200_lstm;

namespace nn_compiler {
namespace runtime {

using nn_compiler::ir::DataType;

class ModelBuilder {
   public:
    using data_store_type = std::unordered_map<int64_t, std::pair<DataType, torch::jit::IValue>>;   // blob id -> (type, value)

    ModelBuilder() = default;
    ~ModelBuilder();

    RetVal preProcess(std::unique_ptr<nn_compiler::ir::NNModel>& model);
    RetVal preloadModel(std::unique_ptr<nn_compiler::ir::NNModel>& model);

    // moves the constants to the device, registers them as blobs; returns (weight blob ids, bias blob ids)
    std::pair<std::vector<int64_t>, std::vector<int64_t>> loadWeightAndBias(const std::vector<at::Tensor>& weights,
                                                                            const std::vector<at::Tensor>& biases);
    bool feasibleForLstmWeightProcess(std::shared_ptr<nn_compiler::ir::NNLayer>& layer);
    RetVal buildLstmParameterVector(std::shared_ptr<nn_compiler::ir::NNLayer>& layer);
    // the B200 counterpart of reArangeLstmWeights: one packed-weight handle per LSTM layer
    RetVal reArangeLstmWeights(std::shared_ptr<nn_compiler::ir::NNLayer>& layer);

    data_store_type getPreLoadedData() { return preloaded_; }
    // packed-weight handle of an LSTM layer (NULL when the layer was not packed)
    pimb200_lstm* getLstmHandle(uint32_t layer_id) const;
    const std::map<uint32_t, pimb200_lstm*>& getLstmHandles() const { return lstm_handles_; }

   private:
    int64_t next_preload_id_ = 0;
    data_store_type preloaded_;
    std::map<uint32_t, pimb200_lstm*> lstm_handles_;
};

}  // namespace runtime
}  // namespace nn_compiler
