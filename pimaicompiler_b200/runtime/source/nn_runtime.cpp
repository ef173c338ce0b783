// NNRuntime (see nn_runtime.h).
#include "nn_runtime.h"

#include <glog/logging.h>

#include "pimb200.h"

namespace nn_compiler {
namespace runtime {

NNRuntime::NNRuntime(std::unique_ptr<nn_compiler::ir::NNModel>& model, std::string model_type) : family_(std::move(model_type)) {
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) pimb200_init(dev);   // stands where PimInitialize and the rocBLAS warm-up were
    builder_ = std::make_shared<ModelBuilder>();
    last_ = builder_->preProcess(model);
    if (last_ == RetVal::SUCCESS) last_ = builder_->preloadModel(model);
    interpreter_ = std::make_shared<StreamExecutor>(std::make_pair(model->getGraphs()[0], builder_->getPreLoadedData()), family_);
    interpreter_->setLstmHandles(builder_->getLstmHandles());
    if (last_ == RetVal::SUCCESS) last_ = interpreter_->preProcess();
}

NNRuntime::~NNRuntime() = default;

void NNRuntime::setProfilePath(const std::string& path) { interpreter_->setProfilePath(path); }

void NNRuntime::inferenceModel(const std::vector<torch::Tensor>& input_tensors, std::vector<torch::Tensor>& output_tensors,
                               bool profiling) {
    if (last_ != RetVal::SUCCESS && !interpreter_) return;
    if (profiling) {
        // as the reference does (runtime/source/nn_runtime.cpp:44-53): untimed runs first, then the profiled one
        for (int i = 0; i < 3; ++i) {
            std::vector<torch::Tensor> scratch;
            last_ = interpreter_->inferenceModel(input_tensors, scratch);
            if (last_ != RetVal::SUCCESS) break;
        }
        if (last_ == RetVal::SUCCESS) last_ = interpreter_->inferenceModelwithProfiling(input_tensors, output_tensors);
    } else {
        last_ = interpreter_->inferenceModel(input_tensors, output_tensors);
    }
    if (last_ != RetVal::SUCCESS) LOG(ERROR) << "inference failed";
}

}  // namespace runtime
}  // namespace nn_compiler
