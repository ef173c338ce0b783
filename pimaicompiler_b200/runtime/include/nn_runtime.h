// NNRuntime(model, model_type) / inferenceModel(inputs, outputs, profiling): the runtime API of the reference
// (runtime/include/nn_runtime.h:22-44) over the B200 executor set.  The rocBLAS warm-up and the PIM library
// start-up / shut-down of the reference (runtime/source/nn_runtime.cpp:32-33, 62-73, 85) are replaced by
// pimb200_init for the current device.
#pragma once

#include "builder/model_builder.h"
#include "executor/stream_executor.h"
#include "ir/include/nn_model.h"

namespace nn_compiler {
namespace runtime {

class NNRuntime {
   public:
    NNRuntime() {}
    NNRuntime(std::unique_ptr<nn_compiler::ir::NNModel>& model, std::string model_type = "");
    ~NNRuntime();

    void inferenceModel(const std::vector<torch::Tensor>& input_tensors, std::vector<torch::Tensor>& output_tensors,
                        bool profiling = false);
    // result of the last inferenceModel / of construction (the reference only logs a failure)
    RetVal lastResult() const { return last_; }
    void setProfilePath(const std::string& path);

   private:
    std::shared_ptr<ModelBuilder> builder_ = nullptr;
    std::shared_ptr<StreamExecutor> interpreter_ = nullptr;
    std::string family_ = "";
    RetVal last_ = RetVal::SUCCESS;
};

}  // namespace runtime
}  // namespace nn_compiler
