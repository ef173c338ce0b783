// PipelineManager(input_file, model_type, gpu_num): compiles a TorchScript file with the reference's compiler and runs
// it through NNRuntime — the class the reference's pybind module exposes (runtime/python/nn_runtime_py.cpp:18-25,
// runtime/python/pipeline_manager/pipeline_manager.{h,cpp}).  With gpu_num > 1 every GPU gets a runtime of its own on a
// worker thread (one replica per device, each with its own copy of the weights); the inputs are split along
// dimension 0 and the replicas' results are concatenated in input order.
#pragma once
#include <torch/script.h>

#include <condition_variable>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "compiler/include/nn_compiler.hpp"
#include "ir/include/nn_model.h"
#include "nn_runtime.h"

namespace NNRuntimeInterface {

class PipelineManager {
   public:
    PipelineManager(const std::string& input_file_path, std::string model_type, int gpu_num = 1, bool profiling = false);
    ~PipelineManager();
    std::vector<torch::Tensor> inferenceModel(const std::vector<torch::Tensor>& input_tensors);
    void setProfilePath(const std::string& path);

   private:
    struct Replica {
        int device = 0;
        std::thread thread;
        std::mutex mu;
        std::condition_variable cv;
        bool has_work = false, done = false, stop = false, failed = false;
        std::string error;
        std::vector<torch::Tensor> inputs, outputs;
    };
    void worker(Replica* r);

    std::string input_file_path_, family_;
    bool is_profiling_ = false;
    std::shared_ptr<nn_compiler::ir::NNModel> compiled_;                 // shared, read-only after compile
    std::shared_ptr<nn_compiler::runtime::NNRuntime> runtime_;           // gpu_num == 1
    std::vector<std::unique_ptr<Replica>> replicas_;                     // gpu_num > 1
};

}  // namespace NNRuntimeInterface
