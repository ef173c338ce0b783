// Stream executor of the runtime, written against the reference's IR (compiled with the reference tree on the include
// path).  Class, method and member meaning follow runtime/include/executor/stream_executor.h of the reference: op
// executors are std::functions registered per ir::LayerType (registerOp), looked up per layer id (preProcess), and
// called by a program-counter loop over the flat layer list in which control ops move the cursor themselves
// (inferenceModel).  What the reference keeps for its device libraries (hip streams, MIOpen handle and descriptors,
// the per-layer MIOpen-vs-ATen timing selection) has no counterpart here: every hot op has one executor, over the
// pimb200 C ABI; the stream an executor launches on is libtorch's current CUDA stream.
#pragma once
#include <ATen/cuda/CUDAEvent.h>
#include <c10/cuda/CUDAStream.h>
#include <cuda_runtime_api.h>
#include <torch/script.h>

#include <functional>
#include <memory>
#include <mutex>
#include <set>
#include <stack>
#include <string>
#include <unordered_map>
#include <vector>

#include "builder/model_builder.h"

namespace nn_compiler {
namespace runtime {

class StreamExecutor;
using OpExecutorFn = std::function<void(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& stream_executor)>;

class StreamExecutor {
   public:
    typedef std::unordered_map<int64_t, std::pair<ir::DataType, torch::jit::IValue>> blob_store_type;

    StreamExecutor(std::pair<std::shared_ptr<ir::NNGraph>, blob_store_type> model, std::string model_type);
    ~StreamExecutor();

    RetVal preProcess();
    RetVal inferenceModel(const std::vector<torch::Tensor>& input_tensors, std::vector<torch::Tensor>& output_tensors);
    // the same run with every op bracketed by CUDA events on the launching stream, written as a Chrome trace
    RetVal inferenceModelwithProfiling(const std::vector<torch::Tensor>& input_tensors,
                                       std::vector<torch::Tensor>& output_tensors);

    void updateBlob(int64_t blob_id, ir::DataType dtype, const torch::jit::IValue& iv);
    std::pair<ir::DataType, torch::jit::IValue>& findBlob(int64_t blob_id);
    bool checkValidBlobID(int64_t blob_id);

    OpExecutorFn findAtenExecutorByType(ir::LayerType& op_type);
    OpExecutorFn getOpExecutor(uint32_t& id);
    void registerOp();

    void setInputTensors(const std::vector<torch::Tensor>& input_tensors);
    void getOutputTensors(std::vector<torch::Tensor>& output_tensors);
    const std::shared_ptr<ir::NNGraph> getGraph();
    std::vector<torch::Tensor> iValueParser(torch::jit::IValue& iv);

    void setCursor(int64_t cursor) { pc_ = cursor; }
    int64_t getCursor() const { return pc_; }

    void pushInLoopConditionStack(int64_t id) { loop_conditions_.push(id); }
    int64_t getTopOfLoopConditionStack() { return loop_conditions_.top(); }
    void popOfLoopConditionStack() { loop_conditions_.pop(); }

    void setModelType(const std::string& model_type) { family_ = model_type; }
    const std::string& getModelType() const { return family_; }

    // ---- what replaces the reference's device-library members ----
    cudaStream_t currentStream() const;             // libtorch's current stream: every executor launches there
    c10::cuda::CUDAStream sideStream(size_t i);     // side streams of MULTISTREAM, from libtorch's pool
    at::cuda::CUDAEvent& event(size_t i);           // events kept across calls
    void setLstmHandles(const std::map<uint32_t, pimb200_lstm*>& handles) { lstm_handles_ = handles; }
    pimb200_lstm* lstmHandle(uint32_t layer_id) const;
    // first non-zero status an executor's C-ABI call returned in this run; turns the run into RetVal::FAILURE
    void setStatus(int s) { if (s != 0 && status_ == 0) status_ = s; }
    int getStatus() const { return status_; }
    void setProfilePath(std::string path) { profile_path_ = std::move(path); }

   private:
    RetVal run(const std::vector<torch::Tensor>& input_tensors, std::vector<torch::Tensor>& output_tensors, bool profiling);
    RetVal checkDeviceStatus();

    std::shared_ptr<ir::NNGraph> program_;
    std::unordered_map<uint32_t, OpExecutorFn> dispatch_;
    std::unordered_map<int, OpExecutorFn> by_type_;   // keyed by ir::LayerType
    int64_t pc_ = 0;                                            // position of the layer being interpreted (control ops move it)
    blob_store_type blobs_;
    std::vector<int64_t> graph_inputs_;
    std::vector<int64_t> graph_outputs_;
    std::stack<int64_t> loop_conditions_;
    std::string family_ = "";
    std::vector<c10::cuda::CUDAStream> streams_;
    std::vector<std::unique_ptr<at::cuda::CUDAEvent>> events_;
    std::map<uint32_t, pimb200_lstm*> lstm_handles_;
    int status_ = 0;
    std::string profile_path_ = "pimb200_profile.json";
    static std::mutex gather_mutex_;   // multi-GPU replicas: guards the copy of results to cuda:0
};

}  // namespace runtime
}  // namespace nn_compiler
