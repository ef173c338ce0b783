// Host-side mirror of the reference's stream executor for the hot path: op executors registered by
// ir::LayerType (runtime/include/executor/stream_executor.h:28, runtime/source/executor/stream_executor.cpp:433-576),
// the blob store they read and publish through (stream_executor.cpp:260-278), and the interpreter loop that
// calls them (stream_executor.cpp:136-202).  The backend handles of the reference (hip streams, MIOpen handle and
// descriptors, PIM) are replaced by the pimb200 C ABI; there is a single executor map, no run-time library selection.
#pragma once
#include <ATen/cuda/CUDAEvent.h>
#include <c10/cuda/CUDAStream.h>
#include <cuda_runtime_api.h>

#include <functional>
#include <memory>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

#include "ir_min.h"
#include "tensor_ops.h"

namespace nn_compiler {
namespace runtime {

class StreamExecutor;
using OpExecutorFn = std::function<void(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& stream_executor)>;

// shape classes of the reference's GEMM router (runtime/include/executor/utils/utils.h:30-36)
using tensor_ops::GEMM_TYPE;
using tensor_ops::getGemmType;

class StreamExecutor {
   public:
    typedef std::unordered_map<int64_t, std::pair<ir::DataType, torch::jit::IValue>> blob_store_type;

    StreamExecutor(std::shared_ptr<ir::NNGraph> graph, std::string model_type);
    ~StreamExecutor();

    RetVal preProcess();  // per-layer executor table, LSTM weight packing ("preload")
    RetVal inferenceModel(const std::vector<torch::Tensor>& input_tensors, std::vector<torch::Tensor>& output_tensors);
    // the same run with every op bracketed by CUDA events on the launching stream; the per-op device times are written
    // as a Chrome trace (runtime/include/executor/utils/profiler.h:54-261 is the reference's writer of that format,
    // runtime/source/executor/stream_executor.cpp:204-258 its per-op loop, which synchronises the device after each op)
    RetVal inferenceModelwithProfiling(const std::vector<torch::Tensor>& input_tensors,
                                       std::vector<torch::Tensor>& output_tensors);
    void setProfilePath(std::string path) { profile_path_ = std::move(path); }
    const std::string& getProfilePath() const { return profile_path_; }

    void updateBlob(int64_t blob_id, ir::DataType dtype, const torch::jit::IValue& iv);
    std::pair<ir::DataType, torch::jit::IValue>& findBlob(int64_t blob_id);
    bool checkValidBlobID(int64_t blob_id);

    void registerOp();
    OpExecutorFn findAtenExecutorByType(ir::LayerType op_type);
    OpExecutorFn getOpExecutor(uint32_t id);

    void setCursor(int64_t c) { cursor_ = c; }
    int64_t getCursor() const { return cursor_; }
    const std::string& getModelType() const { return model_type_; }

    // status of the last C-ABI call an executor made; inferenceModel turns a non-zero value into RetVal::FAILURE
    void setStatus(int s) { if (s != 0 && status_ == 0) status_ = s; }
    int getStatus() const { return status_; }

    cudaStream_t currentStream() const;             // the stream executors launch on (libtorch's current stream)
    c10::cuda::CUDAStream sideStream(size_t i);     // side streams for MULTISTREAM, from libtorch's pool
    at::cuda::CUDAEvent& event(size_t i);           // events kept across calls (no create / destroy per op)

   private:
    std::shared_ptr<ir::NNGraph> graph_;
    std::string model_type_;
    blob_store_type global_blobs_;
    std::unordered_map<int, OpExecutorFn> aten_executor_map_;
    std::vector<OpExecutorFn> op_executor_;
    std::vector<c10::cuda::CUDAStream> streams_;
    std::vector<std::unique_ptr<at::cuda::CUDAEvent>> events_;
    int64_t cursor_ = 0;
    int status_ = 0;
    std::string profile_path_ = "pimb200_profile.json";
    RetVal run(const std::vector<torch::Tensor>& input_tensors, std::vector<torch::Tensor>& output_tensors, bool profiling);
    RetVal checkDeviceStatus();   // synchronises and reads the status words of the kernels with bounded waits
};

// NNRuntime(model, model_type) / inferenceModel(inputs, outputs, profiling) — runtime/include/nn_runtime.h:22-44
class NNRuntime {
   public:
    NNRuntime(std::shared_ptr<ir::NNGraph> graph, std::string model_type = "");
    ~NNRuntime();
    void inferenceModel(const std::vector<torch::Tensor>& input_tensors, std::vector<torch::Tensor>& output_tensors,
                        bool profiling = false);
    RetVal lastResult() const { return last_; }
    void setProfilePath(const std::string& path);   // where inferenceModel(..., profiling = true) writes its Chrome trace

   private:
    std::unique_ptr<StreamExecutor> executor_;
    RetVal last_ = RetVal::SUCCESS;
};

namespace op_executor {
void executeAtenAdd(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& stream_executor);
void executeAtenAddmm(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& stream_executor);
void executeAtenAddmmWithStream(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& stream_executor, void* stream);
void executeAtenBmm(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& stream_executor);
void executeAtenSoftmax(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& stream_executor);   // also log_softmax
void executeAtenArgmax(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& stream_executor);
void executeAtenLayerNorm(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& stream_executor);
void executeAtenTanh(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& stream_executor);
void executeAtenMaskedFill(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& stream_executor);
void executeAtenEmbedding(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& stream_executor);
void executeAtenCat(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& stream_executor);
void executeAtenCopy(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& stream_executor);
void executeAtenLinear(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& stream_executor);
void executeAtenLSTM1(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& stream_executor);
void executeAtenLSTM2(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& stream_executor);
void executeAtenMatmul(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& stream_executor);
void executeAtenMatmulWithStream(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& stream_executor, void* stream);
void executeMultiStream(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& stream_executor);
}  // namespace op_executor

}  // namespace runtime
}  // namespace nn_compiler
