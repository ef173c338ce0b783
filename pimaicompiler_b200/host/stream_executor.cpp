// Registry, blob store, interpreter loop and the GEMM shape classifier of the host-side mirror.
#include "stream_executor.h"

#include <ATen/cuda/CUDAContext.h>

#include <cstdio>

#include "pimb200.h"

namespace nn_compiler {
namespace ir {
AtenLSTM1Layer::~AtenLSTM1Layer() {
    if (packed_) pimb200_lstm_destroy(packed_);
}
}  // namespace ir

namespace runtime {

StreamExecutor::StreamExecutor(std::shared_ptr<ir::NNGraph> graph, std::string model_type)
    : graph_(std::move(graph)), model_type_(std::move(model_type)) {
    registerOp();
}

StreamExecutor::~StreamExecutor() = default;

void StreamExecutor::registerOp() {
    using namespace op_executor;
    auto reg = [&](ir::LayerType t, OpExecutorFn fn) { aten_executor_map_[(int)t] = std::move(fn); };
    reg(ir::LayerType::ATENADD, executeAtenAdd);
    reg(ir::LayerType::ATENADDMM, executeAtenAddmm);
    reg(ir::LayerType::ATENBMM, executeAtenBmm);
    reg(ir::LayerType::ATENCAT, executeAtenCat);
    reg(ir::LayerType::ATENCOPY, executeAtenCopy);
    reg(ir::LayerType::ATENLINEAR, executeAtenLinear);
    reg(ir::LayerType::ATENLSTM1, executeAtenLSTM1);
    reg(ir::LayerType::ATENLSTM2, executeAtenLSTM2);
    reg(ir::LayerType::ATENMATMUL, executeAtenMatmul);
    reg(ir::LayerType::MULTISTREAM, executeMultiStream);
    reg(ir::LayerType::ATENSOFTMAX, executeAtenSoftmax);
    reg(ir::LayerType::ATENLOGSOFTMAX, executeAtenSoftmax);
    reg(ir::LayerType::ATENARGMAX, executeAtenArgmax);
    reg(ir::LayerType::ATENLAYERNORM, executeAtenLayerNorm);
    reg(ir::LayerType::ATENTANH, executeAtenTanh);
    reg(ir::LayerType::ATENMASKEDFILL, executeAtenMaskedFill);
    reg(ir::LayerType::ATENEMBEDDING, executeAtenEmbedding);
    // the one prim op graphs on this path cannot do without: gathers tensor blobs into a list blob
    reg(ir::LayerType::PRIMLISTCONSTRUCT, [](std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& ex) {
        c10::List<at::Tensor> l;
        for (auto id : layer->getInSTensorID()) l.push_back(ex.findBlob(id).second.toTensor());
        ex.updateBlob(layer->getOutSTensorID()[0], ir::DataType::LIST, torch::jit::IValue(l));
    });
}

OpExecutorFn StreamExecutor::findAtenExecutorByType(ir::LayerType op_type) {
    auto it = aten_executor_map_.find((int)op_type);
    return it == aten_executor_map_.end() ? OpExecutorFn() : it->second;
}

OpExecutorFn StreamExecutor::getOpExecutor(uint32_t id) {
    return id < op_executor_.size() ? op_executor_[id] : OpExecutorFn();
}

RetVal StreamExecutor::preProcess() {
    op_executor_.clear();
    for (auto& layer : graph_->getLayers()) {
        auto fn = findAtenExecutorByType(layer->getType());
        if (!fn) return RetVal::FAILURE;  // no executor registered for this node type
        op_executor_.push_back(fn);
        // one-time weight layout step of LSTM nodes (the reference does this in ModelBuilder::preloadModel)
        if (layer->getType() == ir::LayerType::ATENLSTM1 || layer->getType() == ir::LayerType::ATENLSTM2) {
            auto lstm = std::static_pointer_cast<ir::AtenLSTM1Layer>(layer);
            if (lstm->getPackedHandle()) continue;
            tensor_ops::OpContext cx;
            pimb200_lstm* h = tensor_ops::lstmPack(cx, lstm->getParamVector(), lstm->getNumLayers(), lstm->getBidirectional() != 0,
                                                   lstm->getHasBiases() != 0);
            if (!h || cx.status != PIMB200_OK) return RetVal::FAILURE;
            lstm->setPackedHandle(h);
        }
    }
    return RetVal::SUCCESS;
}

void StreamExecutor::updateBlob(int64_t blob_id, ir::DataType dtype, const torch::jit::IValue& iv) {
    global_blobs_[blob_id] = std::make_pair(dtype, iv);
}

std::pair<ir::DataType, torch::jit::IValue>& StreamExecutor::findBlob(int64_t blob_id) {
    auto it = global_blobs_.find(blob_id);
    TORCH_CHECK(it != global_blobs_.end(), "blob ", blob_id, " has not been produced");
    return it->second;
}

bool StreamExecutor::checkValidBlobID(int64_t blob_id) { return global_blobs_.find(blob_id) != global_blobs_.end(); }

cudaStream_t StreamExecutor::currentStream() const { return at::cuda::getCurrentCUDAStream().stream(); }

c10::cuda::CUDAStream StreamExecutor::sideStream(size_t i) {
    while (streams_.size() < 4) streams_.push_back(c10::cuda::getStreamFromPool());
    return streams_[i % streams_.size()];
}

at::cuda::CUDAEvent& StreamExecutor::event(size_t i) {
    while (events_.size() <= i) events_.push_back(std::make_unique<at::cuda::CUDAEvent>(cudaEventDefault));   // timing enabled: the profiler reads them
    return *events_[i];
}

RetVal StreamExecutor::inferenceModel(const std::vector<torch::Tensor>& input_tensors,
                                      std::vector<torch::Tensor>& output_tensors) {
    return run(input_tensors, output_tensors, false);
}

RetVal StreamExecutor::inferenceModelwithProfiling(const std::vector<torch::Tensor>& input_tensors,
                                                   std::vector<torch::Tensor>& output_tensors) {
    return run(input_tensors, output_tensors, true);
}

// A kernel whose bounded wait gave up leaves PIMB200_ERR_TIMEOUT in a device status word; outputs of such a run are
// undefined, so the run is reported as failed.
RetVal StreamExecutor::checkDeviceStatus() {
    if (cudaStreamSynchronize(currentStream()) != cudaSuccess) return RetVal::FAILURE;
    int rc = pimb200_gemm_last_status();
    for (auto& layer : graph_->getLayers()) {
        if (layer->getType() != ir::LayerType::ATENLSTM1 && layer->getType() != ir::LayerType::ATENLSTM2) continue;
        auto lstm = std::static_pointer_cast<ir::AtenLSTM1Layer>(layer);
        if (lstm->getPackedHandle()) {
            const int s = pimb200_lstm_last_status(lstm->getPackedHandle());
            if (rc == PIMB200_OK) rc = s;
        }
    }
    setStatus(rc);
    return rc == PIMB200_OK ? RetVal::SUCCESS : RetVal::FAILURE;
}

RetVal StreamExecutor::run(const std::vector<torch::Tensor>& input_tensors, std::vector<torch::Tensor>& output_tensors,
                           bool profiling) {
    if (input_tensors.size() != graph_->input_ids.size()) return RetVal::FAILURE;
    if (op_executor_.size() != graph_->getLayers().size() && preProcess() != RetVal::SUCCESS) return RetVal::FAILURE;
    status_ = 0;
    for (auto& pb : graph_->preset_blobs)
        if (!checkValidBlobID(pb.first)) updateBlob(pb.first, ir::DataType::TENSOR, torch::jit::IValue(pb.second));
    for (size_t i = 0; i < input_tensors.size(); ++i)
        updateBlob(graph_->input_ids[i], ir::DataType::TENSOR, torch::jit::IValue(input_tensors[i]));
    const auto& layers = graph_->getLayers();
    struct Span { std::string name; size_t e0, e1; };
    std::vector<Span> spans;
    size_t next_event = 16;   // events 0..15 belong to MULTISTREAM
    for (cursor_ = 0; cursor_ < (int64_t)layers.size();) {
        auto layer = layers[cursor_];
        const int64_t before = cursor_;
        if (profiling) {
            event(next_event).record(c10::cuda::getCurrentCUDAStream());
            op_executor_[cursor_](layer, *this);
            event(next_event + 1).record(c10::cuda::getCurrentCUDAStream());
            spans.push_back({layer->getName(), next_event, next_event + 1});
            next_event += 2;
        } else {
            op_executor_[cursor_](layer, *this);
        }
        if (status_ != 0) return RetVal::FAILURE;
        if (cursor_ == before) ++cursor_;  // executors that jump (MULTISTREAM) set the cursor themselves
    }
    if (checkDeviceStatus() != RetVal::SUCCESS) return RetVal::FAILURE;
    if (profiling) {
        // Chrome trace ("traceEvents" of complete events, microseconds): one span per op, laid end to end on the
        // device timeline of the launching stream
        FILE* f = std::fopen(profile_path_.c_str(), "w");
        if (f) {
            std::fprintf(f, "{\"otherData\": {}, \"traceEvents\": [");
            double t0 = 0.0;
            for (size_t i = 0; i < spans.size(); ++i) {
                const double start_us = i == 0 ? 0.0 : 1e3 * event(spans[0].e0).elapsed_time(event(spans[i].e0));
                const double dur_us = 1e3 * event(spans[i].e0).elapsed_time(event(spans[i].e1));
                (void)t0;
                std::fprintf(f, "%s{\"cat\": \"function\", \"dur\": %.3f, \"name\": \"%s\", \"ph\": \"X\", \"pid\": 0, "
                                "\"tid\": 0, \"ts\": %.3f}",
                             i ? ", " : "", dur_us, spans[i].name.c_str(), start_us);
            }
            std::fprintf(f, "]}\n");
            std::fclose(f);
        }
    }
    for (auto id : graph_->output_ids) {
        auto& iv = findBlob(id).second;
        if (iv.isTensor()) {
            output_tensors.push_back(iv.toTensor());
        } else if (iv.isTensorList()) {
            for (const at::Tensor& t : iv.toTensorList()) output_tensors.push_back(t);
        } else if (iv.isTuple()) {
            for (auto& e : iv.toTupleRef().elements())
                if (e.isTensor()) output_tensors.push_back(e.toTensor());
        } else {
            return RetVal::FAILURE;
        }
    }
    return RetVal::SUCCESS;
}

NNRuntime::NNRuntime(std::shared_ptr<ir::NNGraph> graph, std::string model_type) {
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) pimb200_init(dev);  // stands where PimInitialize + the rocBLAS warm-up were
    executor_ = std::make_unique<StreamExecutor>(std::move(graph), std::move(model_type));
    last_ = executor_->preProcess();
}

NNRuntime::~NNRuntime() = default;

void NNRuntime::inferenceModel(const std::vector<torch::Tensor>& input_tensors,
                               std::vector<torch::Tensor>& output_tensors, bool profiling) {
    if (!profiling) {
        last_ = executor_->inferenceModel(input_tensors, output_tensors);
        return;
    }
    // as the reference does (runtime/source/nn_runtime.cpp:44-53): a few untimed runs first, then the profiled one
    for (int i = 0; i < 3 && last_ == RetVal::SUCCESS; ++i) {
        std::vector<torch::Tensor> scratch;
        last_ = executor_->inferenceModel(input_tensors, scratch);
    }
    last_ = executor_->inferenceModelwithProfiling(input_tensors, output_tensors);
}

void NNRuntime::setProfilePath(const std::string& path) { executor_->setProfilePath(path); }

}  // namespace runtime
}  // namespace nn_compiler
