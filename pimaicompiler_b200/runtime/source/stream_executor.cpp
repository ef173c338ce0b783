// Registry, blob store and interpreter loop of the runtime (see executor/stream_executor.h).
#include "executor/stream_executor.h"

#include <ATen/cuda/CUDAContext.h>
#include <glog/logging.h>

#include <cstdio>

#include "executor/op_executor/ops_executor.h"
#include "pimb200.h"

namespace nn_compiler {
namespace runtime {

std::mutex StreamExecutor::gather_mutex_;

StreamExecutor::StreamExecutor(std::pair<std::shared_ptr<ir::NNGraph>, blob_store_type> model, std::string model_type)
    : program_(model.first), blobs_(std::move(model.second)), family_(std::move(model_type)) {
    registerOp();
}

StreamExecutor::~StreamExecutor() = default;

void StreamExecutor::registerOp() {
    using namespace op_executor;
    auto reg = [&](ir::LayerType t, OpExecutorFn fn) { by_type_[(int)t] = std::move(fn); };
    // hot path
    reg(ir::LayerType::ATENADD, executeAtenAdd);
    reg(ir::LayerType::ATENADDMM, executeAtenAddmm);
    reg(ir::LayerType::ATENBMM, executeAtenBmm);
    reg(ir::LayerType::ATENCAT, executeAtenCat);
    reg(ir::LayerType::ATENCOPY, executeAtenCopy);
    reg(ir::LayerType::ATENEMBEDDING, executeAtenEmbedding);
    reg(ir::LayerType::ATENLINEAR, executeAtenLinear);
    reg(ir::LayerType::ATENLSTM1, executeAtenLSTM1);
    reg(ir::LayerType::ATENLSTM2, executeAtenLSTM2);
    reg(ir::LayerType::ATENMATMUL, executeAtenMatmul);
    reg(ir::LayerType::ATENSOFTMAX, executeAtenSoftmax);
    reg(ir::LayerType::ATENLOGSOFTMAX, executeAtenLogSoftmax);
    reg(ir::LayerType::ATENARGMAX, executeAtenArgmax);
    reg(ir::LayerType::ATENTOPK, executeAtenTopk);
    reg(ir::LayerType::ATENTANH, executeAtenTanh);
    reg(ir::LayerType::MULTISTREAM, executeMultiStream);
    // pass-through adapters
    reg(ir::LayerType::ATENITEM, executeAtenItem);
    for (auto t : {ir::LayerType::ATENGT, ir::LayerType::ATENLT, ir::LayerType::ATENGE, ir::LayerType::ATENLE,
                   ir::LayerType::ATENEQ, ir::LayerType::ATENNE})
        reg(t, executeAtenCompare);
    reg(ir::LayerType::ATENTRANSPOSE, executeAtenTranspose);
    reg(ir::LayerType::ATENSELECT, executeAtenSelect);
    reg(ir::LayerType::ATENRELU, executeAtenRelu);
    reg(ir::LayerType::ATENSIZE, executeAtenSize);
    reg(ir::LayerType::ATENINT, executeAtenInt);
    reg(ir::LayerType::ATENUNSQUEEZE, executeAtenUnsqueeze);
    // prim ops
    reg(ir::LayerType::PRIMCONSTANT, executePrimConstant);
    reg(ir::LayerType::PRIMVARIABLE, executePrimVariable);
    reg(ir::LayerType::PRIMLISTCONSTRUCT, executePrimListConstruct);
    reg(ir::LayerType::PRIMLISTUNPACK, executePrimListUnpack);
    reg(ir::LayerType::PRIMTUPLECONSTRUCT, executePrimTupleConstruct);
    reg(ir::LayerType::PRIMTUPLEUNPACK, executePrimTupleUnpack);
    reg(ir::LayerType::PRIMTUPLEINDEX, executePrimTupleIndex);
    reg(ir::LayerType::PRIMIF, executePrimIf);
    reg(ir::LayerType::PRIMENDIF, executePrimEndIf);
    reg(ir::LayerType::PRIMLOOP, executePrimLoop);
    reg(ir::LayerType::PRIMLOOPINDEX, executePrimLoopIndex);
    reg(ir::LayerType::PRIMBLOCK, executePrimBlock);
    reg(ir::LayerType::PRIMENDLOOP, executePrimEndLoop);
}

OpExecutorFn StreamExecutor::findAtenExecutorByType(ir::LayerType& op_type) {
    auto it = by_type_.find((int)op_type);
    return it == by_type_.end() ? OpExecutorFn() : it->second;
}

OpExecutorFn StreamExecutor::getOpExecutor(uint32_t& id) {
    auto it = dispatch_.find(id);
    return it == dispatch_.end() ? OpExecutorFn() : it->second;
}

RetVal StreamExecutor::preProcess() {
    graph_inputs_.clear();
    graph_outputs_.clear();
    dispatch_.clear();
    // 1. one executor per layer id
    for (auto layer : program_->getLayers()) {
        auto type = layer->getType();
        if (type == ir::LayerType::PRIMINPUT || type == ir::LayerType::PRIMOUTPUT) continue;
        auto fn = findAtenExecutorByType(type);
        if (!fn) {
            LOG(ERROR) << "no op executor is registered for " << ir::convertLayerTypeToString(type) << " (layer " << layer->getName()
                       << "): this runtime covers the recurrent / decode hot path and the control ops around it";
            return RetVal::FAILURE;
        }
        dispatch_.insert({layer->getID(), fn});
    }
    // 2. graph inputs / outputs, constants (materialised once and reused by every run), GNMT's pre-allocated cat buffers
    //    (stream_executor.cpp:80-92 of the reference; sizes follow the labelled layers' operands instead of constants)
    int custom_cat_mem_id = 0;
    for (auto layer : program_->getLayers()) {
        const auto type = layer->getType();
        if (family_ == "GNMT" && type == ir::LayerType::ATENLSTM1)
            custom_cat_mem_id = std::static_pointer_cast<ir::AtenLSTM1Layer>(layer)->getCustomCatMemId();
        if (family_ == "GNMT" && type == ir::LayerType::ATENCAT) {
            auto cat_layer = std::static_pointer_cast<ir::AtenCatLayer>(layer);
            auto options = at::TensorOptions().dtype(at::kHalf).device(at::kCUDA);
            const int64_t mem_blob_id = cat_layer->getMemLayerId();
            if (mem_blob_id != -1) {
                blobs_.insert({mem_blob_id, {ir::DataType::TENSOR, torch::jit::IValue(at::zeros({1, 1, 2048}, options))}});
            } else {
                cat_layer->setMemLayerId(custom_cat_mem_id);
                blobs_.insert({custom_cat_mem_id, {ir::DataType::TENSOR, torch::jit::IValue(at::zeros({8, 1, 1024}, options))}});
            }
        }
        if (type == ir::LayerType::PRIMINPUT) {
            graph_inputs_.push_back(layer->getOutSTensorID()[0]);
        } else if (type == ir::LayerType::PRIMOUTPUT) {
            graph_outputs_.push_back(layer->getInSTensorID()[0]);
        } else if (type == ir::LayerType::PRIMCONSTANT) {
            op_executor::executePrimConstant(layer, *this);
        } else if (type == ir::LayerType::PRIMVARIABLE) {
            if (std::static_pointer_cast<ir::PrimVariableLayer>(layer)->getIsConstant()) op_executor::executePrimVariable(layer, *this);
        }
    }
    if (graph_inputs_.empty() || graph_outputs_.empty()) {
        LOG(ERROR) << "the graph needs at least one input and one output";
        return RetVal::FAILURE;
    }
    return RetVal::SUCCESS;
}

void StreamExecutor::updateBlob(int64_t blob_id, ir::DataType dtype, const torch::jit::IValue& iv) {
    blobs_[blob_id] = std::make_pair(dtype, iv);
}

std::pair<ir::DataType, torch::jit::IValue>& StreamExecutor::findBlob(int64_t blob_id) {
    auto it = blobs_.find(blob_id);
    TORCH_CHECK(it != blobs_.end(), "blob ", blob_id, " has not been produced");
    return it->second;
}

bool StreamExecutor::checkValidBlobID(int64_t blob_id) { return blobs_.find(blob_id) != blobs_.end(); }

const std::shared_ptr<ir::NNGraph> StreamExecutor::getGraph() { return program_; }

cudaStream_t StreamExecutor::currentStream() const { return at::cuda::getCurrentCUDAStream().stream(); }

c10::cuda::CUDAStream StreamExecutor::sideStream(size_t i) {
    while (streams_.size() < 4) streams_.push_back(c10::cuda::getStreamFromPool());
    return streams_[i % streams_.size()];
}

at::cuda::CUDAEvent& StreamExecutor::event(size_t i) {
    while (events_.size() <= i) events_.push_back(std::make_unique<at::cuda::CUDAEvent>(cudaEventDefault));
    return *events_[i];
}

pimb200_lstm* StreamExecutor::lstmHandle(uint32_t layer_id) const {
    auto it = lstm_handles_.find(layer_id);
    return it == lstm_handles_.end() ? nullptr : it->second;
}

void StreamExecutor::setInputTensors(const std::vector<torch::Tensor>& input_tensors) {
    TORCH_CHECK(input_tensors.size() == graph_inputs_.size(), "the graph takes ", graph_inputs_.size(), " inputs, ",
                input_tensors.size(), " were given");
    for (size_t k = 0; k < input_tensors.size(); ++k) updateBlob(graph_inputs_[k], ir::DataType::TENSOR, torch::jit::IValue(input_tensors[k]));
}

// tensors of an output value, depth first: tensors as they are, runs of ints as one int64 row, tuples / lists unpacked
std::vector<torch::Tensor> StreamExecutor::iValueParser(torch::jit::IValue& iv) {
    std::vector<torch::Tensor> out;
    auto ints_to_tensor = [](const std::vector<int64_t>& v, bool row) {
        auto t = torch::tensor(v, torch::kLong);
        return row ? t.view({1, (int64_t)v.size()}) : t;
    };
    if (iv.isTensor()) {
        out.push_back(iv.toTensor());
    } else if (iv.isInt()) {
        out.push_back(ints_to_tensor({iv.toInt()}, false));
    } else if (iv.isTuple() || iv.isList()) {
        std::vector<torch::jit::IValue> elems;
        if (iv.isTuple()) {
            for (const auto& e : iv.toTupleRef().elements()) elems.push_back(e);
        } else {
            for (const auto& e : iv.toListRef()) elems.push_back(e);
        }
        std::vector<int64_t> ints;
        for (auto& e : elems) {
            if (e.isInt() && iv.isList()) {
                ints.push_back(e.toInt());
                continue;
            }
            for (auto& t : iValueParser(e)) out.push_back(t);
        }
        if (!ints.empty()) out.push_back(ints_to_tensor(ints, true));
    } else {
        TORCH_CHECK(false, "a graph output of an unsupported kind");
    }
    return out;
}

void StreamExecutor::getOutputTensors(std::vector<torch::Tensor>& output_tensors) {
    for (auto id : graph_outputs_) {
        auto iv = findBlob(id).second;
        for (auto& t : iValueParser(iv)) {
            std::lock_guard<std::mutex> lock(gather_mutex_);
            output_tensors.push_back(t.to("cuda:0"));   // every result ends up on cuda:0, as the reference's does
        }
    }
}

// A kernel whose bounded wait gave up leaves PIMB200_ERR_TIMEOUT in a device status word; outputs of such a run are
// undefined, so the run is reported as failed.
RetVal StreamExecutor::checkDeviceStatus() {
    if (cudaStreamSynchronize(currentStream()) != cudaSuccess) return RetVal::FAILURE;
    int rc = pimb200_gemm_last_status();
    for (auto& kv : lstm_handles_) {
        const int s = pimb200_lstm_last_status(kv.second);
        if (rc == PIMB200_OK) rc = s;
    }
    setStatus(rc);
    return rc == PIMB200_OK ? RetVal::SUCCESS : RetVal::FAILURE;
}

RetVal StreamExecutor::inferenceModel(const std::vector<torch::Tensor>& input_tensors, std::vector<torch::Tensor>& output_tensors) {
    return run(input_tensors, output_tensors, false);
}
RetVal StreamExecutor::inferenceModelwithProfiling(const std::vector<torch::Tensor>& input_tensors,
                                                   std::vector<torch::Tensor>& output_tensors) {
    return run(input_tensors, output_tensors, true);
}

RetVal StreamExecutor::run(const std::vector<torch::Tensor>& input_tensors, std::vector<torch::Tensor>& output_tensors, bool profiling) {
    status_ = 0;
    setInputTensors(input_tensors);
    auto& layers = program_->getLayers();
    const int64_t n_layers = (int64_t)layers.size();
    struct Span { std::string name; size_t e0, e1; };
    std::vector<Span> spans;
    size_t next_event = 16;   // events 0..15 belong to MULTISTREAM
    // layers are ordered inputs, body, outputs; the cursor is the position (= id after UpdateLayerId) of the next layer
    for (pc_ = (int64_t)graph_inputs_.size(); pc_ < n_layers - (int64_t)graph_outputs_.size();) {
        auto layer = layers[pc_];
        const auto type = layer->getType();
        if (type == ir::LayerType::PRIMCONSTANT || type == ir::LayerType::PRIMINPUT || type == ir::LayerType::PRIMOUTPUT) {
            ++pc_;   // constants were materialised by preProcess
            continue;
        }
        uint32_t id = layer->getID();
        auto fn = getOpExecutor(id);
        if (!fn) return RetVal::FAILURE;
        const int64_t before = pc_;
        if (profiling) {
            event(next_event).record(c10::cuda::getCurrentCUDAStream());
            fn(layer, *this);
            event(next_event + 1).record(c10::cuda::getCurrentCUDAStream());
            spans.push_back({layer->getName(), next_event, next_event + 1});
            next_event += 2;
        } else {
            fn(layer, *this);
        }
        if (status_ != 0) {
            LOG(ERROR) << "layer " << layer->getName() << " failed: " << pimb200_status_string(status_);
            return RetVal::FAILURE;
        }
        // control ops (and MULTISTREAM) move the cursor themselves
        if (!ir::isControlOp(type) && pc_ == before) ++pc_;
    }
    if (checkDeviceStatus() != RetVal::SUCCESS) return RetVal::FAILURE;
    if (profiling && !spans.empty()) {
        // Chrome trace ("traceEvents" of complete events, microseconds): one span per executed op, on the device
        // timeline of the launching stream (the reference times each op on the host around a device-wide sync,
        // runtime/source/executor/stream_executor.cpp:204-258, runtime/include/executor/utils/profiler.h:54-261)
        FILE* f = std::fopen(profile_path_.c_str(), "w");
        if (f) {
            std::fprintf(f, "{\"otherData\": {}, \"traceEvents\": [");
            for (size_t i = 0; i < spans.size(); ++i) {
                const double start_us = i == 0 ? 0.0 : 1e3 * event(spans[0].e0).elapsed_time(event(spans[i].e0));
                const double dur_us = 1e3 * event(spans[i].e0).elapsed_time(event(spans[i].e1));
                std::fprintf(f, "%s{\"cat\": \"function\", \"dur\": %.3f, \"name\": \"%s\", \"ph\": \"X\", \"pid\": 0, \"tid\": 0, \"ts\": %.3f}",
                             i ? ", " : "", dur_us, spans[i].name.c_str(), start_us);
            }
            std::fprintf(f, "]}\n");
            std::fclose(f);
        }
    }
    getOutputTensors(output_tensors);
    return RetVal::SUCCESS;
}

}  // namespace runtime
}  // namespace nn_compiler
