// Registry, blob store, interpreter loop and the GEMM shape classifier of the host-side mirror.
#include "stream_executor.h"

#include <ATen/cuda/CUDAContext.h>

#include "pimb200.h"

namespace nn_compiler {
namespace ir {
AtenLSTM1Layer::~AtenLSTM1Layer() {
    if (packed_) pimb200_lstm_destroy(packed_);
}
}  // namespace ir

namespace runtime {

// Same classes as the reference's router (runtime/source/executor/utils/utils.cpp:373-396) on shapes already
// padded to rank 4: vector classes need both leading dims to be 1; an operand is a vector when exactly one of its
// last two extents differs from 1, a matrix when both do.
GEMM_TYPE getGemmType(const std::vector<int64_t>& a, const std::vector<int64_t>& b) {
    if (a.size() != 4 || b.size() != 4) return GEMM_TYPE::UNKNOW;
    const bool lead_one = a[0] == 1 && a[1] == 1 && b[0] == 1 && b[1] == 1;
    if (!lead_one) return GEMM_TYPE::MM;
    const int na = (a[2] != 1) + (a[3] != 1), nb = (b[2] != 1) + (b[3] != 1);
    if (na == 1 && nb == 1) return GEMM_TYPE::VV;
    if (na == 1 && nb == 2) return GEMM_TYPE::VM;
    if (na == 2 && nb == 1) return GEMM_TYPE::MV;
    return GEMM_TYPE::MM;
}

StreamExecutor::StreamExecutor(std::shared_ptr<ir::NNGraph> graph, std::string model_type)
    : graph_(std::move(graph)), model_type_(std::move(model_type)) {
    registerOp();
}

StreamExecutor::~StreamExecutor() {
    for (auto s : streams_) cudaStreamDestroy(s);
}

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
            const auto& pv = lstm->getParamVector();
            if (pv.size() < 2) return RetVal::FAILURE;
            std::vector<const void*> ptrs;
            for (auto& p : pv) {
                if (!p.is_cuda() || p.scalar_type() != at::kHalf || !p.is_contiguous()) return RetVal::FAILURE;
                ptrs.push_back(p.data_ptr());
            }
            const int H = (int)pv[1].size(1), I = (int)pv[0].size(1);
            pimb200_lstm* h = nullptr;
            const int rc = pimb200_lstm_create(ptrs.data(), (int)ptrs.size(), (int)lstm->getNumLayers(),
                                               lstm->getBidirectional(), I, H, lstm->getHasBiases(), &h);
            if (rc != PIMB200_OK) return RetVal::FAILURE;
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

const std::vector<cudaStream_t>& StreamExecutor::streamPool() {
    if (streams_.empty()) {
        for (int i = 0; i < 4; ++i) {
            cudaStream_t s = nullptr;
            if (cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking) == cudaSuccess) streams_.push_back(s);
        }
    }
    return streams_;
}

RetVal StreamExecutor::inferenceModel(const std::vector<torch::Tensor>& input_tensors,
                                      std::vector<torch::Tensor>& output_tensors) {
    if (input_tensors.size() != graph_->input_ids.size()) return RetVal::FAILURE;
    if (op_executor_.size() != graph_->getLayers().size() && preProcess() != RetVal::SUCCESS) return RetVal::FAILURE;
    status_ = 0;
    for (auto& pb : graph_->preset_blobs)
        if (!checkValidBlobID(pb.first)) updateBlob(pb.first, ir::DataType::TENSOR, torch::jit::IValue(pb.second));
    for (size_t i = 0; i < input_tensors.size(); ++i)
        updateBlob(graph_->input_ids[i], ir::DataType::TENSOR, torch::jit::IValue(input_tensors[i]));
    const auto& layers = graph_->getLayers();
    for (cursor_ = 0; cursor_ < (int64_t)layers.size();) {
        auto layer = layers[cursor_];
        const int64_t before = cursor_;
        op_executor_[cursor_](layer, *this);
        if (status_ != 0) return RetVal::FAILURE;
        if (cursor_ == before) ++cursor_;  // executors that jump (MULTISTREAM) set the cursor themselves
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
                               std::vector<torch::Tensor>& output_tensors, bool /*profiling*/) {
    last_ = executor_->inferenceModel(input_tensors, output_tensors);
}

}  // namespace runtime
}  // namespace nn_compiler
