// PipelineManager (see pipeline_manager.h).
#include "pipeline_manager.h"

#include <c10/cuda/CUDAGuard.h>
#include <glog/logging.h>

namespace NNRuntimeInterface {

using nn_compiler::compiler::NNCompiler;
using nn_compiler::runtime::NNRuntime;

namespace {
// A replica's own copy of the compiled model: the layer objects are cloned (the runtime writes preload ids, parameter
// vectors and loop conditions onto them), the runtime reads nothing else of the model.
std::unique_ptr<nn_compiler::ir::NNModel> cloneForReplica(const std::shared_ptr<nn_compiler::ir::NNModel>& src) {
    auto model = std::make_unique<nn_compiler::ir::NNModel>();
    for (auto& g : src->getGraphs()) {
        auto graph = std::make_shared<nn_compiler::ir::NNGraph>();
        graph->setName(g->getName());
        for (auto& layer : g->getLayers()) graph->addLayer(layer->clone());
        for (auto id : g->getGraphInTensorID()) graph->addGraphInTensorID(id);
        for (auto id : g->getGraphOutTensorID()) graph->addGraphOutTensorID(id);
        model->appendGraph(graph);
    }
    return model;
}
std::mutex g_build_mutex;   // replicas prepare their runtimes one at a time
}  // namespace

PipelineManager::PipelineManager(const std::string& input_file_path, std::string model_type, int gpu_num, bool profiling)
    : input_file_path_(input_file_path), family_(std::move(model_type)), is_profiling_(profiling) {
    auto model = std::make_unique<nn_compiler::ir::NNModel>();
    NNCompiler compiler;
    compiler.initialize(input_file_path_, family_);
    compiler.compile(model);
    if (gpu_num <= 1) {
        runtime_ = std::make_shared<NNRuntime>(model, family_);
        if (runtime_->lastResult() != RetVal::SUCCESS) throw std::runtime_error("NNRuntime: the model could not be prepared");
        compiled_ = std::move(model);
        return;
    }
    compiled_ = std::move(model);
    for (int d = 0; d < gpu_num; ++d) {
        replicas_.push_back(std::make_unique<Replica>());
        replicas_.back()->device = d;
    }
    for (auto& r : replicas_) r->thread = std::thread(&PipelineManager::worker, this, r.get());
    // wait until every replica has built its runtime (or failed to)
    for (auto& r : replicas_) {
        std::unique_lock<std::mutex> lk(r->mu);
        r->cv.wait(lk, [&] { return r->done; });
        r->done = false;
        if (r->failed) throw std::runtime_error("replica on cuda:" + std::to_string(r->device) + ": " + r->error);
    }
}

PipelineManager::~PipelineManager() {
    for (auto& r : replicas_) {
        {
            std::lock_guard<std::mutex> lk(r->mu);
            r->stop = true;
        }
        r->cv.notify_all();
        if (r->thread.joinable()) r->thread.join();
    }
}

void PipelineManager::setProfilePath(const std::string& path) {
    if (runtime_) runtime_->setProfilePath(path);
}

// One replica: its own device, its own copy of the compiled model (layers carry per-runtime state), its own runtime.
void PipelineManager::worker(Replica* r) {
    std::shared_ptr<NNRuntime> rt;
    try {
        c10::cuda::CUDAGuard guard(r->device);
        std::lock_guard<std::mutex> build_lock(g_build_mutex);
        auto model = cloneForReplica(compiled_);
        rt = std::make_shared<NNRuntime>(model, family_);
        if (rt->lastResult() != RetVal::SUCCESS) throw std::runtime_error("the model could not be prepared");
    } catch (const std::exception& e) {
        std::lock_guard<std::mutex> lk(r->mu);
        r->failed = true;
        r->error = e.what();
    }
    {
        std::lock_guard<std::mutex> lk(r->mu);
        r->done = true;
    }
    r->cv.notify_all();
    while (true) {
        std::unique_lock<std::mutex> lk(r->mu);
        r->cv.wait(lk, [&] { return r->has_work || r->stop; });
        if (r->stop) return;
        r->has_work = false;
        r->outputs.clear();
        r->failed = false;
        try {
            c10::cuda::CUDAGuard guard(r->device);
            std::vector<torch::Tensor> in;
            for (auto& t : r->inputs) in.push_back(t.to(torch::Device(torch::kCUDA, r->device)));
            rt->inferenceModel(in, r->outputs, is_profiling_);
            if (rt->lastResult() != RetVal::SUCCESS) throw std::runtime_error("inference failed");
        } catch (const std::exception& e) {
            r->failed = true;
            r->error = e.what();
        }
        r->done = true;
        lk.unlock();
        r->cv.notify_all();
    }
}

std::vector<torch::Tensor> PipelineManager::inferenceModel(const std::vector<torch::Tensor>& input_tensors) {
    std::vector<torch::Tensor> outputs;
    if (runtime_) {
        runtime_->inferenceModel(input_tensors, outputs, is_profiling_);
        if (runtime_->lastResult() != RetVal::SUCCESS) throw std::runtime_error("NNRuntime::inferenceModel failed");
        return outputs;
    }
    // replicas: chunk every input along dimension 0 over as many replicas as there are rows
    TORCH_CHECK(!input_tensors.empty() && input_tensors[0].dim() >= 1, "replicated inference needs batched inputs");
    const int64_t rows = input_tensors[0].size(0);
    const int64_t used = std::min<int64_t>(rows, (int64_t)replicas_.size());
    std::vector<std::vector<torch::Tensor>> chunks;
    for (auto& t : input_tensors) chunks.push_back(t.chunk(used, 0));
    for (int64_t i = 0; i < used; ++i) {
        auto& r = replicas_[i];
        {
            std::lock_guard<std::mutex> lk(r->mu);
            r->inputs.clear();
            for (auto& c : chunks) r->inputs.push_back(c[i]);
            r->has_work = true;
            r->done = false;
        }
        r->cv.notify_all();
    }
    std::vector<std::vector<torch::Tensor>> per_replica;
    for (int64_t i = 0; i < used; ++i) {
        auto& r = replicas_[i];
        std::unique_lock<std::mutex> lk(r->mu);
        r->cv.wait(lk, [&] { return r->done; });
        if (r->failed) throw std::runtime_error("replica on cuda:" + std::to_string(r->device) + ": " + r->error);
        per_replica.push_back(r->outputs);
    }
    for (size_t k = 0; k < per_replica[0].size(); ++k) {
        std::vector<torch::Tensor> parts;
        for (auto& o : per_replica) parts.push_back(o.at(k).to("cuda:0"));
        outputs.push_back(at::cat(parts, 0));
    }
    return outputs;
}

}  // namespace NNRuntimeInterface
