// Minimal, interface-compatible subset of the reference's NNIR layer classes — just what the hot-path op
// executors read.  Class, method and enumerator names follow the reference (ir/include/types.h:42-183,
// ir/include/layers/nn_layer.h:22-141, aten_lstm1_layer.h:36-196, aten_addmm_layer.h:20-47,
// aten_linear_layer.h:21-66, aten_cat_layer.h:20-52, multi_stream_layer.h:21-59) so that an executor written
// against these headers reads like one written against the reference's; nothing else of the IR is reproduced.
#pragma once
#include <torch/torch.h>

#include <cstdint>
#include <memory>
#include <string>
#include <vector>

struct pimb200_lstm;

namespace nn_compiler {

enum class RetVal { SUCCESS, FAILURE };  // common/include/types.hpp:21-24

namespace ir {

enum class DataType { UNDEFINED, TENSOR, LIST, TUPLE, INT64, FLOAT64, BOOL, NONE };

enum class LayerType {
    ATENADD, ATENADDMM, ATENBMM, ATENCAT, ATENCOPY, ATENLINEAR, ATENLSTM1, ATENLSTM2, ATENMATMUL, MULTISTREAM,
    ATENSOFTMAX, ATENLOGSOFTMAX, ATENARGMAX, ATENLAYERNORM, ATENTANH, ATENMASKEDFILL, ATENEMBEDDING,
    PRIMINPUT, PRIMOUTPUT, PRIMCONSTANT, PRIMLISTCONSTRUCT
};

inline const char* convertLayerTypeToString(LayerType t) {
    switch (t) {
        case LayerType::ATENADD: return "aten::add";
        case LayerType::ATENADDMM: return "aten::addmm";
        case LayerType::ATENBMM: return "aten::bmm";
        case LayerType::ATENCAT: return "aten::cat";
        case LayerType::ATENCOPY: return "aten::copy_";
        case LayerType::ATENLINEAR: return "aten::linear";
        case LayerType::ATENLSTM1: return "aten::lstm1";
        case LayerType::ATENLSTM2: return "aten::lstm2";
        case LayerType::ATENMATMUL: return "aten::matmul";
        case LayerType::MULTISTREAM: return "MultiStream";
        case LayerType::ATENSOFTMAX: return "aten::softmax";
        case LayerType::ATENLOGSOFTMAX: return "aten::log_softmax";
        case LayerType::ATENARGMAX: return "aten::argmax";
        case LayerType::ATENLAYERNORM: return "aten::layer_norm";
        case LayerType::ATENTANH: return "aten::tanh";
        case LayerType::ATENMASKEDFILL: return "aten::masked_fill";
        case LayerType::ATENEMBEDDING: return "aten::embedding";
        case LayerType::PRIMINPUT: return "prim::Input";
        case LayerType::PRIMOUTPUT: return "prim::Output";
        case LayerType::PRIMCONSTANT: return "prim::Constant";
        case LayerType::PRIMLISTCONSTRUCT: return "prim::ListConstruct";
    }
    return "?";
}

class NNLayer {
   public:
    NNLayer(std::string name, LayerType type) : name_(std::move(name)), type_(type) {}
    virtual ~NNLayer() = default;
    LayerType getType() const { return type_; }
    const std::string& getName() const { return name_; }
    uint32_t getID() const { return id_; }
    void setID(uint32_t id) { id_ = id; }
    const std::vector<int64_t>& getInSTensorID() const { return in_stensor_ids_; }
    const std::vector<int64_t>& getOutSTensorID() const { return out_stensor_ids_; }
    void setInSTensorID(std::vector<int64_t> ids) { in_stensor_ids_ = std::move(ids); }
    void setOutSTensorID(std::vector<int64_t> ids) { out_stensor_ids_ = std::move(ids); }

   private:
    std::string name_;
    LayerType type_;
    uint32_t id_ = 0;
    std::vector<int64_t> in_stensor_ids_, out_stensor_ids_;
};

// where an LSTM output goes when the graph asks for the in-place "custom cat": a slice of a pre-allocated blob
struct OutputAlias {
    int64_t blob_id = -1;     // -1 = allocate a fresh tensor
    int64_t elem_offset = 0;  // first element of the slice inside the blob
};

class AtenLSTM1Layer : public NNLayer {
   public:
    AtenLSTM1Layer(std::string name, LayerType type = LayerType::ATENLSTM1) : NNLayer(std::move(name), type) {}
    ~AtenLSTM1Layer() override;
    void setHasBiases(int v) { has_biases_ = v; }
    void setNumLayers(int64_t v) { num_layers_ = v; }
    void setDropout(double v) { dropout_ = v; }
    void setTrain(int v) { train_ = v; }
    void setBidirectional(int v) { bidirectional_ = v; }
    void setBatchFirst(int v) { batch_first_ = v; }
    void setParamVector(std::vector<at::Tensor> p) { param_vector_ = std::move(p); }
    int getHasBiases() const { return has_biases_; }
    int64_t getNumLayers() const { return num_layers_; }
    double getDropout() const { return dropout_; }
    int getTrain() const { return train_; }
    int getBidirectional() const { return bidirectional_; }
    int getBatchFirst() const { return batch_first_; }
    const std::vector<at::Tensor>& getParamVector() const { return param_vector_; }
    // packed-weight handle (the counterpart of the reference's arranged_weight_), built by ModelBuilder::preloadModel
    pimb200_lstm* getPackedHandle() const { return packed_; }
    void setPackedHandle(pimb200_lstm* h) { packed_ = h; }
    OutputAlias out_alias[3];  // output, h_n, c_n

   private:
    int has_biases_ = 1, train_ = 0, bidirectional_ = 0, batch_first_ = 0;
    int64_t num_layers_ = 1;
    double dropout_ = 0.0;
    std::vector<at::Tensor> param_vector_;
    pimb200_lstm* packed_ = nullptr;
};

class AtenLSTM2Layer : public AtenLSTM1Layer {
   public:
    explicit AtenLSTM2Layer(std::string name) : AtenLSTM1Layer(std::move(name), LayerType::ATENLSTM2) {}
};

class AtenAddmmLayer : public NNLayer {
   public:
    explicit AtenAddmmLayer(std::string name) : NNLayer(std::move(name), LayerType::ATENADDMM) {}
    void setActType(std::string t) { act_type_ = std::move(t); }
    const std::string& getActType() const { return act_type_; }
    double alpha = 1.0, beta = 1.0;

   private:
    std::string act_type_ = "none";
};

class AtenMatmulLayer : public NNLayer {
   public:
    explicit AtenMatmulLayer(std::string name) : NNLayer(std::move(name), LayerType::ATENMATMUL) {}
};

class AtenLinearLayer : public NNLayer {
   public:
    explicit AtenLinearLayer(std::string name) : NNLayer(std::move(name), LayerType::ATENLINEAR) {}
    void setWeights(at::Tensor w) { weights_ = std::move(w); }
    void setBiases(at::Tensor b) { biases_ = std::move(b); }
    const at::Tensor& getWeights() const { return weights_; }
    const at::Tensor& getBiases() const { return biases_; }

   private:
    at::Tensor weights_, biases_;
};

class AtenAddLayer : public NNLayer {
   public:
    explicit AtenAddLayer(std::string name) : NNLayer(std::move(name), LayerType::ATENADD) {}
    double alpha = 1.0;
};

class AtenBmmLayer : public NNLayer {
   public:
    explicit AtenBmmLayer(std::string name) : NNLayer(std::move(name), LayerType::ATENBMM) {}
};

class AtenCatLayer : public NNLayer {
   public:
    explicit AtenCatLayer(std::string name) : NNLayer(std::move(name), LayerType::ATENCAT) {}
    void setDim(int64_t d) { dim_ = d; }
    int64_t getDim() const { return dim_; }
    void setMemLayerId(int64_t id) { mem_layer_id_ = id; }
    int64_t getMemLayerId() const { return mem_layer_id_; }

   private:
    int64_t dim_ = 0;
    int64_t mem_layer_id_ = -1;  // blob of a pre-filled buffer to return instead of copying ("custom cat")
};

class AtenCopyLayer : public NNLayer {
   public:
    explicit AtenCopyLayer(std::string name) : NNLayer(std::move(name), LayerType::ATENCOPY) {}
    int non_blocking = 0;
};

// aten::softmax / aten::log_softmax(self, dim): the attribute the reference's layers carry (dim; dtype is not modelled)
class AtenSoftmaxLayer : public NNLayer {
   public:
    AtenSoftmaxLayer(std::string name, bool log)
        : NNLayer(std::move(name), log ? LayerType::ATENLOGSOFTMAX : LayerType::ATENSOFTMAX) {}
    int64_t dim = -1;
};

// aten::argmax(self, dim, keepdim)
class AtenArgmaxLayer : public NNLayer {
   public:
    explicit AtenArgmaxLayer(std::string name) : NNLayer(std::move(name), LayerType::ATENARGMAX) {}
    int64_t dim = -1;
    int keepdim = 0;
};

// aten::layer_norm(input, normalized_shape, weight, bias, eps) with weight / bias preloaded on the layer
class AtenLayerNormLayer : public NNLayer {
   public:
    explicit AtenLayerNormLayer(std::string name) : NNLayer(std::move(name), LayerType::ATENLAYERNORM) {}
    std::vector<int64_t> normalized_shape;
    at::Tensor weight, bias;
    double eps = 1e-5;
};

class AtenTanhLayer : public NNLayer {
   public:
    explicit AtenTanhLayer(std::string name) : NNLayer(std::move(name), LayerType::ATENTANH) {}
};

// aten::masked_fill(self, mask, value) with a scalar value
class AtenMaskedFillLayer : public NNLayer {
   public:
    explicit AtenMaskedFillLayer(std::string name) : NNLayer(std::move(name), LayerType::ATENMASKEDFILL) {}
    double value = 0.0;
};

// aten::embedding(weight, indices): the table is an input blob, or preloaded on the layer as the reference's
// AtenEmbeddingLayer::getWeights allows
class AtenEmbeddingLayer : public NNLayer {
   public:
    explicit AtenEmbeddingLayer(std::string name) : NNLayer(std::move(name), LayerType::ATENEMBEDDING) {}
    at::Tensor weights;
};

class MultiStreamLayer : public NNLayer {
   public:
    explicit MultiStreamLayer(std::string name) : NNLayer(std::move(name), LayerType::MULTISTREAM) {}
    void setLayers(std::vector<std::shared_ptr<NNLayer>> l) { layers_ = std::move(l); }
    const std::vector<std::shared_ptr<NNLayer>>& getLayers() const { return layers_; }
    int getLayerNum() const { return (int)layers_.size(); }

   private:
    std::vector<std::shared_ptr<NNLayer>> layers_;
};

// prim::ListConstruct of tensors (hx of aten::lstm, the operand list of aten::cat); host-only, no arithmetic
class PrimListConstructLayer : public NNLayer {
   public:
    explicit PrimListConstructLayer(std::string name) : NNLayer(std::move(name), LayerType::PRIMLISTCONSTRUCT) {}
};

// ordered layer list with graph inputs/outputs — the part of NNGraph the interpreter loop walks
class NNGraph {
   public:
    void addLayer(std::shared_ptr<NNLayer> l) {
        l->setID((uint32_t)layers_.size());
        layers_.push_back(std::move(l));
    }
    const std::vector<std::shared_ptr<NNLayer>>& getLayers() const { return layers_; }
    std::vector<int64_t> input_ids, output_ids;
    // blobs that exist before the first layer runs (preloaded constants, pre-allocated cat buffers)
    std::vector<std::pair<int64_t, at::Tensor>> preset_blobs;

   private:
    std::vector<std::shared_ptr<NNLayer>> layers_;
};

}  // namespace ir
}  // namespace nn_compiler
