// Bodies of the hot-path op executors, written against the pimb200 C ABI.
//
// Each function keeps the contract of its namesake in the reference's
// runtime/source/executor/op_executor/aten_ops_executor.cpp (inputs are read from the blob store by in-STensor id,
// attributes from the layer object, results are published with updateBlob), but the device work goes through
// libpimb200.so instead of PIM / MIOpen / the HIP templates.  Shapes outside the hot path (general batched matmul,
// non-unit alpha/beta, mixed dtypes) are forwarded to the same at:: op the reference falls back to.
#include <ATen/cuda/CUDAContext.h>

#include "pimb200.h"
#include "stream_executor.h"

namespace nn_compiler {
namespace runtime {
namespace op_executor {

namespace {

at::Tensor blobTensor(StreamExecutor& ex, int64_t id) {
    auto& iv = ex.findBlob(id).second;
    TORCH_CHECK(iv.isTensor(), "blob ", id, " is not a tensor");
    return iv.toTensor();
}

bool fastHalf(const at::Tensor& t) { return t.defined() && t.is_cuda() && t.scalar_type() == at::kHalf; }

// True when `t` ([K, C] logically) is a transposed view of a contiguous [C, K] matrix, i.e. already K-major.
bool isTransposedKMajor(const at::Tensor& t) {
    return t.dim() == 2 && t.stride(1) == t.size(0) && t.stride(0) == 1;
}

std::vector<int64_t> pad4(at::IntArrayRef s) {
    std::vector<int64_t> v(s.begin(), s.end());
    while (v.size() < 4) v.insert(v.begin(), 1);
    return v;
}

// out = act(L @ R + bias) for the shapes the hot path produces; returns an undefined tensor when the shape is not
// one of them (the caller then uses the library op).  `bias` is 1-D or undefined.  On the vector paths the graph's
// alpha/beta are 1 (the reference hard-sets them, aten_ops.cpp:627-628).
at::Tensor fusedMatmul(StreamExecutor& ex, at::Tensor L, at::Tensor R, const at::Tensor& bias, bool relu,
                       cudaStream_t st) {
    if (!fastHalf(L) || !fastHalf(R) || (bias.defined() && (!fastHalf(bias) || bias.dim() != 1))) return {};
    if (L.dim() > 4 || R.dim() > 4 || L.dim() < 1 || R.dim() < 1) return {};
    const int act = relu ? PIMB200_ACT_RELU : PIMB200_ACT_NONE;
    // libtorch's own shape rule for the result, computed on meta tensors (no device work)
    const auto out_sizes = at::matmul(at::empty(L.sizes(), L.options().device(at::kMeta)),
                                      at::empty(R.sizes(), R.options().device(at::kMeta))).sizes().vec();
    const int64_t K = L.size(-1);
    const int64_t rowsL = L.numel() / K;                       // every leading extent of L is a row
    const int64_t colsR = R.dim() == 1 ? 1 : R.size(-1);
    const int64_t Kr = R.dim() == 1 ? R.size(0) : R.size(-2);
    if (Kr != K || R.numel() != Kr * colsR) return {};         // a batched right operand is not a hot-path shape
    const at::Tensor b = bias.defined() ? bias.contiguous() : bias;
    const void* bp = b.defined() ? b.data_ptr() : nullptr;
    at::Tensor out;
    int rc = PIMB200_OK;
    const GEMM_TYPE type = getGemmType(pad4({rowsL, K}), pad4({K, colsR}));
    if (type == GEMM_TYPE::VV) {
        L = L.contiguous(); R = R.contiguous();
        out = at::empty({1}, L.options());
        rc = pimb200_dot_vv(L.data_ptr(), R.data_ptr(), out.data_ptr(), (int)K, st);
        if (rc == PIMB200_OK && b.defined()) out = relu ? at::relu(out + b) : out + b;
        else if (relu) out = at::relu(out);
    } else if (type == GEMM_TYPE::VM) {
        if (b.defined() && b.numel() != colsR) return {};
        L = L.contiguous();
        at::Tensor A = R.reshape({K, colsR}).contiguous();
        out = at::empty({colsR}, L.options());
        rc = pimb200_gemv_vm(L.data_ptr(), A.data_ptr(), bp, out.data_ptr(), (int)K, (int)colsR, act, st);
    } else if (type == GEMM_TYPE::MV) {
        if (b.defined() && b.numel() != rowsL) return {};
        at::Tensor W = L.reshape({rowsL, K}).contiguous();
        R = R.contiguous();
        out = at::empty({rowsL}, L.options());
        rc = pimb200_gemv_mv(W.data_ptr(), R.data_ptr(), bp, out.data_ptr(), (int)rowsL, (int)K, act, st);
    } else {
        // MM: out[r, c] = sum_k L[r,k] R[k,c].  A 1-D bias follows the reference's MM branch (aten_ops.cpp:695-711):
        // it is indexed by the row of L.
        at::Tensor Lm = L.reshape({rowsL, K}).contiguous();
        at::Tensor Rm = R.reshape({K, colsR});
        at::Tensor Rt = isTransposedKMajor(Rm) ? Rm.t() : Rm.t().contiguous();   // [colsR, K], K-major
        if (b.defined()) {
            if (b.numel() != rowsL) return {};
            at::Tensor Yt = at::empty({colsR, rowsL}, L.options());               // Y^T[c, r]
            rc = pimb200_gemm_wx(Lm.data_ptr(), Rt.data_ptr(), bp, Yt.data_ptr(), (int)rowsL, (int)K, (int)colsR,
                                 (int)K, (int)rowsL, act, 0, st);
            out = Yt.t();
        } else {
            out = at::empty({rowsL, colsR}, L.options());
            rc = pimb200_gemm_wx(Rt.data_ptr(), Lm.data_ptr(), nullptr, out.data_ptr(), (int)colsR, (int)K, (int)rowsL,
                                 (int)K, (int)colsR, act, 0, st);
        }
    }
    ex.setStatus(rc);
    if (rc != PIMB200_OK) return {};
    return out.reshape(out_sizes);
}

void runAddmm(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& ex, cudaStream_t st) {
    auto addmm = std::static_pointer_cast<ir::AtenAddmmLayer>(layer);
    const auto& in = layer->getInSTensorID();
    at::Tensor self = blobTensor(ex, in[0]), mat1 = blobTensor(ex, in[1]), mat2 = blobTensor(ex, in[2]);
    const bool relu = addmm->getActType() == "aten::relu";
    at::Tensor out;
    if (addmm->alpha == 1.0 && addmm->beta == 1.0 && self.dim() == 1) out = fusedMatmul(ex, mat1, mat2, self, relu, st);
    if (!out.defined() && ex.getStatus() == 0) {
        at::Tensor s = self;
        if (self.dim() == 1 && mat2.dim() >= 2 && self.size(0) == mat1.size(-2) && self.size(0) != mat2.size(-1))
            s = self.unsqueeze(1);  // per-row bias of the swapped form
        out = at::addmm(s, mat1.dim() > 2 ? mat1.squeeze(0) : mat1, mat2.dim() > 2 ? mat2.squeeze(0) : mat2,
                        addmm->beta, addmm->alpha);
        if (relu) out = at::relu(out);
    }
    ex.updateBlob(layer->getOutSTensorID()[0], ir::DataType::TENSOR, torch::jit::IValue(out));
}

void runMatmul(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& ex, cudaStream_t st) {
    const auto& in = layer->getInSTensorID();
    at::Tensor a = blobTensor(ex, in[0]), b = blobTensor(ex, in[1]);
    at::Tensor out = fusedMatmul(ex, a, b, at::Tensor(), false, st);
    if (!out.defined() && ex.getStatus() == 0) out = at::matmul(a, b);
    ex.updateBlob(layer->getOutSTensorID()[0], ir::DataType::TENSOR, torch::jit::IValue(out));
}

}  // namespace

void executeAtenAddmm(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& ex) { runAddmm(layer, ex, ex.currentStream()); }
void executeAtenAddmmWithStream(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& ex, void* stream) {
    runAddmm(layer, ex, static_cast<cudaStream_t>(stream));
}
void executeAtenMatmul(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& ex) { runMatmul(layer, ex, ex.currentStream()); }
void executeAtenMatmulWithStream(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& ex, void* stream) {
    runMatmul(layer, ex, static_cast<cudaStream_t>(stream));
}

// aten::linear(x, W, b) with W/b preloaded on the layer (only reached when the linear->addmm rewrite did not fire)
void executeAtenLinear(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& ex) {
    auto lin = std::static_pointer_cast<ir::AtenLinearLayer>(layer);
    at::Tensor x = blobTensor(ex, layer->getInSTensorID()[0]);
    const at::Tensor& W = lin->getWeights();
    const at::Tensor& b = lin->getBiases();
    at::Tensor out;
    if (fastHalf(x) && fastHalf(W) && W.dim() == 2 && (!b.defined() || fastHalf(b))) {
        const int64_t K = W.size(1), N = W.size(0), J = x.numel() / K;
        at::Tensor xc = x.contiguous(), Wc = W.contiguous();
        auto sizes = x.sizes().vec();
        sizes.back() = N;
        out = at::empty(sizes, x.options());
        const void* bp = b.defined() ? b.data_ptr() : nullptr;
        const int rc = J == 1 ? pimb200_gemv_mv(Wc.data_ptr(), xc.data_ptr(), bp, out.data_ptr(), (int)N, (int)K,
                                                PIMB200_ACT_NONE, ex.currentStream())
                              : pimb200_gemm_wx(Wc.data_ptr(), xc.data_ptr(), bp, out.data_ptr(), (int)N, (int)K, (int)J,
                                                (int)K, (int)N, PIMB200_ACT_NONE, 0, ex.currentStream());
        ex.setStatus(rc);
    } else {
        out = at::linear(x, W, b.defined() ? c10::optional<at::Tensor>(b) : c10::nullopt);
    }
    ex.updateBlob(layer->getOutSTensorID()[0], ir::DataType::TENSOR, torch::jit::IValue(out));
}

// fp16 add: same shape, or the second operand one row broadcast over the rows of the first.  aten::add is
// functional, so the result is a new tensor (the reference's kernel writes in place into its first operand).
void executeAtenAdd(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& ex) {
    auto add = std::static_pointer_cast<ir::AtenAddLayer>(layer);
    const auto& in = layer->getInSTensorID();
    at::Tensor a = blobTensor(ex, in[0]), b = blobTensor(ex, in[1]);
    at::Tensor out;
    const bool same = a.sizes() == b.sizes();
    const bool row = !same && a.dim() >= 1 && b.numel() == a.size(-1) && (b.dim() == 0 || b.size(-1) == a.size(-1));
    if (add->alpha == 1.0 && fastHalf(a) && fastHalf(b) && (same || row) && a.numel() > 0) {
        at::Tensor ac = a.contiguous(), bc = b.contiguous();
        out = at::empty_like(ac);
        const int n = (int)ac.size(-1), m = (int)(ac.numel() / n);
        ex.setStatus(pimb200_add_f16(ac.data_ptr(), bc.data_ptr(), out.data_ptr(), m, n, row ? 1 : 0, ex.currentStream()));
    } else {
        out = at::add(a, b, add->alpha);
    }
    ex.updateBlob(layer->getOutSTensorID()[0], ir::DataType::TENSOR, torch::jit::IValue(out));
}

// ---- row-wise glue of the decode path: the device kernels take contiguous fp16 rows along the last dimension;
//      any other dim / dtype keeps the libtorch call the reference makes ----
static bool lastDim(const at::Tensor& t, int64_t dim) { return t.dim() >= 1 && (dim == -1 || dim == t.dim() - 1); }

void executeAtenSoftmax(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& ex) {
    auto sm = std::static_pointer_cast<ir::AtenSoftmaxLayer>(layer);
    const bool log = layer->getType() == ir::LayerType::ATENLOGSOFTMAX;
    at::Tensor x = blobTensor(ex, layer->getInSTensorID()[0]);
    at::Tensor out;
    if (fastHalf(x) && lastDim(x, sm->dim) && x.numel() > 0) {
        at::Tensor xc = x.contiguous();
        out = at::empty_like(xc);
        const long cols = (long)xc.size(-1), rows = (long)(xc.numel() / cols);
        ex.setStatus(pimb200_softmax_rows(xc.data_ptr(), out.data_ptr(), rows, cols, log ? 1 : 0, ex.currentStream()));
    } else {
        out = log ? at::log_softmax(x, sm->dim) : at::softmax(x, sm->dim);
    }
    ex.updateBlob(layer->getOutSTensorID()[0], ir::DataType::TENSOR, torch::jit::IValue(out));
}

void executeAtenArgmax(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& ex) {
    auto am = std::static_pointer_cast<ir::AtenArgmaxLayer>(layer);
    at::Tensor x = blobTensor(ex, layer->getInSTensorID()[0]);
    at::Tensor out;
    if (fastHalf(x) && lastDim(x, am->dim) && x.numel() > 0) {
        at::Tensor xc = x.contiguous();
        auto sizes = xc.sizes().vec();
        const long cols = (long)sizes.back(), rows = (long)(xc.numel() / cols);
        if (am->keepdim) sizes.back() = 1;
        else sizes.pop_back();
        out = at::empty(sizes, xc.options().dtype(at::kLong));
        ex.setStatus(pimb200_argmax_rows(xc.data_ptr(), reinterpret_cast<long long*>(out.data_ptr<int64_t>()), rows, cols,
                                         ex.currentStream()));
    } else {
        out = at::argmax(x, am->dim, am->keepdim != 0);
    }
    ex.updateBlob(layer->getOutSTensorID()[0], ir::DataType::TENSOR, torch::jit::IValue(out));
}

void executeAtenLayerNorm(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& ex) {
    auto ln = std::static_pointer_cast<ir::AtenLayerNormLayer>(layer);
    at::Tensor x = blobTensor(ex, layer->getInSTensorID()[0]);
    at::Tensor out;
    const bool one_dim = ln->normalized_shape.size() == 1 && x.dim() >= 1 && ln->normalized_shape[0] == x.size(-1);
    if (fastHalf(x) && one_dim && x.numel() > 0 && (!ln->weight.defined() || fastHalf(ln->weight)) &&
        (!ln->bias.defined() || fastHalf(ln->bias))) {
        at::Tensor xc = x.contiguous();
        out = at::empty_like(xc);
        const long cols = (long)xc.size(-1), rows = (long)(xc.numel() / cols);
        at::Tensor w = ln->weight.defined() ? ln->weight.contiguous() : at::Tensor();
        at::Tensor b = ln->bias.defined() ? ln->bias.contiguous() : at::Tensor();
        ex.setStatus(pimb200_layer_norm_rows(xc.data_ptr(), w.defined() ? w.data_ptr() : nullptr,
                                             b.defined() ? b.data_ptr() : nullptr, out.data_ptr(), rows, cols,
                                             (float)ln->eps, ex.currentStream()));
    } else {
        out = at::layer_norm(x, ln->normalized_shape,
                             ln->weight.defined() ? c10::optional<at::Tensor>(ln->weight) : c10::nullopt,
                             ln->bias.defined() ? c10::optional<at::Tensor>(ln->bias) : c10::nullopt, ln->eps);
    }
    ex.updateBlob(layer->getOutSTensorID()[0], ir::DataType::TENSOR, torch::jit::IValue(out));
}

void executeAtenTanh(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& ex) {
    at::Tensor x = blobTensor(ex, layer->getInSTensorID()[0]);
    at::Tensor out;
    if (fastHalf(x) && x.numel() > 0) {
        at::Tensor xc = x.contiguous();
        out = at::empty_like(xc);
        ex.setStatus(pimb200_tanh_f16(xc.data_ptr(), out.data_ptr(), (size_t)xc.numel(), ex.currentStream()));
    } else {
        out = at::tanh(x);
    }
    ex.updateBlob(layer->getOutSTensorID()[0], ir::DataType::TENSOR, torch::jit::IValue(out));
}

void executeAtenMaskedFill(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& ex) {
    auto mf = std::static_pointer_cast<ir::AtenMaskedFillLayer>(layer);
    const auto& in = layer->getInSTensorID();
    at::Tensor x = blobTensor(ex, in[0]), mask = blobTensor(ex, in[1]);
    at::Tensor out;
    const bool same = mask.sizes() == x.sizes();
    const bool row = !same && x.dim() >= 1 && mask.numel() == x.size(-1) && mask.dim() >= 1 && mask.size(-1) == x.size(-1);
    if (fastHalf(x) && mask.is_cuda() && mask.scalar_type() == at::kBool && (same || row) && x.numel() > 0) {
        at::Tensor xc = x.contiguous(), mc = mask.contiguous();
        out = at::empty_like(xc);
        ex.setStatus(pimb200_masked_fill_f16(xc.data_ptr(), reinterpret_cast<const unsigned char*>(mc.data_ptr<bool>()),
                                             (float)mf->value, out.data_ptr(), (size_t)xc.numel(), (size_t)mc.numel(),
                                             ex.currentStream()));
    } else {
        out = at::masked_fill(x, mask, mf->value);
    }
    ex.updateBlob(layer->getOutSTensorID()[0], ir::DataType::TENSOR, torch::jit::IValue(out));
}

// aten::embedding.  Indices that already live on the device are used there (the reference reads them back with
// indices.item(), one host synchronisation per decoded token); host indices keep the libtorch call.
void executeAtenEmbedding(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& ex) {
    auto emb = std::static_pointer_cast<ir::AtenEmbeddingLayer>(layer);
    const auto& in = layer->getInSTensorID();
    at::Tensor table = emb->weights.defined() ? emb->weights : blobTensor(ex, in[0]);
    at::Tensor idx = blobTensor(ex, in[emb->weights.defined() ? 0 : 1]);
    at::Tensor out;
    if (table.is_cuda() && table.dim() == 2 && idx.is_cuda() && idx.scalar_type() == at::kLong && idx.numel() > 0) {
        at::Tensor tc = table.contiguous(), ic = idx.contiguous();
        auto sizes = ic.sizes().vec();
        sizes.push_back(tc.size(1));
        out = at::empty(sizes, tc.options());
        ex.setStatus(pimb200_gather_rows(tc.data_ptr(), reinterpret_cast<const long long*>(ic.data_ptr<int64_t>()),
                                         out.data_ptr(), (long)ic.numel(), (size_t)tc.size(1) * tc.element_size(),
                                         (long)tc.size(0), ex.currentStream()));
    } else {
        out = at::embedding(table, idx.to(table.device()));
    }
    ex.updateBlob(layer->getOutSTensorID()[0], ir::DataType::TENSOR, torch::jit::IValue(out));
}

// x[1,1,k] . A[1,k,n] (the GNMT attention context) through the single-row kernel; anything else is at::bmm
void executeAtenBmm(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& ex) {
    const auto& in = layer->getInSTensorID();
    at::Tensor x = blobTensor(ex, in[0]), A = blobTensor(ex, in[1]);
    at::Tensor out;
    if (fastHalf(x) && fastHalf(A) && x.dim() == 3 && A.dim() == 3 && x.size(0) == 1 && A.size(0) == 1 && x.size(1) == 1) {
        at::Tensor xc = x.contiguous(), Ac = A.contiguous();
        out = at::empty({1, 1, A.size(2)}, x.options());
        ex.setStatus(pimb200_bmm_row(xc.data_ptr(), Ac.data_ptr(), out.data_ptr(), (int)A.size(1), (int)A.size(2),
                                     ex.currentStream()));
    } else {
        out = at::bmm(x, A);
    }
    ex.updateBlob(layer->getOutSTensorID()[0], ir::DataType::TENSOR, torch::jit::IValue(out));
}

// aten::cat over a TensorList blob.  When the layer carries the id of a pre-filled buffer (the "custom cat" label of
// the GNMT graphs) that buffer is the result and nothing is copied.
void executeAtenCat(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& ex) {
    auto cat = std::static_pointer_cast<ir::AtenCatLayer>(layer);
    const int64_t out_id = layer->getOutSTensorID()[0];
    if (cat->getMemLayerId() >= 0 && ex.checkValidBlobID(cat->getMemLayerId())) {
        ex.updateBlob(out_id, ir::DataType::TENSOR, ex.findBlob(cat->getMemLayerId()).second);
        return;
    }
    auto& iv = ex.findBlob(layer->getInSTensorID()[0]).second;
    TORCH_CHECK(iv.isTensorList(), "aten::cat expects a tensor list");
    std::vector<at::Tensor> ts;
    for (const at::Tensor& t : iv.toTensorList()) ts.push_back(t);
    TORCH_CHECK(!ts.empty(), "aten::cat of an empty list");
    bool fast = true;
    for (auto& t : ts) fast = fast && t.is_cuda() && t.scalar_type() == ts[0].scalar_type() && t.dim() == ts[0].dim();
    at::Tensor out;
    if (fast && ts[0].dim() > 0) {
        const int64_t nd = ts[0].dim(), dim = (cat->getDim() % nd + nd) % nd;
        auto sizes = ts[0].sizes().vec();
        int64_t total = 0;
        for (auto& t : ts) total += t.size(dim);
        sizes[dim] = total;
        out = at::empty(sizes, ts[0].options());
        int64_t outer = 1;
        for (int64_t d = 0; d < dim; ++d) outer *= sizes[d];
        std::vector<at::Tensor> keep;
        std::vector<const void*> src;
        std::vector<size_t> inner;
        for (auto& t : ts) {
            if (t.numel() == 0) continue;
            keep.push_back(t.contiguous());
            src.push_back(keep.back().data_ptr());
            inner.push_back((size_t)(keep.back().numel() / outer) * keep.back().element_size());
        }
        if (!src.empty() && out.numel() > 0)
            ex.setStatus(pimb200_cat(out.data_ptr(), src.data(), inner.data(), (int)src.size(), (size_t)outer,
                                     ex.currentStream()));
    } else {
        out = at::cat(ts, cat->getDim());
    }
    ex.updateBlob(out_id, ir::DataType::TENSOR, torch::jit::IValue(out));
}

// self.copy_(src): device-to-device copies of equal dtype go through the strided copy kernel; host<->device and
// converting copies stay with the library (runtime/unit-tests/aten_ops_ut.cpp:43-63 exercises both directions)
void executeAtenCopy(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& ex) {
    auto cp = std::static_pointer_cast<ir::AtenCopyLayer>(layer);
    const auto& in = layer->getInSTensorID();
    at::Tensor self = blobTensor(ex, in[0]), src = blobTensor(ex, in[1]);
    if (self.is_cuda() && src.is_cuda() && self.scalar_type() == src.scalar_type() && self.is_contiguous() &&
        src.is_contiguous() && self.numel() == src.numel() && self.numel() > 0) {
        const size_t bytes = (size_t)self.numel() * self.element_size();
        ex.setStatus(pimb200_copy_2d(self.data_ptr(), bytes, src.data_ptr(), bytes, bytes, 1, ex.currentStream()));
    } else {
        at::native::copy_(self, src, cp->non_blocking != 0);
    }
    ex.updateBlob(layer->getOutSTensorID()[0], ir::DataType::TENSOR, torch::jit::IValue(self));
}

namespace {
at::Tensor aliasOrNew(StreamExecutor& ex, const ir::OutputAlias& al, at::IntArrayRef sizes, const at::TensorOptions& opt) {
    if (al.blob_id < 0 || !ex.checkValidBlobID(al.blob_id)) return at::empty(sizes, opt);
    at::Tensor buf = ex.findBlob(al.blob_id).second.toTensor();
    int64_t n = 1;
    for (auto s : sizes) n *= s;
    TORCH_CHECK(al.elem_offset + n <= buf.numel(), "aliased LSTM output does not fit its buffer");
    return buf.view({-1}).narrow(0, al.elem_offset, n).view(sizes);
}
}  // namespace

// aten::lstm, padded input: inputs = (input, hx TensorList [h0, c0]); params and flags live on the layer.
// Publishes (output, h_n, c_n).  Outputs may be slices of pre-allocated blobs (the in-place custom cat).
void executeAtenLSTM1(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& ex) {
    auto lstm = std::static_pointer_cast<ir::AtenLSTM1Layer>(layer);
    const auto& in = layer->getInSTensorID();
    const auto& outs = layer->getOutSTensorID();
    at::Tensor input = blobTensor(ex, in[0]);
    auto& hx_iv = ex.findBlob(in[1]).second;
    TORCH_CHECK(hx_iv.isTensorList(), "aten::lstm expects hx as a tensor list");
    auto hx = hx_iv.toTensorList();
    TORCH_CHECK(hx.size() == 2, "aten::lstm expects hx = [h0, c0]");
    at::Tensor h0 = hx.get(0), c0 = hx.get(1);
    TORCH_CHECK(lstm->getPackedHandle() != nullptr, "LSTM weights were not preloaded");
    TORCH_CHECK(fastHalf(input) && fastHalf(h0) && fastHalf(c0) && input.dim() == 3, "aten::lstm: fp16 CUDA tensors expected");
    input = input.contiguous(); h0 = h0.contiguous(); c0 = c0.contiguous();
    const bool bf = lstm->getBatchFirst() != 0;
    const int64_t T = bf ? input.size(1) : input.size(0), B = bf ? input.size(0) : input.size(1);
    const int64_t H = h0.size(2), D = lstm->getBidirectional() ? 2 : 1, LD = h0.size(0);
    std::vector<int64_t> ysz = bf ? std::vector<int64_t>{B, T, D * H} : std::vector<int64_t>{T, B, D * H};
    at::Tensor y = aliasOrNew(ex, lstm->out_alias[0], ysz, input.options());
    at::Tensor hn = aliasOrNew(ex, lstm->out_alias[1], {LD, B, H}, input.options());
    at::Tensor cn = aliasOrNew(ex, lstm->out_alias[2], {LD, B, H}, input.options());
    ex.setStatus(pimb200_lstm_forward(lstm->getPackedHandle(), input.data_ptr(), (int)T, (int)B, h0.data_ptr(),
                                      c0.data_ptr(), y.data_ptr(), hn.data_ptr(), cn.data_ptr(), bf ? 1 : 0,
                                      ex.currentStream()));
    ex.updateBlob(outs[0], ir::DataType::TENSOR, torch::jit::IValue(y));
    ex.updateBlob(outs[1], ir::DataType::TENSOR, torch::jit::IValue(hn));
    ex.updateBlob(outs[2], ir::DataType::TENSOR, torch::jit::IValue(cn));
}

// aten::lstm, packed sequence: inputs = (data, batch_sizes (CPU int64), hx TensorList)
void executeAtenLSTM2(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& ex) {
    auto lstm = std::static_pointer_cast<ir::AtenLSTM1Layer>(layer);
    const auto& in = layer->getInSTensorID();
    const auto& outs = layer->getOutSTensorID();
    at::Tensor data = blobTensor(ex, in[0]).contiguous();
    at::Tensor bs = blobTensor(ex, in[1]).to(at::kCPU, at::kLong).contiguous();
    auto hx = ex.findBlob(in[2]).second.toTensorList();
    at::Tensor h0 = hx.get(0).contiguous(), c0 = hx.get(1).contiguous();
    TORCH_CHECK(lstm->getPackedHandle() != nullptr, "LSTM weights were not preloaded");
    TORCH_CHECK(fastHalf(data) && fastHalf(h0) && fastHalf(c0) && data.dim() == 2, "aten::lstm: fp16 CUDA tensors expected");
    const int64_t H = h0.size(2), D = lstm->getBidirectional() ? 2 : 1;
    at::Tensor y = at::empty({data.size(0), D * H}, data.options());
    at::Tensor hn = at::empty_like(h0), cn = at::empty_like(c0);
    ex.setStatus(pimb200_lstm_forward_packed(lstm->getPackedHandle(), data.data_ptr(), bs.data_ptr<int64_t>(),
                                             (int)bs.numel(), h0.data_ptr(), c0.data_ptr(), y.data_ptr(), hn.data_ptr(),
                                             cn.data_ptr(), ex.currentStream()));
    ex.updateBlob(outs[0], ir::DataType::TENSOR, torch::jit::IValue(y));
    ex.updateBlob(outs[1], ir::DataType::TENSOR, torch::jit::IValue(hn));
    ex.updateBlob(outs[2], ir::DataType::TENSOR, torch::jit::IValue(cn));
}

// MULTISTREAM: the node's addmm/matmul layers are independent; each runs on its own side stream, ordered after the
// work already queued on the main stream, and the main stream waits for all of them.  The cursor then skips the
// copies of those layers that follow the node in the flat list.
void executeMultiStream(std::shared_ptr<ir::NNLayer>& layer, StreamExecutor& ex) {
    auto ms = std::static_pointer_cast<ir::MultiStreamLayer>(layer);
    const auto& pool = ex.streamPool();
    cudaStream_t main = ex.currentStream();
    cudaEvent_t fork = nullptr;
    cudaEventCreateWithFlags(&fork, cudaEventDisableTiming);
    cudaEventRecord(fork, main);
    std::vector<cudaEvent_t> joins;
    int i = 0;
    for (auto sub : ms->getLayers()) {
        cudaStream_t st = pool.empty() ? main : pool[i % pool.size()];
        if (st != main) cudaStreamWaitEvent(st, fork, 0);
        if (sub->getType() == ir::LayerType::ATENADDMM) executeAtenAddmmWithStream(sub, ex, st);
        else if (sub->getType() == ir::LayerType::ATENMATMUL) executeAtenMatmulWithStream(sub, ex, st);
        else ex.setStatus(PIMB200_ERR_UNSUPPORTED);
        if (st != main) {
            cudaEvent_t j = nullptr;
            cudaEventCreateWithFlags(&j, cudaEventDisableTiming);
            cudaEventRecord(j, st);
            joins.push_back(j);
        }
        ++i;
    }
    for (auto j : joins) {
        cudaStreamWaitEvent(main, j, 0);
        cudaEventDestroy(j);
    }
    cudaEventDestroy(fork);
    ex.setCursor(ex.getCursor() + 1 + ms->getLayerNum());
}

}  // namespace op_executor
}  // namespace runtime
}  // namespace nn_compiler
