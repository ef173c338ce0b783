// Tensor-level bodies of the hot-path operators (see tensor_ops.h).
#include "tensor_ops.h"

#include <atomic>

#include "pimb200.h"

namespace nn_compiler {
namespace runtime {
namespace tensor_ops {

namespace {
std::atomic<long> g_fallbacks{0};
void fellBack() { g_fallbacks.fetch_add(1, std::memory_order_relaxed); }

bool fastHalf(const at::Tensor& t) { return t.defined() && t.is_cuda() && t.scalar_type() == at::kHalf; }
bool lastDim(const at::Tensor& t, int64_t dim) { return t.dim() >= 1 && (dim == -1 || dim == t.dim() - 1); }
// True when `t` ([K, C] logically) is a transposed view of a contiguous [C, K] matrix, i.e. already K-major.
bool isTransposedKMajor(const at::Tensor& t) { return t.dim() == 2 && t.stride(1) == t.size(0) && t.stride(0) == 1; }
c10::optional<at::Tensor> opt(const at::Tensor& t) { return t.defined() ? c10::optional<at::Tensor>(t) : c10::nullopt; }

// out = act(L @ R + bias) for the shapes the hot path produces; an undefined tensor when the shape is not one of them
// (the caller then makes the library call).  `bias` is 1-D or undefined.  On the vector paths the graph's alpha / beta
// are 1 (the reference hard-sets them, aten_ops.cpp:627-628).
at::Tensor fusedMatmul(OpContext& cx, at::Tensor L, at::Tensor R, const at::Tensor& bias, bool relu) {
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
    if (Kr != K) return {};
    const at::Tensor b = bias.defined() ? bias.contiguous() : bias;
    const void* bp = b.defined() ? b.data_ptr() : nullptr;
    at::Tensor out;
    int rc = PIMB200_OK;
    if (R.numel() != Kr * colsR) {
        // a batched right operand: only the stack of column vectors [J, K, 1] under a weight matrix [N, K], which is
        // what SwapAddmmInputs makes of a linear layer over a sequence of J rows (transpose, addmm, transpose back)
        if (L.dim() != 2 || R.dim() != 3 || colsR != 1 || (b.defined() && b.numel() != rowsL)) return {};
        at::Tensor W = L.contiguous();
        at::Tensor X = R.squeeze(-1).contiguous();              // [J, K]; the transposed view of a contiguous [J, 1, K]
        const int64_t J = X.size(0);
        out = at::empty({J, rowsL}, L.options());
        rc = pimb200_gemm_wx(W.data_ptr(), X.data_ptr(), bp, out.data_ptr(), (int)rowsL, (int)K, (int)J, (int)K, (int)rowsL,
                             act, 0, cx.stream);
        cx.note(rc);
        if (rc != PIMB200_OK) return {};
        return out.reshape(out_sizes);
    }
    const GEMM_TYPE type = getGemmType(pad4({rowsL, K}), pad4({K, colsR}));
    if (type == GEMM_TYPE::VV) {
        L = L.contiguous(); R = R.contiguous();
        out = at::empty({1}, L.options());
        rc = pimb200_dot_vv(L.data_ptr(), R.data_ptr(), out.data_ptr(), (int)K, cx.stream);
        if (rc == PIMB200_OK && b.defined()) out = relu ? at::relu(out + b) : out + b;
        else if (relu) out = at::relu(out);
    } else if (type == GEMM_TYPE::VM) {
        if (b.defined() && b.numel() != colsR) return {};
        L = L.contiguous();
        at::Tensor A = R.reshape({K, colsR}).contiguous();
        out = at::empty({colsR}, L.options());
        rc = pimb200_gemv_vm(L.data_ptr(), A.data_ptr(), bp, out.data_ptr(), (int)K, (int)colsR, act, cx.stream);
    } else if (type == GEMM_TYPE::MV) {
        if (b.defined() && b.numel() != rowsL) return {};
        at::Tensor W = L.reshape({rowsL, K}).contiguous();
        R = R.contiguous();
        out = at::empty({rowsL}, L.options());
        rc = pimb200_gemv_mv(W.data_ptr(), R.data_ptr(), bp, out.data_ptr(), (int)rowsL, (int)K, act, cx.stream);
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
                                 (int)K, (int)rowsL, act, 0, cx.stream);
            out = Yt.t();
        } else {
            out = at::empty({rowsL, colsR}, L.options());
            rc = pimb200_gemm_wx(Rt.data_ptr(), Lm.data_ptr(), nullptr, out.data_ptr(), (int)colsR, (int)K, (int)rowsL,
                                 (int)K, (int)colsR, act, 0, cx.stream);
        }
    }
    cx.note(rc);
    if (rc != PIMB200_OK) return {};
    return out.reshape(out_sizes);
}
}  // namespace

long fallbackCount() { return g_fallbacks.load(std::memory_order_relaxed); }
static std::atomic<long> g_grouped{0};
long groupedLaunchCount() { return g_grouped.load(std::memory_order_relaxed); }
void resetFallbackCount() { g_fallbacks.store(0, std::memory_order_relaxed); }

std::vector<int64_t> pad4(at::IntArrayRef s) {
    std::vector<int64_t> v(s.begin(), s.end());
    while (v.size() < 4) v.insert(v.begin(), 1);
    return v;
}

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

at::Tensor addmm(OpContext& cx, const at::Tensor& self, const at::Tensor& mat1, const at::Tensor& mat2, double beta,
                 double alpha, bool relu) {
    at::Tensor out;
    if (alpha == 1.0 && beta == 1.0 && self.dim() == 1) out = fusedMatmul(cx, mat1, mat2, self, relu);
    if (out.defined() || cx.status != 0) return out;
    fellBack();
    at::Tensor s = self;
    if (self.dim() == 1 && mat2.dim() >= 2 && self.size(0) == mat1.size(-2) && self.size(0) != mat2.size(-1))
        s = self.unsqueeze(1);  // per-row bias of the swapped form
    if (mat1.dim() > 2 || mat2.dim() > 2) {
        // operands with leading extents (a sequence of rows behind SwapAddmmInputs' transposes): matmul's shape rule
        out = at::matmul(mat1, mat2);
        if (alpha != 1.0) out = out * alpha;
        out = out + (beta == 1.0 ? s : s * beta);
    } else {
        out = at::addmm(s, mat1, mat2, beta, alpha);
    }
    return relu ? at::relu(out) : out;
}

at::Tensor matmul(OpContext& cx, const at::Tensor& a, const at::Tensor& b) {
    at::Tensor out = fusedMatmul(cx, a, b, at::Tensor(), false);
    if (out.defined() || cx.status != 0) return out;
    fellBack();
    return at::matmul(a, b);
}

std::vector<at::Tensor> groupedMatmul(OpContext& cx, const std::vector<MatmulBranch>& branches) {
    const size_t n = branches.size();
    if (n < 2) return {};
    std::vector<pimb200_gemm_problem> pr(n);
    std::vector<at::Tensor> keep, outs(n);          // operands made contiguous live until the launch is queued
    std::vector<std::vector<int64_t>> shapes(n);
    std::vector<bool> transposed(n, false);
    const bool any_relu = branches[0].relu;
    for (size_t i = 0; i < n; ++i) {
        const MatmulBranch& br = branches[i];
        const at::Tensor& L = br.mat1;
        const at::Tensor& R = br.mat2;
        if (br.relu != any_relu || !fastHalf(L) || !fastHalf(R) || L.dim() < 2 || R.dim() != 2) return {};
        if (br.bias.defined() && (!fastHalf(br.bias) || br.bias.dim() != 1)) return {};
        const int64_t K = L.size(-1), rowsL = L.numel() / K, colsR = R.size(1);
        if (R.size(0) != K || rowsL < 2 || colsR < 2) return {};      // vector classes keep their own kernels
        at::Tensor Lm = L.reshape({rowsL, K}).contiguous();
        at::Tensor Rt = isTransposedKMajor(R) ? R.t() : R.t().contiguous();      // [colsR, K], K-major
        keep.push_back(Lm);
        keep.push_back(Rt);
        auto sizes = L.sizes().vec();
        sizes.back() = colsR;
        shapes[i] = sizes;
        pimb200_gemm_problem& q = pr[i];
        q.act = br.relu ? PIMB200_ACT_RELU : PIMB200_ACT_NONE;
        q.y_is_f32 = 0;
        q.K = (int)K;
        q.ldx = (int)K;
        if (br.bias.defined()) {
            if (br.bias.numel() != rowsL) return {};
            at::Tensor b = br.bias.contiguous();
            keep.push_back(b);
            outs[i] = at::empty({colsR, rowsL}, L.options());         // Y^T[c, r]
            transposed[i] = true;
            q.W = Lm.data_ptr(); q.X = Rt.data_ptr(); q.bias = b.data_ptr(); q.Y = outs[i].data_ptr();
            q.N = (int)rowsL; q.J = (int)colsR; q.ldy = (int)rowsL;
        } else {
            outs[i] = at::empty({rowsL, colsR}, L.options());
            q.W = Rt.data_ptr(); q.X = Lm.data_ptr(); q.bias = nullptr; q.Y = outs[i].data_ptr();
            q.N = (int)colsR; q.J = (int)rowsL; q.ldy = (int)colsR;
        }
    }
    const int rc = pimb200_gemm_wx_grouped(pr.data(), (int)n, cx.stream);
    cx.note(rc);
    if (rc != PIMB200_OK) return {};
    g_grouped.fetch_add(1, std::memory_order_relaxed);
    for (size_t i = 0; i < n; ++i) outs[i] = (transposed[i] ? outs[i].t() : outs[i]).reshape(shapes[i]);
    return outs;
}

at::Tensor linear(OpContext& cx, const at::Tensor& x, const at::Tensor& W, const at::Tensor& b) {
    if (fastHalf(x) && fastHalf(W) && W.dim() == 2 && x.dim() >= 1 && x.size(-1) == W.size(1) && (!b.defined() || fastHalf(b))) {
        const int64_t K = W.size(1), N = W.size(0), J = x.numel() / K;
        at::Tensor xc = x.contiguous(), Wc = W.contiguous(), bc = b.defined() ? b.contiguous() : b;
        auto sizes = x.sizes().vec();
        sizes.back() = N;
        at::Tensor out = at::empty(sizes, x.options());
        const void* bp = bc.defined() ? bc.data_ptr() : nullptr;
        cx.note(J == 1 ? pimb200_gemv_mv(Wc.data_ptr(), xc.data_ptr(), bp, out.data_ptr(), (int)N, (int)K, PIMB200_ACT_NONE,
                                         cx.stream)
                       : pimb200_gemm_wx(Wc.data_ptr(), xc.data_ptr(), bp, out.data_ptr(), (int)N, (int)K, (int)J, (int)K,
                                         (int)N, PIMB200_ACT_NONE, 0, cx.stream));
        return out;
    }
    fellBack();
    return at::linear(x, W, opt(b));
}

// fp16 add: same shape, or the second operand one row broadcast over the rows of the first.  aten::add is functional,
// so the result is a new tensor (the reference's kernel writes in place into its first operand).
at::Tensor add(OpContext& cx, const at::Tensor& a, const at::Tensor& b, double alpha) {
    const bool same = a.sizes() == b.sizes();
    const bool row = !same && a.dim() >= 1 && b.numel() == a.size(-1) && (b.dim() == 0 || b.size(-1) == a.size(-1));
    if (alpha == 1.0 && fastHalf(a) && fastHalf(b) && (same || row) && a.numel() > 0) {
        at::Tensor ac = a.contiguous(), bc = b.contiguous();
        at::Tensor out = at::empty_like(ac);
        const int n = (int)ac.size(-1), m = (int)(ac.numel() / n);
        cx.note(pimb200_add_f16(ac.data_ptr(), bc.data_ptr(), out.data_ptr(), m, n, row ? 1 : 0, cx.stream));
        return out;
    }
    fellBack();
    // libtorch rejects a floating-point alpha on integral operands
    const bool integral = c10::isIntegralType(a.scalar_type(), true) && c10::isIntegralType(b.scalar_type(), true);
    return integral ? at::add(a, b, c10::Scalar((int64_t)alpha)) : at::add(a, b, c10::Scalar(alpha));
}

at::Tensor softmax(OpContext& cx, const at::Tensor& x, int64_t dim, bool log) {
    if (fastHalf(x) && lastDim(x, dim) && x.numel() > 0) {
        at::Tensor xc = x.contiguous();
        at::Tensor out = at::empty_like(xc);
        const long cols = (long)xc.size(-1), rows = (long)(xc.numel() / cols);
        cx.note(pimb200_softmax_rows(xc.data_ptr(), out.data_ptr(), rows, cols, log ? 1 : 0, cx.stream));
        return out;
    }
    fellBack();
    return log ? at::log_softmax(x, dim) : at::softmax(x, dim);
}

at::Tensor argmax(OpContext& cx, const at::Tensor& x, int64_t dim, bool keepdim) {
    if (fastHalf(x) && lastDim(x, dim) && x.numel() > 0) {
        at::Tensor xc = x.contiguous();
        auto sizes = xc.sizes().vec();
        const long cols = (long)sizes.back(), rows = (long)(xc.numel() / cols);
        if (keepdim) sizes.back() = 1;
        else sizes.pop_back();
        at::Tensor out = at::empty(sizes, xc.options().dtype(at::kLong));
        cx.note(pimb200_argmax_rows(xc.data_ptr(), reinterpret_cast<long long*>(out.data_ptr<int64_t>()), rows, cols, cx.stream));
        return out;
    }
    fellBack();
    return at::argmax(x, dim, keepdim);
}

std::tuple<at::Tensor, at::Tensor> topk(OpContext& cx, const at::Tensor& x, int64_t k, int64_t dim, bool largest, bool sorted) {
    if (fastHalf(x) && lastDim(x, dim) && x.numel() > 0 && k >= 1 && k <= 64 && k <= x.size(-1)) {
        at::Tensor xc = x.contiguous();
        auto sizes = xc.sizes().vec();
        const long cols = (long)sizes.back(), rows = (long)(xc.numel() / cols);
        sizes.back() = k;
        at::Tensor vals = at::empty(sizes, xc.options());
        at::Tensor idx = at::empty(sizes, xc.options().dtype(at::kLong));
        cx.note(pimb200_topk_rows(xc.data_ptr(), vals.data_ptr(), reinterpret_cast<long long*>(idx.data_ptr<int64_t>()), rows, cols,
                                  (int)k, largest ? 1 : 0, cx.stream));
        return {vals, idx};
    }
    fellBack();
    return at::topk(x, k, dim, largest, sorted);
}

at::Tensor layerNorm(OpContext& cx, const at::Tensor& x, const std::vector<int64_t>& normalized_shape, const at::Tensor& weight,
                     const at::Tensor& bias, double eps) {
    const bool one_dim = normalized_shape.size() == 1 && x.dim() >= 1 && normalized_shape[0] == x.size(-1);
    if (fastHalf(x) && one_dim && x.numel() > 0 && (!weight.defined() || fastHalf(weight)) && (!bias.defined() || fastHalf(bias))) {
        at::Tensor xc = x.contiguous();
        at::Tensor out = at::empty_like(xc);
        const long cols = (long)xc.size(-1), rows = (long)(xc.numel() / cols);
        at::Tensor w = weight.defined() ? weight.contiguous() : at::Tensor();
        at::Tensor b = bias.defined() ? bias.contiguous() : at::Tensor();
        cx.note(pimb200_layer_norm_rows(xc.data_ptr(), w.defined() ? w.data_ptr() : nullptr, b.defined() ? b.data_ptr() : nullptr,
                                        out.data_ptr(), rows, cols, (float)eps, cx.stream));
        return out;
    }
    fellBack();
    return at::layer_norm(x, normalized_shape, opt(weight), opt(bias), eps);
}

at::Tensor tanh(OpContext& cx, const at::Tensor& x) {
    if (fastHalf(x) && x.numel() > 0) {
        at::Tensor xc = x.contiguous();
        at::Tensor out = at::empty_like(xc);
        cx.note(pimb200_tanh_f16(xc.data_ptr(), out.data_ptr(), (size_t)xc.numel(), cx.stream));
        return out;
    }
    fellBack();
    return at::tanh(x);
}

at::Tensor maskedFill(OpContext& cx, const at::Tensor& x, const at::Tensor& mask, double value) {
    const bool same = mask.sizes() == x.sizes();
    const bool row = !same && x.dim() >= 1 && mask.numel() == x.size(-1) && mask.dim() >= 1 && mask.size(-1) == x.size(-1);
    if (fastHalf(x) && mask.is_cuda() && mask.scalar_type() == at::kBool && (same || row) && x.numel() > 0) {
        at::Tensor xc = x.contiguous(), mc = mask.contiguous();
        at::Tensor out = at::empty_like(xc);
        cx.note(pimb200_masked_fill_f16(xc.data_ptr(), reinterpret_cast<const unsigned char*>(mc.data_ptr<bool>()), (float)value,
                                        out.data_ptr(), (size_t)xc.numel(), (size_t)mc.numel(), cx.stream));
        return out;
    }
    fellBack();
    return at::masked_fill(x, mask, value);
}

at::Tensor embedding(OpContext& cx, const at::Tensor& table, const at::Tensor& idx) {
    if (table.is_cuda() && table.dim() == 2 && idx.is_cuda() && idx.scalar_type() == at::kLong && idx.numel() > 0) {
        at::Tensor tc = table.contiguous(), ic = idx.contiguous();
        auto sizes = ic.sizes().vec();
        sizes.push_back(tc.size(1));
        at::Tensor out = at::empty(sizes, tc.options());
        cx.note(pimb200_gather_rows(tc.data_ptr(), reinterpret_cast<const long long*>(ic.data_ptr<int64_t>()), out.data_ptr(),
                                    (long)ic.numel(), (size_t)tc.size(1) * tc.element_size(), (long)tc.size(0), cx.stream));
        return out;
    }
    fellBack();
    return at::embedding(table, idx.to(table.device()));
}

at::Tensor bmm(OpContext& cx, const at::Tensor& x, const at::Tensor& A) {
    if (fastHalf(x) && fastHalf(A) && x.dim() == 3 && A.dim() == 3 && x.size(0) == 1 && A.size(0) == 1 && x.size(1) == 1 &&
        x.size(2) == A.size(1)) {
        at::Tensor xc = x.contiguous(), Ac = A.contiguous();
        at::Tensor out = at::empty({1, 1, A.size(2)}, x.options());
        cx.note(pimb200_bmm_row(xc.data_ptr(), Ac.data_ptr(), out.data_ptr(), (int)A.size(1), (int)A.size(2), cx.stream));
        return out;
    }
    fellBack();
    return at::bmm(x, A);
}

at::Tensor cat(OpContext& cx, const std::vector<at::Tensor>& ts, int64_t dim_) {
    TORCH_CHECK(!ts.empty(), "aten::cat of an empty list");
    bool fast = true;
    for (auto& t : ts) fast = fast && t.is_cuda() && t.scalar_type() == ts[0].scalar_type() && t.dim() == ts[0].dim();
    if (fast && ts[0].dim() > 0) {
        const int64_t nd = ts[0].dim(), dim = (dim_ % nd + nd) % nd;
        auto sizes = ts[0].sizes().vec();
        int64_t total = 0;
        for (auto& t : ts) total += t.size(dim);
        sizes[dim] = total;
        at::Tensor out = at::empty(sizes, ts[0].options());
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
            cx.note(pimb200_cat(out.data_ptr(), src.data(), inner.data(), (int)src.size(), (size_t)outer, cx.stream));
        return out;
    }
    fellBack();
    return at::cat(ts, dim_);
}

// device-to-device copies of equal dtype go through the strided copy kernel; host<->device and converting copies stay
// with the library (runtime/unit-tests/aten_ops_ut.cpp:43-63 exercises both directions)
at::Tensor copy_(OpContext& cx, at::Tensor self, const at::Tensor& src, bool non_blocking) {
    if (self.is_cuda() && src.is_cuda() && self.scalar_type() == src.scalar_type() && self.is_contiguous() &&
        src.is_contiguous() && self.numel() == src.numel() && self.numel() > 0) {
        const size_t bytes = (size_t)self.numel() * self.element_size();
        cx.note(pimb200_copy_2d(self.data_ptr(), bytes, src.data_ptr(), bytes, bytes, 1, cx.stream));
    } else {
        at::native::copy_(self, src, non_blocking);   // not a hot shape by definition (host side or converting): not counted
    }
    return self;
}

LstmResult lstm(OpContext& cx, pimb200_lstm* handle, const at::Tensor& input_, const at::Tensor& h0_, const at::Tensor& c0_,
                bool bf, bool bidirectional, LstmResult out) {
    TORCH_CHECK(handle != nullptr, "LSTM weights were not preloaded");
    TORCH_CHECK(fastHalf(input_) && fastHalf(h0_) && fastHalf(c0_) && input_.dim() == 3, "aten::lstm: fp16 CUDA tensors expected");
    at::Tensor input = input_.contiguous(), h0 = h0_.contiguous(), c0 = c0_.contiguous();
    const int64_t T = bf ? input.size(1) : input.size(0), B = bf ? input.size(0) : input.size(1);
    const int64_t H = h0.size(2), D = bidirectional ? 2 : 1, LD = h0.size(0);
    if (!out.y.defined()) out.y = at::empty(bf ? std::vector<int64_t>{B, T, D * H} : std::vector<int64_t>{T, B, D * H}, input.options());
    if (!out.hn.defined()) out.hn = at::empty({LD, B, H}, input.options());
    if (!out.cn.defined()) out.cn = at::empty({LD, B, H}, input.options());
    TORCH_CHECK(out.y.is_contiguous() && out.hn.is_contiguous() && out.cn.is_contiguous(), "aten::lstm outputs must be contiguous");
    cx.note(pimb200_lstm_forward(handle, input.data_ptr(), (int)T, (int)B, h0.data_ptr(), c0.data_ptr(), out.y.data_ptr(),
                                 out.hn.data_ptr(), out.cn.data_ptr(), bf ? 1 : 0, cx.stream));
    return out;
}

LstmResult lstmPacked(OpContext& cx, pimb200_lstm* handle, const at::Tensor& data_, const at::Tensor& batch_sizes,
                      const at::Tensor& h0_, const at::Tensor& c0_, bool bidirectional) {
    TORCH_CHECK(handle != nullptr, "LSTM weights were not preloaded");
    at::Tensor data = data_.contiguous(), h0 = h0_.contiguous(), c0 = c0_.contiguous();
    at::Tensor bs = batch_sizes.to(at::kCPU, at::kLong).contiguous();
    TORCH_CHECK(fastHalf(data) && fastHalf(h0) && fastHalf(c0) && data.dim() == 2, "aten::lstm: fp16 CUDA tensors expected");
    const int64_t H = h0.size(2), D = bidirectional ? 2 : 1;
    LstmResult out;
    out.y = at::empty({data.size(0), D * H}, data.options());
    out.hn = at::empty_like(h0);
    out.cn = at::empty_like(c0);
    cx.note(pimb200_lstm_forward_packed(handle, data.data_ptr(), bs.data_ptr<int64_t>(), (int)bs.numel(), h0.data_ptr(),
                                        c0.data_ptr(), out.y.data_ptr(), out.hn.data_ptr(), out.cn.data_ptr(), cx.stream));
    return out;
}

pimb200_lstm* lstmPack(OpContext& cx, const std::vector<at::Tensor>& params, int64_t num_layers, bool bidirectional,
                       bool has_biases) {
    if (params.size() < 2) { cx.note(PIMB200_ERR_BAD_ARG); return nullptr; }
    std::vector<const void*> ptrs;
    for (auto& p : params) {
        if (!p.is_cuda() || p.scalar_type() != at::kHalf || !p.is_contiguous()) { cx.note(PIMB200_ERR_UNSUPPORTED); return nullptr; }
        ptrs.push_back(p.data_ptr());
    }
    pimb200_lstm* h = nullptr;
    cx.note(pimb200_lstm_create(ptrs.data(), (int)ptrs.size(), (int)num_layers, bidirectional ? 1 : 0, (int)params[0].size(1),
                                (int)params[1].size(1), has_biases ? 1 : 0, &h));
    return h;
}

}  // namespace tensor_ops
}  // namespace runtime
}  // namespace nn_compiler
