// Tensor-level bodies of the hot-path operators, independent of any graph IR: each takes libtorch tensors plus the
// operator's attributes, runs the device work through the pimb200 C ABI when the operands have a hot-path form (fp16,
// CUDA, the vector / row shapes the reference offloads or hand-codes) and otherwise makes the libtorch call the
// reference's executor makes (runtime/source/executor/op_executor/aten_ops.cpp).  Both op-executor sets of this
// library (the one over the minimal IR and the one compiled against the reference's own IR headers) are thin
// adapters over these functions.
#pragma once
#include <cuda_runtime_api.h>
#include <torch/torch.h>

#include <tuple>
#include <vector>

struct pimb200_lstm;

namespace nn_compiler {
namespace runtime {
namespace tensor_ops {

// Per-call context: the stream to launch on, the first non-zero C-ABI status, and whether the call left the fast path.
struct OpContext {
    cudaStream_t stream = nullptr;
    int status = 0;
    void note(int rc) {
        if (rc != 0 && status == 0) status = rc;
    }
};

// How often an operator fell back to the libtorch call since the last reset (process-wide).  Tests of hot shapes
// assert that it stays zero.
long fallbackCount();
// MULTISTREAM nodes issued as one grouped launch since the process started (tests assert the path taken)
long groupedLaunchCount();
void resetFallbackCount();

// shape classes of the reference's GEMM router (runtime/include/executor/utils/utils.h:30-36,
// runtime/source/executor/utils/utils.cpp:293-396) on shapes padded to rank 4
enum class GEMM_TYPE { VV, VM, MV, MM, UNKNOW };
std::vector<int64_t> pad4(at::IntArrayRef shape);   // leading ones up to rank 4
GEMM_TYPE getGemmType(const std::vector<int64_t>& self_shape, const std::vector<int64_t>& other_shape);

// out = act(beta * self + alpha * mat1 @ mat2)   (customAtenAddmm, aten_ops.cpp:609-758)
at::Tensor addmm(OpContext& cx, const at::Tensor& self, const at::Tensor& mat1, const at::Tensor& mat2, double beta,
                 double alpha, bool relu);
// out = a @ b   (customAtenMatmul, aten_ops.cpp:760-932)
at::Tensor matmul(OpContext& cx, const at::Tensor& a, const at::Tensor& b);
// The branches of a MULTISTREAM node (stream_ops_executor.cpp:27-50): independent addmm / matmul products.  All of them
// in one grouped launch when every branch is a matrix-class fp16 product (bias indexed by the row of mat1, as in the
// reference's MM branch); an empty vector otherwise (the caller then runs branch by branch on side streams).
struct MatmulBranch {
    at::Tensor bias;   // 1-D or undefined
    at::Tensor mat1, mat2;
    bool relu = false;
};
std::vector<at::Tensor> groupedMatmul(OpContext& cx, const std::vector<MatmulBranch>& branches);
// out = x @ W^T + b   (atenLinear, aten_ops.cpp:304-307)
at::Tensor linear(OpContext& cx, const at::Tensor& x, const at::Tensor& W, const at::Tensor& b);
// out = a + alpha * b   (custom_add for fp16 same-shape / row-broadcast operands, aten_ops_executor.cpp:43-179)
at::Tensor add(OpContext& cx, const at::Tensor& a, const at::Tensor& b, double alpha);
at::Tensor softmax(OpContext& cx, const at::Tensor& x, int64_t dim, bool log);
at::Tensor argmax(OpContext& cx, const at::Tensor& x, int64_t dim, bool keepdim);
// (values, indices) = topk(x, k, dim, largest, sorted)   (atenTopk; the device kernel returns the picks in order)
std::tuple<at::Tensor, at::Tensor> topk(OpContext& cx, const at::Tensor& x, int64_t k, int64_t dim, bool largest, bool sorted);
at::Tensor layerNorm(OpContext& cx, const at::Tensor& x, const std::vector<int64_t>& normalized_shape, const at::Tensor& weight,
                     const at::Tensor& bias, double eps);
at::Tensor tanh(OpContext& cx, const at::Tensor& x);
at::Tensor maskedFill(OpContext& cx, const at::Tensor& x, const at::Tensor& mask, double value);
// table[idx]; indices already on the device stay there (the reference reads them back, aten_ops_executor.cpp:1276-1287)
at::Tensor embedding(OpContext& cx, const at::Tensor& table, const at::Tensor& idx);
// x[1,1,k] @ A[1,k,n] through the single-row kernel (bmm_kernel_xAy, custom_ops.h:435-466); else at::bmm
at::Tensor bmm(OpContext& cx, const at::Tensor& x, const at::Tensor& A);
at::Tensor cat(OpContext& cx, const std::vector<at::Tensor>& ts, int64_t dim);
// self.copy_(src); returns self
at::Tensor copy_(OpContext& cx, at::Tensor self, const at::Tensor& src, bool non_blocking);

// aten::lstm through a packed-weight handle.  `y`, `hn`, `cn` may be given (views into pre-allocated buffers: the
// in-place "custom cat" of the GNMT graphs, miopen_ops_executor.cpp:193-228); undefined ones are allocated.
struct LstmResult {
    at::Tensor y, hn, cn;
};
LstmResult lstm(OpContext& cx, pimb200_lstm* handle, const at::Tensor& input, const at::Tensor& h0, const at::Tensor& c0,
                bool batch_first, bool bidirectional, LstmResult out = {});
LstmResult lstmPacked(OpContext& cx, pimb200_lstm* handle, const at::Tensor& data, const at::Tensor& batch_sizes,
                      const at::Tensor& h0, const at::Tensor& c0, bool bidirectional);
// packs an at::lstm flat parameter list (CUDA fp16, contiguous) into a handle; nullptr + status on failure
pimb200_lstm* lstmPack(OpContext& cx, const std::vector<at::Tensor>& params, int64_t num_layers, bool bidirectional,
                       bool has_biases);

}  // namespace tensor_ops
}  // namespace runtime
}  // namespace nn_compiler
