// Op executors registered by ir::LayerType (names as in the reference's
// runtime/include/executor/op_executor/{aten_ops_executor,prim_ops_executor,stream_ops_executor}.h).
#pragma once
#include "executor/stream_executor.h"

namespace nn_compiler {
namespace runtime {
namespace op_executor {

using Layer = std::shared_ptr<nn_compiler::ir::NNLayer>;

// ---- hot path: device work through the pimb200 C ABI ----
void executeAtenAdd(Layer& layer, StreamExecutor& stream_executor);
void executeAtenAddmm(Layer& layer, StreamExecutor& stream_executor);
void executeAtenBmm(Layer& layer, StreamExecutor& stream_executor);
void executeAtenCat(Layer& layer, StreamExecutor& stream_executor);
void executeAtenCopy(Layer& layer, StreamExecutor& stream_executor);
void executeAtenEmbedding(Layer& layer, StreamExecutor& stream_executor);
void executeAtenLinear(Layer& layer, StreamExecutor& stream_executor);
void executeAtenLSTM1(Layer& layer, StreamExecutor& stream_executor);
void executeAtenLSTM2(Layer& layer, StreamExecutor& stream_executor);
void executeAtenMatmul(Layer& layer, StreamExecutor& stream_executor);
void executeAtenSoftmax(Layer& layer, StreamExecutor& stream_executor);
void executeAtenLogSoftmax(Layer& layer, StreamExecutor& stream_executor);
void executeAtenArgmax(Layer& layer, StreamExecutor& stream_executor);
void executeAtenTopk(Layer& layer, StreamExecutor& stream_executor);
void executeAtenTanh(Layer& layer, StreamExecutor& stream_executor);
void executeMultiStream(Layer& layer, StreamExecutor& stream_executor);

// ---- pass-through adapters (one libtorch call each, no arithmetic of this library) ----
void executeAtenItem(Layer& layer, StreamExecutor& stream_executor);
void executeAtenCompare(Layer& layer, StreamExecutor& stream_executor);   // gt / lt / ge / le / eq / ne by layer type
void executeAtenTranspose(Layer& layer, StreamExecutor& stream_executor);
void executeAtenSelect(Layer& layer, StreamExecutor& stream_executor);
void executeAtenRelu(Layer& layer, StreamExecutor& stream_executor);
void executeAtenSize(Layer& layer, StreamExecutor& stream_executor);
void executeAtenInt(Layer& layer, StreamExecutor& stream_executor);
void executeAtenUnsqueeze(Layer& layer, StreamExecutor& stream_executor);

// ---- prim ops: constants, containers, control flow ----
void executePrimConstant(Layer& layer, StreamExecutor& stream_executor);
void executePrimVariable(Layer& layer, StreamExecutor& stream_executor);
void executePrimListConstruct(Layer& layer, StreamExecutor& stream_executor);
void executePrimListUnpack(Layer& layer, StreamExecutor& stream_executor);
void executePrimTupleConstruct(Layer& layer, StreamExecutor& stream_executor);
void executePrimTupleUnpack(Layer& layer, StreamExecutor& stream_executor);
void executePrimTupleIndex(Layer& layer, StreamExecutor& stream_executor);
void executePrimIf(Layer& layer, StreamExecutor& stream_executor);
void executePrimEndIf(Layer& layer, StreamExecutor& stream_executor);
void executePrimLoop(Layer& layer, StreamExecutor& stream_executor);
void executePrimLoopIndex(Layer& layer, StreamExecutor& stream_executor);
void executePrimBlock(Layer& layer, StreamExecutor& stream_executor);
void executePrimEndLoop(Layer& layer, StreamExecutor& stream_executor);

}  // namespace op_executor
}  // namespace runtime
}  // namespace nn_compiler
