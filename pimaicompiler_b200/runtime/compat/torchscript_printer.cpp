// Replacement unit for the reference's compiler/source/frontend/importer/utils/utils.cpp (a debugging printer of
// TorchScript graphs), which no longer compiles against libtorch 2.x (torch::jit::Function::graph moved to
// GraphFunction, :133).  Implements the interface of compiler/include/frontend/importer/utils/utils.h.
#include "frontend/importer/utils/utils.h"

#include <glog/logging.h>
#include <torch/csrc/jit/api/function_impl.h>

namespace nn_compiler {
namespace frontend {

int TorchscriptPrinter::printGraphRecursive(std::string filename) {
    torch::jit::Module model = torch::jit::load(filename);
    int graphs = 0;
    for (const auto& m : model.named_modules()) {
        for (const auto& method : m.value.get_methods()) {
            LOG(INFO) << m.name << "." << method.name() << ":\n" << method.graph()->toString(true);
            ++graphs;
        }
    }
    return graphs;
}

void TorchscriptPrinter::printNodeRecursive(torch::jit::Node* node, size_t level) {
    const std::string indent(2 * level, ' ');
    LOG(INFO) << indent << node->kind().toQualString() << " (" << node->inputs().size() << " in, "
              << node->outputs().size() << " out)";
    for (torch::jit::Block* block : node->blocks())
        for (torch::jit::Node* inner : block->nodes()) printNodeRecursive(inner, level + 1);
}

void TorchscriptPrinter::printScriptModelRecursive(std::string filename) {
    torch::jit::Module model = torch::jit::load(filename);
    for (const auto& method : model.get_methods())
        for (torch::jit::Node* node : method.graph()->nodes()) printNodeRecursive(node, 0);
}

}  // namespace frontend
}  // namespace nn_compiler
