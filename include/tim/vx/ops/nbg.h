// tim::vx::ops::NBG (reference: include/tim/vx/ops/nbg.h:33-46): an op that stands for a whole
// serialised graph.  `binary` is what Graph::CompileToBinary wrote (this backend's own format; the
// blob states its length in its header); the op's inputs and outputs are bound in the order of the
// serialised graph's InputsTensor() / OutputsTensor().  At Compile the op is expanded into the nodes it
// describes, planned for the GPU the loading graph is bound to.
#ifndef TIM_VX_OPS_NBG_H_
#define TIM_VX_OPS_NBG_H_

#include <cstddef>

#include "tim/vx/builtin_op.h"

namespace tim {
namespace vx {
namespace ops {

class NBG : public BuiltinOp {
 public:
  NBG(Graph* graph, const char* binary, size_t input_count, size_t output_count);
  std::shared_ptr<Operation> Clone(std::shared_ptr<Graph>& graph) const override;
};

}  // namespace ops
}  // namespace vx
}  // namespace tim
#endif  // TIM_VX_OPS_NBG_H_
