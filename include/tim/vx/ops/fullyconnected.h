// tim::vx::ops::FullyConnected (reference: include/tim/vx/ops/fullyconnected.h:44-45).
// Inputs {x, w[, bias]}: dims [0..axis] of x are flattened into K (dim 0
// fastest), the rest is the batch; w [K, N]; output [N, batch...].
#ifndef TIM_VX_OPS_FULLYCONNECTED_H_
#define TIM_VX_OPS_FULLYCONNECTED_H_

#include "tim/vx/builtin_op.h"

namespace tim {
namespace vx {
namespace ops {

class FullyConnected : public BuiltinOp {
 public:
  FullyConnected(Graph* graph, uint32_t axis);
  FullyConnected(Graph* graph, uint32_t axis, uint32_t weights);

  std::shared_ptr<Operation> Clone(std::shared_ptr<Graph>& graph) const override;

 protected:
  uint32_t axis_;
  uint32_t weights_;
};

}  // namespace ops
}  // namespace vx
}  // namespace tim
#endif  // TIM_VX_OPS_FULLYCONNECTED_H_
