// ops::AddN: the sum of num_inputs tensors of one shape
// (reference: include/tim/vx/ops/addn.h:40-45, src/tim/vx/ops/addn.cc:33-41; lowered by
// src/tim/vx/internal/src/ops/vsi_nn_op_addn.c:124-205 to a chain of Add nodes).
#ifndef TIM_VX_OPS_ADDN_H_
#define TIM_VX_OPS_ADDN_H_

#include "tim/vx/builtin_op.h"

namespace tim {
namespace vx {
namespace ops {

class AddN : public BuiltinOp {
 public:
  AddN(Graph* graph, uint32_t num_inputs);
  std::shared_ptr<Operation> Clone(std::shared_ptr<Graph>& graph) const override;
};

}  // namespace ops
}  // namespace vx
}  // namespace tim
#endif  // TIM_VX_OPS_ADDN_H_
