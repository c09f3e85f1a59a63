// ops::InstanceNormalization (reference: include/tim/vx/ops/instancenormalization.h:31-39).  Declared so that
// programs naming it build; not executed by this backend: Graph::Compile fails, naming the op.
#ifndef TIM_VX_OPS_INSTANCENORMALIZATION_H_
#define TIM_VX_OPS_INSTANCENORMALIZATION_H_

#include "tim/vx/builtin_op.h"

namespace tim {
namespace vx {
namespace ops {

class InstanceNormalization : public BuiltinOp {
 public:
  InstanceNormalization(Graph* graph, float eps = 1e-5f, DataLayout input_layout = DataLayout::WHCN);
  std::shared_ptr<Operation> Clone(std::shared_ptr<Graph>& graph) const override;

 protected:
  float eps_;
};

}  // namespace ops
}  // namespace vx
}  // namespace tim
#endif  // TIM_VX_OPS_INSTANCENORMALIZATION_H_
