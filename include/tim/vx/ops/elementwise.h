// tim::vx::ops::Add — quantized elementwise addition
// (reference: include/tim/vx/ops/elementwise.h:69-79).  The reference header
// also declares Minimum, Maximum, Sub, Pow, FloorDiv, Multiply and Div; of the
// elementwise family only the residual Add lies on the quantized CNN path.
#ifndef TIM_VX_OPS_ELEMENTWISE_H_
#define TIM_VX_OPS_ELEMENTWISE_H_

#include "tim/vx/builtin_op.h"

namespace tim {
namespace vx {
namespace ops {

class Add : public BuiltinOp {
 public:
  Add(Graph* graph);
  std::shared_ptr<Operation> Clone(std::shared_ptr<Graph>& graph) const override;
};

}  // namespace ops
}  // namespace vx
}  // namespace tim
#endif  // TIM_VX_OPS_ELEMENTWISE_H_
