// tim::vx::ops::Softmax (reference: include/tim/vx/ops/softmax.h:47):
// out = exp(beta*(x-max)) / sum over `axis`, computed in float32.
#ifndef TIM_VX_OPS_SOFTMAX_H_
#define TIM_VX_OPS_SOFTMAX_H_

#include "tim/vx/builtin_op.h"

namespace tim {
namespace vx {
namespace ops {

class Softmax : public BuiltinOp {
 public:
  Softmax(Graph* graph, float beta, int32_t axis);
  std::shared_ptr<Operation> Clone(std::shared_ptr<Graph>& graph) const override;

 protected:
  float beta_;
  int32_t axis_;
};

}  // namespace ops
}  // namespace vx
}  // namespace tim
#endif  // TIM_VX_OPS_SOFTMAX_H_
