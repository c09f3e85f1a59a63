// ops::Concat: input_cnt tensors joined along `axis`
// (reference: include/tim/vx/ops/concat.h:41-49, src/tim/vx/ops/concat.cc:33-41).
#ifndef TIM_VX_OPS_CONCAT_H_
#define TIM_VX_OPS_CONCAT_H_

#include <vector>

#include "tim/vx/builtin_op.h"

namespace tim {
namespace vx {
namespace ops {

class Concat : public BuiltinOp {
 public:
  Concat(Graph* graph, uint32_t axis, int input_cnt);
  std::shared_ptr<Operation> Clone(std::shared_ptr<Graph>& graph) const override;

 protected:
  uint32_t axis_;
};

}  // namespace ops
}  // namespace vx
}  // namespace tim
#endif  // TIM_VX_OPS_CONCAT_H_
