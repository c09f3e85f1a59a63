// ops::Reshape: the same elements, in WHCN order, under a new shape
// (reference: include/tim/vx/ops/reshape.h:41-46, src/tim/vx/ops/reshape.cc:46-64).
#ifndef TIM_VX_OPS_RESHAPE_H_
#define TIM_VX_OPS_RESHAPE_H_

#include <vector>

#include "tim/vx/builtin_op.h"

namespace tim {
namespace vx {
namespace ops {

class Reshape : public BuiltinOp {
 public:
  Reshape(Graph* graph, const std::vector<uint32_t>& target_shape);
  std::shared_ptr<Operation> Clone(std::shared_ptr<Graph>& graph) const override;

 protected:
  std::vector<uint32_t> size_;
};

}  // namespace ops
}  // namespace vx
}  // namespace tim
#endif  // TIM_VX_OPS_RESHAPE_H_
