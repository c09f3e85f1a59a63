// tim::vx::ops::Relu / Relu6 (reference: include/tim/vx/ops/activations.h:83-85).
// out = quantize(clamp(dequantize(x), 0, [6])).  The reference's other
// activation classes (Tanh, Sigmoid, Gelu, ...) are not on the quantized CNN
// path and are not declared.
#ifndef TIM_VX_OPS_ACTIVATIONS_H_
#define TIM_VX_OPS_ACTIVATIONS_H_

#include "tim/vx/builtin_op.h"

namespace tim {
namespace vx {
namespace ops {

class Relu : public BuiltinOp {
 public:
  Relu(Graph* graph);
  std::shared_ptr<Operation> Clone(std::shared_ptr<Graph>& graph) const override;
};

class Relu6 : public BuiltinOp {
 public:
  Relu6(Graph* graph);
  std::shared_ptr<Operation> Clone(std::shared_ptr<Graph>& graph) const override;
};

}  // namespace ops
}  // namespace vx
}  // namespace tim
#endif  // TIM_VX_OPS_ACTIVATIONS_H_
