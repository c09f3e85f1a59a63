// ops::DataConvert (reference: include/tim/vx/ops/simple_operations.h:41-46,118,
// src/tim/vx/ops/simple_operations.cc:39).
#ifndef TIM_VX_OPS_SIMPLE_OPERATIONS_H_
#define TIM_VX_OPS_SIMPLE_OPERATIONS_H_

#include <vector>

#include "tim/vx/builtin_op.h"

namespace tim {
namespace vx {
namespace ops {

// Of the reference's one-input one-output ops declared with DECLARE_SIMPLE_OP this backend executes
// DataConvert: quantize, dequantize or requantize with the input's and the output's parameters.
class DataConvert : public BuiltinOp {
 public:
  explicit DataConvert(Graph* graph);
  std::shared_ptr<Operation> Clone(std::shared_ptr<Graph>& graph) const override;
};

}  // namespace ops
}  // namespace vx
}  // namespace tim
#endif  // TIM_VX_OPS_SIMPLE_OPERATIONS_H_
