// The one-input one-output ops of the reference's simple_operations.h (include/tim/vx/ops/simple_operations.h:32-154,
// src/tim/vx/ops/simple_operations.cc:28-62).
#ifndef TIM_VX_OPS_SIMPLE_OPERATIONS_H_
#define TIM_VX_OPS_SIMPLE_OPERATIONS_H_

#include <vector>

#include "tim/vx/builtin_op.h"

namespace tim {
namespace vx {
namespace ops {

// This backend executes DataConvert: quantize, dequantize or requantize with the input's and the output's
// parameters.
class DataConvert : public BuiltinOp {
 public:
  explicit DataConvert(Graph* graph);
  std::shared_ptr<Operation> Clone(std::shared_ptr<Graph>& graph) const override;
};

// The other classes of the family are declared so that programs naming them build; they are outside the
// quantized convolutional path, and Graph::Compile fails, naming the op, on a graph that contains one.
#define B2VX_DECLARED_ONLY_OP(NAME)                                                   \
  class NAME : public BuiltinOp {                                                     \
   public:                                                                            \
    explicit NAME(Graph* graph);                                                      \
    std::shared_ptr<Operation> Clone(std::shared_ptr<Graph>& graph) const override;   \
  };
B2VX_DECLARED_ONLY_OP(Neg)
B2VX_DECLARED_ONLY_OP(Abs)
B2VX_DECLARED_ONLY_OP(Sin)
B2VX_DECLARED_ONLY_OP(Exp)
B2VX_DECLARED_ONLY_OP(Log)
B2VX_DECLARED_ONLY_OP(Sqrt)
B2VX_DECLARED_ONLY_OP(Rsqrt)
B2VX_DECLARED_ONLY_OP(Square)
B2VX_DECLARED_ONLY_OP(LogicalNot)
B2VX_DECLARED_ONLY_OP(Floor)
B2VX_DECLARED_ONLY_OP(Ceil)
B2VX_DECLARED_ONLY_OP(Round)
B2VX_DECLARED_ONLY_OP(Cast)
B2VX_DECLARED_ONLY_OP(Rcp)
B2VX_DECLARED_ONLY_OP(Cos)
B2VX_DECLARED_ONLY_OP(Tan)
B2VX_DECLARED_ONLY_OP(ATan)
B2VX_DECLARED_ONLY_OP(ATanh)
B2VX_DECLARED_ONLY_OP(ACosh)
#undef B2VX_DECLARED_ONLY_OP

}  // namespace ops
}  // namespace vx
}  // namespace tim
#endif  // TIM_VX_OPS_SIMPLE_OPERATIONS_H_
