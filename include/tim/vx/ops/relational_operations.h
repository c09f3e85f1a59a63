// Elementwise comparisons (reference: include/tim/vx/ops/relational_operations.h:58-73).  Declared so that
// programs naming them build; not executed by this backend: Graph::Compile fails, naming the op.
#ifndef TIM_VX_OPS_RELATIONAL_OPERATIONS_H_
#define TIM_VX_OPS_RELATIONAL_OPERATIONS_H_

#include "tim/vx/builtin_op.h"

namespace tim {
namespace vx {
namespace ops {

#define B2VX_DECLARED_ONLY_OP(NAME)                                                   \
  class NAME : public BuiltinOp {                                                     \
   public:                                                                            \
    explicit NAME(Graph* graph);                                                      \
    std::shared_ptr<Operation> Clone(std::shared_ptr<Graph>& graph) const override;   \
  };
B2VX_DECLARED_ONLY_OP(Greater)
B2VX_DECLARED_ONLY_OP(GreaterOrEqual)
B2VX_DECLARED_ONLY_OP(Less)
B2VX_DECLARED_ONLY_OP(LessOrEqual)
B2VX_DECLARED_ONLY_OP(NotEqual)
B2VX_DECLARED_ONLY_OP(Equal)
#undef B2VX_DECLARED_ONLY_OP

}  // namespace ops
}  // namespace vx
}  // namespace tim
#endif  // TIM_VX_OPS_RELATIONAL_OPERATIONS_H_
