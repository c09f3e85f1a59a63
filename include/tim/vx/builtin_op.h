// tim::vx::BuiltinOp — an Operation backed by one node of the execution
// backend (reference: include/tim/vx/builtin_op.h:28-39).  `kind` is one of
// the B2VX_NODE_* values of b2vx.h.
#ifndef TIM_VX_BUILTIN_OP_H_
#define TIM_VX_BUILTIN_OP_H_

#include "tim/vx/operation.h"
#define DirectMapOp BuiltinOp

namespace tim {
namespace vx {

class BuiltinOp : public Operation {
 public:
  BuiltinOp(Graph* graph, uint32_t kind, int in_cnt = 0, int out_cnt = 0,
            DataLayout layout = DataLayout::ANY);
};

}  // namespace vx
}  // namespace tim
#endif  // TIM_VX_BUILTIN_OP_H_
