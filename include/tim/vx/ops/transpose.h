// ops::Transpose: output dimension i is input dimension perm[i]
// (reference: include/tim/vx/ops/transpose.h:44-52, src/tim/vx/ops/transpose.cc:34-49).
#ifndef TIM_VX_OPS_TRANSPOSE_H_
#define TIM_VX_OPS_TRANSPOSE_H_

#include <vector>

#include "tim/vx/builtin_op.h"

namespace tim {
namespace vx {
namespace ops {

class Transpose : public BuiltinOp {
 public:
  Transpose(Graph* graph, const std::vector<uint32_t>& perm);
  std::shared_ptr<Operation> Clone(std::shared_ptr<Graph>& graph) const override;

 protected:
  std::vector<uint32_t> perm_;
};

}  // namespace ops
}  // namespace vx
}  // namespace tim
#endif  // TIM_VX_OPS_TRANSPOSE_H_
