// ops::Resize (reference: include/tim/vx/ops/resize.h:47-63).  Declared so that programs naming it build; not
// executed by this backend: Graph::Compile fails, naming the op.
#ifndef TIM_VX_OPS_RESIZE_H_
#define TIM_VX_OPS_RESIZE_H_

#include "tim/vx/builtin_op.h"

namespace tim {
namespace vx {
namespace ops {

class Resize : public BuiltinOp {
 public:
  Resize(Graph* graph, ResizeType type, float factor, bool align_corners, bool half_pixel_centers, int target_height,
         int target_width, DataLayout layout = DataLayout::WHCN);
  std::shared_ptr<Operation> Clone(std::shared_ptr<Graph>& graph) const override;

 protected:
  const ResizeType type_;
  const float factor_;
  const bool align_corners_;
  const bool half_pixel_centers_;
  const int target_height_;
  const int target_width_;
};

}  // namespace ops
}  // namespace vx
}  // namespace tim
#endif  // TIM_VX_OPS_RESIZE_H_
