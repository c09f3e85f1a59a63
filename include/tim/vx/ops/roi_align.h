// ops::RoiAlign (reference: include/tim/vx/ops/roi_align.h:50-68).  Declared so that programs naming it build;
// not executed by this backend: Graph::Compile fails, naming the op.
#ifndef TIM_VX_OPS_ROI_ALIGN_H_
#define TIM_VX_OPS_ROI_ALIGN_H_

#include "tim/vx/builtin_op.h"

namespace tim {
namespace vx {
namespace ops {

class RoiAlign : public BuiltinOp {
 public:
  RoiAlign(Graph* graph, int32_t output_height, int32_t output_width, float height_ratio, float width_ratio,
           int32_t height_sample_num, int32_t width_sample_num, DataLayout input_layout = DataLayout::WHCN);
  std::shared_ptr<Operation> Clone(std::shared_ptr<Graph>& graph) const override;

 protected:
  int32_t output_height_;
  int32_t output_width_;
  float height_ratio_;
  float width_ratio_;
  int32_t height_sample_num_;
  int32_t width_sample_num_;
};

}  // namespace ops
}  // namespace vx
}  // namespace tim
#endif  // TIM_VX_OPS_ROI_ALIGN_H_
