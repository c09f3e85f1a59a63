// ops::GroupedConv2d: input and output channels split into `group` contiguous blocks, block g of the outputs
// reading block g of the inputs; kernel [kw, kh, Ic/group, Oc] (reference:
// include/tim/vx/ops/groupedconv2d.h:56-85, src/tim/vx/ops/groupedconv2d.cc:34-90).
#ifndef TIM_VX_OPS_GROUPEDCONV2D_H_
#define TIM_VX_OPS_GROUPEDCONV2D_H_

#include <array>

#include "tim/vx/builtin_op.h"

namespace tim {
namespace vx {
namespace ops {

class GroupedConv2d : public BuiltinOp {
 public:
  GroupedConv2d(Graph* graph, PadType padding, const std::array<uint32_t, 2>& strides,
                const std::array<uint32_t, 2>& dilation, int32_t grouped_number,
                DataLayout input_layout = DataLayout::WHCN,
                DataLayout kernel_layout = DataLayout::WHIcOc);
  GroupedConv2d(Graph* graph, const std::array<uint32_t, 4>& pad, const std::array<uint32_t, 2>& strides,
                const std::array<uint32_t, 2>& dilation, int32_t group_number,
                DataLayout input_layout = DataLayout::WHCN,
                DataLayout kernel_layout = DataLayout::WHIcOc);

  DataLayout KernelDataLayout() { return kernel_layout_; }
  std::shared_ptr<Operation> Clone(std::shared_ptr<Graph>& graph) const override;

 protected:
  const PadType padding_;
  const std::array<uint32_t, 2> strides_;
  const std::array<uint32_t, 2> dilation_;
  const std::array<uint32_t, 4> pad_;
  const int32_t group_number_;
  const DataLayout kernel_layout_;
};

}  // namespace ops
}  // namespace vx
}  // namespace tim
#endif  // TIM_VX_OPS_GROUPEDCONV2D_H_
