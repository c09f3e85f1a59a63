// tim::vx::ops::Conv2d — 2-D convolution, dense or depthwise.
// Restates include/tim/vx/ops/conv2d.h:59-105 of the reference.
//
// Inputs {x, w[, bias]}: x [W,H,Ic,N]; w [kw,kh,Ic,Oc] for a dense convolution
// or [kw,kh,Ic*multiplier,1] when multiplier >= 1 (depthwise, output channel
// ic*multiplier+m); bias [Oc] int32 with scale s_x*s_w.  Output [Wo,Ho,Oc,N].
// `weights` and `ksize` are hints: the kernel tensor's own shape decides.
// Padding is either a PadType (SAME/VALID; SAME puts the odd element at the
// end) or explicit {left,right,top,bottom}.  dilation 0 is read as 1.
#ifndef TIM_VX_OPS_CONV2D_H_
#define TIM_VX_OPS_CONV2D_H_

#include <array>

#include "tim/vx/builtin_op.h"

namespace tim {
namespace vx {
namespace ops {

class Conv2d : public BuiltinOp {
 public:
  Conv2d(Graph* graph, PadType padding, const std::array<uint32_t, 2>& stride,
         const std::array<uint32_t, 2>& dilation, int32_t multiplier = 0,
         DataLayout input_layout = DataLayout::WHCN,
         DataLayout kernel_layout = DataLayout::WHIcOc);
  Conv2d(Graph* graph, const std::array<uint32_t, 4> pad,
         const std::array<uint32_t, 2>& stride,
         const std::array<uint32_t, 2>& dilation, int32_t multiplier = 0,
         DataLayout input_layout = DataLayout::WHCN,
         DataLayout kernel_layout = DataLayout::WHIcOc);
  Conv2d(Graph* graph, int32_t weights, PadType padding,
         const std::array<uint32_t, 2>& ksize,
         const std::array<uint32_t, 2>& stride,
         const std::array<uint32_t, 2>& dilation, int32_t multiplier = 0,
         DataLayout input_layout = DataLayout::WHCN,
         DataLayout kernel_layout = DataLayout::WHIcOc);
  Conv2d(Graph* graph, int32_t weights, PadType padding,
         const std::array<uint32_t, 2>& ksize,
         const std::array<uint32_t, 2>& stride,
         const std::array<uint32_t, 2>& dilation,
         const std::array<uint32_t, 4>& pad, int32_t multiplier = 0,
         DataLayout input_layout = DataLayout::WHCN,
         DataLayout kernel_layout = DataLayout::WHIcOc);

  DataLayout KernelDataLayout() { return kernel_layout_; }

  std::shared_ptr<Operation> Clone(std::shared_ptr<Graph>& graph) const override;
  const std::vector<std::shared_ptr<Tensor>> ConstantInputsTensor() const override;

 protected:
  const uint32_t weights_;
  const PadType padding_;
  const std::array<uint32_t, 2> ksize_;
  const std::array<uint32_t, 2> stride_;
  const std::array<uint32_t, 2> dilation_;
  const std::array<uint32_t, 4> pad_;
  const int32_t multiplier_;
  const DataLayout kernel_layout_;
};

}  // namespace ops
}  // namespace vx
}  // namespace tim
#endif  // TIM_VX_OPS_CONV2D_H_
