// tim::vx::ops::Pool2d (reference: include/tim/vx/ops/pool2d.h:67-104).
// MAX ignores padding; AVG divides by kw*kh (padding counted); AVG_ANDROID
// divides by the number of in-bounds taps.  Four constructor forms: padding by
// PadType, explicit pad {l,r,t,b}, global pooling (ksize = stride = input
// size), and adaptive pooling (ksize/stride derived from input and output
// size as in src/tim/vx/ops/pool2d.cc:82-93).
#ifndef TIM_VX_OPS_POOL2D_H_
#define TIM_VX_OPS_POOL2D_H_

#include <array>

#include "tim/vx/builtin_op.h"
#include "tim/vx/types.h"

namespace tim {
namespace vx {
namespace ops {

class Pool2d : public BuiltinOp {
 public:
  Pool2d(Graph* graph, PoolType type, PadType padding,
         const std::array<uint32_t, 2>& ksize,
         const std::array<uint32_t, 2>& stride,
         RoundType round_type = RoundType::FLOOR,
         DataLayout layout = DataLayout::WHCN);
  Pool2d(Graph* graph, PoolType type, const std::array<uint32_t, 4>& pad,
         const std::array<uint32_t, 2>& ksize,
         const std::array<uint32_t, 2>& stride,
         RoundType round_type = RoundType::FLOOR,
         DataLayout layout = DataLayout::WHCN);
  Pool2d(Graph* graph, PoolType type, const std::array<uint32_t, 2>& input_size,
         RoundType round_type = RoundType::FLOOR,
         DataLayout layout = DataLayout::WHCN);
  Pool2d(Graph* graph, PoolType type, const std::array<uint32_t, 2>& input_size,
         const std::array<uint32_t, 2>& output_size,
         RoundType round_type = RoundType::FLOOR,
         DataLayout layout = DataLayout::WHCN);

  std::shared_ptr<Operation> Clone(std::shared_ptr<Graph>& graph) const override;
  void Init();

 protected:
  const PoolType type_;
  const PadType padding_;
  std::array<uint32_t, 2> ksize_;
  std::array<uint32_t, 2> stride_;
  const RoundType round_type_;
  const std::array<uint32_t, 4> pad_;
};

}  // namespace ops
}  // namespace vx
}  // namespace tim
#endif  // TIM_VX_OPS_POOL2D_H_
