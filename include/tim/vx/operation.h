// tim::vx::Operation — base of every op class; binds tensors positionally.
// Restates include/tim/vx/operation.h:35-64 of the reference.
#ifndef TIM_VX_OPERATION_H_
#define TIM_VX_OPERATION_H_

#include "tim/vx/graph.h"
#include "tim/vx/tensor.h"

namespace tim {
namespace vx {

class OpImpl;

class Operation {
 public:
  Operation();
  virtual ~Operation();
  virtual std::shared_ptr<Operation> Clone(std::shared_ptr<Graph>& graph) const = 0;

  Operation& BindInput(const std::shared_ptr<Tensor>& tensor);
  Operation& BindOutput(const std::shared_ptr<Tensor>& tensor);
  Operation& BindInputs(const std::vector<std::shared_ptr<Tensor>>& tensors);
  Operation& BindOutputs(const std::vector<std::shared_ptr<Tensor>>& tensors);
  // Kept for source compatibility.  Quantized outputs here always saturate and
  // round to nearest even; only the pooling output-size rounding is a real
  // choice and that is taken from the Pool2d constructor.
  Operation& SetRoundingPolicy(
      OverflowPolicy overflow_policy = OverflowPolicy::SATURATE,
      RoundingPolicy rounding_policy = RoundingPolicy::RTNE,
      RoundType down_scale_size_rounding = RoundType::FLOOR,
      uint32_t accumulator_bits = 0);

  std::unique_ptr<OpImpl>& impl();
  const std::unique_ptr<OpImpl>& impl() const;
  const uint32_t& uid() const;

  virtual const std::vector<std::shared_ptr<Tensor>> ConstantInputsTensor() const;

 protected:
  bool IsAllInputsConst() const;
  std::unique_ptr<OpImpl> impl_;

 private:
  virtual void OnBindInputPostProc(const std::shared_ptr<Tensor>& tensor,
                                   int32_t input_idx);
};

}  // namespace vx
}  // namespace tim
#endif  // TIM_VX_OPERATION_H_
