// tim::transform::LayoutInference: rewrites a graph whose Conv2d / Pool2d ops were declared with the
// front-end layouts (activations CWHN = NHWC, kernels IcWHOc / OcIcWH / IcOcWH) into one that runs in the
// backend's native WHCN / WHIcOc layouts (reference: include/tim/transform/layout_inference.h:41-52,
// src/tim/transform/layout_inference.cc, ops/conv2d_layout_inference.h:42-131).  Returns the new graph and
// the map from the source graph's input and output tensors to their counterparts, which keep the source
// shapes and layouts.
#ifndef TIM_LAYOUT_INFERENCE_H_
#define TIM_LAYOUT_INFERENCE_H_

#include <map>
#include <memory>
#include <utility>
#include <vector>

namespace tim {

namespace vx {
class Context;
class Graph;
class Tensor;
class Operation;
}  // namespace vx

namespace transform {
class IPermuteVector;
std::pair<
    /* graph after layout inference */
    std::shared_ptr<vx::Graph>,
    /* tensor mapping between the original graph and the graph after layout inference */
    std::map<std::shared_ptr<vx::Tensor>, std::shared_ptr<vx::Tensor>>>
LayoutInference(const std::shared_ptr<vx::Graph>& src_graph, std::shared_ptr<vx::Context>& ctx,
                std::map<std::shared_ptr<vx::Tensor>, std::shared_ptr<IPermuteVector>> tensor_pv_map =
                    std::map<std::shared_ptr<vx::Tensor>, std::shared_ptr<IPermuteVector>>());

}  // namespace transform
}  // namespace tim

#endif  // TIM_LAYOUT_INFERENCE_H_
