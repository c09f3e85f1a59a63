// Harness-only stub: the reference's pooling test files also exercise Pool1d,
// which is not on the quantized CNN path.  Tests that build one fail at
// Compile (the op lowers to an unknown node kind) and are reported as such.
#ifndef GOLDEN_SHIM_POOL1D_H_
#define GOLDEN_SHIM_POOL1D_H_
#include "tim/vx/builtin_op.h"
namespace tim { namespace vx { namespace ops {
class Pool1d : public BuiltinOp {
 public:
  template <typename... A>
  Pool1d(Graph* graph, A...) : BuiltinOp(graph, 0xFFFF) {}
  std::shared_ptr<Operation> Clone(std::shared_ptr<Graph>&) const override { return nullptr; }
};
}}}
#endif
