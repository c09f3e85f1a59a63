// tim::vx::Context — entry object of the API (reference: include/tim/vx/context.h:35-45,
// src/tim/vx/context.cc:35-63).  A Context owns one b2vx_context; graphs made
// from it must not outlive it.
#ifndef TIM_VX_CONTEXT_H_
#define TIM_VX_CONTEXT_H_

#include <memory>

namespace tim {
namespace vx {

class CompileOption;
class Graph;

class Context {
 public:
  virtual ~Context() {}
  static std::shared_ptr<Context> Create();

  virtual std::shared_ptr<Graph> CreateGraph() = 0;
  virtual std::shared_ptr<Graph> CreateGraph(const CompileOption& options) = 0;

  // Hardware queries of the reference (Vivante "CL only" parts, stream
  // processor).  A B200 is neither: both return false.
  virtual bool isClOnly() = 0;
  virtual bool hasSP() = 0;
};

}  // namespace vx
}  // namespace tim
#endif  // TIM_VX_CONTEXT_H_
