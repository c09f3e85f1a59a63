// tim::vx::CompileOption (reference: include/tim/vx/compile_option.h:37-55,
// src/tim/vx/compile_option.cc:32-84).  The device id selects the GPU a graph
// is bound to; relax mode is accepted and ignored (there is no reduced-
// precision float path here).
#ifndef TIM_VX_COMPILE_OPTION_H_
#define TIM_VX_COMPILE_OPTION_H_

#include <cstdint>
#include <memory>

namespace tim {
namespace vx {

struct CompileOptionImpl;

class CompileOption {
 public:
  CompileOption();
  ~CompileOption() {}

  bool isRelaxMode() const;
  bool setRelaxMode(bool enable = false);

  void setDeviceId(uint32_t device);
  uint32_t getDeviceId() const;

  static CompileOption DefaultOptions;

 private:
  std::shared_ptr<CompileOptionImpl> impl_;
};

}  // namespace vx
}  // namespace tim
#endif  // TIM_VX_COMPILE_OPTION_H_
