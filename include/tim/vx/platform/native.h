// The in-process ("native") implementation of the platform interfaces
// (reference: include/tim/vx/platform/native.h:34-77): NativeDevice::Enumerate lists the CUDA GPUs of
// this process.
#ifndef TIM_VX_PLATFORM_NATIVE_H_
#define TIM_VX_PLATFORM_NATIVE_H_

#include "tim/vx/platform/platform.h"

namespace tim {
namespace vx {
namespace platform {

class NativeDevice : public IDevice {
 public:
  ~NativeDevice() {}
  virtual bool Submit(const std::shared_ptr<Graph>& graph) = 0;
  virtual bool Trigger(bool async = false, async_callback cb = NULL) = 0;
  virtual bool DeviceExit() = 0;
  virtual void WaitDeviceIdle() = 0;
  virtual std::shared_ptr<IExecutor> CreateExecutor(const int32_t core_index = 0, const int32_t core_count = -1,
                                                    const std::shared_ptr<Context>& context = nullptr) = 0;
  static std::vector<std::shared_ptr<IDevice>> Enumerate();
};

class NativeExecutable : public IExecutable {
 public:
  virtual ~NativeExecutable() {}
  virtual void SetInput(const std::shared_ptr<ITensorHandle>& th) = 0;
  virtual void SetOutput(const std::shared_ptr<ITensorHandle>& th) = 0;
  virtual void SetInputs(const std::vector<std::shared_ptr<ITensorHandle>>& ths) = 0;
  virtual void SetOutputs(const std::vector<std::shared_ptr<ITensorHandle>>& ths) = 0;
  virtual bool Submit(const std::shared_ptr<IExecutable>& ref, bool after = true) = 0;
  virtual bool Trigger(bool async = false) = 0;
  virtual std::shared_ptr<ITensorHandle> AllocateTensor(const TensorSpec& tensor_spec, void* data = nullptr,
                                                        uint32_t size = 0) = 0;
  virtual bool Verify() = 0;
};

class NativeExecutor : public IExecutor {
 public:
  virtual ~NativeExecutor() {}
  virtual bool Submit(const std::shared_ptr<IExecutable>& executable, const std::shared_ptr<IExecutable>& ref,
                      bool after = true) = 0;
  virtual bool Trigger(bool async = false) = 0;
  virtual std::shared_ptr<IExecutable> Compile(const std::shared_ptr<Graph>& graph) = 0;
};

class NativeTensorHandle : public ITensorHandle {
 public:
  virtual bool CopyDataToTensor(const void* data, uint32_t size_in_bytes) = 0;
  virtual bool CopyDataFromTensor(void* data) = 0;
};

}  // namespace platform
}  // namespace vx
}  // namespace tim
#endif  // TIM_VX_PLATFORM_NATIVE_H_
