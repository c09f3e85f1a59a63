// tim::vx::platform — devices, executors, executables and tensor handles: the reference's own
// multi-device surface (include/tim/vx/platform/platform.h:51-144), restated with the same class and
// method names.  Here a device is one CUDA GPU (IDevice::Enumerate lists them all, one "core" each),
// an executor is a work queue bound to a device and a Context, and an executable is a graph that was
// serialised with Graph::CompileToBinary and loaded again as a single ops::NBG node of a graph bound to
// the executor's GPU:
//
//   auto devices = platform::IDevice::Enumerate();
//   auto executor = devices[i]->CreateExecutor();
//   auto executable = platform::Compile(graph, executor);          // graph: any tim::vx graph
//   auto in = executable->AllocateTensor(graph->InputsTensor()[0]->GetSpec());
//   auto out = executable->AllocateTensor(graph->OutputsTensor()[0]->GetSpec());
//   executable->SetInput(in); executable->SetOutput(out);
//   in->CopyDataToTensor(data, bytes);
//   executable->Submit(executable);  executor->Trigger();  out->CopyDataFromTensor(result);
#ifndef TIM_VX_PLATFORM_PLATFORM_H_
#define TIM_VX_PLATFORM_PLATFORM_H_

#include <functional>
#include <memory>
#include <vector>

#include "tim/vx/context.h"
#include "tim/vx/graph.h"
#include "tim/vx/tensor.h"

namespace tim {
namespace vx {
namespace ops {
class NBG;
}

namespace platform {

class IDevice;
class IExecutable;
class IExecutor;
class ITensorHandle;

// executor->Compile(graph)
std::shared_ptr<IExecutable> Compile(const std::shared_ptr<Graph>& graph, const std::shared_ptr<IExecutor>& executor);

class IDevice {
 public:
  using device_id_t = uint32_t;
  using async_callback = std::function<bool(const void*)>;
  using data_t = const void*;
  virtual ~IDevice() {}
  virtual bool Submit(const std::shared_ptr<Graph>& graph) = 0;
  virtual bool Trigger(bool async = false, async_callback cb = NULL) = 0;
  device_id_t Id() const { return device_id_; }
  virtual void WaitDeviceIdle() = 0;
  virtual bool DeviceExit() = 0;
  virtual void RemoteReset();
  uint32_t CoreCount() const { return core_count_; }
  virtual std::shared_ptr<IExecutor> CreateExecutor(const int32_t core_index = 0, const int32_t core_count = -1,
                                                    const std::shared_ptr<Context>& context = nullptr) = 0;
  static std::vector<std::shared_ptr<IDevice>> Enumerate();

 protected:
  device_id_t device_id_ = 0;
  uint32_t core_count_ = 0;
};

class IExecutor {
 public:
  using task = std::weak_ptr<IExecutable>;
  virtual ~IExecutor() {}
  // queue `executable` before or after `ref` (or at the end when ref == executable)
  virtual bool Submit(const std::shared_ptr<IExecutable>& executable, const std::shared_ptr<IExecutable>& ref,
                      bool after = true) = 0;
  // run and drain the queue
  virtual bool Trigger(bool async = false) = 0;
  virtual std::shared_ptr<IExecutable> Compile(const std::shared_ptr<Graph>& graph) = 0;
  virtual std::shared_ptr<IDevice> Device() const { return device_; }
  virtual std::shared_ptr<Context> Contex() const { return context_; }
  virtual uint32_t CoreIndex() const { return core_index_; }
  virtual uint32_t CoreCount() const { return core_count_; }

 protected:
  std::vector<task> tasks_;
  std::shared_ptr<IDevice> device_;
  std::shared_ptr<Context> context_;
  uint32_t core_index_ = 0;
  uint32_t core_count_ = 0;
};

class IExecutable : public std::enable_shared_from_this<IExecutable> {
 public:
  virtual ~IExecutable() {}
  virtual void SetInput(const std::shared_ptr<ITensorHandle>& th) = 0;
  virtual void SetOutput(const std::shared_ptr<ITensorHandle>& th) = 0;
  virtual void SetInputs(const std::vector<std::shared_ptr<ITensorHandle>>& ths) = 0;
  virtual void SetOutputs(const std::vector<std::shared_ptr<ITensorHandle>>& ths) = 0;
  virtual std::vector<std::shared_ptr<ITensorHandle>> GetOutputs() { return output_handles_; }
  virtual std::vector<std::shared_ptr<ITensorHandle>> Getinputs() { return input_handles_; }
  virtual bool Submit(const std::shared_ptr<IExecutable>& ref, bool after = true) = 0;
  virtual bool Trigger(bool async = false) = 0;
  virtual bool Verify() = 0;
  std::shared_ptr<Graph> NBGraph() const { return nb_graph_; }
  virtual std::shared_ptr<ITensorHandle> AllocateTensor(const TensorSpec& tensor_spec, void* data = nullptr,
                                                        uint32_t size = 0) = 0;

 protected:
  std::weak_ptr<IExecutor> executor_;
  std::shared_ptr<Context> context_;
  std::shared_ptr<Graph> nb_graph_;
  std::vector<std::shared_ptr<ITensorHandle>> input_handles_;
  std::vector<std::shared_ptr<ITensorHandle>> output_handles_;
};

class ITensorHandle {
 public:
  virtual ~ITensorHandle() {}
  virtual bool CopyDataToTensor(const void* data, uint32_t size_in_bytes) = 0;
  virtual bool CopyDataFromTensor(void* data) = 0;
  virtual std::shared_ptr<Tensor> GetTensor() const { return tensor_; }
  virtual TensorSpec& GetSpec() { return spec_; }

 protected:
  std::shared_ptr<Tensor> tensor_;
  TensorSpec spec_;
};

}  // namespace platform
}  // namespace vx
}  // namespace tim
#endif  // TIM_VX_PLATFORM_PLATFORM_H_
