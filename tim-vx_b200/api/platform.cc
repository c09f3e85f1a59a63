// tim::vx::platform over this backend: one device per CUDA GPU, executables as serialised graphs
// re-loaded on the executor's GPU.  Behaviour follows the reference's native platform
// (src/tim/vx/platform/native.cc:46-330): Compile serialises the graph and wraps the blob in a new graph
// holding one ops::NBG node, AllocateTensor creates tensors of that graph, Verify compiles it, an
// executor keeps an ordered queue of executables and Trigger runs and drains it.  Where the reference
// binds a sub-device of an NPU, the new graph is simply created with the GPU's index as device id.
#include <cstdio>
#include <vector>

#include "b2vx.h"
#include "tim/vx/compile_option.h"
#include "tim/vx/ops/nbg.h"
#include "tim/vx/platform/native.h"

namespace tim {
namespace vx {
namespace platform {

namespace {

class NativeDeviceImpl : public NativeDevice, public std::enable_shared_from_this<NativeDeviceImpl> {
 public:
  NativeDeviceImpl(device_id_t id, uint32_t core_count) {
    device_id_ = id;
    core_count_ = core_count;
  }
  bool Submit(const std::shared_ptr<Graph>&) override { return true; }
  bool Trigger(bool, async_callback) override { return true; }
  bool DeviceExit() override { return true; }
  void WaitDeviceIdle() override {}   // Graph::Run returns when the GPU is done
  std::shared_ptr<IExecutor> CreateExecutor(const int32_t core_index, const int32_t core_count,
                                            const std::shared_ptr<Context>& context) override;
};

class NativeTensorHandleImpl : public NativeTensorHandle {
 public:
  explicit NativeTensorHandleImpl(const std::shared_ptr<Tensor>& tensor) {
    tensor_ = tensor;
    spec_ = tensor->GetSpec();
  }
  bool CopyDataToTensor(const void* data, uint32_t size_in_bytes) override { return tensor_->CopyDataToTensor(data, size_in_bytes); }
  bool CopyDataFromTensor(void* data) override { return tensor_->CopyDataFromTensor(data); }
};

class NativeExecutorImpl;

class NativeExecutableImpl : public NativeExecutable {
 public:
  NativeExecutableImpl(const std::shared_ptr<IExecutor>& executor, std::vector<char> blob, size_t inputs, size_t outputs)
      : blob_(std::move(blob)) {
    executor_ = executor;
    context_ = executor->Contex();
    CompileOption option;
    option.setDeviceId(executor->Device()->Id());
    nb_graph_ = context_->CreateGraph(option);
    node_ = nb_graph_->CreateOperation<ops::NBG>(blob_.data(), inputs, outputs);
  }
  void SetInput(const std::shared_ptr<ITensorHandle>& th) override {
    node_->BindInput(th->GetTensor());
    input_handles_.push_back(th);
  }
  void SetOutput(const std::shared_ptr<ITensorHandle>& th) override {
    node_->BindOutput(th->GetTensor());
    output_handles_.push_back(th);
  }
  void SetInputs(const std::vector<std::shared_ptr<ITensorHandle>>& ths) override {
    for (const auto& t : ths) SetInput(t);
  }
  void SetOutputs(const std::vector<std::shared_ptr<ITensorHandle>>& ths) override {
    for (const auto& t : ths) SetOutput(t);
  }
  bool Submit(const std::shared_ptr<IExecutable>& ref, bool after) override {
    std::shared_ptr<IExecutor> executor = executor_.lock();
    return executor && executor->Submit(shared_from_this(), ref, after);
  }
  bool Trigger(bool) override { return nb_graph_->Run(); }
  bool Verify() override { return nb_graph_->Compile(); }
  std::shared_ptr<ITensorHandle> AllocateTensor(const TensorSpec& tensor_spec, void* data, uint32_t) override {
    std::shared_ptr<Tensor> tensor = nb_graph_->CreateTensor(tensor_spec, data);
    if (!tensor) return nullptr;
    return std::make_shared<NativeTensorHandleImpl>(tensor);
  }

 private:
  std::vector<char> blob_;
  std::shared_ptr<ops::NBG> node_;
};

class NativeExecutorImpl : public NativeExecutor, public std::enable_shared_from_this<NativeExecutorImpl> {
 public:
  NativeExecutorImpl(const std::shared_ptr<IDevice>& device, int32_t core_count, int32_t core_index,
                     const std::shared_ptr<Context>& context) {
    device_ = device;
    context_ = context ? context : Context::Create();
    // a GPU is one core: the requested range is clipped to it, as the reference clips to its cores
    const int32_t total = static_cast<int32_t>(device->CoreCount());
    if (core_index < 0 || core_index > total - 1) core_index = 0;
    if (core_count <= 0 || core_index + core_count > total) core_count = total - core_index;
    core_index_ = static_cast<uint32_t>(core_index);
    core_count_ = static_cast<uint32_t>(core_count);
  }
  bool Submit(const std::shared_ptr<IExecutable>& executable, const std::shared_ptr<IExecutable>& ref, bool after) override {
    if (!executable || !executable->Verify()) {
      std::fprintf(stderr, "E [platform] executable failed to compile\n");
      return false;
    }
    if (executable == ref) {
      tasks_.push_back(executable);
      return true;
    }
    for (size_t i = 0; i < tasks_.size(); ++i) {
      if (tasks_[i].lock() == ref) {
        tasks_.insert(tasks_.begin() + static_cast<long>(i) + (after ? 1 : 0), executable);
        return true;
      }
    }
    return false;   // ref is not queued
  }
  bool Trigger(bool) override {
    bool ok = false;
    while (!tasks_.empty()) {
      std::shared_ptr<IExecutable> t = tasks_.front().lock();
      tasks_.erase(tasks_.begin());
      if (!t) {
        std::fprintf(stderr, "E [platform] a queued executable no longer exists\n");
        return false;
      }
      ok = t->Trigger();
    }
    device_->WaitDeviceIdle();
    return ok;
  }
  std::shared_ptr<IExecutable> Compile(const std::shared_ptr<Graph>& graph) override {
    size_t bytes = 0;
    if (!graph || !graph->CompileToBinary(nullptr, &bytes)) return nullptr;
    std::vector<char> blob(bytes);
    if (!graph->CompileToBinary(blob.data(), &bytes)) return nullptr;
    return std::make_shared<NativeExecutableImpl>(shared_from_this(), std::move(blob), graph->InputsTensor().size(),
                                                  graph->OutputsTensor().size());
  }
};

std::shared_ptr<IExecutor> NativeDeviceImpl::CreateExecutor(const int32_t core_index, const int32_t core_count,
                                                            const std::shared_ptr<Context>& context) {
  return std::make_shared<NativeExecutorImpl>(shared_from_this(), core_count, core_index, context);
}

}  // namespace

std::shared_ptr<IExecutable> Compile(const std::shared_ptr<Graph>& graph, const std::shared_ptr<IExecutor>& executor) {
  return executor ? executor->Compile(graph) : nullptr;
}

void IDevice::RemoteReset() {}

std::vector<std::shared_ptr<IDevice>> IDevice::Enumerate() { return NativeDevice::Enumerate(); }

std::vector<std::shared_ptr<IDevice>> NativeDevice::Enumerate() {
  std::vector<std::shared_ptr<IDevice>> devices;
  const int32_t n = b2vx_device_count();
  for (int32_t i = 0; i < n; ++i) devices.push_back(std::make_shared<NativeDeviceImpl>(static_cast<device_id_t>(i), 1u));
  return devices;
}

}  // namespace platform
}  // namespace vx
}  // namespace tim
