// Private classes behind the tim::vx interfaces.  Everything here lowers to the
// b2vx C ABI; there is no arithmetic in this layer.
//
// Reference counterparts: ContextImpl (src/tim/vx/context_private.h),
// GraphImpl (src/tim/vx/graph_private.h:43-127), TensorImpl
// (src/tim/vx/tensor_private.h), OpImpl/BuiltinOpImpl (src/tim/vx/op_impl.h,
// src/tim/vx/builtin_op_impl.h).  The reference creates its backend node in the
// op constructor and patches fields as tensors are bound; here an op only
// records its descriptor and bindings, and GraphImpl::Compile emits one
// b2vx_node_* call per op in creation order.
#ifndef TIMVX_B200_API_IMPL_H_
#define TIMVX_B200_API_IMPL_H_

#include <map>
#include <memory>
#include <mutex>
#include <vector>

#include "b2vx.h"
#include "tim/vx/compile_option.h"
#include "tim/vx/context.h"
#include "tim/vx/graph.h"
#include "tim/vx/operation.h"
#include "tim/vx/tensor.h"

namespace tim {
namespace vx {

struct CompileOptionImpl {
  bool relax_mode = false;
  uint32_t device_id = 0;
};

class ContextImpl : public Context {
 public:
  ContextImpl();
  ~ContextImpl() override;
  std::shared_ptr<Graph> CreateGraph() override;
  std::shared_ptr<Graph> CreateGraph(const CompileOption& options) override;
  bool isClOnly() override { return false; }
  bool hasSP() override { return false; }
  b2vx_context* handle() { return ctx_; }

 private:
  b2vx_context* ctx_ = nullptr;
};

class GraphImpl;

class TensorImpl : public Tensor {
 public:
  TensorImpl(GraphImpl* graph, const TensorSpec& spec, const void* data, void* io_handle);
  ~TensorImpl() override;
  bool valid() const { return id_ != B2VX_NO_TENSOR; }

  const ShapeType& GetShape() override;
  DataType GetDataType() override { return spec_.datatype_; }
  const Quantization& GetQuantization() override { return spec_.quantization_; }
  TensorSpec& GetSpec() override { return spec_; }
  uint32_t GetId() override { return id_; }
  bool CopyDataToTensor(const void* data, uint32_t size_in_bytes = 0) override;
  bool CopyDataFromTensor(void* data) override;
  bool SwapHandle(void* new_ptr, bool is_new_ptr_malloc_by_ovxlib, void** old_ptr) override;
  bool SwapHandle(std::shared_ptr<tim::vx::Tensor> tensor) override;
  bool SwapHandleWithCache(std::shared_ptr<tim::vx::Tensor> tensor) override;
  bool FlushCacheForHandle() override;
  bool InvalidateCacheForHandle() override;
  void* map(bool invalidate_cpu_cache = false) override;
  void unmap() override;
  bool IsPlaceHolder() override { return false; }
  bool IsConstTensor() override { return (spec_.attr_ & TensorAttribute::CONSTANT) != 0; }
  bool IsScalar() override { return is_scalar_ != 0; }
  bool SaveTensorToTextByFp32(std::string filename) override;
  void SetScalar(int8_t is_scalar) override { is_scalar_ = is_scalar; }
  void* ConvertTensorToData(uint8_t* tensorData) override;
  float* ConvertTensorToFloat32Data() override;

  void RefreshShape();
  // CONSTANT tensors keep a copy of their data for Graph::CompileToBinary
  const std::vector<uint8_t>& ConstData() const { return const_copy_; }

 private:
  bool EnsureHostBuffer();
  GraphImpl* graph_;
  TensorSpec spec_;
  uint32_t id_ = B2VX_NO_TENSOR;
  void* host_ = nullptr;      // host side of an INPUT/OUTPUT tensor (map, handles)
  bool host_owned_ = false;   // allocated by b2vx_host_alloc
  int8_t is_scalar_ = 0;
  std::vector<uint8_t> const_copy_;
};

// Stand-in for an optional input that was not supplied.
class TensorPlaceholder : public Tensor {
 public:
  const ShapeType& GetShape() override { return spec_.shape_; }
  DataType GetDataType() override { return DataType::UNKNOWN; }
  const Quantization& GetQuantization() override { return spec_.quantization_; }
  TensorSpec& GetSpec() override { return spec_; }
  uint32_t GetId() override { return B2VX_NO_TENSOR; }
  bool CopyDataToTensor(const void*, uint32_t = 0) override { return false; }
  bool CopyDataFromTensor(void*) override { return false; }
  bool SwapHandle(void*, bool, void**) override { return false; }
  bool SwapHandle(std::shared_ptr<tim::vx::Tensor>) override { return false; }
  bool SwapHandleWithCache(std::shared_ptr<tim::vx::Tensor>) override { return false; }
  bool FlushCacheForHandle() override { return false; }
  bool InvalidateCacheForHandle() override { return false; }
  void* map(bool = false) override { return nullptr; }
  void unmap() override {}
  bool IsPlaceHolder() override { return true; }
  bool IsConstTensor() override { return false; }
  bool IsScalar() override { return false; }
  bool SaveTensorToTextByFp32(std::string) override { return false; }
  void SetScalar(int8_t) override {}
  void* ConvertTensorToData(uint8_t*) override { return nullptr; }
  float* ConvertTensorToFloat32Data() override { return nullptr; }

 private:
  TensorSpec spec_;
};

// What an op knows before Compile: its node kind, its descriptor and the
// tensors bound so far.
class OpImpl {
 public:
  OpImpl(Graph* graph, uint32_t kind, int in_cnt, int out_cnt, DataLayout layout);
  Graph* graph_;
  uint32_t kind_;
  int32_t input_cnt_;
  int32_t output_cnt_;
  DataLayout layout_;
  DataLayout kernel_layout_ = DataLayout::WHIcOc;   // Conv2d, GroupedConv2d
  uint32_t uid_;
  std::vector<std::shared_ptr<Tensor>> inputs_tensor_;
  std::vector<std::shared_ptr<Tensor>> outputs_tensor_;
  union {
    b2vx_conv2d_desc conv2d;
    b2vx_fc_desc fc;
    b2vx_pool2d_desc pool2d;
    b2vx_softmax_desc softmax;
    b2vx_dims_desc dims;     // Reshape: target shape; Transpose: permutation
    uint32_t concat_axis;
  } desc_;
  std::vector<uint8_t> blob_;   // ops::NBG: the serialised graph this op stands for
  // Conv2d / Pool2d declared with a front-end layout (CWHN activations, IcWHOc / OcIcWH / IcOcWH kernels):
  // tim::transform::LayoutInference rewrites such a graph; compiled as it stands the op runs as WHCN / WHIcOc.
  bool foreign_layout_ = false;
  // Operation::SetRoundingPolicy, defaults as in include/tim/vx/operation.h of the reference
  OverflowPolicy overflow_policy_ = OverflowPolicy::SATURATE;
  RoundingPolicy rounding_policy_ = RoundingPolicy::RTNE;
  RoundType down_scale_size_rounding_ = RoundType::FLOOR;
  uint32_t accumulator_bits_ = 0;
  const char* name_ = "";       // declared-only ops: the class name, for the message Compile gives
};

// Node kind of ops::NBG inside this layer; it never reaches the C ABI: Compile expands the op into the
// nodes and tensors of its blob.
constexpr uint32_t kNodeKindNbg = 0x4E4247u;
// Node kind of the op classes that are declared for source compatibility only; `name_` says which.
constexpr uint32_t kNodeKindDeclaredOnly = 0x4E4F4Eu;

class GraphImpl : public Graph {
 public:
  GraphImpl(ContextImpl* context, const CompileOption& options);
  ~GraphImpl() override;

  void SetCompileOption(const CompileOption& o) override { options_ = o; }
  std::shared_ptr<Tensor> CreateTensor(const TensorSpec& spec, const void* data = nullptr) override;
  std::shared_ptr<Tensor> CreateTensor(const TensorSpec& spec, const DmaBufferDesc& dmafd) override;
  std::shared_ptr<Tensor> CreateIOTensor(const TensorSpec& spec, void* data = nullptr) override;
  std::shared_ptr<Tensor> CreateTensorPlaceHolder() override;
  bool Compile() override;
  bool CompileToBinary(void* buf, size_t* size) override;
  bool Run() override;
  const std::vector<std::shared_ptr<Tensor>> InputsTensor() const override { return inputs_tensor_; }
  const std::vector<std::shared_ptr<Tensor>> OutputsTensor() const override { return outputs_tensor_; }
  void UpdateTensorConsumersMap(const std::shared_ptr<Tensor>& tensor, const Operation* op) override;
  void RenewTensorConsumersMap(const std::shared_ptr<Tensor>& org_tensor,
                               const std::shared_ptr<Tensor>& dst_tensor,
                               const Operation* op) override;
  void UpdateTensorProducerMap(const std::shared_ptr<Tensor>& tensor, const Operation* op) override;
  const std::vector<std::shared_ptr<Operation>> GetConsumersOp(std::shared_ptr<Tensor> tensor) const override;
  std::shared_ptr<Operation> GetProducerOp(std::shared_ptr<Tensor> tensor) override;
  void PrintGraph() const override;
  std::vector<std::shared_ptr<Operation>>& OpVector() override { return op_vector_; }
  std::map<std::shared_ptr<Tensor>, std::vector<std::shared_ptr<Operation>>>& TensorConsumer() override {
    return tensor_consumers_;
  }
  std::map<std::shared_ptr<Tensor>, std::shared_ptr<Operation>>& TensorProducer() override {
    return tensor_producer_;
  }

  b2vx_graph* handle() { return graph_; }
  ContextImpl* context() { return context_; }
  bool EnsureHandle();
  uint32_t NextOpUid() { return op_uid_++; }
  void LogBackendError(const char* where) const;

 private:
  bool EmitNodes();
  bool ExpandBlob(const OpImpl* op);
  ContextImpl* context_;
  CompileOption options_;
  b2vx_graph* graph_ = nullptr;
  std::vector<std::shared_ptr<Tensor>> inputs_tensor_;
  std::vector<std::shared_ptr<Tensor>> outputs_tensor_;
  std::vector<std::weak_ptr<TensorImpl>> all_tensors_;
  std::map<std::shared_ptr<Tensor>, std::vector<std::shared_ptr<Operation>>> tensor_consumers_;
  std::map<std::shared_ptr<Tensor>, std::shared_ptr<Operation>> tensor_producer_;
  std::once_flag compile_once_;
  bool compiled_ok_ = false;
  uint32_t op_uid_ = 0;
};

}  // namespace vx
}  // namespace tim
#endif  // TIMVX_B200_API_IMPL_H_
