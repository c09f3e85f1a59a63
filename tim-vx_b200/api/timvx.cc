// Implementation of the tim::vx classes on top of the b2vx C ABI.
//
// Behaviour follows the reference's C++ layer: Context (src/tim/vx/context.cc),
// Graph (src/tim/vx/graph.cc:91-394), Tensor (src/tim/vx/tensor.cc:105-592),
// Operation (src/tim/vx/operation.cc:43-97) and the op constructors under
// src/tim/vx/ops/.  Failures are reported as `false` plus one line on stderr,
// never as exceptions.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "impl.h"
#include "tim/vx/builtin_op.h"
#include "tim/vx/ops/addn.h"
#include "tim/vx/ops/instancenormalization.h"
#include "tim/vx/ops/relational_operations.h"
#include "tim/vx/ops/resize.h"
#include "tim/vx/ops/roi_align.h"
#include "tim/vx/ops/concat.h"
#include "tim/vx/ops/reshape.h"
#include "tim/vx/ops/simple_operations.h"
#include "tim/vx/ops/transpose.h"
#include "tim/vx/ops/activations.h"
#include "tim/vx/ops/conv2d.h"
#include "tim/vx/ops/elementwise.h"
#include "tim/vx/ops/fullyconnected.h"
#include "tim/vx/ops/groupedconv2d.h"
#include "tim/vx/ops/nbg.h"
#include "tim/vx/ops/pool2d.h"
#include "tim/vx/ops/softmax.h"

namespace tim {
namespace vx {

namespace {

int log_level() {
  // Same variable and levels as the reference's logger
  // (src/tim/vx/internal/src/vsi_nn_log.c:32-76): 0 none .. 4 debug, default 2.
  static int lvl = [] {
    const char* e = std::getenv("VSI_NN_LOG_LEVEL");
    return e ? std::atoi(e) : 2;
  }();
  return lvl;
}

#define TVX_LOGE(...)                                   \
  do {                                                  \
    if (log_level() >= 1) {                             \
      std::fprintf(stderr, "E [tim-vx/b200] ");         \
      std::fprintf(stderr, __VA_ARGS__);                \
      std::fprintf(stderr, "\n");                       \
    }                                                   \
  } while (0)
#define TVX_LOGW(...)                                   \
  do {                                                  \
    if (log_level() >= 2) {                             \
      std::fprintf(stderr, "W [tim-vx/b200] ");         \
      std::fprintf(stderr, __VA_ARGS__);                \
      std::fprintf(stderr, "\n");                       \
    }                                                   \
  } while (0)

int64_t element_bytes(DataType t) {
  switch (t) {
    case DataType::INT8: case DataType::UINT8: case DataType::BOOL8: return 1;
    case DataType::INT16: case DataType::UINT16: case DataType::FLOAT16: return 2;
    case DataType::INT32: case DataType::UINT32: case DataType::FLOAT32: return 4;
    case DataType::INT64: return 8;
    default: return 0;
  }
}

}  // namespace

// ---------------------------------------------------------------- Quantization / TensorSpec

bool Quantization::operator==(const Quantization& o) const {
  if (type_ != o.type_) return false;
  if (type_ == QuantType::NONE) return true;
  if (type_ == QuantType::DYNAMIC_FIXED_POINT) return fl_ == o.fl_;
  return channel_dim_ == o.channel_dim_ && scales_ == o.scales_ && zero_points_ == o.zero_points_;
}

TensorSpec::TensorSpec(const TensorSpec& other)
    : datatype_(other.datatype_), shape_(other.shape_), attr_(other.attr_),
      quantization_(other.quantization_) {}

TensorSpec& TensorSpec::operator=(const TensorSpec& other) {
  datatype_ = other.datatype_;
  shape_ = other.shape_;
  attr_ = other.attr_;
  quantization_ = other.quantization_;
  return *this;
}

bool TensorSpec::operator==(const TensorSpec& o) const {
  return datatype_ == o.datatype_ && shape_ == o.shape_ && attr_ == o.attr_ &&
         quantization_ == o.quantization_;
}

TensorSpec& TensorSpec::SetDataType(DataType d) { datatype_ = d; return *this; }
TensorSpec& TensorSpec::SetShape(const ShapeType& s) { shape_ = s; return *this; }
TensorSpec& TensorSpec::SetAttribute(TensorAttribute a) { attr_ = a; return *this; }
TensorSpec& TensorSpec::SetQuantization(Quantization& q) { quantization_ = q; return *this; }

TensorSpec TensorSpec::AsTransientSpec() const {
  return TensorSpec(datatype_, ShapeType({}), TensorAttribute::TRANSIENT, quantization_);
}

int64_t TensorSpec::GetElementNum() const {
  int64_t n = 1;
  for (uint32_t d : shape_) n *= d;
  return n;
}
int64_t TensorSpec::GetElementByteSize() const { return element_bytes(datatype_); }
int64_t TensorSpec::GetByteSize() const { return GetElementNum() * GetElementByteSize(); }

// ---------------------------------------------------------------- CompileOption

CompileOption CompileOption::DefaultOptions;

CompileOption::CompileOption() : impl_(new CompileOptionImpl()) {}
bool CompileOption::isRelaxMode() const { return impl_->relax_mode; }
bool CompileOption::setRelaxMode(bool enable) { impl_->relax_mode = enable; return true; }
void CompileOption::setDeviceId(uint32_t device) { impl_->device_id = device; }
uint32_t CompileOption::getDeviceId() const { return impl_->device_id; }

// ---------------------------------------------------------------- Context

std::shared_ptr<Context> Context::Create() { return std::make_shared<ContextImpl>(); }

ContextImpl::ContextImpl() {
  if (b2vx_context_create(&ctx_) != B2VX_OK) {
    TVX_LOGE("b2vx_context_create failed");
    ctx_ = nullptr;
  }
}
ContextImpl::~ContextImpl() {
  if (ctx_) b2vx_context_destroy(ctx_);
}
std::shared_ptr<Graph> ContextImpl::CreateGraph() {
  return std::make_shared<GraphImpl>(this, CompileOption::DefaultOptions);
}
std::shared_ptr<Graph> ContextImpl::CreateGraph(const CompileOption& options) {
  return std::make_shared<GraphImpl>(this, options);
}

// ---------------------------------------------------------------- Tensor

TensorImpl::TensorImpl(GraphImpl* graph, const TensorSpec& spec, const void* data, void* io_handle)
    : graph_(graph), spec_(spec) {
  if (!graph_->EnsureHandle()) return;
  const Quantization& q = spec_.quantization_;
  b2vx_tensor_desc d;
  std::memset(&d, 0, sizeof(d));
  d.dtype = static_cast<int32_t>(spec_.datatype_);
  d.rank = static_cast<uint32_t>(spec_.shape_.size());
  if (d.rank > B2VX_MAX_RANK) {
    TVX_LOGE("tensor rank %u exceeds %u", d.rank, B2VX_MAX_RANK);
    return;
  }
  for (uint32_t i = 0; i < d.rank; ++i) d.dims[i] = spec_.shape_[i];
  d.attr = static_cast<int32_t>(spec_.attr_);
  d.channel_dim = q.ChannelDim();
  switch (q.Type()) {
    case QuantType::NONE:
      d.quant_type = B2VX_QUANT_NONE;
      break;
    case QuantType::ASYMMETRIC:
      d.quant_type = B2VX_QUANT_ASYMMETRIC;
      d.scale = q.Scales().empty() ? 1.0f : q.Scales()[0];
      d.zero_point = q.ZeroPoints().empty() ? 0 : q.ZeroPoints()[0];
      break;
    case QuantType::SYMMETRIC_PER_CHANNEL:
      d.quant_type = B2VX_QUANT_SYMMETRIC_PER_CHANNEL;
      d.n_channel = static_cast<uint32_t>(q.Scales().size());
      d.scales = q.Scales().data();
      d.zero_points = q.ZeroPoints().size() == q.Scales().size() ? q.ZeroPoints().data() : nullptr;
      break;
    default:
      TVX_LOGE("quantization type %d is not supported by this backend", static_cast<int>(q.Type()));
      return;
  }
  uint32_t id = B2VX_NO_TENSOR;
  if (b2vx_tensor_create(graph_->handle(), &d, data, &id) != B2VX_OK) {
    graph_->LogBackendError("CreateTensor");
    return;
  }
  id_ = id;
  host_ = io_handle;
  if (data && (spec_.attr_ & TensorAttribute::CONSTANT)) {
    const uint8_t* p = static_cast<const uint8_t*>(data);
    const_copy_.assign(p, p + static_cast<size_t>(spec_.GetByteSize()));
  }
}

TensorImpl::~TensorImpl() {
  if (host_ && host_owned_) b2vx_host_free(host_);
}

void TensorImpl::RefreshShape() {
  if (!valid()) return;
  b2vx_tensor_desc d;
  if (b2vx_tensor_get_desc(graph_->handle(), id_, &d) != B2VX_OK) return;
  spec_.shape_.assign(d.dims, d.dims + d.rank);
}

const ShapeType& TensorImpl::GetShape() { return spec_.shape_; }

bool TensorImpl::CopyDataToTensor(const void* data, uint32_t /*size_in_bytes*/) {
  if (!valid() || data == nullptr) return false;
  if (spec_.attr_ & TensorAttribute::TRANSIENT) return false;
  size_t bytes = static_cast<size_t>(spec_.GetByteSize());
  if (host_ && host_ != data) std::memcpy(host_, data, bytes);
  if (b2vx_tensor_write(graph_->handle(), id_, data, bytes) != B2VX_OK) {
    graph_->LogBackendError("CopyDataToTensor");
    return false;
  }
  return true;
}

bool TensorImpl::CopyDataFromTensor(void* data) {
  if (!valid() || data == nullptr) return false;
  size_t bytes = static_cast<size_t>(spec_.GetByteSize());
  if (b2vx_tensor_read(graph_->handle(), id_, data, bytes) != B2VX_OK) {
    graph_->LogBackendError("CopyDataFromTensor");
    return false;
  }
  return true;
}

bool TensorImpl::EnsureHostBuffer() {
  if (host_) return true;
  size_t bytes = static_cast<size_t>(spec_.GetByteSize());
  if (bytes == 0) return false;
  if (b2vx_host_alloc(&host_, bytes) != B2VX_OK) {
    host_ = nullptr;
    return false;
  }
  host_owned_ = true;
  return true;
}

// Handle semantics of the reference (src/tim/vx/tensor.cc:243-389): an
// INPUT/OUTPUT tensor has a host side that the caller may own.  Here the host
// side is a plain buffer; unmap()/Flush push it to the GPU, map(true)/
// Invalidate pull the GPU copy into it.
bool TensorImpl::SwapHandle(void* new_ptr, bool /*is_new_ptr_malloc_by_ovxlib*/, void** old_ptr) {
  if (!valid() || !(spec_.attr_ & (TensorAttribute::INPUT | TensorAttribute::OUTPUT))) return false;
  if (old_ptr) *old_ptr = host_owned_ ? nullptr : host_;
  if (host_ && host_owned_) b2vx_host_free(host_);
  host_ = new_ptr;
  host_owned_ = false;
  if (host_ && (spec_.attr_ & TensorAttribute::INPUT)) return FlushCacheForHandle();
  return true;
}

bool TensorImpl::SwapHandle(std::shared_ptr<tim::vx::Tensor> tensor) {
  auto other = std::dynamic_pointer_cast<TensorImpl>(tensor);
  if (!other || other->spec_.GetByteSize() != spec_.GetByteSize()) return false;
  std::swap(host_, other->host_);
  std::swap(host_owned_, other->host_owned_);
  return true;
}

bool TensorImpl::SwapHandleWithCache(std::shared_ptr<tim::vx::Tensor> tensor) {
  if (!SwapHandle(tensor)) return false;
  if (spec_.attr_ & TensorAttribute::INPUT) return host_ ? FlushCacheForHandle() : true;
  return true;
}

bool TensorImpl::FlushCacheForHandle() {
  if (!valid() || !host_) return false;
  return b2vx_tensor_write(graph_->handle(), id_, host_, static_cast<size_t>(spec_.GetByteSize())) == B2VX_OK;
}

bool TensorImpl::InvalidateCacheForHandle() {
  if (!valid() || !host_) return false;
  return b2vx_tensor_read(graph_->handle(), id_, host_, static_cast<size_t>(spec_.GetByteSize())) == B2VX_OK;
}

void* TensorImpl::map(bool invalidate_cpu_cache) {
  if (!valid() || !(spec_.attr_ & (TensorAttribute::INPUT | TensorAttribute::OUTPUT))) return nullptr;
  if (!EnsureHostBuffer()) return nullptr;
  if (invalidate_cpu_cache || (spec_.attr_ & TensorAttribute::OUTPUT)) InvalidateCacheForHandle();
  return host_;
}

void TensorImpl::unmap() {
  if (valid() && host_ && (spec_.attr_ & TensorAttribute::INPUT)) FlushCacheForHandle();
}

float* TensorImpl::ConvertTensorToFloat32Data() {
  // Caller frees with free(), as with vsi_nn_ConvertTensorToFloat32Data.
  if (!valid()) return nullptr;
  size_t n = static_cast<size_t>(spec_.GetElementNum());
  std::vector<uint8_t> raw(static_cast<size_t>(spec_.GetByteSize()));
  if (!CopyDataFromTensor(raw.data())) return nullptr;
  float* out = static_cast<float*>(std::malloc(n * sizeof(float)));
  if (!out) return nullptr;
  std::shared_ptr<Tensor> self(this, [](Tensor*) {});
  if (!utils::DtypeToFloat32(self, raw.data(), out)) {
    std::free(out);
    return nullptr;
  }
  return out;
}

void* TensorImpl::ConvertTensorToData(uint8_t* tensorData) {
  if (!valid()) return nullptr;
  size_t bytes = static_cast<size_t>(spec_.GetByteSize());
  if (tensorData == nullptr) tensorData = static_cast<uint8_t*>(std::malloc(bytes));
  if (tensorData && !CopyDataFromTensor(tensorData)) return nullptr;
  return tensorData;
}

bool TensorImpl::SaveTensorToTextByFp32(std::string filename) {
  float* f = ConvertTensorToFloat32Data();
  if (!f) return false;
  FILE* fp = std::fopen(filename.c_str(), "w");
  if (!fp) {
    std::free(f);
    return false;
  }
  for (int64_t i = 0; i < spec_.GetElementNum(); ++i) std::fprintf(fp, "%f\n", f[i]);
  std::fclose(fp);
  std::free(f);
  return true;
}

namespace utils {

// Element-wise conversions with the tensor's quantization
// (reference: vsi_nn_Float32ToDtype / vsi_nn_DtypeToFloat32 via
// src/tim/vx/tensor.cc:571-587).  Quantization uses f/scale rounded to nearest
// even plus zero point, saturated to the type's range.
bool Float32ToDtype(std::shared_ptr<tim::vx::Tensor> tensor, std::vector<float> fval,
                    uint8_t* tensorData) {
  if (!tensor || !tensorData) return false;
  const Quantization& q = tensor->GetQuantization();
  float scale = q.Scales().empty() ? 1.0f : q.Scales()[0];
  int32_t zp = q.ZeroPoints().empty() ? 0 : q.ZeroPoints()[0];
  for (size_t i = 0; i < fval.size(); ++i) {
    switch (tensor->GetDataType()) {
      case DataType::FLOAT32:
        reinterpret_cast<float*>(tensorData)[i] = fval[i];
        break;
      case DataType::UINT8: {
        double v = std::nearbyint(static_cast<double>(fval[i] / scale)) + zp;
        tensorData[i] = static_cast<uint8_t>(std::min(255.0, std::max(0.0, v)));
        break;
      }
      case DataType::INT8: {
        double v = std::nearbyint(static_cast<double>(fval[i] / scale)) + zp;
        reinterpret_cast<int8_t*>(tensorData)[i] =
            static_cast<int8_t>(std::min(127.0, std::max(-128.0, v)));
        break;
      }
      case DataType::INT32: {
        double v = std::nearbyint(static_cast<double>(fval[i] / scale)) + zp;
        reinterpret_cast<int32_t*>(tensorData)[i] =
            static_cast<int32_t>(std::min(2147483647.0, std::max(-2147483648.0, v)));
        break;
      }
      default:
        return false;
    }
  }
  return true;
}

bool DtypeToFloat32(std::shared_ptr<tim::vx::Tensor> tensor, uint8_t* tensorData, float* data) {
  if (!tensor || !tensorData || !data) return false;
  const Quantization& q = tensor->GetQuantization();
  float scale = q.Scales().empty() ? 1.0f : q.Scales()[0];
  int32_t zp = q.ZeroPoints().empty() ? 0 : q.ZeroPoints()[0];
  int64_t n = tensor->GetSpec().GetElementNum();
  for (int64_t i = 0; i < n; ++i) {
    switch (tensor->GetDataType()) {
      case DataType::FLOAT32: data[i] = reinterpret_cast<float*>(tensorData)[i]; break;
      case DataType::UINT8: data[i] = (static_cast<float>(tensorData[i]) - zp) * scale; break;
      case DataType::INT8:
        data[i] = (static_cast<float>(reinterpret_cast<int8_t*>(tensorData)[i]) - zp) * scale;
        break;
      case DataType::INT32:
        data[i] = (static_cast<float>(reinterpret_cast<int32_t*>(tensorData)[i]) - zp) * scale;
        break;
      default: return false;
    }
  }
  return true;
}

}  // namespace utils

// ---------------------------------------------------------------- Graph

GraphImpl::GraphImpl(ContextImpl* context, const CompileOption& options)
    : context_(context), options_(options) {}

GraphImpl::~GraphImpl() {
  // Ops and tensors hold raw pointers to this graph; release them first.
  op_vector_.clear();
  tensor_consumers_.clear();
  tensor_producer_.clear();
  inputs_tensor_.clear();
  outputs_tensor_.clear();
  if (graph_) b2vx_graph_destroy(graph_);
}

bool GraphImpl::EnsureHandle() {
  if (graph_) return true;
  if (!context_ || !context_->handle()) return false;
  int32_t dev = static_cast<int32_t>(options_.getDeviceId());
  if (const char* e = std::getenv("B2VX_DEVICE")) dev = std::atoi(e);
  if (b2vx_graph_create(context_->handle(), dev, &graph_) != B2VX_OK) {
    LogBackendError("CreateGraph");
    graph_ = nullptr;
    return false;
  }
  return true;
}

void GraphImpl::LogBackendError(const char* where) const {
  TVX_LOGE("%s: %s", where, context_ && context_->handle() ? b2vx_last_error(context_->handle()) : "no context");
}

std::shared_ptr<Tensor> GraphImpl::CreateTensor(const TensorSpec& spec, const void* data) {
  auto t = std::make_shared<TensorImpl>(this, spec, data, nullptr);
  if (!t->valid()) return nullptr;
  if (spec.attr_ & TensorAttribute::INPUT) inputs_tensor_.push_back(t);
  if (spec.attr_ & TensorAttribute::OUTPUT) outputs_tensor_.push_back(t);
  all_tensors_.push_back(t);
  return t;
}

std::shared_ptr<Tensor> GraphImpl::CreateTensor(const TensorSpec& /*spec*/, const DmaBufferDesc& /*dmafd*/) {
  TVX_LOGE("dma-buf backed tensors are not supported");
  return nullptr;
}

std::shared_ptr<Tensor> GraphImpl::CreateIOTensor(const TensorSpec& spec, void* data) {
  if (!(spec.attr_ & (TensorAttribute::INPUT | TensorAttribute::OUTPUT))) {
    TVX_LOGE("CreateIOTensor needs an INPUT or OUTPUT spec");
    return nullptr;
  }
  auto t = std::make_shared<TensorImpl>(this, spec, nullptr, data);
  if (!t->valid()) return nullptr;
  // As in the reference (src/tim/vx/tensor.cc:126-137) IO tensors made here
  // are not appended to the graph's input/output lists.
  all_tensors_.push_back(t);
  return t;
}

std::shared_ptr<Tensor> GraphImpl::CreateTensorPlaceHolder() {
  return std::make_shared<TensorPlaceholder>();
}

void GraphImpl::UpdateTensorConsumersMap(const std::shared_ptr<Tensor>& tensor, const Operation* op) {
  for (const auto& sp : op_vector_) {
    if (sp.get() == op) {
      tensor_consumers_[tensor].push_back(sp);
      return;
    }
  }
}

void GraphImpl::RenewTensorConsumersMap(const std::shared_ptr<Tensor>& org_tensor,
                                        const std::shared_ptr<Tensor>& dst_tensor,
                                        const Operation* op) {
  auto it = tensor_consumers_.find(org_tensor);
  if (it != tensor_consumers_.end()) {
    auto& v = it->second;
    v.erase(std::remove_if(v.begin(), v.end(), [op](const std::shared_ptr<Operation>& p) { return p.get() == op; }),
            v.end());
    if (v.empty()) tensor_consumers_.erase(it);
  }
  UpdateTensorConsumersMap(dst_tensor, op);
}

void GraphImpl::UpdateTensorProducerMap(const std::shared_ptr<Tensor>& tensor, const Operation* op) {
  for (const auto& sp : op_vector_) {
    if (sp.get() == op) {
      tensor_producer_[tensor] = sp;
      return;
    }
  }
}

const std::vector<std::shared_ptr<Operation>> GraphImpl::GetConsumersOp(std::shared_ptr<Tensor> tensor) const {
  auto it = tensor_consumers_.find(tensor);
  if (it == tensor_consumers_.end()) return {};
  return it->second;
}

std::shared_ptr<Operation> GraphImpl::GetProducerOp(std::shared_ptr<Tensor> tensor) {
  auto it = tensor_producer_.find(tensor);
  return it == tensor_producer_.end() ? nullptr : it->second;
}

const std::vector<std::shared_ptr<Tensor>> Graph::GetConstantInputs() const {
  std::vector<std::shared_ptr<Tensor>> out;
  for (const auto& op : op_vector_) {
    auto c = op->ConstantInputsTensor();
    out.insert(out.end(), c.begin(), c.end());
  }
  return out;
}

bool GraphImpl::EmitNodes() {
  for (const auto& op : op_vector_) {
    OpImpl* p = op->impl().get();
    auto in = [&](size_t i) -> uint32_t {
      return i < p->inputs_tensor_.size() && p->inputs_tensor_[i] ? p->inputs_tensor_[i]->GetId() : B2VX_NO_TENSOR;
    };
    auto out = [&](size_t i) -> uint32_t {
      return i < p->outputs_tensor_.size() && p->outputs_tensor_[i] ? p->outputs_tensor_[i]->GetId() : B2VX_NO_TENSOR;
    };
    // As in the reference, the layouts named in an op's constructor only inform tim::transform::LayoutInference;
    // a graph compiled without it runs every op as WHCN / WHIcOc (its conv2d_test.cc relies on that).
    if (p->foreign_layout_) TVX_LOGW("an op names a CWHN / front-end kernel layout and runs as WHCN / WHIcOc: layout inference was not applied");
    if (p->overflow_policy_ != OverflowPolicy::SATURATE || p->rounding_policy_ != RoundingPolicy::RTNE) {
      TVX_LOGE("SetRoundingPolicy: this backend saturates and rounds to nearest even; OverflowPolicy::WRAP and RoundingPolicy::TO_ZERO are not supported");
      return false;
    }
    b2vx_status st = B2VX_UNSUPPORTED;
    switch (p->kind_) {
      case B2VX_NODE_CONV2D: st = b2vx_node_conv2d(graph_, in(0), in(1), in(2), out(0), &p->desc_.conv2d); break;
      case B2VX_NODE_FULLY_CONNECTED:
        st = b2vx_node_fully_connected(graph_, in(0), in(1), in(2), out(0), &p->desc_.fc);
        break;
      case B2VX_NODE_POOL2D: st = b2vx_node_pool2d(graph_, in(0), out(0), &p->desc_.pool2d); break;
      case B2VX_NODE_ADD: st = b2vx_node_add(graph_, in(0), in(1), out(0)); break;
      case B2VX_NODE_RELU: st = b2vx_node_relu(graph_, in(0), out(0)); break;
      case B2VX_NODE_RELU6: st = b2vx_node_relu6(graph_, in(0), out(0)); break;
      case B2VX_NODE_SOFTMAX: st = b2vx_node_softmax(graph_, in(0), out(0), &p->desc_.softmax); break;
      case B2VX_NODE_RESHAPE: st = b2vx_node_reshape(graph_, in(0), out(0), &p->desc_.dims); break;
      case B2VX_NODE_TRANSPOSE: st = b2vx_node_transpose(graph_, in(0), out(0), &p->desc_.dims); break;
      case B2VX_NODE_DATACONVERT: st = b2vx_node_dataconvert(graph_, in(0), out(0)); break;
      case B2VX_NODE_CONCAT: {
        std::vector<uint32_t> ids;
        for (size_t k = 0; k < p->inputs_tensor_.size(); ++k) ids.push_back(in(k));
        st = b2vx_node_concat(graph_, ids.data(), static_cast<uint32_t>(ids.size()), p->desc_.concat_axis, out(0));
        break;
      }
      case B2VX_NODE_ADDN: {
        std::vector<uint32_t> ids;
        for (size_t k = 0; k < p->inputs_tensor_.size(); ++k) ids.push_back(in(k));
        st = b2vx_node_addn(graph_, ids.data(), static_cast<uint32_t>(ids.size()), out(0));
        break;
      }
      case kNodeKindNbg: st = ExpandBlob(p) ? B2VX_OK : B2VX_INVALID_ARG; break;
      case kNodeKindDeclaredOnly:
        TVX_LOGE("ops::%s is declared for source compatibility only; this backend does not execute it", p->name_);
        return false;
      default: break;
    }
    if (st != B2VX_OK) {
      LogBackendError("AddNode");
      return false;
    }
  }
  return true;
}

bool GraphImpl::Compile() {
  std::call_once(compile_once_, [this] {
    if (!EnsureHandle()) return;
    if (!EmitNodes()) return;
    if (b2vx_graph_compile(graph_) != B2VX_OK) {
      LogBackendError("Compile");
      return;
    }
    for (auto& w : all_tensors_) {
      if (auto t = w.lock()) t->RefreshShape();
    }
    compiled_ok_ = true;
  });
  return compiled_ok_;
}

// ---------------------------------------------------------------- serialised graphs
//
// Graph::CompileToBinary (src/tim/vx/graph.cc:385-387 hands this to vsi_nn_GenerateNBG) writes what
// this layer recorded: every tensor an op touches (descriptor, quantization, constant data) and every
// op (kind, descriptor, bindings), plus which tensors are the graph's inputs and outputs, in order.
// ops::NBG (include/tim/vx/ops/nbg.h) takes such a blob; at Compile it is expanded into the nodes it
// describes, its graph inputs and outputs replaced by the tensors bound to the op.  The format is
// this backend's own ("B2VB", little endian, version 2); kernels are planned again on load, for the
// GPU the loading graph is bound to.
namespace {

constexpr uint32_t kBlobMagic = 0x42563242u;   // "B2VB"
constexpr uint32_t kBlobVersion = 2;

struct BlobWriter {
  std::vector<uint8_t> b;
  template <typename T> void put(const T& v) {
    const uint8_t* p = reinterpret_cast<const uint8_t*>(&v);
    b.insert(b.end(), p, p + sizeof(T));
  }
  void bytes(const void* p, size_t n) {
    const uint8_t* q = static_cast<const uint8_t*>(p);
    b.insert(b.end(), q, q + n);
  }
};

struct BlobReader {
  const uint8_t* p;
  size_t left;
  bool ok = true;
  template <typename T> T get() {
    T v{};
    if (left < sizeof(T)) { ok = false; return v; }
    std::memcpy(&v, p, sizeof(T));
    p += sizeof(T);
    left -= sizeof(T);
    return v;
  }
  const uint8_t* bytes(size_t n) {
    if (left < n) { ok = false; return nullptr; }
    const uint8_t* q = p;
    p += n;
    left -= n;
    return q;
  }
};

}  // namespace

bool GraphImpl::CompileToBinary(void* buf, size_t* size) {
  if (!size) return false;
  if (op_vector_.empty()) {   // as vsi_nn_GenerateNBG on a graph without nodes (src/tim/vx/graph_test.cc:32-38 expects false)
    TVX_LOGE("CompileToBinary: the graph has no operation");
    return false;
  }
  std::map<const Tensor*, uint32_t> index;
  std::vector<std::shared_ptr<Tensor>> tensors;
  auto add = [&](const std::shared_ptr<Tensor>& t) {
    if (!t || t->IsPlaceHolder()) return;
    if (index.emplace(t.get(), static_cast<uint32_t>(tensors.size())).second) tensors.push_back(t);
  };
  for (const auto& op : op_vector_) {
    if (op->impl()->kind_ == kNodeKindNbg) {
      TVX_LOGE("CompileToBinary: a graph that contains an NBG op cannot be serialised again");
      return false;
    }
    for (const auto& t : op->impl()->inputs_tensor_) add(t);
    for (const auto& t : op->impl()->outputs_tensor_) add(t);
  }
  BlobWriter w;
  w.put(kBlobMagic);
  w.put(kBlobVersion);
  w.put<uint64_t>(0);   // total size, patched below
  w.put(static_cast<uint32_t>(tensors.size()));
  w.put(static_cast<uint32_t>(op_vector_.size()));
  w.put(static_cast<uint32_t>(inputs_tensor_.size()));
  w.put(static_cast<uint32_t>(outputs_tensor_.size()));
  for (const auto& t : tensors) {
    TensorSpec& sp = t->GetSpec();
    const Quantization& q = sp.quantization_;
    w.put(static_cast<int32_t>(sp.datatype_));
    w.put(static_cast<int32_t>(sp.attr_));
    // TRANSIENT tensors go in without a shape, as the user declared them (Compile infers it again)
    const bool shapeless = sp.attr_ == TensorAttribute::TRANSIENT;
    w.put(static_cast<uint32_t>(shapeless ? 0 : sp.shape_.size()));
    if (!shapeless) for (uint32_t d : sp.shape_) w.put(d);
    w.put(static_cast<int32_t>(q.Type()));
    w.put(static_cast<int32_t>(q.ChannelDim()));
    w.put(static_cast<uint32_t>(q.Scales().size()));
    for (float v : q.Scales()) w.put(v);
    w.put(static_cast<uint32_t>(q.ZeroPoints().size()));
    for (int32_t v : q.ZeroPoints()) w.put(v);
    const std::vector<uint8_t>& data = static_cast<TensorImpl*>(t.get())->ConstData();
    if ((sp.attr_ & TensorAttribute::CONSTANT) && data.empty()) {
      TVX_LOGE("CompileToBinary: a CONSTANT tensor was created without data");
      return false;
    }
    w.put(static_cast<uint64_t>(data.size()));
    w.bytes(data.data(), data.size());
  }
  auto put_ids = [&](const std::vector<std::shared_ptr<Tensor>>& v) {
    w.put(static_cast<uint32_t>(v.size()));
    for (const auto& t : v) w.put(t && !t->IsPlaceHolder() ? index[t.get()] : B2VX_NO_TENSOR);
  };
  for (const auto& op : op_vector_) {
    const OpImpl* p = op->impl().get();
    w.put(p->kind_);
    w.bytes(&p->desc_, sizeof(p->desc_));
    put_ids(p->inputs_tensor_);
    put_ids(p->outputs_tensor_);
  }
  for (const auto& t : inputs_tensor_) w.put(index.count(t.get()) ? index[t.get()] : B2VX_NO_TENSOR);
  for (const auto& t : outputs_tensor_) w.put(index.count(t.get()) ? index[t.get()] : B2VX_NO_TENSOR);
  const uint64_t total = w.b.size();
  std::memcpy(w.b.data() + 8, &total, sizeof(total));
  if (buf) {
    if (*size < total) {
      TVX_LOGE("CompileToBinary: buffer of %zu bytes, %llu needed", *size, static_cast<unsigned long long>(total));
      return false;
    }
    std::memcpy(buf, w.b.data(), total);
  }
  *size = static_cast<size_t>(total);
  return true;
}

bool GraphImpl::ExpandBlob(const OpImpl* op) {
  BlobReader r{op->blob_.data(), op->blob_.size()};
  if (r.get<uint32_t>() != kBlobMagic || r.get<uint32_t>() != kBlobVersion) {
    TVX_LOGE("NBG: not a graph serialised by this backend");
    return false;
  }
  r.get<uint64_t>();
  const uint32_t n_tensors = r.get<uint32_t>(), n_ops = r.get<uint32_t>(), n_in = r.get<uint32_t>(), n_out = r.get<uint32_t>();
  if (!r.ok || op->inputs_tensor_.size() != n_in || op->outputs_tensor_.size() != n_out) {
    TVX_LOGE("NBG: the blob has %u inputs and %u outputs, the op has %zu and %zu bound", n_in, n_out,
             op->inputs_tensor_.size(), op->outputs_tensor_.size());
    return false;
  }
  struct Rec {
    b2vx_tensor_desc d;
    std::vector<float> scales;
    std::vector<int32_t> zps;
    const uint8_t* data = nullptr;
    uint64_t bytes = 0;
  };
  std::vector<Rec> recs(n_tensors);
  for (Rec& t : recs) {
    std::memset(&t.d, 0, sizeof(t.d));
    t.d.dtype = r.get<int32_t>();
    t.d.attr = r.get<int32_t>();
    t.d.rank = r.get<uint32_t>();
    if (!r.ok || t.d.rank > B2VX_MAX_RANK) return false;
    for (uint32_t i = 0; i < t.d.rank; ++i) t.d.dims[i] = r.get<uint32_t>();
    const int32_t qtype = r.get<int32_t>();
    t.d.channel_dim = r.get<int32_t>();
    const uint32_t ns = r.get<uint32_t>();
    if (!r.ok || ns > (1u << 24)) return false;
    t.scales.resize(ns);
    for (float& v : t.scales) v = r.get<float>();
    const uint32_t nz = r.get<uint32_t>();
    if (!r.ok || nz > (1u << 24)) return false;
    t.zps.resize(nz);
    for (int32_t& v : t.zps) v = r.get<int32_t>();
    switch (static_cast<QuantType>(qtype)) {
      case QuantType::NONE: t.d.quant_type = B2VX_QUANT_NONE; break;
      case QuantType::ASYMMETRIC:
        t.d.quant_type = B2VX_QUANT_ASYMMETRIC;
        t.d.scale = t.scales.empty() ? 1.0f : t.scales[0];
        t.d.zero_point = t.zps.empty() ? 0 : t.zps[0];
        break;
      case QuantType::SYMMETRIC_PER_CHANNEL:
        t.d.quant_type = B2VX_QUANT_SYMMETRIC_PER_CHANNEL;
        t.d.n_channel = ns;
        break;
      default: return false;
    }
    t.bytes = r.get<uint64_t>();
    t.data = r.bytes(static_cast<size_t>(t.bytes));
    if (!r.ok) return false;
  }
  struct OpRec {
    uint32_t kind;
    decltype(OpImpl::desc_) desc;
    std::vector<uint32_t> in, out;
  };
  std::vector<OpRec> ops(n_ops);
  for (OpRec& o : ops) {
    o.kind = r.get<uint32_t>();
    const uint8_t* d = r.bytes(sizeof(o.desc));
    if (!r.ok) return false;
    std::memcpy(&o.desc, d, sizeof(o.desc));
    o.in.resize(r.get<uint32_t>());
    if (!r.ok || o.in.size() > 16) return false;
    for (uint32_t& v : o.in) v = r.get<uint32_t>();
    o.out.resize(r.get<uint32_t>());
    if (!r.ok || o.out.size() > 16) return false;
    for (uint32_t& v : o.out) v = r.get<uint32_t>();
  }
  std::vector<uint32_t> id(n_tensors, B2VX_NO_TENSOR);
  for (uint32_t k = 0; k < n_in; ++k) {
    const uint32_t t = r.get<uint32_t>();
    if (!r.ok || t >= n_tensors || !op->inputs_tensor_[k]) return false;
    id[t] = op->inputs_tensor_[k]->GetId();
  }
  for (uint32_t k = 0; k < n_out; ++k) {
    const uint32_t t = r.get<uint32_t>();
    if (!r.ok || t >= n_tensors || !op->outputs_tensor_[k]) return false;
    id[t] = op->outputs_tensor_[k]->GetId();
  }
  for (uint32_t t = 0; t < n_tensors; ++t) {
    if (id[t] != B2VX_NO_TENSOR) continue;
    Rec& rec = recs[t];
    if (rec.d.quant_type == B2VX_QUANT_SYMMETRIC_PER_CHANNEL) {
      rec.d.scales = rec.scales.data();
      rec.d.zero_points = rec.zps.size() == rec.scales.size() ? rec.zps.data() : nullptr;
    }
    // a blob input or output that the op does not bind cannot occur (counts were checked); everything
    // else is created as recorded
    if (b2vx_tensor_create(graph_, &rec.d, rec.bytes ? rec.data : nullptr, &id[t]) != B2VX_OK) {
      LogBackendError("NBG tensor");
      return false;
    }
  }
  auto at = [&](const std::vector<uint32_t>& v, size_t i) -> uint32_t {
    return i < v.size() && v[i] != B2VX_NO_TENSOR && v[i] < n_tensors ? id[v[i]] : B2VX_NO_TENSOR;
  };
  for (OpRec& o : ops) {
    b2vx_status st = B2VX_UNSUPPORTED;
    switch (o.kind) {
      case B2VX_NODE_CONV2D: st = b2vx_node_conv2d(graph_, at(o.in, 0), at(o.in, 1), at(o.in, 2), at(o.out, 0), &o.desc.conv2d); break;
      case B2VX_NODE_FULLY_CONNECTED:
        st = b2vx_node_fully_connected(graph_, at(o.in, 0), at(o.in, 1), at(o.in, 2), at(o.out, 0), &o.desc.fc);
        break;
      case B2VX_NODE_POOL2D: st = b2vx_node_pool2d(graph_, at(o.in, 0), at(o.out, 0), &o.desc.pool2d); break;
      case B2VX_NODE_ADD: st = b2vx_node_add(graph_, at(o.in, 0), at(o.in, 1), at(o.out, 0)); break;
      case B2VX_NODE_RELU: st = b2vx_node_relu(graph_, at(o.in, 0), at(o.out, 0)); break;
      case B2VX_NODE_RELU6: st = b2vx_node_relu6(graph_, at(o.in, 0), at(o.out, 0)); break;
      case B2VX_NODE_SOFTMAX: st = b2vx_node_softmax(graph_, at(o.in, 0), at(o.out, 0), &o.desc.softmax); break;
      case B2VX_NODE_RESHAPE: st = b2vx_node_reshape(graph_, at(o.in, 0), at(o.out, 0), &o.desc.dims); break;
      case B2VX_NODE_TRANSPOSE: st = b2vx_node_transpose(graph_, at(o.in, 0), at(o.out, 0), &o.desc.dims); break;
      case B2VX_NODE_DATACONVERT: st = b2vx_node_dataconvert(graph_, at(o.in, 0), at(o.out, 0)); break;
      case B2VX_NODE_CONCAT: {
        std::vector<uint32_t> ids;
        for (size_t k = 0; k < o.in.size(); ++k) ids.push_back(at(o.in, k));
        st = b2vx_node_concat(graph_, ids.data(), static_cast<uint32_t>(ids.size()), o.desc.concat_axis, at(o.out, 0));
        break;
      }
      case B2VX_NODE_ADDN: {
        std::vector<uint32_t> ids;
        for (size_t k = 0; k < o.in.size(); ++k) ids.push_back(at(o.in, k));
        st = b2vx_node_addn(graph_, ids.data(), static_cast<uint32_t>(ids.size()), at(o.out, 0));
        break;
      }
      default: break;
    }
    if (st != B2VX_OK) {
      LogBackendError("NBG node");
      return false;
    }
  }
  return true;
}

bool GraphImpl::Run() {
  if (!Compile()) return false;
  if (b2vx_graph_run(graph_) != B2VX_OK) {
    LogBackendError("Run");
    return false;
  }
  return true;
}

void GraphImpl::PrintGraph() const {
  if (graph_) b2vx_graph_print(graph_);
}

// ---------------------------------------------------------------- Operation

OpImpl::OpImpl(Graph* graph, uint32_t kind, int in_cnt, int out_cnt, DataLayout layout)
    : graph_(graph), kind_(kind), input_cnt_(in_cnt), output_cnt_(out_cnt), layout_(layout),
      uid_(static_cast<GraphImpl*>(graph)->NextOpUid()) {
  std::memset(&desc_, 0, sizeof(desc_));
}

Operation::Operation() {}
Operation::~Operation() {}

std::unique_ptr<OpImpl>& Operation::impl() { return impl_; }
const std::unique_ptr<OpImpl>& Operation::impl() const { return impl_; }
const uint32_t& Operation::uid() const { return impl_->uid_; }

Operation& Operation::BindInput(const std::shared_ptr<Tensor>& tensor) {
  impl_->inputs_tensor_.push_back(tensor);
  if (tensor && !tensor->IsPlaceHolder()) impl_->graph_->UpdateTensorConsumersMap(tensor, this);
  OnBindInputPostProc(tensor, static_cast<int32_t>(impl_->inputs_tensor_.size()) - 1);
  return *this;
}

Operation& Operation::BindOutput(const std::shared_ptr<Tensor>& tensor) {
  impl_->outputs_tensor_.push_back(tensor);
  if (tensor) impl_->graph_->UpdateTensorProducerMap(tensor, this);
  return *this;
}

Operation& Operation::BindInputs(const std::vector<std::shared_ptr<Tensor>>& tensors) {
  for (const auto& t : tensors) BindInput(t);
  return *this;
}

Operation& Operation::BindOutputs(const std::vector<std::shared_ptr<Tensor>>& tensors) {
  for (const auto& t : tensors) BindOutput(t);
  return *this;
}

// BuiltinOpImpl::SetRoundingPolicy (src/tim/vx/builtin_op_impl.cc:65-74) writes the four values into the node's
// vx_param.  This backend saturates and rounds to nearest even, always; the values are kept, and Compile refuses a
// graph with an op that asked for anything else instead of quietly computing something the caller did not order.
Operation& Operation::SetRoundingPolicy(OverflowPolicy overflow_policy, RoundingPolicy rounding_policy,
                                        RoundType down_scale_size_rounding, uint32_t accumulator_bits) {
  impl_->overflow_policy_ = overflow_policy;
  impl_->rounding_policy_ = rounding_policy;
  impl_->down_scale_size_rounding_ = down_scale_size_rounding;
  impl_->accumulator_bits_ = accumulator_bits;
  return *this;
}

const std::vector<std::shared_ptr<Tensor>> Operation::ConstantInputsTensor() const {
  if (IsAllInputsConst()) return impl_->inputs_tensor_;
  return {};
}

bool Operation::IsAllInputsConst() const {
  for (const auto& t : impl_->inputs_tensor_) {
    if (!t || !t->IsConstTensor()) return false;
  }
  return true;
}

void Operation::OnBindInputPostProc(const std::shared_ptr<Tensor>&, int32_t) {}

BuiltinOp::BuiltinOp(Graph* graph, uint32_t kind, int in_cnt, int out_cnt, DataLayout layout) {
  impl_.reset(new OpImpl(graph, kind, in_cnt, out_cnt, layout));
}

// ---------------------------------------------------------------- ops

namespace ops {

Conv2d::Conv2d(Graph* graph, PadType padding, const std::array<uint32_t, 2>& stride,
               const std::array<uint32_t, 2>& dilation, int32_t multiplier, DataLayout input_layout,
               DataLayout kernel_layout)
    : Conv2d(graph, 0, padding, {0, 0}, stride, dilation, {0, 0, 0, 0}, multiplier, input_layout, kernel_layout) {}

Conv2d::Conv2d(Graph* graph, const std::array<uint32_t, 4> pad, const std::array<uint32_t, 2>& stride,
               const std::array<uint32_t, 2>& dilation, int32_t multiplier, DataLayout input_layout,
               DataLayout kernel_layout)
    : Conv2d(graph, 0, PadType::AUTO, {0, 0}, stride, dilation, pad, multiplier, input_layout, kernel_layout) {}

Conv2d::Conv2d(Graph* graph, int32_t weights, PadType padding, const std::array<uint32_t, 2>& ksize,
               const std::array<uint32_t, 2>& stride, const std::array<uint32_t, 2>& dilation,
               int32_t multiplier, DataLayout input_layout, DataLayout kernel_layout)
    : Conv2d(graph, weights, padding, ksize, stride, dilation, {0, 0, 0, 0}, multiplier, input_layout,
             kernel_layout) {}

Conv2d::Conv2d(Graph* graph, int32_t weights, PadType padding, const std::array<uint32_t, 2>& ksize,
               const std::array<uint32_t, 2>& stride, const std::array<uint32_t, 2>& dilation,
               const std::array<uint32_t, 4>& pad, int32_t multiplier, DataLayout input_layout,
               DataLayout kernel_layout)
    : BuiltinOp(graph, B2VX_NODE_CONV2D, 0, 0, input_layout),
      weights_(weights), padding_(padding), ksize_(ksize), stride_(stride), dilation_(dilation),
      pad_(pad), multiplier_(multiplier), kernel_layout_(kernel_layout) {
  b2vx_conv2d_desc& d = impl_->desc_.conv2d;
  d.weights = weights_;
  d.pad_type = static_cast<int32_t>(padding_);
  for (int i = 0; i < 2; ++i) {
    d.ksize[i] = ksize_[i];
    d.stride[i] = stride_[i];
    d.dilation[i] = dilation_[i];
  }
  for (int i = 0; i < 4; ++i) d.pad[i] = pad_[i];
  d.multiplier = multiplier_;
  impl_->kernel_layout_ = kernel_layout;
  impl_->foreign_layout_ = (input_layout != DataLayout::WHCN && input_layout != DataLayout::ANY) ||
                           (kernel_layout != DataLayout::WHIcOc && kernel_layout != DataLayout::ANY);
}

GroupedConv2d::GroupedConv2d(Graph* graph, PadType padding, const std::array<uint32_t, 2>& strides,
                             const std::array<uint32_t, 2>& dilation, int32_t grouped_number, DataLayout input_layout,
                             DataLayout kernel_layout)
    : BuiltinOp(graph, B2VX_NODE_CONV2D, 3, 1, input_layout), padding_(padding), strides_(strides), dilation_(dilation),
      pad_({0, 0, 0, 0}), group_number_(grouped_number), kernel_layout_(kernel_layout) {
  b2vx_conv2d_desc& d = impl_->desc_.conv2d;
  d.pad_type = static_cast<int32_t>(padding_);
  for (int i = 0; i < 2; ++i) {
    d.stride[i] = strides_[i];
    d.dilation[i] = dilation_[i];
  }
  d.group = group_number_;
  impl_->kernel_layout_ = kernel_layout;
  impl_->foreign_layout_ = (input_layout != DataLayout::WHCN && input_layout != DataLayout::ANY) ||
                           (kernel_layout != DataLayout::WHIcOc && kernel_layout != DataLayout::ANY);
}

GroupedConv2d::GroupedConv2d(Graph* graph, const std::array<uint32_t, 4>& pad, const std::array<uint32_t, 2>& strides,
                             const std::array<uint32_t, 2>& dilation, int32_t group_number, DataLayout input_layout,
                             DataLayout kernel_layout)
    : BuiltinOp(graph, B2VX_NODE_CONV2D, 3, 1, input_layout), padding_(PadType::AUTO), strides_(strides), dilation_(dilation),
      pad_(pad), group_number_(group_number), kernel_layout_(kernel_layout) {
  b2vx_conv2d_desc& d = impl_->desc_.conv2d;
  d.pad_type = static_cast<int32_t>(padding_);
  for (int i = 0; i < 2; ++i) {
    d.stride[i] = strides_[i];
    d.dilation[i] = dilation_[i];
  }
  for (int i = 0; i < 4; ++i) d.pad[i] = pad_[i];
  d.group = group_number_;
  impl_->kernel_layout_ = kernel_layout;
  impl_->foreign_layout_ = (input_layout != DataLayout::WHCN && input_layout != DataLayout::ANY) ||
                           (kernel_layout != DataLayout::WHIcOc && kernel_layout != DataLayout::ANY);
}

std::shared_ptr<Operation> GroupedConv2d::Clone(std::shared_ptr<Graph>& graph) const {
  if (padding_ == PadType::AUTO)
    return graph->CreateOperation<GroupedConv2d>(pad_, strides_, dilation_, group_number_, impl_->layout_, kernel_layout_);
  return graph->CreateOperation<GroupedConv2d>(padding_, strides_, dilation_, group_number_, impl_->layout_, kernel_layout_);
}

std::shared_ptr<Operation> Conv2d::Clone(std::shared_ptr<Graph>& graph) const {
  return graph->CreateOperation<Conv2d>(static_cast<int32_t>(weights_), padding_, ksize_, stride_, dilation_, pad_,
                                        multiplier_, impl_->layout_, kernel_layout_);
}

const std::vector<std::shared_ptr<Tensor>> Conv2d::ConstantInputsTensor() const {
  if (IsAllInputsConst()) return {impl_->inputs_tensor_[0]};
  return {};
}

FullyConnected::FullyConnected(Graph* graph, uint32_t axis) : FullyConnected(graph, axis, 0) {}

FullyConnected::FullyConnected(Graph* graph, uint32_t axis, uint32_t weights)
    : BuiltinOp(graph, B2VX_NODE_FULLY_CONNECTED), axis_(axis), weights_(weights) {
  impl_->desc_.fc.axis = axis;
  impl_->desc_.fc.weights = weights;
}

std::shared_ptr<Operation> FullyConnected::Clone(std::shared_ptr<Graph>& graph) const {
  return graph->CreateOperation<FullyConnected>(axis_, weights_);
}

Pool2d::Pool2d(Graph* graph, PoolType type, PadType padding, const std::array<uint32_t, 2>& ksize,
               const std::array<uint32_t, 2>& stride, RoundType round_type, DataLayout layout)
    : BuiltinOp(graph, B2VX_NODE_POOL2D, 1, 1, layout),
      type_(type), padding_(padding), ksize_(ksize), stride_(stride), round_type_(round_type),
      pad_({0, 0, 0, 0}) {
  Init();
}

Pool2d::Pool2d(Graph* graph, PoolType type, const std::array<uint32_t, 4>& pad,
               const std::array<uint32_t, 2>& ksize, const std::array<uint32_t, 2>& stride,
               RoundType round_type, DataLayout layout)
    : BuiltinOp(graph, B2VX_NODE_POOL2D, 1, 1, layout),
      type_(type), padding_(PadType::AUTO), ksize_(ksize), stride_(stride), round_type_(round_type), pad_(pad) {
  Init();
}

Pool2d::Pool2d(Graph* graph, PoolType type, const std::array<uint32_t, 2>& input_size, RoundType round_type,
               DataLayout layout)
    : BuiltinOp(graph, B2VX_NODE_POOL2D, 1, 1, layout),
      type_(type), padding_(PadType::AUTO), ksize_(input_size), stride_(input_size), round_type_(round_type),
      pad_({0, 0, 0, 0}) {
  Init();
}

Pool2d::Pool2d(Graph* graph, PoolType type, const std::array<uint32_t, 2>& input_size,
               const std::array<uint32_t, 2>& output_size, RoundType round_type, DataLayout layout)
    : BuiltinOp(graph, B2VX_NODE_POOL2D, 1, 1, layout),
      type_(type), padding_(PadType::AUTO), round_type_(round_type), pad_({0, 0, 0, 0}) {
  for (int i = 0; i < 2; ++i) {
    stride_[i] = static_cast<uint32_t>(std::floor(input_size[i] / static_cast<float>(output_size[i])));
    ksize_[i] = input_size[i] - (output_size[i] - 1) * stride_[i];
  }
  Init();
}

void Pool2d::Init() {
  impl_->foreign_layout_ = impl_->layout_ != DataLayout::WHCN && impl_->layout_ != DataLayout::ANY;
  b2vx_pool2d_desc& d = impl_->desc_.pool2d;
  d.type = static_cast<int32_t>(type_);
  d.pad_type = static_cast<int32_t>(padding_);
  d.round_type = static_cast<int32_t>(round_type_);
  for (int i = 0; i < 2; ++i) {
    d.ksize[i] = ksize_[i];
    d.stride[i] = stride_[i];
  }
  for (int i = 0; i < 4; ++i) d.pad[i] = pad_[i];
}

std::shared_ptr<Operation> Pool2d::Clone(std::shared_ptr<Graph>& graph) const {
  if (padding_ != PadType::AUTO) return graph->CreateOperation<Pool2d>(type_, padding_, ksize_, stride_, round_type_, impl_->layout_);
  return graph->CreateOperation<Pool2d>(type_, pad_, ksize_, stride_, round_type_, impl_->layout_);
}

// ---- declared-only ops (see the headers): one- and two-input families, then the three the reference's
// layout inference tests build
#define B2VX_DECLARED_ONLY_OP(NAME, INPUTS)                                                          \
  NAME::NAME(Graph* graph) : BuiltinOp(graph, kNodeKindDeclaredOnly, INPUTS, 1) { impl_->name_ = #NAME; } \
  std::shared_ptr<Operation> NAME::Clone(std::shared_ptr<Graph>& graph) const { return graph->CreateOperation<NAME>(); }
B2VX_DECLARED_ONLY_OP(Neg, 1)
B2VX_DECLARED_ONLY_OP(Abs, 1)
B2VX_DECLARED_ONLY_OP(Sin, 1)
B2VX_DECLARED_ONLY_OP(Exp, 1)
B2VX_DECLARED_ONLY_OP(Log, 1)
B2VX_DECLARED_ONLY_OP(Sqrt, 1)
B2VX_DECLARED_ONLY_OP(Rsqrt, 1)
B2VX_DECLARED_ONLY_OP(Square, 1)
B2VX_DECLARED_ONLY_OP(LogicalNot, 1)
B2VX_DECLARED_ONLY_OP(Floor, 1)
B2VX_DECLARED_ONLY_OP(Ceil, 1)
B2VX_DECLARED_ONLY_OP(Round, 1)
B2VX_DECLARED_ONLY_OP(Cast, 1)
B2VX_DECLARED_ONLY_OP(Rcp, 1)
B2VX_DECLARED_ONLY_OP(Cos, 1)
B2VX_DECLARED_ONLY_OP(Tan, 1)
B2VX_DECLARED_ONLY_OP(ATan, 1)
B2VX_DECLARED_ONLY_OP(ATanh, 1)
B2VX_DECLARED_ONLY_OP(ACosh, 1)
B2VX_DECLARED_ONLY_OP(Greater, 2)
B2VX_DECLARED_ONLY_OP(GreaterOrEqual, 2)
B2VX_DECLARED_ONLY_OP(Less, 2)
B2VX_DECLARED_ONLY_OP(LessOrEqual, 2)
B2VX_DECLARED_ONLY_OP(NotEqual, 2)
B2VX_DECLARED_ONLY_OP(Equal, 2)
#undef B2VX_DECLARED_ONLY_OP

InstanceNormalization::InstanceNormalization(Graph* graph, float eps, DataLayout input_layout)
    : BuiltinOp(graph, kNodeKindDeclaredOnly, 3, 1, input_layout), eps_(eps) { impl_->name_ = "InstanceNormalization"; }
std::shared_ptr<Operation> InstanceNormalization::Clone(std::shared_ptr<Graph>& graph) const {
  return graph->CreateOperation<InstanceNormalization>(eps_, impl_->layout_);
}

Resize::Resize(Graph* graph, ResizeType type, float factor, bool align_corners, bool half_pixel_centers, int target_height,
               int target_width, DataLayout layout)
    : BuiltinOp(graph, kNodeKindDeclaredOnly, 1, 1, layout), type_(type), factor_(factor), align_corners_(align_corners),
      half_pixel_centers_(half_pixel_centers), target_height_(target_height), target_width_(target_width) { impl_->name_ = "Resize"; }
std::shared_ptr<Operation> Resize::Clone(std::shared_ptr<Graph>& graph) const {
  return graph->CreateOperation<Resize>(type_, factor_, align_corners_, half_pixel_centers_, target_height_, target_width_, impl_->layout_);
}

RoiAlign::RoiAlign(Graph* graph, int32_t output_height, int32_t output_width, float height_ratio, float width_ratio,
                   int32_t height_sample_num, int32_t width_sample_num, DataLayout input_layout)
    : BuiltinOp(graph, kNodeKindDeclaredOnly, 3, 1, input_layout), output_height_(output_height), output_width_(output_width),
      height_ratio_(height_ratio), width_ratio_(width_ratio), height_sample_num_(height_sample_num),
      width_sample_num_(width_sample_num) { impl_->name_ = "RoiAlign"; }
std::shared_ptr<Operation> RoiAlign::Clone(std::shared_ptr<Graph>& graph) const {
  return graph->CreateOperation<RoiAlign>(output_height_, output_width_, height_ratio_, width_ratio_, height_sample_num_,
                                          width_sample_num_, impl_->layout_);
}

AddN::AddN(Graph* graph, uint32_t num_inputs) : BuiltinOp(graph, B2VX_NODE_ADDN, static_cast<int>(num_inputs), 1) {}
std::shared_ptr<Operation> AddN::Clone(std::shared_ptr<Graph>& graph) const {
  return graph->CreateOperation<AddN>(static_cast<uint32_t>(impl_->input_cnt_));
}

Add::Add(Graph* graph) : BuiltinOp(graph, B2VX_NODE_ADD, 2, 1) {}
std::shared_ptr<Operation> Add::Clone(std::shared_ptr<Graph>& graph) const { return graph->CreateOperation<Add>(); }

Relu::Relu(Graph* graph) : BuiltinOp(graph, B2VX_NODE_RELU, 1, 1) {}
std::shared_ptr<Operation> Relu::Clone(std::shared_ptr<Graph>& graph) const { return graph->CreateOperation<Relu>(); }

NBG::NBG(Graph* graph, const char* binary, size_t input_count, size_t output_count)
    : BuiltinOp(graph, kNodeKindNbg, static_cast<int>(input_count), static_cast<int>(output_count)) {
  // the blob states its own length in its header (the reference's constructor takes no size either)
  // and nothing of it is trusted before the first eight bytes say it is a blob of this backend and this version:
  // a vendor-format NBG file, which the reference's API takes here, leaves the op empty and Compile fails cleanly
  uint32_t magic = 0, version = 0;
  uint64_t total = 0;
  if (binary) {
    std::memcpy(&magic, binary, sizeof(magic));
    std::memcpy(&version, binary + 4, sizeof(version));
  }
  if (binary && magic == kBlobMagic && version == kBlobVersion) std::memcpy(&total, binary + 8, sizeof(total));
  if (total >= 32 && total < (1ull << 40)) impl_->blob_.assign(binary, binary + total);
}
std::shared_ptr<Operation> NBG::Clone(std::shared_ptr<Graph>& graph) const {
  return graph->CreateOperation<NBG>(reinterpret_cast<const char*>(impl_->blob_.data()), impl_->input_cnt_, impl_->output_cnt_);
}

Reshape::Reshape(Graph* graph, const std::vector<uint32_t>& target_shape)
    : BuiltinOp(graph, B2VX_NODE_RESHAPE, 1, 1), size_(target_shape) {
  b2vx_dims_desc& d = impl_->desc_.dims;
  d.rank = static_cast<uint32_t>(target_shape.size() <= B2VX_MAX_RANK ? target_shape.size() : 0);   // rank 0 is refused when the node is added
  for (uint32_t i = 0; i < d.rank; ++i) d.v[i] = target_shape[i];
}
std::shared_ptr<Operation> Reshape::Clone(std::shared_ptr<Graph>& graph) const { return graph->CreateOperation<Reshape>(size_); }

Transpose::Transpose(Graph* graph, const std::vector<uint32_t>& perm) : BuiltinOp(graph, B2VX_NODE_TRANSPOSE, 1, 1), perm_(perm) {
  b2vx_dims_desc& d = impl_->desc_.dims;
  d.rank = static_cast<uint32_t>(perm.size() <= B2VX_MAX_RANK ? perm.size() : 0);
  for (uint32_t i = 0; i < d.rank; ++i) d.v[i] = perm[i];
}
std::shared_ptr<Operation> Transpose::Clone(std::shared_ptr<Graph>& graph) const { return graph->CreateOperation<Transpose>(perm_); }

Concat::Concat(Graph* graph, uint32_t axis, int input_cnt) : BuiltinOp(graph, B2VX_NODE_CONCAT, input_cnt, 1), axis_(axis) {
  impl_->desc_.concat_axis = axis;
}
std::shared_ptr<Operation> Concat::Clone(std::shared_ptr<Graph>& graph) const {
  return graph->CreateOperation<Concat>(axis_, impl_->input_cnt_);
}

DataConvert::DataConvert(Graph* graph) : BuiltinOp(graph, B2VX_NODE_DATACONVERT, 1, 1) {}
std::shared_ptr<Operation> DataConvert::Clone(std::shared_ptr<Graph>& graph) const { return graph->CreateOperation<DataConvert>(); }

Relu6::Relu6(Graph* graph) : BuiltinOp(graph, B2VX_NODE_RELU6, 1, 1) {}
std::shared_ptr<Operation> Relu6::Clone(std::shared_ptr<Graph>& graph) const { return graph->CreateOperation<Relu6>(); }

Softmax::Softmax(Graph* graph, float beta, int32_t axis)
    : BuiltinOp(graph, B2VX_NODE_SOFTMAX, 1, 1), beta_(beta), axis_(axis) {
  impl_->desc_.softmax.beta = beta;
  impl_->desc_.softmax.axis = axis;
}
std::shared_ptr<Operation> Softmax::Clone(std::shared_ptr<Graph>& graph) const {
  return graph->CreateOperation<Softmax>(beta_, axis_);
}

}  // namespace ops
}  // namespace vx
}  // namespace tim

// The b2vx_graph behind a tim::vx::Graph, for tools that read back the launch
// plan or time it (creates the backend graph if it does not exist yet).
extern "C" void* timvx_graph_backend_handle(tim::vx::Graph* graph) {
  auto* impl = static_cast<tim::vx::GraphImpl*>(graph);
  if (!impl || !impl->EnsureHandle()) return nullptr;
  return impl->handle();
}
