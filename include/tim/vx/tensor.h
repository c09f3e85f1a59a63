// tim::vx::Quantization / TensorSpec / Tensor.
// Restates the public surface of include/tim/vx/tensor.h:40-175 of the
// reference.  Shapes are listed fastest dimension first (W,H,C,N).
#ifndef TIM_VX_TENSOR_H_
#define TIM_VX_TENSOR_H_

#include <cstdint>
#include <iostream>
#include <memory>
#include <string>
#include <vector>

#include "tim/vx/types.h"

namespace tim {
namespace vx {

using ShapeType = std::vector<uint32_t>;

// Quantization parameters of one tensor.  Per-tensor forms keep one scale and
// one zero point; the per-channel form keeps one pair per slice along
// channel_dim.  The reference's own tests build ASYMMETRIC parameters through
// the four-argument constructor with one-element vectors
// (src/tim/vx/ops/conv2d_test.cc:1012-1019), which must keep working.
class Quantization {
 public:
  Quantization() : type_(QuantType::NONE) {}
  Quantization(QuantType type, float scale, int32_t zero_point)
      : type_(type), scales_({scale}), zero_points_({zero_point}) {}
  Quantization(QuantType type, int32_t channel_dim, std::vector<float> scales,
               std::vector<int32_t> zero_points)
      : type_(type),
        channel_dim_(channel_dim),
        scales_(std::move(scales)),
        zero_points_(std::move(zero_points)) {}
  Quantization(QuantType type, int8_t fl) : type_(type), fl_(fl) {}

  QuantType& Type() { return type_; }
  const QuantType& Type() const { return type_; }
  Quantization& SetType(QuantType type) { type_ = type; return *this; }

  int32_t& ChannelDim() { return channel_dim_; }
  const int32_t& ChannelDim() const { return channel_dim_; }
  Quantization& SetChannelDim(int32_t dim) { channel_dim_ = dim; return *this; }

  std::vector<float>& Scales() { return scales_; }
  const std::vector<float>& Scales() const { return scales_; }
  Quantization& SetScales(std::vector<float> scales) { scales_ = scales; return *this; }

  std::vector<int32_t>& ZeroPoints() { return zero_points_; }
  const std::vector<int32_t>& ZeroPoints() const { return zero_points_; }
  Quantization& SetZeroPoints(std::vector<int32_t> zps) { zero_points_ = zps; return *this; }

  const std::int8_t& Fl() const { return fl_; }

  bool operator==(const Quantization& other) const;

 protected:
  QuantType type_{QuantType::NONE};
  int32_t channel_dim_{-1};
  std::vector<float> scales_;
  std::vector<int32_t> zero_points_;
  int8_t fl_ = 0;
};

struct TensorSpec {
  TensorSpec() {}
  TensorSpec(DataType datatype, const ShapeType& shape, TensorAttribute attr)
      : datatype_(datatype), shape_(shape), attr_(attr) {}
  TensorSpec(DataType datatype, const ShapeType& shape, TensorAttribute attr,
             const Quantization& quantization)
      : TensorSpec(datatype, shape, attr) {
    quantization_ = quantization;
  }
  TensorSpec(const TensorSpec& other);
  TensorSpec& operator=(const TensorSpec& other);
  bool operator==(const TensorSpec& other) const;

  TensorSpec& SetDataType(DataType datatype);
  TensorSpec& SetShape(const ShapeType& shape);
  TensorSpec& SetAttribute(TensorAttribute attr);
  TensorSpec& SetQuantization(Quantization& quantization);
  TensorSpec AsTransientSpec() const;

  int64_t GetElementNum() const;
  int64_t GetElementByteSize() const;
  int64_t GetByteSize() const;

  inline DataType& GetDataType() { return datatype_; }
  inline ShapeType& GetShapeType() { return shape_; }
  inline TensorAttribute& GetTensorAttribute() { return attr_; }
  inline Quantization& GetQuantization() { return quantization_; }

  DataType datatype_{DataType::UNKNOWN};
  ShapeType shape_;
  TensorAttribute attr_{TensorAttribute::TRANSIENT};
  Quantization quantization_;
};

struct DmaBufferDesc {
  int64_t fd;
};

class Tensor {
 public:
  virtual ~Tensor() {}
  virtual const ShapeType& GetShape() = 0;
  virtual DataType GetDataType() = 0;
  virtual const Quantization& GetQuantization() = 0;
  virtual TensorSpec& GetSpec() = 0;
  virtual uint32_t GetId() = 0;
  // Host -> tensor.  As in the reference (src/tim/vx/tensor.cc:154-166) the
  // size argument is advisory: the whole tensor is always copied.
  virtual bool CopyDataToTensor(const void* data, uint32_t size_in_bytes = 0) = 0;
  virtual bool CopyDataFromTensor(void* data) = 0;
  virtual bool SwapHandle(void* new_ptr, bool is_new_ptr_malloc_by_ovxlib,
                          void** old_ptr) = 0;
  virtual bool SwapHandle(std::shared_ptr<tim::vx::Tensor> tensor) = 0;
  virtual bool SwapHandleWithCache(std::shared_ptr<tim::vx::Tensor> tensor) = 0;
  virtual bool FlushCacheForHandle() = 0;
  virtual bool InvalidateCacheForHandle() = 0;
  virtual void* map(bool invalidate_cpu_cache = false) = 0;
  virtual void unmap() = 0;
  virtual bool IsPlaceHolder() = 0;
  virtual bool IsConstTensor() = 0;
  virtual bool IsScalar() = 0;
  virtual bool SaveTensorToTextByFp32(std::string filename) = 0;
  virtual void SetScalar(int8_t is_scalar) = 0;
  virtual void* ConvertTensorToData(uint8_t* tensorData) = 0;
  virtual float* ConvertTensorToFloat32Data() = 0;
};

namespace utils {
bool Float32ToDtype(std::shared_ptr<tim::vx::Tensor> tensor,
                    std::vector<float> fval, uint8_t* tensorData);
bool DtypeToFloat32(std::shared_ptr<tim::vx::Tensor> tensor,
                    uint8_t* tensorData, float* data);
}  // namespace utils

}  // namespace vx
}  // namespace tim
#endif  // TIM_VX_TENSOR_H_
