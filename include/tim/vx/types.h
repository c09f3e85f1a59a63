// tim::vx enumerations used by the quantized-inference path.
// Restates include/tim/vx/types.h:30-88 of the reference: enumerator names and
// numeric values are part of the drop-in surface (user code passes them by
// name, the C ABI in b2vx.h receives them by value).
#ifndef TIM_VX_TYPES_H_
#define TIM_VX_TYPES_H_

namespace tim {
namespace vx {

enum class DataType {
  UNKNOWN, INT8, UINT8, INT16, UINT16, INT32, UINT32, INT64,
  FLOAT16, FLOAT32, BOOL8, INT4, UINT4
};

enum class QuantType {
  NONE, ASYMMETRIC, SYMMETRIC_PER_CHANNEL, ASYMMETRIC_PER_CHANNEL,
  DYNAMIC_FIXED_POINT
};

enum TensorAttribute {
  CONSTANT = 1 << 0,
  TRANSIENT = 1 << 1,
  VARIABLE = 1 << 2,
  INPUT = 1 << 3,
  OUTPUT = 1 << 4
};

enum class PadType { NONE = -1, AUTO, VALID, SAME };
enum class PoolType { MAX, AVG, L2, AVG_ANDROID };
enum class RoundType { CEILING, FLOOR };
enum class OverflowPolicy { WRAP, SATURATE };
enum class RoundingPolicy { TO_ZERO, RTNE };
enum class ResizeType { NEAREST_NEIGHBOR, BILINEAR, AREA };

// Only WHCN activations and WHIcOc kernels are executed by this backend; the
// other enumerators exist so that user code naming them still compiles.
enum class DataLayout {
  ANY, WHCN, CWHN, IcWHOc, OcIcWH, IcOcWH, WHIcOc, WCN, WIcOc,
  WHDCN, WHDIcOc, CWHDN, OcIcWHD
};

}  // namespace vx
}  // namespace tim
#endif  // TIM_VX_TYPES_H_
