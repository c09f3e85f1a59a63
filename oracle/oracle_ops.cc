// CPU oracle — TEST INFRASTRUCTURE ONLY (see oracle_ops.h for scope, sources
// and parity status).  Plain loops, int32 accumulation, and the reference's
// float requantization sequence replayed operation for operation.  Build with
// -ffp-contract=off so no multiply-add is fused.
#include "oracle_ops.h"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <limits>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

enum { DT_INT8 = 1, DT_UINT8 = 2, DT_INT32 = 5, DT_FLOAT32 = 9 };

inline bool is_quant_dtype(int32_t dt) { return dt == DT_INT8 || dt == DT_UINT8; }

// type_get_range (src/tim/vx/internal/include/utils/vsi_nn_dtype_util_prv.h:170-207)
inline void dtype_range(int32_t dt, int32_t* lo, int32_t* hi) {
  switch (dt) {
    case DT_INT8: *lo = -128; *hi = 127; break;
    case DT_UINT8: *lo = 0; *hi = 255; break;
    default: *lo = std::numeric_limits<int32_t>::min(); *hi = std::numeric_limits<int32_t>::max(); break;
  }
}

inline int32_t load_q(const void* p, int32_t dt, size_t i) {
  return dt == DT_UINT8 ? static_cast<int32_t>(static_cast<const uint8_t*>(p)[i])
                        : static_cast<int32_t>(static_cast<const int8_t*>(p)[i]);
}

inline void store_q(void* p, int32_t dt, size_t i, int32_t v) {
  if (dt == DT_UINT8) static_cast<uint8_t*>(p)[i] = static_cast<uint8_t>(v);
  else if (dt == DT_INT8) static_cast<int8_t*>(p)[i] = static_cast<int8_t>(v);
  else static_cast<int32_t*>(p)[i] = v;
}

inline float q_scale(const orc_quant& q, uint32_t c) { return q.per_channel ? q.scales[c] : q.scale; }
inline int32_t q_zp(const orc_quant& q, uint32_t c) {
  return q.per_channel ? (q.zps ? q.zps[c] : 0) : q.zp;
}

// simple_round (src/tim/vx/internal/include/utils/vsi_nn_math.h:183-189): the
// add and the floor are done in float, as there.
inline float simple_round(float x) {
  float r = floorf(fabsf(x) + 0.5f);
  return std::signbit(x) ? -r : r;
}

}  // namespace

extern "C" {

// vsi_rint (src/tim/vx/internal/include/utils/vsi_nn_math.h:191-210): ties (to
// within 1e-8) go to the even integer, everything else through simple_round.
double orc_rint(double x) {
  double inter;
  double decimal = std::modf(x, &inter);
  if (std::fabs(std::fabs(decimal) - 0.5) < 1e-8) {
    inter += static_cast<double>(static_cast<int32_t>(inter) % 2);
    return inter;
  }
  return static_cast<double>(simple_round(static_cast<float>(x)));
}

// fp32_to_affine (src/tim/vx/internal/include/utils/vsi_nn_dtype_util_prv.h:228-254).
// One deliberate difference: the double -> int32 conversion saturates, where
// the reference's C cast is undefined beyond +-2^31 (x86 yields INT_MIN, which
// would clamp a huge positive value to the type's minimum).
int32_t orc_fp32_to_affine(float in, float scale, int32_t zero_point, int32_t dtype) {
  int32_t lo, hi;
  dtype_range(dtype, &lo, &hi);
  if (std::isinf(in)) return std::signbit(in) ? lo : hi;
  double v = orc_rint(static_cast<double>(in / scale)) + static_cast<double>(zero_point);
  int32_t data;
  if (!(v == v)) data = 0;
  else if (v >= 2147483647.0) data = std::numeric_limits<int32_t>::max();
  else if (v <= -2147483648.0) data = std::numeric_limits<int32_t>::min();
  else data = static_cast<int32_t>(v);
  return std::max(lo, std::min(hi, data));
}

// affine_to_fp32 (vsi_nn_dtype_util_prv.h:256-266)
float orc_affine_to_fp32(int32_t val, float scale, int32_t zero_point) {
  return (static_cast<float>(val) - static_cast<float>(zero_point)) * scale;
}

// vsi_nn_ComputeFilterSize (src/tim/vx/internal/src/utils/vsi_nn_util.c:483-511)
uint32_t orc_filter_size(uint32_t in, uint32_t ksize, uint32_t pad0, uint32_t pad1, uint32_t stride,
                         uint32_t dilation, int32_t round_type) {
  if (stride == 0) {
    if (in == ksize) stride = 1;
    else return 0;
  }
  if (dilation > 1) ksize = dilation * (ksize - 1) + 1;
  int64_t span = static_cast<int64_t>(in) + pad0 + pad1 - ksize;
  if (span < 0) return 0;
  uint32_t out = round_type == 0 /* CEILING */ ? static_cast<uint32_t>((span + stride - 1) / stride)
                                               : static_cast<uint32_t>(span / stride);
  return out + 1;
}

// vsi_nn_compute_padding_per_axis (vsi_nn_util.c:535-553): SAME gives
// out = ceil(in/stride) and splits the total padding front = total/2,
// end = total - front; VALID gives no padding.
void orc_same_valid_padding(uint32_t in, uint32_t ksize, uint32_t stride, uint32_t dilation,
                            int32_t pad_type, uint32_t out_pad[2]) {
  if (dilation == 0) dilation = 1;
  if (stride == 0) stride = 1;
  int64_t eff = static_cast<int64_t>(ksize - 1) * dilation + 1;
  int64_t out;
  if (pad_type == 2 /* SAME */) out = (static_cast<int64_t>(in) + stride - 1) / stride;
  else out = (static_cast<int64_t>(in) + stride - eff) / stride;
  int64_t total = (out - 1) * stride + eff - in;
  if (total < 0) total = 0;
  out_pad[0] = static_cast<uint32_t>(total / 2);
  out_pad[1] = static_cast<uint32_t>(total - total / 2);
}

int32_t orc_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

}  // extern "C"

namespace {

// One output plane [Ho][Wo] of a convolution, accumulated tap by tap so the
// inner loop runs along W.  Taps that fall into the padding contribute
// nothing: padding is zero in the real domain, i.e. x == zero point.
// Accumulation order per output element: ic (outer), ky, kx (inner); the
// float path depends on that order, the integer path does not.
template <typename XT, typename WT, typename AccT>
void conv_plane(const orc_conv2d_args& a, uint32_t n, uint32_t oc, uint32_t ic_begin, uint32_t ic_end,
                uint32_t w_ch_for_ic0, bool depthwise, AccT zx, AccT zw, AccT* acc) {
  const XT* x = static_cast<const XT*>(a.x);
  const WT* w = static_cast<const WT*>(a.w);
  const uint32_t dx = a.dilation[0] ? a.dilation[0] : 1, dy = a.dilation[1] ? a.dilation[1] : 1;
  const uint32_t sx = a.stride[0], sy = a.stride[1];
  for (uint32_t ic = ic_begin; ic < ic_end; ++ic) {
    // dense: weight [kx,ky,ic,oc]; depthwise: weight [kx,ky,oc,0]
    const size_t wbase = depthwise ? static_cast<size_t>(oc) * a.kh * a.kw
                                   : (static_cast<size_t>(oc) * a.w_ic + (ic - ic_begin + w_ch_for_ic0)) * a.kh * a.kw;
    const XT* xin = x + (static_cast<size_t>(n) * a.C + ic) * a.H * a.W;
    for (uint32_t ky = 0; ky < a.kh; ++ky) {
      for (uint32_t kx = 0; kx < a.kw; ++kx) {
        const AccT wv = static_cast<AccT>(w[wbase + ky * a.kw + kx]) - zw;
        // wo range with 0 <= wo*sx - pad_left + kx*dx < W
        int64_t off = static_cast<int64_t>(kx) * dx - a.pad_left;
        int64_t wo_lo = off >= 0 ? 0 : (-off + sx - 1) / sx;
        int64_t wo_hi = (static_cast<int64_t>(a.W) - 1 - off) / sx;  // inclusive
        if (static_cast<int64_t>(a.W) - 1 - off < 0) continue;
        wo_hi = std::min<int64_t>(wo_hi, static_cast<int64_t>(a.Wo) - 1);
        for (uint32_t ho = 0; ho < a.Ho; ++ho) {
          int64_t hi = static_cast<int64_t>(ho) * sy - a.pad_top + static_cast<int64_t>(ky) * dy;
          if (hi < 0 || hi >= static_cast<int64_t>(a.H)) continue;
          const XT* row = xin + hi * a.W + off;
          AccT* arow = acc + static_cast<size_t>(ho) * a.Wo;
          if (sx == 1) {
            for (int64_t wo = wo_lo; wo <= wo_hi; ++wo) arow[wo] += (static_cast<AccT>(row[wo]) - zx) * wv;
          } else {
            for (int64_t wo = wo_lo; wo <= wo_hi; ++wo) arow[wo] += (static_cast<AccT>(row[wo * sx]) - zx) * wv;
          }
        }
      }
    }
  }
}

template <typename XT, typename WT>
int32_t conv2d_quant(const orc_conv2d_args& a) {
  const bool depthwise = a.multiplier >= 1;
  const int32_t* bias = static_cast<const int32_t*>(a.bias);
  const size_t plane = static_cast<size_t>(a.Wo) * a.Ho;
  const int64_t jobs = static_cast<int64_t>(a.N) * a.Oc;
#pragma omp parallel
  {
    std::vector<int32_t> acc(plane);
#pragma omp for schedule(dynamic, 1)
    for (int64_t job = 0; job < jobs; ++job) {
      const uint32_t n = static_cast<uint32_t>(job / a.Oc), oc = static_cast<uint32_t>(job % a.Oc);
      std::fill(acc.begin(), acc.end(), 0);
      const int32_t zx = a.xq.zp, zw = q_zp(a.wq, oc);
      if (depthwise) {
        const uint32_t ic = oc / static_cast<uint32_t>(a.multiplier);
        conv_plane<XT, WT, int32_t>(a, n, oc, ic, ic + 1, 0, true, zx, zw, acc.data());
      } else if (a.group > 1) {
        // grouped (vsi_nn_op_grouped_conv2d.c): output block g reads input block g
        const uint32_t per_in = a.C / static_cast<uint32_t>(a.group), per_out = a.Oc / static_cast<uint32_t>(a.group);
        const uint32_t gi = oc / per_out;
        conv_plane<XT, WT, int32_t>(a, n, oc, gi * per_in, (gi + 1) * per_in, 0, false, zx, zw, acc.data());
      } else {
        conv_plane<XT, WT, int32_t>(a, n, oc, 0, a.C, 0, false, zx, zw, acc.data());
      }
      // The accumulator is a quantized value with scale s_x*s_w[oc] and zero
      // point 0 (the bias quantization): affine_to_fp32 then fp32_to_affine.
      const float acc_scale = a.xq.scale * q_scale(a.wq, oc);
      const size_t obase = (static_cast<size_t>(n) * a.Oc + oc) * plane;
      for (size_t i = 0; i < plane; ++i) {
        int32_t v = acc[i] + (bias ? bias[oc] : 0);
        if (a.acc_out) a.acc_out[obase + i] = v;
        float real = orc_affine_to_fp32(v, acc_scale, 0);
        if (a.y_dtype == DT_FLOAT32) static_cast<float*>(a.y)[obase + i] = real;
        else store_q(a.y, a.y_dtype, obase + i, orc_fp32_to_affine(real, a.yq.scale, a.yq.zp, a.y_dtype));
      }
    }
  }
  return 0;
}

int32_t conv2d_float(const orc_conv2d_args& a) {
  const bool depthwise = a.multiplier >= 1;
  const float* bias = static_cast<const float*>(a.bias);
  const size_t plane = static_cast<size_t>(a.Wo) * a.Ho;
  const int64_t jobs = static_cast<int64_t>(a.N) * a.Oc;
#pragma omp parallel
  {
    std::vector<float> acc(plane);
#pragma omp for schedule(dynamic, 1)
    for (int64_t job = 0; job < jobs; ++job) {
      const uint32_t n = static_cast<uint32_t>(job / a.Oc), oc = static_cast<uint32_t>(job % a.Oc);
      std::fill(acc.begin(), acc.end(), 0.0f);
      if (depthwise) {
        const uint32_t ic = oc / static_cast<uint32_t>(a.multiplier);
        conv_plane<float, float, float>(a, n, oc, ic, ic + 1, 0, true, 0.0f, 0.0f, acc.data());
      } else if (a.group > 1) {
        const uint32_t per_in = a.C / static_cast<uint32_t>(a.group), per_out = a.Oc / static_cast<uint32_t>(a.group);
        const uint32_t gi = oc / per_out;
        conv_plane<float, float, float>(a, n, oc, gi * per_in, (gi + 1) * per_in, 0, false, 0.0f, 0.0f, acc.data());
      } else {
        conv_plane<float, float, float>(a, n, oc, 0, a.C, 0, false, 0.0f, 0.0f, acc.data());
      }
      const size_t obase = (static_cast<size_t>(n) * a.Oc + oc) * plane;
      float* y = static_cast<float*>(a.y);
      for (size_t i = 0; i < plane; ++i) y[obase + i] = acc[i] + (bias ? bias[oc] : 0.0f);
    }
  }
  return 0;
}

}  // namespace

extern "C" {

int32_t orc_conv2d(const orc_conv2d_args* a) {
  if (a->x_dtype == DT_FLOAT32) {
    if (a->w_dtype != DT_FLOAT32 || a->y_dtype != DT_FLOAT32) return -1;
    return conv2d_float(*a);
  }
  if (!is_quant_dtype(a->x_dtype) || !is_quant_dtype(a->w_dtype)) return -1;
  if (!is_quant_dtype(a->y_dtype) && a->y_dtype != DT_FLOAT32) return -1;
  if (a->x_dtype == DT_UINT8 && a->w_dtype == DT_UINT8) return conv2d_quant<uint8_t, uint8_t>(*a);
  if (a->x_dtype == DT_UINT8 && a->w_dtype == DT_INT8) return conv2d_quant<uint8_t, int8_t>(*a);
  if (a->x_dtype == DT_INT8 && a->w_dtype == DT_INT8) return conv2d_quant<int8_t, int8_t>(*a);
  return conv2d_quant<int8_t, uint8_t>(*a);
}

// vxFullyConnectedLayer (prebuilt-sdk/x86_64_linux/include/VX/vx_khr_nn.h:875-915)
// on the 2-D operands the reference's op_compute builds
// (src/tim/vx/internal/src/ops/vsi_nn_op_fullconnect2.c:45-138).
int32_t orc_fully_connected(const orc_fc_args* a) {
  if (a->x_dtype == DT_FLOAT32) {
    if (a->w_dtype != DT_FLOAT32 || a->y_dtype != DT_FLOAT32) return -1;
    const float* x = static_cast<const float*>(a->x);
    const float* w = static_cast<const float*>(a->w);
    const float* bias = static_cast<const float*>(a->bias);
    float* y = static_cast<float*>(a->y);
#pragma omp parallel for collapse(2)
    for (uint32_t b = 0; b < a->batch; ++b) {
      for (uint32_t n = 0; n < a->N; ++n) {
        float acc = 0.0f;
        for (uint32_t k = 0; k < a->K; ++k) acc += x[static_cast<size_t>(b) * a->K + k] * w[static_cast<size_t>(n) * a->K + k];
        y[static_cast<size_t>(b) * a->N + n] = acc + (bias ? bias[n] : 0.0f);
      }
    }
    return 0;
  }
  if (!is_quant_dtype(a->x_dtype) || !is_quant_dtype(a->w_dtype)) return -1;
  const int32_t* bias = static_cast<const int32_t*>(a->bias);
#pragma omp parallel for collapse(2)
  for (uint32_t b = 0; b < a->batch; ++b) {
    for (uint32_t n = 0; n < a->N; ++n) {
      const int32_t zx = a->xq.zp, zw = q_zp(a->wq, n);
      int32_t acc = 0;
      const size_t xb = static_cast<size_t>(b) * a->K, wb = static_cast<size_t>(n) * a->K;
      if (a->x_dtype == DT_UINT8 && a->w_dtype == DT_INT8) {
        const uint8_t* x = static_cast<const uint8_t*>(a->x) + xb;
        const int8_t* w = static_cast<const int8_t*>(a->w) + wb;
        for (uint32_t k = 0; k < a->K; ++k) acc += (static_cast<int32_t>(x[k]) - zx) * (static_cast<int32_t>(w[k]) - zw);
      } else if (a->x_dtype == DT_UINT8 && a->w_dtype == DT_UINT8) {
        const uint8_t* x = static_cast<const uint8_t*>(a->x) + xb;
        const uint8_t* w = static_cast<const uint8_t*>(a->w) + wb;
        for (uint32_t k = 0; k < a->K; ++k) acc += (static_cast<int32_t>(x[k]) - zx) * (static_cast<int32_t>(w[k]) - zw);
      } else {
        for (uint32_t k = 0; k < a->K; ++k)
          acc += (load_q(a->x, a->x_dtype, xb + k) - zx) * (load_q(a->w, a->w_dtype, wb + k) - zw);
      }
      acc += bias ? bias[n] : 0;
      const size_t o = static_cast<size_t>(b) * a->N + n;
      if (a->acc_out) a->acc_out[o] = acc;
      float real = orc_affine_to_fp32(acc, a->xq.scale * q_scale(a->wq, n), 0);
      if (a->y_dtype == DT_FLOAT32) static_cast<float*>(a->y)[o] = real;
      else store_q(a->y, a->y_dtype, o, orc_fp32_to_affine(real, a->yq.scale, a->yq.zp, a->y_dtype));
    }
  }
  return 0;
}

// vxPoolingLayer2 (vx_khr_nn.h:1693-1744).  MAX looks at in-bounds taps only.
// AVG divides by kw*kh (padding counts as real zero); AVG_ANDROID divides by
// the in-bounds tap count — the distinction the reference's float tests make
// (src/tim/vx/ops/avg_pool_test.cc:404-579).  Quantized averages sum (q - zp)
// in int32 and convert once: avg = (sum * s_in) / divisor in float.
int32_t orc_pool2d(const orc_pool2d_args* a) {
  const bool is_float = a->dtype == DT_FLOAT32;
  if (!is_float && !is_quant_dtype(a->dtype)) return -1;
  if (a->type < 0 || a->type > 3) return -1;
  const bool same_quant = is_float || (a->xq.scale == a->yq.scale && a->xq.zp == a->yq.zp);
  const int64_t planes = static_cast<int64_t>(a->N) * a->C;
#pragma omp parallel for schedule(static)
  for (int64_t p = 0; p < planes; ++p) {
    const size_t ibase = static_cast<size_t>(p) * a->H * a->W;
    const size_t obase = static_cast<size_t>(p) * a->Ho * a->Wo;
    for (uint32_t ho = 0; ho < a->Ho; ++ho) {
      for (uint32_t wo = 0; wo < a->Wo; ++wo) {
        int32_t count = 0, qsum = 0, qmax = std::numeric_limits<int32_t>::min();
        float fsum = 0.0f, fmax = -std::numeric_limits<float>::infinity(), fsq = 0.0f;
        for (uint32_t ky = 0; ky < a->ksize[1]; ++ky) {
          int64_t hi = static_cast<int64_t>(ho) * a->stride[1] - a->pad_top + ky;
          if (hi < 0 || hi >= static_cast<int64_t>(a->H)) continue;
          for (uint32_t kx = 0; kx < a->ksize[0]; ++kx) {
            int64_t wi = static_cast<int64_t>(wo) * a->stride[0] - a->pad_left + kx;
            if (wi < 0 || wi >= static_cast<int64_t>(a->W)) continue;
            const size_t idx = ibase + hi * a->W + wi;
            ++count;
            if (is_float) {
              float v = static_cast<const float*>(a->x)[idx];
              fsum += v;
              fmax = std::max(fmax, v);
              const float sq = v * v;
              fsq = fsq + sq;
            } else {
              int32_t v = load_q(a->x, a->dtype, idx);
              qsum += v - a->xq.zp;
              qmax = std::max(qmax, v);
              const float real = orc_affine_to_fp32(v, a->xq.scale, a->xq.zp);
              const float sq = real * real;
              fsq = fsq + sq;
            }
          }
        }
        const size_t o = obase + static_cast<size_t>(ho) * a->Wo + wo;
        const float div = a->type == 1 ? static_cast<float>(a->ksize[0] * a->ksize[1]) : static_cast<float>(count);
        if (a->type == 2) {
          // L2: sqrt(mean of x^2) over the taps inside the input, in float (squares added in tap order).  The
          // reference only lowers the type (src/tim/vx/type_utils.cc:99-100, VX_NN_POOLING_L2); it holds neither a
          // formula nor a vector for it: parity unpinned.
          const float r = count ? std::sqrt(fsq / static_cast<float>(count)) : 0.0f;
          if (is_float) static_cast<float*>(a->y)[o] = r;
          else store_q(a->y, a->dtype, o, orc_fp32_to_affine(r, a->yq.scale, a->yq.zp, a->dtype));
        } else if (is_float) {
          float r = a->type == 0 ? (count ? fmax : 0.0f) : (count ? fsum / div : 0.0f);
          static_cast<float*>(a->y)[o] = r;
        } else if (a->type == 0) {
          int32_t q = count ? qmax : a->xq.zp;
          if (!same_quant)
            q = orc_fp32_to_affine(orc_affine_to_fp32(q, a->xq.scale, a->xq.zp), a->yq.scale, a->yq.zp, a->dtype);
          store_q(a->y, a->dtype, o, q);
        } else {
          float avg = count ? (static_cast<float>(qsum) * a->xq.scale) / div : 0.0f;
          store_q(a->y, a->dtype, o, orc_fp32_to_affine(avg, a->yq.scale, a->yq.zp, a->dtype));
        }
      }
    }
  }
  return 0;
}

// vxTensorAddNode with saturation (prebuilt-sdk/x86_64_linux/include/VX/vx_nodes.h:838-853):
// both operands are taken to real values, summed in float and quantized with
// the output parameters — the convention the reference's visible quantized
// binary kernels use (src/tim/vx/internal/src/libnnext/ops/cl/maximum.cl:50-75).
// Shapes broadcast numpy-style (src/tim/vx/internal/src/ops/vsi_nn_op_eltwise.c:147-214).
int32_t orc_add(const void* a, int32_t a_dtype, const uint32_t* a_dims, orc_quant aq,
                const void* b, int32_t b_dtype, const uint32_t* b_dims, orc_quant bq,
                void* y, int32_t y_dtype, const uint32_t* y_dims, orc_quant yq, uint32_t rank) {
  if (rank > 8) return -1;
  size_t total = 1;
  size_t astride[8], bstride[8];
  size_t as = 1, bs = 1;
  for (uint32_t d = 0; d < rank; ++d) {
    astride[d] = a_dims[d] == 1 && y_dims[d] != 1 ? 0 : as;
    bstride[d] = b_dims[d] == 1 && y_dims[d] != 1 ? 0 : bs;
    as *= a_dims[d];
    bs *= b_dims[d];
    total *= y_dims[d];
  }
  auto to_real = [](const void* p, int32_t dt, size_t i, const orc_quant& q) -> float {
    if (dt == DT_FLOAT32) return static_cast<const float*>(p)[i];
    int32_t v = dt == DT_INT32 ? static_cast<const int32_t*>(p)[i] : load_q(p, dt, i);
    return orc_affine_to_fp32(v, q.scale, q.zp);
  };
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < static_cast<int64_t>(total); ++i) {
    size_t rem = static_cast<size_t>(i), ai = 0, bi = 0;
    for (uint32_t d = 0; d < rank; ++d) {
      size_t c = rem % y_dims[d];
      rem /= y_dims[d];
      ai += c * astride[d];
      bi += c * bstride[d];
    }
    float r = to_real(a, a_dtype, ai, aq) + to_real(b, b_dtype, bi, bq);
    if (y_dtype == DT_FLOAT32) static_cast<float*>(y)[i] = r;
    else store_q(y, y_dtype, static_cast<size_t>(i), orc_fp32_to_affine(r, yq.scale, yq.zp, y_dtype));
  }
  return 0;
}

// ops::AddN (src/tim/vx/internal/src/ops/vsi_nn_op_addn.c:124-205: a chain of n-1 Add nodes): every Add
// dequantizes its inputs and adds them in float; the intermediate sums stay float32 here and only the
// last one is quantized, with the output's parameters.
int32_t orc_addn(const void* const* x, const int32_t* dtypes, const orc_quant* q, uint32_t n,
                 void* y, int32_t y_dtype, orc_quant yq, uint64_t elems) {
  if (n < 2) return -1;
  auto to_real = [](const void* p, int32_t dt, size_t i, const orc_quant& qq) -> float {
    if (dt == DT_FLOAT32) return static_cast<const float*>(p)[i];
    int32_t v = dt == DT_INT32 ? static_cast<const int32_t*>(p)[i] : load_q(p, dt, i);
    return orc_affine_to_fp32(v, qq.scale, qq.zp);
  };
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < static_cast<int64_t>(elems); ++i) {
    float r = to_real(x[0], dtypes[0], static_cast<size_t>(i), q[0]);
    for (uint32_t k = 1; k < n; ++k) r = r + to_real(x[k], dtypes[k], static_cast<size_t>(i), q[k]);
    if (y_dtype == DT_FLOAT32) static_cast<float*>(y)[i] = r;
    else store_q(y, y_dtype, static_cast<size_t>(i), orc_fp32_to_affine(r, yq.scale, yq.zp, y_dtype));
  }
  return 0;
}

// vxActivationLayer RELU / RELU6 (src/tim/vx/internal/src/ops/vsi_nn_op_relu.c:48,
// src/tim/vx/internal/src/kernel/vx/eltwise_unary_vx.c:333-352): clamp in the
// real domain, then quantize with the output parameters.
int32_t orc_relu(const void* x, int32_t x_dtype, orc_quant xq, void* y, int32_t y_dtype, orc_quant yq,
                 uint64_t n, float upper) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < static_cast<int64_t>(n); ++i) {
    float r = x_dtype == DT_FLOAT32 ? static_cast<const float*>(x)[i]
                                    : orc_affine_to_fp32(load_q(x, x_dtype, i), xq.scale, xq.zp);
    r = r < 0.0f ? 0.0f : r;
    if (upper >= 0.0f && r > upper) r = upper;
    if (y_dtype == DT_FLOAT32) static_cast<float*>(y)[i] = r;
    else store_q(y, y_dtype, i, orc_fp32_to_affine(r, yq.scale, yq.zp, y_dtype));
  }
  return 0;
}

// vxSoftmaxLayer2 (src/tim/vx/internal/src/kernel/vx/softmax_vx.c:88):
// exp(beta*(x - max)) / sum along one axis, in float32.
int32_t orc_softmax(const void* x, int32_t x_dtype, orc_quant xq, void* y, int32_t y_dtype, orc_quant yq,
                    const uint32_t* dims, uint32_t rank, int32_t axis, float beta) {
  if (axis < 0) axis += static_cast<int32_t>(rank);
  if (axis < 0 || axis >= static_cast<int32_t>(rank)) return -1;
  size_t inner = 1, outer = 1;
  for (int32_t d = 0; d < axis; ++d) inner *= dims[d];
  for (uint32_t d = axis + 1; d < rank; ++d) outer *= dims[d];
  const size_t len = dims[axis];
  auto real_at = [&](size_t i) -> float {
    return x_dtype == DT_FLOAT32 ? static_cast<const float*>(x)[i]
                                 : orc_affine_to_fp32(load_q(x, x_dtype, i), xq.scale, xq.zp);
  };
  for (size_t o = 0; o < outer; ++o) {
    for (size_t in = 0; in < inner; ++in) {
      const size_t base = o * len * inner + in;
      float m = -std::numeric_limits<float>::infinity();
      for (size_t k = 0; k < len; ++k) m = std::max(m, real_at(base + k * inner));
      float sum = 0.0f;
      for (size_t k = 0; k < len; ++k) sum += expf(beta * (real_at(base + k * inner) - m));
      for (size_t k = 0; k < len; ++k) {
        float r = expf(beta * (real_at(base + k * inner) - m)) / sum;
        const size_t idx = base + k * inner;
        if (y_dtype == DT_FLOAT32) static_cast<float*>(y)[idx] = r;
        else store_q(y, y_dtype, idx, orc_fp32_to_affine(r, yq.scale, yq.zp, y_dtype));
      }
    }
  }
  return 0;
}

}  // extern "C"
