// Device-side float -> quantized conversion shared by every kernel.
//
// Replays fp32_to_affine of the reference
// (src/tim/vx/internal/include/utils/vsi_nn_dtype_util_prv.h:228-254):
//     q = clamp((int32)(vsi_rint(real / scale) + zero_point), lo, hi),
// with vsi_rint (src/tim/vx/internal/include/utils/vsi_nn_math.h:191-210):
// exact .5 fractions go to the even integer, everything else goes through
// floorf(fabsf(x) + 0.5f) computed in float.  The reference tests the tie in
// double with a 1e-8 window; for a value that came from a float division that
// window contains only the exact tie, so the float test below is equivalent.
// Every step uses an explicit round-to-nearest intrinsic so that no
// multiply-add is fused and the result is bit-identical to the CPU sequence.
#ifndef B2VX_REQUANT_CUH_
#define B2VX_REQUANT_CUH_

#include "kernels.h"

namespace b2vx {

__device__ __forceinline__ int requant(float real, const OutQuant& q) {
  if (isinf(real)) return real < 0.0f ? q.lo : q.hi;
  const float x = __fdiv_rn(real, q.scale);
  const float ax = fabsf(x);
  const float fl = floorf(ax);
  float r;
  if (__fsub_rn(ax, fl) == 0.5f) {
    r = __fadd_rn(fl, static_cast<float>(static_cast<int>(fl) & 1));
  } else {
    r = floorf(__fadd_rn(ax, 0.5f));
  }
  r = copysignf(r, x);
  // (int32)(double(r) + zero_point), saturating; r is integer-valued.
  long long v = static_cast<long long>(__float2int_rn(r)) + q.zp;
  v = v < q.lo ? q.lo : v;
  v = v > q.hi ? q.hi : v;
  return static_cast<int>(v);
}

// Fast form of the same conversion for hot epilogues.  Returns q - lo, in
// [0, span] with span = hi - lo.  inv_scale = 1/scale (rounded), addc =
// zp - lo - 0x4B400000.
//
// t = real*inv_scale differs from the reference's real/scale by at most a
// couple of ulps, and the reference's rounding differs from round-to-nearest-
// even only within one ulp of a .5 fraction.  So whenever t is farther than
// |t|*2^-20 from every .5 fraction, RTNE(t) is the reference's result; RTNE
// comes from adding 1.5*2^23, which leaves the integer in the low mantissa
// bits.  The rare near-tie element (about |t|*2e-6 of them) takes the exact
// sequence.  |t| is clamped to 2^16 first: beyond that the output saturates
// whatever the rounding (|zp| and the output range are at most 8 bits).
__device__ __forceinline__ int requant_fast(float real, const OutQuant& q, float inv_scale, int addc, int span) {
  float t = __fmul_rn(real, inv_scale);
  t = fminf(fmaxf(t, -65536.0f), 65536.0f);
  const float r = __fadd_rn(t, 12582912.0f);
  const float d = __fsub_rn(t, __fsub_rn(r, 12582912.0f));
  const float thr = fmaf(fabsf(t), -9.5367431640625e-7f, 0.5f);
  int u = __vimin_s32_relu(__float_as_int(r) + addc, span);
  if (fabsf(d) > thr) u = requant(real, q) - q.lo;
  return u;
}

}  // namespace b2vx
#endif  // B2VX_REQUANT_CUH_
