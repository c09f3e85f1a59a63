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

// The same conversion for 32-bit outputs, where the rounded quotient itself can leave the int32 range:
// the reference adds the zero point in double and saturates afterwards.
__device__ __forceinline__ int requant_wide(float real, const OutQuant& q) {
  if (isinf(real)) return real < 0.0f ? q.lo : q.hi;
  const float x = __fdiv_rn(real, q.scale);
  if (!(x == x)) return max(q.lo, min(q.hi, 0));
  const float ax = fabsf(x);
  const float fl = floorf(ax);
  float r;
  if (__fsub_rn(ax, fl) == 0.5f) {
    r = __fadd_rn(fl, static_cast<float>(static_cast<int>(fl) & 1));   // a .5 fraction exists only below 2^23
  } else {
    r = floorf(__fadd_rn(ax, 0.5f));
  }
  r = copysignf(fminf(r, 1.0e12f), x);
  long long v = __float2ll_rn(r) + q.zp;
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


// ---- two float32 lanes per instruction (sm_100 packed arithmetic) -----------
// Each half is an IEEE round-to-nearest operation, bit-identical to the scalar
// intrinsic; the point is one issue slot for two results in instruction-bound
// requantization loops.
#ifdef B2VX_F2_INTRINSICS
// float2 values and the sm_100 packed intrinsics: the compiler keeps each value in a register pair.
typedef float2 f32x2;
__device__ __forceinline__ f32x2 f2_pack(float lo, float hi) { return make_float2(lo, hi); }
__device__ __forceinline__ f32x2 f2_pack_bits(uint32_t lo, uint32_t hi) { return make_float2(__uint_as_float(lo), __uint_as_float(hi)); }
__device__ __forceinline__ void f2_unpack(f32x2 v, float& lo, float& hi) { lo = v.x; hi = v.y; }
__device__ __forceinline__ void f2_unpack_bits(f32x2 v, uint32_t& lo, uint32_t& hi) { lo = __float_as_uint(v.x); hi = __float_as_uint(v.y); }
__device__ __forceinline__ f32x2 f2_add(f32x2 a, f32x2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ f32x2 f2_mul(f32x2 a, f32x2 b) { return __fmul2_rn(a, b); }
// Caution: a packed product consumed by a packed addition was observed to come back as one fused
// multiply-add on sm_100a (product unrounded) despite the .rn qualifiers.  Where the reference rounds
// the product and the sum separately, compute the product with the scalar __fmul_rn instead.
__device__ __forceinline__ f32x2 f2_fma(f32x2 a, f32x2 b, f32x2 c) { return __ffma2_rn(a, b, c); }
#else
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 f2_pack(float lo, float hi) {
  f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ f32x2 f2_pack_bits(uint32_t lo, uint32_t hi) {
  f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
  return r;
}
__device__ __forceinline__ void f2_unpack(f32x2 v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ void f2_unpack_bits(f32x2 v, uint32_t& lo, uint32_t& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=r"(lo), "=r"(hi) : "l"(v));
}
__device__ __forceinline__ f32x2 f2_add(f32x2 a, f32x2 b) {
  f32x2 r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ f32x2 f2_mul(f32x2 a, f32x2 b) {
  f32x2 r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ f32x2 f2_fma(f32x2 a, f32x2 b, f32x2 c) {
  f32x2 r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
#endif
// d = sat_u8(a) << 8 | sat_u8(b) | c << 16 (or the s8 form): saturating narrow + pack in one instruction.
__device__ __forceinline__ uint32_t pack_sat_u8(int hi, int lo, uint32_t upper) {
  uint32_t d;
  asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(hi), "r"(lo), "r"(upper));
  return d;
}
__device__ __forceinline__ uint32_t pack_sat_s8(int hi, int lo, uint32_t upper) {
  uint32_t d;
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(hi), "r"(lo), "r"(upper));
  return d;
}

// Host-side test for the two-sided fast rounding used by the hot loops: the value real/scale must stay
// far inside the range where adding 1.5*2^23 leaves the integer in the low mantissa bits.
#define B2VX_FAST_ROUND_LIMIT 2097152.0f   /* 2^21 */

// Requantization of one 16-column chunk of an accumulator row: acc + folded bias -> float ->
// * accumulator scale -> quantized bytes (the exact sequence is requant() in requant.cuh).
//
// Fast form.  The reference computes q = R(real / scale) + zp with R = round-half-even except within an
// ulp of a .5 fraction.  r_hi and r_lo round real*(1/scale)*(1 +- 2^-21) + zp to the nearest integer in
// one fused multiply-add each: adding 1.5*2^23 + zp leaves the integer in the low mantissa bits, and
// as long as real/scale stays above -1.5*2^23 (the host checks a bound on it when the plan is made, and
// sets exact_only otherwise) the bit pattern is monotone, so the saturating narrow below stays right.
// The reference's quotient (one rounding, of a divisor within half an ulp of 1/scale) lies strictly
// between the two products; when both give the same byte after saturation, that byte is the
// reference's result.  Elements that disagree are redone with the exact code.  Float work is done two
// lanes per instruction (f32x2) and four results are narrowed and packed by two cvt.pack.sat.
struct RequantConsts {
  f32x2 inv_hi2, inv_lo2, magic2;
  float inv_hi, inv_lo, magic;
  OutQuant oq;
  int out_signed;
  uint32_t out_flip;
  int exact_only;
};

// Four rounded values (bit patterns of r = t + magic) -> four saturated bytes.  The magic constant carries
// zp, plus 128 for int8 outputs, so that the saturation is always the unsigned one; out_flip
// (0x80808080 for int8, else 0) turns the biased bytes back into two's complement afterwards.
__device__ __forceinline__ uint32_t sat_pack4(uint32_t b0, uint32_t b1, uint32_t b2, uint32_t b3) {
  const int v0 = static_cast<int>(b0) - 0x4B400000, v1 = static_cast<int>(b1) - 0x4B400000;
  const int v2 = static_cast<int>(b2) - 0x4B400000, v3 = static_cast<int>(b3) - 0x4B400000;
  return pack_sat_u8(v1, v0, pack_sat_u8(v3, v2, 0u));
}

// Constants of one output quantization for requant_chunk16.
__device__ __forceinline__ RequantConsts make_requant_consts(const OutQuant& oq, int exact_only) {
  RequantConsts rc;
  const float inv = __frcp_rn(oq.scale);
  rc.inv_hi = __fmul_rn(inv, 1.000000476837158203125f);    // 1 + 2^-21
  rc.inv_lo = __fmul_rn(inv, 0.999999523162841796875f);    // 1 - 2^-21
  rc.out_signed = oq.lo < 0;
  rc.magic = 12582912.0f + static_cast<float>(oq.zp + (rc.out_signed ? 128 : 0));
  rc.inv_hi2 = f2_pack(rc.inv_hi, rc.inv_hi);
  rc.inv_lo2 = f2_pack(rc.inv_lo, rc.inv_lo);
  rc.magic2 = f2_pack(rc.magic, rc.magic);
  rc.oq = oq;
  rc.out_flip = rc.out_signed ? 0x80808080u : 0u;
  rc.exact_only = exact_only;
  return rc;
}

// EXTRA: the row has a term to subtract from every accumulator (sub = dz * S of this row) and/or a
// border correction (corr: 16 values for this chunk's channels, or null); without EXTRA both are
// ignored.  A template parameter because as run-time conditions they were compiled into instructions
// every chunk pays for.
template <bool EXTRA>
__device__ __forceinline__ uint4 requant_chunk16(const int (&acc)[16], const int* bias, const float* scale,
                                                 const RequantConsts& rc, int sub, const int32_t* corr) {
  f32x2 real[8];
#pragma unroll
  for (int g4 = 0; g4 < 4; ++g4) {
    int4 b4 = *reinterpret_cast<const int4*>(bias + g4 * 4);
    if (EXTRA) {
      b4.x -= sub; b4.y -= sub; b4.z -= sub; b4.w -= sub;
      if (corr) {
        const int4 c4 = __ldg(reinterpret_cast<const int4*>(corr + g4 * 4));
        b4.x += c4.x; b4.y += c4.y; b4.z += c4.z; b4.w += c4.w;
      }
    }
    const float4 s4 = *reinterpret_cast<const float4*>(scale + g4 * 4);
    real[2 * g4] = f2_mul(f2_pack(__int2float_rn(acc[g4 * 4 + 0] + b4.x), __int2float_rn(acc[g4 * 4 + 1] + b4.y)), f2_pack(s4.x, s4.y));
    real[2 * g4 + 1] = f2_mul(f2_pack(__int2float_rn(acc[g4 * 4 + 2] + b4.z), __int2float_rn(acc[g4 * 4 + 3] + b4.w)), f2_pack(s4.z, s4.w));
  }
  uint32_t wh[4], wl[4];
#pragma unroll
  for (int g4 = 0; g4 < 4; ++g4) {
    uint32_t h0, h1, h2, h3, l0, l1, l2, l3;
    f2_unpack_bits(f2_fma(real[2 * g4], rc.inv_hi2, rc.magic2), h0, h1);
    f2_unpack_bits(f2_fma(real[2 * g4 + 1], rc.inv_hi2, rc.magic2), h2, h3);
    f2_unpack_bits(f2_fma(real[2 * g4], rc.inv_lo2, rc.magic2), l0, l1);
    f2_unpack_bits(f2_fma(real[2 * g4 + 1], rc.inv_lo2, rc.magic2), l2, l3);
    wh[g4] = sat_pack4(h0, h1, h2, h3);
    wl[g4] = sat_pack4(l0, l1, l2, l3);
  }
  uint32_t differ = (wh[0] ^ wl[0]) | (wh[1] ^ wl[1]) | (wh[2] ^ wl[2]) | (wh[3] ^ wl[3]);
  // Opaque to the optimizer: otherwise it notices that each per-element test below implies this one,
  // drops it, and every chunk pays for sixteen tests.
  asm volatile("" : "+r"(differ));
  if (differ != 0u || rc.exact_only) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const uint32_t m = 0xFFu << (8 * (i & 3));
      if (((wh[i >> 2] ^ wl[i >> 2]) & m) != 0u || rc.exact_only) {
        float lo, hi;
        f2_unpack(real[i >> 1], lo, hi);
        const uint32_t q = (static_cast<uint32_t>(requant((i & 1) ? hi : lo, rc.oq)) ^ rc.out_flip) & 0xFFu;
        wh[i >> 2] = (wh[i >> 2] & ~m) | (q << (8 * (i & 3)));
      }
    }
  }
  return make_uint4(wh[0] ^ rc.out_flip, wh[1] ^ rc.out_flip, wh[2] ^ rc.out_flip, wh[3] ^ rc.out_flip);
}

// Quantized Add of four byte pairs through the 64 KB table (entry (a, b) at a*256 + (b ^ ((a & 31) << 2)),
// which spreads pairs that share b over the shared-memory banks): build the indices, four byte loads, pack.
__device__ __forceinline__ uint32_t add_lut_word(uint32_t aw, uint32_t bw, const uint8_t* tab) {
  uint32_t p01 = __byte_perm(bw, aw, 0x5140), p23 = __byte_perm(bw, aw, 0x7362);   // [b0 a0 b1 a1], [b2 a2 b3 a3]
  p01 ^= (p01 >> 6) & 0x007C007Cu;
  p23 ^= (p23 >> 6) & 0x007C007Cu;
  const uint32_t r0 = tab[p01 & 0xFFFFu], r1 = tab[p01 >> 16], r2 = tab[p23 & 0xFFFFu], r3 = tab[p23 >> 16];
  return __byte_perm(__byte_perm(r0, r1, 0x0040), __byte_perm(r2, r3, 0x0040), 0x5410);
}

}  // namespace b2vx
#endif  // B2VX_REQUANT_CUH_
