// CUDA-core kernels of the quantized-inference path: layout converters, the
// any-shape quantized convolution, depthwise convolution, pooling, Add, Relu,
// Softmax, im2col and the float32 variants.  All work on channels-last
// storage (kernels.h) with 128-bit or 32-bit accesses along the channel axis.
#include "kernels.h"
#include "requant.cuh"

namespace b2vx {
namespace {

constexpr int kThreads = 256;

inline unsigned grid_for(long long n, int threads) { return static_cast<unsigned>((n + threads - 1) / threads); }

// ---------------------------------------------------------------- layout

template <typename T>
__global__ void whcn_to_cl_kernel(const T* __restrict__ src, T* __restrict__ dst, int N, int C, int H, int W, int Cp) {
  const long long total = static_cast<long long>(N) * H * W * Cp;
  long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i >= total) return;
  int c = static_cast<int>(i % Cp);
  long long r = i / Cp;
  int w = static_cast<int>(r % W); r /= W;
  int h = static_cast<int>(r % H);
  int n = static_cast<int>(r / H);
  dst[i] = c < C ? src[((static_cast<long long>(n) * C + c) * H + h) * W + w] : T(0);
}

template <typename T>
__global__ void cl_to_whcn_kernel(const T* __restrict__ src, T* __restrict__ dst, int N, int C, int H, int W, int Cp) {
  const long long total = static_cast<long long>(N) * C * H * W;
  long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i >= total) return;
  int w = static_cast<int>(i % W);
  long long r = i / W;
  int h = static_cast<int>(r % H); r /= H;
  int c = static_cast<int>(r % C);
  int n = static_cast<int>(r / C);
  dst[i] = src[((static_cast<long long>(n) * H + h) * W + w) * Cp + c];
}

// ---------------------------------------------------------------- quantized conv, CUDA cores

template <bool XS>
__device__ __forceinline__ int dp4(unsigned a, unsigned b, int c) {
  int d;
  if (XS) asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  else asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

// One thread: one output pixel x 16 output channels.  A warp shares its 16
// weight rows, so weight loads are warp-uniform 128-bit loads served by L1.
template <bool XS>
__global__ void __launch_bounds__(128) conv_simt_kernel(const uint8_t* __restrict__ x, const int8_t* __restrict__ w8,
                                                       int Kp, ConvGeom g, ContractEpilogue e, uint8_t* __restrict__ y) {
  constexpr int OCT = 16;
  const long long P = static_cast<long long>(g.N) * g.Ho * g.Wo;
  const long long p = blockIdx.x * 128LL + threadIdx.x;
  const int oc0 = blockIdx.y * OCT;
  if (p >= P) return;
  const int wo = static_cast<int>(p % g.Wo);
  const long long t = p / g.Wo;
  const int ho = static_cast<int>(t % g.Ho);
  const int n = static_cast<int>(t / g.Ho);

  int acc[OCT];
#pragma unroll
  for (int o = 0; o < OCT; ++o) acc[o] = 0;
  int S = 0;
  const bool need_s = e.dz != nullptr;
  const int8_t* ones = w8 + static_cast<size_t>(g.Ocp) * Kp;
  const int chunks = g.Cp >> 4;

  for (int ky = 0; ky < g.kh; ++ky) {
    const int hi = ho * g.sy - g.pt + ky * g.dy;
    for (int kx = 0; kx < g.kw; ++kx) {
      const int wi = wo * g.sx - g.pl + kx * g.dx;
      const int tap = ky * g.kw + kx;
      if (hi < 0 || hi >= g.H || wi < 0 || wi >= g.W) {
        if (e.tapc) {
#pragma unroll
          for (int o = 0; o < OCT; ++o) acc[o] -= e.tapc[static_cast<size_t>(tap) * g.Ocp + oc0 + o];
        }
        continue;
      }
      const uint4* xp = reinterpret_cast<const uint4*>(x + ((static_cast<size_t>(n) * g.H + hi) * g.W + wi) * g.Cp);
      const int8_t* wt = w8 + static_cast<size_t>(tap) * g.Cp;
      for (int ch = 0; ch < chunks; ++ch) {
        const uint4 xv = xp[ch];
#pragma unroll
        for (int o = 0; o < OCT; ++o) {
          const uint4 wv = __ldg(reinterpret_cast<const uint4*>(wt + static_cast<size_t>(oc0 + o) * Kp + ch * 16));
          int a = acc[o];
          a = dp4<XS>(xv.x, wv.x, a);
          a = dp4<XS>(xv.y, wv.y, a);
          a = dp4<XS>(xv.z, wv.z, a);
          a = dp4<XS>(xv.w, wv.w, a);
          acc[o] = a;
        }
        if (need_s) {
          const uint4 ov = __ldg(reinterpret_cast<const uint4*>(ones + static_cast<size_t>(tap) * g.Cp + ch * 16));
          S = dp4<XS>(xv.x, ov.x, S);
          S = dp4<XS>(xv.y, ov.y, S);
          S = dp4<XS>(xv.z, ov.z, S);
          S = dp4<XS>(xv.w, ov.w, S);
        }
      }
    }
  }

  uint32_t packed[4] = {0, 0, 0, 0};
#pragma unroll
  for (int o = 0; o < OCT; ++o) {
    const int oc = oc0 + o;
    int v = acc[o] + e.bias_full[oc];
    if (need_s) v -= e.dz[oc] * S;
    const float real = __fmul_rn(__int2float_rn(v), e.acc_scale[oc]);
    const int q = requant(real, e.out);
    packed[o >> 2] |= static_cast<uint32_t>(q & 0xFF) << ((o & 3) * 8);
  }
  *reinterpret_cast<uint4*>(y + static_cast<size_t>(p) * g.Ocp + oc0) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
}

// ---------------------------------------------------------------- depthwise, quantized

// One thread: one output pixel x 4 output channels (one 32-bit word).
template <bool XS>
__global__ void depthwise_q_kernel(const uint8_t* __restrict__ x, int zx, const int16_t* __restrict__ wd,
                                   const int32_t* __restrict__ bias, const float* __restrict__ acc_scale,
                                   int multiplier, ConvGeom g, OutQuant out, uint8_t* __restrict__ y) {
  const int words = g.Ocp >> 2;
  const long long total = static_cast<long long>(g.N) * g.Ho * g.Wo * words;
  long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i >= total) return;
  const int cw = static_cast<int>(i % words);
  const long long p = i / words;
  const int wo = static_cast<int>(p % g.Wo);
  const long long t = p / g.Wo;
  const int ho = static_cast<int>(t % g.Ho);
  const int n = static_cast<int>(t / g.Ho);
  const int oc0 = cw * 4;
  int acc[4] = {0, 0, 0, 0};
  for (int ky = 0; ky < g.kh; ++ky) {
    const int hi = ho * g.sy - g.pt + ky * g.dy;
    if (hi < 0 || hi >= g.H) continue;
    for (int kx = 0; kx < g.kw; ++kx) {
      const int wi = wo * g.sx - g.pl + kx * g.dx;
      if (wi < 0 || wi >= g.W) continue;
      const uint8_t* px = x + ((static_cast<size_t>(n) * g.H + hi) * g.W + wi) * g.Cp;
      const int16_t* pw = wd + static_cast<size_t>(ky * g.kw + kx) * g.Ocp + oc0;
      int xv[4];
      if (multiplier == 1) {
        const uint32_t word = *reinterpret_cast<const uint32_t*>(px + oc0);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint32_t b = (word >> (8 * j)) & 0xFF;
          xv[j] = XS ? static_cast<int>(static_cast<int8_t>(b)) : static_cast<int>(b);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int ic = (oc0 + j) / multiplier;
          const uint8_t b = ic < g.C ? px[ic] : static_cast<uint8_t>(zx);
          xv[j] = XS ? static_cast<int>(static_cast<int8_t>(b)) : static_cast<int>(b);
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[j] += (xv[j] - zx) * static_cast<int>(pw[j]);
    }
  }
  uint32_t word = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int oc = oc0 + j;
    const int v = acc[j] + bias[oc];
    const float real = __fmul_rn(__int2float_rn(v), acc_scale[oc]);
    word |= static_cast<uint32_t>(requant(real, out) & 0xFF) << (8 * j);
  }
  *reinterpret_cast<uint32_t*>(y + static_cast<size_t>(p) * g.Ocp + oc0) = word;
}

// ---------------------------------------------------------------- float32 conv

// One thread per output element; the sum runs ic (outer), ky, kx (inner) with
// separate multiply and add, the order and rounding of the CPU oracle.
__global__ void conv_f32_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias,
                                int multiplier, int w_ic, ConvGeom g, float* __restrict__ y) {
  const long long total = static_cast<long long>(g.N) * g.Ho * g.Wo * g.Oc;
  long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i >= total) return;
  const int oc = static_cast<int>(i % g.Oc);
  const long long p = i / g.Oc;
  const int wo = static_cast<int>(p % g.Wo);
  const long long t = p / g.Wo;
  const int ho = static_cast<int>(t % g.Ho);
  const int n = static_cast<int>(t / g.Ho);
  const bool depthwise = multiplier >= 1;
  const int ic_begin = depthwise ? oc / multiplier : 0;
  const int ic_end = depthwise ? ic_begin + 1 : g.C;
  float acc = 0.0f;
  for (int ic = ic_begin; ic < ic_end; ++ic) {
    const float* wk = depthwise ? w + static_cast<size_t>(oc) * g.kh * g.kw
                                : w + (static_cast<size_t>(oc) * w_ic + ic) * g.kh * g.kw;
    for (int ky = 0; ky < g.kh; ++ky) {
      const int hi = ho * g.sy - g.pt + ky * g.dy;
      if (hi < 0 || hi >= g.H) continue;
      for (int kx = 0; kx < g.kw; ++kx) {
        const int wi = wo * g.sx - g.pl + kx * g.dx;
        if (wi < 0 || wi >= g.W) continue;
        const float xv = x[((static_cast<size_t>(n) * g.H + hi) * g.W + wi) * g.Cp + ic];
        acc = __fadd_rn(acc, __fmul_rn(xv, wk[ky * g.kw + kx]));
      }
    }
  }
  if (bias) acc = __fadd_rn(acc, bias[oc]);
  y[static_cast<size_t>(p) * g.Ocp + oc] = acc;
}

// ---------------------------------------------------------------- pooling

template <bool XS>
__global__ void pool_q_kernel(const uint8_t* __restrict__ x, int type, float in_scale, int in_zp, int same_quant,
                              ConvGeom g, OutQuant out, uint8_t* __restrict__ y) {
  const int words = g.Cp >> 2;
  const long long total = static_cast<long long>(g.N) * g.Ho * g.Wo * words;
  long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i >= total) return;
  const int cw = static_cast<int>(i % words);
  const long long p = i / words;
  const int wo = static_cast<int>(p % g.Wo);
  const long long t = p / g.Wo;
  const int ho = static_cast<int>(t % g.Ho);
  const int n = static_cast<int>(t / g.Ho);
  int sum[4] = {0, 0, 0, 0};
  int mx[4] = {INT_MIN, INT_MIN, INT_MIN, INT_MIN};
  int count = 0;
  for (int ky = 0; ky < g.kh; ++ky) {
    const int hi = ho * g.sy - g.pt + ky;
    if (hi < 0 || hi >= g.H) continue;
    for (int kx = 0; kx < g.kw; ++kx) {
      const int wi = wo * g.sx - g.pl + kx;
      if (wi < 0 || wi >= g.W) continue;
      const uint32_t word =
          *reinterpret_cast<const uint32_t*>(x + ((static_cast<size_t>(n) * g.H + hi) * g.W + wi) * g.Cp + cw * 4);
      ++count;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t b = (word >> (8 * j)) & 0xFF;
        const int v = XS ? static_cast<int>(static_cast<int8_t>(b)) : static_cast<int>(b);
        sum[j] += v - in_zp;
        mx[j] = max(mx[j], v);
      }
    }
  }
  const float div = type == 1 ? static_cast<float>(g.kw * g.kh) : static_cast<float>(count);
  uint32_t word = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    int q;
    if (type == 0) {
      q = count ? mx[j] : in_zp;
      if (!same_quant) q = requant(__fmul_rn(__fsub_rn(__int2float_rn(q), __int2float_rn(in_zp)), in_scale), out);
    } else {
      const float avg = count ? __fdiv_rn(__fmul_rn(__int2float_rn(sum[j]), in_scale), div) : 0.0f;
      q = requant(avg, out);
    }
    word |= static_cast<uint32_t>(q & 0xFF) << (8 * j);
  }
  *reinterpret_cast<uint32_t*>(y + static_cast<size_t>(p) * g.Cp + cw * 4) = word;
}

__global__ void pool_f32_kernel(const float* __restrict__ x, int type, ConvGeom g, float* __restrict__ y) {
  const long long total = static_cast<long long>(g.N) * g.Ho * g.Wo * g.C;
  long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i >= total) return;
  const int c = static_cast<int>(i % g.C);
  const long long p = i / g.C;
  const int wo = static_cast<int>(p % g.Wo);
  const long long t = p / g.Wo;
  const int ho = static_cast<int>(t % g.Ho);
  const int n = static_cast<int>(t / g.Ho);
  float sum = 0.0f, mx = -INFINITY;
  int count = 0;
  for (int ky = 0; ky < g.kh; ++ky) {
    const int hi = ho * g.sy - g.pt + ky;
    if (hi < 0 || hi >= g.H) continue;
    for (int kx = 0; kx < g.kw; ++kx) {
      const int wi = wo * g.sx - g.pl + kx;
      if (wi < 0 || wi >= g.W) continue;
      const float v = x[((static_cast<size_t>(n) * g.H + hi) * g.W + wi) * g.Cp + c];
      sum = __fadd_rn(sum, v);
      mx = fmaxf(mx, v);
      ++count;
    }
  }
  const float div = type == 1 ? static_cast<float>(g.kw * g.kh) : static_cast<float>(count);
  float r = 0.0f;
  if (count) r = type == 0 ? mx : __fdiv_rn(sum, div);
  y[static_cast<size_t>(p) * g.Cp + c] = r;
}

// ---------------------------------------------------------------- elementwise

template <bool S>
__device__ __forceinline__ int byte_at(uint32_t word, int j) {
  const uint32_t b = (word >> (8 * j)) & 0xFF;
  return S ? static_cast<int>(static_cast<int8_t>(b)) : static_cast<int>(b);
}

// 16 elements per thread, 128-bit loads and stores.  The two dequantizations
// ((q - zp) * scale, 256 possible values each) are tabulated in shared memory
// by the block; the sum is requantized with requant_fast.
template <bool AS, bool BS>
__global__ void add_q_kernel(const uint4* __restrict__ a, float sa, int za, const uint4* __restrict__ b, float sb, int zb,
                             OutQuant out, uint4* __restrict__ y, size_t n16) {
  __shared__ float fa[256], fb[256];
  for (int i = threadIdx.x; i < 256; i += blockDim.x) {
    const int qa = AS ? static_cast<int>(static_cast<int8_t>(i)) : i;
    const int qb = BS ? static_cast<int>(static_cast<int8_t>(i)) : i;
    fa[i] = __fmul_rn(__fsub_rn(__int2float_rn(qa), __int2float_rn(za)), sa);
    fb[i] = __fmul_rn(__fsub_rn(__int2float_rn(qb), __int2float_rn(zb)), sb);
  }
  __syncthreads();
  const float inv_scale = __frcp_rn(out.scale);
  const int span = out.hi - out.lo, addc = out.zp - out.lo - 0x4B400000;
  const uint32_t sign_fix = out.lo < 0 ? 0x80808080u : 0u;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n16; i += stride) {
    const uint4 av = a[i], bv = b[i];
    const uint32_t aw[4] = {av.x, av.y, av.z, av.w}, bw[4] = {bv.x, bv.y, bv.z, bv.w};
    uint32_t ow[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      uint32_t word = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float r = __fadd_rn(fa[(aw[k] >> (8 * j)) & 0xFF], fb[(bw[k] >> (8 * j)) & 0xFF]);
        word |= static_cast<uint32_t>(requant_fast(r, out, inv_scale, addc, span)) << (8 * j);
      }
      ow[k] = word ^ sign_fix;
    }
    y[i] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
  }
}

__global__ void add_f32_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ y, size_t n) {
  size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (i < n) y[i] = __fadd_rn(a[i], b[i]);
}

// Any 8-bit -> 8-bit pointwise map (Relu, Relu6 with arbitrary input/output
// quantization) as a 256-entry table built on the host with the reference's
// float sequence; 16 elements per thread.
__global__ void lut_q_kernel(const uint4* __restrict__ x, const uint8_t* __restrict__ lut, uint4* __restrict__ y, size_t n16) {
  __shared__ uint8_t t[256];
  for (int i = threadIdx.x; i < 256; i += blockDim.x) t[i] = lut[i];
  __syncthreads();
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n16; i += stride) {
    const uint4 xv = x[i];
    const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
    uint32_t ow[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      ow[k] = static_cast<uint32_t>(t[xw[k] & 0xFF]) | (static_cast<uint32_t>(t[(xw[k] >> 8) & 0xFF]) << 8) |
              (static_cast<uint32_t>(t[(xw[k] >> 16) & 0xFF]) << 16) | (static_cast<uint32_t>(t[xw[k] >> 24]) << 24);
    }
    y[i] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
  }
}

__global__ void relu_f32_kernel(const float* __restrict__ x, float upper, float* __restrict__ y, size_t n) {
  size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (i >= n) return;
  float r = x[i];
  r = r < 0.0f ? 0.0f : r;
  if (upper >= 0.0f && r > upper) r = upper;
  y[i] = r;
}

// ---------------------------------------------------------------- softmax

__device__ __forceinline__ float load_real(const void* x, int kind, long long i, float s, int z) {
  if (kind == 2) return static_cast<const float*>(x)[i];
  const int v = kind == 1 ? static_cast<int>(static_cast<const int8_t*>(x)[i]) : static_cast<int>(static_cast<const uint8_t*>(x)[i]);
  return __fmul_rn(__fsub_rn(__int2float_rn(v), __int2float_rn(z)), s);
}

// One thread per slice; slices are short (class scores).
__global__ void softmax_kernel(const void* __restrict__ x, int x_kind, float sx, int zx, void* __restrict__ y, int y_kind,
                               OutQuant out, float beta, SoftmaxGeom g) {
  const long long slices = static_cast<long long>(g.o[0]) * g.o[1] * g.o[2];
  long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i >= slices) return;
  const int a = static_cast<int>(i % g.o[0]);
  const long long r = i / g.o[0];
  const int b = static_cast<int>(r % g.o[1]);
  const int c = static_cast<int>(r / g.o[1]);
  const long long xb = a * g.xs[0] + b * g.xs[1] + c * g.xs[2];
  const long long yb = a * g.ys[0] + b * g.ys[1] + c * g.ys[2];
  float m = -INFINITY;
  for (int k = 0; k < g.len; ++k) m = fmaxf(m, load_real(x, x_kind, xb + k * g.x_stride, sx, zx));
  float sum = 0.0f;
  for (int k = 0; k < g.len; ++k)
    sum = __fadd_rn(sum, expf(__fmul_rn(beta, __fsub_rn(load_real(x, x_kind, xb + k * g.x_stride, sx, zx), m))));
  for (int k = 0; k < g.len; ++k) {
    const float v = __fdiv_rn(expf(__fmul_rn(beta, __fsub_rn(load_real(x, x_kind, xb + k * g.x_stride, sx, zx), m))), sum);
    const long long idx = yb + k * g.y_stride;
    if (y_kind == 2) static_cast<float*>(y)[idx] = v;
    else static_cast<uint8_t*>(y)[idx] = static_cast<uint8_t>(requant(v, out) & 0xFF);
  }
}

// ---------------------------------------------------------------- im2col

// One thread writes 16 consecutive bytes of one im2col row.
__global__ void im2col_kernel(const uint8_t* __restrict__ x, int Cs, int Kp, int zx, ConvGeom g, uint8_t* __restrict__ col) {
  const int chunks = Kp >> 4;
  const long long total = static_cast<long long>(g.N) * g.Ho * g.Wo * chunks;
  long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i >= total) return;
  const int ch = static_cast<int>(i % chunks);
  const long long p = i / chunks;
  const int wo = static_cast<int>(p % g.Wo);
  const long long t = p / g.Wo;
  const int ho = static_cast<int>(t % g.Ho);
  const int n = static_cast<int>(t / g.Ho);
  const int K = g.kh * g.kw * Cs;
  const int k0 = ch * 16;
  uint4 v;
  if (Cs == g.Cp && k0 < K) {
    // a 16-byte chunk never straddles taps when the channel stride is Cp
    const int tap = k0 / Cs, c0 = k0 - tap * Cs;
    const int ky = tap / g.kw, kx = tap - ky * g.kw;
    const int hi = ho * g.sy - g.pt + ky * g.dy, wi = wo * g.sx - g.pl + kx * g.dx;
    if (hi >= 0 && hi < g.H && wi >= 0 && wi < g.W) {
      v = *reinterpret_cast<const uint4*>(x + ((static_cast<size_t>(n) * g.H + hi) * g.W + wi) * g.Cp + c0);
    } else {
      const uint32_t z = (zx & 0xFF) * 0x01010101u;
      v = make_uint4(z, z, z, z);
    }
  } else {
    uint32_t w4[4] = {0, 0, 0, 0};
    for (int j = 0; j < 16; ++j) {
      const int k = k0 + j;
      uint32_t b = 0;
      if (k < K) {
        const int tap = k / Cs, c = k - tap * Cs;
        const int ky = tap / g.kw, kx = tap - ky * g.kw;
        const int hi = ho * g.sy - g.pt + ky * g.dy, wi = wo * g.sx - g.pl + kx * g.dx;
        if (c >= g.C) b = 0;
        else if (hi >= 0 && hi < g.H && wi >= 0 && wi < g.W)
          b = x[((static_cast<size_t>(n) * g.H + hi) * g.W + wi) * g.Cp + c];
        else b = zx & 0xFF;
      }
      w4[j >> 2] |= b << ((j & 3) * 8);
    }
    v = make_uint4(w4[0], w4[1], w4[2], w4[3]);
  }
  *reinterpret_cast<uint4*>(col + static_cast<size_t>(p) * Kp + k0) = v;
}

// im2col from a WHCN input: one block per (image, output row).  The input rows the
// block needs (C*kh of them, padding materialised with the zero point) are staged
// in shared memory with coalesced loads; every thread then assembles 16-byte
// pieces of im2col rows from a per-k offset table.
__global__ void im2col_whcn_kernel(const uint8_t* __restrict__ x, int Kp, int zx, ConvGeom g, int rowlen,
                                   uint8_t* __restrict__ col) {
  extern __shared__ uint8_t sm[];
  const int n = blockIdx.y, ho = blockIdx.x;
  const int rows = g.C * g.kh;
  const int K = rows * g.kw;
  int* koff = reinterpret_cast<int*>(sm);                    // [Kp]
  uint8_t* img = sm + static_cast<size_t>(Kp) * sizeof(int);   // [rows][rowlen]
  for (int k = threadIdx.x; k < Kp; k += blockDim.x) {
    int off = -1;
    if (k < K) {
      const int r = k / g.kw, kx = k - r * g.kw;
      off = r * rowlen + kx * g.dx;
    }
    koff[k] = off;
  }
  for (int idx = threadIdx.x; idx < rows * rowlen; idx += blockDim.x) {
    const int r = idx / rowlen, j = idx - r * rowlen;
    const int c = r / g.kh, ky = r - c * g.kh;
    const int hi = ho * g.sy - g.pt + ky * g.dy, wi = j - g.pl;
    uint8_t v = static_cast<uint8_t>(zx);
    if (hi >= 0 && hi < g.H && wi >= 0 && wi < g.W) v = x[((static_cast<size_t>(n) * g.C + c) * g.H + hi) * g.W + wi];
    img[idx] = v;
  }
  __syncthreads();
  const int chunks = Kp >> 4;
  uint8_t* out = col + (static_cast<size_t>(n) * g.Ho + ho) * g.Wo * Kp;
  for (int q = threadIdx.x; q < g.Wo * chunks; q += blockDim.x) {
    const int wo = q / chunks, ch = q - wo * chunks;
    const int base = wo * g.sx;
    uint32_t w4[4] = {0, 0, 0, 0};
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const int off = koff[ch * 16 + j];
      const uint32_t b = off >= 0 ? img[off + base] : 0u;
      w4[j >> 2] |= b << ((j & 3) * 8);
    }
    *reinterpret_cast<uint4*>(out + static_cast<size_t>(wo) * Kp + ch * 16) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
  }
}

}  // namespace

// ---------------------------------------------------------------- wrappers

void launch_whcn_to_cl(const void* src, void* dst, int N, int C, int H, int W, int Cp, int elem, cudaStream_t s) {
  const long long total = static_cast<long long>(N) * H * W * Cp;
  if (total == 0) return;
  if (elem == 1)
    whcn_to_cl_kernel<uint8_t><<<grid_for(total, kThreads), kThreads, 0, s>>>(static_cast<const uint8_t*>(src),
                                                                           static_cast<uint8_t*>(dst), N, C, H, W, Cp);
  else
    whcn_to_cl_kernel<uint32_t><<<grid_for(total, kThreads), kThreads, 0, s>>>(static_cast<const uint32_t*>(src),
                                                                            static_cast<uint32_t*>(dst), N, C, H, W, Cp);
}

void launch_cl_to_whcn(const void* src, void* dst, int N, int C, int H, int W, int Cp, int elem, cudaStream_t s) {
  const long long total = static_cast<long long>(N) * C * H * W;
  if (total == 0) return;
  if (elem == 1)
    cl_to_whcn_kernel<uint8_t><<<grid_for(total, kThreads), kThreads, 0, s>>>(static_cast<const uint8_t*>(src),
                                                                           static_cast<uint8_t*>(dst), N, C, H, W, Cp);
  else
    cl_to_whcn_kernel<uint32_t><<<grid_for(total, kThreads), kThreads, 0, s>>>(static_cast<const uint32_t*>(src),
                                                                            static_cast<uint32_t*>(dst), N, C, H, W, Cp);
}

void launch_conv_simt(const void* x, int x_signed, const int8_t* w8, int Kp, const ConvGeom& g,
                      const ContractEpilogue& e, void* y, cudaStream_t s) {
  const long long P = static_cast<long long>(g.N) * g.Ho * g.Wo;
  if (P == 0) return;
  dim3 grid(grid_for(P, 128), g.Ocp / 16);
  if (x_signed)
    conv_simt_kernel<true><<<grid, 128, 0, s>>>(static_cast<const uint8_t*>(x), w8, Kp, g, e, static_cast<uint8_t*>(y));
  else
    conv_simt_kernel<false><<<grid, 128, 0, s>>>(static_cast<const uint8_t*>(x), w8, Kp, g, e, static_cast<uint8_t*>(y));
}

void launch_depthwise_q(const void* x, int x_signed, int zx, const int16_t* wd, const int32_t* bias,
                        const float* acc_scale, int multiplier, const ConvGeom& g, OutQuant out, void* y,
                        cudaStream_t s) {
  const long long total = static_cast<long long>(g.N) * g.Ho * g.Wo * (g.Ocp / 4);
  if (total == 0) return;
  if (x_signed)
    depthwise_q_kernel<true><<<grid_for(total, kThreads), kThreads, 0, s>>>(static_cast<const uint8_t*>(x), zx, wd, bias,
                                                                         acc_scale, multiplier, g, out,
                                                                         static_cast<uint8_t*>(y));
  else
    depthwise_q_kernel<false><<<grid_for(total, kThreads), kThreads, 0, s>>>(static_cast<const uint8_t*>(x), zx, wd, bias,
                                                                          acc_scale, multiplier, g, out,
                                                                          static_cast<uint8_t*>(y));
}

void launch_conv_f32(const float* x, const float* w, const float* bias, int multiplier, int w_ic, const ConvGeom& g,
                     float* y, cudaStream_t s) {
  const long long total = static_cast<long long>(g.N) * g.Ho * g.Wo * g.Oc;
  if (total == 0) return;
  conv_f32_kernel<<<grid_for(total, kThreads), kThreads, 0, s>>>(x, w, bias, multiplier, w_ic, g, y);
}

void launch_pool_q(const void* x, int is_signed, int type, float in_scale, int in_zp, int same_quant, const ConvGeom& g,
                   OutQuant out, void* y, cudaStream_t s) {
  const long long total = static_cast<long long>(g.N) * g.Ho * g.Wo * (g.Cp / 4);
  if (total == 0) return;
  if (is_signed)
    pool_q_kernel<true><<<grid_for(total, kThreads), kThreads, 0, s>>>(static_cast<const uint8_t*>(x), type, in_scale, in_zp,
                                                                    same_quant, g, out, static_cast<uint8_t*>(y));
  else
    pool_q_kernel<false><<<grid_for(total, kThreads), kThreads, 0, s>>>(static_cast<const uint8_t*>(x), type, in_scale,
                                                                     in_zp, same_quant, g, out, static_cast<uint8_t*>(y));
}

void launch_pool_f32(const float* x, int type, const ConvGeom& g, float* y, cudaStream_t s) {
  const long long total = static_cast<long long>(g.N) * g.Ho * g.Wo * g.C;
  if (total == 0) return;
  pool_f32_kernel<<<grid_for(total, kThreads), kThreads, 0, s>>>(x, type, g, y);
}

void launch_add_q(const void* a, int a_signed, float sa, int za, const void* b, int b_signed, float sb, int zb,
                  OutQuant out, int /*out_signed*/, void* y, size_t n, cudaStream_t s) {
  const size_t n16 = n / 16;
  if (n16 == 0) return;
  unsigned grid = grid_for(static_cast<long long>(n16), kThreads);
  if (grid > 148u * 16u) grid = 148u * 16u;
  const uint4* pa = static_cast<const uint4*>(a);
  const uint4* pb = static_cast<const uint4*>(b);
  uint4* py = static_cast<uint4*>(y);
  if (a_signed && b_signed) add_q_kernel<true, true><<<grid, kThreads, 0, s>>>(pa, sa, za, pb, sb, zb, out, py, n16);
  else if (a_signed) add_q_kernel<true, false><<<grid, kThreads, 0, s>>>(pa, sa, za, pb, sb, zb, out, py, n16);
  else if (b_signed) add_q_kernel<false, true><<<grid, kThreads, 0, s>>>(pa, sa, za, pb, sb, zb, out, py, n16);
  else add_q_kernel<false, false><<<grid, kThreads, 0, s>>>(pa, sa, za, pb, sb, zb, out, py, n16);
}

void launch_add_f32(const float* a, const float* b, float* y, size_t n, cudaStream_t s) {
  if (n == 0) return;
  add_f32_kernel<<<grid_for(static_cast<long long>(n), kThreads), kThreads, 0, s>>>(a, b, y, n);
}

void launch_lut_q(const void* x, const uint8_t* lut, void* y, size_t n, cudaStream_t s) {
  const size_t n16 = n / 16;
  if (n16 == 0) return;
  unsigned grid = grid_for(static_cast<long long>(n16), kThreads);
  if (grid > 148u * 16u) grid = 148u * 16u;
  lut_q_kernel<<<grid, kThreads, 0, s>>>(static_cast<const uint4*>(x), lut, static_cast<uint4*>(y), n16);
}

void launch_relu_f32(const float* x, float upper, float* y, size_t n, cudaStream_t s) {
  if (n == 0) return;
  relu_f32_kernel<<<grid_for(static_cast<long long>(n), kThreads), kThreads, 0, s>>>(x, upper, y, n);
}

void launch_softmax(const void* x, int x_kind, float sx, int zx, void* y, int y_kind, OutQuant out, float beta,
                    const SoftmaxGeom& g, cudaStream_t s) {
  const long long slices = static_cast<long long>(g.o[0]) * g.o[1] * g.o[2];
  if (slices == 0 || g.len == 0) return;
  softmax_kernel<<<grid_for(slices, 128), 128, 0, s>>>(x, x_kind, sx, zx, y, y_kind, out, beta, g);
}

void launch_im2col(const void* x, int Cs, int Kp, int zx, const ConvGeom& g, void* col, cudaStream_t s) {
  const long long total = static_cast<long long>(g.N) * g.Ho * g.Wo * (Kp / 16);
  if (total == 0) return;
  im2col_kernel<<<grid_for(total, kThreads), kThreads, 0, s>>>(static_cast<const uint8_t*>(x), Cs, Kp, zx, g,
                                                             static_cast<uint8_t*>(col));
}

void launch_im2col_whcn(const void* x, int Kp, int zx, const ConvGeom& g, void* col, cudaStream_t s) {
  if (g.N == 0 || g.Ho == 0 || g.Wo == 0) return;
  // input columns a row of outputs touches, counted from -pad_left
  const int rowlen = (g.Wo - 1) * g.sx + (g.kw - 1) * g.dx + 1;
  const size_t smem = static_cast<size_t>(Kp) * sizeof(int) + static_cast<size_t>(g.C) * g.kh * rowlen;
  dim3 grid(g.Ho, g.N);
  im2col_whcn_kernel<<<grid, 256, smem, s>>>(static_cast<const uint8_t*>(x), Kp, zx, g, rowlen, static_cast<uint8_t*>(col));
}

}  // namespace b2vx
