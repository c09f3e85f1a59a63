// CUDA-core kernels of the quantized-inference path: layout converters, the
// any-shape quantized convolution, depthwise convolution, pooling, Add, Relu,
// Softmax, im2col and the float32 variants.  All work on channels-last
// storage (kernels.h) with 128-bit or 32-bit accesses along the channel axis.
#include <cmath>
#include <cstdlib>
#include <cstring>

#include "kernels.h"
#include "pdl.cuh"
#include "requant.cuh"

namespace b2vx {
namespace {

constexpr int kThreads = 256;

inline unsigned grid_for(long long n, int threads) { return static_cast<unsigned>((n + threads - 1) / threads); }

// ---------------------------------------------------------------- layout

// A WHCN image is a [C][H*W] matrix (pixels contiguous), the channels-last image its transpose
// [H*W][Cp].  Both converters move 64-channel x 64-pixel byte tiles through shared memory so that
// either side is touched in 64-byte runs; a thread transposes one 4 x 4 byte block in registers.
// Shared tile: [64 pixels][16 words of 4 channels], the four 16-byte chunks of a pixel XOR-swizzled
// with the pixel's block index to spread the banks.

// 4 x 4 byte transpose: r[j] holds bytes (j, 0..3); on return r[i] holds bytes (0..3, i).
__device__ __forceinline__ void transpose4x4(uint32_t (&r)[4]) {
  const uint32_t t0 = __byte_perm(r[0], r[1], 0x5140), t1 = __byte_perm(r[0], r[1], 0x7362);
  const uint32_t t2 = __byte_perm(r[2], r[3], 0x5140), t3 = __byte_perm(r[2], r[3], 0x7362);
  r[0] = __byte_perm(t0, t2, 0x5410);
  r[1] = __byte_perm(t0, t2, 0x7632);
  r[2] = __byte_perm(t1, t3, 0x5410);
  r[3] = __byte_perm(t1, t3, 0x7632);
}

template <bool ALIGNED>
__global__ void __launch_bounds__(256) whcn_to_cl_u8_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int C,
                                                            int HW, int Cp) {
  pdl_wait();
  pdl_trigger();
  __shared__ uint4 tile[64 * 4];
  const int p0 = blockIdx.x * 64, c0 = blockIdx.y * 64, n = blockIdx.z;
  const int t = threadIdx.x;
  {
    const int pb = t & 15, cb = t >> 4;
    const int p = p0 + 4 * pb;
    uint32_t r[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = c0 + 4 * cb + j;
      r[j] = 0;
      if (c < C) {
        const uint8_t* row = src + (static_cast<size_t>(n) * C + c) * HW;
        if (ALIGNED) {
          if (p < HW) r[j] = *reinterpret_cast<const uint32_t*>(row + p);
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i)
            if (p + i < HW) r[j] |= static_cast<uint32_t>(row[p + i]) << (8 * i);
        }
      }
    }
    transpose4x4(r);   // r[i] = pixel 4*pb+i, channels 4*cb .. 4*cb+3
    uint32_t* words = reinterpret_cast<uint32_t*>(tile);
#pragma unroll
    for (int i = 0; i < 4; ++i) words[(4 * pb + i) * 16 + (((cb >> 2) ^ (pb & 3)) << 2) + (cb & 3)] = r[i];
  }
  __syncthreads();
  {
    const int px = t >> 2, chunk = t & 3;
    const int p = p0 + px, c = c0 + 16 * chunk;
    if (p < HW && c < Cp)
      *reinterpret_cast<uint4*>(dst + (static_cast<size_t>(n) * HW + p) * Cp + c) = tile[px * 4 + (chunk ^ ((px >> 2) & 3))];
  }
}

template <bool ALIGNED>
__global__ void __launch_bounds__(256) cl_to_whcn_u8_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int C,
                                                            int HW, int Cp) {
  pdl_wait();
  pdl_trigger();
  __shared__ uint4 tile[64 * 4];
  const int p0 = blockIdx.x * 64, c0 = blockIdx.y * 64, n = blockIdx.z;
  const int t = threadIdx.x;
  {
    const int px = t >> 2, chunk = t & 3;
    const int p = p0 + px, c = c0 + 16 * chunk;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (p < HW && c < Cp) v = *reinterpret_cast<const uint4*>(src + (static_cast<size_t>(n) * HW + p) * Cp + c);
    tile[px * 4 + (chunk ^ ((px >> 2) & 3))] = v;
  }
  __syncthreads();
  {
    const int pb = t & 15, cb = t >> 4;
    const int p = p0 + 4 * pb;
    const uint32_t* words = reinterpret_cast<const uint32_t*>(tile);
    uint32_t r[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) r[i] = words[(4 * pb + i) * 16 + (((cb >> 2) ^ (pb & 3)) << 2) + (cb & 3)];
    transpose4x4(r);   // r[j] = channel 4*cb+j, pixels 4*pb .. 4*pb+3
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = c0 + 4 * cb + j;
      if (c >= C) continue;
      uint8_t* row = dst + (static_cast<size_t>(n) * C + c) * HW;
      if (ALIGNED) {
        if (p < HW) *reinterpret_cast<uint32_t*>(row + p) = r[j];
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (p + i < HW) row[p + i] = static_cast<uint8_t>(r[j] >> (8 * i));
      }
    }
  }
}

// 32-bit elements: the classic 32 x 32 tile with a padded row.
__global__ void __launch_bounds__(256) whcn_to_cl_u32_kernel(const uint32_t* __restrict__ src, uint32_t* __restrict__ dst, int C,
                                                             int HW, int Cp) {
  __shared__ uint32_t tile[32][33];
  const int p0 = blockIdx.x * 32, c0 = blockIdx.y * 32, n = blockIdx.z;
  const int lx = threadIdx.x & 31, ly = threadIdx.x >> 5;
  for (int j = ly; j < 32; j += 8) {
    const int c = c0 + j, p = p0 + lx;
    tile[j][lx] = (c < C && p < HW) ? src[(static_cast<size_t>(n) * C + c) * HW + p] : 0u;
  }
  __syncthreads();
  for (int j = ly; j < 32; j += 8) {
    const int p = p0 + j, c = c0 + lx;
    if (p < HW && c < Cp) dst[(static_cast<size_t>(n) * HW + p) * Cp + c] = tile[lx][j];
  }
}

__global__ void __launch_bounds__(256) cl_to_whcn_u32_kernel(const uint32_t* __restrict__ src, uint32_t* __restrict__ dst, int C,
                                                             int HW, int Cp) {
  __shared__ uint32_t tile[32][33];
  const int p0 = blockIdx.x * 32, c0 = blockIdx.y * 32, n = blockIdx.z;
  const int lx = threadIdx.x & 31, ly = threadIdx.x >> 5;
  for (int j = ly; j < 32; j += 8) {
    const int p = p0 + j, c = c0 + lx;
    tile[j][lx] = (p < HW && c < Cp) ? src[(static_cast<size_t>(n) * HW + p) * Cp + c] : 0u;
  }
  __syncthreads();
  for (int j = ly; j < 32; j += 8) {
    const int c = c0 + j, p = p0 + lx;
    if (c < C && p < HW) dst[(static_cast<size_t>(n) * C + c) * HW + p] = tile[lx][j];
  }
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

// ---------------------------------------------------------------- depthwise, quantized, multiplier 1

// A block owns a slab of up to 64 channels and a run of output-pixel pairs; a thread owns 16 channels
// (one 128-bit access) of two horizontally adjacent output pixels.  The slab's weights sit in shared
// memory as one 32-bit word per (tap, channel): w - zw as a 16-bit half placed so that one dp2a
// multiplies it with that channel's byte of an input word (channel c of a word: half c & 1, byte pair
// c >> 1), i.e. one instruction per multiply-accumulate with no byte extraction.  Out-of-bounds taps
// read as the input zero point, so the zero-point term is a per-channel constant folded into the bias:
//   acc = sum_taps x * (w - zw)  +  [bias - zx * sum_taps (w - zw)].
// Signed inputs are biased by 128 on load (and zx with them).  The epilogue is the 16-value
// requantization shared with the tensor-core GEMM.
struct DwParams {
  ConvGeom g;
  const uint32_t* wtab;      // [taps][Ocp] words
  const uint32_t* wtab_v;    // 3x3 windows: [6][Ocp] words for the strip form (see depthwise_strip_kernel), else null
  const int32_t* bias_full;  // [Ocp]
  const float* acc_scale;    // [Ocp]
  OutQuant out;
  uint32_t x_flip;           // 0x80808080 for int8 input
  uint32_t zx_word;          // biased zero point replicated into four bytes
  int exact_only;
  int slab;                  // channels per block: min(Ocp, 64)
};

template <int MODE>
__device__ __forceinline__ int dp2a_su(uint32_t w16x2, uint32_t x8x4, int c) {
  int d;
  if (MODE == 0) asm("dp2a.lo.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(w16x2), "r"(x8x4), "r"(c));
  else asm("dp2a.hi.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(w16x2), "r"(x8x4), "r"(c));
  return d;
}

__device__ __forceinline__ void dw_mac16(int (&acc)[16], const uint4& x, const uint4 (&w)[4]) {
  const uint32_t xw[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    acc[4 * k + 0] = dp2a_su<0>(w[k].x, xw[k], acc[4 * k + 0]);
    acc[4 * k + 1] = dp2a_su<0>(w[k].y, xw[k], acc[4 * k + 1]);
    acc[4 * k + 2] = dp2a_su<1>(w[k].z, xw[k], acc[4 * k + 2]);
    acc[4 * k + 3] = dp2a_su<1>(w[k].w, xw[k], acc[4 * k + 3]);
  }
}

// KH, KW > 0: window known at compile time, both tap loops unroll and the loads of all taps can be in
// flight together (the kernel is latency-bound otherwise); 0: any window.
template <int KH, int KW, bool XS>
__global__ void __launch_bounds__(256, 2) depthwise_q16_kernel(const uint8_t* __restrict__ x, DwParams p, uint8_t* __restrict__ y) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ uint4 dw_smem[];               // [taps][slab / 4] groups of four weight words
  const ConvGeom& g = p.g;
  const int kh = KH ? KH : g.kh, kw = KW ? KW : g.kw;
  const int taps = kh * kw;
  const int c_slab = blockIdx.y * p.slab;
  const int slab_ch = min(p.slab, g.Ocp - c_slab);   // multiple of 16
  const int quads = p.slab >> 2;
  for (int i = threadIdx.x; i < taps * quads; i += blockDim.x) {
    const int t = i / quads, q = i - t * quads;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (4 * q < slab_ch) v = *reinterpret_cast<const uint4*>(p.wtab + static_cast<size_t>(t) * g.Ocp + c_slab + 4 * q);
    dw_smem[i] = v;
  }
  __syncthreads();
  const int chunks = p.slab >> 4;                   // thread mapping is the same in every slab
  const int pairs_w = (g.Wo + 1) >> 1;
  const long long total_pairs = static_cast<long long>(g.N) * g.Ho * pairs_w;
  const int pairs_per_block = blockDim.x / chunks;
  const int chunk = threadIdx.x % chunks;
  const int local_pair = threadIdx.x / chunks;
  if (local_pair >= pairs_per_block || 16 * chunk >= slab_ch) return;
  const long long pair = static_cast<long long>(blockIdx.x) * pairs_per_block + local_pair;
  if (pair >= total_pairs) return;
  const int pw = static_cast<int>(pair % pairs_w);
  const long long t2 = pair / pairs_w;
  const int ho = static_cast<int>(t2 % g.Ho);
  const int n = static_cast<int>(t2 / g.Ho);
  const int wo0 = 2 * pw;
  const bool second = wo0 + 1 < g.Wo;
  const int c0 = c_slab + 16 * chunk;
  const uint4 zx4 = make_uint4(p.zx_word, p.zx_word, p.zx_word, p.zx_word);
  int acc0[16], acc1[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) { acc0[i] = 0; acc1[i] = 0; }
  const uint8_t* img = x + static_cast<size_t>(n) * g.H * g.W * g.Cp + c0;
#pragma unroll
  for (int ky = 0; ky < kh; ++ky) {
    const int hi = ho * g.sy - g.pt + ky * g.dy;
    const bool row_ok = hi >= 0 && hi < g.H;
    const uint8_t* rowp = img + static_cast<size_t>(row_ok ? hi : 0) * g.W * g.Cp;
#pragma unroll
    for (int kx = 0; kx < kw; ++kx) {
      const uint4* wq = dw_smem + (ky * kw + kx) * quads + 4 * chunk;
      const uint4 w[4] = {wq[0], wq[1], wq[2], wq[3]};
      const int wi0 = wo0 * g.sx - g.pl + kx * g.dx, wi1 = wi0 + g.sx;
      uint4 xa = zx4, xb = zx4;
      if (row_ok && wi0 >= 0 && wi0 < g.W) {
        xa = __ldg(reinterpret_cast<const uint4*>(rowp + static_cast<size_t>(wi0) * g.Cp));
        if (XS) { xa.x ^= 0x80808080u; xa.y ^= 0x80808080u; xa.z ^= 0x80808080u; xa.w ^= 0x80808080u; }
      }
      if (second && row_ok && wi1 >= 0 && wi1 < g.W) {
        xb = __ldg(reinterpret_cast<const uint4*>(rowp + static_cast<size_t>(wi1) * g.Cp));
        if (XS) { xb.x ^= 0x80808080u; xb.y ^= 0x80808080u; xb.z ^= 0x80808080u; xb.w ^= 0x80808080u; }
      }
      dw_mac16(acc0, xa, w);
      dw_mac16(acc1, xb, w);
    }
  }
  const RequantConsts rc = make_requant_consts(p.out, p.exact_only);
  uint8_t* out = y + ((static_cast<size_t>(n) * g.Ho + ho) * g.Wo + wo0) * g.Ocp + c0;
  *reinterpret_cast<uint4*>(out) = requant_chunk16<false>(acc0, p.bias_full + c0, p.acc_scale + c0, rc, 0, nullptr);
  if (second) *reinterpret_cast<uint4*>(out + g.Ocp) = requant_chunk16<false>(acc1, p.bias_full + c0, p.acc_scale + c0, rc, 0, nullptr);
}

// The same computation with the input staged in shared memory: a block owns a slab of CK = 1, 2 or 4
// 16-channel chunks (whichever wastes fewest channels) of a TH x TW tile of output pixels, TW = 8 or
// 16 and TH = 256 / (8 * CK), copies the input patch it needs (halo included, the zero point where the
// patch leaves the image, signed bytes already biased) with independent 128-bit loads that are all
// in flight together, and then computes from shared memory with no bounds checks.  Several blocks
// per SM overlap one block's copy with another's arithmetic.  A thread owns one chunk of pixel
// (row q / 8, column q % 8) of the tile and, when TW = 16, of the pixel 8 columns to the right.
template <int KH, int KW, bool XS>
__global__ void __launch_bounds__(256, (KH == 3 ? 3 : 2)) depthwise_q16s_kernel(const uint8_t* __restrict__ x, DwParams p, int tw_shift,
                                                                int ck_shift, int IH, int IW, uint8_t* __restrict__ y) {
  extern __shared__ uint4 dw_smem[];               // [taps][4 * CK] weight quads, then [IH][IW][CK] input chunks
  const ConvGeom& g = p.g;
  const int kh = KH ? KH : g.kh, kw = KW ? KW : g.kw;
  const int taps = kh * kw;
  const int TW = 1 << tw_shift, CK = 1 << ck_shift;
  const int TH = 32 >> ck_shift;                    // 256 threads = CK chunks x 8 columns x TH rows
  const int tiles_w = (g.Wo + TW - 1) >> tw_shift, tiles_h = (g.Ho + TH - 1) / TH;
  int tile = blockIdx.x;
  const int tile_w = tile % tiles_w; tile /= tiles_w;
  const int tile_h = tile % tiles_h;
  const int n = tile / tiles_h;
  const int c_slab = blockIdx.y * 16 * CK;
  const int slab_chunks = min(16 * CK, g.Ocp - c_slab) >> 4;
  const int ho0 = tile_h * TH, wo0 = tile_w * TW;
  const int hi0 = ho0 * g.sy - g.pt, wi0 = wo0 * g.sx - g.pl;
  uint4* wsm = dw_smem;
  uint4* xsm = dw_smem + taps * 4 * CK;
  pdl_trigger();
  for (int i = threadIdx.x; i < taps * 4 * CK; i += 256) {
    const int t = i >> (2 + ck_shift), q = i & (4 * CK - 1);
    uint4 v = make_uint4(0, 0, 0, 0);
    if ((q >> 2) < slab_chunks) v = *reinterpret_cast<const uint4*>(p.wtab + static_cast<size_t>(t) * g.Ocp + c_slab + 4 * q);
    wsm[i] = v;
  }
  pdl_wait();   // weights are constants; the input is the first thing another kernel produced
  const int chunk = threadIdx.x & (CK - 1);
  {
    const uint4 zx4 = make_uint4(p.zx_word, p.zx_word, p.zx_word, p.zx_word);
    const uint8_t* img = x + static_cast<size_t>(n) * g.H * g.W * g.Cp + c_slab;
    const int units = IH * IW * CK;
    const int ppi = 256 >> ck_shift;               // staged pixels per step
    int pix = threadIdx.x >> ck_shift;
    int ih = pix / IW, iw = pix - ih * IW;
    const int step_h = ppi / IW, step_w = ppi - step_h * IW;
#pragma unroll 4
    for (int u = threadIdx.x; u < units; u += 256) {
      const int hi = hi0 + ih, wi = wi0 + iw;
      uint4 v = zx4;
      if (chunk < slab_chunks && hi >= 0 && hi < g.H && wi >= 0 && wi < g.W) {
        v = __ldg(reinterpret_cast<const uint4*>(img + (static_cast<size_t>(hi) * g.W + wi) * g.Cp + 16 * chunk));
        if (XS) { v.x ^= 0x80808080u; v.y ^= 0x80808080u; v.z ^= 0x80808080u; v.w ^= 0x80808080u; }
      }
      xsm[u] = v;
      ih += step_h; iw += step_w;
      if (iw >= IW) { iw -= IW; ++ih; }
    }
  }
  __syncthreads();
  if (chunk >= slab_chunks) return;
  const int q = threadIdx.x >> ck_shift;           // 0 .. 8*TH-1
  const int tr = q >> 3, tc = q & 7;
  const bool two = TW == 16;
  int acc0[16], acc1[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) { acc0[i] = 0; acc1[i] = 0; }
  const uint4* xrow0 = xsm + (((tr * g.sy) * IW + tc * g.sx) << ck_shift) + chunk;
  const int second_off = (8 * g.sx) << ck_shift;
#pragma unroll
  for (int ky = 0; ky < kh; ++ky) {
#pragma unroll
    for (int kx = 0; kx < kw; ++kx) {
      const uint4* wq = wsm + (((ky * kw + kx) << ck_shift) + chunk) * 4;
      const uint4 w[4] = {wq[0], wq[1], wq[2], wq[3]};
      const uint4* xp = xrow0 + ((ky * g.dy * IW + kx * g.dx) << ck_shift);
      dw_mac16(acc0, xp[0], w);
      if (two) dw_mac16(acc1, xp[second_off], w);
    }
  }
  const RequantConsts rc = make_requant_consts(p.out, p.exact_only);
  const int ho = ho0 + tr, wo = wo0 + tc, c0 = c_slab + 16 * chunk;
  if (ho >= g.Ho) return;
  uint8_t* out = y + ((static_cast<size_t>(n) * g.Ho + ho) * g.Wo + wo) * g.Ocp + c0;
  if (wo < g.Wo) *reinterpret_cast<uint4*>(out) = requant_chunk16<false>(acc0, p.bias_full + c0, p.acc_scale + c0, rc, 0, nullptr);
  if (two && wo + 8 < g.Wo)
    *reinterpret_cast<uint4*>(out + 8 * g.Ocp) = requant_chunk16<false>(acc1, p.bias_full + c0, p.acc_scale + c0, rc, 0, nullptr);
}

// The 3x3 form for strides 1 and 2: a thread owns FOUR channels (one 32-bit word of a pixel) of a strip of eight
// horizontally adjacent output pixels.  Its 36 weight words and its bias / scale live in registers, every input word of the strip's
// three rows is read from shared memory once (10 or 17 32-bit loads per row) and feeds up to three outputs, so
// the arithmetic runs at 9.4 or 5.6 multiply-accumulates per shared-memory load instead of 5.3 per 128-bit load,
// and a warp's load is one or two 128-byte wavefronts instead of four.  (The 16-channel form above spends more
// shared-memory cycles than issue slots.)  A block's 256 threads are CW = 4, 8 or 16 channel words x 64, 32 or 16
// strips, the strips laid out as NI images x SEG strips per row x TH rows (powers of two, chosen by the launcher).
// Consecutive strips of a warp are consecutive rows; the patch's row pitch is chosen so that their words fall in
// different banks.
#ifndef B2VX_DW_BLOCKS
#define B2VX_DW_BLOCKS 4   // resident blocks per SM the strip kernel is compiled for (64 registers per thread)
#endif
struct DwStripGeom {
  int ck_shift;    // 16-channel chunks per slab: 1 << ck_shift
  int seg_shift;   // strips per tile row
  int th_shift;    // tile rows
  int ni_shift;    // images per tile (more than one only when a tile covers a whole image)
  int IH, IW;      // input patch of one image
  int pitch;       // bytes between patch rows
  int tiles_w;     // tiles per output row
  int iw_recip;    // 65536 / IW + 1: (pixel * iw_recip) >> 16 = pixel / IW for pixel < 256
  int step_h, step_w;   // (256 / CK) / IW and (256 / CK) % IW: how a thread's patch pixel advances per staging round
  int tiles_h, n_groups;   // pipelined form: tile rows per image, groups of NI images
  int patch_bytes;         // pipelined form: NI * IH * pitch rounded up to 128
};

__device__ __forceinline__ uint4 requant16_packed(f32x2 (&real)[8], const RequantConsts& rc) {
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
  asm volatile("" : "+r"(differ));   // keeps the one test per sixteen values (see requant_chunk16)
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

// Four pixels x four channels: acc[4 * pixel + channel] already holds the folded bias; one word per pixel comes back.
// The arithmetic is requant_chunk16's (same two-sided rounding, same exact path for the rare disagreement).
__device__ __forceinline__ uint4 requant_4x4(const int (&acc)[16], const float4& s4, const RequantConsts& rc) {
  f32x2 real[8];
  const f32x2 s01 = f2_pack(s4.x, s4.y), s23 = f2_pack(s4.z, s4.w);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    real[2 * j] = f2_mul(f2_pack(__int2float_rn(acc[4 * j + 0]), __int2float_rn(acc[4 * j + 1])), s01);
    real[2 * j + 1] = f2_mul(f2_pack(__int2float_rn(acc[4 * j + 2]), __int2float_rn(acc[4 * j + 3])), s23);
  }
  return requant16_packed(real, rc);
}

// Grid: x = tile column + tiles_w * tile row, y = group of NI images, z = channel slab.
template <int S, bool XS, int CKS>
__global__ void __launch_bounds__(256, B2VX_DW_BLOCKS) depthwise_strip_kernel(const uint8_t* __restrict__ x, DwParams p, DwStripGeom t,
                                                                 uint8_t* __restrict__ y) {
  extern __shared__ uint4 dw_smem[];               // [NI][IH] patch rows of t.pitch bytes: [IW][CK] 16-channel chunks
  const ConvGeom& g = p.g;
  constexpr int CK = 1 << CKS, CW = 4 * CK, PXB = 16 * CK;   // chunks, words and bytes of a pixel of the slab
  const int TH = 1 << t.th_shift, SEG = 1 << t.seg_shift, NI = 1 << t.ni_shift;
  const unsigned tile_h = blockIdx.x / static_cast<unsigned>(t.tiles_w), tile_w = blockIdx.x - tile_h * t.tiles_w;
  const int n0 = blockIdx.y << t.ni_shift;
  const int c_slab = blockIdx.z * PXB;
  const int slab_chunks = min(PXB, g.Ocp - c_slab) >> 4;
  const int ho0 = tile_h << t.th_shift, wo0 = tile_w << (3 + t.seg_shift);
  const int hi0 = ho0 * S - g.pt, wi0 = wo0 * S - g.pl;
  pdl_trigger();
  const int cw = threadIdx.x & (CW - 1);
  const int strip = threadIdx.x >> (2 + CKS);
  const bool active = (cw >> 2) < slab_chunks;
  pdl_wait();   // the input is the first thing another kernel produced
  uint8_t* const xsm = reinterpret_cast<uint8_t*>(dw_smem);
  {
    const uint4 zx4 = make_uint4(p.zx_word, p.zx_word, p.zx_word, p.zx_word);
    const int chunk = threadIdx.x & (CK - 1);
    const int units = t.IH * t.IW * CK;
    const unsigned pix0 = threadIdx.x >> CKS;
    const int ih0 = static_cast<int>((pix0 * static_cast<unsigned>(t.iw_recip)) >> 16);   // pix0 / IW (pix0 < 256)
    const int iw0 = static_cast<int>(pix0) - ih0 * t.IW;
    const bool chunk_ok = chunk < slab_chunks;
    const uint32_t img_bytes = static_cast<uint32_t>(g.H) * g.W * g.Cp;
    for (int ni = 0; ni < NI; ++ni) {
      const bool img_ok = chunk_ok && n0 + ni < g.N;
      const uint8_t* img = x + static_cast<size_t>(img_ok ? n0 + ni : 0) * img_bytes + c_slab + 16 * chunk;
      uint8_t* dst = xsm + ni * t.IH * t.pitch + 16 * chunk;
      int ih = ih0, iw = iw0;
#pragma unroll 4
      for (int u = threadIdx.x; u < units; u += 256) {
        const int hi = hi0 + ih, wi = wi0 + iw;
        uint4 v = zx4;
        if (img_ok && static_cast<unsigned>(hi) < static_cast<unsigned>(g.H) && static_cast<unsigned>(wi) < static_cast<unsigned>(g.W)) {
          v = __ldg(reinterpret_cast<const uint4*>(img + static_cast<uint32_t>(hi * g.W + wi) * static_cast<uint32_t>(g.Cp)));
          if (XS) { v.x ^= 0x80808080u; v.y ^= 0x80808080u; v.z ^= 0x80808080u; v.w ^= 0x80808080u; }
        }
        *reinterpret_cast<uint4*>(dst + ih * t.pitch + iw * PXB) = v;
        ih += t.step_h; iw += t.step_w;
        if (iw >= t.IW) { iw -= t.IW; ++ih; }
      }
    }
  }
  // this thread's constants, requested while the block's copies land (they stay in L1/L2 between blocks);
  // threads past the last channel read the last words and never use them
  uint4 wp[3], ws[3];                             // per window column: rows 0 and 1 as a pair, row 2 alone
  const int c0 = min(c_slab + 4 * cw, g.Ocp - 4);
#pragma unroll
  for (int k = 0; k < 3; ++k) {
    wp[k] = __ldg(reinterpret_cast<const uint4*>(p.wtab_v + static_cast<size_t>(k) * g.Ocp + c0));
    ws[k] = __ldg(reinterpret_cast<const uint4*>(p.wtab_v + static_cast<size_t>(3 + k) * g.Ocp + c0));
  }
  const int4 b4 = __ldg(reinterpret_cast<const int4*>(p.bias_full + c0));
  const float4 s4 = __ldg(reinterpret_cast<const float4*>(p.acc_scale + c0));
  __syncthreads();
  if (!active) return;
  const int r = strip & (TH - 1);
  const int sgm = (strip >> t.th_shift) & (SEG - 1);
  const int ni = strip >> (t.th_shift + t.seg_shift);
  const int n = n0 + ni, ho = ho0 + r, wo = wo0 + 8 * sgm;
  if (n >= g.N || ho >= g.Ho || wo >= g.Wo) return;
  int acc[2][16];
  const uint8_t* rowp = xsm + (ni * t.IH + r * S) * t.pitch + (8 * sgm * S) * PXB + 4 * cw;
  const uint8_t* rowp1 = rowp + t.pitch;
  const uint8_t* rowp2 = rowp1 + t.pitch;
#pragma unroll
  for (int ic = 0; ic < 7 * S + 3; ++ic) {
    const uint32_t x0 = *reinterpret_cast<const uint32_t*>(rowp + ic * PXB);
    const uint32_t x1 = *reinterpret_cast<const uint32_t*>(rowp1 + ic * PXB);
    const uint32_t x2 = *reinterpret_cast<const uint32_t*>(rowp2 + ic * PXB);
    // rows 0 and 1 of this column, byte-interleaved: [r0.c0 r1.c0 r0.c1 r1.c1] and [r0.c2 r1.c2 r0.c3 r1.c3], so that one
    // dp2a against the pair (w[0][kx], w[1][kx]) of a channel does two multiply-accumulates
    const uint32_t p01 = __byte_perm(x0, x1, 0x5140), p23 = __byte_perm(x0, x1, 0x7362);
#pragma unroll
    for (int kx = 0; kx < 3; ++kx) {
      if (ic - kx >= 0 && (ic - kx) % S == 0 && (ic - kx) / S < 8) {
        const int j = (ic - kx) / S;
        int* a = &acc[j >> 2][4 * (j & 3)];
        const bool first = kx == 0;   // an output's first product starts from the folded bias
        a[0] = dp2a_su<0>(wp[kx].x, p01, first ? b4.x : a[0]);
        a[1] = dp2a_su<1>(wp[kx].y, p01, first ? b4.y : a[1]);
        a[2] = dp2a_su<0>(wp[kx].z, p23, first ? b4.z : a[2]);
        a[3] = dp2a_su<1>(wp[kx].w, p23, first ? b4.w : a[3]);
        a[0] = dp2a_su<0>(ws[kx].x, x2, a[0]);
        a[1] = dp2a_su<0>(ws[kx].y, x2, a[1]);
        a[2] = dp2a_su<1>(ws[kx].z, x2, a[2]);
        a[3] = dp2a_su<1>(ws[kx].w, x2, a[3]);
      }
    }
  }
  const RequantConsts rc = make_requant_consts(p.out, p.exact_only);
  uint8_t* out = y + ((static_cast<size_t>(n) * g.Ho + ho) * g.Wo + wo) * g.Ocp + c_slab + 4 * cw;
  const uint4 q0 = requant_4x4(acc[0], s4, rc);
  const uint4 q1 = requant_4x4(acc[1], s4, rc);
  const uint32_t q[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
  for (int j = 0; j < 8; ++j)
    if (wo + j < g.Wo) *reinterpret_cast<uint32_t*>(out + j * g.Ocp) = q[j];
}

// The strip form as a pipeline: a block stays on one channel slab, keeps its weights in registers and walks over
// that slab's tiles (grid x = blocks per slab, z = slab).  The patch of the next tile is copied with 16-byte
// asynchronous copies into the second of two buffers while the block computes the current one, so the copy
// latency that a one-tile block pays in full is hidden.  Signed input bytes arrive as they are and are biased by
// 128 when they are read from shared memory.
__device__ __forceinline__ void cp_async16(uint32_t dst_smem, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_smem), "l"(src) : "memory");
}

template <int S, bool XS, int CKS>
__global__ void __launch_bounds__(256, 3) depthwise_strip_pipe_kernel(const uint8_t* __restrict__ x, DwParams p, DwStripGeom t,
                                                                      uint8_t* __restrict__ y) {
  extern __shared__ uint4 dw_smem[];               // two patches of t.patch_bytes
  const ConvGeom& g = p.g;
  constexpr int CK = 1 << CKS, CW = 4 * CK, PXB = 16 * CK;
  const int TH = 1 << t.th_shift, SEG = 1 << t.seg_shift, NI = 1 << t.ni_shift;
  const int c_slab = blockIdx.z * PXB;
  const int slab_chunks = min(PXB, g.Ocp - c_slab) >> 4;
  pdl_trigger();
  const int cw = threadIdx.x & (CW - 1);
  const int strip = threadIdx.x >> (2 + CKS);
  const bool active = (cw >> 2) < slab_chunks;
  const int r = strip & (TH - 1);
  const int sgm = (strip >> t.th_shift) & (SEG - 1);
  const int ni_s = strip >> (t.th_shift + t.seg_shift);
  const uint32_t row_off = (ni_s * t.IH + r * S) * t.pitch + (8 * sgm * S) * PXB + 4 * cw;
  // staging role of this thread
  const int chunk = threadIdx.x & (CK - 1);
  const int units = t.IH * t.IW * CK;
  const unsigned pix0 = threadIdx.x >> CKS;
  const int ih0 = static_cast<int>((pix0 * static_cast<unsigned>(t.iw_recip)) >> 16);
  const int iw0 = static_cast<int>(pix0) - ih0 * t.IW;
  const bool chunk_ok = chunk < slab_chunks;
  const uint32_t img_bytes = static_cast<uint32_t>(g.H) * g.W * g.Cp;
  const uint32_t zraw = p.zx_word ^ p.x_flip;       // the zero point as the input stores it
  const uint4 zx4 = make_uint4(zraw, zraw, zraw, zraw);
  const uint32_t smem0 = static_cast<uint32_t>(__cvta_generic_to_shared(dw_smem));
  uint8_t* const xsm = reinterpret_cast<uint8_t*>(dw_smem);
  const unsigned tiles_xy = static_cast<unsigned>(t.tiles_w) * t.tiles_h;
  const unsigned T = tiles_xy * t.n_groups;

  auto locate = [&](unsigned L, int& n0, int& ho0, int& wo0) {
    const unsigned ng = L / tiles_xy, txy = L - ng * tiles_xy;
    const unsigned th = txy / static_cast<unsigned>(t.tiles_w), tw = txy - th * t.tiles_w;
    n0 = ng << t.ni_shift;
    ho0 = th << t.th_shift;
    wo0 = tw << (3 + t.seg_shift);
  };
  auto stage = [&](unsigned L, uint32_t buf_off) {
    int n0, ho0, wo0;
    locate(L, n0, ho0, wo0);
    const int hi0 = ho0 * S - g.pt, wi0 = wo0 * S - g.pl;
    for (int ni = 0; ni < NI; ++ni) {
      const bool img_ok = chunk_ok && n0 + ni < g.N;
      const uint8_t* img = x + static_cast<size_t>(img_ok ? n0 + ni : 0) * img_bytes + c_slab + 16 * chunk;
      const uint32_t dst = buf_off + ni * t.IH * t.pitch + 16 * chunk;
      int ih = ih0, iw = iw0;
#pragma unroll 2
      for (int u = threadIdx.x; u < units; u += 256) {
        const int hi = hi0 + ih, wi = wi0 + iw;
        const uint32_t d = dst + ih * t.pitch + iw * PXB;
        if (img_ok && static_cast<unsigned>(hi) < static_cast<unsigned>(g.H) && static_cast<unsigned>(wi) < static_cast<unsigned>(g.W))
          cp_async16(smem0 + d, img + static_cast<uint32_t>(hi * g.W + wi) * static_cast<uint32_t>(g.Cp));
        else
          *reinterpret_cast<uint4*>(xsm + d) = zx4;
        ih += t.step_h; iw += t.step_w;
        if (iw >= t.IW) { iw -= t.IW; ++ih; }
      }
    }
  };

  pdl_wait();   // the input is the first thing another kernel produced
  unsigned L = blockIdx.x;
  if (L < T) stage(L, 0u);
  asm volatile("cp.async.commit_group;" ::: "memory");
  uint4 wp[3], ws[3];
  const int c0 = min(c_slab + 4 * cw, g.Ocp - 4);
#pragma unroll
  for (int k = 0; k < 3; ++k) {
    wp[k] = __ldg(reinterpret_cast<const uint4*>(p.wtab_v + static_cast<size_t>(k) * g.Ocp + c0));
    ws[k] = __ldg(reinterpret_cast<const uint4*>(p.wtab_v + static_cast<size_t>(3 + k) * g.Ocp + c0));
  }
  const int4 b4 = __ldg(reinterpret_cast<const int4*>(p.bias_full + c0));
  const float4 s4 = __ldg(reinterpret_cast<const float4*>(p.acc_scale + c0));
  const RequantConsts rc = make_requant_consts(p.out, p.exact_only);
  uint32_t cur = 0u, nxt = static_cast<uint32_t>(t.patch_bytes);
  for (; L < T; L += gridDim.x) {
    if (L + gridDim.x < T) stage(L + gridDim.x, nxt);     // that buffer was read two tiles ago; a barrier has passed since
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 1;" ::: "memory");  // this thread's copies of the current tile have landed
    __syncthreads();                                       // ... and everybody else's
    int n0, ho0, wo0;
    locate(L, n0, ho0, wo0);
    const int n = n0 + ni_s, ho = ho0 + r, wo = wo0 + 8 * sgm;
    if (active && n < g.N && ho < g.Ho && wo < g.Wo) {
      int acc[2][16];
      const uint8_t* rowp = xsm + cur + row_off;
      const uint8_t* rowp1 = rowp + t.pitch;
      const uint8_t* rowp2 = rowp1 + t.pitch;
#pragma unroll
      for (int ic = 0; ic < 7 * S + 3; ++ic) {
        uint32_t x0 = *reinterpret_cast<const uint32_t*>(rowp + ic * PXB);
        uint32_t x1 = *reinterpret_cast<const uint32_t*>(rowp1 + ic * PXB);
        uint32_t x2 = *reinterpret_cast<const uint32_t*>(rowp2 + ic * PXB);
        if (XS) { x0 ^= 0x80808080u; x1 ^= 0x80808080u; x2 ^= 0x80808080u; }
        const uint32_t p01 = __byte_perm(x0, x1, 0x5140), p23 = __byte_perm(x0, x1, 0x7362);
#pragma unroll
        for (int kx = 0; kx < 3; ++kx) {
          if (ic - kx >= 0 && (ic - kx) % S == 0 && (ic - kx) / S < 8) {
            const int j = (ic - kx) / S;
            int* a = &acc[j >> 2][4 * (j & 3)];
            const bool first = kx == 0;
            a[0] = dp2a_su<0>(wp[kx].x, p01, first ? b4.x : a[0]);
            a[1] = dp2a_su<1>(wp[kx].y, p01, first ? b4.y : a[1]);
            a[2] = dp2a_su<0>(wp[kx].z, p23, first ? b4.z : a[2]);
            a[3] = dp2a_su<1>(wp[kx].w, p23, first ? b4.w : a[3]);
            a[0] = dp2a_su<0>(ws[kx].x, x2, a[0]);
            a[1] = dp2a_su<0>(ws[kx].y, x2, a[1]);
            a[2] = dp2a_su<1>(ws[kx].z, x2, a[2]);
            a[3] = dp2a_su<1>(ws[kx].w, x2, a[3]);
          }
        }
      }
      uint8_t* out = y + ((static_cast<size_t>(n) * g.Ho + ho) * g.Wo + wo) * g.Ocp + c_slab + 4 * cw;
      const uint4 q0 = requant_4x4(acc[0], s4, rc);
      const uint4 q1 = requant_4x4(acc[1], s4, rc);
      const uint32_t q[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (wo + j < g.Wo) *reinterpret_cast<uint32_t*>(out + j * g.Ocp) = q[j];
    }
    __syncthreads();                                       // the current buffer may be overwritten from here on
    const uint32_t tmp = cur; cur = nxt; nxt = tmp;
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
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
  float sq[4] = {0.0f, 0.0f, 0.0f, 0.0f};   // type 2 (L2): squares of the real values, added in tap order
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
        if (type == 2) {
          const float real = __fmul_rn(__int2float_rn(v - in_zp), in_scale);
          sq[j] = __fadd_rn(sq[j], __fmul_rn(real, real));
        }
      }
    }
  }
  const float div = type == 1 ? static_cast<float>(g.kw * g.kh) : static_cast<float>(count);
  uint32_t word = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    int q;
    if (type == 2) {
      q = requant(count ? __fsqrt_rn(__fdiv_rn(sq[j], __int2float_rn(count))) : 0.0f, out);
    } else if (type == 0) {
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

// The same pooling with 16 channels (one 128-bit access) per thread and byte-SIMD arithmetic: max with
// __vmaxu4/__vmaxs4, sums as packed 16-bit pairs (so the window may hold at most 256 taps).
// K = 2 or 3: a K x K window known at compile time, so that all its loads are in flight together; 0: any window.
template <bool XS, int K>
__global__ void __launch_bounds__(256) pool_q16_kernel(const uint8_t* __restrict__ x, int type, float in_scale, int in_zp,
                                                       int same_quant, ConvGeom g, OutQuant out, uint8_t* __restrict__ y) {
  pdl_wait();
  pdl_trigger();
  const int chunks = g.Cp >> 4;
  const long long total = static_cast<long long>(g.N) * g.Ho * g.Wo * chunks;
  long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i >= total) return;
  const int ch = static_cast<int>(i % chunks);
  const long long p = i / chunks;
  const int wo = static_cast<int>(p % g.Wo);
  const long long t = p / g.Wo;
  const int ho = static_cast<int>(t % g.Ho);
  const int n = static_cast<int>(t / g.Ho);
  const int h_lo = max(0, ho * g.sy - g.pt), h_hi = min(g.H, ho * g.sy - g.pt + g.kh);
  const int w_lo = max(0, wo * g.sx - g.pl), w_hi = min(g.W, wo * g.sx - g.pl + g.kw);
  const int count = max(0, h_hi - h_lo) * max(0, w_hi - w_lo);
  const uint32_t flip = XS ? 0x80808080u : 0u;       // signed bytes are handled as value + 128
  uint32_t mx[4] = {0u, 0u, 0u, 0u};                 // unsigned max of the biased bytes
  uint32_t even[4] = {0u, 0u, 0u, 0u}, odd[4] = {0u, 0u, 0u, 0u};   // 16-bit sums of bytes 0,2 and 1,3 of each word
  auto take = [&](const uint4& v) {
    const uint32_t w4[4] = {v.x ^ flip, v.y ^ flip, v.z ^ flip, v.w ^ flip};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      if (type == 0) {
        mx[k] = __vmaxu4(mx[k], w4[k]);
      } else {
        even[k] += w4[k] & 0x00FF00FFu;
        odd[k] += (w4[k] >> 8) & 0x00FF00FFu;
      }
    }
  };
  if (K > 0) {
    const uint8_t* img = x + static_cast<size_t>(n) * g.H * g.W * g.Cp + ch * 16;
    constexpr int KK = K > 0 ? K * K : 1;
    uint4 v[KK];
    bool ok[KK];
#pragma unroll
    for (int ky = 0; ky < K; ++ky) {
#pragma unroll
      for (int kx = 0; kx < K; ++kx) {
        const int hi = ho * g.sy - g.pt + ky, wi = wo * g.sx - g.pl + kx;
        ok[ky * K + kx] = hi >= 0 && hi < g.H && wi >= 0 && wi < g.W;
        v[ky * K + kx] = make_uint4(0, 0, 0, 0);
        if (ok[ky * K + kx]) v[ky * K + kx] = __ldg(reinterpret_cast<const uint4*>(img + (static_cast<size_t>(hi) * g.W + wi) * g.Cp));
      }
    }
#pragma unroll
    for (int t9 = 0; t9 < K * K; ++t9)
      if (ok[t9]) take(v[t9]);
  } else {
    for (int hi = h_lo; hi < h_hi; ++hi) {
      const uint8_t* rowp = x + ((static_cast<size_t>(n) * g.H + hi) * g.W) * g.Cp + ch * 16;
      for (int wi = w_lo; wi < w_hi; ++wi) take(*reinterpret_cast<const uint4*>(rowp + static_cast<size_t>(wi) * g.Cp));
    }
  }
  const int bias = XS ? 128 : 0;
  const float div = type == 1 ? static_cast<float>(g.kw * g.kh) : static_cast<float>(count);
  uint32_t o[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    if (type == 0 && same_quant) {
      o[k] = count ? (mx[k] ^ flip) : (static_cast<uint32_t>(in_zp & 0xFF) * 0x01010101u);
      continue;
    }
    uint32_t word = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int q;
      if (type == 0) {
        q = count ? static_cast<int>((mx[k] >> (8 * j)) & 0xFF) - bias : in_zp;
        q = requant(__fmul_rn(__fsub_rn(__int2float_rn(q), __int2float_rn(in_zp)), in_scale), out);
      } else {
        const uint32_t pair = (j & 1) ? odd[k] : even[k];
        const int sum = static_cast<int>((pair >> (16 * (j >> 1))) & 0xFFFF) - count * (in_zp + bias);
        const float avg = count ? __fdiv_rn(__fmul_rn(__int2float_rn(sum), in_scale), div) : 0.0f;
        q = requant(avg, out);
      }
      word |= static_cast<uint32_t>(q & 0xFF) << (8 * j);
    }
    o[k] = word;
  }
  *reinterpret_cast<uint4*>(y + static_cast<size_t>(p) * g.Cp + ch * 16) = make_uint4(o[0], o[1], o[2], o[3]);
}

// Max pooling whose output keeps the input's quantization, K x K window with stride S (3x3 / 2 and 2x2 / 2 are the
// common ones): a thread produces a 2 x 2 block of outputs for 16 channels from the (K + S) x (K + S) input patch the
// four windows share, row by row: one horizontal maximum per output column and input row, handed to the output rows whose
// window contains that row.  25 loads and about 130 byte-SIMD maxima for four 3x3 / 2 outputs, where one output per thread
// costs 9 loads and 36 maxima each.  Taps outside the image are skipped by clamping their coordinates into the window's
// valid part (a repeated tap does not change a maximum; every window of an existing output has a valid tap).
template <bool XS, int K, int S>
__global__ void __launch_bounds__(256) pool_max2x2_kernel(const uint8_t* __restrict__ x, ConvGeom g, uint8_t* __restrict__ y) {
  pdl_wait();
  pdl_trigger();
  constexpr int P = K + S;   // patch extent
  const int chunks = g.Cp >> 4;
  const int wo2n = (g.Wo + 1) >> 1, ho2n = (g.Ho + 1) >> 1;
  const long long total = static_cast<long long>(g.N) * ho2n * wo2n * chunks;
  const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i >= total) return;
  const int ch = static_cast<int>(i % chunks);
  const long long p = i / chunks;
  const int wo = static_cast<int>(p % wo2n) * 2;
  const long long t = p / wo2n;
  const int ho = static_cast<int>(t % ho2n) * 2;
  const int n = static_cast<int>(t / ho2n);
  const int w0 = wo * S - g.pl, h0 = ho * S - g.pt;
  const bool has_w1 = wo + 1 < g.Wo, has_h1 = ho + 1 < g.Ho;
  // columns of the patch, each clamped into the valid part of the window(s) it belongs to
  int col[P];
#pragma unroll
  for (int c = 0; c < P; ++c) {
    // window 0 holds patch columns [0, K), window 1 [S, S + K); a column of window 1 only (c >= K) is clamped into window
    // 1's range, which starts at w0 + S
    const int lo = c >= K ? max(w0 + S, 0) : max(w0, 0);
    col[c] = min(max(w0 + c, lo), g.W - 1);
  }
  const uint32_t flip = XS ? 0x80808080u : 0u;
  const uint8_t* img = x + static_cast<size_t>(n) * g.H * g.W * g.Cp + ch * 16;
  uint32_t o[2][2][4];   // [output row][output column][word]; bytes biased to unsigned
#pragma unroll
  for (int a = 0; a < 2; ++a)
#pragma unroll
    for (int b = 0; b < 2; ++b)
#pragma unroll
      for (int k = 0; k < 4; ++k) o[a][b][k] = 0u;
#pragma unroll
  for (int r = 0; r < P; ++r) {
    const int lo = r >= K ? max(h0 + S, 0) : max(h0, 0);
    const int hr = min(max(h0 + r, lo), g.H - 1);
    const uint8_t* rowp = img + static_cast<size_t>(hr) * g.W * g.Cp;
    uint4 v[P];
#pragma unroll
    for (int c = 0; c < P; ++c) v[c] = __ldg(reinterpret_cast<const uint4*>(rowp + static_cast<size_t>(col[c]) * g.Cp));
    uint32_t m[2][4];
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      m[b][0] = m[b][1] = m[b][2] = m[b][3] = 0u;
#pragma unroll
      for (int c = b * S; c < b * S + K; ++c) {
        m[b][0] = __vmaxu4(m[b][0], v[c].x ^ flip);
        m[b][1] = __vmaxu4(m[b][1], v[c].y ^ flip);
        m[b][2] = __vmaxu4(m[b][2], v[c].z ^ flip);
        m[b][3] = __vmaxu4(m[b][3], v[c].w ^ flip);
      }
    }
#pragma unroll
    for (int a = 0; a < 2; ++a) {
      if (r >= a * S && r < a * S + K) {   // (known at compile time: the loops are unrolled)
#pragma unroll
        for (int b = 0; b < 2; ++b)
#pragma unroll
          for (int k = 0; k < 4; ++k) o[a][b][k] = __vmaxu4(o[a][b][k], m[b][k]);
      }
    }
  }
#pragma unroll
  for (int a = 0; a < 2; ++a) {
    if (a == 1 && !has_h1) break;
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      if (b == 1 && !has_w1) break;
      const size_t pix = (static_cast<size_t>(n) * g.Ho + ho + a) * g.Wo + wo + b;
      *reinterpret_cast<uint4*>(y + pix * g.Cp + ch * 16) = make_uint4(o[a][b][0] ^ flip, o[a][b][1] ^ flip, o[a][b][2] ^ flip, o[a][b][3] ^ flip);
    }
  }
}

// Large windows with few outputs (global average pooling): one warp per (output pixel, 16-channel
// chunk), the lanes share out the window's taps and combine their byte-SIMD maxima / packed sums by
// shuffles, so the 49 loads of a 7x7 window are in flight together instead of queued in one thread.
template <bool XS>
__global__ void __launch_bounds__(256) pool_q16_warp_kernel(const uint8_t* __restrict__ x, int type, float in_scale, int in_zp,
                                                            int same_quant, ConvGeom g, OutQuant out, uint8_t* __restrict__ y) {
  pdl_wait();
  pdl_trigger();
  const int chunks = g.Cp >> 4;
  const long long total = static_cast<long long>(g.N) * g.Ho * g.Wo * chunks;
  const long long i = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (i >= total) return;
  const int ch = static_cast<int>(i % chunks);
  const long long p = i / chunks;
  const int wo = static_cast<int>(p % g.Wo);
  const long long t = p / g.Wo;
  const int ho = static_cast<int>(t % g.Ho);
  const int n = static_cast<int>(t / g.Ho);
  const int h_lo = max(0, ho * g.sy - g.pt), h_hi = min(g.H, ho * g.sy - g.pt + g.kh);
  const int w_lo = max(0, wo * g.sx - g.pl), w_hi = min(g.W, wo * g.sx - g.pl + g.kw);
  const int ww = max(0, w_hi - w_lo);
  const int count = max(0, h_hi - h_lo) * ww;
  const uint32_t flip = XS ? 0x80808080u : 0u;
  uint32_t mx[4] = {0u, 0u, 0u, 0u}, even[4] = {0u, 0u, 0u, 0u}, odd[4] = {0u, 0u, 0u, 0u};
  const uint8_t* base = x + static_cast<size_t>(n) * g.H * g.W * g.Cp + ch * 16;
  for (int tap = lane; tap < count; tap += 32) {
    const int r = tap / ww, c = tap - r * ww;
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(base + (static_cast<size_t>(h_lo + r) * g.W + (w_lo + c)) * g.Cp));
    const uint32_t w4[4] = {v.x ^ flip, v.y ^ flip, v.z ^ flip, v.w ^ flip};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      mx[k] = __vmaxu4(mx[k], w4[k]);
      even[k] += w4[k] & 0x00FF00FFu;
      odd[k] += (w4[k] >> 8) & 0x00FF00FFu;
    }
  }
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      mx[k] = __vmaxu4(mx[k], __shfl_xor_sync(0xffffffffu, mx[k], off));
      even[k] += __shfl_xor_sync(0xffffffffu, even[k], off);     // 16-bit lanes: at most 256 taps x 255
      odd[k] += __shfl_xor_sync(0xffffffffu, odd[k], off);
    }
  }
  if (lane >= 4) return;
  const int k = lane;                                           // lane k finishes word k of the chunk
  const int bias = XS ? 128 : 0;
  const float div = type == 1 ? static_cast<float>(g.kw * g.kh) : static_cast<float>(count);
  uint32_t word = 0;
  if (type == 0 && same_quant) {
    word = count ? (mx[k] ^ flip) : (static_cast<uint32_t>(in_zp & 0xFF) * 0x01010101u);
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int q;
      if (type == 0) {
        q = count ? static_cast<int>((mx[k] >> (8 * j)) & 0xFF) - bias : in_zp;
        q = requant(__fmul_rn(__fsub_rn(__int2float_rn(q), __int2float_rn(in_zp)), in_scale), out);
      } else {
        const uint32_t pair = (j & 1) ? odd[k] : even[k];
        const int sum = static_cast<int>((pair >> (16 * (j >> 1))) & 0xFFFF) - count * (in_zp + bias);
        const float avg = count ? __fdiv_rn(__fmul_rn(__int2float_rn(sum), in_scale), div) : 0.0f;
        q = requant(avg, out);
      }
      word |= static_cast<uint32_t>(q & 0xFF) << (8 * j);
    }
  }
  *reinterpret_cast<uint32_t*>(y + static_cast<size_t>(p) * g.Cp + ch * 16 + 4 * k) = word;
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
  float sum = 0.0f, mx = -INFINITY, sq = 0.0f;
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
      sq = __fadd_rn(sq, __fmul_rn(v, v));
      ++count;
    }
  }
  const float div = type == 1 ? static_cast<float>(g.kw * g.kh) : static_cast<float>(count);
  float r = 0.0f;
  if (count) r = type == 0 ? mx : (type == 2 ? __fsqrt_rn(__fdiv_rn(sq, __int2float_rn(count))) : __fdiv_rn(sum, div));
  y[static_cast<size_t>(p) * g.Cp + c] = r;
}

// ---------------------------------------------------------------- elementwise

template <bool S>
__device__ __forceinline__ int byte_at(uint32_t word, int j) {
  const uint32_t b = (word >> (8 * j)) & 0xFF;
  return S ? static_cast<int>(static_cast<int8_t>(b)) : static_cast<int>(b);
}

// Quantized Add, 16 elements per thread and step, 128-bit loads and stores.
//
// Per element the reference computes (qa - za)*sa + (qb - zb)*sb in float and requantizes the sum.
// Here a byte becomes the float 2^23 + q by a byte permute into a float's mantissa (signed inputs are
// biased by 128 first), the zero point is removed by an exact float subtraction, and every float
// operation handles two elements (f32x2).  Rounding: r = sum*inv + (1.5*2^23 + zp) leaves
// rint(sum*inv) + zp in the low mantissa bits; it is evaluated with inv*(1 +- 2^-21) and the two results
// agree unless sum/scale lies within about 2^-21 (relative) of a .5 fraction, in which case that
// element is redone with the exact sequence.  FAST = false is the exact sequence only, for
// scale ratios so extreme that the magic-number addition could leave its binade.
struct AddParams {
  float sa, sb, scale;          // input scales, output scale
  float ca, cb;                 // -(2^23 + za [+128]), -(2^23 + zb [+128])
  float inv_hi, inv_lo, magic;  // 1/scale * (1 +- 2^-21), 1.5*2^23 + zp
  int za, zb;
  uint32_t a_flip, b_flip;      // 0x80808080 for signed inputs
  OutQuant out;
  int out_signed;
};

__device__ __forceinline__ int add_q_exact(uint32_t aw, uint32_t bw, int j, const AddParams& p) {
  const int qa = static_cast<int>((aw >> (8 * j)) & 0xFF) - (p.a_flip ? 128 : 0);
  const int qb = static_cast<int>((bw >> (8 * j)) & 0xFF) - (p.b_flip ? 128 : 0);
  const float fa = __fmul_rn(__int2float_rn(qa - p.za), p.sa), fb = __fmul_rn(__int2float_rn(qb - p.zb), p.sb);
  return requant(__fadd_rn(fa, fb), p.out);
}

// aw, bw: four input bytes each, signed inputs already biased by 128
template <bool FAST>
__device__ __forceinline__ uint32_t add_q_word(uint32_t aw, uint32_t bw, const AddParams& p) {
  int v[4];
  uint32_t d[4];
  if (FAST) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint32_t a0 = __byte_perm(aw, 0x4B000000u, h ? 0x7542 : 0x7540), a1 = __byte_perm(aw, 0x4B000000u, h ? 0x7543 : 0x7541);
      const uint32_t b0 = __byte_perm(bw, 0x4B000000u, h ? 0x7542 : 0x7540), b1 = __byte_perm(bw, 0x4B000000u, h ? 0x7543 : 0x7541);
      // The two products are scalar mul.rn (never contracted): a packed multiply feeding the packed
      // addition came back fused into one multiply-add on sm_100a, i.e. with the product unrounded,
      // also when it was written as fma(a, b, -0).
      float da0, da1, db0, db1;
      f2_unpack(f2_add(f2_pack_bits(a0, a1), f2_pack(p.ca, p.ca)), da0, da1);
      f2_unpack(f2_add(f2_pack_bits(b0, b1), f2_pack(p.cb, p.cb)), db0, db1);
      const f32x2 fa = f2_pack(__fmul_rn(da0, p.sa), __fmul_rn(da1, p.sa));
      const f32x2 fb = f2_pack(__fmul_rn(db0, p.sb), __fmul_rn(db1, p.sb));
      const f32x2 sum = f2_add(fa, fb);
      const f32x2 m = f2_pack(p.magic, p.magic);
      uint32_t h0, h1, l0, l1;
      f2_unpack_bits(f2_fma(sum, f2_pack(p.inv_hi, p.inv_hi), m), h0, h1);
      f2_unpack_bits(f2_fma(sum, f2_pack(p.inv_lo, p.inv_lo), m), l0, l1);
      d[2 * h] = h0 ^ l0;
      d[2 * h + 1] = h1 ^ l1;
      v[2 * h] = static_cast<int>(h0) - 0x4B400000;
      v[2 * h + 1] = static_cast<int>(h1) - 0x4B400000;
    }
  } else {
    d[0] = d[1] = d[2] = d[3] = 1u;
  }
  if (d[0] | d[1] | d[2] | d[3]) {
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (d[j]) v[j] = add_q_exact(aw, bw, j, p);
  }
  return p.out_signed ? pack_sat_s8(v[1], v[0], pack_sat_s8(v[3], v[2], 0u)) : pack_sat_u8(v[1], v[0], pack_sat_u8(v[3], v[2], 0u));
}

template <bool FAST>
__global__ void __launch_bounds__(256) add_q_kernel(const uint4* __restrict__ a, const uint4* __restrict__ b, AddParams p,
                                                    uint4* __restrict__ y, size_t n16) {
  pdl_wait();
  pdl_trigger();
  // Two groups per step, all four loads issued before any arithmetic: the kernel needs about 64 KB of
  // loads in flight per SM to keep HBM busy.
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n16; i += 2 * stride) {
    const size_t i2 = i + stride;
    const bool two = i2 < n16;
    uint4 av = __ldcs(a + i), bv = __ldcs(b + i);
    uint4 av2 = make_uint4(0, 0, 0, 0), bv2 = make_uint4(0, 0, 0, 0);
    if (two) { av2 = __ldcs(a + i2); bv2 = __ldcs(b + i2); }
    av.x ^= p.a_flip; av.y ^= p.a_flip; av.z ^= p.a_flip; av.w ^= p.a_flip;
    bv.x ^= p.b_flip; bv.y ^= p.b_flip; bv.z ^= p.b_flip; bv.w ^= p.b_flip;
    uint4 o;
    o.x = add_q_word<FAST>(av.x, bv.x, p);
    o.y = add_q_word<FAST>(av.y, bv.y, p);
    o.z = add_q_word<FAST>(av.z, bv.z, p);
    o.w = add_q_word<FAST>(av.w, bv.w, p);
    y[i] = o;
    if (two) {
      av2.x ^= p.a_flip; av2.y ^= p.a_flip; av2.z ^= p.a_flip; av2.w ^= p.a_flip;
      bv2.x ^= p.b_flip; bv2.y ^= p.b_flip; bv2.z ^= p.b_flip; bv2.w ^= p.b_flip;
      o.x = add_q_word<FAST>(av2.x, bv2.x, p);
      o.y = add_q_word<FAST>(av2.y, bv2.y, p);
      o.z = add_q_word<FAST>(av2.z, bv2.z, p);
      o.w = add_q_word<FAST>(av2.w, bv2.w, p);
      y[i2] = o;
    }
  }
}

// Quantized Add by table: the result is a function of the two input bytes, so a 64 KB table (built on the
// host with the reference's float sequence) answers every element exactly, whatever the share of
// near-tie sums that would send the arithmetic kernel to its exact path.  The table lives in shared
// memory; entry (a, b) sits at a*256 + (b ^ ((a & 31) << 2)), which spreads pairs that share b over
// the banks.  Per element: build the index, one byte load, pack.
__global__ void __launch_bounds__(1024) add_q_lut_kernel(const uint4* __restrict__ a, const uint4* __restrict__ b,
                                                        const uint4* __restrict__ table, uint4* __restrict__ y, size_t n16) {
  pdl_trigger();
  extern __shared__ uint4 tab4[];
  for (int i = threadIdx.x; i < 4096; i += blockDim.x) tab4[i] = table[i];   // a constant of the graph
  __syncthreads();
  pdl_wait();
  const uint8_t* tab = reinterpret_cast<const uint8_t*>(tab4);
  // Four groups per step with all eight loads issued first, to keep enough bytes in flight.
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n16; i += 4 * stride) {
    uint4 av[4], bv[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const size_t ik = i + k * stride;
      if (ik < n16) { av[k] = __ldcs(a + ik); bv[k] = __ldcs(b + ik); }
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const size_t ik = i + k * stride;
      if (ik < n16) {
        uint4 o;
        o.x = add_lut_word(av[k].x, bv[k].x, tab);
        o.y = add_lut_word(av[k].y, bv[k].y, tab);
        o.z = add_lut_word(av[k].z, bv[k].z, tab);
        o.w = add_lut_word(av[k].w, bv[k].w, tab);
        y[ik] = o;
      }
    }
  }
}

// Add with numpy-style broadcasting (equal ranks, a dimension of 1 repeats): one output element per
// thread, operand indices from per-axis strides (0 along a broadcast axis), the exact float sequence.
// A slow path by design; the equal-shape case never comes here.
struct BroadcastGeom {
  int N, H, W, C, Cp;                  // output
  long long as[4], bs[4];              // element strides of a and b along (n, h, w, c); 0 = broadcast
};
template <typename T>
__global__ void add_broadcast_kernel(const T* __restrict__ a, float sa, int za, int a_signed, const T* __restrict__ b, float sb,
                                     int zb, int b_signed, OutQuant out, BroadcastGeom g, T* __restrict__ y) {
  const long long total = static_cast<long long>(g.N) * g.H * g.W * g.C;
  long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i >= total) return;
  const int c = static_cast<int>(i % g.C);
  long long r = i / g.C;
  const int w = static_cast<int>(r % g.W); r /= g.W;
  const int h = static_cast<int>(r % g.H);
  const int n = static_cast<int>(r / g.H);
  const long long ai = n * g.as[0] + h * g.as[1] + w * g.as[2] + c * g.as[3];
  const long long bi = n * g.bs[0] + h * g.bs[1] + w * g.bs[2] + c * g.bs[3];
  const size_t yi = ((static_cast<size_t>(n) * g.H + h) * g.W + w) * g.Cp + c;
  if (sizeof(T) == 4) {
    reinterpret_cast<float*>(y)[yi] = __fadd_rn(reinterpret_cast<const float*>(a)[ai], reinterpret_cast<const float*>(b)[bi]);
  } else {
    const int qa = a_signed ? static_cast<int>(static_cast<int8_t>(a[ai])) : static_cast<int>(a[ai]);
    const int qb = b_signed ? static_cast<int>(static_cast<int8_t>(b[bi])) : static_cast<int>(b[bi]);
    const float fa = __fmul_rn(__fsub_rn(__int2float_rn(qa), __int2float_rn(za)), sa);
    const float fb = __fmul_rn(__fsub_rn(__int2float_rn(qb), __int2float_rn(zb)), sb);
    y[yi] = static_cast<T>(requant(__fadd_rn(fa, fb), out) & 0xFF);
  }
}

__global__ void add_f32_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ y, size_t n) {
  size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (i < n) y[i] = __fadd_rn(a[i], b[i]);
}

// Add on 32-bit integer tensors (the reference's platform sample adds INT32 vectors): the same real-domain
// sequence as the 8-bit kernels, with the int32 range as the saturation bounds.
__global__ void add_i32_kernel(const int* __restrict__ a, float sa, int za, const int* __restrict__ b, float sb, int zb,
                               OutQuant out, int* __restrict__ y, size_t n) {
  size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (i >= n) return;
  const float fa = __fmul_rn(__fsub_rn(__int2float_rn(a[i]), __int2float_rn(za)), sa);
  const float fb = __fmul_rn(__fsub_rn(__int2float_rn(b[i]), __int2float_rn(zb)), sb);
  y[i] = requant_wide(__fadd_rn(fa, fb), out);
}

// Move between two storages under a logical shape (see RelayoutParams): the general form behind Reshape,
// Transpose, Concat and DataConvert.  A thread takes a run of up to 16 consecutive positions of iteration
// dimension 0 (the one with the smallest output stride), so neighbouring threads write neighbouring runs and
// the coordinates are worked out once per run.  IndexT: 32-bit when the element count allows.
__device__ __forceinline__ void relayout_one(const uint8_t* __restrict__ in, uint8_t* __restrict__ out, const RelayoutParams& p,
                                             long long src, long long o) {
  switch (p.convert) {
    case 0:
      if (p.elem == 1) out[o] = in[src];
      else reinterpret_cast<uint32_t*>(out)[o] = reinterpret_cast<const uint32_t*>(in)[src];
      break;
    case 1:
      out[o] = __ldg(p.lut + in[src]);
      break;
    case 2:
      out[o] = static_cast<uint8_t>(requant(reinterpret_cast<const float*>(in)[src], p.out) & 0xFF);
      break;
    default: {
      const int q = p.in_signed ? static_cast<int>(static_cast<int8_t>(in[src])) : static_cast<int>(in[src]);
      reinterpret_cast<float*>(out)[o] = __fmul_rn(__fsub_rn(__int2float_rn(q), __int2float_rn(p.in_zp)), p.in_scale);
      break;
    }
  }
}

template <typename IndexT>
__global__ void relayout_kernel(const uint8_t* __restrict__ in, uint8_t* __restrict__ out, RelayoutParams p, int run, int runs0,
                                long long n_threads) {
  const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (tid >= n_threads) return;
  IndexT rem = static_cast<IndexT>(tid);
  const int c0 = static_cast<int>(rem % static_cast<IndexT>(runs0)) * run;
  rem /= static_cast<IndexT>(runs0);
  long long o = c0 * p.ostride[0], src = c0 * p.istride[0], lin = c0 * p.lstride[0];
#pragma unroll
  for (int k = 1; k < 4; ++k) {
    if (k < p.rank) {
      const long long c = static_cast<long long>(rem % static_cast<IndexT>(p.dims[k]));
      rem /= static_cast<IndexT>(p.dims[k]);
      o += c * p.ostride[k];
      src += c * p.istride[k];
      lin += c * p.lstride[k];
    }
  }
  const int count = min(run, p.dims[0] - c0);
  if (count == 16 && p.convert == 0 && p.elem == 1 && !p.reshape && p.ostride[0] == 1 && p.istride[0] == 1 &&
      ((reinterpret_cast<uintptr_t>(in + src) | reinterpret_cast<uintptr_t>(out + o)) & 15) == 0) {
    // both sides contiguous along the run: one 16-byte copy
    *reinterpret_cast<uint4*>(out + o) = *reinterpret_cast<const uint4*>(in + src);
    return;
  }
  for (int e = 0; e < count; ++e) {
    long long s = src;
    if (p.reshape) {
      IndexT l = static_cast<IndexT>(lin);
      s = 0;
#pragma unroll
      for (int k = 0; k < 4; ++k) {   // unused dimensions have extent 1
        s += static_cast<long long>(l % static_cast<IndexT>(p.idims[k])) * p.istride[k];
        l /= static_cast<IndexT>(p.idims[k]);
      }
    }
    relayout_one(in, out, p, s, o);
    o += p.ostride[0];
    src += p.istride[0];
    lin += p.lstride[0];
  }
}

// Byte transpose between a dimension that is contiguous in the output (iteration dimension 0) and one that is
// contiguous in the input (dimension kb): 32 x 32 tiles through shared memory, so that both the reads and the
// writes of a warp are 32 consecutive bytes.  The remaining dimensions are spread over blockIdx.z.
__global__ void relayout_tiled_kernel(const uint8_t* __restrict__ in, uint8_t* __restrict__ out, RelayoutParams p, int kb) {
  __shared__ uint8_t tile[32][33];
  long long ibase = 0, obase = 0;
  unsigned rest = blockIdx.z;
#pragma unroll
  for (int k = 1; k < 4; ++k) {
    if (k < p.rank && k != kb) {
      const unsigned c = rest % static_cast<unsigned>(p.dims[k]);
      rest /= static_cast<unsigned>(p.dims[k]);
      ibase += c * p.istride[k];
      obase += c * p.ostride[k];
    }
  }
  const int a0 = blockIdx.x * 32, b0 = blockIdx.y * 32;
  const int tx = threadIdx.x, ty = threadIdx.y;
#pragma unroll
  for (int i = 0; i < 32; i += 8) {
    const int a = a0 + ty + i, b = b0 + tx;
    if (a < p.dims[0] && b < p.dims[kb]) tile[ty + i][tx] = in[ibase + a * p.istride[0] + b];
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 32; i += 8) {
    const int a = a0 + tx, b = b0 + ty + i;
    if (a < p.dims[0] && b < p.dims[kb]) out[obase + a + b * p.ostride[kb]] = tile[tx][ty + i];
  }
}

__global__ void concat_c16_kernel(const uint4* __restrict__ in, int in_pitch16, int in16, uint4* __restrict__ out, int out_pitch16,
                                  int off16, long long total) {
  const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i >= total) return;
  const long long pix = i / in16;
  const int j = static_cast<int>(i - pix * in16);
  out[pix * out_pitch16 + off16 + j] = in[pix * in_pitch16 + j];
}

// Any 8-bit -> 8-bit pointwise map (Relu, Relu6 with arbitrary input/output
// quantization) as a 256-entry table built on the host with the reference's
// float sequence; 16 elements per thread.
__global__ void lut_q_kernel(const uint4* __restrict__ x, const uint8_t* __restrict__ lut, uint4* __restrict__ y, size_t n16) {
  pdl_wait();
  pdl_trigger();
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
  pdl_wait();
  pdl_trigger();
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

// im2col from a WHCN input with few channels, K index = (ky*C + c)*8 + kx (filter rows padded to 8
// taps, kw <= 8, dilation 1): the 8 bytes of one (pixel, ky, c) are 8 consecutive input bytes, so a
// 16-byte piece of the matrix is two unaligned 8-byte reads of the staged rows instead of sixteen
// gathered bytes.  The byte in the padding slot (kx >= kw) belongs to the neighbouring pixel; its
// weight is zero.  One block per output row (n, ho); staged rows have pitch `pitch` (a multiple of 4,
// at least 8 bytes beyond the last input column used).
template <int PADK>
__global__ void __launch_bounds__(256) im2col_whcn8_kernel(const uint8_t* __restrict__ x, int Kp, int zx, ConvGeom g, int pitch,
                                                           uint8_t* __restrict__ col) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ uint32_t sm_words[];
  uint8_t* img = reinterpret_cast<uint8_t*>(sm_words);     // [kh*C][pitch]
  const int n = blockIdx.y, ho = blockIdx.x;
  const int rows = g.kh * g.C;
  // Staged column j holds input column j - lead; lead = pad_left rounded up to 4 keeps input words
  // aligned with shared-memory words.  First everything becomes the zero point, then the in-bounds
  // part of each row is copied (as 32-bit words when the input rows allow it).
  const int lead = (g.pl + 3) & ~3;
  const uint32_t zx_word = static_cast<uint32_t>(zx & 0xFF) * 0x01010101u;
  const int pitch_w = pitch >> 2;
  for (int idx = threadIdx.x; idx < rows * pitch_w; idx += blockDim.x) sm_words[idx] = zx_word;
  __syncthreads();
  const int copy_cols = min(g.W, pitch - lead);            // input columns that fit in a staged row
  if ((g.W & 3) == 0 && (reinterpret_cast<uintptr_t>(x) & 3) == 0) {
    const int wpr = copy_cols >> 2;                         // whole words; the ragged rest below
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int r = warp; r < rows; r += 8) {                  // a warp per staged row, lanes along it
      const int ky = r / g.C, c = r - ky * g.C;
      const int hi = ho * g.sy - g.pt + ky;
      if (hi < 0 || hi >= g.H) continue;
      const uint32_t* src = reinterpret_cast<const uint32_t*>(x + ((static_cast<size_t>(n) * g.C + c) * g.H + hi) * g.W);
      uint32_t* dst = sm_words + r * pitch_w + (lead >> 2);
      for (int w = lane; w < wpr; w += 32) dst[w] = __ldg(src + w);
    }
    const int rest = copy_cols & 3;
    for (int idx = threadIdx.x; idx < rows * rest; idx += blockDim.x) {
      const int r = idx / rest, wi = (copy_cols & ~3) + (idx - r * rest);
      const int ky = r / g.C, c = r - ky * g.C;
      const int hi = ho * g.sy - g.pt + ky;
      if (hi >= 0 && hi < g.H) img[r * pitch + lead + wi] = x[((static_cast<size_t>(n) * g.C + c) * g.H + hi) * g.W + wi];
    }
  } else {
    for (int idx = threadIdx.x; idx < rows * copy_cols; idx += blockDim.x) {
      const int r = idx / copy_cols, wi = idx - r * copy_cols;
      const int ky = r / g.C, c = r - ky * g.C;
      const int hi = ho * g.sy - g.pt + ky;
      if (hi >= 0 && hi < g.H) img[r * pitch + lead + wi] = x[((static_cast<size_t>(n) * g.C + c) * g.H + hi) * g.W + wi];
    }
  }
  __syncthreads();
  const int shift0 = lead - g.pl;                          // staged column of output pixel 0, tap 0
  const int chunks = Kp >> 4;
  uint8_t* out = col + (static_cast<size_t>(n) * g.Ho + ho) * g.Wo * Kp;
  // piece q = wo * chunks + ch; a thread's next piece is 256 further, stepped without divisions
  int wo = threadIdx.x / chunks, ch = threadIdx.x - wo * chunks;
  const int step_wo = 256 / chunks, step_ch = 256 - step_wo * chunks;
  for (int q = threadIdx.x; q < g.Wo * chunks; q += 256, wo += step_wo, ch += step_ch) {
    if (ch >= chunks) { ch -= chunks; ++wo; }
    uint32_t w4[4] = {0, 0, 0, 0};
    if (PADK == 8) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int r = 2 * ch + h;
        if (r < rows) {
          const int byte = r * pitch + wo * g.sx + shift0;
          const uint32_t* wp = sm_words + (byte >> 2);
          const uint32_t sh = (byte & 3) * 8;
          const uint32_t a0 = wp[0], a1 = wp[1], a2 = wp[2];
          w4[2 * h] = __funnelshift_r(a0, a1, sh);
          w4[2 * h + 1] = __funnelshift_r(a1, a2, sh);
        }
      }
    } else {
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        const int r = 4 * ch + h;
        if (r < rows) {
          const int byte = r * pitch + wo * g.sx + shift0;
          const uint32_t* wp = sm_words + (byte >> 2);
          w4[h] = __funnelshift_r(wp[0], wp[1], (byte & 3) * 8);
        }
      }
    }
    *reinterpret_cast<uint4*>(out + static_cast<size_t>(wo) * Kp + ch * 16) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
  }
}

// ---------------------------------------------------------------- FullyConnected with few rows (M <= 16)

// Decode-like shapes are bound by streaming the weights once; a 128-row tensor-core tile would spend its
// time on pipeline latency with a handful of CTAs.  Here a block of eight warps owns CH = 4 output
// channels and all M input rows, and its 256 lanes split K in 16-byte slices: a lane loads the four
// weight slices (the only HBM traffic, coalesced along K) and the M input slices (L1/L2-resident) and
// issues 4*4*M dp4a.  With K = 4096 every load of the block is in flight at once, and there are
// Ocp/4 blocks to fill the machine.  The CH*MT partial sums per lane are combined inside the warp by a
// halving exchange (each step a lane gives away half of its values: 31 shuffles for 32 values
// instead of 5 per value), then across the eight warps through shared memory.  HAS_DZ: the weights
// keep a zero point dz, removed as dz * sum(x) accumulated alongside (K must then be unpadded).
template <int CH, int MT, bool XS, bool HAS_DZ>
__global__ void __launch_bounds__(256, 2) fc_small_m_kernel(const uint8_t* __restrict__ A, const int8_t* __restrict__ B, int M, int Kp,
                                                         int Oc, int Ocp, ContractEpilogue ep, uint8_t* __restrict__ D, int ldd) {
  pdl_wait();
  pdl_trigger();
  constexpr int V = CH * MT;                        // partial sums per lane: 4 ... 64
  constexpr int KEEP = V >= 64 ? 2 : 1;             // values a lane still holds after the exchange
  __shared__ int partial[8][32 * KEEP];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c0 = blockIdx.x * CH;
  int v[V];
#pragma unroll
  for (int i = 0; i < V; ++i) v[i] = 0;
  int sx[MT];
#pragma unroll
  for (int m = 0; m < MT; ++m) sx[m] = 0;
  const int8_t* brow = B + static_cast<size_t>(c0) * Kp;
#pragma unroll 1
  for (int k = threadIdx.x * 16; k < Kp; k += 256 * 16) {
    uint4 w[CH];
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      w[c] = make_uint4(0, 0, 0, 0);
      if (c0 + c < Ocp) w[c] = __ldcs(reinterpret_cast<const uint4*>(brow + static_cast<size_t>(c) * Kp + k));
    }
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      const int row = m < M ? m : M - 1;            // rows beyond M repeat the last one; their sums are dropped
      const uint4 x = __ldg(reinterpret_cast<const uint4*>(A + static_cast<size_t>(row) * Kp + k));
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        int a = v[c * MT + m];
        a = dp4<XS>(x.x, w[c].x, a);
        a = dp4<XS>(x.y, w[c].y, a);
        a = dp4<XS>(x.z, w[c].z, a);
        a = dp4<XS>(x.w, w[c].w, a);
        v[c * MT + m] = a;
      }
      if (HAS_DZ) {
        int t = sx[m];
        t = dp4<XS>(x.x, 0x01010101u, t);
        t = dp4<XS>(x.y, 0x01010101u, t);
        t = dp4<XS>(x.z, 0x01010101u, t);
        t = dp4<XS>(x.w, 0x01010101u, t);
        sx[m] = t;
      }
    }
  }
  if (HAS_DZ) {
#pragma unroll
    for (int c = 0; c < CH; ++c)
#pragma unroll
      for (int m = 0; m < MT; ++m) v[c * MT + m] -= ep.dz_uniform * sx[m];
  }
  // Halving exchange.  Step s (offset 16 >> s) starts with V >> s values per lane: a lane keeps the
  // upper half if its offset bit is set, else the lower half, each added to the partner's copy.  Once
  // a single value is left the remaining steps are plain butterfly additions, after which the lanes
  // with those bits set hold duplicates.
  int idx = 0;
  bool owner = true;
#pragma unroll
  for (int step = 0; step < 5; ++step) {
    const int off = 16 >> step;
    if ((V >> step) > 1) {
      const int n = (V >> step) >> 1;
      const bool upper = (lane & off) != 0;
#pragma unroll
      for (int j = 0; j < n; ++j) {
        const int send = upper ? v[j] : v[j + n];
        const int keep = upper ? v[j + n] : v[j];
        v[j] = keep + __shfl_xor_sync(0xffffffffu, send, off);
      }
      if (upper) idx += n;
    } else {
      v[0] += __shfl_xor_sync(0xffffffffu, v[0], off);
      if (lane & off) owner = false;
    }
  }
#pragma unroll
  for (int j = 0; j < KEEP; ++j) partial[warp][lane * KEEP + j] = v[j];
  __syncthreads();
  if (warp == 0 && owner) {
#pragma unroll
    for (int j = 0; j < KEEP; ++j) {
      int total = 0;
#pragma unroll
      for (int w8 = 0; w8 < 8; ++w8) total += partial[w8][lane * KEEP + j];
      const int id = idx + j;
      const int c = id / MT, m = id - c * MT;
      const int oc = c0 + c;
      if (m < M && oc < Oc) {
        const int acc = total + ep.bias_full[oc];
        const float real = __fmul_rn(__int2float_rn(acc), ep.acc_scale[oc]);
        D[static_cast<size_t>(m) * ldd + oc] = static_cast<uint8_t>(requant(real, ep.out) & 0xFF);
      }
    }
  }
}

}  // namespace

// ---------------------------------------------------------------- wrappers

void launch_whcn_to_cl(const void* src, void* dst, int N, int C, int H, int W, int Cp, int elem, cudaStream_t s) {
  const int HW = H * W;
  if (N == 0 || HW == 0 || Cp == 0) return;
  if (elem == 1) {
    const dim3 grid((HW + 63) / 64, (Cp + 63) / 64, N);
    const bool aligned = (HW & 3) == 0 && (reinterpret_cast<uintptr_t>(src) & 3) == 0;
    if (aligned) launch_pdl(whcn_to_cl_u8_kernel<true>, dim3(grid), dim3(256), 0, s, static_cast<const uint8_t*>(src), static_cast<uint8_t*>(dst), C, HW, Cp);
    else launch_pdl(whcn_to_cl_u8_kernel<false>, dim3(grid), dim3(256), 0, s, static_cast<const uint8_t*>(src), static_cast<uint8_t*>(dst), C, HW, Cp);
  } else {
    const dim3 grid((HW + 31) / 32, (Cp + 31) / 32, N);
    whcn_to_cl_u32_kernel<<<grid, 256, 0, s>>>(static_cast<const uint32_t*>(src), static_cast<uint32_t*>(dst), C, HW, Cp);
  }
}

void launch_cl_to_whcn(const void* src, void* dst, int N, int C, int H, int W, int Cp, int elem, cudaStream_t s) {
  const int HW = H * W;
  if (N == 0 || HW == 0 || C == 0) return;
  if (elem == 1) {
    const dim3 grid((HW + 63) / 64, (C + 63) / 64, N);
    const bool aligned = (HW & 3) == 0 && (reinterpret_cast<uintptr_t>(dst) & 3) == 0;
    if (aligned) launch_pdl(cl_to_whcn_u8_kernel<true>, dim3(grid), dim3(256), 0, s, static_cast<const uint8_t*>(src), static_cast<uint8_t*>(dst), C, HW, Cp);
    else launch_pdl(cl_to_whcn_u8_kernel<false>, dim3(grid), dim3(256), 0, s, static_cast<const uint8_t*>(src), static_cast<uint8_t*>(dst), C, HW, Cp);
  } else {
    const dim3 grid((HW + 31) / 32, (C + 31) / 32, N);
    cl_to_whcn_u32_kernel<<<grid, 256, 0, s>>>(static_cast<const uint32_t*>(src), static_cast<uint32_t*>(dst), C, HW, Cp);
  }
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

namespace {
constexpr int kDwStripSmem = 72 * 1024;

// Tile shape of the strip form for one layer: the candidate (channel chunks per slab, strips per row, rows, images
// per tile) with the lowest estimated instruction count over the whole layer.  A block always runs its 256 threads
// through the arithmetic of 32 outputs each (about 540 instructions) and stages its patch at about 15 instructions
// per 16-byte unit, so the estimate is blocks * (540 + 15 * units / 256); ties go to the wider slab.
bool choose_dw_strip(const ConvGeom& g, DwStripGeom* best, double* best_cost) {
  const int S = g.sx, nchunks = g.Ocp / 16;
  bool found = false;
  for (int cs = 2; cs >= 0; --cs) {
    const int CK = 1 << cs, strips = 64 >> cs, slabs = (nchunks + CK - 1) / CK, px_bytes = 64 >> (2 - cs);
    for (int ss = 0; ss <= 3; ++ss) {
      const int SEG = 1 << ss, TW = 8 * SEG;
      if (SEG > strips || (ss > 0 && 8 * (SEG / 2) >= g.Wo)) continue;   // a row of strips no wider than needed
      for (int ts = 0; (SEG << ts) <= strips; ++ts) {
        const int TH = 1 << ts;
        if (ts > 0 && (TH / 2) >= g.Ho) continue;
        const int NI = strips / (SEG * TH);
        if (NI > 1 && (TH < g.Ho || TW < g.Wo)) continue;                 // several images only as whole images
        int ns = 0;
        while ((1 << ns) < NI) ++ns;
        const int IH = (TH - 1) * S + 3, IW = (TW - 1) * S + 3;
        // rows of a warp's consecutive strips (S patch rows apart) should start px_bytes apart modulo 128
        int pitch = IW * px_bytes;
        for (int k = 0; k < 8 && (S * pitch) % 128 != px_bytes % 128; ++k) pitch += 16;
        if ((S * pitch) % 128 != px_bytes % 128) pitch = IW * px_bytes;
        if (static_cast<size_t>(NI) * IH * pitch > static_cast<size_t>(kDwStripSmem) || IW > 255) continue;
        if ((g.N + NI - 1) / NI > 65535 || slabs > 65535) continue;
        const double blocks = static_cast<double>((g.Wo + TW - 1) / TW) * ((g.Ho + TH - 1) / TH) * ((g.N + NI - 1) / NI) * slabs;
        const double cost = blocks * (540.0 + 15.0 * (static_cast<double>(NI) * IH * IW * CK) / 256.0);
        if (!found || cost < *best_cost) {
          found = true;
          *best_cost = cost;
          best->ck_shift = cs; best->seg_shift = ss; best->th_shift = ts; best->ni_shift = ns;
          best->IH = IH; best->IW = IW; best->pitch = pitch;
        }
      }
    }
  }
  return found;
}
}  // namespace

void launch_depthwise_q16(const void* x, int x_signed, int zx, const uint32_t* wtab, const uint32_t* wtab_v, const int32_t* bias_full,
                          const float* acc_scale, const ConvGeom& g, OutQuant out, int exact_only, void* y, cudaStream_t s) {
  if (static_cast<long long>(g.N) * g.Ho * g.Wo == 0) return;
  DwParams p;
  p.g = g;
  p.wtab = wtab;
  p.wtab_v = wtab_v;
  p.bias_full = bias_full;
  p.acc_scale = acc_scale;
  p.out = out;
  p.x_flip = x_signed ? 0x80808080u : 0u;
  p.zx_word = static_cast<uint32_t>((zx + (x_signed ? 128 : 0)) & 0xFF) * 0x01010101u;
  p.exact_only = exact_only;
  p.slab = g.Ocp < 64 ? g.Ocp : 64;
  const int chunks = p.slab / 16;
  const int pairs_per_block = 256 / chunks;
  const long long total_pairs = static_cast<long long>(g.N) * g.Ho * ((g.Wo + 1) / 2);
  const dim3 grid(static_cast<unsigned>((total_pairs + pairs_per_block - 1) / pairs_per_block), (g.Ocp + p.slab - 1) / p.slab);
  const size_t smem = static_cast<size_t>(g.kh) * g.kw * (p.slab / 4) * sizeof(uint4);
  const uint8_t* xp = static_cast<const uint8_t*>(x);
  uint8_t* yp = static_cast<uint8_t*>(y);
  // 3x3 windows at stride 1 or 2: the strip form (B2VX_DW_STRIP=0 keeps the 16-channel form below)
  const char* strip_env = std::getenv("B2VX_DW_STRIP");   // read per launch, so that one process can run both forms
  const bool no_strip = strip_env && std::strcmp(strip_env, "0") == 0;
  if (!no_strip && wtab_v != nullptr && g.kh == 3 && g.kw == 3 && g.dx == 1 && g.dy == 1 && g.sx == g.sy && (g.sx == 1 || g.sx == 2)) {
    DwStripGeom best{};
    double best_cost = 0.0;
    if (choose_dw_strip(g, &best, &best_cost)) {
      const int CK = 1 << best.ck_shift, TH = 1 << best.th_shift, TW = 8 << best.seg_shift, NI = 1 << best.ni_shift;
      const size_t smem_t = static_cast<size_t>(NI) * best.IH * best.pitch;
      best.tiles_w = (g.Wo + TW - 1) / TW;
      best.iw_recip = 65536 / best.IW + 1;
      best.step_h = (256 / CK) / best.IW;
      best.step_w = (256 / CK) % best.IW;
      const dim3 grid_t(static_cast<unsigned>(best.tiles_w * ((g.Ho + TH - 1) / TH)), static_cast<unsigned>((g.N + NI - 1) / NI),
                        static_cast<unsigned>((g.Ocp / 16 + CK - 1) / CK));
      using StripFn = void (*)(const uint8_t*, DwParams, DwStripGeom, uint8_t*);
      static const StripFn fns[2][2][3] = {
          {{depthwise_strip_kernel<1, false, 0>, depthwise_strip_kernel<1, false, 1>, depthwise_strip_kernel<1, false, 2>},
           {depthwise_strip_kernel<1, true, 0>, depthwise_strip_kernel<1, true, 1>, depthwise_strip_kernel<1, true, 2>}},
          {{depthwise_strip_kernel<2, false, 0>, depthwise_strip_kernel<2, false, 1>, depthwise_strip_kernel<2, false, 2>},
           {depthwise_strip_kernel<2, true, 0>, depthwise_strip_kernel<2, true, 1>, depthwise_strip_kernel<2, true, 2>}}};
      static const StripFn pipe_fns[2][2][3] = {
          {{depthwise_strip_pipe_kernel<1, false, 0>, depthwise_strip_pipe_kernel<1, false, 1>, depthwise_strip_pipe_kernel<1, false, 2>},
           {depthwise_strip_pipe_kernel<1, true, 0>, depthwise_strip_pipe_kernel<1, true, 1>, depthwise_strip_pipe_kernel<1, true, 2>}},
          {{depthwise_strip_pipe_kernel<2, false, 0>, depthwise_strip_pipe_kernel<2, false, 1>, depthwise_strip_pipe_kernel<2, false, 2>},
           {depthwise_strip_pipe_kernel<2, true, 0>, depthwise_strip_pipe_kernel<2, true, 1>, depthwise_strip_pipe_kernel<2, true, 2>}}};
      static int sms_of[64] = {0};
      static bool attr_set_t[64] = {false};
      int dev = 0;
      cudaGetDevice(&dev);
      if (dev < 0 || dev >= 64 || !attr_set_t[dev]) {
        for (int a = 0; a < 2; ++a)
          for (int b = 0; b < 2; ++b)
            for (int c = 0; c < 3; ++c) {
              cudaFuncSetAttribute(fns[a][b][c], cudaFuncAttributeMaxDynamicSharedMemorySize, kDwStripSmem);
              cudaFuncSetAttribute(pipe_fns[a][b][c], cudaFuncAttributeMaxDynamicSharedMemorySize, kDwStripSmem);
            }
        if (dev >= 0 && dev < 64) {
          cudaDeviceGetAttribute(&sms_of[dev], cudaDevAttrMultiProcessorCount, dev);
          attr_set_t[dev] = true;
        }
      }
      // Pipelined form (two patches per block, three blocks per SM) when both patches fit and the layer is large;
      // B2VX_DW_PIPE=0 keeps one tile per block, =1 pipelines every layer whose patches fit.
      const char* pipe_env = std::getenv("B2VX_DW_PIPE");   // read per launch plan: "0" never, "1" whenever it fits
      const bool no_pipe = pipe_env && std::strcmp(pipe_env, "0") == 0, force_pipe = pipe_env && std::strcmp(pipe_env, "1") == 0;
      best.tiles_h = (g.Ho + TH - 1) / TH;
      best.n_groups = (g.N + NI - 1) / NI;
      best.patch_bytes = static_cast<int>((smem_t + 127) & ~static_cast<size_t>(127));
      const int sms = (dev >= 0 && dev < 64 && sms_of[dev] > 0) ? sms_of[dev] : 148;
      // (measured on MobileNetV2 at batch 64: the pipeline wins from about four tiles per resident block on, below
      // that the one-tile blocks, which the hardware schedules one by one, finish sooner)
      const long long all_tiles = static_cast<long long>(grid_t.x) * grid_t.y * grid_t.z;
      if (!no_pipe && 2 * static_cast<size_t>(best.patch_bytes) <= static_cast<size_t>(kDwStripSmem) && (force_pipe || all_tiles >= 12LL * sms)) {
        const long long tiles = static_cast<long long>(grid_t.x) * grid_t.y;
        long long gx = (3LL * sms) / grid_t.z;
        if (gx < 1) gx = 1;
        if (gx > tiles) gx = tiles;
        const dim3 grid_p(static_cast<unsigned>(gx), 1, grid_t.z);
        launch_pdl(pipe_fns[g.sx - 1][x_signed ? 1 : 0][best.ck_shift], grid_p, dim3(256), 2 * static_cast<size_t>(best.patch_bytes), s, xp, p, best, yp);
        return;
      }
      launch_pdl(fns[g.sx - 1][x_signed ? 1 : 0][best.ck_shift], grid_t, dim3(256), smem_t, s, xp, p, best, yp);
      return;
    }
  }
  {
    // staged form when the input patch of a TH x TW output tile fits comfortably in shared memory
    const int tw_shift = g.Wo <= 8 ? 3 : 4;
    const int TW = 1 << tw_shift;
    // chunks per slab: the choice of 4, 2, 1 that leaves the fewest idle channel chunks (ties: the larger)
    const int nchunks = g.Ocp / 16;
    int ck_shift = 2, best_waste = 1 << 30;
    for (int cs = 2; cs >= 0; --cs) {
      const int ck = 1 << cs, waste = (nchunks + ck - 1) / ck * ck - nchunks;
      if (waste < best_waste) { best_waste = waste; ck_shift = cs; }
    }
    const int CK = 1 << ck_shift, TH = 32 >> ck_shift;
    const int IH = (TH - 1) * g.sy + (g.kh - 1) * g.dy + 1, IW = (TW - 1) * g.sx + (g.kw - 1) * g.dx + 1;
    const size_t smem_s = (static_cast<size_t>(g.kh) * g.kw * 4 * CK + static_cast<size_t>(IH) * IW * CK) * sizeof(uint4);
    if (smem_s <= 72 * 1024) {
      const dim3 grid_s(static_cast<unsigned>(((g.Wo + TW - 1) / TW) * ((g.Ho + TH - 1) / TH) * g.N), (nchunks + CK - 1) / CK);
      static bool attr_set[64] = {false};
      int dev = 0;
      cudaGetDevice(&dev);
      if (dev < 0 || dev >= 64 || !attr_set[dev]) {
        cudaFuncSetAttribute(depthwise_q16s_kernel<3, 3, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 72 * 1024);
        cudaFuncSetAttribute(depthwise_q16s_kernel<3, 3, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 72 * 1024);
        cudaFuncSetAttribute(depthwise_q16s_kernel<0, 0, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 72 * 1024);
        cudaFuncSetAttribute(depthwise_q16s_kernel<0, 0, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 72 * 1024);
        if (dev >= 0 && dev < 64) attr_set[dev] = true;
      }
      if (g.kh == 3 && g.kw == 3) {
        if (x_signed) launch_pdl(depthwise_q16s_kernel<3, 3, true>, dim3(grid_s), dim3(256), smem_s, s, xp, p, tw_shift, ck_shift, IH, IW, yp);
        else launch_pdl(depthwise_q16s_kernel<3, 3, false>, dim3(grid_s), dim3(256), smem_s, s, xp, p, tw_shift, ck_shift, IH, IW, yp);
      } else {
        if (x_signed) launch_pdl(depthwise_q16s_kernel<0, 0, true>, dim3(grid_s), dim3(256), smem_s, s, xp, p, tw_shift, ck_shift, IH, IW, yp);
        else launch_pdl(depthwise_q16s_kernel<0, 0, false>, dim3(grid_s), dim3(256), smem_s, s, xp, p, tw_shift, ck_shift, IH, IW, yp);
      }
      return;
    }
  }
  if (g.kh == 3 && g.kw == 3) {
    if (x_signed) launch_pdl(depthwise_q16_kernel<3, 3, true>, dim3(grid), dim3(256), smem, s, xp, p, yp);
    else launch_pdl(depthwise_q16_kernel<3, 3, false>, dim3(grid), dim3(256), smem, s, xp, p, yp);
  } else {
    if (x_signed) launch_pdl(depthwise_q16_kernel<0, 0, true>, dim3(grid), dim3(256), smem, s, xp, p, yp);
    else launch_pdl(depthwise_q16_kernel<0, 0, false>, dim3(grid), dim3(256), smem, s, xp, p, yp);
  }
}

void launch_conv_f32(const float* x, const float* w, const float* bias, int multiplier, int w_ic, const ConvGeom& g,
                     float* y, cudaStream_t s) {
  const long long total = static_cast<long long>(g.N) * g.Ho * g.Wo * g.Oc;
  if (total == 0) return;
  conv_f32_kernel<<<grid_for(total, kThreads), kThreads, 0, s>>>(x, w, bias, multiplier, w_ic, g, y);
}

void launch_pool_q(const void* x, int is_signed, int type, float in_scale, int in_zp, int same_quant, const ConvGeom& g,
                   OutQuant out, void* y, cudaStream_t s) {
  const uint8_t* xp = static_cast<const uint8_t*>(x);
  uint8_t* yp = static_cast<uint8_t*>(y);
  if (type != 2 && g.kw * g.kh <= 256 && g.dx == 1 && g.dy == 1) {   // (L2 pooling runs the general kernel)
    const long long total = static_cast<long long>(g.N) * g.Ho * g.Wo * (g.Cp / 16);
    if (total == 0) return;
    if (g.kw * g.kh >= 32 && total <= 148LL * 2048 / 32 * 8) {
      // few outputs, many taps each: a warp per output chunk
      if (is_signed) launch_pdl(pool_q16_warp_kernel<true>, dim3(grid_for(total * 32, 256)), dim3(256), 0, s, xp, type, in_scale, in_zp, same_quant, g, out, yp);
      else launch_pdl(pool_q16_warp_kernel<false>, dim3(grid_for(total * 32, 256)), dim3(256), 0, s, xp, type, in_scale, in_zp, same_quant, g, out, yp);
      return;
    }
    // Max pooling that keeps the quantization, 3x3 or 2x2 window, stride 2, padding smaller than the window: 2 x 2 outputs per
    // thread (B2VX_POOL_2X2=0: one output per thread as for every other pooling)
    static const bool no_2x2 = [] { const char* e = std::getenv("B2VX_POOL_2X2"); return e && std::strcmp(e, "0") == 0; }();
    if (!no_2x2 && type == 0 && same_quant && g.kw == g.kh && (g.kw == 3 || g.kw == 2) && g.sx == 2 && g.sy == 2 && g.pl < g.kw && g.pt < g.kh &&
        (g.Wo - 1) * 2 - g.pl <= g.W - 1 && (g.Ho - 1) * 2 - g.pt <= g.H - 1) {   // every window holds a tap of the image
      const long long blocks4 = static_cast<long long>(g.N) * ((g.Ho + 1) / 2) * ((g.Wo + 1) / 2) * (g.Cp / 16);
      const dim3 grid4(grid_for(blocks4, 256));
      if (g.kw == 3) {
        if (is_signed) launch_pdl(pool_max2x2_kernel<true, 3, 2>, grid4, dim3(256), 0, s, xp, g, yp);
        else launch_pdl(pool_max2x2_kernel<false, 3, 2>, grid4, dim3(256), 0, s, xp, g, yp);
      } else {
        if (is_signed) launch_pdl(pool_max2x2_kernel<true, 2, 2>, grid4, dim3(256), 0, s, xp, g, yp);
        else launch_pdl(pool_max2x2_kernel<false, 2, 2>, grid4, dim3(256), 0, s, xp, g, yp);
      }
      return;
    }
    const dim3 grid(grid_for(total, 256));
#define B2VX_POOL_LAUNCH(XS_, K_) launch_pdl(pool_q16_kernel<XS_, K_>, grid, dim3(256), 0, s, xp, type, in_scale, in_zp, same_quant, g, out, yp)
    if (g.kw == 3 && g.kh == 3) { if (is_signed) B2VX_POOL_LAUNCH(true, 3); else B2VX_POOL_LAUNCH(false, 3); }
    else if (g.kw == 2 && g.kh == 2) { if (is_signed) B2VX_POOL_LAUNCH(true, 2); else B2VX_POOL_LAUNCH(false, 2); }
    else { if (is_signed) B2VX_POOL_LAUNCH(true, 0); else B2VX_POOL_LAUNCH(false, 0); }
#undef B2VX_POOL_LAUNCH
    return;
  }
  const long long total = static_cast<long long>(g.N) * g.Ho * g.Wo * (g.Cp / 4);
  if (total == 0) return;
  if (is_signed) pool_q_kernel<true><<<grid_for(total, kThreads), kThreads, 0, s>>>(xp, type, in_scale, in_zp, same_quant, g, out, yp);
  else pool_q_kernel<false><<<grid_for(total, kThreads), kThreads, 0, s>>>(xp, type, in_scale, in_zp, same_quant, g, out, yp);
}

void launch_pool_f32(const float* x, int type, const ConvGeom& g, float* y, cudaStream_t s) {
  const long long total = static_cast<long long>(g.N) * g.Ho * g.Wo * g.C;
  if (total == 0) return;
  pool_f32_kernel<<<grid_for(total, kThreads), kThreads, 0, s>>>(x, type, g, y);
}

void launch_add_q(const void* a, int a_signed, float sa, int za, const void* b, int b_signed, float sb, int zb,
                  OutQuant out, int out_signed, void* y, size_t n, cudaStream_t s) {
  const size_t n16 = n / 16;
  if (n16 == 0) return;
  AddParams p;
  p.sa = sa; p.sb = sb; p.scale = out.scale;
  p.za = za; p.zb = zb;
  p.a_flip = a_signed ? 0x80808080u : 0u;
  p.b_flip = b_signed ? 0x80808080u : 0u;
  p.ca = -(8388608.0f + static_cast<float>(za + (a_signed ? 128 : 0)));
  p.cb = -(8388608.0f + static_cast<float>(zb + (b_signed ? 128 : 0)));
  const float inv = 1.0f / out.scale;
  p.inv_hi = inv * (1.0f + 4.76837158203125e-7f);
  p.inv_lo = inv * (1.0f - 4.76837158203125e-7f);
  p.magic = 12582912.0f + static_cast<float>(out.zp);
  p.out = out;
  p.out_signed = out_signed;
  // the saturating pack clamps to the type's range; a narrower range or a huge scale ratio takes the exact path
  const bool full_range = out_signed ? (out.lo == -128 && out.hi == 127) : (out.lo == 0 && out.hi == 255);
  const float bound = 256.0f * (fabsf(sa) + fabsf(sb)) * fabsf(inv) + 512.0f;
  const bool fast = full_range && bound < B2VX_FAST_ROUND_LIMIT && out.scale > 0.0f && std::isfinite(inv);
  // two 16-element steps per thread keep enough loads in flight; at most 8 blocks per SM
  unsigned grid = grid_for(static_cast<long long>((n16 + 3) / 4), 256);
  if (grid > 148u * 8u) grid = 148u * 8u;
  const uint4* pa = static_cast<const uint4*>(a);
  const uint4* pb = static_cast<const uint4*>(b);
  uint4* py = static_cast<uint4*>(y);
  if (fast) launch_pdl(add_q_kernel<true>, dim3(grid), dim3(256), 0, s, pa, pb, p, py, n16);
  else launch_pdl(add_q_kernel<false>, dim3(grid), dim3(256), 0, s, pa, pb, p, py, n16);
}

// AddN: one element per thread (the op is rare on the path; the two-input case runs the tuned Add kernels).
template <int ELEM>
__global__ void __launch_bounds__(256) addn_kernel(AddNParams p, void* __restrict__ y, size_t n) {
  pdl_wait();
  pdl_trigger();
  const size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (i >= n) return;
  float r = 0.0f;
#pragma unroll 1
  for (int k = 0; k < p.n_in; ++k) {
    float v;
    if (ELEM == 4) {
      v = static_cast<const float*>(p.x[k])[i];
    } else {
      const int q = p.is_signed[k] ? static_cast<int>(static_cast<const int8_t*>(p.x[k])[i]) : static_cast<int>(static_cast<const uint8_t*>(p.x[k])[i]);
      v = __fmul_rn(__int2float_rn(q - p.zp[k]), p.scale[k]);
    }
    r = k == 0 ? v : __fadd_rn(r, v);
  }
  if (ELEM == 4) static_cast<float*>(y)[i] = r;
  else static_cast<uint8_t*>(y)[i] = static_cast<uint8_t>(requant(r, p.out) & 0xFF);
}

void launch_addn(const AddNParams& p, int elem, void* y, size_t n, cudaStream_t s) {
  if (n == 0) return;
  const unsigned grid = grid_for(static_cast<long long>(n), 256);
  if (elem == 4) launch_pdl(addn_kernel<4>, dim3(grid), dim3(256), 0, s, p, y, n);
  else launch_pdl(addn_kernel<1>, dim3(grid), dim3(256), 0, s, p, y, n);
}

void launch_add_q_lut(const void* a, const void* b, const uint8_t* table, void* y, size_t n, cudaStream_t s) {
  const size_t n16 = n / 16;
  if (n16 == 0) return;
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !attr_set[dev]) {
    cudaFuncSetAttribute(add_q_lut_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536);
    if (dev >= 0 && dev < 64) attr_set[dev] = true;
  }
  // three 64 KB blocks per SM; every block should have enough elements to repay its table load
  // 1024 threads share one table: two blocks (64 warps, the SM's maximum) per SM
  unsigned grid = grid_for(static_cast<long long>((n16 + 7) / 8), 1024);
  if (grid > 148u * 2u) grid = 148u * 2u;
  launch_pdl(add_q_lut_kernel, dim3(grid), dim3(1024), 65536, s, static_cast<const uint4*>(a), static_cast<const uint4*>(b),
                                            reinterpret_cast<const uint4*>(table), static_cast<uint4*>(y), n16);
}

void launch_add_broadcast(const void* a, int a_signed, float sa, int za, const int a_dims[5], const void* b, int b_signed, float sb,
                          int zb, const int b_dims[5], OutQuant out, const int y_dims[5], int elem, void* y, cudaStream_t s) {
  BroadcastGeom g;
  g.N = y_dims[0]; g.H = y_dims[1]; g.W = y_dims[2]; g.C = y_dims[3]; g.Cp = y_dims[4];
  auto strides = [&](const int d[5], long long st[4]) {
    const long long full[4] = {static_cast<long long>(d[1]) * d[2] * d[4], static_cast<long long>(d[2]) * d[4], d[4], 1};
    for (int k = 0; k < 4; ++k) st[k] = (d[k] == 1 && y_dims[k] != 1) ? 0 : full[k];
  };
  strides(a_dims, g.as);
  strides(b_dims, g.bs);
  const long long total = static_cast<long long>(g.N) * g.H * g.W * g.C;
  if (total == 0) return;
  if (elem == 4)
    add_broadcast_kernel<uint32_t><<<grid_for(total, kThreads), kThreads, 0, s>>>(static_cast<const uint32_t*>(a), sa, za, a_signed,
                                                                                static_cast<const uint32_t*>(b), sb, zb, b_signed, out, g,
                                                                                static_cast<uint32_t*>(y));
  else
    add_broadcast_kernel<uint8_t><<<grid_for(total, kThreads), kThreads, 0, s>>>(static_cast<const uint8_t*>(a), sa, za, a_signed,
                                                                               static_cast<const uint8_t*>(b), sb, zb, b_signed, out, g,
                                                                               static_cast<uint8_t*>(y));
}

void launch_add_i32(const int* a, float sa, int za, const int* b, float sb, int zb, OutQuant out, int* y, size_t n, cudaStream_t s) {
  if (n == 0) return;
  add_i32_kernel<<<grid_for(static_cast<long long>(n), kThreads), kThreads, 0, s>>>(a, sa, za, b, sb, zb, out, y, n);
}

void launch_add_f32(const float* a, const float* b, float* y, size_t n, cudaStream_t s) {
  if (n == 0) return;
  add_f32_kernel<<<grid_for(static_cast<long long>(n), kThreads), kThreads, 0, s>>>(a, b, y, n);
}

void launch_relayout(const void* in, void* out, const RelayoutParams& p, cudaStream_t s) {
  if (p.total <= 0) return;
  const uint8_t* ip0 = static_cast<const uint8_t*>(in);
  uint8_t* op0 = static_cast<uint8_t*>(out);
  if (p.convert == 0 && p.elem == 1 && !p.reshape && p.rank >= 2 && p.ostride[0] == 1 && p.istride[0] != 1 && p.dims[0] >= 16) {
    int kb = -1;
    for (int k = 1; k < p.rank; ++k)
      if (p.istride[k] == 1 && p.dims[k] >= 16) kb = k;
    long long others = 1;
    for (int k = 1; k < p.rank; ++k)
      if (k != kb) others *= p.dims[k];
    if (kb > 0 && others <= 65535 && (p.dims[kb] + 31) / 32 <= 65535) {
      const dim3 grid((p.dims[0] + 31) / 32, (p.dims[kb] + 31) / 32, static_cast<unsigned>(others));
      relayout_tiled_kernel<<<grid, dim3(32, 8), 0, s>>>(ip0, op0, p, kb);
      return;
    }
  }
  const int run = p.dims[0] < 16 ? p.dims[0] : 16;
  const int runs0 = (p.dims[0] + run - 1) / run;
  const long long n_threads = p.total / p.dims[0] * runs0;
  const uint8_t* ip = static_cast<const uint8_t*>(in);
  uint8_t* op = static_cast<uint8_t*>(out);
  if (p.total < (1ll << 31)) relayout_kernel<unsigned><<<grid_for(n_threads, kThreads), kThreads, 0, s>>>(ip, op, p, run, runs0, n_threads);
  else relayout_kernel<unsigned long long><<<grid_for(n_threads, kThreads), kThreads, 0, s>>>(ip, op, p, run, runs0, n_threads);
}

void launch_concat_c16(const void* in, int in_pitch16, int in16, void* out, int out_pitch16, int off16, long long pixels, cudaStream_t s) {
  const long long total = pixels * in16;
  if (total <= 0) return;
  concat_c16_kernel<<<grid_for(total, kThreads), kThreads, 0, s>>>(static_cast<const uint4*>(in), in_pitch16, in16, static_cast<uint4*>(out),
                                                                   out_pitch16, off16, total);
}

void launch_lut_q(const void* x, const uint8_t* lut, void* y, size_t n, cudaStream_t s) {
  const size_t n16 = n / 16;
  if (n16 == 0) return;
  unsigned grid = grid_for(static_cast<long long>(n16), kThreads);
  if (grid > 148u * 16u) grid = 148u * 16u;
  launch_pdl(lut_q_kernel, dim3(grid), dim3(kThreads), 0, s, static_cast<const uint4*>(x), lut, static_cast<uint4*>(y), n16);
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

// The same shapes with 9 to 16 rows (and large ones with fewer): weight streaming through the warp-level
// integer MMA, mma.sync m16n8k32: the sixteen input rows are the MMA's M, eight output channels its N.
// A block of eight warps owns 32 output channels (four n-tiles per warp, so that the input fragments
// are loaded once for four MMAs) and splits K in 64-byte pieces among its warps.  K is a reduction
// dimension, so any assignment of bytes to the MMA's k positions is right as long as both operands use
// the same one: a lane's 16-byte load of a weight row (k bytes 16q .. 16q+15 of the piece, q = lane % 4)
// feeds two MMAs, words (0,1) and (2,3), and the same words of the two input rows it loads are the A
// fragments.  All HBM traffic is 128-bit loads of 128 contiguous bytes per row and step.  (Tried and dropped:
// 16-byte asynchronous copies into a six-deep ring in shared memory, 1.4 times slower.)  Partial sums of the
// eight warps meet in shared memory; the requantization is the exact sequence.
// HAS_DZ: weights keep a zero point dz, removed as dz * sum(x) from an MMA against all-ones bytes.
template <bool XS>
__device__ __forceinline__ void mma_m16n8k32(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  if (XS)
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  else
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <bool XS, bool HAS_DZ>
__global__ void __launch_bounds__(256, 2) fc_mma16_kernel(const uint8_t* __restrict__ A, const int8_t* __restrict__ B, int M, int Kp,
                                                          int Oc, int Ocp, ContractEpilogue ep, uint8_t* __restrict__ D, int ldd) {
  pdl_wait();
  pdl_trigger();
  constexpr int NT = 4;                              // n-tiles of eight channels per warp
  __shared__ int partial[8][16][NT * 8 + 1];
  __shared__ int s_sum[8][16];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int q = lane & 3, r = lane >> 2;             // k quarter of a piece; row (and channel within an n-tile)
  const int c0 = blockIdx.x * (NT * 8);
  int acc[NT][4];
#pragma unroll
  for (int t = 0; t < NT; ++t)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[t][i] = 0;
  int accs[4] = {0, 0, 0, 0};
  const bool row_lo = r < M, row_hi = r + 8 < M;
  const uint8_t* a_lo = A + static_cast<size_t>(row_lo ? r : 0) * Kp + q * 16;
  const uint8_t* a_hi = A + static_cast<size_t>(row_hi ? r + 8 : 0) * Kp + q * 16;
  const int8_t* b_row[NT];
  bool b_ok[NT];
#pragma unroll
  for (int t = 0; t < NT; ++t) {
    const int ch = c0 + 8 * t + r;
    b_ok[t] = ch < Ocp;
    b_row[t] = B + static_cast<size_t>(b_ok[t] ? ch : 0) * Kp + q * 16;
  }
  // Every warp takes one contiguous eighth of K (in whole pieces), so that its successive loads of a weight row
  // are neighbours in memory; two pieces (128 bytes per row) per step, all ten loads issued before the first MMA.
  const int pieces = (Kp + 63) >> 6;
  const int per_warp = (pieces + 7) >> 3;
  const int p_begin = warp * per_warp, p_end = min(pieces, p_begin + per_warp);
  const uint4 zero4 = make_uint4(0, 0, 0, 0);
#pragma unroll 1
  for (int p0 = p_begin; p0 < p_end; p0 += 2) {
    uint4 w[2][NT], xl[2], xh[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int k = (p0 + u) * 64;
      const bool k_ok = p0 + u < p_end && k + q * 16 < Kp;
#pragma unroll
      for (int t = 0; t < NT; ++t) w[u][t] = (k_ok && b_ok[t]) ? __ldcs(reinterpret_cast<const uint4*>(b_row[t] + k)) : zero4;
      xl[u] = (k_ok && row_lo) ? __ldg(reinterpret_cast<const uint4*>(a_lo + k)) : zero4;
      xh[u] = (k_ok && row_hi) ? __ldg(reinterpret_cast<const uint4*>(a_hi + k)) : zero4;
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        mma_m16n8k32<XS>(acc[t], xl[u].x, xh[u].x, xl[u].y, xh[u].y, w[u][t].x, w[u][t].y);
        mma_m16n8k32<XS>(acc[t], xl[u].z, xh[u].z, xl[u].w, xh[u].w, w[u][t].z, w[u][t].w);
      }
      if (HAS_DZ) {
        mma_m16n8k32<XS>(accs, xl[u].x, xh[u].x, xl[u].y, xh[u].y, 0x01010101u, 0x01010101u);
        mma_m16n8k32<XS>(accs, xl[u].z, xh[u].z, xl[u].w, xh[u].w, 0x01010101u, 0x01010101u);
      }
    }
  }
  // accumulator layout: c0, c1 = (row r, channels 2q, 2q+1), c2, c3 = (row r + 8, the same channels)
#pragma unroll
  for (int t = 0; t < NT; ++t) {
    partial[warp][r][8 * t + 2 * q] = acc[t][0];
    partial[warp][r][8 * t + 2 * q + 1] = acc[t][1];
    partial[warp][r + 8][8 * t + 2 * q] = acc[t][2];
    partial[warp][r + 8][8 * t + 2 * q + 1] = acc[t][3];
  }
  if (HAS_DZ && q == 0) {
    s_sum[warp][r] = accs[0];
    s_sum[warp][r + 8] = accs[2];
  }
  __syncthreads();
  for (int o = threadIdx.x; o < 16 * NT * 8; o += 256) {
    const int m = o / (NT * 8), c = o - m * (NT * 8);
    const int oc = c0 + c;
    if (m >= M || oc >= Oc) continue;
    int total = 0, sx = 0;
#pragma unroll
    for (int w8 = 0; w8 < 8; ++w8) {
      total += partial[w8][m][c];
      if (HAS_DZ) sx += s_sum[w8][m];
    }
    if (HAS_DZ) total -= ep.dz_uniform * sx;
    const float real = __fmul_rn(__int2float_rn(total + ep.bias_full[oc]), ep.acc_scale[oc]);
    D[static_cast<size_t>(m) * ldd + oc] = static_cast<uint8_t>(requant(real, ep.out) & 0xFF);
  }
}

template <int CH, int MT>
static void launch_fc_small_m_t(const void* A, int a_signed, const int8_t* B, int M, int Kp, int Oc, int Ocp,
                                const ContractEpilogue& e, void* D, int ldd, cudaStream_t s) {
  const uint8_t* a = static_cast<const uint8_t*>(A);
  uint8_t* d = static_cast<uint8_t*>(D);
  const unsigned grid = static_cast<unsigned>((Ocp + CH - 1) / CH);   // one block per channel group
  const bool dz = e.dz_uniform != 0;
  if (a_signed) {
    if (dz) launch_pdl(fc_small_m_kernel<CH, MT, true, true>, dim3(grid), dim3(256), 0, s, a, B, M, Kp, Oc, Ocp, e, d, ldd);
    else launch_pdl(fc_small_m_kernel<CH, MT, true, false>, dim3(grid), dim3(256), 0, s, a, B, M, Kp, Oc, Ocp, e, d, ldd);
  } else {
    if (dz) launch_pdl(fc_small_m_kernel<CH, MT, false, true>, dim3(grid), dim3(256), 0, s, a, B, M, Kp, Oc, Ocp, e, d, ldd);
    else launch_pdl(fc_small_m_kernel<CH, MT, false, false>, dim3(grid), dim3(256), 0, s, a, B, M, Kp, Oc, Ocp, e, d, ldd);
  }
}

void launch_fc_small_m(const void* A, int a_signed, const int8_t* B, int M, int Kp, int Oc, int Ocp, const ContractEpilogue& e,
                       void* D, int ldd, cudaStream_t s) {
  if (M <= 0 || Ocp <= 0) return;
  // B2VX_FC_MMA=0 keeps every shape on the dp4a kernel; 1 sends every shape to the MMA kernel (tuning aids)
  static const int fc_mma = [] { const char* v = std::getenv("B2VX_FC_MMA"); return v ? std::atoi(v) : -1; }();
  const bool use_mma = fc_mma == 1 || (fc_mma != 0 && M > 1);
  if (use_mma && M <= 16) {
    const uint8_t* a = static_cast<const uint8_t*>(A);
    uint8_t* d = static_cast<uint8_t*>(D);
    const unsigned grid = static_cast<unsigned>((Ocp + 31) / 32);
    const bool dz = e.dz_uniform != 0;
    if (a_signed) {
      if (dz) launch_pdl(fc_mma16_kernel<true, true>, dim3(grid), dim3(256), 0, s, a, B, M, Kp, Oc, Ocp, e, d, ldd);
      else launch_pdl(fc_mma16_kernel<true, false>, dim3(grid), dim3(256), 0, s, a, B, M, Kp, Oc, Ocp, e, d, ldd);
    } else {
      if (dz) launch_pdl(fc_mma16_kernel<false, true>, dim3(grid), dim3(256), 0, s, a, B, M, Kp, Oc, Ocp, e, d, ldd);
      else launch_pdl(fc_mma16_kernel<false, false>, dim3(grid), dim3(256), 0, s, a, B, M, Kp, Oc, Ocp, e, d, ldd);
    }
    return;
  }
  if (M <= 1) launch_fc_small_m_t<4, 1>(A, a_signed, B, M, Kp, Oc, Ocp, e, D, ldd, s);
  else if (M <= 4) launch_fc_small_m_t<4, 4>(A, a_signed, B, M, Kp, Oc, Ocp, e, D, ldd, s);
  else if (M <= 8) launch_fc_small_m_t<4, 8>(A, a_signed, B, M, Kp, Oc, Ocp, e, D, ldd, s);
  else launch_fc_small_m_t<4, 16>(A, a_signed, B, M, Kp, Oc, Ocp, e, D, ldd, s);
}

void launch_im2col_whcn8(const void* x, int Kp, int zx, const ConvGeom& g, int padk, void* col, cudaStream_t s) {
  if (g.N == 0 || g.Ho == 0 || g.Wo == 0) return;
  const int pitch = im2col_whcn8_pitch(g, padk);
  const size_t smem = static_cast<size_t>(g.C) * g.kh * pitch + 16;
  dim3 grid(g.Ho, g.N);
  if (padk == 8)
    launch_pdl(im2col_whcn8_kernel<8>, dim3(grid), dim3(256), smem, s, static_cast<const uint8_t*>(x), Kp, zx, g, pitch,
               static_cast<uint8_t*>(col));
  else
    launch_pdl(im2col_whcn8_kernel<4>, dim3(grid), dim3(256), smem, s, static_cast<const uint8_t*>(x), Kp, zx, g, pitch,
               static_cast<uint8_t*>(col));
}
int im2col_whcn8_pitch(const ConvGeom& g, int padk) {
  // up to 3 bytes of alignment lead, the padk-byte read of the last pixel, the last word of the funnel
  // shift; 4 mod 64 spreads consecutive rows over the banks
  const int need = 3 + (g.Wo - 1) * g.sx + padk + 4;
  int pitch = (need + 3) & ~3;
  while ((pitch & 63) != 4) pitch += 4;
  return pitch;
}

void launch_im2col_whcn(const void* x, int Kp, int zx, const ConvGeom& g, void* col, cudaStream_t s) {
  if (g.N == 0 || g.Ho == 0 || g.Wo == 0) return;
  // input columns a row of outputs touches, counted from -pad_left
  const int rowlen = (g.Wo - 1) * g.sx + (g.kw - 1) * g.dx + 1;
  const size_t smem = static_cast<size_t>(Kp) * sizeof(int) + static_cast<size_t>(g.C) * g.kh * rowlen;
  dim3 grid(g.Ho, g.N);
  launch_pdl(im2col_whcn_kernel, dim3(grid), dim3(256), smem, s, static_cast<const uint8_t*>(x), Kp, zx, g, rowlen, static_cast<uint8_t*>(col));
}

}  // namespace b2vx
