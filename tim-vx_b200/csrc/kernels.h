// Launch wrappers of the sm_100a kernels behind the b2vx C ABI.
//
// Device layout of an activation tensor with tim::vx shape [W,H,C,N] (lower
// ranks are padded with ones: [K,B] is C=K, N=B): channels-last, dense,
//     addr(n,h,w,c) = ((n*H + h)*W + w)*Cp + c,   Cp = C rounded up to 16 bytes,
// so a pixel's channels are one contiguous, 16-byte aligned run — the unit of
// every 128-bit load below and the K-contiguous ("K-major") operand layout the
// tensor-core GEMM wants.  Bytes in the channel padding are don't-care: packed
// weights are zero there, and per-channel kernels carry them along untouched.
//
// Quantized outputs are produced by replaying the reference's float sequence
// (affine_to_fp32 then fp32_to_affine,
// src/tim/vx/internal/include/utils/vsi_nn_dtype_util_prv.h:228-266, with the
// vsi_rint tie rule of include/utils/vsi_nn_math.h:191-210) with explicit
// round-to-nearest intrinsics, never a fused multiply-add.
#ifndef B2VX_KERNELS_H_
#define B2VX_KERNELS_H_

#include <cuda_runtime.h>
#include <stdint.h>

namespace b2vx {

// Output quantization of a kernel: q = clamp(rint(real / scale) + zp, lo, hi).
struct OutQuant {
  float scale;
  int32_t zp;
  int32_t lo;
  int32_t hi;
};

// Geometry of one convolution / pooling window sweep over channels-last data.
struct ConvGeom {
  int N, H, W, C, Cp;        // input
  int Ho, Wo, Oc, Ocp;       // output
  int kh, kw, sy, sx, dy, dx, pt, pl;
};

// Per-output-channel epilogue tables of a quantized contraction (device
// pointers, Ocp entries each; tapc is [kh*kw][Ocp] or null).
//   acc = A - dz[oc]*S + bias_full[oc] - sum over out-of-bounds taps of tapc[tap][oc]
//   real = float(acc) * acc_scale[oc]
// A is the raw sum of x*w8 over in-bounds taps (w8 = weight shifted into int8),
// S the raw sum of x over the same taps (needed only when some dz != 0).
struct ContractEpilogue {
  const int32_t* bias_full;
  const float* acc_scale;
  const int32_t* dz;         // null when all zero
  const int32_t* tapc;       // null when the input zero point is 0 or there is no padding
  OutQuant out;
  int out_is_float;          // write float(acc)*acc_scale instead of quantizing
  // Tensor-core epilogue only: 1 = requantize with the exact sequence only.  The fast form needs
  // |acc * acc_scale / out.scale| < 2^21 for every possible accumulator, which the planner checks
  // from K, the bias and the scales.
  int exact_only;
  // Tensor-core path, weights with one zero point left over (dz_uniform = zw - 128 for uint8 weights):
  // the packed weights carry an all-ones row per N tile, whose accumulator column is S.
  int dz_uniform;
  // Tensor-core implicit convolution with a non-zero input zero point and padding: out-of-bounds taps
  // read as 0 instead of the zero point, which the bias folding assumed.  Output rows/columns are
  // classified by their set of out-of-bounds taps (row_class[Ho], col_class[Wo], class 0 = none) and
  // border_corr[(row_class * n_col_classes + col_class) * Ocp + oc] is added to the accumulator.
  const int32_t* border_corr;   // null = no correction
  const uint8_t* row_class;
  const uint8_t* col_class;
  int n_col_classes;
  // Tensor-core path, residual Add fused into the epilogue: the convolution's own quantized byte q
  // (quantization `out`) and the byte r at the same position of `add_residual` (a channels-last tensor
  // of the output's shape) are replaced by add_table[q*256 + (r ^ ((q & 31) << 2))], the 64 KB table
  // of the Add that follows (launch_add_q_lut's layout, first operand = this convolution).
  const uint8_t* add_residual;  // null = no fused Add
  const uint8_t* add_table;
};

// ---- layout converters (elem = 1 or 4 bytes) -------------------------------
void launch_whcn_to_cl(const void* src, void* dst, int N, int C, int H, int W, int Cp, int elem, cudaStream_t s);
void launch_cl_to_whcn(const void* src, void* dst, int N, int C, int H, int W, int Cp, int elem, cudaStream_t s);

// ---- quantized contraction on CUDA cores (any shape; the fallback path) ----
// w8: [rows][Kp] int8, row oc holds K = (tap*Cp + c), Ocp rows; when e.dz != null
// one more row (index Ocp) follows: the all-ones row whose dot product is S.
void launch_conv_simt(const void* x, int x_signed, const int8_t* w8, int Kp, const ConvGeom& g,
                      const ContractEpilogue& e, void* y, cudaStream_t s);

// ---- depthwise convolution, quantized: wd [kh*kw][Ocp] int16 = w - zw -------
void launch_depthwise_q(const void* x, int x_signed, int zx, const int16_t* wd, const int32_t* bias,
                        const float* acc_scale, int multiplier, const ConvGeom& g, OutQuant out,
                        void* y, cudaStream_t s);

// The multiplier-1 case, 16 channels x 2 pixels per thread with the weights in shared memory:
// wtab [kh*kw][Ocp] words, each w - zw as a 16-bit half in position (channel & 1);
// bias_full = bias - zx' * sum_taps (w - zw) with zx' = zx (+128 for int8 input).  Needs kh*kw <= 64.
// wtab_v (3x3 windows; else null) selects, for strides 1 and 2 without dilation, the form with 4 channels x 8 pixels
// per thread: [6][Ocp] words, row kx < 3 = the halves (w[0][kx] - zw, w[1][kx] - zw) of a channel, row 3 + kx = wtab's
// row of tap (2, kx).
void launch_depthwise_q16(const void* x, int x_signed, int zx, const uint32_t* wtab, const uint32_t* wtab_v, const int32_t* bias_full,
                          const float* acc_scale, const ConvGeom& g, OutQuant out, int exact_only, void* y, cudaStream_t s);

// ---- float32 convolution (dense or depthwise), accumulation order ic,ky,kx --
// w: original WHIcOc layout; bias may be null.
void launch_conv_f32(const float* x, const float* w, const float* bias, int multiplier, int w_ic,
                     const ConvGeom& g, float* y, cudaStream_t s);

// ---- pooling: type 0 max, 1 avg (divide by kw*kh), 2 L2 (sqrt of the mean square over valid taps), 3 avg over valid taps ----
void launch_pool_q(const void* x, int is_signed, int type, float in_scale, int in_zp, int same_quant,
                   const ConvGeom& g, OutQuant out, void* y, cudaStream_t s);
void launch_pool_f32(const float* x, int type, const ConvGeom& g, float* y, cudaStream_t s);

// ---- elementwise over n elements of channels-last storage -------------------
void launch_add_q(const void* a, int a_signed, float sa, int za, const void* b, int b_signed, float sb, int zb,
                  OutQuant out, int out_signed, void* y, size_t n, cudaStream_t s);
// The same Add through a 64 KB byte table in shared memory (exact whatever the data; chosen for large
// tensors): table[a*256 + (b ^ ((a & 31) << 2))] = quantized sum for raw input bytes a, b.
void launch_add_q_lut(const void* a, const void* b, const uint8_t* table, void* y, size_t n, cudaStream_t s);
void launch_add_f32(const float* a, const float* b, float* y, size_t n, cudaStream_t s);
void launch_add_i32(const int* a, float sa, int za, const int* b, float sb, int zb, OutQuant out, int* y, size_t n, cudaStream_t s);
// Add with broadcasting over channels-last operands; dims = {N, H, W, C, Cp} of a, b and the output
// (a dimension of 1 repeats along the output's), elem = 1 (quantized) or 4 (float32).
void launch_add_broadcast(const void* a, int a_signed, float sa, int za, const int a_dims[5], const void* b, int b_signed, float sb,
                          int zb, const int b_dims[5], OutQuant out, const int y_dims[5], int elem, void* y, cudaStream_t s);
// ops::AddN over n_in (2..16) same-shaped channels-last tensors of n elements each: dequantize, add in float32 from
// left to right, quantize once.  elem = 1: int8/uint8 inputs and output; 4: float32 throughout.
struct AddNParams {
  const void* x[16];
  float scale[16];
  int zp[16];
  int is_signed[16];
  int n_in;
  OutQuant out;
  int out_signed;
};
void launch_addn(const AddNParams& p, int elem, void* y, size_t n, cudaStream_t s);
// y[i] = lut[x[i]] over n bytes: Relu/Relu6 between any two 8-bit quantizations,
// the 256-entry device table being built on the host with the reference's float sequence
void launch_lut_q(const void* x, const uint8_t* lut, void* y, size_t n, cudaStream_t s);

// Data movement between storages (Reshape, Transpose, Concat pieces, DataConvert).  The iteration space is a
// logical shape of up to four dimensions, dimension 0 fastest (the host lists the dimensions by increasing
// output stride, so that consecutive threads write neighbouring bytes); each element goes from
//   in  + sum(coord_in[k]  * istride[k])      to      out + sum(coord[k] * ostride[k])
// (strides in elements) where coord_in = coord, or, with `reshape`, the coordinates of the same dense
// linear index under the input's own shape idims.
struct RelayoutParams {
  int rank;
  int dims[4];
  long long ostride[4];
  long long istride[4];
  int reshape;
  long long lstride[4];   // reshape: dense (WHCN-order) strides of the iteration dimensions, to form the linear index
  int idims[4];
  long long total;
  // 0: raw copy of `elem`-byte elements; 1: bytes through the 256-entry table `lut`;
  // 2: float32 -> 8-bit with `out` (requant); 3: 8-bit (in_signed) -> float32 with in_scale / in_zp
  int convert;
  int elem;
  const uint8_t* lut;
  OutQuant out;
  float in_scale;
  int in_zp;
  int in_signed;
};
void launch_relayout(const void* in, void* out, const RelayoutParams& p, cudaStream_t s);
// Concat of 8-bit channels-last tensors along the channel axis when every extent is a multiple of 16:
// per pixel, in16 16-byte pieces go to out + pixel * out_pitch16 + off16.
void launch_concat_c16(const void* in, int in_pitch16, int in16, void* out, int out_pitch16, int off16, long long pixels, cudaStream_t s);
// upper < 0: relu, else clamp to [0, upper]
void launch_relu_f32(const float* x, float upper, float* y, size_t n, cudaStream_t s);

// ---- softmax along one axis of a channels-last tensor ----------------------
// Input and output may differ in element size (u8 in, f32 out), hence in
// channel padding, so each side has its own element strides.  The reduced axis
// is (len, x_stride/y_stride); the other three axes enumerate the slices.
struct SoftmaxGeom {
  int len; long long x_stride, y_stride;
  int o[3]; long long xs[3], ys[3];
};
// x_kind: 0 u8, 1 s8, 2 f32.  y_kind likewise.
void launch_softmax(const void* x, int x_kind, float sx, int zx, void* y, int y_kind, OutQuant out, float beta,
                    const SoftmaxGeom& g, cudaStream_t s);

// ---- FullyConnected / 1x1-on-one-pixel with at most 16 rows, on CUDA cores ----
// D[M][ldd] = requant(A[M][Kp] * B[Ocp][Kp]^T): B is the packed weight matrix with plain row order
// (one N tile, no ones row), e.bias_full / e.acc_scale / e.out / e.dz_uniform as for the GEMM; with
// dz_uniform != 0 every byte of A's rows must be real data (K == Kp).
void launch_fc_small_m(const void* A, int a_signed, const int8_t* B, int M, int Kp, int Oc, int Ocp, const ContractEpilogue& e,
                       void* D, int ldd, cudaStream_t s);

// ---- explicit im2col for the tensor-core GEMM -------------------------------
// col [M][Kp] bytes, M = N*Ho*Wo, K index = tap*Cs + c with Cs = g.C (dense) or
// g.Cp; out-of-bounds taps are filled with the input zero point, the K tail
// (and the channel padding when Cs = Cp) with zero.
void launch_im2col(const void* x, int Cs, int Kp, int zx, const ConvGeom& g, void* col, cudaStream_t s);

// The same matrix straight from a WHCN tensor [N][C][H][W] with few channels (network inputs):
// K index = (c*kh + ky)*kw + kx, the kernel tensor's own element order.
void launch_im2col_whcn(const void* x, int Kp, int zx, const ConvGeom& g, void* col, cudaStream_t s);
// The same for filters up to padk = 8 or 4 wide (dilation 1) with K index = (ky*C + c)*padk + kx: every (pixel, ky, c)
// contributes padk consecutive input bytes, slot kx >= kw carrying a don't-care byte (zero weight).
// Shared memory needed per block: C * kh * im2col_whcn8_pitch(g, padk) + 16 bytes.
void launch_im2col_whcn8(const void* x, int Kp, int zx, const ConvGeom& g, int padk, void* col, cudaStream_t s);
int im2col_whcn8_pitch(const ConvGeom& g, int padk);

// ---- int8 GEMM on tcgen05 tensor cores --------------------------------------
// D[M][ldd] (u8/s8) = requant(A[M][Kp] (u8 or s8) * B[Np][Kp]^T (s8)), K-major
// operands fed by TMA, int32 accumulation in tensor memory.  Returns a CUDA
// error code; the kernel's bounded waits report through *status (device int,
// 0 = ok).
struct GemmTcPlan;   // opaque: tensor maps + launch geometry, built once at compile
// N tiling of a GEMM: n_tiles tiles of `data` output channels each.  The packed weight matrix has
// n_tiles * rows rows; inside a tile, rows [0, data) are output channels, and when rows > data row
// `data` is the all-ones row (S column) and the rest is zero.
struct GemmTcTiling {
  int n_tiles, data, rows;
};
// Picks the tiling for M x Ocp x Kp from a small cost model (waves of tiles over the SMs, operand
// bytes per tile, epilogue work per tile).  with_s: reserve 16 rows per tile for the ones row.
GemmTcTiling gemm_tc_choose_tiling(long long M, int Ocp, int Kp, int with_s);
// tiling == null: ceil(Np / 256) equal tiles of Np / n_tiles rows, no ones row.
GemmTcPlan* gemm_tc_plan_create(const void* A, int a_signed, const int8_t* B, int M, int Np, int Kp, int Oc,
                                void* D, int ldd, int d_signed, const ContractEpilogue& e, int* status,
                                char* err, size_t err_len, const GemmTcTiling* tiling = nullptr);
// Implicit-GEMM convolution on the same kernel: X is the channels-last input [N][H][W][Cp], B is
// [Np][kh*kw*Cp] with K = tap*Cp + c, D the channels-last output.  Filter taps are fetched as
// shifted 4-D TMA boxes; positions in the padding read as zero, so with a non-zero input zero point
// and padding the epilogue needs e.border_corr.
GemmTcPlan* gemm_tc_conv_plan_create(const void* X, int x_signed, const int8_t* B, const ConvGeom& g, int Np, void* D,
                                     const ContractEpilogue& e, int* status, char* err, size_t err_len,
                                     const GemmTcTiling* tiling = nullptr);
// The plain-GEMM plan built inside caller-provided storage (gemm_tc_plan_bytes() bytes, 64-byte aligned)
// instead of on the heap; not to be passed to gemm_tc_plan_destroy.
size_t gemm_tc_plan_bytes(void);
GemmTcPlan* gemm_tc_plan_build_in(void* storage, size_t storage_bytes, const void* A, int a_signed, const int8_t* B, int M,
                                  int Np, int Kp, void* D, int ldd, const ContractEpilogue& e, int* status, char* err,
                                  size_t err_len);
void gemm_tc_plan_destroy(GemmTcPlan* p);
// 1 when an implicit-convolution plan loads one input patch per tile and runs the taps on shifted views of it.
int gemm_tc_plan_is_halo(const GemmTcPlan* p);
cudaError_t gemm_tc_launch(const GemmTcPlan* p, cudaStream_t s);
// 1 when this build and device can run the tensor-core path.
int gemm_tc_available(void);
// Measured dense int8 rate of the tensor pipe on the current device, TOP/s (issue-rate microbenchmark: operands in
// shared memory, no epilogue); 0 when it cannot run.  status: device int for the bounded waits, as for the GEMM.
double gemm_tc_measure_int8_peak(int reps, int* sm_count, int* status);

}  // namespace b2vx
#endif  // B2VX_KERNELS_H_
