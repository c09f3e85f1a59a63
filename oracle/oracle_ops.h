/*
 * CPU oracle for the quantized-inference path — TEST INFRASTRUCTURE ONLY.
 *
 * A plain restatement, on the CPU, of what the reference computes for Conv2d
 * (dense and depthwise), FullyConnected, Pool2d, Add, Relu, Relu6 and Softmax
 * on WHCN tensors.  Only tests, the smoke check and the benchmark's CPU
 * baseline may call it; the product never does.
 *
 * The reference's arithmetic for these ops lives in a closed driver
 * (libOpenVX.so; calls at src/tim/vx/internal/src/kernel/vx/convolutional.c:534,
 * src/tim/vx/internal/src/ops/vsi_nn_op_fullconnect2.c:118,
 * src/tim/vx/internal/src/ops/vsi_nn_op_pool.c:144,
 * src/tim/vx/internal/src/kernel/vx/eltwise_vx.c:58), so this file follows the
 * visible definitions instead: the op equations in
 * prebuilt-sdk/x86_64_linux/include/VX/vx_khr_nn.h:836-915,1693-1744, the
 * rounding and saturation helpers in
 * src/tim/vx/internal/include/utils/vsi_nn_dtype_util_prv.h:170-266 and
 * src/tim/vx/internal/include/utils/vsi_nn_math.h:183-210, and the shape rules
 * in src/tim/vx/internal/src/utils/vsi_nn_util.c:203-235,483-588.
 *
 * Parity status: pinned by the reference's own unit-test vectors for
 * u8xu8 and s8xs8 (per-tensor and per-channel) convolution, depthwise
 * convolution, average pooling (within the 1 LSB those tests allow) and the
 * float32 index/padding tests.  u8 activations with per-channel s8 weights,
 * quantized FullyConnected, quantized Add/Relu/Relu6/MaxPool and whole
 * networks have no reference vector: for those this oracle is the definition
 * ("parity unpinned").
 *
 * All tensors are dense, dims[0] fastest.  dtype codes are the B2VX_DT_*
 * values of b2vx.h (1 = int8, 2 = uint8, 5 = int32, 9 = float32).
 */
#ifndef ORACLE_OPS_H_
#define ORACLE_OPS_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Quantization of one tensor.  per_channel != 0: scales[n] / zps[n] (zps may
 * be NULL = all zero); otherwise scale / zp.  A float32 tensor ignores it. */
typedef struct orc_quant {
  int32_t per_channel;
  float scale;
  int32_t zp;
  int32_t n;
  const float* scales;
  const int32_t* zps;
} orc_quant;

typedef struct orc_conv2d_args {
  /* input [W,H,C,N] */
  const void* x; int32_t x_dtype; uint32_t W, H, C, N; orc_quant xq;
  /* weights [kw,kh,Ic,Oc]; depthwise: [kw,kh,C*multiplier,1] */
  const void* w; int32_t w_dtype; uint32_t kw, kh, w_ic, w_oc; orc_quant wq;
  /* bias [Oc]: int32 for quantized inputs, float32 for float; may be NULL */
  const void* bias;
  /* output [Wo,Ho,Oc,N] */
  void* y; int32_t y_dtype; uint32_t Wo, Ho, Oc; orc_quant yq;
  uint32_t stride[2]; uint32_t dilation[2]; uint32_t pad_left, pad_top;
  int32_t multiplier;      /* >= 1: depthwise */
  int32_t group;           /* > 1: grouped, weights [kw,kh,C/group,Oc] */
  int32_t* acc_out;        /* optional [Wo,Ho,Oc,N] int32 accumulators (bias included) */
} orc_conv2d_args;

typedef struct orc_fc_args {
  const void* x; int32_t x_dtype; uint32_t K, batch; orc_quant xq;   /* x [K,batch] */
  const void* w; int32_t w_dtype; uint32_t N; orc_quant wq;          /* w [K,N]     */
  const void* bias;
  void* y; int32_t y_dtype; orc_quant yq;                            /* y [N,batch] */
  int32_t* acc_out;
} orc_fc_args;

typedef struct orc_pool2d_args {
  const void* x; int32_t dtype; uint32_t W, H, C, N; orc_quant xq;
  void* y; uint32_t Wo, Ho; orc_quant yq;
  int32_t type;            /* B2VX_POOL_* */
  uint32_t ksize[2]; uint32_t stride[2]; uint32_t pad_left, pad_top;
} orc_pool2d_args;

/* rounding / saturation */
double orc_rint(double x);
int32_t orc_fp32_to_affine(float in, float scale, int32_t zero_point, int32_t dtype);
float orc_affine_to_fp32(int32_t val, float scale, int32_t zero_point);

/* shape rules */
uint32_t orc_filter_size(uint32_t in, uint32_t ksize, uint32_t pad0, uint32_t pad1,
                         uint32_t stride, uint32_t dilation, int32_t round_type);
void orc_same_valid_padding(uint32_t in, uint32_t ksize, uint32_t stride, uint32_t dilation,
                            int32_t pad_type, uint32_t out_pad[2]);

/* ops; return 0 on success, -1 on an unsupported dtype combination */
int32_t orc_conv2d(const orc_conv2d_args* a);
int32_t orc_fully_connected(const orc_fc_args* a);
int32_t orc_pool2d(const orc_pool2d_args* a);
/* numpy-style broadcast of a [a_dims] and b [b_dims] into y [y_dims], rank <= 8 */
int32_t orc_add(const void* a, int32_t a_dtype, const uint32_t* a_dims, orc_quant aq,
                const void* b, int32_t b_dtype, const uint32_t* b_dims, orc_quant bq,
                void* y, int32_t y_dtype, const uint32_t* y_dims, orc_quant yq, uint32_t rank);
// ops::AddN: the sum of n same-shaped tensors, dequantized, added in float32 from left to right and quantized once
// (src/tim/vx/internal/src/ops/vsi_nn_op_addn.c:124-205 chains n-1 Add nodes; see b2vx.h for the intermediate type).
int32_t orc_addn(const void* const* x, const int32_t* dtypes, const orc_quant* q, uint32_t n,
                 void* y, int32_t y_dtype, orc_quant yq, uint64_t elems);
/* upper < 0: plain relu; otherwise clamp to [0, upper] */
int32_t orc_relu(const void* x, int32_t x_dtype, orc_quant xq, void* y, int32_t y_dtype,
                 orc_quant yq, uint64_t n, float upper);
/* softmax along `axis` of a rank-`rank` tensor; output float32 or quantized */
int32_t orc_softmax(const void* x, int32_t x_dtype, orc_quant xq, void* y, int32_t y_dtype,
                    orc_quant yq, const uint32_t* dims, uint32_t rank, int32_t axis, float beta);

/* number of OpenMP threads the ops will use */
int32_t orc_num_threads(void);

#ifdef __cplusplus
}
#endif
#endif /* ORACLE_OPS_H_ */
