/*
 * b2vx — C ABI of the B200-native execution backend behind the tim::vx API.
 *
 * This is the layer the tim::vx C++ classes lower to.  In the reference that
 * lower layer is the ovxlib C API (vsi_nn_CreateGraph, vsi_nn_AddTensor,
 * vsi_nn_AddNode, vsi_nn_SetupGraph, vsi_nn_VerifyGraph, vsi_nn_RunGraph,
 * vsi_nn_CopyDataToTensor, vsi_nn_CopyTensorToBuffer ...), whose call sites are
 * cited beside each entry point below (paths are relative to the reference
 * project root).  ovxlib's node structs are written to directly by the C++
 * layer (src/tim/vx/ops/conv2d.cc:71-81), so instead of cloning struct layouts
 * this ABI passes one plain descriptor per node kind.
 *
 * Conventions
 *   - opaque handles, POD descriptors, plain pointers and sizes only;
 *   - every call returns a b2vx_status; b2vx_last_error() gives the text;
 *   - tensors are addressed by a uint32 id that is local to their graph;
 *   - shapes are tim::vx order (dims[0] fastest: W,H,C,N for activations,
 *     W,H,Ic,Oc for convolution weights, K,N for fully-connected weights);
 *   - host pointers are borrowed for the duration of a call only;
 *   - the library owns all device memory; a graph is bound to one GPU;
 *   - a graph is not thread-safe; distinct graphs may be driven from distinct
 *     threads and may live on distinct GPUs.
 */
#ifndef B2VX_H_
#define B2VX_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B2VX_MAX_RANK 8u
#define B2VX_NO_TENSOR 0xFFFFFFFFu

typedef struct b2vx_context b2vx_context;
typedef struct b2vx_graph b2vx_graph;

typedef int32_t b2vx_status;
enum {
  B2VX_OK = 0,
  B2VX_INVALID_ARG = 1,
  B2VX_UNSUPPORTED = 2,
  B2VX_SHAPE_MISMATCH = 3,
  B2VX_QUANT_MISMATCH = 4,
  B2VX_OOM = 5,
  B2VX_CUDA_ERROR = 6,
  B2VX_DEVICE_TIMEOUT = 7,
  B2VX_BAD_STATE = 8
};

/* Values equal tim::vx::DataType (include/tim/vx/types.h:30-44). */
enum {
  B2VX_DT_UNKNOWN = 0,
  B2VX_DT_INT8 = 1,
  B2VX_DT_UINT8 = 2,
  B2VX_DT_INT16 = 3,
  B2VX_DT_UINT16 = 4,
  B2VX_DT_INT32 = 5,
  B2VX_DT_UINT32 = 6,
  B2VX_DT_INT64 = 7,
  B2VX_DT_FLOAT16 = 8,
  B2VX_DT_FLOAT32 = 9,
  B2VX_DT_BOOL8 = 10
};

/* Values equal tim::vx::QuantType (include/tim/vx/types.h:46-52). */
enum {
  B2VX_QUANT_NONE = 0,
  B2VX_QUANT_ASYMMETRIC = 1,
  B2VX_QUANT_SYMMETRIC_PER_CHANNEL = 2
};

/* Bits equal tim::vx::TensorAttribute (include/tim/vx/types.h:54-60). */
enum {
  B2VX_ATTR_CONSTANT = 1,
  B2VX_ATTR_TRANSIENT = 2,
  B2VX_ATTR_VARIABLE = 4,
  B2VX_ATTR_INPUT = 8,
  B2VX_ATTR_OUTPUT = 16
};

/* Values equal tim::vx::PadType / PoolType / RoundType (types.h:62-66). */
enum { B2VX_PAD_NONE = -1, B2VX_PAD_AUTO = 0, B2VX_PAD_VALID = 1, B2VX_PAD_SAME = 2 };
enum { B2VX_POOL_MAX = 0, B2VX_POOL_AVG = 1, B2VX_POOL_L2 = 2, B2VX_POOL_AVG_ANDROID = 3 };
enum { B2VX_ROUND_CEILING = 0, B2VX_ROUND_FLOOR = 1 };

enum {
  B2VX_NODE_CONV2D = 1,
  B2VX_NODE_FULLY_CONNECTED = 2,
  B2VX_NODE_POOL2D = 3,
  B2VX_NODE_ADD = 4,
  B2VX_NODE_RELU = 5,
  B2VX_NODE_RELU6 = 6,
  B2VX_NODE_SOFTMAX = 7,
  B2VX_NODE_RESHAPE = 8,
  B2VX_NODE_TRANSPOSE = 9,
  B2VX_NODE_CONCAT = 10,
  B2VX_NODE_DATACONVERT = 11,
  B2VX_NODE_ADDN = 12
};

/* most tensors one node reads (Concat) */
#define B2VX_MAX_NODE_INPUTS 16

/* Replaces vsi_nn_tensor_attr_t as filled by PackTensorDtype and
 * TensorImpl::Init (src/tim/vx/tensor.cc:40-99,391-459).  rank == 0 with the
 * TRANSIENT attribute means "shape inferred at compile" (tensor.cc:401-407).
 * For per-channel quantization scales/zero_points hold n_channel entries and
 * channel_dim names the axis they run along; otherwise scale/zero_point are
 * used and the arrays may be NULL. */
typedef struct b2vx_tensor_desc {
  int32_t dtype;
  uint32_t rank;
  uint32_t dims[B2VX_MAX_RANK];
  int32_t attr;
  int32_t quant_type;
  float scale;
  int32_t zero_point;
  int32_t channel_dim;
  uint32_t n_channel;
  const float* scales;
  const int32_t* zero_points;
} b2vx_tensor_desc;

/* Replaces vsi_nn_conv2d_param as written by ops::Conv2d
 * (src/tim/vx/ops/conv2d.cc:56-82).  multiplier >= 1 selects depthwise
 * (src/tim/vx/internal/src/ops/vsi_nn_op_conv2d.c:62-66).  pad = {left,right,
 * top,bottom}; it is used when pad_type is AUTO or NONE
 * (src/tim/vx/type_utils.cc:78-91) and recomputed for SAME/VALID
 * (src/tim/vx/internal/src/utils/vsi_nn_util.c:555-588).  dilation 0 means 1. */
typedef struct b2vx_conv2d_desc {
  uint32_t weights;
  int32_t pad_type;
  uint32_t ksize[2];
  uint32_t stride[2];
  uint32_t dilation[2];
  uint32_t pad[4];
  int32_t multiplier;
  /* ops::GroupedConv2d (src/tim/vx/ops/groupedconv2d.cc:34-68): input and output channels split into
   * `group` contiguous blocks, block g of the outputs reading block g of the inputs; the kernel is
   * [kw, kh, Ic/group, Oc].  0 and 1 mean an ordinary convolution. */
  int32_t group;
} b2vx_conv2d_desc;

/* Replaces vsi_nn_fcl_param (src/tim/vx/ops/fullyconnected.cc:37-41). */
typedef struct b2vx_fc_desc {
  uint32_t axis;
  uint32_t weights;
} b2vx_fc_desc;

/* Replaces vsi_nn_pool_param (src/tim/vx/ops/pool2d.cc:35-108). */
typedef struct b2vx_pool2d_desc {
  int32_t type;
  int32_t pad_type;
  uint32_t ksize[2];
  uint32_t stride[2];
  uint32_t pad[4];
  int32_t round_type;
} b2vx_pool2d_desc;

/* A list of up to B2VX_MAX_RANK numbers: a target shape (Reshape) or a permutation (Transpose). */
typedef struct b2vx_dims_desc {
  uint32_t rank;
  uint32_t v[8];
} b2vx_dims_desc;

/* Replaces vsi_nn_softmax_param (src/tim/vx/ops/softmax.cc:33-37). */
typedef struct b2vx_softmax_desc {
  float beta;
  int32_t axis;
} b2vx_softmax_desc;

/* One row of the compiled launch plan, for PrintGraph-style reporting and for
 * counting launches in a benchmark. */
typedef struct b2vx_kernel_info {
  char name[48];
  uint32_t node_index;
  uint64_t ops;            /* 2*MAC for contractions, 0 otherwise            */
  uint64_t bytes;          /* algorithmic bytes: unique inputs+outputs+consts */
  float last_ms;           /* filled by b2vx_graph_profile, else 0           */
} b2vx_kernel_info;

/* ---- context: vsi_nn_CreateContext / vsi_nn_ReleaseContext
 *      (src/tim/vx/context.cc:35-43) ---- */
b2vx_status b2vx_context_create(b2vx_context** out);
void b2vx_context_destroy(b2vx_context* ctx);
const char* b2vx_last_error(const b2vx_context* ctx);
/* Number of CUDA devices visible to the process (0 when none). */
int32_t b2vx_device_count(void);

/* ---- graph: vsi_nn_CreateGraph / vsi_nn_ReleaseGraph
 *      (src/tim/vx/graph.cc:91-99) ---- */
b2vx_status b2vx_graph_create(b2vx_context* ctx, int32_t device_id, b2vx_graph** out);
void b2vx_graph_destroy(b2vx_graph* g);

/* ---- tensors: vsi_nn_AddTensor / vsi_nn_AddTensorFromHandle
 *      (src/tim/vx/tensor.cc:391-459).  const_data is copied when non-NULL. */
b2vx_status b2vx_tensor_create(b2vx_graph* g, const b2vx_tensor_desc* desc,
                               const void* const_data, uint32_t* out_id);
/* vsi_nn_GetTensor / attr readback; after compile the inferred shape is
 * reported.  scales/zero_points pointers in *out stay owned by the graph. */
b2vx_status b2vx_tensor_get_desc(b2vx_graph* g, uint32_t id, b2vx_tensor_desc* out);
/* vsi_nn_CopyDataToTensor (src/tim/vx/tensor.cc:154-192): host -> tensor, the
 * whole tensor, WHCN order.  bytes must equal the tensor's byte size. */
b2vx_status b2vx_tensor_write(b2vx_graph* g, uint32_t id, const void* src, size_t bytes);
/* vsi_nn_CopyTensorToBuffer (src/tim/vx/tensor.cc:194-228): tensor -> host. */
b2vx_status b2vx_tensor_read(b2vx_graph* g, uint32_t id, void* dst, size_t bytes);

/* ---- nodes: vsi_nn_AddNode + nn_param writes + input/output binding
 *      (src/tim/vx/builtin_op_impl.cc:30-63).  bias may be B2VX_NO_TENSOR. */
b2vx_status b2vx_node_conv2d(b2vx_graph* g, uint32_t x, uint32_t w, uint32_t bias,
                             uint32_t y, const b2vx_conv2d_desc* d);
b2vx_status b2vx_node_fully_connected(b2vx_graph* g, uint32_t x, uint32_t w,
                                      uint32_t bias, uint32_t y, const b2vx_fc_desc* d);
b2vx_status b2vx_node_pool2d(b2vx_graph* g, uint32_t x, uint32_t y, const b2vx_pool2d_desc* d);
b2vx_status b2vx_node_add(b2vx_graph* g, uint32_t a, uint32_t b, uint32_t y);
b2vx_status b2vx_node_relu(b2vx_graph* g, uint32_t x, uint32_t y);
b2vx_status b2vx_node_relu6(b2vx_graph* g, uint32_t x, uint32_t y);
b2vx_status b2vx_node_softmax(b2vx_graph* g, uint32_t x, uint32_t y, const b2vx_softmax_desc* d);
/* Data movement between the compute nodes, as the reference's exported graphs use it
 * (samples/multi_device/vx_mobilenet.cc:570-571,832-840; vx_resnet50.cc:1347-1349).
 * Reshape (src/tim/vx/ops/reshape.cc:34-47): same elements in WHCN order under a new shape.
 * Transpose (src/tim/vx/ops/transpose.cc:34-45): output dimension i is input dimension perm[i].
 * Concat (src/tim/vx/ops/concat.cc:33-41): inputs joined along `axis`; 8-bit inputs whose
 * quantization differs from the output's are requantized.
 * DataConvert (src/tim/vx/ops/simple_operations.cc): quantize / dequantize / requantize. */
b2vx_status b2vx_node_reshape(b2vx_graph* g, uint32_t x, uint32_t y, const b2vx_dims_desc* shape);
b2vx_status b2vx_node_transpose(b2vx_graph* g, uint32_t x, uint32_t y, const b2vx_dims_desc* perm);
b2vx_status b2vx_node_concat(b2vx_graph* g, const uint32_t* inputs, uint32_t n_inputs, uint32_t axis, uint32_t y);
b2vx_status b2vx_node_dataconvert(b2vx_graph* g, uint32_t x, uint32_t y);
/* ops::AddN (src/tim/vx/ops/addn.cc -> vsi_nn_op_addn.c:124-205, which chains
 * n-1 Add nodes): y = x0 + x1 + ... over 2 to 16 tensors of one shape, all
 * int8/uint8 (any scales) or all float32.  The inputs are dequantized, summed in
 * float32 from left to right, and the sum is quantized once with the output's
 * parameters; with two inputs this is exactly the Add node.  (The reference's
 * intermediate sums of quantized inputs are float16 on hardware without the SP
 * unit; float16 is outside this backend, the sums here stay float32.) */
b2vx_status b2vx_node_addn(b2vx_graph* g, const uint32_t* inputs, uint32_t n_inputs, uint32_t y);

/* ---- compile / run: vsi_nn_SetupGraph + vsi_nn_VerifyGraph
 *      (src/tim/vx/graph.cc:328-383) and vsi_nn_RunGraph (graph.cc:389-391).
 * compile validates dtypes and quantization, sorts nodes, infers TRANSIENT
 * shapes, packs weights and builds the launch plan; it is idempotent.  run
 * compiles on first use, launches the plan and waits for it. */
b2vx_status b2vx_graph_compile(b2vx_graph* g);
b2vx_status b2vx_graph_run(b2vx_graph* g);
/* Launch the plan on the graph's stream without waiting. */
b2vx_status b2vx_graph_run_async(b2vx_graph* g);
/* Wait for everything queued on the graph's stream. */
b2vx_status b2vx_graph_sync(b2vx_graph* g);
/* Use the caller's cudaStream_t (passed as void*) for all later work of this
 * graph; NULL restores the graph's own stream. */
b2vx_status b2vx_graph_set_stream(b2vx_graph* g, void* cuda_stream);
/* vsi_nn_PrintGraph (src/tim/vx/graph.cc:393): one line per planned kernel. */
b2vx_status b2vx_graph_print(b2vx_graph* g);
/* Launch plan readback: count, then one row per kernel. */
b2vx_status b2vx_graph_kernel_count(b2vx_graph* g, uint32_t* out);
b2vx_status b2vx_graph_kernel_info(b2vx_graph* g, uint32_t index, b2vx_kernel_info* out);
/* Run the plan `iters` times with one CUDA-event pair around each kernel and
 * store the mean per-kernel time in b2vx_kernel_info::last_ms. */
b2vx_status b2vx_graph_profile(b2vx_graph* g, uint32_t iters);

/* ---- a convolution for callers that cannot allocate -------------------------
 * No counterpart in the reference (there, every buffer belongs to the driver).
 *
 * Some callers of this library never get to call cudaMalloc: a plugin that lives
 * inside a server whose device memory was carved up at start-up, a control loop
 * with a hard deadline (the driver's allocator takes locks and can stall the
 * whole device), a process running so close to the memory limit that an
 * allocation in the middle of a request may fail.  The graph API above allocates
 * tensors, packed weights and scratch at compile time; this entry point
 * allocates nothing, neither on the device nor through any library: the caller
 * passes every input and output as a device pointer, and the one intermediate
 * the operation needs, the im2col matrix, lives in a fixed array of
 * B2VX_NOALLOC_SCRATCH_BYTES inside the library.  Every GPU that loads the
 * library holds that array until the process exits.
 *
 * The operation: a first-layer quantized convolution (uint8 image with fewer
 * than 16 channels, int8 weights, uint8 output; at most 256 output channels),
 * computed exactly as a Conv2d node of the graph API computes it.
 *   x_whcn     uint8, tim::vx order [W,H,C,N] (N slowest)
 *   w8         int8 [Ocp][Kp]: row oc holds that channel's weights in the kernel
 *              tensor's own order, k = (c*kh + ky)*kw + kx, zero padded to
 *              Kp = K rounded up to 16; Ocp = oc rounded up to 16, extra rows zero
 *   bias_full  int32 [Ocp]: bias[oc] - in_zero_point * sum_k w8[oc][k]; padding 0
 *   acc_scale  float [Ocp]: in_scale * weight_scale[oc]; padding 0
 *   y_cl       uint8 [N*Ho*Wo][Ocp], channels-last; Wo/Ho follow from the explicit
 *              pad {left,right,top,bottom} with floor rounding
 * All pointers are device pointers aligned to 16 bytes.  The call returns when
 * y_cl is complete.  A problem whose im2col matrix (N*Ho*Wo*Kp bytes) exceeds
 * the array is refused with B2VX_INVALID_ARG and a message in err.
 *
 * The first call on a GPU resolves the array's device address (once, also when
 * several threads make their first call together); make that call before any
 * stream capture.  All calls on one GPU share the array: calls whose kernels
 * overlap on the GPU (other streams, other threads) race.  Extents, strides,
 * dilations and paddings above INT_MAX/4, filters with kw*kh*c > 65536 and zero
 * points outside 0..255 are refused with B2VX_INVALID_ARG. */
#define B2VX_NOALLOC_SCRATCH_BYTES (16u * 1024u * 1024u)
typedef struct b2vx_conv2d_noalloc_desc {
  uint32_t n, h, w, c;
  uint32_t kw, kh, oc;
  uint32_t stride[2];
  uint32_t dilation[2];
  uint32_t pad[4];
  int32_t in_zero_point;
  float out_scale;
  int32_t out_zero_point;
} b2vx_conv2d_noalloc_desc;
b2vx_status b2vx_conv2d_first_layer_noalloc(const b2vx_conv2d_noalloc_desc* d, const void* x_whcn, const int8_t* w8,
                                            const int32_t* bias_full, const float* acc_scale, void* y_cl,
                                            void* cuda_stream, char* err, size_t err_len);

/* Measurement aid with no counterpart in the reference: the dense int8 rate of
 * the tensor pipe of GPU `device_id`, in TOP/s (2 x multiply-accumulate), from
 * an issue-rate microbenchmark (tcgen05.mma.kind::i8 on operands resident in
 * shared memory, no epilogue, every SM, about 10 ms per repetition, best of
 * `reps`).  It is the denominator of the "fraction of int8 peak" figures. */
b2vx_status b2vx_measure_int8_peak(int32_t device_id, int32_t reps, double* tops_out, int32_t* sm_count_out);

/* Pinned host memory for callers that want asynchronous tensor_write/read. */
b2vx_status b2vx_host_alloc(void** out, size_t bytes);
void b2vx_host_free(void* p);

#ifdef __cplusplus
}
#endif
#endif /* B2VX_H_ */
