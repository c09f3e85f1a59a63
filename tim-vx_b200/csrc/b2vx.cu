// b2vx C ABI on CUDA: graph bookkeeping, validation, shape inference, weight
// packing and the launch plan.  (Entry points are documented in b2vx.h.)
//
// What Compile does — the part the reference spreads over vsi_nn_SetupGraph /
// vsi_nn_VerifyGraph (src/tim/vx/internal/src/vsi_nn_graph.c:1450-1603) and
// the closed driver's vxVerifyGraph:
//   1. order nodes by data dependency;
//   2. per node: dtype/quantization checks, padding and output-shape rules
//      (vsi_nn_op_conv2d.c:199-287, vsi_nn_op_pool.c:324-427,
//      vsi_nn_op_fullconnect2.c:154-196, vsi_nn_util.c:483-588);
//   3. give every activation tensor channels-last device storage (kernels.h);
//   4. pack constants for the kernel chosen per node: int8-shifted weight
//      matrix [rows][Kp], folded bias (bias - zx*sum(w) + K*zx*dz), per-tap
//      border corrections, per-channel accumulator scales;
//   5. record one launch closure per kernel.
// Run replays the closures on the graph's stream.
//
// There is no CPU execution path: without a CUDA device graph creation fails.
#include <cuda_runtime.h>

#include <algorithm>
#include <array>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <memory>
#include <string>
#include <vector>

#include "b2vx.h"
#include "kernels.h"

using namespace b2vx;

namespace {

size_t dtype_size(int32_t dt) {
  switch (dt) {
    case B2VX_DT_INT8: case B2VX_DT_UINT8: case B2VX_DT_BOOL8: return 1;
    case B2VX_DT_INT16: case B2VX_DT_UINT16: case B2VX_DT_FLOAT16: return 2;
    case B2VX_DT_INT32: case B2VX_DT_UINT32: case B2VX_DT_FLOAT32: return 4;
    case B2VX_DT_INT64: return 8;
    default: return 0;
  }
}
bool is_q8(int32_t dt) { return dt == B2VX_DT_INT8 || dt == B2VX_DT_UINT8; }
int round_up(int v, int m) { return (v + m - 1) / m * m; }

struct TensorRec {
  b2vx_tensor_desc d;
  std::vector<float> scales;
  std::vector<int32_t> zps;
  bool has_shape = false;
  std::vector<uint8_t> host;   // constants, and data written before compile (WHCN order)
  bool host_valid = false;
  // device side
  int W = 1, H = 1, C = 1, N = 1, Cp = 0;
  void* d_cl = nullptr;        // channels-last storage
  void* d_io = nullptr;        // WHCN copy for graph inputs/outputs (== d_cl when both layouts coincide)
  size_t cl_bytes = 0, io_bytes = 0;
  bool is_activation = false;
  bool cl_used = false;        // some kernel reads the channels-last copy (decides whether a graph input is converted)
  bool io_direct = false;      // a graph output whose producer writes the WHCN copy itself (no conversion at the end)

  size_t elems() const {
    size_t n = 1;
    for (uint32_t i = 0; i < d.rank; ++i) n *= d.dims[i];
    return n;
  }
  size_t bytes() const { return elems() * dtype_size(d.dtype); }
  float scale() const { return d.quant_type == B2VX_QUANT_ASYMMETRIC ? d.scale : 1.0f; }
  int32_t zp() const { return d.quant_type == B2VX_QUANT_ASYMMETRIC ? d.zero_point : 0; }
  bool same_layouts() const { return H == 1 && W == 1 && Cp == C; }
};

struct NodeRec {
  int32_t kind;
  uint32_t in[B2VX_MAX_NODE_INPUTS];   // unused slots hold B2VX_NO_TENSOR
  uint32_t out;
  union {
    b2vx_conv2d_desc conv;
    b2vx_fc_desc fc;
    b2vx_pool2d_desc pool;
    b2vx_softmax_desc softmax;
    b2vx_dims_desc dims;      // Reshape: target shape; Transpose: permutation
    uint32_t concat_axis;
  } p;
  uint32_t pad[4];
  bool removed = false;   // folded into its producer at compile
  int fuse_add = -1;      // index of the Add node this convolution's epilogue may absorb
  uint32_t fuse_residual = B2VX_NO_TENSOR;   // that Add's other operand
};

struct Step {
  b2vx_kernel_info info;
  std::function<cudaError_t(cudaStream_t)> fn;
  const void* tag = nullptr;   // identifies a step to code that runs after the list was edited (steps are inserted in front of others)
};

}  // namespace

struct b2vx_context {
  std::string err;
};

struct b2vx_graph {
  b2vx_context* ctx = nullptr;
  int device = 0;
  cudaStream_t own_stream = nullptr;
  cudaStream_t stream = nullptr;
  std::vector<TensorRec> tensors;
  std::vector<NodeRec> nodes;
  std::vector<uint32_t> order;
  std::vector<Step> steps;
  std::vector<void*> allocs;
  std::vector<GemmTcPlan*> gemm_plans;
  std::vector<std::function<b2vx_status()>> finalizers;   // run once device scratch exists
  void* scratch = nullptr;
  size_t scratch_bytes = 0;
  int* d_status = nullptr;
  int* h_status = nullptr;
  bool compiled = false;
  bool use_tc = false;
  bool fuse_add = true;      // residual Add into the preceding convolution's epilogue (B2VX_FUSE_ADD=0 disables)
  int fuse_request = -1;     // set while planning a convolution that may absorb an Add: that Add's node index
  uint32_t fuse_residual = B2VX_NO_TENSOR;
  bool fuse_done = false;
  bool fc_small_m = true;    // FullyConnected with <= 16 rows on the CUDA-core streaming kernel
  int add_mode = 0;          // quantized Add: 0 choose by size, 1 table kernel, 2 arithmetic kernel
  // the whole launch plan captured once as a CUDA graph; replays cost one launch on the host
  cudaGraphExec_t exec = nullptr;
  bool capture_failed = false;
  bool use_cuda_graph = true;
};

namespace {

b2vx_status fail(b2vx_graph* g, b2vx_status st, const std::string& msg) {
  if (g && g->ctx) g->ctx->err = msg;
  return st;
}

#define CUDA_TRY(g, expr)                                                                         \
  do {                                                                                            \
    cudaError_t _e = (expr);                                                                      \
    if (_e != cudaSuccess)                                                                        \
      return fail((g), B2VX_CUDA_ERROR, std::string(#expr) + ": " + cudaGetErrorString(_e));      \
  } while (0)

bool valid_id(const b2vx_graph* g, uint32_t id) { return id < g->tensors.size(); }

// Makes the graph's GPU current for the duration of a call.  A host thread that has not chosen a device yet
// reports device 0; going back to it afterwards would create a context on GPU 0 in a process that works on
// another GPU (and did, in worker threads of multi-GPU runs, at a cost of milliseconds per call), so the
// previous device is restored only if this process already has a context there.
struct DeviceGuard {
  int prev = -1;
  explicit DeviceGuard(int dev) {
    cudaGetDevice(&prev);
    if (prev != dev) cudaSetDevice(dev);
    else prev = -1;
  }
  ~DeviceGuard() {
    if (prev < 0) return;
    typedef int (*StateFn)(int, unsigned int*, int*);   // cuDevicePrimaryCtxGetState(CUdevice, unsigned*, int*)
    static const StateFn state = [] {
      void* fn = nullptr;
      cudaDriverEntryPointQueryResult q;
      if (cudaGetDriverEntryPoint("cuDevicePrimaryCtxGetState", &fn, cudaEnableDefault, &q) != cudaSuccess ||
          q != cudaDriverEntryPointSuccess)
        fn = nullptr;
      return reinterpret_cast<StateFn>(fn);
    }();
    unsigned int flags = 0;
    int active = 1;
    if (state && state(prev, &flags, &active) == 0 && !active) return;   // ordinal == CUdevice handle for cudart devices
    cudaSetDevice(prev);
  }
};

b2vx_status dev_alloc(b2vx_graph* g, void** out, size_t bytes) {
  *out = nullptr;
  if (bytes == 0) bytes = 16;
  cudaError_t e = cudaMalloc(out, bytes);
  if (e != cudaSuccess) return fail(g, B2VX_OOM, std::string("cudaMalloc: ") + cudaGetErrorString(e));
  g->allocs.push_back(*out);
  return B2VX_OK;
}

template <typename T>
b2vx_status upload(b2vx_graph* g, const std::vector<T>& v, T** out) {
  void* p = nullptr;
  b2vx_status st = dev_alloc(g, &p, v.size() * sizeof(T));
  if (st != B2VX_OK) return st;
  if (!v.empty()) CUDA_TRY(g, cudaMemcpy(p, v.data(), v.size() * sizeof(T), cudaMemcpyHostToDevice));
  *out = static_cast<T*>(p);
  return B2VX_OK;
}

// ---------------------------------------------------------------- shapes

// vsi_nn_ComputeFilterSize (src/tim/vx/internal/src/utils/vsi_nn_util.c:483-511)
uint32_t filter_size(uint32_t in, uint32_t k, uint32_t pad0, uint32_t pad1, uint32_t stride, uint32_t dilation, int32_t round_type) {
  if (stride == 0) {
    if (in != k) return 0;
    stride = 1;
  }
  if (dilation > 1) k = dilation * (k - 1) + 1;
  const int64_t span = static_cast<int64_t>(in) + pad0 + pad1 - k;
  if (span < 0) return 0;
  const uint32_t steps = round_type == B2VX_ROUND_CEILING ? static_cast<uint32_t>((span + stride - 1) / stride)
                                                          : static_cast<uint32_t>(span / stride);
  return steps + 1;
}

// vsi_nn_compute_padding (vsi_nn_util.c:535-588): SAME -> out = ceil(in/stride),
// odd padding goes to the end; VALID -> none; AUTO/NONE -> the explicit values.
void resolve_pads(int32_t pad_type, const uint32_t in[2], const uint32_t k[2], const uint32_t stride[2],
                  const uint32_t dil[2], const uint32_t explicit_pad[4], uint32_t out[4]) {
  for (int i = 0; i < 4; ++i) out[i] = explicit_pad[i];
  if (pad_type != B2VX_PAD_SAME && pad_type != B2VX_PAD_VALID) return;
  uint32_t d[2] = {dil[0], dil[1]};
  if (d[0] == 0 && d[1] == 0) d[0] = d[1] = 1;
  for (int a = 0; a < 2; ++a) {
    const uint32_t dl = d[a] ? d[a] : 1, st = stride[a] ? stride[a] : 1;
    const int64_t eff = static_cast<int64_t>(k[a] - 1) * dl + 1;
    const int64_t o = pad_type == B2VX_PAD_SAME ? (static_cast<int64_t>(in[a]) + st - 1) / st
                                                : (static_cast<int64_t>(in[a]) + st - eff) / st;
    int64_t total = (o - 1) * st + eff - in[a];
    if (total < 0) total = 0;
    out[2 * a] = static_cast<uint32_t>(total / 2);
    out[2 * a + 1] = static_cast<uint32_t>(total - total / 2);
  }
}

// A declared output shape wins over the inferred one; for conv/pool it may be
// smaller in W/H (the reference's own depthwise padding test relies on that:
// src/tim/vx/ops/depthwiseConv_test.cc:268-330).
b2vx_status set_shape(b2vx_graph* g, uint32_t id, const std::vector<uint32_t>& dims, const char* what, bool spatial_may_shrink) {
  TensorRec& t = g->tensors[id];
  if (t.has_shape) {
    bool ok = t.d.rank == dims.size();
    for (size_t i = 0; ok && i < dims.size(); ++i) {
      if (spatial_may_shrink && i < 2) ok = t.d.dims[i] >= 1 && t.d.dims[i] <= dims[i];
      else ok = t.d.dims[i] == dims[i];
    }
    if (!ok) return fail(g, B2VX_SHAPE_MISMATCH, std::string(what) + ": declared output shape differs from the inferred one");
    return B2VX_OK;
  }
  t.d.rank = static_cast<uint32_t>(dims.size());
  for (size_t i = 0; i < dims.size(); ++i) t.d.dims[i] = dims[i];
  t.has_shape = true;
  return B2VX_OK;
}

b2vx_status infer_node(b2vx_graph* g, NodeRec& n) {
  const TensorRec& x = g->tensors[n.in[0]];
  if (!x.has_shape) return fail(g, B2VX_SHAPE_MISMATCH, "node input has no shape");
  switch (n.kind) {
    case B2VX_NODE_CONV2D: {
      const TensorRec& w = g->tensors[n.in[1]];
      if (x.d.rank < 3 || x.d.rank > 4 || w.d.rank != 4) return fail(g, B2VX_SHAPE_MISMATCH, "conv2d: input must be rank 3/4 and kernel rank 4");
      const b2vx_conv2d_desc& c = n.p.conv;
      const uint32_t in2[2] = {x.d.dims[0], x.d.dims[1]}, k2[2] = {w.d.dims[0], w.d.dims[1]};
      resolve_pads(c.pad_type, in2, k2, c.stride, c.dilation, c.pad, n.pad);
      const uint32_t wo = filter_size(in2[0], k2[0], n.pad[0], n.pad[1], c.stride[0], c.dilation[0], B2VX_ROUND_FLOOR);
      const uint32_t ho = filter_size(in2[1], k2[1], n.pad[2], n.pad[3], c.stride[1], c.dilation[1], B2VX_ROUND_FLOOR);
      if (wo == 0 || ho == 0) return fail(g, B2VX_SHAPE_MISMATCH, "conv2d: kernel larger than padded input");
      const uint32_t oc = c.weights > 0 ? c.weights : (c.multiplier > 0 ? x.d.dims[2] * c.multiplier : w.d.dims[3]);
      std::vector<uint32_t> dims = {wo, ho, oc};
      if (x.d.rank == 4) dims.push_back(x.d.dims[3]);
      return set_shape(g, n.out, dims, "conv2d", true);
    }
    case B2VX_NODE_FULLY_CONNECTED: {
      const TensorRec& w = g->tensors[n.in[1]];
      if (w.d.rank != 2 || n.p.fc.axis >= x.d.rank) return fail(g, B2VX_SHAPE_MISMATCH, "fully_connected: weights must be rank 2 and axis inside the input rank");
      std::vector<uint32_t> dims = {n.p.fc.weights ? n.p.fc.weights : w.d.dims[1]};
      for (uint32_t i = n.p.fc.axis + 1; i < x.d.rank; ++i) dims.push_back(x.d.dims[i]);
      if (dims.size() == 1) dims.push_back(1);
      TensorRec& y = g->tensors[n.out];
      if (y.has_shape) {
        size_t want = 1;
        for (uint32_t v : dims) want *= v;
        if (y.elems() != want || y.d.dims[0] != dims[0]) return fail(g, B2VX_SHAPE_MISMATCH, "fully_connected: declared output shape");
        return B2VX_OK;
      }
      return set_shape(g, n.out, dims, "fully_connected", false);
    }
    case B2VX_NODE_POOL2D: {
      if (x.d.rank < 3 || x.d.rank > 4) return fail(g, B2VX_SHAPE_MISMATCH, "pool2d: input must be rank 3 or 4");
      const b2vx_pool2d_desc& c = n.p.pool;
      const uint32_t in2[2] = {x.d.dims[0], x.d.dims[1]}, dil[2] = {1, 1};
      resolve_pads(c.pad_type, in2, c.ksize, c.stride, dil, c.pad, n.pad);
      const uint32_t wo = filter_size(in2[0], c.ksize[0], n.pad[0], n.pad[1], c.stride[0], 1, c.round_type);
      const uint32_t ho = filter_size(in2[1], c.ksize[1], n.pad[2], n.pad[3], c.stride[1], 1, c.round_type);
      if (wo == 0 || ho == 0) return fail(g, B2VX_SHAPE_MISMATCH, "pool2d: window larger than padded input");
      std::vector<uint32_t> dims = {wo, ho};
      for (uint32_t i = 2; i < x.d.rank; ++i) dims.push_back(x.d.dims[i]);
      return set_shape(g, n.out, dims, "pool2d", true);
    }
    case B2VX_NODE_ADD: {
      const TensorRec& b = g->tensors[n.in[1]];
      if (!b.has_shape) return fail(g, B2VX_SHAPE_MISMATCH, "add: input has no shape");
      // numpy-style broadcast per dimension (vsi_nn_op_eltwise.c:147-214); operands of different rank
      // map to different storage axes here, so equal ranks are required (pad the shape with ones)
      if (b.d.rank != x.d.rank) return fail(g, B2VX_UNSUPPORTED, "add: operands must have the same rank (pad the smaller shape with ones)");
      std::vector<uint32_t> dims(x.d.rank);
      for (uint32_t i = 0; i < x.d.rank; ++i) {
        const uint32_t da = x.d.dims[i], db = b.d.dims[i];
        if (da != db && da != 1 && db != 1) return fail(g, B2VX_SHAPE_MISMATCH, "add: shapes do not broadcast");
        dims[i] = std::max(da, db);
      }
      return set_shape(g, n.out, dims, "add", false);
    }
    case B2VX_NODE_RESHAPE: {
      // src/tim/vx/ops/reshape.cc:46-58: the target shape is the output's shape; element counts must agree
      const b2vx_dims_desc& d = n.p.dims;
      std::vector<uint32_t> dims(d.v, d.v + d.rank);
      size_t want = 1;
      for (uint32_t v : dims) want *= v;
      if (want != x.elems()) return fail(g, B2VX_SHAPE_MISMATCH, "reshape: element count changes");
      TensorRec& y = g->tensors[n.out];
      if (y.has_shape) return y.elems() == want ? B2VX_OK : fail(g, B2VX_SHAPE_MISMATCH, "reshape: declared output size");
      return set_shape(g, n.out, dims, "reshape", false);
    }
    case B2VX_NODE_TRANSPOSE: {
      // vsi_nn_op_permute.c op_setup: out.size[i] = in.size[perm[i]]
      const b2vx_dims_desc& d = n.p.dims;
      if (d.rank != x.d.rank) return fail(g, B2VX_SHAPE_MISMATCH, "transpose: permutation length != input rank");
      std::vector<uint32_t> dims(d.rank);
      uint32_t seen = 0;
      for (uint32_t i = 0; i < d.rank; ++i) {
        if (d.v[i] >= d.rank || (seen >> d.v[i]) & 1u) return fail(g, B2VX_INVALID_ARG, "transpose: not a permutation");
        seen |= 1u << d.v[i];
        dims[i] = x.d.dims[d.v[i]];
      }
      return set_shape(g, n.out, dims, "transpose", false);
    }
    case B2VX_NODE_ADDN: {
      for (uint32_t id : n.in) {
        if (id == B2VX_NO_TENSOR) continue;
        const TensorRec& t = g->tensors[id];
        if (!t.has_shape || t.d.rank != x.d.rank) return fail(g, B2VX_SHAPE_MISMATCH, "addn: input shapes differ");
        for (uint32_t i = 0; i < x.d.rank; ++i)
          if (t.d.dims[i] != x.d.dims[i]) return fail(g, B2VX_SHAPE_MISMATCH, "addn: input shapes differ");
      }
      return set_shape(g, n.out, std::vector<uint32_t>(x.d.dims, x.d.dims + x.d.rank), "addn", false);
    }
    case B2VX_NODE_CONCAT: {
      // vsi_nn_op_concat.c op_setup: all dimensions but `axis` agree; the axis extents add up
      const uint32_t axis = n.p.concat_axis;
      if (axis >= x.d.rank) return fail(g, B2VX_SHAPE_MISMATCH, "concat: axis outside the input rank");
      std::vector<uint32_t> dims(x.d.dims, x.d.dims + x.d.rank);
      dims[axis] = 0;
      for (uint32_t id : n.in) {
        if (id == B2VX_NO_TENSOR) continue;
        const TensorRec& t = g->tensors[id];
        if (!t.has_shape || t.d.rank != x.d.rank) return fail(g, B2VX_SHAPE_MISMATCH, "concat: input ranks differ");
        for (uint32_t i = 0; i < x.d.rank; ++i)
          if (i != axis && t.d.dims[i] != x.d.dims[i]) return fail(g, B2VX_SHAPE_MISMATCH, "concat: input shapes differ off the axis");
        dims[axis] += t.d.dims[axis];
      }
      return set_shape(g, n.out, dims, "concat", false);
    }
    default:
      return set_shape(g, n.out, std::vector<uint32_t>(x.d.dims, x.d.dims + x.d.rank), "unary", false);
  }
}

// tim::vx dims -> (W,H,C,N): rank 4 as is, rank 3 = [W,H,C], rank 2 = [C,N], rank 1 = [C].
void map_dims(TensorRec& t) {
  t.W = t.H = t.C = t.N = 1;
  const uint32_t* d = t.d.dims;
  switch (t.d.rank) {
    case 4: t.W = d[0]; t.H = d[1]; t.C = d[2]; t.N = d[3]; break;
    case 3: t.W = d[0]; t.H = d[1]; t.C = d[2]; break;
    case 2: t.C = d[0]; t.N = d[1]; break;
    case 1: t.C = d[0]; break;
    default: break;
  }
  const int per16 = static_cast<int>(16 / dtype_size(t.d.dtype));
  t.Cp = round_up(t.C, per16);
  t.cl_bytes = static_cast<size_t>(t.N) * t.H * t.W * t.Cp * dtype_size(t.d.dtype);
  t.io_bytes = t.bytes();
}

// Channels-last storage of a tensor a kernel is about to read.
const void* cl_in(TensorRec& t) {
  t.cl_used = true;
  return t.d_cl;
}

OutQuant out_quant(const TensorRec& t) {
  OutQuant q;
  q.scale = t.scale();
  q.zp = t.zp();
  if (t.d.dtype == B2VX_DT_INT8) { q.lo = -128; q.hi = 127; }
  else if (t.d.dtype == B2VX_DT_UINT8) { q.lo = 0; q.hi = 255; }
  else { q.lo = INT32_MIN; q.hi = INT32_MAX; }
  return q;
}

// Host copy of the device requantization (requant.cuh): fp32_to_affine of the
// reference with its vsi_rint tie rule, in plain IEEE float operations.
int host_requant(float real, const OutQuant& q) {
  if (std::isinf(real)) return real < 0.0f ? q.lo : q.hi;
  const float x = real / q.scale;
  const float ax = std::fabs(x);
  const float fl = std::floor(ax);
  float r;
  if (ax - fl == 0.5f) r = fl + static_cast<float>(static_cast<long long>(fl) & 1);
  else r = std::floor(ax + 0.5f);
  r = std::copysign(r, x);
  double v = static_cast<double>(r) + q.zp;
  if (!(v == v)) v = 0;
  v = std::max(static_cast<double>(q.lo), std::min(static_cast<double>(q.hi), v));
  return static_cast<int>(v);
}

// Relu / Relu6 from one 8-bit quantization to another as a byte table:
// quantize(clamp(dequantize(q), 0, upper)).
std::vector<uint8_t> relu_table(const TensorRec& x, const TensorRec& y, float upper) {
  std::vector<uint8_t> lut(256);
  const OutQuant oq = out_quant(y);
  const bool xs = x.d.dtype == B2VX_DT_INT8;
  for (int i = 0; i < 256; ++i) {
    const int q = xs ? static_cast<int>(static_cast<int8_t>(i)) : i;
    float r = (static_cast<float>(q) - static_cast<float>(x.zp())) * x.scale();
    r = r < 0.0f ? 0.0f : r;
    if (upper >= 0.0f && r > upper) r = upper;
    lut[i] = static_cast<uint8_t>(host_requant(r, oq) & 0xFF);
  }
  return lut;
}

b2vx_kernel_info make_info(const char* name, uint32_t node, uint64_t ops, uint64_t bytes) {
  b2vx_kernel_info i;
  std::memset(&i, 0, sizeof(i));
  std::snprintf(i.name, sizeof(i.name), "%s", name);
  i.node_index = node;
  i.ops = ops;
  i.bytes = bytes;
  return i;
}

ConvGeom conv_geom(const TensorRec& x, const TensorRec& y, int kw, int kh, const uint32_t stride[2], const uint32_t dil[2], const uint32_t pad[4]) {
  ConvGeom g;
  g.N = x.N; g.H = x.H; g.W = x.W; g.C = x.C; g.Cp = x.Cp;
  g.Ho = y.H; g.Wo = y.W; g.Oc = y.C; g.Ocp = y.Cp;
  g.kh = kh; g.kw = kw;
  g.sx = stride[0] ? stride[0] : 1; g.sy = stride[1] ? stride[1] : 1;
  g.dx = dil[0] ? dil[0] : 1; g.dy = dil[1] ? dil[1] : 1;
  g.pl = pad[0]; g.pt = pad[2];
  return g;
}

// vsi_nn_QuantCheck (src/tim/vx/internal/src/utils/vsi_nn_dtype_util.c:368-441):
// only same-dtype, same-quantization-kind triples are checked (so per-channel weights
// under a per-tensor input, whose quantization kinds differ, pass unchecked there and
// here: no per-channel comparison of bias scales exists to mirror); the bias scale
// has to equal s_in*s_w within max(min(.)*1e-5, 1e-8)
// (src/tim/vx/internal/src/quantization/vsi_nn_asymmetric_affine.c:59-112).
bool quant_check(const TensorRec& x, const TensorRec& w, const TensorRec* b) {
  if (x.d.dtype != w.d.dtype || x.d.quant_type != w.d.quant_type) return true;
  if (b && b->d.quant_type != x.d.quant_type) return true;
  if (!is_q8(x.d.dtype) || x.d.quant_type != B2VX_QUANT_ASYMMETRIC) return true;
  if (!b || b->d.scale == 0.0f) return true;
  const double prod = static_cast<double>(x.d.scale) * static_cast<double>(w.d.scale), bs = b->d.scale;
  return std::fabs(prod - bs) <= std::max(std::min(prod, bs) * 1e-5, 1e-8);
}

// ---------------------------------------------------------------- contraction planning (conv2d dense, fully connected)

struct PackedContraction {
  std::vector<int8_t> w8;          // [rows][Kp]
  std::vector<int32_t> bias_full;  // [Ocp]
  std::vector<float> acc_scale;    // [Ocp]
  std::vector<int32_t> dz;         // [Ocp]
  std::vector<int32_t> tapc;       // [taps][Ocp]
  bool need_s = false;
  int rows = 0, Kp = 0;
  // largest |accumulator * acc_scale| any output channel can reach, the accumulator being the true
  // sum((x - zx)*(w - zw)) + bias with every product at the end of the input type's range that makes it largest
  double real_max = 0.0;
};

// Weight element (kx,ky,ic,oc) of a WHIcOc kernel as a signed value together
// with the zero point that still has to be subtracted from it: u8 weights are
// shifted by 128 into int8 (dz = zw-128), s8 weights are kept (dz = zw).
// K index by k_order: 0 tap*Cs + ic; 1 ic*taps + tap (the kernel tensor's own order, used with the
// WHCN im2col); 2 / 3 (ky*C + ic)*8 + kx / (ky*C + ic)*4 + kx (filter rows padded to 8 / 4 taps, used with the row-of-8 / row-of-4 im2col).  Rows come in n_tiles tiles of tile_rows rows: output channel oc is row
// (oc / tile_data) * tile_rows + oc % tile_data; when some dz != 0 and tile_rows > tile_data, row
// tile_data of every tile is the all-ones row (its dot product with an input row is S).
void pack_contraction(const TensorRec& x, const TensorRec& w, const TensorRec* bias, int kw, int kh, int C, int Cs,
                      int Kp, int Oc, int Ocp, int n_tiles, int tile_data, int tile_rows, int k_order,
                      PackedContraction* out) {
  const int rows = n_tiles * tile_rows;
  const int taps = kw * kh;
  const bool w_u8 = w.d.dtype == B2VX_DT_UINT8;
  const bool per_ch = w.d.quant_type == B2VX_QUANT_SYMMETRIC_PER_CHANNEL;
  auto kidx = [&](int t, int ic) -> size_t {
    if (k_order == 1) return static_cast<size_t>(ic) * taps + t;
    if (k_order == 2 || k_order == 3) return (static_cast<size_t>(t / kw) * C + ic) * (k_order == 2 ? 8 : 4) + t % kw;
    return static_cast<size_t>(t) * Cs + ic;
  };
  out->rows = rows;
  out->Kp = Kp;
  out->bias_full.assign(Ocp, 0);
  out->acc_scale.assign(Ocp, 0.0f);
  out->dz.assign(Ocp, 0);
  out->tapc.assign(static_cast<size_t>(taps) * Ocp, 0);
  out->need_s = false;
  const int zx = x.zp();
  const float sx = x.scale();
  std::vector<int64_t> tapsum(taps);
  const int32_t* b = bias ? reinterpret_cast<const int32_t*>(bias->host.data()) : nullptr;
  const int x_lo = (x.d.dtype == B2VX_DT_INT8 ? -128 : 0) - zx, x_hi = (x.d.dtype == B2VX_DT_INT8 ? 127 : 255) - zx;
  out->real_max = 0.0;
  for (int oc = 0; oc < Oc; ++oc) {
    const int zw = per_ch ? (w.zps.empty() ? 0 : w.zps[oc]) : w.zp();
    const float sw = per_ch ? w.scales[oc] : w.scale();
    const int dz = w_u8 ? zw - 128 : zw;
    out->dz[oc] = dz;
    if (dz != 0) out->need_s = true;
    out->acc_scale[oc] = sx * sw;
  }
  out->w8.assign(static_cast<size_t>(rows) * Kp, 0);
  for (int oc = 0; oc < Oc; ++oc) {
    std::fill(tapsum.begin(), tapsum.end(), 0);
    int64_t pos = 0, neg = 0;
    int8_t* row = out->w8.data() + (static_cast<size_t>(oc / tile_data) * tile_rows + oc % tile_data) * Kp;
    for (int ic = 0; ic < C; ++ic) {
      for (int t = 0; t < taps; ++t) {
        const size_t src = (static_cast<size_t>(oc) * C + ic) * taps + t;   // WHIcOc, W fastest: tap = ky*kw + kx
        const int v = w_u8 ? static_cast<int>(w.host[src]) - 128 : static_cast<int>(reinterpret_cast<const int8_t*>(w.host.data())[src]);
        row[kidx(t, ic)] = static_cast<int8_t>(v);
        tapsum[t] += v;
        const int64_t wr = v - out->dz[oc];   // the real weight minus its zero point
        const int64_t p0 = wr * x_lo, p1 = wr * x_hi;
        pos += p0 > p1 ? p0 : p1;
        neg += p0 < p1 ? p0 : p1;
      }
    }
    const double hi = static_cast<double>(pos + (b ? b[oc] : 0)), lo = static_cast<double>(neg + (b ? b[oc] : 0));
    out->real_max = std::max(out->real_max, std::max(std::fabs(hi), std::fabs(lo)) * std::fabs(static_cast<double>(out->acc_scale[oc])));
    int64_t all = 0;
    for (int t = 0; t < taps; ++t) {
      // contribution of one fully in-bounds tap beyond the raw products:
      //   -zx*sum_c(w8) + C*zx*dz
      const int64_t tc = -static_cast<int64_t>(zx) * tapsum[t] + static_cast<int64_t>(C) * zx * out->dz[oc];
      out->tapc[static_cast<size_t>(t) * Ocp + oc] = static_cast<int32_t>(tc);
      all += tc;
    }
    out->bias_full[oc] = static_cast<int32_t>((b ? b[oc] : 0) + all);
  }
  if (tile_rows > tile_data && out->need_s) {
    for (int tile = 0; tile < n_tiles; ++tile) {
      int8_t* ones = out->w8.data() + (static_cast<size_t>(tile) * tile_rows + tile_data) * Kp;
      for (int t = 0; t < taps; ++t)
        for (int ic = 0; ic < C; ++ic) ones[kidx(t, ic)] = 1;
    }
  }
}

// Element strides of a tensor's channels-last storage per logical (WHCN-order) dimension.
void cl_strides(const TensorRec& t, long long s[4]) {
  s[0] = s[1] = s[2] = s[3] = 0;
  switch (t.d.rank) {
    case 4: s[3] = static_cast<long long>(t.H) * t.W * t.Cp;   // fall through
    case 3: s[0] = t.Cp; s[1] = static_cast<long long>(t.W) * t.Cp; s[2] = 1; break;
    case 2: s[0] = 1; s[1] = t.Cp; break;
    default: s[0] = 1; break;
  }
}

// Element strides of the dense WHCN-order copy (dimension 0 fastest).
void dense_strides(const TensorRec& t, long long s[4]) {
  long long acc = 1;
  for (uint32_t k = 0; k < 4; ++k) {
    s[k] = k < t.d.rank ? acc : 0;
    if (k < t.d.rank) acc *= t.d.dims[k];
  }
}

// Lists the iteration dimensions by increasing output stride: consecutive threads then write neighbouring
// elements.  `with_istride`: the input strides belong to the iteration dimensions and move with them.
void sort_by_output_stride(RelayoutParams& p, bool with_istride) {
  for (int a = 0; a < p.rank; ++a)
    for (int b = a + 1; b < p.rank; ++b)
      if (p.ostride[b] < p.ostride[a] || (p.ostride[b] == p.ostride[a] && p.dims[b] < p.dims[a])) {
        std::swap(p.dims[a], p.dims[b]);
        std::swap(p.ostride[a], p.ostride[b]);
        std::swap(p.lstride[a], p.lstride[b]);
        if (with_istride) std::swap(p.istride[a], p.istride[b]);
      }
}

RelayoutParams relayout_base(const TensorRec& shape_of) {
  RelayoutParams p;
  std::memset(&p, 0, sizeof(p));
  p.rank = static_cast<int>(shape_of.d.rank);
  p.total = 1;
  for (int k = 0; k < 4; ++k) {
    p.dims[k] = k < p.rank ? static_cast<int>(shape_of.d.dims[k]) : 1;
    p.idims[k] = 1;
    p.total *= p.dims[k];
  }
  p.elem = static_cast<int>(dtype_size(shape_of.d.dtype));
  return p;
}

b2vx_status plan_contraction(b2vx_graph* g, uint32_t node_index, const char* label, TensorRec& x, TensorRec& w,
                             TensorRec* bias, TensorRec& y, int kw, int kh, const uint32_t stride[2],
                             const uint32_t dil[2], const uint32_t pad[4]) {
  // float32 layers accept a kernel and a bias produced at run time (a graph input, or the Transpose that layout
  // inference puts behind one); the quantized paths pack their weights when the graph is compiled
  const bool runtime_ok = x.d.dtype == B2VX_DT_FLOAT32;
  if (!w.host_valid && !(runtime_ok && w.is_activation)) return fail(g, B2VX_UNSUPPORTED, std::string(label) + ": weights must be a CONSTANT tensor with data");
  if (bias && !bias->host_valid && !(runtime_ok && bias->is_activation))
    return fail(g, B2VX_UNSUPPORTED, std::string(label) + ": bias must be a CONSTANT tensor with data");
  const ConvGeom geo = conv_geom(x, y, kw, kh, stride, dil, pad);
  const uint64_t P = static_cast<uint64_t>(y.N) * y.H * y.W;
  const uint64_t macs = P * y.C * static_cast<uint64_t>(kw) * kh * x.C;
  const uint64_t abytes = x.elems() * dtype_size(x.d.dtype) + y.elems() * dtype_size(y.d.dtype) + w.bytes() +
                          (bias ? bias->bytes() : 0);

  // ---- float32
  if (x.d.dtype == B2VX_DT_FLOAT32) {
    if (w.d.dtype != B2VX_DT_FLOAT32 || y.d.dtype != B2VX_DT_FLOAT32 || (bias && bias->d.dtype != B2VX_DT_FLOAT32))
      return fail(g, B2VX_UNSUPPORTED, std::string(label) + ": float32 input needs float32 weights, bias and output");
    float *dw = nullptr, *db = nullptr;
    b2vx_status st = B2VX_OK;
    if (w.host_valid) {
      std::vector<float> wv(reinterpret_cast<const float*>(w.host.data()), reinterpret_cast<const float*>(w.host.data()) + w.elems());
      st = upload(g, wv, &dw);
      if (st != B2VX_OK) return st;
    } else {
      // run-time kernel: every run first copies it from its storage into the dense [kw, kh, Ic, Oc] order the kernel reads
      void* dense = nullptr;
      st = dev_alloc(g, &dense, w.bytes());
      if (st != B2VX_OK) return st;
      dw = static_cast<float*>(dense);
      RelayoutParams rp = relayout_base(w);
      dense_strides(w, rp.ostride);
      cl_strides(w, rp.istride);
      const void* wp = cl_in(w);
      Step sw;
      sw.info = make_info("kernel_to_dense", node_index, 0, 2 * w.bytes());
      sw.fn = [=](cudaStream_t st2) { launch_relayout(wp, dense, rp, st2); return cudaGetLastError(); };
      g->steps.push_back(std::move(sw));
    }
    if (bias && bias->host_valid) {
      std::vector<float> bv(reinterpret_cast<const float*>(bias->host.data()), reinterpret_cast<const float*>(bias->host.data()) + bias->elems());
      st = upload(g, bv, &db);
      if (st != B2VX_OK) return st;
    } else if (bias) {
      db = static_cast<float*>(const_cast<void*>(cl_in(*bias)));   // rank 1: the storage is the dense vector
    }
    const float* xp = static_cast<const float*>(cl_in(x));
    float* yp = static_cast<float*>(y.d_cl);
    const int w_ic = x.C;
    Step s;
    s.info = make_info("conv_f32", node_index, 2 * macs, abytes);
    s.fn = [=](cudaStream_t st2) { launch_conv_f32(xp, dw, db, 0, w_ic, geo, yp, st2); return cudaGetLastError(); };
    g->steps.push_back(std::move(s));
    return B2VX_OK;
  }

  // ---- quantized
  if (!is_q8(x.d.dtype) || !is_q8(w.d.dtype) || !is_q8(y.d.dtype))
    return fail(g, B2VX_UNSUPPORTED, std::string(label) + ": supported types are int8/uint8 activations and weights, or all float32");
  if (bias && bias->d.dtype != B2VX_DT_INT32) return fail(g, B2VX_UNSUPPORTED, std::string(label) + ": bias of a quantized op must be int32");
  if (x.d.quant_type != B2VX_QUANT_ASYMMETRIC || y.d.quant_type != B2VX_QUANT_ASYMMETRIC)
    return fail(g, B2VX_QUANT_MISMATCH, std::string(label) + ": activations must use ASYMMETRIC quantization");
  if (w.d.quant_type == B2VX_QUANT_SYMMETRIC_PER_CHANNEL) {
    if (static_cast<int>(w.scales.size()) != y.C) return fail(g, B2VX_QUANT_MISMATCH, std::string(label) + ": per-channel scale count != output channels");
  } else if (w.d.quant_type != B2VX_QUANT_ASYMMETRIC) {
    return fail(g, B2VX_QUANT_MISMATCH, std::string(label) + ": weights need ASYMMETRIC or SYMMETRIC_PER_CHANNEL quantization");
  }
  if (!quant_check(x, w, bias)) return fail(g, B2VX_QUANT_MISMATCH, std::string(label) + ": bias scale != input scale * weight scale");

  const int taps = kw * kh;
  const bool x_signed = x.d.dtype == B2VX_DT_INT8;
  const bool has_pad = pad[0] || pad[1] || pad[2] || pad[3];
  bool any_dz = false, dz_is_uniform = true;
  int dz_value = 0;
  {
    const bool w_u8 = w.d.dtype == B2VX_DT_UINT8;
    if (w.d.quant_type == B2VX_QUANT_SYMMETRIC_PER_CHANNEL) {
      for (size_t i = 0; i < w.zps.size(); ++i) {
        const int dz = w_u8 ? w.zps[i] - 128 : w.zps[i];
        any_dz = any_dz || dz != 0;
        if (i == 0) dz_value = dz;
        else dz_is_uniform = dz_is_uniform && dz == dz_value;
      }
    } else {
      dz_value = w_u8 ? w.zp() - 128 : w.zp();
      any_dz = dz_value != 0;
    }
  }
  // The im2col matrix is the input itself when the window is 1x1/stride 1/no
  // padding, or when the window covers the whole (unpadded) input.
  const bool identity_1x1 = kw == 1 && kh == 1 && geo.sx == 1 && geo.sy == 1 && !has_pad;
  const bool identity_full = kw == x.W && kh == x.H && !has_pad && y.W == 1 && y.H == 1 && geo.dx == 1 && geo.dy == 1;
  const bool tc_ok = g->use_tc && (!any_dz || dz_is_uniform);   // one leftover weight zero point: the S column handles it

  ContractEpilogue ep;
  std::memset(&ep, 0, sizeof(ep));
  ep.out = out_quant(y);
  PackedContraction pk;

  if (tc_ok) {
    // Four ways to present the input to the GEMM kernel:
    //   identity  the channels-last input already is the A matrix (1x1/s1, or a window = whole input);
    //   implicit  filter taps fetched as shifted 4-D TMA boxes, zero fill as padding; with a non-zero input
    //             zero point the border pixels get a per-class correction in the epilogue;
    //   whcn      first layers with < 16 channels: im2col straight from the WHCN graph input, K = (c,ky,kx);
    //   im2col    everything else: explicit matrix in scratch memory, padding filled with zx.
    //   whcn8     the same with filter rows of 2..8 taps padded to 4 or 8, K = (ky,c,kx'): whole input words per piece;
    enum { IDENTITY, IMPLICIT, WHCN, WHCN8, IM2COL } mode;
    const int padk = kw <= 4 ? 4 : 8;   // whcn8 mode: bytes per (pixel, ky, c)
    static const bool allow_strided = [] { const char* e = std::getenv("B2VX_IMPLICIT_STRIDED"); return !(e && e[0] == '0'); }();
    const bool strided = geo.sx != 1 || geo.sy != 1;
    // Border classes of an implicit convolution: output rows (columns) grouped by which ky (kx) fall
    // outside the input.  Few classes exist (3 x 3 for a 3x3/stride-1 SAME convolution).
    std::vector<uint8_t> row_class(y.H, 0), col_class(y.W, 0);
    std::vector<uint32_t> row_masks(1, 0u), col_masks(1, 0u);   // class id -> bitmask of out-of-bounds taps
    bool classes_ok = kh <= 32 && kw <= 32;
    const bool need_border = x.zp() != 0 && has_pad;
    if (need_border && classes_ok) {
      auto classify = [&](int out_n, int in_n, int k, int stride_, int dil_, int pad0, std::vector<uint8_t>& cls,
                          std::vector<uint32_t>& masks) {
        for (int o = 0; o < out_n; ++o) {
          uint32_t m = 0;
          for (int t = 0; t < k; ++t) {
            const int i = o * stride_ - pad0 + t * dil_;
            if (i < 0 || i >= in_n) m |= 1u << t;
          }
          size_t id = 0;
          while (id < masks.size() && masks[id] != m) ++id;
          if (id == masks.size()) masks.push_back(m);
          if (id > 255) return false;
          cls[o] = static_cast<uint8_t>(id);
        }
        return true;
      };
      classes_ok = classify(y.H, x.H, kh, geo.sy, geo.dy, geo.pt, row_class, row_masks) &&
                   classify(y.W, x.W, kw, geo.sx, geo.dx, geo.pl, col_class, col_masks) &&
                   row_masks.size() * col_masks.size() <= 256;
    }
    if (identity_1x1 || identity_full) mode = IDENTITY;
    else if (x.C >= 16 && (!need_border || classes_ok) && (!strided || allow_strided)) mode = IMPLICIT;
    else if (x.C < 16 && (x.d.attr & B2VX_ATTR_INPUT) && x.d_io != nullptr && kw >= 2 && kw <= 8 && geo.dx == 1 && geo.dy == 1 &&
             static_cast<size_t>(x.C) * kh * im2col_whcn8_pitch(geo, padk) + 16 <= 40u * 1024u)
      mode = WHCN8;  // filter rows of up to 8 (or 4) taps: 8 (or 4) consecutive input bytes per (pixel, ky, c)
    else if (x.C < 16 && (x.d.attr & B2VX_ATTR_INPUT) && x.d_io != nullptr &&
             static_cast<size_t>(x.C) * kh * ((geo.Wo - 1) * geo.sx + (kw - 1) * geo.dx + 1) + 4u * round_up(taps * x.C, 16) <= 40u * 1024u)
      mode = WHCN;   // the staging rows of one output row fit in shared memory
    else mode = IM2COL;
    int Cs, Kp, M;
    const void* A = nullptr;
    const bool need_im2col = mode == WHCN || mode == WHCN8 || mode == IM2COL;
    if (mode == IDENTITY && identity_1x1) { Cs = x.Cp; Kp = x.Cp; M = static_cast<int>(P); A = cl_in(x); }
    else if (mode == IDENTITY) { Cs = x.Cp; Kp = taps * x.Cp; M = y.N; A = cl_in(x); }
    else if (mode == IMPLICIT) { Cs = x.Cp; Kp = taps * x.Cp; M = static_cast<int>(P); A = cl_in(x); }
    else if (mode == WHCN) { Cs = x.C; Kp = round_up(taps * x.C, 16); M = static_cast<int>(P); }
    else if (mode == WHCN8) {
      // rows of the matrix are read by TMA in 64- or 128-byte pieces: a pitch that is a multiple of 64
      // keeps every piece on whole 32-byte sectors
      Cs = x.C; Kp = round_up(kh * x.C * padk, 16); if (Kp > 64) Kp = round_up(Kp, 64); M = static_cast<int>(P);
    }
    else { Cs = x.C < 16 ? x.C : x.Cp; Kp = round_up(taps * Cs, 16); M = static_cast<int>(P); }
    // Few rows (decode-like FullyConnected, 1x1 on a handful of pixels): weight streaming on CUDA cores.
    // (B2VX_FC_SMALL_M=0, read when the graph is created, keeps such shapes on the tensor-core kernel)
    // Measured at N = K = 4096: faster than the 128-row tile up to 8 rows (1.8x at one row); at 16 rows the
    // dp4a rate bounds it and the tensor-core kernel is level or better.
    if (g->fc_small_m && mode == IDENTITY && M <= 16 && (!any_dz || x.C == x.Cp)) {
      pack_contraction(x, w, bias, kw, kh, x.C, Cs, Kp, y.C, y.Cp, 1, y.Cp, y.Cp, 0, &pk);
      int8_t* dw8s = nullptr; int32_t* dbias_s = nullptr; float* dscale_s = nullptr;
      b2vx_status sts = upload(g, pk.w8, &dw8s);
      if (sts == B2VX_OK) sts = upload(g, pk.bias_full, &dbias_s);
      if (sts == B2VX_OK) sts = upload(g, pk.acc_scale, &dscale_s);
      if (sts != B2VX_OK) return sts;
      ep.bias_full = dbias_s;
      ep.acc_scale = dscale_s;
      ep.dz_uniform = any_dz ? dz_value : 0;
      void* ycl_s = y.d_cl;
      const int ldd_s = y.Cp, oc_s = y.C, ocp_s = y.Cp;
      Step s_fc;
      s_fc.info = make_info("fc_small_m", node_index, 2 * macs, abytes);
      s_fc.fn = [=](cudaStream_t st2) {
        launch_fc_small_m(A, x_signed, dw8s, M, Kp, oc_s, ocp_s, ep, ycl_s, ldd_s, st2);
        return cudaGetLastError();
      };
      g->steps.push_back(std::move(s_fc));
      return B2VX_OK;
    }
    const GemmTcTiling tiling = gemm_tc_choose_tiling(M, y.Cp, Kp, any_dz ? 1 : 0);
    const int Np = tiling.n_tiles * tiling.rows;
    pack_contraction(x, w, bias, kw, kh, x.C, Cs, Kp, y.C, y.Cp, tiling.n_tiles, tiling.data, tiling.rows, mode == WHCN ? 1 : (mode == WHCN8 ? (padk == 8 ? 2 : 3) : 0), &pk);
    ep.dz_uniform = any_dz ? dz_value : 0;
    if (mode == IMPLICIT && need_border) {
      // correction of class (r, c) = minus the folded contribution of every tap that is out of bounds there
      const size_t ncls = row_masks.size() * col_masks.size();
      std::vector<int32_t> corr(ncls * y.Cp, 0);
      for (size_t r = 0; r < row_masks.size(); ++r)
        for (size_t c = 0; c < col_masks.size(); ++c)
          for (int ky = 0; ky < kh; ++ky)
            for (int kx = 0; kx < kw; ++kx) {
              if (!((row_masks[r] >> ky) & 1u) && !((col_masks[c] >> kx) & 1u)) continue;
              const int32_t* tc = pk.tapc.data() + static_cast<size_t>(ky * kw + kx) * y.Cp;
              int32_t* dst = corr.data() + (r * col_masks.size() + c) * y.Cp;
              for (int oc = 0; oc < y.Cp; ++oc) dst[oc] -= tc[oc];
            }
      int32_t* dcorr = nullptr; uint8_t *drow = nullptr, *dcol = nullptr;
      b2vx_status stc = upload(g, corr, &dcorr);
      if (stc == B2VX_OK) stc = upload(g, row_class, &drow);
      if (stc == B2VX_OK) stc = upload(g, col_class, &dcol);
      if (stc != B2VX_OK) return stc;
      ep.border_corr = dcorr;
      ep.row_class = drow;
      ep.col_class = dcol;
      ep.n_col_classes = static_cast<int>(col_masks.size());
    }
    int8_t* dw8 = nullptr; int32_t* dbias = nullptr; float* dscale = nullptr;
    b2vx_status st = upload(g, pk.w8, &dw8);
    if (st == B2VX_OK) st = upload(g, pk.bias_full, &dbias);
    if (st == B2VX_OK) st = upload(g, pk.acc_scale, &dscale);
    if (st != B2VX_OK) return st;
    ep.bias_full = dbias;
    ep.acc_scale = dscale;
    {
      // largest |acc * acc_scale / out scale| any input can produce: decides whether the epilogue may
      // use its fast rounding (valid below 2^21)
      // (bounded per output channel from the weights themselves; the integer the epilogue converts is that true
      // accumulator: the S term of a weight zero point and the border corrections are already in it)
      const double tmax = pk.real_max / std::fabs(static_cast<double>(ep.out.scale));
      ep.exact_only = !(tmax < 2097152.0);
    }
    void* fused_out = nullptr;
    if (g->fuse_request >= 0) {
      // absorb the Add that follows: table over (this convolution's byte, the residual's byte)
      NodeRec& ad = g->nodes[g->fuse_request];
      TensorRec& res = g->tensors[g->fuse_residual];
      TensorRec& ao = g->tensors[ad.out];
      if (res.Cp == y.Cp && ao.Cp == y.Cp && res.cl_bytes == y.cl_bytes && ao.cl_bytes == y.cl_bytes) {
        const bool ys = y.d.dtype == B2VX_DT_INT8, rs = res.d.dtype == B2VX_DT_INT8;
        const OutQuant aq = out_quant(ao);
        std::vector<uint8_t> table(65536);
        for (int iq = 0; iq < 256; ++iq) {
          const int q = ys ? static_cast<int>(static_cast<int8_t>(iq)) : iq;
          const float fq = (static_cast<float>(q) - static_cast<float>(y.zp())) * y.scale();
          for (int ir = 0; ir < 256; ++ir) {
            const int r = rs ? static_cast<int>(static_cast<int8_t>(ir)) : ir;
            const float fr = (static_cast<float>(r) - static_cast<float>(res.zp())) * res.scale();
            // operand order of the float addition as in the Add node (addition commutes, kept for the record)
            const float sum = ad.in[0] == g->fuse_residual ? fr + fq : fq + fr;
            table[iq * 256 + (ir ^ ((iq & 31) << 2))] = static_cast<uint8_t>(host_requant(sum, aq) & 0xFF);
          }
        }
        uint8_t* dtab = nullptr;
        const b2vx_status stt = upload(g, table, &dtab);
        if (stt != B2VX_OK) return stt;
        ep.add_residual = static_cast<const uint8_t*>(cl_in(res));
        ep.add_table = dtab;
        fused_out = ao.d_cl;
        g->fuse_done = true;
      }
    }
    if (need_im2col) {
      const size_t need = static_cast<size_t>(M) * Kp;
      g->scratch_bytes = std::max(g->scratch_bytes, need);
    }
    // The GEMM plan bakes the A address into a TMA tensor map; for the im2col
    // form that address is the graph's scratch buffer, which is sized over all
    // nodes and allocated after planning, so plan creation is deferred to a
    // finalizer that Compile runs at its end.
    const int zx = x.zp();
    const std::string lbl = label;
    void* ycl = fused_out ? fused_out : y.d_cl;
    const int ldd = y.Cp, Oc = y.C, y_signed = y.d.dtype == B2VX_DT_INT8;
    if (mode == WHCN8) {
      const void* xio = x.d_io;
      Step s_col;
      s_col.info = make_info(padk == 8 ? "im2col_whcn8" : "im2col_whcn4", node_index, 0, x.elems() + static_cast<uint64_t>(M) * Kp);
      s_col.fn = [=](cudaStream_t st2) {
        launch_im2col_whcn8(xio, Kp, zx, geo, padk, g->scratch, st2);
        return cudaGetLastError();
      };
      g->steps.push_back(std::move(s_col));
    } else if (mode == WHCN) {
      const void* xio = x.d_io;
      Step s_col;
      s_col.info = make_info("im2col_whcn", node_index, 0, x.elems() + static_cast<uint64_t>(M) * Kp);
      s_col.fn = [=](cudaStream_t st2) {
        launch_im2col_whcn(xio, Kp, zx, geo, g->scratch, st2);
        return cudaGetLastError();
      };
      g->steps.push_back(std::move(s_col));
    } else if (mode == IM2COL) {
      const void* xcl = cl_in(x);
      Step s_col;
      s_col.info = make_info("im2col", node_index, 0, x.elems() + static_cast<uint64_t>(M) * Kp);
      s_col.fn = [=](cudaStream_t st2) {
        launch_im2col(xcl, Cs, Kp, zx, geo, g->scratch, st2);
        return cudaGetLastError();
      };
      g->steps.push_back(std::move(s_col));
    }
    auto plan_holder = std::make_shared<GemmTcPlan*>(nullptr);
    const bool implicit = mode == IMPLICIT;
    g->finalizers.push_back([=]() -> b2vx_status {
      char err[160] = {0};
      GemmTcPlan* pl;
      if (implicit) {
        pl = gemm_tc_conv_plan_create(A, x_signed, dw8, geo, Np, ycl, ep, g->d_status, err, sizeof(err), &tiling);
      } else {
        const void* Aptr = need_im2col ? g->scratch : A;
        pl = gemm_tc_plan_create(Aptr, x_signed, dw8, M, Np, Kp, Oc, ycl, ldd, y_signed, ep, g->d_status, err, sizeof(err), &tiling);
      }
      if (!pl) return fail(g, B2VX_UNSUPPORTED, lbl + ": " + err);
      g->gemm_plans.push_back(pl);
      *plan_holder = pl;
      if (implicit && gemm_tc_plan_is_halo(pl)) {
        // "gemm_i8_tc(implicit...)" -> "gemm_i8_tc(halo...)": one input patch per tile instead of one box per tap
        for (Step& st : g->steps) {
          if (st.tag != plan_holder.get()) continue;
          std::string name = st.info.name;
          const size_t at = name.find("implicit");
          if (at != std::string::npos) {
            name.replace(at, 8, "halo");
            std::snprintf(st.info.name, sizeof(st.info.name), "%s", name.c_str());
          }
        }
      }
      return B2VX_OK;
    });
    Step s_gemm;
    {
      std::string kname = implicit ? "gemm_i8_tc(implicit" : (need_im2col ? "gemm_i8_tc(im2col" : "gemm_i8_tc(");
      if (fused_out) kname += kname.back() == '(' ? "+add" : ",+add";
      kname += ")";
      if (kname == "gemm_i8_tc()") kname = "gemm_i8_tc";
      s_gemm.info = make_info(kname.c_str(), node_index, 2 * macs, abytes + (fused_out ? y.bytes() : 0));
    }
    s_gemm.fn = [=](cudaStream_t st2) -> cudaError_t { return gemm_tc_launch(*plan_holder, st2); };
    s_gemm.tag = plan_holder.get();
    g->steps.push_back(std::move(s_gemm));
    return B2VX_OK;
  }

  // CUDA-core path: K = tap*Cp + c, out-of-bounds taps are skipped and corrected per tap.
  const int Kp = taps * x.Cp;
  pack_contraction(x, w, bias, kw, kh, x.C, x.Cp, Kp, y.C, y.Cp, 1, y.Cp, y.Cp + 1, 0, &pk);
  int8_t* dw8 = nullptr; int32_t *dbias = nullptr, *ddz = nullptr, *dtapc = nullptr; float* dscale = nullptr;
  b2vx_status st = upload(g, pk.w8, &dw8);
  if (st == B2VX_OK) st = upload(g, pk.bias_full, &dbias);
  if (st == B2VX_OK) st = upload(g, pk.acc_scale, &dscale);
  if (st == B2VX_OK && pk.need_s) st = upload(g, pk.dz, &ddz);
  if (st == B2VX_OK && has_pad && x.zp() != 0) st = upload(g, pk.tapc, &dtapc);
  if (st != B2VX_OK) return st;
  ep.bias_full = dbias;
  ep.acc_scale = dscale;
  ep.dz = ddz;
  ep.tapc = dtapc;
  const void* xcl = cl_in(x);
  void* ycl = y.d_cl;
  Step s;
  s.info = make_info("conv_simt", node_index, 2 * macs, abytes);
  s.fn = [=](cudaStream_t st2) { launch_conv_simt(xcl, x_signed, dw8, Kp, geo, ep, ycl, st2); return cudaGetLastError(); };
  g->steps.push_back(std::move(s));
  return B2VX_OK;
}

// ---------------------------------------------------------------- per-node planning

b2vx_status plan_conv(b2vx_graph* g, uint32_t idx, NodeRec& n) {
  TensorRec& x = g->tensors[n.in[0]];
  TensorRec& w = g->tensors[n.in[1]];
  TensorRec* bias = n.in[2] != B2VX_NO_TENSOR ? &g->tensors[n.in[2]] : nullptr;
  TensorRec& y = g->tensors[n.out];
  const b2vx_conv2d_desc& c = n.p.conv;
  const int kw = w.d.dims[0], kh = w.d.dims[1];
  if (c.multiplier < 1) {
    if (static_cast<int>(w.d.dims[2]) != x.C || static_cast<int>(w.d.dims[3]) != y.C)
      return fail(g, B2VX_SHAPE_MISMATCH, "conv2d: kernel shape does not match input/output channels");
    if (w.d.quant_type == B2VX_QUANT_SYMMETRIC_PER_CHANNEL && w.d.channel_dim != 3)
      return fail(g, B2VX_QUANT_MISMATCH, "conv2d: per-channel weights must use channel_dim 3");
    return plan_contraction(g, idx, "conv2d", x, w, bias, y, kw, kh, c.stride, c.dilation, n.pad);
  }
  // depthwise
  if (static_cast<int>(w.d.dims[2]) != x.C * c.multiplier || y.C != x.C * c.multiplier)
    return fail(g, B2VX_SHAPE_MISMATCH, "depthwise conv2d: kernel channels != input channels * multiplier");
  if (!w.host_valid || (bias && !bias->host_valid)) return fail(g, B2VX_UNSUPPORTED, "depthwise conv2d: weights and bias must be constants");
  const ConvGeom geo = conv_geom(x, y, kw, kh, c.stride, c.dilation, n.pad);
  const uint64_t macs = static_cast<uint64_t>(y.N) * y.H * y.W * y.C * kw * kh;
  const uint64_t abytes = x.bytes() + y.bytes() + w.bytes() + (bias ? bias->bytes() : 0);
  if (x.d.dtype == B2VX_DT_FLOAT32) {
    if (w.d.dtype != B2VX_DT_FLOAT32 || y.d.dtype != B2VX_DT_FLOAT32 || (bias && bias->d.dtype != B2VX_DT_FLOAT32))
      return fail(g, B2VX_UNSUPPORTED, "depthwise conv2d: float32 input needs float32 weights, bias and output");
    float *dw = nullptr, *db = nullptr;
    std::vector<float> wv(reinterpret_cast<const float*>(w.host.data()), reinterpret_cast<const float*>(w.host.data()) + w.elems());
    b2vx_status st = upload(g, wv, &dw);
    if (st != B2VX_OK) return st;
    if (bias) {
      std::vector<float> bv(reinterpret_cast<const float*>(bias->host.data()), reinterpret_cast<const float*>(bias->host.data()) + bias->elems());
      st = upload(g, bv, &db);
      if (st != B2VX_OK) return st;
    }
    const float* xp = static_cast<const float*>(cl_in(x));
    float* yp = static_cast<float*>(y.d_cl);
    const int mult = c.multiplier;
    Step s;
    s.info = make_info("depthwise_f32", idx, 2 * macs, abytes);
    s.fn = [=](cudaStream_t st2) { launch_conv_f32(xp, dw, db, mult, 0, geo, yp, st2); return cudaGetLastError(); };
    g->steps.push_back(std::move(s));
    return B2VX_OK;
  }
  if (!is_q8(x.d.dtype) || !is_q8(w.d.dtype) || !is_q8(y.d.dtype) || (bias && bias->d.dtype != B2VX_DT_INT32))
    return fail(g, B2VX_UNSUPPORTED, "depthwise conv2d: unsupported dtype combination");
  const bool per_ch = w.d.quant_type == B2VX_QUANT_SYMMETRIC_PER_CHANNEL;
  if (per_ch && static_cast<int>(w.scales.size()) != y.C) return fail(g, B2VX_QUANT_MISMATCH, "depthwise conv2d: per-channel scale count != channels");
  if (per_ch && w.d.channel_dim != 2) return fail(g, B2VX_QUANT_MISMATCH, "depthwise conv2d: per-channel weights must use channel_dim 2");
  if (!quant_check(x, w, bias)) return fail(g, B2VX_QUANT_MISMATCH, "depthwise conv2d: bias scale != input scale * weight scale");
  const int taps = kw * kh;
  std::vector<int16_t> wd(static_cast<size_t>(taps) * y.Cp, 0);
  std::vector<int32_t> bv(y.Cp, 0);
  std::vector<float> sc(y.Cp, 0.0f);
  const bool w_u8 = w.d.dtype == B2VX_DT_UINT8;
  for (int oc = 0; oc < y.C; ++oc) {
    const int zw = per_ch ? (w.zps.empty() ? 0 : w.zps[oc]) : w.zp();
    for (int t = 0; t < taps; ++t) {
      const size_t src = static_cast<size_t>(oc) * taps + t;
      const int v = w_u8 ? static_cast<int>(w.host[src]) : static_cast<int>(reinterpret_cast<const int8_t*>(w.host.data())[src]);
      wd[static_cast<size_t>(t) * y.Cp + oc] = static_cast<int16_t>(v - zw);
    }
    bv[oc] = bias ? reinterpret_cast<const int32_t*>(bias->host.data())[oc] : 0;
    sc[oc] = x.scale() * (per_ch ? w.scales[oc] : w.scale());
  }
  int16_t* dwd = nullptr; int32_t* db = nullptr; float* dsc = nullptr;
  b2vx_status st = upload(g, wd, &dwd);
  if (st == B2VX_OK) st = upload(g, bv, &db);
  if (st == B2VX_OK) st = upload(g, sc, &dsc);
  if (st != B2VX_OK) return st;
  const void* xcl = cl_in(x);
  void* ycl = y.d_cl;
  const int xs = x.d.dtype == B2VX_DT_INT8, zx = x.zp(), mult = c.multiplier;
  const OutQuant oq = out_quant(y);
  if (mult == 1 && taps <= 64) {
    // dp2a kernel: weights as positioned 16-bit halves, zero-point term folded into the bias
    std::vector<uint32_t> wtab(static_cast<size_t>(taps) * y.Cp, 0u);
    std::vector<int32_t> bfull(y.Cp, 0);
    const int zx_eff = zx + (xs ? 128 : 0);
    double bmax = 0.0, smax = 0.0;
    for (int oc = 0; oc < y.C; ++oc) {
      int64_t wsum = 0;
      for (int t = 0; t < taps; ++t) {
        const int v = wd[static_cast<size_t>(t) * y.Cp + oc];
        wsum += v;
        wtab[static_cast<size_t>(t) * y.Cp + oc] = (static_cast<uint32_t>(v) & 0xFFFFu) << (16 * (oc & 1));
      }
      bfull[oc] = static_cast<int32_t>(bv[oc] - static_cast<int64_t>(zx_eff) * wsum);
      bmax = std::max(bmax, std::fabs(static_cast<double>(bfull[oc])));
      smax = std::max(smax, std::fabs(static_cast<double>(sc[oc])));
    }
    const double tmax = (static_cast<double>(taps) * 255.0 * 255.0 + bmax) * smax / std::fabs(static_cast<double>(oq.scale));
    const int exact_only = !(tmax < 2097152.0);
    uint32_t* dwt = nullptr; int32_t* dbf = nullptr; uint32_t* dwv = nullptr;
    st = upload(g, wtab, &dwt);
    if (st == B2VX_OK) st = upload(g, bfull, &dbf);
    if (st == B2VX_OK && kh == 3 && kw == 3) {
      // strip form of the kernel: window rows 0 and 1 of a column as the two halves of one word, row 2 as in wtab
      std::vector<uint32_t> wv(static_cast<size_t>(6) * y.Cp, 0u);
      for (int oc = 0; oc < y.C; ++oc)
        for (int kx = 0; kx < 3; ++kx) {
          const uint32_t r0 = static_cast<uint32_t>(wd[static_cast<size_t>(kx) * y.Cp + oc]) & 0xFFFFu;
          const uint32_t r1 = static_cast<uint32_t>(wd[static_cast<size_t>(3 + kx) * y.Cp + oc]) & 0xFFFFu;
          wv[static_cast<size_t>(kx) * y.Cp + oc] = r0 | (r1 << 16);
          wv[static_cast<size_t>(3 + kx) * y.Cp + oc] = wtab[static_cast<size_t>(6 + kx) * y.Cp + oc];
        }
      st = upload(g, wv, &dwv);
    }
    if (st != B2VX_OK) return st;
    Step s16;
    s16.info = make_info("depthwise_q16", idx, 2 * macs, abytes);
    s16.fn = [=](cudaStream_t st2) { launch_depthwise_q16(xcl, xs, zx, dwt, dwv, dbf, dsc, geo, oq, exact_only, ycl, st2); return cudaGetLastError(); };
    g->steps.push_back(std::move(s16));
    return B2VX_OK;
  }
  Step s;
  s.info = make_info("depthwise_q", idx, 2 * macs, abytes);
  s.fn = [=](cudaStream_t st2) { launch_depthwise_q(xcl, xs, zx, dwd, db, dsc, mult, geo, oq, ycl, st2); return cudaGetLastError(); };
  g->steps.push_back(std::move(s));
  return B2VX_OK;
}

b2vx_status plan_fc(b2vx_graph* g, uint32_t idx, NodeRec& n) {
  TensorRec& x = g->tensors[n.in[0]];
  TensorRec& w = g->tensors[n.in[1]];
  TensorRec* bias = n.in[2] != B2VX_NO_TENSOR ? &g->tensors[n.in[2]] : nullptr;
  TensorRec& y = g->tensors[n.out];
  // dims [0..axis] flatten into K; everything after must be the batch (N) axis.
  size_t K = 1;
  for (uint32_t i = 0; i <= n.p.fc.axis; ++i) K *= x.d.dims[i];
  const size_t batch = x.elems() / K;
  if (K != static_cast<size_t>(x.W) * x.H * x.C || static_cast<int>(batch) != x.N)
    return fail(g, B2VX_UNSUPPORTED, "fully_connected: axis must flatten every non-batch dimension");
  if (w.d.dims[0] != K) return fail(g, B2VX_SHAPE_MISMATCH, "fully_connected: weight K != flattened input size");
  if (w.d.quant_type == B2VX_QUANT_SYMMETRIC_PER_CHANNEL && w.d.channel_dim != 1)
    return fail(g, B2VX_QUANT_MISMATCH, "fully_connected: per-channel weights must use channel_dim 1");
  // A weight [K,N] with k = x + W*(y + H*c) is a WHIcOc kernel [W,H,C,N]: the
  // op is a convolution whose window is the whole input.
  TensorRec yv = y;   // view of the output as [1,1,N_out,batch]
  yv.W = 1; yv.H = 1; yv.C = static_cast<int>(w.d.dims[1]); yv.N = x.N;
  if (static_cast<size_t>(yv.C) * yv.N != y.elems() || y.C != yv.C || y.N != yv.N)
    return fail(g, B2VX_SHAPE_MISMATCH, "fully_connected: output must be [weights, batch]");
  const uint32_t one[2] = {1, 1}, nopad[4] = {0, 0, 0, 0};
  return plan_contraction(g, idx, "fully_connected", x, w, bias, y, x.W, x.H, one, one, nopad);
}

b2vx_status plan_pool(b2vx_graph* g, uint32_t idx, NodeRec& n) {
  TensorRec& x = g->tensors[n.in[0]];
  TensorRec& y = g->tensors[n.out];
  const b2vx_pool2d_desc& c = n.p.pool;
  if (c.type != B2VX_POOL_MAX && c.type != B2VX_POOL_AVG && c.type != B2VX_POOL_L2 && c.type != B2VX_POOL_AVG_ANDROID)
    return fail(g, B2VX_UNSUPPORTED, "pool2d: the type must be MAX, AVG, L2 or AVG_ANDROID");
  if (x.d.dtype != y.d.dtype) return fail(g, B2VX_UNSUPPORTED, "pool2d: input and output dtype must match");
  const uint32_t one[2] = {1, 1};
  const ConvGeom geo = conv_geom(x, y, c.ksize[0], c.ksize[1], c.stride, one, n.pad);
  const uint64_t abytes = x.bytes() + y.bytes();
  const int type = c.type;
  Step s;
  if (x.d.dtype == B2VX_DT_FLOAT32) {
    const float* xp = static_cast<const float*>(cl_in(x));
    float* yp = static_cast<float*>(y.d_cl);
    s.info = make_info("pool_f32", idx, 0, abytes);
    s.fn = [=](cudaStream_t st2) { launch_pool_f32(xp, type, geo, yp, st2); return cudaGetLastError(); };
  } else if (is_q8(x.d.dtype)) {
    const void* xp = cl_in(x);
    void* yp = y.d_cl;
    const int sg = x.d.dtype == B2VX_DT_INT8, zx = x.zp(), same = x.scale() == y.scale() && x.zp() == y.zp();
    const float sx = x.scale();
    const OutQuant oq = out_quant(y);
    s.info = make_info("pool_q", idx, 0, abytes);
    s.fn = [=](cudaStream_t st2) { launch_pool_q(xp, sg, type, sx, zx, same, geo, oq, yp, st2); return cudaGetLastError(); };
  } else {
    return fail(g, B2VX_UNSUPPORTED, "pool2d: unsupported dtype");
  }
  g->steps.push_back(std::move(s));
  return B2VX_OK;
}

b2vx_status plan_add(b2vx_graph* g, uint32_t idx, NodeRec& n) {
  TensorRec& a = g->tensors[n.in[0]];
  TensorRec& b = g->tensors[n.in[1]];
  TensorRec& y = g->tensors[n.out];
  const uint64_t abytes = a.bytes() + b.bytes() + y.bytes();
  Step s;
  const bool same_shape = a.N == y.N && a.H == y.H && a.W == y.W && a.C == y.C && b.N == y.N && b.H == y.H && b.W == y.W && b.C == y.C;
  if (!same_shape) {
    const bool all_f32 = a.d.dtype == B2VX_DT_FLOAT32 && b.d.dtype == B2VX_DT_FLOAT32 && y.d.dtype == B2VX_DT_FLOAT32;
    const bool all_q8 = is_q8(a.d.dtype) && is_q8(b.d.dtype) && is_q8(y.d.dtype);
    if (!all_f32 && !all_q8) return fail(g, B2VX_UNSUPPORTED, "add: operands must be all int8/uint8 or all float32");
    const void *ap = cl_in(a), *bp = cl_in(b);
    void* yp = y.d_cl;
    const int as = a.d.dtype == B2VX_DT_INT8, bs = b.d.dtype == B2VX_DT_INT8;
    const float sa = all_q8 ? a.scale() : 1.0f, sb = all_q8 ? b.scale() : 1.0f;
    const int za = all_q8 ? a.zp() : 0, zb = all_q8 ? b.zp() : 0;
    const OutQuant oq = out_quant(y);
    const std::array<int, 5> ad = {a.N, a.H, a.W, a.C, a.Cp}, bd = {b.N, b.H, b.W, b.C, b.Cp}, yd = {y.N, y.H, y.W, y.C, y.Cp};
    const int elem = all_f32 ? 4 : 1;
    s.info = make_info("add_broadcast", idx, 0, abytes);
    s.fn = [=](cudaStream_t st2) {
      launch_add_broadcast(ap, as, sa, za, ad.data(), bp, bs, sb, zb, bd.data(), oq, yd.data(), elem, yp, st2);
      return cudaGetLastError();
    };
    g->steps.push_back(std::move(s));
    return B2VX_OK;
  }
  if (a.d.dtype == B2VX_DT_FLOAT32 && b.d.dtype == B2VX_DT_FLOAT32 && y.d.dtype == B2VX_DT_FLOAT32) {
    const float *ap = static_cast<const float*>(cl_in(a)), *bp = static_cast<const float*>(cl_in(b));
    float* yp = static_cast<float*>(y.d_cl);
    const size_t nel = y.cl_bytes / 4;
    s.info = make_info("add_f32", idx, 0, abytes);
    s.fn = [=](cudaStream_t st2) { launch_add_f32(ap, bp, yp, nel, st2); return cudaGetLastError(); };
  } else if (is_q8(a.d.dtype) && is_q8(b.d.dtype) && is_q8(y.d.dtype)) {
    const void *ap = cl_in(a), *bp = cl_in(b);
    void* yp = y.d_cl;
    const int as = a.d.dtype == B2VX_DT_INT8, bs = b.d.dtype == B2VX_DT_INT8, ys = y.d.dtype == B2VX_DT_INT8;
    const float sa = a.scale(), sb = b.scale();
    const int za = a.zp(), zb = b.zp();
    const OutQuant oq = out_quant(y);
    const size_t nel = y.cl_bytes;
    // B2VX_ADD_KERNEL=lut|alu forces one of the two kernels (read when the graph is created)
    // The arithmetic kernel is the faster one unless many byte pairs give a sum whose quotient by the
    // output scale is (nearly) a .5 fraction, each of which costs it an exact re-evaluation: scales in a
    // simple ratio do that (0.4*i + 0.7*j hits .5 for one pair in ten).  Count such pairs; large tensors
    // with more than 2% of them use the table kernel.
    bool use_lut = g->add_mode == 1;
    if (g->add_mode == 0 && nel >= (size_t(1) << 23)) {
      int near = 0;
      const float inv = 1.0f / oq.scale;
      for (int ia = 0; ia < 256; ia += 3) {
        const float fa = (static_cast<float>(as ? static_cast<int>(static_cast<int8_t>(ia)) : ia) - static_cast<float>(za)) * sa;
        for (int ib = 0; ib < 256; ib += 5) {
          const float fb = (static_cast<float>(bs ? static_cast<int>(static_cast<int8_t>(ib)) : ib) - static_cast<float>(zb)) * sb;
          const double t = static_cast<double>(fa + fb) * inv;
          const double frac = std::fabs(t) - std::floor(std::fabs(t));
          if (std::fabs(frac - 0.5) < std::fabs(t) * 1e-6 + 1e-9) ++near;
        }
      }
      use_lut = near * 50 > 86 * 52;   // 86 x 52 pairs sampled
    }
    if (use_lut) {
      // every pair of input bytes through the reference's float sequence, once
      std::vector<uint8_t> table(65536);
      for (int ia = 0; ia < 256; ++ia) {
        const int qa = as ? static_cast<int>(static_cast<int8_t>(ia)) : ia;
        const float fa = (static_cast<float>(qa) - static_cast<float>(za)) * sa;
        for (int ib = 0; ib < 256; ++ib) {
          const int qb = bs ? static_cast<int>(static_cast<int8_t>(ib)) : ib;
          const float fb = (static_cast<float>(qb) - static_cast<float>(zb)) * sb;
          table[ia * 256 + (ib ^ ((ia & 31) << 2))] = static_cast<uint8_t>(host_requant(fa + fb, oq) & 0xFF);
        }
      }
      uint8_t* dtab = nullptr;
      const b2vx_status st = upload(g, table, &dtab);
      if (st != B2VX_OK) return st;
      s.info = make_info("add_q_lut", idx, 0, abytes);
      s.fn = [=](cudaStream_t st2) { launch_add_q_lut(ap, bp, dtab, yp, nel, st2); return cudaGetLastError(); };
    } else {
      s.info = make_info("add_q", idx, 0, abytes);
      s.fn = [=](cudaStream_t st2) { launch_add_q(ap, as, sa, za, bp, bs, sb, zb, oq, ys, yp, nel, st2); return cudaGetLastError(); };
    }
  } else if (a.d.dtype == B2VX_DT_INT32 && b.d.dtype == B2VX_DT_INT32 && y.d.dtype == B2VX_DT_INT32) {
    const int *ap = static_cast<const int*>(cl_in(a)), *bp = static_cast<const int*>(cl_in(b));
    int* yp = static_cast<int*>(y.d_cl);
    const float sa = a.scale(), sb = b.scale();
    const int za = a.zp(), zb = b.zp();
    const OutQuant oq = out_quant(y);
    const size_t nel = y.cl_bytes / 4;
    s.info = make_info("add_i32", idx, 0, abytes);
    s.fn = [=](cudaStream_t st2) { launch_add_i32(ap, sa, za, bp, sb, zb, oq, yp, nel, st2); return cudaGetLastError(); };
  } else {
    return fail(g, B2VX_UNSUPPORTED, "add: operands must be all int8/uint8, all int32 or all float32");
  }
  g->steps.push_back(std::move(s));
  return B2VX_OK;
}

// ops::AddN: two inputs are an Add; more run the one-element-per-thread kernel over the channels-last storages
// (all operands have one shape, hence one storage layout).
b2vx_status plan_addn(b2vx_graph* g, uint32_t idx, NodeRec& n) {
  uint32_t cnt = 0;
  for (uint32_t id : n.in) cnt += id != B2VX_NO_TENSOR ? 1u : 0u;
  if (cnt == 2) return plan_add(g, idx, n);
  TensorRec& y = g->tensors[n.out];
  const bool f32 = y.d.dtype == B2VX_DT_FLOAT32;
  if (!f32 && !is_q8(y.d.dtype)) return fail(g, B2VX_UNSUPPORTED, "addn: operands must be all int8/uint8 or all float32");
  AddNParams p;
  std::memset(&p, 0, sizeof(p));
  uint64_t abytes = y.bytes();
  for (uint32_t id : n.in) {
    if (id == B2VX_NO_TENSOR) continue;
    TensorRec& t = g->tensors[id];
    if (f32 ? t.d.dtype != B2VX_DT_FLOAT32 : !is_q8(t.d.dtype)) return fail(g, B2VX_UNSUPPORTED, "addn: operands must be all int8/uint8 or all float32");
    if (t.cl_bytes != y.cl_bytes) return fail(g, B2VX_SHAPE_MISMATCH, "addn: operand storage differs from the output's");
    p.x[p.n_in] = cl_in(t);
    p.scale[p.n_in] = f32 ? 1.0f : t.scale();
    p.zp[p.n_in] = f32 ? 0 : t.zp();
    p.is_signed[p.n_in] = t.d.dtype == B2VX_DT_INT8;
    ++p.n_in;
    abytes += t.bytes();
  }
  p.out = out_quant(y);
  p.out_signed = y.d.dtype == B2VX_DT_INT8;
  void* yp = y.d_cl;
  const size_t nel = f32 ? y.cl_bytes / 4 : y.cl_bytes;
  const int elem = f32 ? 4 : 1;
  Step s;
  s.info = make_info("addn", idx, 0, abytes);
  s.fn = [=](cudaStream_t st2) { launch_addn(p, elem, yp, nel, st2); return cudaGetLastError(); };
  g->steps.push_back(std::move(s));
  return B2VX_OK;
}

// Reshape, Transpose, DataConvert: one pass from the input's storage to the output's.
b2vx_status plan_move(b2vx_graph* g, uint32_t idx, NodeRec& n) {
  TensorRec& x = g->tensors[n.in[0]];
  TensorRec& y = g->tensors[n.out];
  if (x.d.rank > 4 || y.d.rank > 4) return fail(g, B2VX_UNSUPPORTED, "reshape/transpose/dataconvert: rank above 4");
  RelayoutParams p = relayout_base(y);
  // A graph input is read from its WHCN copy as the caller wrote it, and a graph output that nothing else
  // reads is written in WHCN order, which saves the layout conversions before and after.
  const bool x_dense = (x.d.attr & (B2VX_ATTR_INPUT | B2VX_ATTR_VARIABLE)) != 0 && x.d_io != nullptr && x.d_io != x.d_cl;
  int consumers = 0;
  for (const NodeRec& m : g->nodes) {
    if (m.removed) continue;
    for (uint32_t id : m.in) consumers += id == n.out;
  }
  const bool y_dense = (y.d.attr & B2VX_ATTR_OUTPUT) != 0 && consumers == 0 && y.d_io != nullptr && y.d_io != y.d_cl;
  long long xs[4];
  if (x_dense) dense_strides(x, xs);
  else cl_strides(x, xs);
  if (y_dense) dense_strides(y, p.ostride);
  else cl_strides(y, p.ostride);
  dense_strides(y, p.lstride);
  const char* name = "reshape";
  if (n.kind == B2VX_NODE_TRANSPOSE) {
    name = "transpose";
    for (uint32_t k = 0; k < y.d.rank; ++k) p.istride[k] = xs[n.p.dims.v[k]];
  } else if (n.kind == B2VX_NODE_RESHAPE) {
    p.reshape = 1;
    for (int k = 0; k < 4; ++k) p.istride[k] = xs[k];
    for (uint32_t k = 0; k < x.d.rank; ++k) p.idims[k] = static_cast<int>(x.d.dims[k]);
  } else {
    name = "dataconvert";
    for (int k = 0; k < 4; ++k) p.istride[k] = xs[k];
  }
  sort_by_output_stride(p, !p.reshape);
  if (n.kind != B2VX_NODE_DATACONVERT) {
    if (x.d.dtype != y.d.dtype) return fail(g, B2VX_UNSUPPORTED, "reshape/transpose: input and output dtype differ");
  } else if (is_q8(x.d.dtype) && is_q8(y.d.dtype)) {
    // requantize: every input byte through dequantize + quantize, once, on the host
    std::vector<uint8_t> lut(256);
    const OutQuant oq = out_quant(y);
    for (int i = 0; i < 256; ++i) {
      const int q = x.d.dtype == B2VX_DT_INT8 ? static_cast<int>(static_cast<int8_t>(i)) : i;
      lut[i] = static_cast<uint8_t>(host_requant((static_cast<float>(q) - static_cast<float>(x.zp())) * x.scale(), oq) & 0xFF);
    }
    uint8_t* dlut = nullptr;
    const b2vx_status st = upload(g, lut, &dlut);
    if (st != B2VX_OK) return st;
    // same shape, one byte per element: the two storages have the same layout, so the whole storage goes
    // through the table 16 bytes at a time
    const void* xp8 = cl_in(x);
    void* yp8 = y.d_cl;
    const size_t nbytes = y.cl_bytes;
    Step s8;
    s8.info = make_info("requantize_lut", idx, 0, x.bytes() + y.bytes());
    s8.fn = [=](cudaStream_t st2) { launch_lut_q(xp8, dlut, yp8, nbytes, st2); return cudaGetLastError(); };
    g->steps.push_back(std::move(s8));
    return B2VX_OK;
  } else if (x.d.dtype == B2VX_DT_FLOAT32 && is_q8(y.d.dtype)) {
    p.convert = 2;
    p.out = out_quant(y);
  } else if (is_q8(x.d.dtype) && y.d.dtype == B2VX_DT_FLOAT32) {
    p.convert = 3;
    p.in_scale = x.scale();
    p.in_zp = x.zp();
    p.in_signed = x.d.dtype == B2VX_DT_INT8;
  } else if (x.d.dtype == y.d.dtype && x.d.dtype == B2VX_DT_FLOAT32) {
    p.convert = 0;
  } else {
    return fail(g, B2VX_UNSUPPORTED, "dataconvert: supported are 8-bit <-> 8-bit, float32 <-> 8-bit and float32 -> float32");
  }
  const void* xp = x_dense ? x.d_io : cl_in(x);
  void* yp = y_dense ? y.d_io : y.d_cl;
  if (y_dense) y.io_direct = true;
  Step s;
  s.info = make_info(name, idx, 0, x.bytes() + y.bytes());
  s.fn = [=](cudaStream_t st2) { launch_relayout(xp, yp, p, st2); return cudaGetLastError(); };
  g->steps.push_back(std::move(s));
  return B2VX_OK;
}

// Concat: one pass per input into its slice of the output.
b2vx_status plan_concat(b2vx_graph* g, uint32_t idx, NodeRec& n) {
  TensorRec& y = g->tensors[n.out];
  if (y.d.rank > 4) return fail(g, B2VX_UNSUPPORTED, "concat: rank above 4");
  const uint32_t axis = n.p.concat_axis;
  long long ys[4];
  cl_strides(y, ys);
  long long offset = 0;   // along the axis, in elements of that dimension
  for (uint32_t id : n.in) {
    if (id == B2VX_NO_TENSOR) continue;
    TensorRec& t = g->tensors[id];
    if (t.d.dtype != y.d.dtype) return fail(g, B2VX_UNSUPPORTED, "concat: input and output dtype differ");
    const bool convert = is_q8(t.d.dtype) && (t.scale() != y.scale() || t.zp() != y.zp());
    const void* tp = cl_in(t);
    const size_t es = dtype_size(y.d.dtype);
    uint8_t* yp = static_cast<uint8_t*>(y.d_cl) + static_cast<size_t>(offset * ys[axis]) * es;
    Step s;
    const bool channel_axis = (y.d.rank == 3 || y.d.rank == 4) && axis == 2;
    if (channel_axis && es == 1 && !convert && t.C % 16 == 0 && offset % 16 == 0) {
      const int in16 = t.C / 16, in_pitch16 = t.Cp / 16, out_pitch16 = y.Cp / 16;
      const long long pixels = static_cast<long long>(t.N) * t.H * t.W;
      s.info = make_info("concat_c16", idx, 0, 2 * t.bytes());
      s.fn = [=](cudaStream_t st2) { launch_concat_c16(tp, in_pitch16, in16, yp, out_pitch16, 0, pixels, st2); return cudaGetLastError(); };
    } else {
      RelayoutParams p = relayout_base(t);
      for (int k = 0; k < 4; ++k) p.ostride[k] = ys[k];
      cl_strides(t, p.istride);
      sort_by_output_stride(p, true);
      if (convert) {
        std::vector<uint8_t> lut(256);
        const OutQuant oq = out_quant(y);
        for (int i = 0; i < 256; ++i) {
          const int q = t.d.dtype == B2VX_DT_INT8 ? static_cast<int>(static_cast<int8_t>(i)) : i;
          lut[i] = static_cast<uint8_t>(host_requant((static_cast<float>(q) - static_cast<float>(t.zp())) * t.scale(), oq) & 0xFF);
        }
        uint8_t* dlut = nullptr;
        const b2vx_status st = upload(g, lut, &dlut);
        if (st != B2VX_OK) return st;
        p.convert = 1;
        p.lut = dlut;
      }
      s.info = make_info("concat", idx, 0, 2 * t.bytes());
      s.fn = [=](cudaStream_t st2) { launch_relayout(tp, yp, p, st2); return cudaGetLastError(); };
    }
    g->steps.push_back(std::move(s));
    offset += t.d.dims[axis];
  }
  return B2VX_OK;
}

b2vx_status plan_relu(b2vx_graph* g, uint32_t idx, NodeRec& n) {
  TensorRec& x = g->tensors[n.in[0]];
  TensorRec& y = g->tensors[n.out];
  const float upper = n.kind == B2VX_NODE_RELU6 ? 6.0f : -1.0f;
  const uint64_t abytes = x.bytes() + y.bytes();
  Step s;
  if (x.d.dtype == B2VX_DT_FLOAT32 && y.d.dtype == B2VX_DT_FLOAT32) {
    const float* xp = static_cast<const float*>(cl_in(x));
    float* yp = static_cast<float*>(y.d_cl);
    const size_t nel = y.cl_bytes / 4;
    s.info = make_info("relu_f32", idx, 0, abytes);
    s.fn = [=](cudaStream_t st2) { launch_relu_f32(xp, upper, yp, nel, st2); return cudaGetLastError(); };
  } else if (is_q8(x.d.dtype) && is_q8(y.d.dtype)) {
    const void* xp = cl_in(x);
    void* yp = y.d_cl;
    uint8_t* dlut = nullptr;
    b2vx_status st = upload(g, relu_table(x, y, upper), &dlut);
    if (st != B2VX_OK) return st;
    const size_t nel = y.cl_bytes;
    s.info = make_info("relu_lut_q", idx, 0, abytes);
    s.fn = [=](cudaStream_t st2) { launch_lut_q(xp, dlut, yp, nel, st2); return cudaGetLastError(); };
  } else {
    return fail(g, B2VX_UNSUPPORTED, "relu: input and output must be both int8/uint8 or both float32");
  }
  g->steps.push_back(std::move(s));
  return B2VX_OK;
}

b2vx_status plan_softmax(b2vx_graph* g, uint32_t idx, NodeRec& n) {
  TensorRec& x = g->tensors[n.in[0]];
  TensorRec& y = g->tensors[n.out];
  int axis = n.p.softmax.axis;
  if (axis < 0) axis += static_cast<int>(x.d.rank);
  if (axis < 0 || axis >= static_cast<int>(x.d.rank)) return fail(g, B2VX_INVALID_ARG, "softmax: axis out of range");
  auto kind_of = [](int32_t dt) { return dt == B2VX_DT_UINT8 ? 0 : dt == B2VX_DT_INT8 ? 1 : dt == B2VX_DT_FLOAT32 ? 2 : -1; };
  const int xk = kind_of(x.d.dtype), yk = kind_of(y.d.dtype);
  if (xk < 0 || yk < 0) return fail(g, B2VX_UNSUPPORTED, "softmax: unsupported dtype");
  // which of (W,H,C,N) the axis is
  static const int map4[4] = {0, 1, 2, 3}, map3[3] = {0, 1, 2}, map2[2] = {2, 3}, map1[1] = {2};
  const int* mp = x.d.rank == 4 ? map4 : x.d.rank == 3 ? map3 : x.d.rank == 2 ? map2 : map1;
  const int which = mp[axis];
  const long long ext[4] = {x.W, x.H, x.C, x.N};
  const long long xst[4] = {x.Cp, static_cast<long long>(x.W) * x.Cp, 1, static_cast<long long>(x.H) * x.W * x.Cp};
  const long long yst[4] = {y.Cp, static_cast<long long>(y.W) * y.Cp, 1, static_cast<long long>(y.H) * y.W * y.Cp};
  SoftmaxGeom sg;
  sg.len = static_cast<int>(ext[which]);
  sg.x_stride = xst[which];
  sg.y_stride = yst[which];
  for (int i = 0, k = 0; i < 4; ++i) {
    if (i == which) continue;
    sg.o[k] = static_cast<int>(ext[i]);
    sg.xs[k] = xst[i];
    sg.ys[k] = yst[i];
    ++k;
  }
  const void* xp = cl_in(x);
  void* yp = y.d_cl;
  const float sx = x.scale(), beta = n.p.softmax.beta;
  const int zx = x.zp();
  const OutQuant oq = out_quant(y);
  Step st;
  st.info = make_info("softmax", idx, 0, x.bytes() + y.bytes());
  st.fn = [=](cudaStream_t st2) { launch_softmax(xp, xk, sx, zx, yp, yk, oq, beta, sg, st2); return cudaGetLastError(); };
  g->steps.push_back(std::move(st));
  return B2VX_OK;
}

b2vx_status add_node(b2vx_graph* g, int32_t kind, uint32_t i0, uint32_t i1, uint32_t i2, uint32_t out, const NodeRec* proto) {
  if (!g) return B2VX_INVALID_ARG;
  if (g->compiled) return fail(g, B2VX_BAD_STATE, "graph is already compiled");
  if (!valid_id(g, i0) || !valid_id(g, out)) return fail(g, B2VX_INVALID_ARG, "node: bad tensor id");
  if (i1 != B2VX_NO_TENSOR && !valid_id(g, i1)) return fail(g, B2VX_INVALID_ARG, "node: bad tensor id");
  if (i2 != B2VX_NO_TENSOR && !valid_id(g, i2)) return fail(g, B2VX_INVALID_ARG, "node: bad tensor id");
  NodeRec n;
  if (proto) n = *proto;
  else std::memset(&n, 0, sizeof(n));
  n.kind = kind;
  for (uint32_t& id : n.in) id = B2VX_NO_TENSOR;
  n.in[0] = i0; n.in[1] = i1; n.in[2] = i2; n.out = out;
  n.removed = false;
  n.fuse_add = -1;
  n.fuse_residual = B2VX_NO_TENSOR;
  g->nodes.push_back(n);
  return B2VX_OK;
}

}  // namespace

// ================================================================== C ABI

extern "C" {

b2vx_status b2vx_context_create(b2vx_context** out) {
  if (!out) return B2VX_INVALID_ARG;
  *out = new b2vx_context();
  return B2VX_OK;
}
void b2vx_context_destroy(b2vx_context* ctx) { delete ctx; }
const char* b2vx_last_error(const b2vx_context* ctx) { return ctx ? ctx->err.c_str() : ""; }

int32_t b2vx_device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

b2vx_status b2vx_graph_create(b2vx_context* ctx, int32_t device_id, b2vx_graph** out) {
  if (!ctx || !out) return B2VX_INVALID_ARG;
  const int n = b2vx_device_count();
  if (n <= 0) {
    ctx->err = "no CUDA device: this backend has no CPU execution path";
    return B2VX_CUDA_ERROR;
  }
  if (device_id < 0 || device_id >= n) {
    ctx->err = "device id out of range";
    return B2VX_INVALID_ARG;
  }
  b2vx_graph* g = new b2vx_graph();
  g->ctx = ctx;
  g->device = device_id;
  DeviceGuard guard(device_id);
  if (cudaStreamCreateWithFlags(&g->own_stream, cudaStreamNonBlocking) != cudaSuccess ||
      cudaMalloc(reinterpret_cast<void**>(&g->d_status), sizeof(int)) != cudaSuccess ||
      cudaMemset(g->d_status, 0, sizeof(int)) != cudaSuccess ||
      cudaHostAlloc(reinterpret_cast<void**>(&g->h_status), sizeof(int), cudaHostAllocDefault) != cudaSuccess) {
    ctx->err = std::string("graph_create: ") + cudaGetErrorString(cudaGetLastError());
    delete g;
    return B2VX_CUDA_ERROR;
  }
  *g->h_status = 0;
  g->stream = g->own_stream;
  const char* k = std::getenv("B2VX_CONV_KERNEL");
  g->use_tc = gemm_tc_available() && !(k && std::strcmp(k, "simt") == 0);
  const char* fa = std::getenv("B2VX_FUSE_ADD");
  g->fuse_add = !(fa && fa[0] == '0');
  const char* fs = std::getenv("B2VX_FC_SMALL_M");
  g->fc_small_m = !(fs && fs[0] == '0');
  const char* ak = std::getenv("B2VX_ADD_KERNEL");
  g->add_mode = !ak ? 0 : (std::strcmp(ak, "lut") == 0 ? 1 : 2);
  const char* cg = std::getenv("B2VX_CUDA_GRAPH");
  g->use_cuda_graph = !(cg && cg[0] == '0');
  *out = g;
  return B2VX_OK;
}

void b2vx_graph_destroy(b2vx_graph* g) {
  if (!g) return;
  DeviceGuard guard(g->device);
  cudaStreamSynchronize(g->stream);
  if (g->exec) cudaGraphExecDestroy(g->exec);
  for (GemmTcPlan* p : g->gemm_plans) gemm_tc_plan_destroy(p);
  for (void* p : g->allocs) cudaFree(p);
  if (g->d_status) cudaFree(g->d_status);
  if (g->h_status) cudaFreeHost(g->h_status);
  if (g->own_stream) cudaStreamDestroy(g->own_stream);
  delete g;
}

b2vx_status b2vx_tensor_create(b2vx_graph* g, const b2vx_tensor_desc* desc, const void* const_data, uint32_t* out_id) {
  if (!g || !desc || !out_id) return B2VX_INVALID_ARG;
  if (g->compiled) return fail(g, B2VX_BAD_STATE, "graph is already compiled");
  if (desc->rank > 4) return fail(g, B2VX_UNSUPPORTED, "tensor: rank above 4 is not supported on this path");
  if (desc->dtype != B2VX_DT_INT8 && desc->dtype != B2VX_DT_UINT8 && desc->dtype != B2VX_DT_INT32 && desc->dtype != B2VX_DT_FLOAT32)
    return fail(g, B2VX_UNSUPPORTED, "tensor: dtype must be int8, uint8, int32 or float32");
  if (desc->quant_type != B2VX_QUANT_NONE && desc->quant_type != B2VX_QUANT_ASYMMETRIC &&
      desc->quant_type != B2VX_QUANT_SYMMETRIC_PER_CHANNEL)
    return fail(g, B2VX_UNSUPPORTED, "tensor: quantization type not supported");
  TensorRec t;
  t.d = *desc;
  if (desc->quant_type == B2VX_QUANT_SYMMETRIC_PER_CHANNEL) {
    if (!desc->scales || desc->n_channel == 0) return fail(g, B2VX_INVALID_ARG, "tensor: per-channel scales missing");
    t.scales.assign(desc->scales, desc->scales + desc->n_channel);
    if (desc->zero_points) t.zps.assign(desc->zero_points, desc->zero_points + desc->n_channel);
  }
  if (desc->quant_type == B2VX_QUANT_ASYMMETRIC && is_q8(desc->dtype) && !(desc->scale > 0.0f))
    return fail(g, B2VX_QUANT_MISMATCH, "tensor: scale must be positive");
  t.d.scales = nullptr;
  t.d.zero_points = nullptr;
  t.has_shape = desc->rank > 0;
  for (uint32_t i = 0; i < desc->rank; ++i)
    if (desc->dims[i] == 0) return fail(g, B2VX_INVALID_ARG, "tensor: zero-sized dimension");
  if (const_data) {
    if (!t.has_shape) return fail(g, B2VX_INVALID_ARG, "tensor: data given without a shape");
    t.host.assign(static_cast<const uint8_t*>(const_data), static_cast<const uint8_t*>(const_data) + t.bytes());
    t.host_valid = true;
  }
  g->tensors.push_back(std::move(t));
  *out_id = static_cast<uint32_t>(g->tensors.size() - 1);
  return B2VX_OK;
}

b2vx_status b2vx_tensor_get_desc(b2vx_graph* g, uint32_t id, b2vx_tensor_desc* out) {
  if (!g || !out || !valid_id(g, id)) return B2VX_INVALID_ARG;
  TensorRec& t = g->tensors[id];
  *out = t.d;
  if (!t.has_shape) out->rank = 0;
  out->n_channel = static_cast<uint32_t>(t.scales.size());
  out->scales = t.scales.empty() ? nullptr : t.scales.data();
  out->zero_points = t.zps.empty() ? nullptr : t.zps.data();
  return B2VX_OK;
}

b2vx_status b2vx_tensor_write(b2vx_graph* g, uint32_t id, const void* src, size_t bytes) {
  if (!g || !src || !valid_id(g, id)) return B2VX_INVALID_ARG;
  TensorRec& t = g->tensors[id];
  if (t.d.attr & B2VX_ATTR_TRANSIENT) return fail(g, B2VX_BAD_STATE, "tensor_write: transient tensors cannot be written");
  if (!t.has_shape || bytes != t.bytes()) return fail(g, B2VX_INVALID_ARG, "tensor_write: byte size does not match the tensor");
  if (!g->compiled) {
    t.host.assign(static_cast<const uint8_t*>(src), static_cast<const uint8_t*>(src) + bytes);
    t.host_valid = true;
    return B2VX_OK;
  }
  if (t.d.attr & B2VX_ATTR_CONSTANT) return fail(g, B2VX_BAD_STATE, "tensor_write: constants are frozen at compile");
  if (!t.d_io) return fail(g, B2VX_BAD_STATE, "tensor_write: tensor has no device storage");
  DeviceGuard guard(g->device);
  CUDA_TRY(g, cudaMemcpyAsync(t.d_io, src, bytes, cudaMemcpyHostToDevice, g->stream));
  CUDA_TRY(g, cudaStreamSynchronize(g->stream));
  return B2VX_OK;
}

b2vx_status b2vx_tensor_read(b2vx_graph* g, uint32_t id, void* dst, size_t bytes) {
  if (!g || !dst || !valid_id(g, id)) return B2VX_INVALID_ARG;
  TensorRec& t = g->tensors[id];
  if (!t.has_shape || bytes != t.bytes()) return fail(g, B2VX_INVALID_ARG, "tensor_read: byte size does not match the tensor");
  if (!g->compiled) {
    if (!t.host_valid) return fail(g, B2VX_BAD_STATE, "tensor_read: tensor holds no data yet");
    std::memcpy(dst, t.host.data(), bytes);
    return B2VX_OK;
  }
  if (!t.is_activation) {
    if (!t.host_valid) return fail(g, B2VX_BAD_STATE, "tensor_read: tensor holds no data");
    std::memcpy(dst, t.host.data(), bytes);
    return B2VX_OK;
  }
  DeviceGuard guard(g->device);
  if (t.d_io) {
    CUDA_TRY(g, cudaMemcpyAsync(dst, t.d_io, bytes, cudaMemcpyDeviceToHost, g->stream));
    CUDA_TRY(g, cudaStreamSynchronize(g->stream));
    return B2VX_OK;
  }
  // intermediate tensor: convert on the fly (debugging / per-layer checks)
  void* tmp = nullptr;
  CUDA_TRY(g, cudaMalloc(&tmp, bytes));
  launch_cl_to_whcn(t.d_cl, tmp, t.N, t.C, t.H, t.W, t.Cp, static_cast<int>(dtype_size(t.d.dtype)), g->stream);
  cudaError_t e = cudaMemcpyAsync(dst, tmp, bytes, cudaMemcpyDeviceToHost, g->stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(g->stream);
  cudaFree(tmp);
  if (e != cudaSuccess) return fail(g, B2VX_CUDA_ERROR, std::string("tensor_read: ") + cudaGetErrorString(e));
  return B2VX_OK;
}

b2vx_status b2vx_node_conv2d(b2vx_graph* g, uint32_t x, uint32_t w, uint32_t bias, uint32_t y, const b2vx_conv2d_desc* d) {
  if (!g || !d) return B2VX_INVALID_ARG;
  if (!valid_id(g, w)) return fail(g, B2VX_INVALID_ARG, "conv2d: weight tensor missing");
  NodeRec n;
  std::memset(&n, 0, sizeof(n));
  n.p.conv = *d;
  return add_node(g, B2VX_NODE_CONV2D, x, w, bias, y, &n);
}

b2vx_status b2vx_node_fully_connected(b2vx_graph* g, uint32_t x, uint32_t w, uint32_t bias, uint32_t y, const b2vx_fc_desc* d) {
  if (!g || !d) return B2VX_INVALID_ARG;
  if (!valid_id(g, w)) return fail(g, B2VX_INVALID_ARG, "fully_connected: weight tensor missing");
  NodeRec n;
  std::memset(&n, 0, sizeof(n));
  n.p.fc = *d;
  return add_node(g, B2VX_NODE_FULLY_CONNECTED, x, w, bias, y, &n);
}

b2vx_status b2vx_node_pool2d(b2vx_graph* g, uint32_t x, uint32_t y, const b2vx_pool2d_desc* d) {
  if (!g || !d) return B2VX_INVALID_ARG;
  NodeRec n;
  std::memset(&n, 0, sizeof(n));
  n.p.pool = *d;
  return add_node(g, B2VX_NODE_POOL2D, x, B2VX_NO_TENSOR, B2VX_NO_TENSOR, y, &n);
}

b2vx_status b2vx_node_add(b2vx_graph* g, uint32_t a, uint32_t b, uint32_t y) {
  if (!g) return B2VX_INVALID_ARG;
  if (!valid_id(g, b)) return fail(g, B2VX_INVALID_ARG, "add: second input missing");
  return add_node(g, B2VX_NODE_ADD, a, b, B2VX_NO_TENSOR, y, nullptr);
}
b2vx_status b2vx_node_relu(b2vx_graph* g, uint32_t x, uint32_t y) {
  return add_node(g, B2VX_NODE_RELU, x, B2VX_NO_TENSOR, B2VX_NO_TENSOR, y, nullptr);
}
b2vx_status b2vx_node_relu6(b2vx_graph* g, uint32_t x, uint32_t y) {
  return add_node(g, B2VX_NODE_RELU6, x, B2VX_NO_TENSOR, B2VX_NO_TENSOR, y, nullptr);
}
b2vx_status b2vx_node_reshape(b2vx_graph* g, uint32_t x, uint32_t y, const b2vx_dims_desc* shape) {
  if (!g) return B2VX_INVALID_ARG;
  if (!shape || shape->rank == 0 || shape->rank > B2VX_MAX_RANK) return fail(g, B2VX_INVALID_ARG, "reshape: bad shape");
  NodeRec n;
  std::memset(&n, 0, sizeof(n));
  n.p.dims = *shape;
  return add_node(g, B2VX_NODE_RESHAPE, x, B2VX_NO_TENSOR, B2VX_NO_TENSOR, y, &n);
}
b2vx_status b2vx_node_transpose(b2vx_graph* g, uint32_t x, uint32_t y, const b2vx_dims_desc* perm) {
  if (!g) return B2VX_INVALID_ARG;
  if (!perm || perm->rank == 0 || perm->rank > B2VX_MAX_RANK) return fail(g, B2VX_INVALID_ARG, "transpose: bad permutation");
  NodeRec n;
  std::memset(&n, 0, sizeof(n));
  n.p.dims = *perm;
  return add_node(g, B2VX_NODE_TRANSPOSE, x, B2VX_NO_TENSOR, B2VX_NO_TENSOR, y, &n);
}
b2vx_status b2vx_node_concat(b2vx_graph* g, const uint32_t* inputs, uint32_t n_inputs, uint32_t axis, uint32_t y) {
  if (!g) return B2VX_INVALID_ARG;
  if (!inputs || n_inputs == 0 || n_inputs > B2VX_MAX_NODE_INPUTS) return fail(g, B2VX_INVALID_ARG, "concat: 1 to 16 inputs");
  for (uint32_t i = 0; i < n_inputs; ++i)
    if (!valid_id(g, inputs[i])) return fail(g, B2VX_INVALID_ARG, "concat: bad tensor id");
  NodeRec n;
  std::memset(&n, 0, sizeof(n));
  n.p.concat_axis = axis;
  const b2vx_status st = add_node(g, B2VX_NODE_CONCAT, inputs[0], B2VX_NO_TENSOR, B2VX_NO_TENSOR, y, &n);
  if (st != B2VX_OK) return st;
  for (uint32_t i = 0; i < n_inputs; ++i) g->nodes.back().in[i] = inputs[i];
  return B2VX_OK;
}
b2vx_status b2vx_node_addn(b2vx_graph* g, const uint32_t* inputs, uint32_t n_inputs, uint32_t y) {
  if (!g) return B2VX_INVALID_ARG;
  if (!inputs || n_inputs < 2 || n_inputs > B2VX_MAX_NODE_INPUTS) return fail(g, B2VX_INVALID_ARG, "addn: 2 to 16 inputs");
  for (uint32_t i = 0; i < n_inputs; ++i)
    if (!valid_id(g, inputs[i])) return fail(g, B2VX_INVALID_ARG, "addn: bad tensor id");
  const b2vx_status st = add_node(g, B2VX_NODE_ADDN, inputs[0], B2VX_NO_TENSOR, B2VX_NO_TENSOR, y, nullptr);
  if (st != B2VX_OK) return st;
  for (uint32_t i = 0; i < n_inputs; ++i) g->nodes.back().in[i] = inputs[i];
  return B2VX_OK;
}
b2vx_status b2vx_node_dataconvert(b2vx_graph* g, uint32_t x, uint32_t y) {
  return add_node(g, B2VX_NODE_DATACONVERT, x, B2VX_NO_TENSOR, B2VX_NO_TENSOR, y, nullptr);
}
b2vx_status b2vx_node_softmax(b2vx_graph* g, uint32_t x, uint32_t y, const b2vx_softmax_desc* d) {
  if (!g || !d) return B2VX_INVALID_ARG;
  NodeRec n;
  std::memset(&n, 0, sizeof(n));
  n.p.softmax = *d;
  return add_node(g, B2VX_NODE_SOFTMAX, x, B2VX_NO_TENSOR, B2VX_NO_TENSOR, y, &n);
}

b2vx_status b2vx_graph_compile(b2vx_graph* g) {
  if (!g) return B2VX_INVALID_ARG;
  if (g->compiled) return B2VX_OK;
  DeviceGuard guard(g->device);
  // 1. order
  std::vector<char> ready(g->tensors.size(), 0), done(g->nodes.size(), 0);
  for (size_t i = 0; i < g->tensors.size(); ++i)
    ready[i] = (g->tensors[i].d.attr & (B2VX_ATTR_CONSTANT | B2VX_ATTR_INPUT | B2VX_ATTR_VARIABLE)) != 0;
  for (const NodeRec& n : g->nodes) ready[n.out] = 0;
  g->order.clear();
  for (bool progress = true; progress;) {
    progress = false;
    for (size_t i = 0; i < g->nodes.size(); ++i) {
      if (done[i]) continue;
      NodeRec& n = g->nodes[i];
      bool ok = true;
      for (uint32_t id : n.in) ok = ok && (id == B2VX_NO_TENSOR || ready[id]);
      if (!ok) continue;
      b2vx_status st = infer_node(g, n);
      if (st != B2VX_OK) return st;
      ready[n.out] = 1;
      done[i] = 1;
      g->order.push_back(static_cast<uint32_t>(i));
      progress = true;
    }
  }
  if (g->order.size() != g->nodes.size()) return fail(g, B2VX_BAD_STATE, "graph has a cycle or a node whose input is never produced");

  // 1a. A grouped convolution (ops::GroupedConv2d) runs as an ordinary one whose kernel is block diagonal:
  // the kernel [kw, kh, Ic/group, Oc] is spread into [kw, kh, Ic, Oc] with the real value zero (the weight
  // zero point) everywhere outside the blocks, which adds nothing to any accumulator.  The tensor cores do
  // `group` times the arithmetic the layer needs; what it buys is one code path.
  for (size_t ni = 0; ni < g->nodes.size(); ++ni) {
    if (g->nodes[ni].kind != B2VX_NODE_CONV2D || g->nodes[ni].p.conv.group <= 1) continue;
    const int group = g->nodes[ni].p.conv.group;
    if (g->nodes[ni].p.conv.multiplier >= 1) return fail(g, B2VX_UNSUPPORTED, "conv2d: group and multiplier together");
    const TensorRec& w = g->tensors[g->nodes[ni].in[1]];
    const TensorRec& x = g->tensors[g->nodes[ni].in[0]];
    if (!w.host_valid) return fail(g, B2VX_UNSUPPORTED, "grouped conv2d: the kernel must be a constant");
    if (w.d.rank != 4 || x.d.rank < 3) return fail(g, B2VX_SHAPE_MISMATCH, "grouped conv2d: kernel rank 4, input rank 3 or 4");
    const uint32_t kk = w.d.dims[0] * w.d.dims[1], icg = w.d.dims[2], oc_n = w.d.dims[3], ic_n = x.d.dims[2];
    if (icg * static_cast<uint32_t>(group) != ic_n || oc_n % static_cast<uint32_t>(group))
      return fail(g, B2VX_SHAPE_MISMATCH, "grouped conv2d: kernel must be [kw, kh, C/group, Oc] with Oc a multiple of group");
    TensorRec full = w;
    full.d.dims[2] = ic_n;
    const size_t es = dtype_size(w.d.dtype);
    full.host.assign(static_cast<size_t>(kk) * ic_n * oc_n * es, 0);
    if (es == 1) std::memset(full.host.data(), w.zp() & 0xFF, full.host.size());   // real zero of an 8-bit kernel
    const uint32_t per_out = oc_n / static_cast<uint32_t>(group);
    for (uint32_t oc = 0; oc < oc_n; ++oc) {
      const uint32_t gi = oc / per_out;
      std::memcpy(full.host.data() + (static_cast<size_t>(oc) * ic_n + gi * icg) * kk * es,
                  w.host.data() + static_cast<size_t>(oc) * icg * kk * es, static_cast<size_t>(icg) * kk * es);
    }
    g->tensors.push_back(std::move(full));
    g->nodes[ni].in[1] = static_cast<uint32_t>(g->tensors.size() - 1);
    g->nodes[ni].p.conv.group = 1;
  }

  // 1b. A Relu/Relu6 between identical 8-bit quantizations whose byte table is the
  // identity (zero point at the bottom of the range, nothing to clamp) changes no
  // byte: its producer writes straight into the Relu's output tensor.
  for (NodeRec& r : g->nodes) {
    if (r.kind != B2VX_NODE_RELU && r.kind != B2VX_NODE_RELU6) continue;
    TensorRec& tin = g->tensors[r.in[0]];
    TensorRec& tout = g->tensors[r.out];
    if (!is_q8(tin.d.dtype) || tin.d.dtype != tout.d.dtype) continue;
    if (tin.d.quant_type != B2VX_QUANT_ASYMMETRIC || tout.d.quant_type != B2VX_QUANT_ASYMMETRIC) continue;
    if (tin.scale() != tout.scale() || tin.zp() != tout.zp()) continue;
    if (tin.d.attr != B2VX_ATTR_TRANSIENT) continue;
    int consumers = 0;
    NodeRec* producer = nullptr;
    for (NodeRec& n : g->nodes) {
      if (n.removed) continue;
      for (uint32_t id : n.in) consumers += id == r.in[0];
      if (n.out == r.in[0]) producer = &n;
    }
    if (consumers != 1 || !producer) continue;
    const std::vector<uint8_t> lut = relu_table(tin, tout, r.kind == B2VX_NODE_RELU6 ? 6.0f : -1.0f);
    bool identity = true;
    for (int i = 0; i < 256; ++i) identity = identity && lut[i] == i;
    if (!identity) continue;
    producer->out = r.out;
    r.removed = true;
  }

  // 1c. A quantized Add one of whose operands is the output of a convolution that nothing else reads
  // can be done in that convolution's epilogue (tensor-core path): the convolution's byte and the
  // other operand's byte index the Add's 64 KB table.  The absorbing convolution is the operand
  // produced later in the order; the other operand is then ready when it runs.  Whether the fusion
  // happens is decided when the convolution is planned (it needs the tensor-core path).
  if (g->fuse_add && g->use_tc) {
    std::vector<int> pos(g->nodes.size(), -1);
    for (size_t i = 0; i < g->order.size(); ++i) pos[g->order[i]] = static_cast<int>(i);
    for (size_t ai = 0; ai < g->nodes.size(); ++ai) {
      NodeRec& ad = g->nodes[ai];
      if (ad.removed || ad.kind != B2VX_NODE_ADD) continue;
      const TensorRec& t0 = g->tensors[ad.in[0]];
      const TensorRec& t1 = g->tensors[ad.in[1]];
      const TensorRec& to = g->tensors[ad.out];
      if (!is_q8(t0.d.dtype) || !is_q8(t1.d.dtype) || !is_q8(to.d.dtype)) continue;
      if (t0.d.rank != t1.d.rank || !std::equal(t0.d.dims, t0.d.dims + t0.d.rank, t1.d.dims)) continue;
      int best = -1, best_operand = -1;
      for (int k = 0; k < 2; ++k) {
        const uint32_t tid = ad.in[k];
        if (g->tensors[tid].d.attr != B2VX_ATTR_TRANSIENT) continue;
        int consumers = 0, producer = -1;
        for (size_t ni = 0; ni < g->nodes.size(); ++ni) {
          const NodeRec& n = g->nodes[ni];
          if (n.removed) continue;
          for (uint32_t id : n.in) consumers += id == tid;
          if (n.out == tid) producer = static_cast<int>(ni);
        }
        if (consumers != 1 || producer < 0) continue;
        const NodeRec& pn = g->nodes[producer];
        if (pn.kind != B2VX_NODE_CONV2D || pn.p.conv.multiplier >= 1 || pn.fuse_add >= 0) continue;
        if (best < 0 || pos[producer] > pos[best]) { best = producer; best_operand = k; }
      }
      if (best < 0) continue;
      // the other operand must exist before the absorbing convolution runs
      const uint32_t other = ad.in[1 - best_operand];
      int other_producer = -1;
      for (size_t ni = 0; ni < g->nodes.size(); ++ni)
        if (!g->nodes[ni].removed && g->nodes[ni].out == other) other_producer = static_cast<int>(ni);
      if (other_producer >= 0 && pos[other_producer] > pos[best]) continue;
      g->nodes[best].fuse_add = static_cast<int>(ai);
      g->nodes[best].fuse_residual = other;
    }
  }

  // 2. which tensors are activations (touched by a node as data, not as weights/bias)
  for (const NodeRec& n : g->nodes) {
    if (n.removed) continue;
    g->tensors[n.in[0]].is_activation = true;
    g->tensors[n.out].is_activation = true;
    if (n.kind == B2VX_NODE_CONCAT || n.kind == B2VX_NODE_ADDN) {
      for (uint32_t id : n.in)
        if (id != B2VX_NO_TENSOR) g->tensors[id].is_activation = true;
    }
    if (n.kind == B2VX_NODE_CONV2D || n.kind == B2VX_NODE_FULLY_CONNECTED) {
      // a kernel or bias that is not a constant lives on the device like any other tensor
      for (int k = 1; k <= 2; ++k)
        if (n.in[k] != B2VX_NO_TENSOR && !g->tensors[n.in[k]].host_valid && !(g->tensors[n.in[k]].d.attr & B2VX_ATTR_CONSTANT))
          g->tensors[n.in[k]].is_activation = true;
    }
    if (n.kind == B2VX_NODE_ADD) g->tensors[n.in[1]].is_activation = true;
    // 32-bit integer activations exist only around Add (the reference's platform sample adds INT32 vectors) and
    // the nodes that move elements without looking at them
    else if (n.kind != B2VX_NODE_RESHAPE && n.kind != B2VX_NODE_TRANSPOSE && n.kind != B2VX_NODE_CONCAT &&
             (g->tensors[n.in[0]].d.dtype == B2VX_DT_INT32 || g->tensors[n.out].d.dtype == B2VX_DT_INT32))
      return fail(g, B2VX_UNSUPPORTED, "int32 activations are supported by Add, Reshape, Transpose and Concat only");
  }
  for (TensorRec& t : g->tensors) {
    if (!t.is_activation) continue;
    if (!t.has_shape) return fail(g, B2VX_SHAPE_MISMATCH, "an activation tensor has no shape");
    map_dims(t);
    b2vx_status st = dev_alloc(g, &t.d_cl, t.cl_bytes);
    if (st != B2VX_OK) return st;
    CUDA_TRY(g, cudaMemsetAsync(t.d_cl, 0, t.cl_bytes, g->stream));
    const bool io = (t.d.attr & (B2VX_ATTR_INPUT | B2VX_ATTR_OUTPUT | B2VX_ATTR_CONSTANT | B2VX_ATTR_VARIABLE)) != 0;
    if (io) {
      if (t.same_layouts()) t.d_io = t.d_cl;
      else {
        st = dev_alloc(g, &t.d_io, t.io_bytes);
        if (st != B2VX_OK) return st;
      }
    }
  }

  // 3. plan: nodes first (they record which inputs they read in channels-last form), then the
  //    input conversions are put in front and the output conversions behind
  g->steps.clear();
  for (uint32_t idx : g->order) {
    NodeRec& n = g->nodes[idx];
    if (n.removed) continue;
    b2vx_status st = B2VX_UNSUPPORTED;
    switch (n.kind) {
      case B2VX_NODE_CONV2D:
        g->fuse_request = n.fuse_add;
        g->fuse_residual = n.fuse_residual;
        g->fuse_done = false;
        st = plan_conv(g, idx, n);
        if (st == B2VX_OK && g->fuse_done) g->nodes[n.fuse_add].removed = true;   // the Add happens in this node's kernel
        g->fuse_request = -1;
        break;
      case B2VX_NODE_FULLY_CONNECTED: st = plan_fc(g, idx, n); break;
      case B2VX_NODE_POOL2D: st = plan_pool(g, idx, n); break;
      case B2VX_NODE_ADD: st = plan_add(g, idx, n); break;
      case B2VX_NODE_RELU:
      case B2VX_NODE_RELU6: st = plan_relu(g, idx, n); break;
      case B2VX_NODE_SOFTMAX: st = plan_softmax(g, idx, n); break;
      case B2VX_NODE_RESHAPE:
      case B2VX_NODE_TRANSPOSE:
      case B2VX_NODE_DATACONVERT: st = plan_move(g, idx, n); break;
      case B2VX_NODE_CONCAT: st = plan_concat(g, idx, n); break;
      case B2VX_NODE_ADDN: st = plan_addn(g, idx, n); break;
      default: return fail(g, B2VX_UNSUPPORTED, "unknown node kind");
    }
    if (st != B2VX_OK) return st;
  }
  {
    std::vector<Step> head;
    for (size_t i = 0; i < g->tensors.size(); ++i) {
      TensorRec& t = g->tensors[i];
      if (!t.is_activation || !t.cl_used || !(t.d.attr & (B2VX_ATTR_INPUT | B2VX_ATTR_VARIABLE))) continue;
      if (t.d_io == t.d_cl) continue;
      const void* src = t.d_io;
      void* dst = t.d_cl;
      const int N = t.N, C = t.C, H = t.H, W = t.W, Cp = t.Cp, el = static_cast<int>(dtype_size(t.d.dtype));
      Step s;
      s.info = make_info("whcn_to_cl", B2VX_NO_TENSOR, 0, t.io_bytes + t.cl_bytes);
      s.fn = [=](cudaStream_t st2) { launch_whcn_to_cl(src, dst, N, C, H, W, Cp, el, st2); return cudaGetLastError(); };
      head.push_back(std::move(s));
    }
    g->steps.insert(g->steps.begin(), std::make_move_iterator(head.begin()), std::make_move_iterator(head.end()));
  }
  for (size_t i = 0; i < g->tensors.size(); ++i) {
    TensorRec& t = g->tensors[i];
    if (!t.is_activation || !(t.d.attr & B2VX_ATTR_OUTPUT)) continue;
    if (t.d_io == t.d_cl || t.io_direct) continue;
    const void* src = t.d_cl;
    void* dst = t.d_io;
    const int N = t.N, C = t.C, H = t.H, W = t.W, Cp = t.Cp, el = static_cast<int>(dtype_size(t.d.dtype));
    Step s;
    s.info = make_info("cl_to_whcn", B2VX_NO_TENSOR, 0, t.io_bytes + t.cl_bytes);
    s.fn = [=](cudaStream_t st2) { launch_cl_to_whcn(src, dst, N, C, H, W, Cp, el, st2); return cudaGetLastError(); };
    g->steps.push_back(std::move(s));
  }
  if (g->scratch_bytes) {
    b2vx_status st = dev_alloc(g, &g->scratch, g->scratch_bytes);
    if (st != B2VX_OK) return st;
  }
  for (auto& f : g->finalizers) {
    b2vx_status st = f();
    if (st != B2VX_OK) return st;
  }
  g->finalizers.clear();

  // 4. data that was supplied before compile: inputs written early, constant activations
  for (TensorRec& t : g->tensors) {
    if (!t.is_activation || !t.host_valid || !t.d_io) continue;
    CUDA_TRY(g, cudaMemcpyAsync(t.d_io, t.host.data(), t.io_bytes, cudaMemcpyHostToDevice, g->stream));
    if ((t.d.attr & B2VX_ATTR_CONSTANT) && t.d_io != t.d_cl)
      launch_whcn_to_cl(t.d_io, t.d_cl, t.N, t.C, t.H, t.W, t.Cp, static_cast<int>(dtype_size(t.d.dtype)), g->stream);
  }
  CUDA_TRY(g, cudaStreamSynchronize(g->stream));
  CUDA_TRY(g, cudaGetLastError());
  g->compiled = true;
  return B2VX_OK;
}

b2vx_status b2vx_graph_run_async(b2vx_graph* g) {
  if (!g) return B2VX_INVALID_ARG;
  b2vx_status st = b2vx_graph_compile(g);
  if (st != B2VX_OK) return st;
  DeviceGuard guard(g->device);
  if (g->use_cuda_graph && !g->exec && !g->capture_failed && !g->steps.empty()) {
    // Record the plan once; on any failure fall back to launching kernel by kernel.
    cudaGraph_t graph = nullptr;
    bool ok = cudaStreamBeginCapture(g->stream, cudaStreamCaptureModeThreadLocal) == cudaSuccess;
    if (ok) {
      for (Step& s : g->steps) ok = ok && s.fn(g->stream) == cudaSuccess;
      ok = (cudaStreamEndCapture(g->stream, &graph) == cudaSuccess) && ok && graph != nullptr;
    }
    if (ok) ok = cudaGraphInstantiate(&g->exec, graph, 0) == cudaSuccess;
    if (graph) cudaGraphDestroy(graph);
    if (!ok) {
      cudaGetLastError();
      g->exec = nullptr;
      g->capture_failed = true;
    }
  }
  if (g->exec) {
    cudaError_t e = cudaGraphLaunch(g->exec, g->stream);
    if (e != cudaSuccess) return fail(g, B2VX_CUDA_ERROR, std::string("cudaGraphLaunch: ") + cudaGetErrorString(e));
    return B2VX_OK;
  }
  for (Step& s : g->steps) {
    cudaError_t e = s.fn(g->stream);
    if (e != cudaSuccess) {
      return fail(g, B2VX_CUDA_ERROR, std::string(s.info.name) + ": " + cudaGetErrorString(e));
    }
  }
  return B2VX_OK;
}

b2vx_status b2vx_graph_sync(b2vx_graph* g) {
  if (!g) return B2VX_INVALID_ARG;
  DeviceGuard guard(g->device);
  CUDA_TRY(g, cudaMemcpyAsync(g->h_status, g->d_status, sizeof(int), cudaMemcpyDeviceToHost, g->stream));
  CUDA_TRY(g, cudaStreamSynchronize(g->stream));
  if (*g->h_status != 0) {
    const int code = *g->h_status;
    cudaMemsetAsync(g->d_status, 0, sizeof(int), g->stream);
    return fail(g, B2VX_DEVICE_TIMEOUT, "a tensor-core kernel gave up waiting on a barrier (code " + std::to_string(code) + ")");
  }
  return B2VX_OK;
}

b2vx_status b2vx_graph_run(b2vx_graph* g) {
  b2vx_status st = b2vx_graph_run_async(g);
  if (st != B2VX_OK) return st;
  return b2vx_graph_sync(g);
}

b2vx_status b2vx_graph_set_stream(b2vx_graph* g, void* cuda_stream) {
  if (!g) return B2VX_INVALID_ARG;
  DeviceGuard guard(g->device);
  cudaStreamSynchronize(g->stream);
  g->stream = cuda_stream ? static_cast<cudaStream_t>(cuda_stream) : g->own_stream;
  return B2VX_OK;
}

b2vx_status b2vx_graph_kernel_count(b2vx_graph* g, uint32_t* out) {
  if (!g || !out) return B2VX_INVALID_ARG;
  *out = static_cast<uint32_t>(g->steps.size());
  return B2VX_OK;
}

b2vx_status b2vx_graph_kernel_info(b2vx_graph* g, uint32_t index, b2vx_kernel_info* out) {
  if (!g || !out || index >= g->steps.size()) return B2VX_INVALID_ARG;
  *out = g->steps[index].info;
  return B2VX_OK;
}

b2vx_status b2vx_graph_print(b2vx_graph* g) {
  if (!g) return B2VX_INVALID_ARG;
  std::fprintf(stderr, "b2vx graph: %zu tensors, %zu nodes, %zu kernels, device %d, tensor cores %s\n", g->tensors.size(),
               g->nodes.size(), g->steps.size(), g->device, g->use_tc ? "on" : "off");
  for (size_t i = 0; i < g->steps.size(); ++i) {
    const b2vx_kernel_info& k = g->steps[i].info;
    std::fprintf(stderr, "  [%3zu] %-22s node %-4d ops %-12llu bytes %-12llu %8.3f ms\n", i, k.name,
                 k.node_index == B2VX_NO_TENSOR ? -1 : static_cast<int>(k.node_index),
                 static_cast<unsigned long long>(k.ops), static_cast<unsigned long long>(k.bytes), k.last_ms);
  }
  return B2VX_OK;
}

b2vx_status b2vx_graph_profile(b2vx_graph* g, uint32_t iters) {
  if (!g) return B2VX_INVALID_ARG;
  if (iters == 0) iters = 1;
  b2vx_status st = b2vx_graph_run(g);   // warm-up
  if (st != B2VX_OK) return st;
  DeviceGuard guard(g->device);
  std::vector<cudaEvent_t> ev(g->steps.size() + 1);
  for (auto& e : ev) CUDA_TRY(g, cudaEventCreate(&e));
  std::vector<double> total(g->steps.size(), 0.0);
  // Per-kernel times from events recorded between the kernels.  Submitted launch by launch, the host
  // cannot keep up with kernels of a few microseconds and the gaps would be booked to the kernels, so
  // the sequence (kernels + event records) is captured into a CUDA graph and replayed; direct
  // submission is the fallback.
  cudaGraphExec_t exec = nullptr;
  if (g->use_cuda_graph) {
    cudaGraph_t graph = nullptr;
    bool ok = cudaStreamBeginCapture(g->stream, cudaStreamCaptureModeThreadLocal) == cudaSuccess;
    if (ok) {
      ok = cudaEventRecordWithFlags(ev[0], g->stream, cudaEventRecordExternal) == cudaSuccess;
      for (size_t i = 0; ok && i < g->steps.size(); ++i) {
        ok = g->steps[i].fn(g->stream) == cudaSuccess &&
             cudaEventRecordWithFlags(ev[i + 1], g->stream, cudaEventRecordExternal) == cudaSuccess;
      }
      ok = (cudaStreamEndCapture(g->stream, &graph) == cudaSuccess) && ok && graph != nullptr;
    }
    if (ok) ok = cudaGraphInstantiate(&exec, graph, 0) == cudaSuccess;
    if (graph) cudaGraphDestroy(graph);
    if (!ok) {
      exec = nullptr;
      cudaGetLastError();
    }
  }
  for (uint32_t it = 0; it < iters; ++it) {
    if (exec) {
      CUDA_TRY(g, cudaGraphLaunch(exec, g->stream));
    } else {
      CUDA_TRY(g, cudaEventRecord(ev[0], g->stream));
      for (size_t i = 0; i < g->steps.size(); ++i) {
        cudaError_t e = g->steps[i].fn(g->stream);
        if (e != cudaSuccess) return fail(g, B2VX_CUDA_ERROR, std::string(g->steps[i].info.name) + ": " + cudaGetErrorString(e));
        CUDA_TRY(g, cudaEventRecord(ev[i + 1], g->stream));
      }
    }
    CUDA_TRY(g, cudaStreamSynchronize(g->stream));
    for (size_t i = 0; i < g->steps.size(); ++i) {
      float ms = 0.0f;
      CUDA_TRY(g, cudaEventElapsedTime(&ms, ev[i], ev[i + 1]));
      total[i] += ms;
    }
  }
  if (exec) cudaGraphExecDestroy(exec);
  for (size_t i = 0; i < g->steps.size(); ++i) g->steps[i].info.last_ms = static_cast<float>(total[i] / iters);
  for (auto& e : ev) cudaEventDestroy(e);
  return b2vx_graph_sync(g);
}

b2vx_status b2vx_measure_int8_peak(int32_t device_id, int32_t reps, double* tops_out, int32_t* sm_count_out) {
  if (!tops_out || reps < 1 || reps > 100) return B2VX_INVALID_ARG;
  *tops_out = 0.0;
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || device_id < 0 || device_id >= count) return B2VX_INVALID_ARG;
  DeviceGuard guard(device_id);
  if (!gemm_tc_available()) return B2VX_UNSUPPORTED;
  int* d_status = nullptr;
  if (cudaMalloc(reinterpret_cast<void**>(&d_status), sizeof(int)) != cudaSuccess) return B2VX_OOM;
  cudaMemset(d_status, 0, sizeof(int));
  int sms = 0, h_status = 0;
  const double tops = gemm_tc_measure_int8_peak(reps, &sms, d_status);
  cudaMemcpy(&h_status, d_status, sizeof(int), cudaMemcpyDeviceToHost);
  cudaFree(d_status);
  if (h_status != 0) return B2VX_DEVICE_TIMEOUT;
  if (tops <= 0.0) return B2VX_CUDA_ERROR;
  *tops_out = tops;
  if (sm_count_out) *sm_count_out = sms;
  return B2VX_OK;
}

b2vx_status b2vx_host_alloc(void** out, size_t bytes) {
  if (!out) return B2VX_INVALID_ARG;
  if (cudaHostAlloc(out, bytes ? bytes : 1, cudaHostAllocDefault) != cudaSuccess) {
    cudaGetLastError();
    *out = nullptr;
    return B2VX_OOM;
  }
  return B2VX_OK;
}
void b2vx_host_free(void* p) {
  if (p) cudaFreeHost(p);
}

}  // extern "C"
