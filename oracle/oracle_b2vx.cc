// The b2vx C ABI implemented on the CPU oracle — TEST INFRASTRUCTURE ONLY.
//
// Exports the same symbols as the product library (include/b2vx.h) so that the
// tim::vx C++ layer, and anything written against it, can be linked against
// the oracle instead of the CUDA backend: the reference's own unit tests run
// this way on a machine without a GPU, and whole networks built through the
// tim::vx API get an independent CPU result to compare the GPU result with.
// Graph bookkeeping and shape inference are restated here independently of the
// product (reference: src/tim/vx/internal/src/vsi_nn_graph.c:389-560,1450-1639
// and the op_setup functions of vsi_nn_op_conv2d.c:199-287, vsi_nn_op_pool.c:324-427,
// vsi_nn_op_fullconnect2.c:154-196, vsi_nn_op_eltwise.c:147-214).
//
// With B2VX_CAPTURE_DIR set, every graph run is also written out as a JSON
// case (tensors, nodes, inputs, oracle outputs, and any expectation the test
// harness attaches through orc_capture_expect_pair), which is how the golden
// fixtures under tests/golden/ are produced.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "b2vx.h"
#include "oracle_ops.h"

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

struct OTensor {
  b2vx_tensor_desc d;
  std::vector<float> scales;
  std::vector<int32_t> zps;
  std::vector<uint8_t> data;
  bool has_shape = false;   // shape known (declared, or inferred at compile)
  bool declared = false;    // shape given by the caller
  bool written = false;
  size_t elems() const {
    size_t n = 1;
    for (uint32_t i = 0; i < d.rank; ++i) n *= d.dims[i];
    return n;
  }
  size_t bytes() const { return elems() * dtype_size(d.dtype); }
  orc_quant quant() const {
    orc_quant q;
    std::memset(&q, 0, sizeof(q));
    if (d.quant_type == B2VX_QUANT_SYMMETRIC_PER_CHANNEL) {
      q.per_channel = 1;
      q.n = static_cast<int32_t>(scales.size());
      q.scales = scales.data();
      q.zps = zps.empty() ? nullptr : zps.data();
    } else if (d.quant_type == B2VX_QUANT_ASYMMETRIC) {
      q.scale = d.scale;
      q.zp = d.zero_point;
    } else {
      q.scale = 1.0f;
    }
    return q;
  }
};

struct ONode {
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
  uint32_t pad_resolved[4];
};

struct Expectation {
  uint32_t tensor;
  int32_t dtype;
  double tol;
  std::vector<uint8_t> data;
};

}  // namespace

struct b2vx_context {
  std::string err;
};

struct b2vx_graph {
  b2vx_context* ctx;
  std::vector<OTensor> tensors;
  std::vector<ONode> nodes;
  std::vector<uint32_t> order;
  bool compiled = false;
  bool ran = false;
  uint32_t last_read = B2VX_NO_TENSOR;
  std::vector<Expectation> expects;
  std::map<uint32_t, std::vector<uint8_t>> captured_inputs;
  std::string case_name;
};

namespace {

std::string g_case_name;
b2vx_graph* g_last_graph = nullptr;
int g_case_serial = 0;

b2vx_status fail(b2vx_graph* g, b2vx_status st, const std::string& msg) {
  if (g && g->ctx) g->ctx->err = msg;
  return st;
}

bool valid_id(const b2vx_graph* g, uint32_t id) { return id < g->tensors.size(); }

// ---------------------------------------------------------------- capture

void json_bytes(FILE* f, const uint8_t* p, size_t n) {
  static const char* hex = "0123456789abcdef";
  std::fputc('"', f);
  for (size_t i = 0; i < n; ++i) {
    std::fputc(hex[p[i] >> 4], f);
    std::fputc(hex[p[i] & 15], f);
  }
  std::fputc('"', f);
}

void write_case(b2vx_graph* g) {
  const char* dir = std::getenv("B2VX_CAPTURE_DIR");
  if (!dir || !g->ran) return;
  char path[1024];
  std::string safe = g->case_name.empty() ? std::string("case") : g->case_name;
  for (char& c : safe) if (!((c >= 'a' && c <= 'z') || (c >= 'A' && c <= 'Z') || (c >= '0' && c <= '9') || c == '_' || c == '.')) c = '_';
  std::snprintf(path, sizeof(path), "%s/%s__%03d.json", dir, safe.c_str(), g_case_serial++);
  FILE* f = std::fopen(path, "w");
  if (!f) return;
  std::fprintf(f, "{\"name\": \"%s\",\n \"tensors\": [\n", g->case_name.c_str());
  for (size_t i = 0; i < g->tensors.size(); ++i) {
    const OTensor& t = g->tensors[i];
    std::fprintf(f, "  {\"id\": %zu, \"dtype\": %d, \"dims\": [", i, t.d.dtype);
    for (uint32_t k = 0; k < t.d.rank; ++k) std::fprintf(f, "%s%u", k ? ", " : "", t.d.dims[k]);
    std::fprintf(f, "], \"attr\": %d, \"quant_type\": %d, \"scale\": %.9g, \"zero_point\": %d, \"channel_dim\": %d, \"scales\": [",
                 t.d.attr, t.d.quant_type, t.d.scale, t.d.zero_point, t.d.channel_dim);
    for (size_t k = 0; k < t.scales.size(); ++k) std::fprintf(f, "%s%.9g", k ? ", " : "", t.scales[k]);
    std::fprintf(f, "], \"zero_points\": [");
    for (size_t k = 0; k < t.zps.size(); ++k) std::fprintf(f, "%s%d", k ? ", " : "", t.zps[k]);
    std::fprintf(f, "], \"declared_rank\": %u, \"data\": ", t.declared ? t.d.rank : 0);
    bool keep = (t.d.attr & B2VX_ATTR_CONSTANT) || (t.d.attr & B2VX_ATTR_OUTPUT);
    auto in_it = g->captured_inputs.find(static_cast<uint32_t>(i));
    if (in_it != g->captured_inputs.end()) json_bytes(f, in_it->second.data(), in_it->second.size());
    else if (keep && !t.data.empty()) json_bytes(f, t.data.data(), t.data.size());
    else std::fprintf(f, "null");
    std::fprintf(f, "}%s\n", i + 1 < g->tensors.size() ? "," : "");
  }
  std::fprintf(f, " ],\n \"nodes\": [\n");
  for (size_t i = 0; i < g->nodes.size(); ++i) {
    const ONode& n = g->nodes[i];
    std::fprintf(f, "  {\"kind\": %d, \"in\": [%u, %u, %u", n.kind, n.in[0], n.in[1], n.in[2]);
    for (uint32_t k = 3; k < B2VX_MAX_NODE_INPUTS && n.in[k] != B2VX_NO_TENSOR; ++k) std::fprintf(f, ", %u", n.in[k]);
    std::fprintf(f, "], \"out\": %u", n.out);
    if (n.kind == B2VX_NODE_CONV2D) {
      const b2vx_conv2d_desc& c = n.p.conv;
      std::fprintf(f, ", \"weights\": %u, \"pad_type\": %d, \"ksize\": [%u, %u], \"stride\": [%u, %u], \"dilation\": [%u, %u], \"pad\": [%u, %u, %u, %u], \"multiplier\": %d, \"group\": %d",
                   c.weights, c.pad_type, c.ksize[0], c.ksize[1], c.stride[0], c.stride[1], c.dilation[0], c.dilation[1],
                   c.pad[0], c.pad[1], c.pad[2], c.pad[3], c.multiplier, c.group);
    } else if (n.kind == B2VX_NODE_FULLY_CONNECTED) {
      std::fprintf(f, ", \"axis\": %u, \"weights\": %u", n.p.fc.axis, n.p.fc.weights);
    } else if (n.kind == B2VX_NODE_POOL2D) {
      const b2vx_pool2d_desc& c = n.p.pool;
      std::fprintf(f, ", \"type\": %d, \"pad_type\": %d, \"ksize\": [%u, %u], \"stride\": [%u, %u], \"pad\": [%u, %u, %u, %u], \"round_type\": %d",
                   c.type, c.pad_type, c.ksize[0], c.ksize[1], c.stride[0], c.stride[1], c.pad[0], c.pad[1], c.pad[2], c.pad[3],
                   c.round_type);
    } else if (n.kind == B2VX_NODE_SOFTMAX) {
      std::fprintf(f, ", \"beta\": %.9g, \"axis\": %d", n.p.softmax.beta, n.p.softmax.axis);
    } else if (n.kind == B2VX_NODE_RESHAPE || n.kind == B2VX_NODE_TRANSPOSE) {
      std::fprintf(f, ", \"dims\": [");
      for (uint32_t k = 0; k < n.p.dims.rank; ++k) std::fprintf(f, "%s%u", k ? ", " : "", n.p.dims.v[k]);
      std::fprintf(f, "]");
    } else if (n.kind == B2VX_NODE_CONCAT) {
      std::fprintf(f, ", \"axis\": %u", n.p.concat_axis);
    }
    std::fprintf(f, "}%s\n", i + 1 < g->nodes.size() ? "," : "");
  }
  std::fprintf(f, " ],\n \"expect\": [\n");
  for (size_t i = 0; i < g->expects.size(); ++i) {
    const Expectation& e = g->expects[i];
    std::fprintf(f, "  {\"tensor\": %u, \"dtype\": %d, \"tol\": %.9g, \"data\": ", e.tensor, e.dtype, e.tol);
    json_bytes(f, e.data.data(), e.data.size());
    std::fprintf(f, "}%s\n", i + 1 < g->expects.size() ? "," : "");
  }
  std::fprintf(f, " ]\n}\n");
  std::fclose(f);
}

// ---------------------------------------------------------------- shape inference

void resolve_pads(int32_t pad_type, const uint32_t in[2], const uint32_t k[2], const uint32_t stride[2],
                  const uint32_t dil[2], const uint32_t explicit_pad[4], uint32_t out[4]) {
  // vsi_nn_compute_padding (src/tim/vx/internal/src/utils/vsi_nn_util.c:555-588):
  // AUTO (and NONE, which the C++ layer turns into AUTO) keeps the explicit
  // pads; dilation {0,0} means {1,1}.
  for (int i = 0; i < 4; ++i) out[i] = explicit_pad[i];
  if (pad_type != B2VX_PAD_SAME && pad_type != B2VX_PAD_VALID) return;
  uint32_t d0 = dil[0], d1 = dil[1];
  if (d0 == 0 && d1 == 0) d0 = d1 = 1;
  orc_same_valid_padding(in[0], k[0], stride[0], d0, pad_type, out);
  orc_same_valid_padding(in[1], k[1], stride[1], d1, pad_type, out + 2);
}

// A declared output shape is kept, as in the reference's op_setup functions
// (they only fill shapes left as "auto").  For conv/pool it may be smaller in
// W/H than the inferred one: the reference's own test
// src/tim/vx/ops/depthwiseConv_test.cc:268-330 declares 1x1 where SAME padding
// gives 1x2 and expects the first window only.
b2vx_status set_shape(b2vx_graph* g, uint32_t id, const std::vector<uint32_t>& dims, const char* what,
                      bool spatial_may_shrink = false) {
  OTensor& t = g->tensors[id];
  if (t.has_shape) {
    bool same = t.d.rank == dims.size();
    for (size_t i = 0; same && i < dims.size(); ++i) {
      if (spatial_may_shrink && i < 2) same = t.d.dims[i] >= 1 && t.d.dims[i] <= dims[i];
      else same = t.d.dims[i] == dims[i];
    }
    if (!same) return fail(g, B2VX_SHAPE_MISMATCH, std::string(what) + ": declared output shape differs from the inferred one");
    return B2VX_OK;
  }
  t.d.rank = static_cast<uint32_t>(dims.size());
  for (size_t i = 0; i < dims.size(); ++i) t.d.dims[i] = dims[i];
  t.has_shape = true;
  return B2VX_OK;
}

b2vx_status infer_node(b2vx_graph* g, ONode& n) {
  const OTensor& x = g->tensors[n.in[0]];
  if (!x.has_shape) return fail(g, B2VX_SHAPE_MISMATCH, "input shape unknown");
  switch (n.kind) {
    case B2VX_NODE_CONV2D: {
      const OTensor& w = g->tensors[n.in[1]];
      if (x.d.rank < 3 || x.d.rank > 4 || w.d.rank != 4) return fail(g, B2VX_SHAPE_MISMATCH, "conv2d: rank");
      const b2vx_conv2d_desc& c = n.p.conv;
      uint32_t in2[2] = {x.d.dims[0], x.d.dims[1]}, k2[2] = {w.d.dims[0], w.d.dims[1]};
      resolve_pads(c.pad_type, in2, k2, c.stride, c.dilation, c.pad, n.pad_resolved);
      uint32_t wo = orc_filter_size(in2[0], k2[0], n.pad_resolved[0], n.pad_resolved[1], c.stride[0], c.dilation[0], B2VX_ROUND_FLOOR);
      uint32_t ho = orc_filter_size(in2[1], k2[1], n.pad_resolved[2], n.pad_resolved[3], c.stride[1], c.dilation[1], B2VX_ROUND_FLOOR);
      uint32_t oc = c.weights > 0 ? c.weights : (c.multiplier > 0 ? x.d.dims[2] * c.multiplier : w.d.dims[3]);
      if (wo == 0 || ho == 0) return fail(g, B2VX_SHAPE_MISMATCH, "conv2d: empty output");
      std::vector<uint32_t> dims = {wo, ho, oc};
      if (x.d.rank == 4) dims.push_back(x.d.dims[3]);
      return set_shape(g, n.out, dims, "conv2d", true);
    }
    case B2VX_NODE_FULLY_CONNECTED: {
      const OTensor& w = g->tensors[n.in[1]];
      if (w.d.rank != 2 || n.p.fc.axis >= x.d.rank) return fail(g, B2VX_SHAPE_MISMATCH, "fully_connected: rank/axis");
      std::vector<uint32_t> dims = {n.p.fc.weights ? n.p.fc.weights : w.d.dims[1]};
      for (uint32_t i = n.p.fc.axis + 1; i < x.d.rank; ++i) dims.push_back(x.d.dims[i]);
      if (dims.size() == 1) dims.push_back(1);
      OTensor& y = g->tensors[n.out];
      if (y.has_shape) {
        // A declared output only has to hold the same number of elements.
        size_t want = 1;
        for (uint32_t v : dims) want *= v;
        if (y.elems() != want) return fail(g, B2VX_SHAPE_MISMATCH, "fully_connected: output size");
        return B2VX_OK;
      }
      return set_shape(g, n.out, dims, "fully_connected");
    }
    case B2VX_NODE_POOL2D: {
      if (x.d.rank < 3 || x.d.rank > 4) return fail(g, B2VX_SHAPE_MISMATCH, "pool2d: rank");
      const b2vx_pool2d_desc& c = n.p.pool;
      uint32_t in2[2] = {x.d.dims[0], x.d.dims[1]};
      uint32_t dil[2] = {1, 1};
      resolve_pads(c.pad_type, in2, c.ksize, c.stride, dil, c.pad, n.pad_resolved);
      uint32_t wo = orc_filter_size(in2[0], c.ksize[0], n.pad_resolved[0], n.pad_resolved[1], c.stride[0], 1, c.round_type);
      uint32_t ho = orc_filter_size(in2[1], c.ksize[1], n.pad_resolved[2], n.pad_resolved[3], c.stride[1], 1, c.round_type);
      if (wo == 0 || ho == 0) return fail(g, B2VX_SHAPE_MISMATCH, "pool2d: empty output");
      std::vector<uint32_t> dims = {wo, ho};
      for (uint32_t i = 2; i < x.d.rank; ++i) dims.push_back(x.d.dims[i]);
      return set_shape(g, n.out, dims, "pool2d", true);
    }
    case B2VX_NODE_ADDN: {
      for (uint32_t id : n.in) {
        if (id == B2VX_NO_TENSOR) continue;
        const OTensor& t = g->tensors[id];
        if (!t.has_shape || t.d.rank != x.d.rank) return fail(g, B2VX_SHAPE_MISMATCH, "addn: input shapes differ");
        for (uint32_t i = 0; i < x.d.rank; ++i)
          if (t.d.dims[i] != x.d.dims[i]) return fail(g, B2VX_SHAPE_MISMATCH, "addn: input shapes differ");
      }
      return set_shape(g, n.out, std::vector<uint32_t>(x.d.dims, x.d.dims + x.d.rank), "addn");
    }
    case B2VX_NODE_ADD: {
      const OTensor& b = g->tensors[n.in[1]];
      if (!b.has_shape) return fail(g, B2VX_SHAPE_MISMATCH, "add: input shape unknown");
      uint32_t rank = std::max(x.d.rank, b.d.rank);
      std::vector<uint32_t> dims(rank);
      for (uint32_t i = 0; i < rank; ++i) {
        uint32_t da = i < x.d.rank ? x.d.dims[i] : 1, db = i < b.d.rank ? b.d.dims[i] : 1;
        if (da != db && da != 1 && db != 1) return fail(g, B2VX_SHAPE_MISMATCH, "add: shapes do not broadcast");
        dims[i] = std::max(da, db);
      }
      return set_shape(g, n.out, dims, "add");
    }
    case B2VX_NODE_RESHAPE: {
      // src/tim/vx/ops/reshape.cc:46-58: the target shape is the output's shape; element counts must agree
      const b2vx_dims_desc& d = n.p.dims;
      std::vector<uint32_t> dims(d.v, d.v + d.rank);
      size_t want = 1;
      for (uint32_t v : dims) want *= v;
      if (want != x.elems()) return fail(g, B2VX_SHAPE_MISMATCH, "reshape: element count changes");
      OTensor& y = g->tensors[n.out];
      if (y.has_shape) return y.elems() == want ? B2VX_OK : fail(g, B2VX_SHAPE_MISMATCH, "reshape: declared output size");
      return set_shape(g, n.out, dims, "reshape");
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
      return set_shape(g, n.out, dims, "transpose");
    }
    case B2VX_NODE_CONCAT: {
      // vsi_nn_op_concat.c op_setup: all dimensions but `axis` agree; the axis extents add up
      const uint32_t axis = n.p.concat_axis;
      if (axis >= x.d.rank) return fail(g, B2VX_SHAPE_MISMATCH, "concat: axis outside the input rank");
      std::vector<uint32_t> dims(x.d.dims, x.d.dims + x.d.rank);
      dims[axis] = 0;
      for (uint32_t id : n.in) {
        if (id == B2VX_NO_TENSOR) continue;
        const OTensor& t = g->tensors[id];
        if (!t.has_shape || t.d.rank != x.d.rank) return fail(g, B2VX_SHAPE_MISMATCH, "concat: input ranks differ");
        for (uint32_t i = 0; i < x.d.rank; ++i)
          if (i != axis && t.d.dims[i] != x.d.dims[i]) return fail(g, B2VX_SHAPE_MISMATCH, "concat: input shapes differ off the axis");
        dims[axis] += t.d.dims[axis];
      }
      return set_shape(g, n.out, dims, "concat");
    }
    default: {
      std::vector<uint32_t> dims(x.d.dims, x.d.dims + x.d.rank);
      return set_shape(g, n.out, dims, "unary");
    }
  }
}

// ---------------------------------------------------------------- execution

b2vx_status exec_node(b2vx_graph* g, ONode& n) {
  OTensor& x = g->tensors[n.in[0]];
  OTensor& y = g->tensors[n.out];
  y.data.assign(y.bytes(), 0);
  int32_t rc = -1;
  switch (n.kind) {
    case B2VX_NODE_CONV2D: {
      OTensor& w = g->tensors[n.in[1]];
      orc_conv2d_args a;
      std::memset(&a, 0, sizeof(a));
      a.x = x.data.data(); a.x_dtype = x.d.dtype;
      a.W = x.d.dims[0]; a.H = x.d.dims[1]; a.C = x.d.dims[2]; a.N = x.d.rank == 4 ? x.d.dims[3] : 1;
      a.xq = x.quant();
      a.w = w.data.data(); a.w_dtype = w.d.dtype;
      a.kw = w.d.dims[0]; a.kh = w.d.dims[1]; a.w_ic = w.d.dims[2]; a.w_oc = w.d.dims[3];
      a.wq = w.quant();
      a.bias = n.in[2] != B2VX_NO_TENSOR ? g->tensors[n.in[2]].data.data() : nullptr;
      a.y = y.data.data(); a.y_dtype = y.d.dtype;
      a.Wo = y.d.dims[0]; a.Ho = y.d.dims[1]; a.Oc = y.d.dims[2];
      a.yq = y.quant();
      a.stride[0] = n.p.conv.stride[0]; a.stride[1] = n.p.conv.stride[1];
      a.dilation[0] = n.p.conv.dilation[0]; a.dilation[1] = n.p.conv.dilation[1];
      a.pad_left = n.pad_resolved[0]; a.pad_top = n.pad_resolved[2];
      a.multiplier = n.p.conv.multiplier;
      a.group = n.p.conv.group;
      if (a.group > 1) {
        if (a.multiplier >= 1) return fail(g, B2VX_UNSUPPORTED, "conv2d: group and multiplier together");
        if (a.C % a.group || a.Oc % a.group || a.w_ic * static_cast<uint32_t>(a.group) != a.C || a.w_oc != a.Oc)
          return fail(g, B2VX_SHAPE_MISMATCH, "grouped conv2d: kernel must be [kw, kh, C/group, Oc] with C and Oc multiples of group");
      } else if (a.multiplier >= 1) {
        if (a.w_ic != a.C * static_cast<uint32_t>(a.multiplier) || a.Oc != a.w_ic)
          return fail(g, B2VX_SHAPE_MISMATCH, "depthwise conv2d: kernel channels != C*multiplier");
      } else if (a.w_ic != a.C || a.w_oc != a.Oc) {
        return fail(g, B2VX_SHAPE_MISMATCH, "conv2d: kernel shape does not match input/output channels");
      }
      rc = orc_conv2d(&a);
      break;
    }
    case B2VX_NODE_FULLY_CONNECTED: {
      OTensor& w = g->tensors[n.in[1]];
      orc_fc_args a;
      std::memset(&a, 0, sizeof(a));
      size_t K = 1;
      for (uint32_t i = 0; i <= n.p.fc.axis; ++i) K *= x.d.dims[i];
      if (K != w.d.dims[0]) return fail(g, B2VX_SHAPE_MISMATCH, "fully_connected: K mismatch");
      a.x = x.data.data(); a.x_dtype = x.d.dtype; a.K = static_cast<uint32_t>(K);
      a.batch = static_cast<uint32_t>(x.elems() / K); a.xq = x.quant();
      a.w = w.data.data(); a.w_dtype = w.d.dtype; a.N = w.d.dims[1]; a.wq = w.quant();
      a.bias = n.in[2] != B2VX_NO_TENSOR ? g->tensors[n.in[2]].data.data() : nullptr;
      a.y = y.data.data(); a.y_dtype = y.d.dtype; a.yq = y.quant();
      rc = orc_fully_connected(&a);
      break;
    }
    case B2VX_NODE_POOL2D: {
      orc_pool2d_args a;
      std::memset(&a, 0, sizeof(a));
      if (x.d.dtype != y.d.dtype) return fail(g, B2VX_UNSUPPORTED, "pool2d: input/output dtype differ");
      a.x = x.data.data(); a.dtype = x.d.dtype;
      a.W = x.d.dims[0]; a.H = x.d.dims[1]; a.C = x.d.dims[2]; a.N = x.d.rank == 4 ? x.d.dims[3] : 1;
      a.xq = x.quant();
      a.y = y.data.data(); a.Wo = y.d.dims[0]; a.Ho = y.d.dims[1]; a.yq = y.quant();
      a.type = n.p.pool.type;
      a.ksize[0] = n.p.pool.ksize[0]; a.ksize[1] = n.p.pool.ksize[1];
      a.stride[0] = n.p.pool.stride[0] ? n.p.pool.stride[0] : 1;
      a.stride[1] = n.p.pool.stride[1] ? n.p.pool.stride[1] : 1;
      a.pad_left = n.pad_resolved[0]; a.pad_top = n.pad_resolved[2];
      rc = orc_pool2d(&a);
      break;
    }
    case B2VX_NODE_ADD: {
      OTensor& b = g->tensors[n.in[1]];
      uint32_t rank = y.d.rank, ad[8], bd[8];
      for (uint32_t i = 0; i < rank; ++i) {
        ad[i] = i < x.d.rank ? x.d.dims[i] : 1;
        bd[i] = i < b.d.rank ? b.d.dims[i] : 1;
      }
      rc = orc_add(x.data.data(), x.d.dtype, ad, x.quant(), b.data.data(), b.d.dtype, bd, b.quant(),
                   y.data.data(), y.d.dtype, y.d.dims, y.quant(), rank);
      break;
    }
    case B2VX_NODE_ADDN: {
      const void* ptrs[B2VX_MAX_NODE_INPUTS];
      int32_t dts[B2VX_MAX_NODE_INPUTS];
      orc_quant qs[B2VX_MAX_NODE_INPUTS];
      uint32_t cnt = 0;
      for (uint32_t id : n.in) {
        if (id == B2VX_NO_TENSOR) continue;
        OTensor& t = g->tensors[id];
        ptrs[cnt] = t.data.data(); dts[cnt] = t.d.dtype; qs[cnt] = t.quant();
        ++cnt;
      }
      rc = orc_addn(ptrs, dts, qs, cnt, y.data.data(), y.d.dtype, y.quant(), y.elems());
      break;
    }
    case B2VX_NODE_RELU:
    case B2VX_NODE_RELU6:
      rc = orc_relu(x.data.data(), x.d.dtype, x.quant(), y.data.data(), y.d.dtype, y.quant(), x.elems(),
                    n.kind == B2VX_NODE_RELU6 ? 6.0f : -1.0f);
      break;
    case B2VX_NODE_RESHAPE:
      if (x.d.dtype != y.d.dtype) return fail(g, B2VX_UNSUPPORTED, "reshape: input/output dtype differ");
      std::memcpy(y.data.data(), x.data.data(), y.bytes());
      rc = 0;
      break;
    case B2VX_NODE_TRANSPOSE: {
      if (x.d.dtype != y.d.dtype) return fail(g, B2VX_UNSUPPORTED, "transpose: input/output dtype differ");
      const size_t es = dtype_size(x.d.dtype);
      const uint32_t rank = x.d.rank;
      size_t istride[8], s0 = 1;
      for (uint32_t i = 0; i < rank; ++i) { istride[i] = s0; s0 *= x.d.dims[i]; }
      const size_t total = y.elems();
      for (size_t o = 0; o < total; ++o) {
        size_t rem = o, src = 0;
        for (uint32_t i = 0; i < rank; ++i) {
          const size_t c = rem % y.d.dims[i];
          rem /= y.d.dims[i];
          src += c * istride[n.p.dims.v[i]];
        }
        std::memcpy(y.data.data() + o * es, x.data.data() + src * es, es);
      }
      rc = 0;
      break;
    }
    case B2VX_NODE_CONCAT: {
      const uint32_t axis = n.p.concat_axis, rank = y.d.rank;
      const size_t es = dtype_size(y.d.dtype);
      size_t inner = 1, outer = 1;
      for (uint32_t i = 0; i < axis; ++i) inner *= y.d.dims[i];
      for (uint32_t i = axis + 1; i < rank; ++i) outer *= y.d.dims[i];
      size_t offset = 0;   // along the axis
      for (uint32_t id : n.in) {
        if (id == B2VX_NO_TENSOR) continue;
        OTensor& t = g->tensors[id];
        if (t.d.dtype != y.d.dtype) return fail(g, B2VX_UNSUPPORTED, "concat: input/output dtype differ");
        const orc_quant tq = t.quant(), yq = y.quant();
        const bool q8 = t.d.dtype == B2VX_DT_UINT8 || t.d.dtype == B2VX_DT_INT8;
        const bool convert = q8 && (tq.scale != yq.scale || tq.zp != yq.zp);
        const size_t ext = t.d.dims[axis];
        for (size_t o = 0; o < outer; ++o)
          for (size_t a = 0; a < ext; ++a) {
            const size_t src = (o * ext + a) * inner, dst = (o * y.d.dims[axis] + offset + a) * inner;
            if (!convert) {
              std::memcpy(y.data.data() + dst * es, t.data.data() + src * es, inner * es);
            } else {
              for (size_t i = 0; i < inner; ++i) {
                const int32_t v = t.d.dtype == B2VX_DT_UINT8 ? static_cast<int32_t>(t.data[src + i])
                                                             : static_cast<int32_t>(static_cast<int8_t>(t.data[src + i]));
                const int32_t q = orc_fp32_to_affine(orc_affine_to_fp32(v, tq.scale, tq.zp), yq.scale, yq.zp, y.d.dtype);
                y.data[dst + i] = static_cast<uint8_t>(q & 0xFF);
              }
            }
          }
        offset += ext;
      }
      rc = 0;
      break;
    }
    case B2VX_NODE_DATACONVERT: {
      // dequantize with the input's parameters, quantize with the output's (float32 passes through)
      const orc_quant xq = x.quant(), yq = y.quant();
      const size_t total = x.elems();
      rc = 0;
      for (size_t i = 0; i < total && rc == 0; ++i) {
        float real;
        switch (x.d.dtype) {
          case B2VX_DT_FLOAT32: real = reinterpret_cast<const float*>(x.data.data())[i]; break;
          case B2VX_DT_UINT8: real = orc_affine_to_fp32(x.data[i], xq.scale, xq.zp); break;
          case B2VX_DT_INT8: real = orc_affine_to_fp32(static_cast<int8_t>(x.data[i]), xq.scale, xq.zp); break;
          case B2VX_DT_INT32: real = orc_affine_to_fp32(reinterpret_cast<const int32_t*>(x.data.data())[i], xq.scale, xq.zp); break;
          default: rc = -1; real = 0.0f; break;
        }
        switch (y.d.dtype) {
          case B2VX_DT_FLOAT32: reinterpret_cast<float*>(y.data.data())[i] = real; break;
          case B2VX_DT_UINT8: case B2VX_DT_INT8:
            y.data[i] = static_cast<uint8_t>(orc_fp32_to_affine(real, yq.scale, yq.zp, y.d.dtype) & 0xFF);
            break;
          case B2VX_DT_INT32: reinterpret_cast<int32_t*>(y.data.data())[i] = orc_fp32_to_affine(real, yq.scale, yq.zp, y.d.dtype); break;
          default: rc = -1; break;
        }
      }
      break;
    }
    case B2VX_NODE_SOFTMAX:
      rc = orc_softmax(x.data.data(), x.d.dtype, x.quant(), y.data.data(), y.d.dtype, y.quant(), x.d.dims,
                       x.d.rank, n.p.softmax.axis, n.p.softmax.beta);
      break;
    default: break;
  }
  if (rc != 0) return fail(g, B2VX_UNSUPPORTED, "oracle: unsupported dtype combination");
  return B2VX_OK;
}

bool supported_dtype(int32_t dt) {
  return dt == B2VX_DT_INT8 || dt == B2VX_DT_UINT8 || dt == B2VX_DT_INT32 || dt == B2VX_DT_FLOAT32;
}

b2vx_status add_node(b2vx_graph* g, int32_t kind, uint32_t i0, uint32_t i1, uint32_t i2, uint32_t out, ONode* proto) {
  if (!g) return B2VX_INVALID_ARG;
  if (g->compiled) return fail(g, B2VX_BAD_STATE, "graph already compiled");
  if (!valid_id(g, i0) || !valid_id(g, out)) return fail(g, B2VX_INVALID_ARG, "node: bad tensor id");
  if (i1 != B2VX_NO_TENSOR && !valid_id(g, i1)) return fail(g, B2VX_INVALID_ARG, "node: bad tensor id");
  if (i2 != B2VX_NO_TENSOR && !valid_id(g, i2)) return fail(g, B2VX_INVALID_ARG, "node: bad tensor id");
  ONode n = proto ? *proto : ONode();
  if (!proto) std::memset(&n, 0, sizeof(n));
  n.kind = kind;
  for (uint32_t& id : n.in) id = B2VX_NO_TENSOR;
  n.in[0] = i0; n.in[1] = i1; n.in[2] = i2; n.out = out;
  g->nodes.push_back(n);
  return B2VX_OK;
}

}  // namespace

extern "C" {

// Hooks for the golden-vector harness (not part of b2vx.h).
void orc_capture_set_case(const char* name) { g_case_name = name ? name : ""; }
// a and b are the two sides of a vector comparison made right after a tensor
// read; the side that equals what was read is the actual output, the other one
// is the expectation to record.
void orc_capture_expect_pair(const void* a, const void* b, size_t bytes, int32_t dtype, double tol) {
  b2vx_graph* g = g_last_graph;
  if (!g || g->last_read == B2VX_NO_TENSOR) return;
  const OTensor& t = g->tensors[g->last_read];
  const void* expected = a;
  if (t.data.size() == bytes && std::memcmp(a, t.data.data(), bytes) == 0 && std::memcmp(b, t.data.data(), bytes) != 0)
    expected = b;
  Expectation e;
  e.tensor = g->last_read;
  e.dtype = dtype;
  e.tol = tol;
  e.data.assign(static_cast<const uint8_t*>(expected), static_cast<const uint8_t*>(expected) + bytes);
  g->expects.push_back(std::move(e));
}

b2vx_status b2vx_context_create(b2vx_context** out) {
  if (!out) return B2VX_INVALID_ARG;
  *out = new b2vx_context();
  return B2VX_OK;
}
void b2vx_context_destroy(b2vx_context* ctx) { delete ctx; }
const char* b2vx_last_error(const b2vx_context* ctx) { return ctx ? ctx->err.c_str() : ""; }
// the host counts as one device, so that device-enumerating callers (tim::vx::platform) work on the oracle too
int32_t b2vx_device_count(void) { return 1; }

b2vx_status b2vx_graph_create(b2vx_context* ctx, int32_t, b2vx_graph** out) {
  if (!ctx || !out) return B2VX_INVALID_ARG;
  b2vx_graph* g = new b2vx_graph();
  g->ctx = ctx;
  g->case_name = g_case_name;
  *out = g;
  return B2VX_OK;
}

void b2vx_graph_destroy(b2vx_graph* g) {
  if (!g) return;
  write_case(g);
  if (g_last_graph == g) g_last_graph = nullptr;
  delete g;
}

b2vx_status b2vx_tensor_create(b2vx_graph* g, const b2vx_tensor_desc* desc, const void* const_data, uint32_t* out_id) {
  if (!g || !desc || !out_id) return B2VX_INVALID_ARG;
  if (desc->rank > B2VX_MAX_RANK) return fail(g, B2VX_INVALID_ARG, "tensor: rank too large");
  if (!supported_dtype(desc->dtype)) return fail(g, B2VX_UNSUPPORTED, "tensor: dtype not supported on this path");
  OTensor t;
  t.d = *desc;
  if (desc->quant_type == B2VX_QUANT_SYMMETRIC_PER_CHANNEL) {
    if (!desc->scales || desc->n_channel == 0) return fail(g, B2VX_INVALID_ARG, "tensor: per-channel scales missing");
    t.scales.assign(desc->scales, desc->scales + desc->n_channel);
    if (desc->zero_points) t.zps.assign(desc->zero_points, desc->zero_points + desc->n_channel);
  }
  t.d.scales = nullptr;
  t.d.zero_points = nullptr;
  t.has_shape = desc->rank > 0;
  t.declared = t.has_shape;
  if (const_data) {
    if (!t.has_shape) return fail(g, B2VX_INVALID_ARG, "tensor: data without a shape");
    t.data.assign(static_cast<const uint8_t*>(const_data), static_cast<const uint8_t*>(const_data) + t.bytes());
    t.written = true;
  }
  g->tensors.push_back(std::move(t));
  *out_id = static_cast<uint32_t>(g->tensors.size() - 1);
  return B2VX_OK;
}

b2vx_status b2vx_tensor_get_desc(b2vx_graph* g, uint32_t id, b2vx_tensor_desc* out) {
  if (!g || !out || !valid_id(g, id)) return B2VX_INVALID_ARG;
  OTensor& t = g->tensors[id];
  *out = t.d;
  if (!t.has_shape) out->rank = 0;
  out->n_channel = static_cast<uint32_t>(t.scales.size());
  out->scales = t.scales.empty() ? nullptr : t.scales.data();
  out->zero_points = t.zps.empty() ? nullptr : t.zps.data();
  return B2VX_OK;
}

b2vx_status b2vx_tensor_write(b2vx_graph* g, uint32_t id, const void* src, size_t bytes) {
  if (!g || !src || !valid_id(g, id)) return B2VX_INVALID_ARG;
  OTensor& t = g->tensors[id];
  if (t.d.attr & B2VX_ATTR_TRANSIENT) return fail(g, B2VX_BAD_STATE, "tensor_write: transient tensor");
  if (!t.has_shape || bytes != t.bytes()) return fail(g, B2VX_INVALID_ARG, "tensor_write: byte size mismatch");
  t.data.assign(static_cast<const uint8_t*>(src), static_cast<const uint8_t*>(src) + bytes);
  t.written = true;
  if (t.d.attr & B2VX_ATTR_INPUT) g->captured_inputs[id] = t.data;
  return B2VX_OK;
}

b2vx_status b2vx_tensor_read(b2vx_graph* g, uint32_t id, void* dst, size_t bytes) {
  if (!g || !dst || !valid_id(g, id)) return B2VX_INVALID_ARG;
  OTensor& t = g->tensors[id];
  if (!t.has_shape || bytes != t.bytes()) return fail(g, B2VX_INVALID_ARG, "tensor_read: byte size mismatch");
  if (t.data.size() != bytes) return fail(g, B2VX_BAD_STATE, "tensor_read: tensor holds no data yet");
  std::memcpy(dst, t.data.data(), bytes);
  g->last_read = id;
  g_last_graph = g;
  return B2VX_OK;
}

b2vx_status b2vx_node_conv2d(b2vx_graph* g, uint32_t x, uint32_t w, uint32_t bias, uint32_t y, const b2vx_conv2d_desc* d) {
  if (!d) return B2VX_INVALID_ARG;
  ONode n;
  std::memset(&n, 0, sizeof(n));
  n.p.conv = *d;
  if (g && (!valid_id(g, w))) return fail(g, B2VX_INVALID_ARG, "conv2d: weight tensor missing");
  return add_node(g, B2VX_NODE_CONV2D, x, w, bias, y, &n);
}

b2vx_status b2vx_node_fully_connected(b2vx_graph* g, uint32_t x, uint32_t w, uint32_t bias, uint32_t y, const b2vx_fc_desc* d) {
  if (!d) return B2VX_INVALID_ARG;
  ONode n;
  std::memset(&n, 0, sizeof(n));
  n.p.fc = *d;
  if (g && (!valid_id(g, w))) return fail(g, B2VX_INVALID_ARG, "fully_connected: weight tensor missing");
  return add_node(g, B2VX_NODE_FULLY_CONNECTED, x, w, bias, y, &n);
}

b2vx_status b2vx_node_pool2d(b2vx_graph* g, uint32_t x, uint32_t y, const b2vx_pool2d_desc* d) {
  if (!d) return B2VX_INVALID_ARG;
  ONode n;
  std::memset(&n, 0, sizeof(n));
  n.p.pool = *d;
  return add_node(g, B2VX_NODE_POOL2D, x, B2VX_NO_TENSOR, B2VX_NO_TENSOR, y, &n);
}

b2vx_status b2vx_node_add(b2vx_graph* g, uint32_t a, uint32_t b, uint32_t y) {
  if (g && !valid_id(g, b)) return fail(g, B2VX_INVALID_ARG, "add: second input missing");
  return add_node(g, B2VX_NODE_ADD, a, b, B2VX_NO_TENSOR, y, nullptr);
}
b2vx_status b2vx_node_relu(b2vx_graph* g, uint32_t x, uint32_t y) {
  return add_node(g, B2VX_NODE_RELU, x, B2VX_NO_TENSOR, B2VX_NO_TENSOR, y, nullptr);
}
b2vx_status b2vx_node_relu6(b2vx_graph* g, uint32_t x, uint32_t y) {
  return add_node(g, B2VX_NODE_RELU6, x, B2VX_NO_TENSOR, B2VX_NO_TENSOR, y, nullptr);
}
b2vx_status b2vx_node_reshape(b2vx_graph* g, uint32_t x, uint32_t y, const b2vx_dims_desc* shape) {
  if (!g || !shape || shape->rank == 0 || shape->rank > B2VX_MAX_RANK) return g ? fail(g, B2VX_INVALID_ARG, "reshape: bad shape") : B2VX_INVALID_ARG;
  ONode n;
  std::memset(&n, 0, sizeof(n));
  n.p.dims = *shape;
  return add_node(g, B2VX_NODE_RESHAPE, x, B2VX_NO_TENSOR, B2VX_NO_TENSOR, y, &n);
}
b2vx_status b2vx_node_transpose(b2vx_graph* g, uint32_t x, uint32_t y, const b2vx_dims_desc* perm) {
  if (!g || !perm || perm->rank == 0 || perm->rank > B2VX_MAX_RANK) return g ? fail(g, B2VX_INVALID_ARG, "transpose: bad permutation") : B2VX_INVALID_ARG;
  ONode n;
  std::memset(&n, 0, sizeof(n));
  n.p.dims = *perm;
  return add_node(g, B2VX_NODE_TRANSPOSE, x, B2VX_NO_TENSOR, B2VX_NO_TENSOR, y, &n);
}
b2vx_status b2vx_node_concat(b2vx_graph* g, const uint32_t* inputs, uint32_t n_inputs, uint32_t axis, uint32_t y) {
  if (!g) return B2VX_INVALID_ARG;
  if (!inputs || n_inputs == 0 || n_inputs > B2VX_MAX_NODE_INPUTS) return fail(g, B2VX_INVALID_ARG, "concat: 1 to 16 inputs");
  for (uint32_t i = 0; i < n_inputs; ++i)
    if (!valid_id(g, inputs[i])) return fail(g, B2VX_INVALID_ARG, "concat: bad tensor id");
  ONode n;
  std::memset(&n, 0, sizeof(n));
  n.p.concat_axis = axis;
  b2vx_status st = add_node(g, B2VX_NODE_CONCAT, inputs[0], B2VX_NO_TENSOR, B2VX_NO_TENSOR, y, &n);
  if (st != B2VX_OK) return st;
  for (uint32_t i = 0; i < n_inputs; ++i) g->nodes.back().in[i] = inputs[i];
  return B2VX_OK;
}
b2vx_status b2vx_node_addn(b2vx_graph* g, const uint32_t* inputs, uint32_t n_inputs, uint32_t y) {
  if (!g) return B2VX_INVALID_ARG;
  if (!inputs || n_inputs < 2 || n_inputs > B2VX_MAX_NODE_INPUTS) return fail(g, B2VX_INVALID_ARG, "addn: 2 to 16 inputs");
  for (uint32_t i = 0; i < n_inputs; ++i)
    if (!valid_id(g, inputs[i])) return fail(g, B2VX_INVALID_ARG, "addn: bad tensor id");
  b2vx_status st = add_node(g, B2VX_NODE_ADDN, inputs[0], B2VX_NO_TENSOR, B2VX_NO_TENSOR, y, nullptr);
  if (st != B2VX_OK) return st;
  for (uint32_t i = 0; i < n_inputs; ++i) g->nodes.back().in[i] = inputs[i];
  return B2VX_OK;
}
b2vx_status b2vx_node_dataconvert(b2vx_graph* g, uint32_t x, uint32_t y) {
  return add_node(g, B2VX_NODE_DATACONVERT, x, B2VX_NO_TENSOR, B2VX_NO_TENSOR, y, nullptr);
}
b2vx_status b2vx_node_softmax(b2vx_graph* g, uint32_t x, uint32_t y, const b2vx_softmax_desc* d) {
  if (!d) return B2VX_INVALID_ARG;
  ONode n;
  std::memset(&n, 0, sizeof(n));
  n.p.softmax = *d;
  return add_node(g, B2VX_NODE_SOFTMAX, x, B2VX_NO_TENSOR, B2VX_NO_TENSOR, y, &n);
}

b2vx_status b2vx_graph_compile(b2vx_graph* g) {
  if (!g) return B2VX_INVALID_ARG;
  if (g->compiled) return B2VX_OK;
  // Topological order: a node is ready when every input tensor is a constant,
  // a graph input, or the output of an already ordered node.
  std::vector<char> ready(g->tensors.size(), 0), done(g->nodes.size(), 0);
  for (size_t i = 0; i < g->tensors.size(); ++i)
    ready[i] = (g->tensors[i].d.attr & (B2VX_ATTR_CONSTANT | B2VX_ATTR_INPUT | B2VX_ATTR_VARIABLE)) != 0;
  for (const ONode& n : g->nodes)
    ready[n.out] = 0;
  g->order.clear();
  bool progress = true;
  while (progress) {
    progress = false;
    for (size_t i = 0; i < g->nodes.size(); ++i) {
      if (done[i]) continue;
      ONode& n = g->nodes[i];
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
  if (g->order.size() != g->nodes.size()) return fail(g, B2VX_BAD_STATE, "graph has a cycle or an unfed input");
  g->compiled = true;
  return B2VX_OK;
}

b2vx_status b2vx_graph_run(b2vx_graph* g) {
  if (!g) return B2VX_INVALID_ARG;
  b2vx_status st = b2vx_graph_compile(g);
  if (st != B2VX_OK) return st;
  for (size_t i = 0; i < g->tensors.size(); ++i) {
    OTensor& t = g->tensors[i];
    if ((t.d.attr & (B2VX_ATTR_INPUT | B2VX_ATTR_CONSTANT)) && t.data.size() != t.bytes()) t.data.assign(t.bytes(), 0);
  }
  for (uint32_t idx : g->order) {
    st = exec_node(g, g->nodes[idx]);
    if (st != B2VX_OK) return st;
  }
  g->ran = true;
  return B2VX_OK;
}

b2vx_status b2vx_graph_run_async(b2vx_graph* g) { return b2vx_graph_run(g); }
b2vx_status b2vx_graph_sync(b2vx_graph* g) { return g ? B2VX_OK : B2VX_INVALID_ARG; }
b2vx_status b2vx_graph_set_stream(b2vx_graph* g, void*) { return g ? B2VX_OK : B2VX_INVALID_ARG; }

b2vx_status b2vx_graph_print(b2vx_graph* g) {
  if (!g) return B2VX_INVALID_ARG;
  for (size_t i = 0; i < g->nodes.size(); ++i)
    std::fprintf(stderr, "oracle node %zu kind %d in [%u %u %u] out %u\n", i, g->nodes[i].kind, g->nodes[i].in[0],
                 g->nodes[i].in[1], g->nodes[i].in[2], g->nodes[i].out);
  return B2VX_OK;
}

b2vx_status b2vx_graph_kernel_count(b2vx_graph* g, uint32_t* out) {
  if (!g || !out) return B2VX_INVALID_ARG;
  *out = 0;
  return B2VX_OK;
}
b2vx_status b2vx_graph_kernel_info(b2vx_graph*, uint32_t, b2vx_kernel_info*) { return B2VX_INVALID_ARG; }
b2vx_status b2vx_graph_profile(b2vx_graph* g, uint32_t) { return b2vx_graph_run(g); }

b2vx_status b2vx_host_alloc(void** out, size_t bytes) {
  if (!out) return B2VX_INVALID_ARG;
  *out = std::malloc(bytes ? bytes : 1);
  return *out ? B2VX_OK : B2VX_OOM;
}
void b2vx_host_free(void* p) { std::free(p); }

}  // extern "C"
