// Layout inference over the public graph interface.  Where the reference pushes a permute vector
// through every op class (src/tim/transform/ops/*_layout_inference.h), this version keeps, for every
// tensor of the source graph, up to two tensors of the new graph: one in the source's own layout and one
// in WHCN.  Ops that care about the layout (Conv2d, Pool2d declared CWHN) ask for the WHCN form, ops
// that do not (Relu, Relu6, Add, DataConvert) run in whichever form all their inputs already have, the
// rest run in the source layout; a Transpose is inserted only when the form an op asks for does not exist
// yet.  Constant kernels are permuted on the host once.  Chains such as conv -> relu -> add -> conv
// therefore stay in WHCN with one Transpose at the graph's input and one at its output.
#include <algorithm>
#include <cstdio>
#include <cstring>

#include "impl.h"
#include "tim/transform/layout_inference.h"
#include "tim/vx/ops.h"

namespace tim {
namespace transform {

class IPermuteVector {};   // callers may pass permute vectors for the inputs; they are taken as aligned

namespace {

using TensorPtr = std::shared_ptr<vx::Tensor>;
using Perm = std::vector<uint32_t>;

// output dimension i = input dimension perm[i] (ops::Transpose)
const Perm kCWHN2WHCN = {1, 2, 0, 3};
const Perm kWHCN2CWHN = {2, 0, 1, 3};

vx::ShapeType permuted(const vx::ShapeType& shape, const Perm& perm) {
  if (shape.size() != perm.size()) return shape;   // shape not known yet (or not rank 4): left to inference
  vx::ShapeType out(shape.size());
  for (size_t i = 0; i < perm.size(); ++i) out[i] = shape[perm[i]];
  return out;
}

// Elements of a dense tensor (dimension 0 fastest) reordered as ops::Transpose would.
std::vector<uint8_t> permute_data(const std::vector<uint8_t>& data, const vx::ShapeType& shape, const Perm& perm, size_t elem) {
  const size_t rank = shape.size();
  std::vector<size_t> istride(rank, 1);
  for (size_t i = 1; i < rank; ++i) istride[i] = istride[i - 1] * shape[i - 1];
  const vx::ShapeType oshape = permuted(shape, perm);
  size_t total = 1;
  for (uint32_t v : shape) total *= v;
  std::vector<uint8_t> out(data.size());
  for (size_t o = 0; o < total; ++o) {
    size_t rem = o, src = 0;
    for (size_t i = 0; i < rank; ++i) {
      src += (rem % oshape[i]) * istride[perm[i]];
      rem /= oshape[i];
    }
    std::memcpy(out.data() + o * elem, data.data() + src * elem, elem);
  }
  return out;
}

struct Forms {
  TensorPtr src;    // in the source graph's layout
  TensorPtr whcn;   // permuted CWHN -> WHCN
};

struct Inference {
  std::shared_ptr<vx::Graph> graph;
  std::map<TensorPtr, Forms> forms;

  TensorPtr transpose(const TensorPtr& from, const Perm& perm, const vx::TensorSpec& like, bool as_output) {
    vx::TensorSpec spec(like);
    spec.SetAttribute(as_output ? vx::TensorAttribute::OUTPUT : vx::TensorAttribute::TRANSIENT);
    if (!as_output) spec.SetShape(permuted(from->GetShape(), perm));
    TensorPtr to = graph->CreateTensor(spec);
    auto op = graph->CreateOperation<vx::ops::Transpose>(perm);
    (*op).BindInput(from).BindOutput(to);
    return to;
  }
  TensorPtr in_source_layout(const TensorPtr& t) {
    Forms& f = forms[t];
    if (!f.src && f.whcn) f.src = transpose(f.whcn, kWHCN2CWHN, t->GetSpec(), false);
    return f.src;
  }
  TensorPtr in_whcn(const TensorPtr& t) {
    Forms& f = forms[t];
    if (!f.whcn && f.src) f.whcn = transpose(f.src, kCWHN2WHCN, t->GetSpec(), false);
    return f.whcn;
  }
  // a constant of the source graph, copied as it is
  TensorPtr constant(const TensorPtr& t) {
    Forms& f = forms[t];
    if (!f.src) f.src = graph->CreateTensor(t->GetSpec(), static_cast<vx::TensorImpl*>(t.get())->ConstData().data());
    return f.src;
  }
};

bool is_const(const TensorPtr& t) { return t && t->IsConstTensor(); }

size_t element_count(const TensorPtr& t) {
  size_t n = 1;
  for (uint32_t v : t->GetShape()) n *= v;
  return n;
}

// A rank-4 constant operand of an op that runs in WHCN: its elements (and the channel dimension of a per-channel
// quantization) permuted CWHN -> WHCN on the host, as the reference's layout inference permutes the constant inputs of
// an elementwise op together with the others.
TensorPtr constant_whcn(Inference& inf, const TensorPtr& t) {
  Forms& f = inf.forms[t];
  if (f.whcn) return f.whcn;
  vx::TensorSpec spec(t->GetSpec());
  const vx::ShapeType shape = spec.GetShapeType();
  const std::vector<uint8_t>& data = static_cast<vx::TensorImpl*>(t.get())->ConstData();
  const std::vector<uint8_t> moved = permute_data(data, shape, kCWHN2WHCN, data.size() / std::max<size_t>(1, element_count(t)));
  spec.SetShape(permuted(shape, kCWHN2WHCN));
  vx::Quantization q = spec.GetQuantization();
  if (q.Type() == vx::QuantType::SYMMETRIC_PER_CHANNEL && q.ChannelDim() >= 0 && q.ChannelDim() < 4) {
    for (int32_t i = 0; i < 4; ++i)
      if (static_cast<int32_t>(kCWHN2WHCN[i]) == q.ChannelDim()) { q.SetChannelDim(i); break; }
    spec.SetQuantization(q);
  }
  f.whcn = inf.graph->CreateTensor(spec, moved.data());
  return f.whcn;
}

// A constant kernel in WHIcOc, permuted on the host; depthwise kernels end as [W, H, C*multiplier, 1].
TensorPtr native_kernel(Inference& inf, const TensorPtr& w, vx::DataLayout layout, bool depthwise) {
  Perm perm;
  switch (layout) {
    case vx::DataLayout::IcWHOc: perm = {1, 2, 0, 3}; break;   // nnapi, tflite
    case vx::DataLayout::OcIcWH: perm = {2, 3, 1, 0}; break;   // TVM
    case vx::DataLayout::IcOcWH: perm = {2, 3, 0, 1}; break;
    default: break;
  }
  vx::TensorSpec spec(w->GetSpec());
  const std::vector<uint8_t>& data = static_cast<vx::TensorImpl*>(w.get())->ConstData();
  std::vector<uint8_t> moved;
  const uint8_t* bytes = data.data();
  if (!perm.empty() && spec.GetShapeType().size() == 4) {
    moved = permute_data(data, spec.GetShapeType(), perm, static_cast<size_t>(spec.GetElementByteSize()));
    bytes = moved.data();
    vx::Quantization q = spec.GetQuantization();
    if (q.Type() == vx::QuantType::SYMMETRIC_PER_CHANNEL) {
      for (uint32_t i = 0; i < 4; ++i)
        if (static_cast<int32_t>(perm[i]) == q.ChannelDim()) { q.SetChannelDim(static_cast<int32_t>(i)); break; }
      spec.SetQuantization(q);
    }
    spec.SetShape(permuted(spec.GetShapeType(), perm));
  }
  if (depthwise && spec.GetShapeType().size() == 4 && spec.GetShapeType()[2] == 1 && spec.GetShapeType()[3] != 1) {
    // [W, H, 1, C*m] holds the same bytes as the native depthwise kernel [W, H, C*m, 1]
    vx::ShapeType s = spec.GetShapeType();
    std::swap(s[2], s[3]);
    vx::Quantization q = spec.GetQuantization();
    if (q.Type() == vx::QuantType::SYMMETRIC_PER_CHANNEL && q.ChannelDim() == 3) {
      q.SetChannelDim(2);
      spec.SetQuantization(q);
    }
    spec.SetShape(s);
  }
  return inf.graph->CreateTensor(spec, bytes);
}

}  // namespace

std::pair<std::shared_ptr<vx::Graph>, std::map<std::shared_ptr<vx::Tensor>, std::shared_ptr<vx::Tensor>>> LayoutInference(
    const std::shared_ptr<vx::Graph>& src_graph, std::shared_ptr<vx::Context>& ctx,
    std::map<std::shared_ptr<vx::Tensor>, std::shared_ptr<IPermuteVector>> tensor_pv_map) {
  (void)tensor_pv_map;
  Inference inf;
  inf.graph = ctx->CreateGraph();
  std::map<TensorPtr, TensorPtr> io_map;
  for (const TensorPtr& t : src_graph->InputsTensor()) {
    inf.forms[t].src = inf.graph->CreateTensor(t->GetSpec());
    io_map[t] = inf.forms[t].src;
  }
  const std::vector<TensorPtr> outputs = src_graph->OutputsTensor();
  auto is_output = [&](const TensorPtr& t) { return std::find(outputs.begin(), outputs.end(), t) != outputs.end(); };
  // a graph output is produced into a tensor that keeps the source's spec; where an op runs in WHCN the
  // result goes through one more Transpose into it
  auto result_tensor = [&](const TensorPtr& t) {
    TensorPtr n = inf.graph->CreateTensor(t->GetSpec());
    if (is_output(t)) io_map[t] = n;
    return n;
  };

  std::vector<std::shared_ptr<vx::Operation>> pending = src_graph->OpVector();
  bool progress = true;
  while (!pending.empty() && progress) {
    progress = false;
    for (size_t k = 0; k < pending.size(); ++k) {
      const std::shared_ptr<vx::Operation> op = pending[k];
      vx::OpImpl* impl = op->impl().get();
      bool ready = true;
      for (const TensorPtr& t : impl->inputs_tensor_) {
        if (!t || is_const(t)) continue;
        const auto it = inf.forms.find(t);
        ready = ready && it != inf.forms.end() && (it->second.src || it->second.whcn);
      }
      if (!ready) continue;
      const uint32_t kind = impl->kind_;
      const bool cwhn = impl->layout_ == vx::DataLayout::CWHN;
      std::shared_ptr<vx::Graph> g = inf.graph;
      std::shared_ptr<vx::Operation> clone = op->Clone(g);
      clone->impl()->layout_ = vx::DataLayout::WHCN;
      clone->impl()->foreign_layout_ = false;
      clone->impl()->kernel_layout_ = vx::DataLayout::WHIcOc;
      const TensorPtr out = impl->outputs_tensor_.empty() ? nullptr : impl->outputs_tensor_[0];
      if ((kind == B2VX_NODE_CONV2D || kind == B2VX_NODE_POOL2D) && cwhn) {
        clone->BindInput(inf.in_whcn(impl->inputs_tensor_[0]));
        if (kind == B2VX_NODE_CONV2D) {
          const TensorPtr w = impl->inputs_tensor_[1];
          const bool depthwise = impl->desc_.conv2d.multiplier > 0;
          if (is_const(w)) {
            clone->BindInput(native_kernel(inf, w, impl->kernel_layout_, depthwise));
          } else {
            // a kernel fed at run time: permuted by a Transpose node
            Perm perm;
            switch (impl->kernel_layout_) {
              case vx::DataLayout::IcWHOc: perm = {1, 2, 0, 3}; break;
              case vx::DataLayout::OcIcWH: perm = {2, 3, 1, 0}; break;
              case vx::DataLayout::IcOcWH: perm = {2, 3, 0, 1}; break;
              default: break;
            }
            TensorPtr wn = inf.in_source_layout(w);
            clone->BindInput(perm.empty() ? wn : inf.transpose(wn, perm, w->GetSpec(), false));
          }
          if (impl->inputs_tensor_.size() > 2 && impl->inputs_tensor_[2]) {
            const TensorPtr b = impl->inputs_tensor_[2];
            clone->BindInput(is_const(b) ? inf.constant(b) : inf.in_source_layout(b));
          }
        }
        vx::TensorSpec spec(out->GetSpec());
        spec.SetAttribute(vx::TensorAttribute::TRANSIENT);
        spec.SetShape(permuted(out->GetSpec().GetShapeType(), kCWHN2WHCN));
        TensorPtr y = inf.graph->CreateTensor(spec);
        clone->BindOutput(y);
        inf.forms[out].whcn = y;
      } else if (kind == B2VX_NODE_CONV2D && !cwhn) {
        // WHCN activations; the kernel may still come in a front-end layout
        clone->BindInput(inf.in_source_layout(impl->inputs_tensor_[0]));
        const TensorPtr w = impl->inputs_tensor_[1];
        if (is_const(w)) {
          clone->BindInput(native_kernel(inf, w, impl->kernel_layout_, impl->desc_.conv2d.multiplier > 0));
        } else {
          Perm perm;
          switch (impl->kernel_layout_) {
            case vx::DataLayout::IcWHOc: perm = {1, 2, 0, 3}; break;
            case vx::DataLayout::OcIcWH: perm = {2, 3, 1, 0}; break;
            case vx::DataLayout::IcOcWH: perm = {2, 3, 0, 1}; break;
            default: break;
          }
          TensorPtr wn = inf.in_source_layout(w);
          clone->BindInput(perm.empty() ? wn : inf.transpose(wn, perm, w->GetSpec(), false));
        }
        if (impl->inputs_tensor_.size() > 2 && impl->inputs_tensor_[2]) {
          const TensorPtr b = impl->inputs_tensor_[2];
          clone->BindInput(is_const(b) ? inf.constant(b) : inf.in_source_layout(b));
        }
        inf.forms[out].src = result_tensor(out);
        clone->BindOutput(inf.forms[out].src);
      } else {
        // layout-agnostic ops follow their inputs into WHCN when every non-constant input is there already
        const bool agnostic = kind == B2VX_NODE_RELU || kind == B2VX_NODE_RELU6 || kind == B2VX_NODE_ADD || kind == B2VX_NODE_DATACONVERT;
        bool all_whcn = agnostic;
        for (const TensorPtr& t : impl->inputs_tensor_) {
          if (!t) continue;
          if (!is_const(t)) all_whcn = all_whcn && inf.forms[t].whcn != nullptr;   // a WHCN form exists for rank-4 tensors only
          // a constant operand goes along when it has all four dimensions (it is permuted) or a single element (any
          // layout); one of lower rank would broadcast against other dimensions after the permutation, so such an op
          // stays in the source layout
          else all_whcn = all_whcn && (t->GetShape().size() == 4 || element_count(t) == 1);
        }
        for (const TensorPtr& t : impl->inputs_tensor_) {
          if (!t) continue;
          if (is_const(t)) clone->BindInput(all_whcn && t->GetShape().size() == 4 ? constant_whcn(inf, t) : inf.constant(t));
          else clone->BindInput(all_whcn ? inf.in_whcn(t) : inf.in_source_layout(t));
        }
        for (const TensorPtr& o : impl->outputs_tensor_) {
          if (all_whcn) {
            vx::TensorSpec spec(o->GetSpec());
            spec.SetAttribute(vx::TensorAttribute::TRANSIENT);
            spec.SetShape(permuted(o->GetSpec().GetShapeType(), kCWHN2WHCN));
            inf.forms[o].whcn = inf.graph->CreateTensor(spec);
            clone->BindOutput(inf.forms[o].whcn);
          } else {
            inf.forms[o].src = result_tensor(o);
            clone->BindOutput(inf.forms[o].src);
          }
        }
      }
      pending.erase(pending.begin() + static_cast<long>(k));
      --k;
      progress = true;
    }
  }
  if (!pending.empty()) std::fprintf(stderr, "E [tim-vx/b200] LayoutInference: %zu ops have inputs that nothing produces\n", pending.size());
  // graph outputs that exist only in WHCN: back to the source layout, into a tensor with the source's spec
  for (const TensorPtr& t : outputs) {
    Forms& f = inf.forms[t];
    if (f.src || !f.whcn) continue;
    f.src = inf.transpose(f.whcn, kWHCN2CWHN, t->GetSpec(), true);
    io_map[t] = f.src;
  }
  return std::make_pair(inf.graph, io_map);
}

}  // namespace transform
}  // namespace tim
