// tim::transform::LayoutInference through the public headers.
//  1. The two convolution cases of the reference's own test (src/tim/transform/layout_inference_test.cc:9-121):
//     a float 2x2 averaging kernel over a 3x3 image, declared CWHN / IcWHOc with a constant kernel, and
//     declared WHCN / IcWHOc with the kernel fed at run time; both must give 0.875 four times and keep the
//     source's output shape.
//  2. A quantized NHWC network (Conv2d 3x3 -> Relu -> depthwise 3x3 -> Add with the Relu output -> AVG pool
//     -> FullyConnected), every tensor and kernel in the front-end layouts, against the same network written
//     natively in WHCN / WHIcOc with the data permuted by hand: the logits must be the same bytes, and the
//     inferred graph must not contain more Transposes than the one at its input and the one in front of the
//     FullyConnected.
// Exits non-zero on any mismatch; prints the logits so that two builds can be compared.
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <vector>

#include "tim/transform/layout_inference.h"
#include "tim/vx/context.h"
#include "tim/vx/graph.h"
#include "tim/vx/ops.h"
#include "tim/vx/tensor.h"

using namespace tim::vx;

static uint32_t lcg_state = 4242;
static uint8_t next_byte() {
  lcg_state = lcg_state * 1664525u + 1013904223u;
  return static_cast<uint8_t>(lcg_state >> 24);
}
static Quantization quant(float s, int32_t z) { return Quantization(QuantType::ASYMMETRIC, s, z); }

static int reference_cases() {
  auto ctx = Context::Create();
  {
    auto src = ctx->CreateGraph();
    ShapeType input_shape({1, 3, 3, 1}), kernel_shape({1, 2, 2, 1}), output_shape({1, 2, 2, 1});
    auto input = src->CreateTensor(TensorSpec(DataType::FLOAT32, input_shape, TensorAttribute::INPUT));
    std::vector<float> kernel_data = {0.25f, 0.25f, 0.25f, 0.25f}, bias_data = {0.0f};
    auto kernel = src->CreateTensor(TensorSpec(DataType::FLOAT32, kernel_shape, TensorAttribute::CONSTANT), kernel_data.data());
    auto bias = src->CreateTensor(TensorSpec(DataType::FLOAT32, ShapeType({1}), TensorAttribute::CONSTANT), bias_data.data());
    auto output = src->CreateTensor(TensorSpec(DataType::FLOAT32, output_shape, TensorAttribute::OUTPUT));
    auto conv = src->CreateOperation<ops::Conv2d>(1, PadType::AUTO, std::array<uint32_t, 2>({2, 2}), std::array<uint32_t, 2>({1, 1}),
                                                  std::array<uint32_t, 2>({0, 0}), std::array<uint32_t, 4>({0, 0, 0, 0}), 0,
                                                  DataLayout::CWHN, DataLayout::IcWHOc);
    (*conv).BindInputs({input, kernel, bias}).BindOutput(output);
    auto transform = tim::transform::LayoutInference(src, ctx);
    auto infer = transform.first;
    auto io = transform.second;
    if (!infer->Compile()) return 10;
    std::vector<float> in = {1.0f, 1.0f, 1.0f, 1.0f, 0.5f, 1.0f, 1.0f, 1.0f, 1.0f};
    if (!io[src->InputsTensor()[0]]->CopyDataToTensor(in.data(), in.size() * sizeof(float))) return 11;
    if (!infer->Run()) return 12;
    auto out_t = io[src->OutputsTensor()[0]];
    if (out_t->GetShape() != output_shape) return 13;
    std::vector<float> out(4);
    if (!out_t->CopyDataFromTensor(out.data())) return 14;
    for (float v : out)
      if (v != 0.875f) return 15;
  }
  {
    auto src = ctx->CreateGraph();
    ShapeType input_shape({3, 3, 1, 1}), kernel_shape({1, 2, 2, 1}), output_shape({2, 2, 1, 1});
    auto input = src->CreateTensor(TensorSpec(DataType::FLOAT32, input_shape, TensorAttribute::INPUT));
    auto kernel = src->CreateTensor(TensorSpec(DataType::FLOAT32, kernel_shape, TensorAttribute::INPUT));
    auto bias = src->CreateTensor(TensorSpec(DataType::FLOAT32, ShapeType({1}), TensorAttribute::INPUT));
    auto output = src->CreateTensor(TensorSpec(DataType::FLOAT32, output_shape, TensorAttribute::OUTPUT));
    auto conv = src->CreateOperation<ops::Conv2d>(0, PadType::AUTO, std::array<uint32_t, 2>({0, 0}), std::array<uint32_t, 2>({1, 1}),
                                                  std::array<uint32_t, 2>({1, 1}), std::array<uint32_t, 4>({0, 0, 0, 0}), 0,
                                                  DataLayout::WHCN, DataLayout::IcWHOc);
    (*conv).BindInputs({input, kernel, bias}).BindOutput(output);
    auto transform = tim::transform::LayoutInference(src, ctx);
    auto infer = transform.first;
    auto io = transform.second;
    if (!infer->Compile()) return 20;
    std::vector<float> in = {1.0f, 1.0f, 1.0f, 1.0f, 0.5f, 1.0f, 1.0f, 1.0f, 1.0f}, k = {0.25f, 0.25f, 0.25f, 0.25f}, b = {0.0f};
    if (!io[src->InputsTensor()[0]]->CopyDataToTensor(in.data(), in.size() * 4) ||
        !io[src->InputsTensor()[1]]->CopyDataToTensor(k.data(), k.size() * 4) ||
        !io[src->InputsTensor()[2]]->CopyDataToTensor(b.data(), b.size() * 4))
      return 21;
    if (!infer->Run()) return 22;
    auto out_t = io[src->OutputsTensor()[0]];
    if (out_t->GetShape() != output_shape) return 23;
    std::vector<float> out(4);
    if (!out_t->CopyDataFromTensor(out.data())) return 24;
    for (float v : out)
      if (v != 0.875f) return 25;
  }
  return 0;
}

constexpr uint32_t W = 12, H = 10, C = 8, N = 2, OC = 16, CLASSES = 10;

struct Weights {
  std::vector<uint8_t> conv;   // IcWHOc [C, 3, 3, OC]
  std::vector<uint8_t> dw;     // IcWHOc [1, 3, 3, OC]
  std::vector<uint8_t> fc;     // [K, CLASSES] with K counted over the NHWC-flattened pooled tensor
  std::vector<int32_t> conv_b, dw_b, fc_b;
  std::vector<uint8_t> channel_offset;   // [OC]: the constant operand of an Add
};

// element (i0, i1, i2, i3) of a dense tensor with dimension 0 fastest
static size_t at4(const uint32_t d[4], uint32_t i0, uint32_t i1, uint32_t i2, uint32_t i3) {
  return ((static_cast<size_t>(i3) * d[2] + i2) * d[1] + i1) * d[0] + i0;
}

static std::vector<uint8_t> run_network(const std::shared_ptr<Context>& ctx, const Weights& wts, const std::vector<uint8_t>& image_nhwc,
                                        bool nhwc, int* transposes) {
  auto g = ctx->CreateGraph();
  const DataLayout act = nhwc ? DataLayout::CWHN : DataLayout::WHCN, ker = nhwc ? DataLayout::IcWHOc : DataLayout::WHIcOc;
  const uint32_t PW = W / 2, PH = H / 2;
  // data in the layout of this variant
  std::vector<uint8_t> image = image_nhwc, conv_w = wts.conv, dw_w = wts.dw, fc_w = wts.fc;
  if (!nhwc) {
    const uint32_t dn[4] = {C, W, H, N}, dw4[4] = {W, H, C, N};
    for (uint32_t n = 0; n < N; ++n) for (uint32_t h = 0; h < H; ++h) for (uint32_t w = 0; w < W; ++w) for (uint32_t c = 0; c < C; ++c)
      image[at4(dw4, w, h, c, n)] = image_nhwc[at4(dn, c, w, h, n)];
    const uint32_t kn[4] = {C, 3, 3, OC}, kw[4] = {3, 3, C, OC};
    for (uint32_t o = 0; o < OC; ++o) for (uint32_t y = 0; y < 3; ++y) for (uint32_t x = 0; x < 3; ++x) for (uint32_t c = 0; c < C; ++c)
      conv_w[at4(kw, x, y, c, o)] = wts.conv[at4(kn, c, x, y, o)];
    // depthwise [1, 3, 3, OC] -> [3, 3, OC, 1]
    for (uint32_t o = 0; o < OC; ++o) for (uint32_t y = 0; y < 3; ++y) for (uint32_t x = 0; x < 3; ++x)
      dw_w[(o * 3 + y) * 3 + x] = wts.dw[(o * 3 + y) * 3 + x];
    // the FullyConnected flattens [PW, PH, OC] here but [OC, PW, PH] in the NHWC variant: reorder K
    const uint32_t K = PW * PH * OC;
    for (uint32_t j = 0; j < CLASSES; ++j)
      for (uint32_t c = 0; c < OC; ++c) for (uint32_t h = 0; h < PH; ++h) for (uint32_t w = 0; w < PW; ++w)
        fc_w[j * K + (c * PH + h) * PW + w] = wts.fc[j * K + (h * PW + w) * OC + c];
  }
  auto shape = [&](uint32_t w, uint32_t h, uint32_t c) { return nhwc ? ShapeType({c, w, h, N}) : ShapeType({w, h, c, N}); };
  auto input = g->CreateTensor(TensorSpec(DataType::UINT8, shape(W, H, C), TensorAttribute::INPUT, quant(0.02f, 128)));
  auto cw = g->CreateTensor(TensorSpec(DataType::UINT8, nhwc ? ShapeType({C, 3, 3, OC}) : ShapeType({3, 3, C, OC}), TensorAttribute::CONSTANT,
                                       quant(0.01f, 125)), conv_w.data());
  auto cb = g->CreateTensor(TensorSpec(DataType::INT32, ShapeType({OC}), TensorAttribute::CONSTANT, quant(0.02f * 0.01f, 0)), wts.conv_b.data());
  auto dwt = g->CreateTensor(TensorSpec(DataType::UINT8, nhwc ? ShapeType({1, 3, 3, OC}) : ShapeType({3, 3, OC, 1}), TensorAttribute::CONSTANT,
                                        quant(0.02f, 130)), dw_w.data());
  auto db = g->CreateTensor(TensorSpec(DataType::INT32, ShapeType({OC}), TensorAttribute::CONSTANT, quant(0.05f * 0.02f, 0)), wts.dw_b.data());
  auto fw = g->CreateTensor(TensorSpec(DataType::UINT8, ShapeType({PW * PH * OC, CLASSES}), TensorAttribute::CONSTANT, quant(0.005f, 128)), fc_w.data());
  auto fb = g->CreateTensor(TensorSpec(DataType::INT32, ShapeType({CLASSES}), TensorAttribute::CONSTANT, quant(0.06f * 0.005f, 0)), wts.fc_b.data());
  auto transient = [&](float s, int32_t z) { return g->CreateTensor(TensorSpec(DataType::UINT8, {}, TensorAttribute::TRANSIENT, quant(s, z))); };
  auto t1 = transient(0.05f, 20), t2a = transient(0.05f, 20), t2 = transient(0.05f, 20), t3 = transient(0.07f, 90), t4 = transient(0.06f, 50), t5 = transient(0.06f, 50);
  auto logits = g->CreateTensor(TensorSpec(DataType::UINT8, ShapeType({CLASSES, N}), TensorAttribute::OUTPUT, quant(0.1f, 128)));
  const std::array<uint32_t, 2> one = {1, 1}, three = {3, 3}, two = {2, 2};
  const std::array<uint32_t, 4> nopad = {0, 0, 0, 0};
  auto conv = g->CreateOperation<ops::Conv2d>(static_cast<int32_t>(OC), PadType::SAME, three, one, one, nopad, 0, act, ker);
  (*conv).BindInputs({input, cw, cb}).BindOutput(t1);
  auto relu = g->CreateOperation<ops::Relu>();
  (*relu).BindInput(t1).BindOutput(t2a);
  // an elementwise op with a constant operand that has all four dimensions (one value per channel): layout
  // inference has to permute the constant together with the activation it is added to
  auto per_channel = g->CreateTensor(TensorSpec(DataType::UINT8, nhwc ? ShapeType({OC, 1, 1, 1}) : ShapeType({1, 1, OC, 1}), TensorAttribute::CONSTANT,
                                                quant(0.03f, 100)), wts.channel_offset.data());
  auto addc = g->CreateOperation<ops::Add>();
  (*addc).BindInputs({t2a, per_channel}).BindOutput(t2);
  auto dw = g->CreateOperation<ops::Conv2d>(static_cast<int32_t>(OC), PadType::SAME, three, one, one, nopad, 1, act, ker);
  (*dw).BindInputs({t2, dwt, db}).BindOutput(t3);
  auto add = g->CreateOperation<ops::Add>();
  (*add).BindInputs({t3, t2}).BindOutput(t4);
  auto pool = g->CreateOperation<ops::Pool2d>(PoolType::AVG, PadType::VALID, two, two, RoundType::FLOOR, act);
  (*pool).BindInput(t4).BindOutput(t5);
  auto fc = g->CreateOperation<ops::FullyConnected>(2, CLASSES);
  (*fc).BindInputs({t5, fw, fb}).BindOutput(logits);

  std::shared_ptr<Graph> run = g;
  std::shared_ptr<Tensor> in_t = input, out_t = logits;
  if (nhwc) {
    auto c2 = ctx;
    auto transform = tim::transform::LayoutInference(g, c2);
    run = transform.first;
    in_t = transform.second[input];
    out_t = transform.second[logits];
    int count = 0;
    for (const auto& op : run->OpVector())
      if (dynamic_cast<ops::Transpose*>(op.get())) ++count;
    if (transposes) *transposes = count;
  }
  std::vector<uint8_t> out(CLASSES * N);
  if (!run->Compile() || !in_t->CopyDataToTensor(image.data(), image.size()) || !run->Run() || !out_t->CopyDataFromTensor(out.data())) out.clear();
  return out;
}

int main() {
  const int rc = reference_cases();
  if (rc) { std::fprintf(stderr, "reference case failed at step %d\n", rc); return rc; }
  auto ctx = Context::Create();
  Weights w;
  w.conv.resize(C * 9 * OC); for (auto& v : w.conv) v = next_byte();
  w.dw.resize(9 * OC); for (auto& v : w.dw) v = next_byte();
  w.fc.resize((W / 2) * (H / 2) * OC * CLASSES); for (auto& v : w.fc) v = next_byte();
  w.conv_b.resize(OC); for (auto& v : w.conv_b) v = static_cast<int32_t>(next_byte()) * 16 - 2000;
  w.dw_b.resize(OC); for (auto& v : w.dw_b) v = static_cast<int32_t>(next_byte()) * 4 - 500;
  w.channel_offset.resize(OC); for (auto& v : w.channel_offset) v = next_byte();
  w.fc_b.resize(CLASSES); for (auto& v : w.fc_b) v = static_cast<int32_t>(next_byte()) * 8 - 1000;
  std::vector<uint8_t> image(C * W * H * N);
  for (auto& v : image) v = next_byte();
  int transposes = -1;
  const std::vector<uint8_t> native = run_network(ctx, w, image, false, nullptr);
  const std::vector<uint8_t> inferred = run_network(ctx, w, image, true, &transposes);
  if (native.empty() || inferred.empty()) { std::fprintf(stderr, "a graph failed to compile or run\n"); return 30; }
  if (native != inferred) { std::fprintf(stderr, "inferred NHWC graph differs from the native WHCN graph\n"); return 31; }
  bool varied = false;
  for (size_t i = 1; i < native.size(); ++i) varied = varied || native[i] != native[0];
  if (!varied) { std::fprintf(stderr, "constant logits\n"); return 32; }
  if (transposes != 2) { std::fprintf(stderr, "%d Transposes in the inferred graph, expected 2\n", transposes); return 33; }
  std::printf("logits");
  for (uint8_t v : native) std::printf(" %u", v);
  std::printf("\nok layout inference\n");
  return 0;
}
