// Reshape, Transpose, Concat and DataConvert through the public tim::vx headers, the way the reference's
// exported graphs use them (samples/multi_device/vx_mobilenet.cc:570-571,832-840 permute the NHWC image and
// flatten the logits; vx_resnet50.cc:1347-1349 concatenates along the channel axis):
//
//   image u8 [C=3, W=8, H=6, N=2] --Transpose{1,2,0,3}--> [W, H, C, N] --Conv2d 3x3 (3 -> 16)--+
//   side  u8 [W, H, 32, N] (other scale) ------------------------------------------------------+--Concat axis 2
//   --> [W, H, 48, N] --Reshape--> [W*H*48, N] --DataConvert--> float32 [W*H*48, N]
//
// The program checks the result against its own straightforward loops for everything but the
// convolution (whose bytes it reads back through a second output), then serialises the graph
// (CompileToBinary), reloads it through ops::NBG and requires the same bytes.  It prints
// "out <checksum> <first values>" so that two builds (CPU oracle, CUDA) can be compared, and exits
// non-zero on any mismatch.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <vector>

#include "tim/vx/context.h"
#include "tim/vx/graph.h"
#include "tim/vx/ops.h"
#include "tim/vx/tensor.h"

using namespace tim::vx;

static uint32_t lcg_state = 77;
static uint8_t next_byte() {
  lcg_state = lcg_state * 1664525u + 1013904223u;
  return static_cast<uint8_t>(lcg_state >> 24);
}
static Quantization quant(float s, int32_t z) { return Quantization(QuantType::ASYMMETRIC, s, z); }

constexpr uint32_t W = 8, H = 6, C = 3, N = 2, OC = 16, SIDE = 32;
constexpr float kConvScale = 0.05f, kSideScale = 0.031f, kCatScale = 0.04f;
constexpr int32_t kConvZp = 7, kSideZp = 120, kCatZp = 60;

struct Built {
  std::shared_ptr<Graph> graph;
  std::shared_ptr<Tensor> image, side, conv_out, result;
};

static Built build(const std::shared_ptr<Context>& context) {
  Built b;
  b.graph = context->CreateGraph();
  auto& g = b.graph;
  b.image = g->CreateTensor(TensorSpec(DataType::UINT8, {C, W, H, N}, TensorAttribute::INPUT, quant(0.02f, 128)));
  b.side = g->CreateTensor(TensorSpec(DataType::UINT8, {W, H, SIDE, N}, TensorAttribute::INPUT, quant(kSideScale, kSideZp)));
  auto whcn = g->CreateTensor(TensorSpec(DataType::UINT8, {}, TensorAttribute::TRANSIENT, quant(0.02f, 128)));
  std::vector<uint8_t> wdata(3 * 3 * C * OC);
  for (auto& v : wdata) v = next_byte();
  auto weight = g->CreateTensor(TensorSpec(DataType::UINT8, {3, 3, C, OC}, TensorAttribute::CONSTANT, quant(0.01f, 131)), wdata.data());
  std::vector<int32_t> bdata(OC);
  for (auto& v : bdata) v = static_cast<int32_t>(next_byte()) * 8 - 1000;
  auto bias = g->CreateTensor(TensorSpec(DataType::INT32, {OC}, TensorAttribute::CONSTANT, quant(0.02f * 0.01f, 0)), bdata.data());
  // the convolution's result is also a graph output, so that the program can read its bytes
  b.conv_out = g->CreateTensor(TensorSpec(DataType::UINT8, {W, H, OC, N}, TensorAttribute::OUTPUT, quant(kConvScale, kConvZp)));
  auto cat = g->CreateTensor(TensorSpec(DataType::UINT8, {}, TensorAttribute::TRANSIENT, quant(kCatScale, kCatZp)));
  auto flat = g->CreateTensor(TensorSpec(DataType::UINT8, {}, TensorAttribute::TRANSIENT, quant(kCatScale, kCatZp)));
  b.result = g->CreateTensor(TensorSpec(DataType::FLOAT32, {W * H * (OC + SIDE), N}, TensorAttribute::OUTPUT));

  auto transpose = g->CreateOperation<ops::Transpose>(std::vector<uint32_t>{1, 2, 0, 3});
  (*transpose).BindInput(b.image).BindOutput(whcn);
  auto conv = g->CreateOperation<ops::Conv2d>(PadType::SAME, std::array<uint32_t, 2>{1, 1}, std::array<uint32_t, 2>{1, 1});
  (*conv).BindInputs({whcn, weight, bias}).BindOutput(b.conv_out);
  auto concat = g->CreateOperation<ops::Concat>(2, 2);
  (*concat).BindInputs({b.conv_out, b.side}).BindOutput(cat);
  auto reshape = g->CreateOperation<ops::Reshape>(std::vector<uint32_t>{W * H * (OC + SIDE), N});
  (*reshape).BindInput(cat).BindOutput(flat);
  auto convert = g->CreateOperation<ops::DataConvert>();
  (*convert).BindInput(flat).BindOutput(b.result);
  return b;
}

// fp32_to_affine of the reference for in-range values: round half to even, add the zero point, clamp
static uint8_t requant(float real, float scale, int32_t zp) {
  const float q = std::nearbyintf(real / scale) + static_cast<float>(zp);
  return static_cast<uint8_t>(q < 0.0f ? 0.0f : (q > 255.0f ? 255.0f : q));
}

int main() {
  auto context = Context::Create();
  Built b = build(context);
  std::vector<uint8_t> image(C * W * H * N), side(W * H * SIDE * N);
  for (auto& v : image) v = next_byte();
  for (auto& v : side) v = next_byte();
  if (!b.graph->Compile()) { std::fprintf(stderr, "compile failed\n"); return 1; }
  if (!b.image->CopyDataToTensor(image.data(), image.size()) || !b.side->CopyDataToTensor(side.data(), side.size())) return 2;
  if (!b.graph->Run()) { std::fprintf(stderr, "run failed\n"); return 3; }
  std::vector<uint8_t> conv(W * H * OC * N);
  std::vector<float> got(W * H * (OC + SIDE) * N);
  if (!b.conv_out->CopyDataFromTensor(conv.data()) || !b.result->CopyDataFromTensor(got.data())) return 4;

  // expectation from the convolution's bytes: concat along the channel axis with requantization of both
  // operands, flattened in WHCN order, dequantized
  size_t bad = 0;
  for (uint32_t n = 0; n < N; ++n)
    for (uint32_t c = 0; c < OC + SIDE; ++c)
      for (uint32_t h = 0; h < H; ++h)
        for (uint32_t w = 0; w < W; ++w) {
          float real;
          if (c < OC) real = (static_cast<float>(conv[((n * OC + c) * H + h) * W + w]) - static_cast<float>(kConvZp)) * kConvScale;
          else real = (static_cast<float>(side[((n * SIDE + (c - OC)) * H + h) * W + w]) - static_cast<float>(kSideZp)) * kSideScale;
          const uint8_t q = requant(real, kCatScale, kCatZp);
          const float want = (static_cast<float>(q) - static_cast<float>(kCatZp)) * kCatScale;
          const float have = got[((n * (OC + SIDE) + c) * H + h) * W + w];
          if (want != have) ++bad;
        }
  if (bad) { std::fprintf(stderr, "%zu elements differ from the expectation\n", bad); return 5; }
  // the convolution must have seen the transposed image: a constant output would mean it did not
  bool varied = false;
  for (size_t i = 1; i < conv.size(); ++i) varied = varied || conv[i] != conv[0];
  if (!varied) { std::fprintf(stderr, "convolution output is constant\n"); return 6; }

  // serialise, reload through ops::NBG, same bytes
  size_t bytes = 0;
  if (!b.graph->CompileToBinary(nullptr, &bytes) || bytes == 0) return 7;
  std::vector<char> blob(bytes);
  if (!b.graph->CompileToBinary(blob.data(), &bytes)) return 8;
  auto g2 = context->CreateGraph();
  auto in0 = g2->CreateTensor(b.image->GetSpec());
  auto in1 = g2->CreateTensor(b.side->GetSpec());
  auto out0 = g2->CreateTensor(b.conv_out->GetSpec());
  auto out1 = g2->CreateTensor(b.result->GetSpec());
  auto nbg = g2->CreateOperation<ops::NBG>(blob.data(), 2, 2);
  (*nbg).BindInputs({in0, in1}).BindOutputs({out0, out1});
  if (!g2->Compile()) { std::fprintf(stderr, "reloaded graph failed to compile\n"); return 9; }
  if (!in0->CopyDataToTensor(image.data(), image.size()) || !in1->CopyDataToTensor(side.data(), side.size()) || !g2->Run()) return 10;
  std::vector<float> again(got.size());
  if (!out1->CopyDataFromTensor(again.data())) return 11;
  if (std::memcmp(again.data(), got.data(), got.size() * sizeof(float)) != 0) { std::fprintf(stderr, "reloaded graph differs\n"); return 12; }

  uint32_t sum = 0;
  for (uint8_t v : conv) sum = sum * 31u + v;
  for (float v : got) { uint32_t u; std::memcpy(&u, &v, 4); sum = sum * 31u + u; }
  std::printf("out %08x", sum);
  for (int i = 0; i < 8; ++i) std::printf(" %.4f", got[i * 97]);
  std::printf("\nok movement ops\n");
  return 0;
}
