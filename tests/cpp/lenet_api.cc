// LeNet-5 written against the public tim::vx headers only, the way user code
// of the reference is written (compare samples/lenet/lenet_asymu8.cc:115-317):
// Context::Create, CreateGraph, CreateTensor with TensorSpec/Quantization,
// CreateOperation<Op>(...).BindInputs(...).BindOutputs(...), Compile,
// CopyDataToTensor, Run, CopyDataFromTensor.  Weights and the input image are
// seeded pseudo-random bytes.  Prints the uint8 logits and the float32
// probabilities of each image, one line per image, so that two builds (CPU
// oracle, CUDA) can be compared textually.
#include <array>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "tim/vx/context.h"
#include "tim/vx/graph.h"
#include "tim/vx/operation.h"
#include "tim/vx/ops/activations.h"
#include "tim/vx/ops/conv2d.h"
#include "tim/vx/ops/fullyconnected.h"
#include "tim/vx/ops/pool2d.h"
#include "tim/vx/ops/softmax.h"
#include "tim/vx/tensor.h"

static uint32_t lcg_state = 12345;
static uint8_t next_byte() {
  lcg_state = lcg_state * 1664525u + 1013904223u;
  return static_cast<uint8_t>(lcg_state >> 24);
}

int main(int argc, char** argv) {
  const uint32_t batch = argc > 1 ? static_cast<uint32_t>(std::atoi(argv[1])) : 2;
  using namespace tim::vx;
  auto context = Context::Create();
  auto graph = context->CreateGraph();

  auto quant = [](float s, int32_t z) { return Quantization(QuantType::ASYMMETRIC, s, z); };
  auto weights = [&](const ShapeType& shape, float s, int32_t z) {
    TensorSpec spec(DataType::UINT8, shape, TensorAttribute::CONSTANT, quant(s, z));
    std::vector<uint8_t> data(static_cast<size_t>(spec.GetElementNum()));
    for (auto& v : data) v = next_byte();
    return graph->CreateTensor(spec, data.data());
  };
  auto bias = [&](uint32_t n, float s) {
    TensorSpec spec(DataType::INT32, {n}, TensorAttribute::CONSTANT, quant(s, 0));
    std::vector<int32_t> data(n);
    for (auto& v : data) v = static_cast<int32_t>(next_byte()) * 8 - 1000;
    return graph->CreateTensor(spec, data.data());
  };
  auto transient = [&](float s, int32_t z) {
    return graph->CreateTensor(TensorSpec(DataType::UINT8, {}, TensorAttribute::TRANSIENT, quant(s, z)));
  };

  const float s_in = 1.0f / 255.0f;
  auto input = graph->CreateTensor(TensorSpec(DataType::UINT8, {28, 28, 1, batch}, TensorAttribute::INPUT, quant(s_in, 0)));
  auto w1 = weights({5, 5, 1, 20}, 0.004f, 120);
  auto b1 = bias(20, s_in * 0.004f);
  auto c1 = transient(0.02f, 140), p1 = transient(0.02f, 140);
  auto w2 = weights({5, 5, 20, 50}, 0.0012f, 128);
  auto b2 = bias(50, 0.02f * 0.0012f);
  auto c2 = transient(0.04f, 141), p2 = transient(0.04f, 141);
  auto w3 = weights({800, 500}, 0.0007f, 130);
  auto b3 = bias(500, 0.04f * 0.0007f);
  auto f3 = transient(0.02f, 0), r3 = transient(0.02f, 0);
  auto w4 = weights({500, 10}, 0.0016f, 135);
  auto b4 = bias(10, 0.02f * 0.0016f);
  auto logits = graph->CreateTensor(TensorSpec(DataType::UINT8, {10, batch}, TensorAttribute::OUTPUT, quant(0.06f, 80)));
  auto prob = graph->CreateTensor(TensorSpec(DataType::FLOAT32, {10, batch}, TensorAttribute::OUTPUT));

  auto conv1 = graph->CreateOperation<ops::Conv2d>(20, PadType::VALID, std::array<uint32_t, 2>({5, 5}),
                                                   std::array<uint32_t, 2>({1, 1}), std::array<uint32_t, 2>({1, 1}));
  (*conv1).BindInputs({input, w1, b1}).BindOutputs({c1});
  auto pool1 = graph->CreateOperation<ops::Pool2d>(PoolType::MAX, PadType::NONE, std::array<uint32_t, 2>({2, 2}),
                                                   std::array<uint32_t, 2>({2, 2}));
  (*pool1).BindInputs({c1}).BindOutputs({p1});
  auto conv2 = graph->CreateOperation<ops::Conv2d>(50, PadType::VALID, std::array<uint32_t, 2>({5, 5}),
                                                   std::array<uint32_t, 2>({1, 1}), std::array<uint32_t, 2>({1, 1}));
  (*conv2).BindInputs({p1, w2, b2}).BindOutputs({c2});
  auto pool2 = graph->CreateOperation<ops::Pool2d>(PoolType::MAX, PadType::NONE, std::array<uint32_t, 2>({2, 2}),
                                                   std::array<uint32_t, 2>({2, 2}));
  (*pool2).BindInputs({c2}).BindOutputs({p2});
  auto fc3 = graph->CreateOperation<ops::FullyConnected>(2, 500);
  (*fc3).BindInputs({p2, w3, b3}).BindOutputs({f3});
  auto relu = graph->CreateOperation<ops::Relu>();
  (*relu).BindInput(f3).BindOutput(r3);
  auto fc4 = graph->CreateOperation<ops::FullyConnected>(0, 10);
  (*fc4).BindInputs({r3, w4, b4}).BindOutputs({logits});
  auto softmax = graph->CreateOperation<ops::Softmax>(1.0f, 0);
  (*softmax).BindInput(logits).BindOutput(prob);

  if (!graph->Compile()) { std::printf("Compile failed\n"); return 1; }
  if (c1->GetShape() != ShapeType({24, 24, 20, batch})) { std::printf("shape inference failed\n"); return 1; }
  std::vector<uint8_t> image(28 * 28 * batch);
  for (auto& v : image) v = next_byte();
  if (!input->CopyDataToTensor(image.data(), static_cast<uint32_t>(image.size()))) { std::printf("copy in failed\n"); return 1; }
  if (!graph->Run()) { std::printf("Run failed\n"); return 1; }
  std::vector<uint8_t> q(10 * batch);
  std::vector<float> pr(10 * batch);
  if (!logits->CopyDataFromTensor(q.data()) || !prob->CopyDataFromTensor(pr.data())) { std::printf("copy out failed\n"); return 1; }
  for (uint32_t n = 0; n < batch; ++n) {
    std::printf("logits");
    for (int i = 0; i < 10; ++i) std::printf(" %u", q[n * 10 + i]);
    std::printf(" prob");
    for (int i = 0; i < 10; ++i) std::printf(" %.5f", pr[n * 10 + i]);
    std::printf("\n");
  }
  return 0;
}
