// The platform surface (tim/vx/platform/platform.h) the way the reference's multi-device sample uses
// it (compare samples/lenet_multi_device/lenet_multi_device.cc:120-178): a small quantized network with
// a residual Add is built once; its output through Graph::Run is the yardstick; then for every
// enumerated device an executor compiles the graph into an executable, tensors are allocated from
// it, and the executable runs through the executor's queue.  Also checked: the size query of
// CompileToBinary, loading the blob by hand into a graph with an ops::NBG node, and queue order with
// two executables.  Prints "device <i> <bytes...>" lines (so two builds can be compared) and exits
// non-zero on any mismatch.
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <vector>

#include "tim/vx/context.h"
#include "tim/vx/graph.h"
#include "tim/vx/ops/activations.h"
#include "tim/vx/ops/conv2d.h"
#include "tim/vx/ops/elementwise.h"
#include "tim/vx/ops/fullyconnected.h"
#include "tim/vx/ops/nbg.h"
#include "tim/vx/ops/pool2d.h"
#include "tim/vx/platform/native.h"
#include "tim/vx/platform/platform.h"
#include "tim/vx/tensor.h"

using namespace tim::vx;

static uint32_t lcg_state = 2024;
static uint8_t next_byte() {
  lcg_state = lcg_state * 1664525u + 1013904223u;
  return static_cast<uint8_t>(lcg_state >> 24);
}

static Quantization quant(float s, int32_t z) { return Quantization(QuantType::ASYMMETRIC, s, z); }

// conv3x3(16->32)+relu -> conv1x1(32->32) -> add(skip) -> relu -> maxpool2 -> fc(10)
static std::shared_ptr<Graph> build(const std::shared_ptr<Context>& context, uint32_t batch) {
  auto graph = context->CreateGraph();
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
  auto x = graph->CreateTensor(TensorSpec(DataType::UINT8, {12, 12, 16, batch}, TensorAttribute::INPUT, quant(0.02f, 0)));
  auto w1 = weights({3, 3, 16, 32}, 0.004f, 131);
  auto b1 = bias(32, 0.02f * 0.004f);
  auto t1 = transient(0.05f, 0), r1 = transient(0.05f, 0);
  auto w2 = weights({1, 1, 32, 32}, 0.006f, 125);
  auto b2 = bias(32, 0.05f * 0.006f);
  auto t2 = transient(0.07f, 120), s2 = transient(0.09f, 0), r2 = transient(0.09f, 0), p2 = transient(0.09f, 0);
  auto w3 = weights({6 * 6 * 32, 10}, 0.003f, 128);
  auto b3 = bias(10, 0.09f * 0.003f);
  auto y = graph->CreateTensor(TensorSpec(DataType::UINT8, {10, batch}, TensorAttribute::OUTPUT, quant(0.2f, 128)));
  const std::array<uint32_t, 2> one = {1, 1}, two = {2, 2};
  graph->CreateOperation<ops::Conv2d>(PadType::SAME, one, one)->BindInputs({x, w1, b1}).BindOutputs({t1});
  graph->CreateOperation<ops::Relu>()->BindInput(t1).BindOutput(r1);
  graph->CreateOperation<ops::Conv2d>(PadType::VALID, one, one)->BindInputs({r1, w2, b2}).BindOutputs({t2});
  graph->CreateOperation<ops::Add>()->BindInputs({t2, r1}).BindOutputs({s2});
  graph->CreateOperation<ops::Relu>()->BindInput(s2).BindOutput(r2);
  graph->CreateOperation<ops::Pool2d>(PoolType::MAX, PadType::VALID, two, two)->BindInput(r2).BindOutput(p2);
  graph->CreateOperation<ops::FullyConnected>(2, 10)->BindInputs({p2, w3, b3}).BindOutputs({y});
  return graph;
}

static void print_row(const char* tag, size_t idx, const std::vector<uint8_t>& v) {
  std::printf("%s %zu", tag, idx);
  for (uint8_t b : v) std::printf(" %u", b);
  std::printf("\n");
}

int main() {
  const uint32_t batch = 3;
  auto context = Context::Create();
  auto graph = build(context, batch);
  std::vector<uint8_t> input(12 * 12 * 16 * batch), input2(input.size());
  for (auto& v : input) v = next_byte();
  for (auto& v : input2) v = next_byte();

  // 1. the yardstick: the graph itself
  std::vector<uint8_t> want(10 * batch), want2(10 * batch);
  if (!graph->Compile()) return std::fprintf(stderr, "graph does not compile\n"), 1;
  graph->InputsTensor()[0]->CopyDataToTensor(input.data(), static_cast<uint32_t>(input.size()));
  if (!graph->Run() || !graph->OutputsTensor()[0]->CopyDataFromTensor(want.data())) return 2;
  graph->InputsTensor()[0]->CopyDataToTensor(input2.data(), static_cast<uint32_t>(input2.size()));
  if (!graph->Run() || !graph->OutputsTensor()[0]->CopyDataFromTensor(want2.data())) return 2;
  print_row("graph", 0, want);

  // 2. serialise; size query first
  size_t bytes = 0;
  if (!graph->CompileToBinary(nullptr, &bytes) || bytes == 0) return std::fprintf(stderr, "size query failed\n"), 3;
  std::vector<char> blob(bytes);
  size_t too_small = bytes - 1;
  std::vector<char> small(too_small);
  if (graph->CompileToBinary(small.data(), &too_small)) return std::fprintf(stderr, "short buffer accepted\n"), 3;
  if (!graph->CompileToBinary(blob.data(), &bytes)) return 3;

  // 3. load by hand: a fresh graph with one NBG node
  {
    auto g2 = context->CreateGraph();
    auto in = g2->CreateTensor(graph->InputsTensor()[0]->GetSpec());
    auto out = g2->CreateTensor(graph->OutputsTensor()[0]->GetSpec());
    g2->CreateOperation<ops::NBG>(blob.data(), 1, 1)->BindInput(in).BindOutput(out);
    std::vector<uint8_t> got(want.size());
    if (!g2->Compile()) return std::fprintf(stderr, "NBG graph does not compile\n"), 4;
    in->CopyDataToTensor(input.data(), static_cast<uint32_t>(input.size()));
    if (!g2->Run() || !out->CopyDataFromTensor(got.data())) return 4;
    if (got != want) return std::fprintf(stderr, "NBG graph output differs\n"), 4;
    size_t again = 0;
    if (g2->CompileToBinary(nullptr, &again)) return std::fprintf(stderr, "re-serialising an NBG graph must fail\n"), 4;
  }

  // 4. every device through the platform interfaces
  auto devices = platform::IDevice::Enumerate();
  if (devices.empty()) return std::fprintf(stderr, "no device enumerated\n"), 5;
  for (size_t d = 0; d < devices.size(); ++d) {
    if (devices[d]->Id() != d || devices[d]->CoreCount() < 1) return 5;
    auto executor = devices[d]->CreateExecutor();
    auto exe_a = platform::Compile(graph, executor);
    auto exe_b = executor->Compile(graph);
    if (!exe_a || !exe_b) return std::fprintf(stderr, "platform compile failed\n"), 6;
    auto in_a = exe_a->AllocateTensor(graph->InputsTensor()[0]->GetSpec());
    auto out_a = exe_a->AllocateTensor(graph->OutputsTensor()[0]->GetSpec());
    auto in_b = exe_b->AllocateTensor(graph->InputsTensor()[0]->GetSpec());
    auto out_b = exe_b->AllocateTensor(graph->OutputsTensor()[0]->GetSpec());
    exe_a->SetInput(in_a);
    exe_a->SetOutput(out_a);
    exe_b->SetInputs({in_b});
    exe_b->SetOutputs({out_b});
    in_a->CopyDataToTensor(input.data(), static_cast<uint32_t>(input.size()));
    in_b->CopyDataToTensor(input2.data(), static_cast<uint32_t>(input2.size()));
    // queue: b first, then a in front of it; an executable that is not queued cannot be a reference
    if (!exe_b->Submit(exe_b)) return 7;
    if (!exe_a->Submit(exe_b, false)) return 7;
    auto exe_c = executor->Compile(graph);
    if (executor->Submit(exe_b, exe_c, true)) return std::fprintf(stderr, "submit after an unqueued reference succeeded\n"), 7;
    if (!executor->Trigger()) return 8;
    std::vector<uint8_t> got_a(want.size()), got_b(want.size());
    if (!out_a->CopyDataFromTensor(got_a.data()) || !out_b->CopyDataFromTensor(got_b.data())) return 8;
    if (got_a != want || got_b != want2) return std::fprintf(stderr, "device %zu: executable output differs from the graph's\n", d), 9;
    print_row("device", d, got_a);
  }
  std::printf("ok %zu devices\n", devices.size());
  return 0;
}
