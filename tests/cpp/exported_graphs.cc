// Runs the three graphs the reference ships as generated source (samples/multi_device/vx_lenet.cc,
// vx_mobilenet.cc, vx_resnet50.cc: acuitylite::<net>::construct_graph), compiled unmodified from the reference
// tree and linked with this driver (oracle/Makefile, target ref-samples).  samples/multi_device/multi_device.cc
// itself wants all three coefficient files; the tree holds only LeNet's, so this driver calls the constructors
// directly: LeNet with its real coefficients and digit image, the other two with seeded stand-in coefficient
// files of the length their constructors read (oracle/make_export_blobs.py) and the reference's input images.
//
// usage: exported_graphs <directory with lenet.export.data, lenet_input_1_1_28_28_uint8.bin, mobilenet.export.data,
//        mobilenet_1_224_224_3_uint8.bin, resnet50.export.data, resnet50_1_3_224_224_uint8.bin>
// Prints, per network, the output size, a hash of the output bytes, the best class and its probability.
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <functional>
#include <string>
#include <vector>

#include "tim/vx/context.h"
#include "tim/vx/graph.h"
#include "tim/vx/tensor.h"
#include "vx_lenet.h"
#include "vx_mobilenet.h"
#include "vx_resnet50.h"

static std::vector<char> slurp(const std::string& path) {
  std::ifstream f(path, std::ios::binary);
  return std::vector<char>((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
}

static int run_one(const char* name, const std::function<void(std::shared_ptr<tim::vx::Graph>, const char*)>& construct,
                   std::vector<std::shared_ptr<tim::vx::Tensor>>& inputs, std::vector<std::shared_ptr<tim::vx::Tensor>>& outputs,
                   const std::string& coef, const std::string& image) {
  auto ctx = tim::vx::Context::Create();
  auto graph = ctx->CreateGraph();
  inputs.clear();
  outputs.clear();
  construct(graph, coef.c_str());
  if (inputs.empty() || outputs.empty()) { std::fprintf(stderr, "%s: constructor bound no input or output\n", name); return 1; }
  if (!graph->Compile()) { std::fprintf(stderr, "%s: Compile failed\n", name); return 2; }
  std::vector<char> in = slurp(image);
  if (in.size() != inputs[0]->GetSpec().GetByteSize()) {
    std::fprintf(stderr, "%s: input file has %zu bytes, the tensor %zu\n", name, in.size(), static_cast<size_t>(inputs[0]->GetSpec().GetByteSize()));
    return 3;
  }
  if (!inputs[0]->CopyDataToTensor(in.data(), static_cast<uint32_t>(in.size()))) return 4;
  if (!graph->Run()) { std::fprintf(stderr, "%s: Run failed\n", name); return 5; }
  const size_t bytes = outputs[0]->GetSpec().GetByteSize();
  std::vector<float> out(bytes / sizeof(float));
  if (!outputs[0]->CopyDataFromTensor(out.data())) return 6;
  uint64_t h = 1469598103934665603ull;   // FNV-1a over the output bytes
  const unsigned char* p = reinterpret_cast<const unsigned char*>(out.data());
  for (size_t i = 0; i < bytes; ++i) { h ^= p[i]; h *= 1099511628211ull; }
  size_t best = 0;
  for (size_t i = 1; i < out.size(); ++i)
    if (out[i] > out[best]) best = i;
  std::printf("%s: %zu outputs, hash %016llx, top-1 class %zu, probability %.6f\n", name, out.size(), static_cast<unsigned long long>(h), best,
              static_cast<double>(out[best]));
  return 0;
}

int main(int argc, char** argv) {
  if (argc < 2) { std::fprintf(stderr, "usage: %s <data directory>\n", argv[0]); return 64; }
  const std::string d = std::string(argv[1]) + "/";
  int rc = run_one("lenet", acuitylite::lenet::construct_graph, acuitylite::lenet::inputs_tensor, acuitylite::lenet::outputs_tensor,
                   d + "lenet.export.data", d + "lenet_input_1_1_28_28_uint8.bin");
  if (rc) return rc;
  rc = run_one("mobilenet", acuitylite::mobilenet::construct_graph, acuitylite::mobilenet::inputs_tensor, acuitylite::mobilenet::outputs_tensor,
               d + "mobilenet.export.data", d + "mobilenet_1_224_224_3_uint8.bin");
  if (rc) return 10 + rc;
  rc = run_one("resnet50", acuitylite::resnet50::construct_graph, acuitylite::resnet50::inputs_tensor, acuitylite::resnet50::outputs_tensor,
               d + "resnet50.export.data", d + "resnet50_1_3_224_224_uint8.bin");
  if (rc) return 20 + rc;
  std::printf("ok exported graphs\n");
  return 0;
}
