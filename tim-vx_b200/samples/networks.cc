// Synthetic networks on the tim::vx API (see networks.h).
//
// Quantization parameters are chosen analytically so that activations keep a
// usable spread without a calibration pass: the builder tracks estimates of
// the mean and mean square of each activation's real values, sets every
// layer's output scale to a few standard deviations per 255 steps, and gives
// each output channel the bias that cancels the expected accumulator (the
// role batch-norm folding plays in a trained network) plus seeded noise.
#include "networks.h"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "tim/vx/context.h"
#include "tim/vx/compile_option.h"
#include "tim/vx/graph.h"
#include "tim/vx/ops.h"
#include "tim/vx/tensor.h"

using namespace tim::vx;

extern "C" void* timvx_graph_backend_handle(tim::vx::Graph* graph);

namespace {

// splitmix64: counter-based, identical on every platform.
struct Rng {
  uint64_t s;
  explicit Rng(uint64_t seed) : s(seed * 0x9E3779B97F4A7C15ull + 0x1234567ull) {}
  uint64_t next() {
    uint64_t z = (s += 0x9E3779B97F4A7C15ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
  }
  int range(int lo, int hi) { return lo + static_cast<int>(next() % static_cast<uint64_t>(hi - lo + 1)); }
  float uniform(float lo, float hi) { return lo + (hi - lo) * static_cast<float>((next() >> 11) * (1.0 / 9007199254740992.0)); }
};

struct Act {
  std::shared_ptr<Tensor> t;
  float scale;
  int zp;
  double ms;       // estimate of E[real^2]
  double mean;     // estimate of E[real]
  uint32_t W, H, C;
};

}  // namespace

struct b2vx_net {
  std::shared_ptr<Context> ctx;
  std::shared_ptr<Graph> graph;
  std::shared_ptr<Tensor> input, output;
  std::vector<std::shared_ptr<Tensor>> keep;
  uint32_t W = 0, H = 0, C = 0, batch = 0, classes = 0;
  uint64_t macs = 0;
  Rng rng{1};
  enum WeightKind { S8_PER_CHANNEL, U8_ZP128, U8_ASYM } wkind = S8_PER_CHANNEL;

  // uint8 weights of one layer, [oc][per_oc]: with zero point 128 plain uniform bytes; otherwise every
  // channel is drawn in mirrored pairs (w, 2*zw - w) from the widest range symmetric about the zero
  // point, so that a channel's weights sum to zero in the real domain (what a trained, batch-norm
  // folded layer roughly has) and the accumulator does not depend on the input's mean.  Returns the
  // variance of one (w - zw).
  double fill_u8_weights(std::vector<uint8_t>& wd, size_t oc, size_t per_oc, int zw, bool plain) {
    if (plain) {
      for (auto& v : wd) v = static_cast<uint8_t>(rng.range(0, 255));
      return (256.0 * 256.0 - 1.0) / 12.0;
    }
    const int half = std::min(zw, 255 - zw);
    for (size_t i = 0; i < oc; ++i) {
      uint8_t* row = wd.data() + i * per_oc;
      size_t k = 0;
      for (; k + 1 < per_oc; k += 2) {
        const int d = rng.range(-half, half);
        row[k] = static_cast<uint8_t>(zw + d);
        row[k + 1] = static_cast<uint8_t>(zw - d);
      }
      if (k < per_oc) row[k] = static_cast<uint8_t>(zw);
      // shuffle so that mirrored values are not neighbours
      for (size_t j = per_oc; j > 1; --j) std::swap(row[j - 1], row[static_cast<size_t>(rng.next() % j)]);
    }
    const double n = 2.0 * half + 1.0;
    return (n * n - 1.0) / 12.0;
  }

  std::shared_ptr<Tensor> transient(float scale, int zp) {
    Quantization q(QuantType::ASYMMETRIC, scale, zp);
    TensorSpec spec(DataType::UINT8, {}, TensorAttribute::TRANSIENT, q);
    auto t = graph->CreateTensor(spec);
    keep.push_back(t);
    return t;
  }

  // Convolution (dense, or depthwise when multiplier == 1) with seeded weights.
  // act: 0 none (output zero point 128), 1 relu, 6 relu6 — for 1 and 6 the
  // conv output and the activation output share quantization with zero point 0.
  Act conv(const Act& x, uint32_t k, uint32_t oc, uint32_t stride, int act, bool depthwise = false,
           std::shared_ptr<Tensor> out_override = nullptr, float* out_scale_io = nullptr) {
    const uint32_t ic = x.C;
    const uint32_t fan_in = depthwise ? k * k : k * k * ic;
    std::vector<uint32_t> wshape = depthwise ? std::vector<uint32_t>{k, k, oc, 1} : std::vector<uint32_t>{k, k, ic, oc};
    const size_t wcount = static_cast<size_t>(k) * k * (depthwise ? oc : static_cast<size_t>(ic) * oc);
    std::shared_ptr<Tensor> w, b;
    double w_var;   // variance of one real weight around its mean
    std::vector<int32_t> bias(oc);
    const size_t per_oc = wcount / oc;
    const double mean_xq = x.mean / x.scale;   // expected (q - zero point) of the input
    if (wkind == S8_PER_CHANNEL) {
      std::vector<float> ws(oc), bs(oc);
      std::vector<int32_t> zeros(oc, 0);
      // U(0.001,0.01) per channel, rescaled by fan-in so accumulators stay in range
      const float shrink = 1.0f / std::sqrt(static_cast<float>(fan_in) / 64.0f);
      double s2 = 0;
      for (uint32_t i = 0; i < oc; ++i) {
        ws[i] = rng.uniform(0.001f, 0.01f) * shrink;
        bs[i] = x.scale * ws[i];
        s2 += static_cast<double>(ws[i]) * ws[i];
      }
      std::vector<int8_t> wd(wcount);
      for (auto& v : wd) v = static_cast<int8_t>(rng.range(-127, 127));
      for (uint32_t i = 0; i < oc; ++i) {
        long long sum = 0;
        for (size_t k = 0; k < per_oc; ++k) sum += wd[i * per_oc + k];
        bias[i] = static_cast<int32_t>(std::llround(-mean_xq * static_cast<double>(sum))) + rng.range(-1000, 1000);
      }
      Quantization wq(QuantType::SYMMETRIC_PER_CHANNEL, depthwise ? 2 : 3, ws, zeros);
      Quantization bq(QuantType::SYMMETRIC_PER_CHANNEL, 0, bs, zeros);
      w = graph->CreateTensor(TensorSpec(DataType::INT8, wshape, TensorAttribute::CONSTANT, wq), wd.data());
      b = graph->CreateTensor(TensorSpec(DataType::INT32, {oc}, TensorAttribute::CONSTANT, bq), bias.data());
      w_var = (s2 / oc) * (127.0 * 128.0 / 3.0);   // uniform integer in [-127,127]
    } else {
      const int zw = wkind == U8_ZP128 ? 128 : rng.range(100, 156);
      const float sw = wkind == U8_ZP128 ? 0.01f : rng.uniform(0.005f, 0.05f) / std::sqrt(static_cast<float>(fan_in) / 16.0f);
      std::vector<uint8_t> wd(wcount);
      const double q_var = fill_u8_weights(wd, oc, per_oc, zw, wkind == U8_ZP128);
      for (uint32_t i = 0; i < oc; ++i) {
        long long sum = 0;
        for (size_t k = 0; k < per_oc; ++k) sum += static_cast<int>(wd[i * per_oc + k]) - zw;
        bias[i] = static_cast<int32_t>(std::llround(-mean_xq * static_cast<double>(sum))) + rng.range(-1000, 1000);
      }
      Quantization wq(QuantType::ASYMMETRIC, sw, zw);
      Quantization bq(QuantType::ASYMMETRIC, x.scale * sw, 0);
      w = graph->CreateTensor(TensorSpec(DataType::UINT8, wshape, TensorAttribute::CONSTANT, wq), wd.data());
      b = graph->CreateTensor(TensorSpec(DataType::INT32, {oc}, TensorAttribute::CONSTANT, bq), bias.data());
      w_var = static_cast<double>(sw) * sw * q_var;
    }
    keep.push_back(w);
    keep.push_back(b);
    // with the mean cancelled by the bias, the accumulator is roughly N(0, fan_in * E[x^2] * var(w))
    const double var = static_cast<double>(fan_in) * x.ms * w_var;
    const float sigma = static_cast<float>(std::sqrt(std::max(var, 1e-12)));
    float s_out;
    int z_out;
    double ms_out, mean_out;
    if (act == 0) { s_out = 6.0f * sigma / 255.0f; z_out = 128; ms_out = var; mean_out = 0.0; }
    else if (act == 1) { s_out = 3.0f * sigma / 255.0f; z_out = 0; ms_out = var / 2; mean_out = 0.3989 * sigma; }
    else { s_out = std::min(3.0f * sigma, 6.0f) / 255.0f; z_out = 0; ms_out = std::min(var / 2, 12.0); mean_out = std::min(0.3989 * sigma, 2.0); }
    if (out_scale_io && *out_scale_io > 0) s_out = *out_scale_io;
    if (out_scale_io) *out_scale_io = s_out;

    const uint32_t pad_total = k - 1;   // "SAME"-style explicit padding: front = total/2, odd element at the end for stride 2
    uint32_t pl = pad_total / 2, pr = pad_total - pl;
    if (stride == 2 && k > 1) { pl = (k - 1) / 2; pr = (k - 1) / 2; }
    const uint32_t Wo = (x.W + pl + pr - k) / stride + 1, Ho = (x.H + pl + pr - k) / stride + 1;
    auto y = out_override ? out_override : transient(s_out, z_out);
    auto op = graph->CreateOperation<ops::Conv2d>(static_cast<int32_t>(oc), PadType::AUTO, std::array<uint32_t, 2>({k, k}),
                                                  std::array<uint32_t, 2>({stride, stride}), std::array<uint32_t, 2>({1, 1}),
                                                  std::array<uint32_t, 4>({pl, pr, pl, pr}), depthwise ? 1 : 0);
    (*op).BindInputs({x.t, w, b}).BindOutputs({y});
    macs += static_cast<uint64_t>(Wo) * Ho * oc * fan_in;
    Act r{y, s_out, z_out, ms_out, mean_out, Wo, Ho, oc};
    if (act == 1 || act == 6) {
      auto z = transient(s_out, z_out);
      if (act == 1) {
        auto relu = graph->CreateOperation<ops::Relu>();
        (*relu).BindInput(y).BindOutput(z);
      } else {
        auto relu = graph->CreateOperation<ops::Relu6>();
        (*relu).BindInput(y).BindOutput(z);
      }
      r.t = z;
    }
    return r;
  }

  Act add(const Act& a, const Act& b, bool relu) {
    const double mean = a.mean + b.mean;
    const double var = std::max(a.ms + b.ms + 2.0 * a.mean * b.mean - mean * mean, 1e-12) + mean * mean;
    const float sigma = static_cast<float>(std::sqrt(var));
    const float s = relu ? 3.5f * sigma / 255.0f : 6.0f * sigma / 255.0f;
    const int zp = relu ? 0 : 128;
    auto y = transient(s, zp);
    auto op = graph->CreateOperation<ops::Add>();
    (*op).BindInputs({a.t, b.t}).BindOutputs({y});
    Act r{y, s, zp, relu ? var / 2 + mean * mean / 2 : var, relu ? std::max(mean, 0.3989 * sigma) : mean, a.W, a.H, a.C};
    if (relu) {
      auto z = transient(s, zp);
      auto ro = graph->CreateOperation<ops::Relu>();
      (*ro).BindInput(y).BindOutput(z);
      r.t = z;
    }
    return r;
  }

  Act fc(const Act& x, uint32_t axis, uint32_t K, uint32_t n_out, bool output_tensor) {
    std::shared_ptr<Tensor> w, b;
    std::vector<int32_t> bias(n_out);
    const double mean_xq = x.mean / x.scale;
    double w_var;
    if (wkind == S8_PER_CHANNEL) {
      std::vector<float> ws(n_out), bs(n_out);
      std::vector<int32_t> zeros(n_out, 0);
      const float shrink = 1.0f / std::sqrt(static_cast<float>(K) / 64.0f);
      double s2 = 0;
      for (uint32_t i = 0; i < n_out; ++i) {
        ws[i] = rng.uniform(0.001f, 0.01f) * shrink;
        bs[i] = x.scale * ws[i];
        s2 += static_cast<double>(ws[i]) * ws[i];
      }
      std::vector<int8_t> wd(static_cast<size_t>(K) * n_out);
      for (auto& v : wd) v = static_cast<int8_t>(rng.range(-127, 127));
      for (uint32_t i = 0; i < n_out; ++i) {
        long long sum = 0;
        for (uint32_t k = 0; k < K; ++k) sum += wd[static_cast<size_t>(i) * K + k];
        bias[i] = static_cast<int32_t>(std::llround(-mean_xq * static_cast<double>(sum))) + rng.range(-1000, 1000);
      }
      w = graph->CreateTensor(TensorSpec(DataType::INT8, {K, n_out}, TensorAttribute::CONSTANT,
                                         Quantization(QuantType::SYMMETRIC_PER_CHANNEL, 1, ws, zeros)), wd.data());
      b = graph->CreateTensor(TensorSpec(DataType::INT32, {n_out}, TensorAttribute::CONSTANT,
                                         Quantization(QuantType::SYMMETRIC_PER_CHANNEL, 0, bs, zeros)), bias.data());
      w_var = (s2 / n_out) * (127.0 * 128.0 / 3.0);
    } else {
      const int zw = wkind == U8_ZP128 ? 128 : rng.range(100, 156);
      const float sw = wkind == U8_ZP128 ? 0.01f : rng.uniform(0.005f, 0.05f) / std::sqrt(static_cast<float>(K) / 16.0f);
      std::vector<uint8_t> wd(static_cast<size_t>(K) * n_out);
      const double q_var = fill_u8_weights(wd, n_out, K, zw, wkind == U8_ZP128);
      for (uint32_t i = 0; i < n_out; ++i) {
        long long sum = 0;
        for (uint32_t k = 0; k < K; ++k) sum += static_cast<int>(wd[static_cast<size_t>(i) * K + k]) - zw;
        bias[i] = static_cast<int32_t>(std::llround(-mean_xq * static_cast<double>(sum))) + rng.range(-1000, 1000);
      }
      w = graph->CreateTensor(TensorSpec(DataType::UINT8, {K, n_out}, TensorAttribute::CONSTANT,
                                         Quantization(QuantType::ASYMMETRIC, sw, zw)), wd.data());
      b = graph->CreateTensor(TensorSpec(DataType::INT32, {n_out}, TensorAttribute::CONSTANT,
                                         Quantization(QuantType::ASYMMETRIC, x.scale * sw, 0)), bias.data());
      w_var = static_cast<double>(sw) * sw * q_var;
    }
    keep.push_back(w);
    keep.push_back(b);
    const double var = static_cast<double>(K) * x.ms * w_var;
    const float s_out = 6.0f * static_cast<float>(std::sqrt(std::max(var, 1e-12))) / 255.0f;
    std::shared_ptr<Tensor> y;
    if (output_tensor) {
      y = graph->CreateTensor(TensorSpec(DataType::UINT8, {n_out, batch}, TensorAttribute::OUTPUT,
                                         Quantization(QuantType::ASYMMETRIC, s_out, 128)));
      keep.push_back(y);
    } else {
      y = transient(s_out, 128);
    }
    auto op = graph->CreateOperation<ops::FullyConnected>(axis, n_out);
    (*op).BindInputs({x.t, w, b}).BindOutputs({y});
    macs += static_cast<uint64_t>(K) * n_out;
    return Act{y, s_out, 128, var, 0.0, 1, 1, n_out};
  }

  Act make_input(uint32_t w, uint32_t h, uint32_t c, float scale, int zp) {
    W = w; H = h; C = c;
    input = graph->CreateTensor(TensorSpec(DataType::UINT8, {w, h, c, batch}, TensorAttribute::INPUT,
                                           Quantization(QuantType::ASYMMETRIC, scale, zp)));
    // uniform 0..255: E[(q-zp)^2] * scale^2
    const double m = 127.5 - zp;
    return Act{input, scale, zp, static_cast<double>(scale) * scale * (m * m + (256.0 * 256.0 - 1.0) / 12.0), scale * m, w, h, c};
  }

  bool build_resnet50() {
    wkind = S8_PER_CHANNEL;
    classes = 1000;
    Act x = make_input(224, 224, 3, 0.02f, 128);
    x = conv(x, 7, 64, 2, 1);
    {
      // MaxPool 3x3/2 with pad {0,1,0,1} and CEILING, as the reference's exported graph does
      // (samples/multi_device/vx_resnet50.cc:1318-1323)
      auto y = transient(x.scale, x.zp);
      auto op = graph->CreateOperation<ops::Pool2d>(PoolType::MAX, std::array<uint32_t, 4>({0, 1, 0, 1}),
                                                    std::array<uint32_t, 2>({3, 3}), std::array<uint32_t, 2>({2, 2}),
                                                    RoundType::CEILING);
      (*op).BindInput(x.t).BindOutput(y);
      x.t = y; x.W = 56; x.H = 56;
    }
    const int blocks[4] = {3, 4, 6, 3};
    const uint32_t widths[4] = {64, 128, 256, 512};
    for (int s = 0; s < 4; ++s) {
      for (int blk = 0; blk < blocks[s]; ++blk) {
        const uint32_t stride = (blk == 0 && s > 0) ? 2 : 1;
        Act shortcut = x;
        if (blk == 0) shortcut = conv(x, 1, widths[s] * 4, stride, 0);   // projection shortcut
        Act y = conv(x, 1, widths[s], 1, 1);
        y = conv(y, 3, widths[s], stride, 1);                            // v1.5: stride on the 3x3
        y = conv(y, 1, widths[s] * 4, 1, 0);
        x = add(y, shortcut, true);
      }
    }
    {
      auto y = transient(x.scale, x.zp);
      auto op = graph->CreateOperation<ops::Pool2d>(PoolType::AVG, std::array<uint32_t, 2>({7, 7}));
      (*op).BindInput(x.t).BindOutput(y);
      x.t = y; x.W = 1; x.H = 1;
    }
    Act out = fc(x, 2, 2048, 1000, true);
    output = out.t;
    return true;
  }

  bool build_mobilenetv2() {
    wkind = U8_ASYM;
    classes = 1000;
    Act x = make_input(224, 224, 3, 0.02f, 128);
    x = conv(x, 3, 32, 2, 6);
    const int cfg[7][4] = {{1, 16, 1, 1}, {6, 24, 2, 2}, {6, 32, 3, 2}, {6, 64, 4, 2}, {6, 96, 3, 1}, {6, 160, 3, 2}, {6, 320, 1, 1}};
    for (const auto& c : cfg) {
      for (int i = 0; i < c[2]; ++i) {
        const uint32_t stride = i == 0 ? c[3] : 1;
        const Act in = x;
        Act y = x;
        if (c[0] != 1) y = conv(y, 1, in.C * c[0], 1, 6);
        y = conv(y, 3, y.C, stride, 6, true);
        y = conv(y, 1, c[1], 1, 0);
        if (stride == 1 && in.C == static_cast<uint32_t>(c[1])) y = add(y, in, false);
        x = y;
      }
    }
    x = conv(x, 1, 1280, 1, 6);
    {
      auto y = transient(x.scale, x.zp);
      auto op = graph->CreateOperation<ops::Pool2d>(PoolType::AVG, std::array<uint32_t, 2>({7, 7}));
      (*op).BindInput(x.t).BindOutput(y);
      x.t = y; x.W = 1; x.H = 1;
    }
    Act out = fc(x, 2, 1280, 1000, true);
    output = out.t;
    return true;
  }

  bool build_lenet() {
    // Synthetic quantization of the benchmark configuration: input scale 1/255 zp 0, uint8 weights
    // scale 0.01 zp 128, every activation scale 0.05 zp 128.
    wkind = U8_ZP128;
    classes = 10;
    Act x = make_input(28, 28, 1, 1.0f / 255.0f, 0);
    auto fixed = [&](Act a) { return a; };
    (void)fixed;
    auto conv_fixed = [&](const Act& in, uint32_t k, uint32_t oc) {
      float s = 0.05f;
      // valid padding: override the SAME-style pads the helper would use
      auto y = transient(0.05f, 128);
      std::vector<uint8_t> wd(static_cast<size_t>(k) * k * in.C * oc);
      for (auto& v : wd) v = static_cast<uint8_t>(rng.range(0, 255));
      std::vector<int32_t> bias(oc);
      for (auto& v : bias) v = rng.range(-1000, 1000);
      auto w = graph->CreateTensor(TensorSpec(DataType::UINT8, {k, k, in.C, oc}, TensorAttribute::CONSTANT,
                                              Quantization(QuantType::ASYMMETRIC, 0.01f, 128)), wd.data());
      auto b = graph->CreateTensor(TensorSpec(DataType::INT32, {oc}, TensorAttribute::CONSTANT,
                                              Quantization(QuantType::ASYMMETRIC, in.scale * 0.01f, 0)), bias.data());
      keep.push_back(w); keep.push_back(b);
      auto op = graph->CreateOperation<ops::Conv2d>(static_cast<int32_t>(oc), PadType::VALID, std::array<uint32_t, 2>({k, k}),
                                                    std::array<uint32_t, 2>({1, 1}), std::array<uint32_t, 2>({1, 1}));
      (*op).BindInputs({in.t, w, b}).BindOutputs({y});
      const uint32_t Wo = in.W - k + 1;
      macs += static_cast<uint64_t>(Wo) * Wo * oc * k * k * in.C;
      return Act{y, s, 128, 1.0, 0.0, Wo, Wo, oc};
    };
    auto pool = [&](const Act& in) {
      auto y = transient(in.scale, in.zp);
      auto op = graph->CreateOperation<ops::Pool2d>(PoolType::MAX, PadType::NONE, std::array<uint32_t, 2>({2, 2}),
                                                    std::array<uint32_t, 2>({2, 2}));
      (*op).BindInput(in.t).BindOutput(y);
      return Act{y, in.scale, in.zp, in.ms, in.mean, in.W / 2, in.H / 2, in.C};
    };
    x = pool(conv_fixed(x, 5, 20));
    x = pool(conv_fixed(x, 5, 50));
    auto fc_fixed = [&](const Act& in, uint32_t axis, uint32_t K, uint32_t n_out, bool last) {
      std::vector<uint8_t> wd(static_cast<size_t>(K) * n_out);
      for (auto& v : wd) v = static_cast<uint8_t>(rng.range(0, 255));
      std::vector<int32_t> bias(n_out);
      for (auto& v : bias) v = rng.range(-1000, 1000);
      auto w = graph->CreateTensor(TensorSpec(DataType::UINT8, {K, n_out}, TensorAttribute::CONSTANT,
                                              Quantization(QuantType::ASYMMETRIC, 0.01f, 128)), wd.data());
      auto b = graph->CreateTensor(TensorSpec(DataType::INT32, {n_out}, TensorAttribute::CONSTANT,
                                              Quantization(QuantType::ASYMMETRIC, in.scale * 0.01f, 0)), bias.data());
      keep.push_back(w); keep.push_back(b);
      std::shared_ptr<Tensor> y;
      if (last) {
        y = graph->CreateTensor(TensorSpec(DataType::UINT8, {n_out, batch}, TensorAttribute::OUTPUT,
                                           Quantization(QuantType::ASYMMETRIC, 0.05f, 128)));
        keep.push_back(y);
      } else {
        y = transient(0.05f, 128);
      }
      auto op = graph->CreateOperation<ops::FullyConnected>(axis, n_out);
      (*op).BindInputs({in.t, w, b}).BindOutputs({y});
      macs += static_cast<uint64_t>(K) * n_out;
      return Act{y, 0.05f, 128, 1.0, 0.0, 1, 1, n_out};
    };
    x = fc_fixed(x, 2, 800, 500, false);
    {
      auto z = transient(0.05f, 128);
      auto relu = graph->CreateOperation<ops::Relu>();
      (*relu).BindInput(x.t).BindOutput(z);
      x.t = z;
    }
    x = fc_fixed(x, 0, 500, 10, true);
    output = x.t;
    // Softmax tail of the sample, float32 output
    auto prob = graph->CreateTensor(TensorSpec(DataType::FLOAT32, {10, batch}, TensorAttribute::OUTPUT));
    keep.push_back(prob);
    auto sm = graph->CreateOperation<ops::Softmax>(1.0f, 0);
    (*sm).BindInput(output).BindOutput(prob);
    return true;
  }
};

extern "C" {

b2vx_net* b2vx_net_create(const char* name, int32_t batch, uint64_t seed, int32_t device) {
  if (!name || batch <= 0) return nullptr;
  auto net = std::make_unique<b2vx_net>();
  net->ctx = Context::Create();
  CompileOption opt;
  opt.setDeviceId(static_cast<uint32_t>(device));
  net->graph = net->ctx->CreateGraph(opt);
  net->batch = static_cast<uint32_t>(batch);
  net->rng = Rng(seed);
  const std::string n = name;
  bool ok = false;
  if (n == "resnet50") ok = net->build_resnet50();
  else if (n == "mobilenetv2") ok = net->build_mobilenetv2();
  else if (n == "lenet") ok = net->build_lenet();
  else std::fprintf(stderr, "b2vx_net_create: unknown network '%s'\n", name);
  if (!ok || !net->input || !net->output) return nullptr;
  if (!net->graph->Compile()) {
    std::fprintf(stderr, "b2vx_net_create: Compile failed for '%s'\n", name);
    return nullptr;
  }
  return net.release();
}

void b2vx_net_destroy(b2vx_net* net) { delete net; }

size_t b2vx_net_input_bytes(const b2vx_net* net) { return static_cast<size_t>(net->W) * net->H * net->C * net->batch; }
size_t b2vx_net_output_bytes(const b2vx_net* net) { return static_cast<size_t>(net->classes) * net->batch; }

void b2vx_net_synthetic_input(const b2vx_net* net, uint64_t seed, uint8_t* dst) {
  Rng r(seed ^ 0xABCDEF);
  const size_t n = b2vx_net_input_bytes(net);
  size_t i = 0;
  while (i + 8 <= n) {
    uint64_t v = r.next();
    std::memcpy(dst + i, &v, 8);
    i += 8;
  }
  for (; i < n; ++i) dst[i] = static_cast<uint8_t>(r.next());
}

int32_t b2vx_net_set_input(b2vx_net* net, const void* data) {
  return net->input->CopyDataToTensor(data, static_cast<uint32_t>(b2vx_net_input_bytes(net))) ? 0 : -1;
}
int32_t b2vx_net_run(b2vx_net* net) { return net->graph->Run() ? 0 : -1; }
int32_t b2vx_net_get_output(b2vx_net* net, void* data) { return net->output->CopyDataFromTensor(data) ? 0 : -1; }
void* b2vx_net_graph_handle(b2vx_net* net) { return timvx_graph_backend_handle(net->graph.get()); }
uint64_t b2vx_net_macs_per_image(const b2vx_net* net) { return net->macs; }

}  // extern "C"
