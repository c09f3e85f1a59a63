// b2vx_conv2d_first_layer_noalloc — the first-layer convolution for callers that cannot allocate
// device memory.
//
// Who that is: code that runs inside someone else's memory budget — a plugin of a serving process
// whose device memory is handed out once at start-up, a real-time loop that must not enter the
// driver's allocator (cudaMalloc takes locks and may synchronise the whole device), a library loaded
// into a process that runs close to the memory limit, where an allocation in the middle of a request
// can simply fail.  Such callers own every buffer they pass in, and the one thing this convolution needs
// beyond its inputs and outputs — the im2col matrix between its two kernels — lives in the fixed
// array below instead of in memory obtained per graph.
//
// The price: every GPU that loads the library carries kScratchBytes of device memory until the process
// exits, problems whose im2col matrix is larger are refused, and all calls on one GPU share the array,
// so two calls whose kernels overlap on the GPU (different streams, different threads) corrupt each
// other.  The array keeps whatever the previous call left; nothing in it needs to start at zero except
// the status word, which every call clears before its kernels run.
#include <cuda_runtime.h>

#include <climits>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "b2vx.h"
#include "kernels.h"

namespace {

constexpr size_t kScratchBytes = B2VX_NOALLOC_SCRATCH_BYTES;
constexpr int kMaxDevices = 64;

// In host code these two names are host-side stand-ins, not device addresses: they may only be
// handed to cudaGetSymbolAddress (done once per device in setup()), never to a kernel.
static __device__ __align__(256) unsigned char g_scratch[kScratchBytes];
static __device__ __align__(256) int g_status[64];

struct PerDevice {
  std::once_flag once;      // first calls on one GPU from several threads: one of them does the set-up, the others wait
  cudaError_t error = cudaSuccess;
  unsigned char* scratch = nullptr;   // device address of g_scratch on this device
  int* status = nullptr;              // device address of g_status on this device
};
PerDevice g_dev[kMaxDevices];

b2vx_status fail(char* err, size_t err_len, b2vx_status st, const char* msg) {
  if (err && err_len) std::snprintf(err, err_len, "%s", msg);
  return st;
}

// Once per device, with that device current: resolve the device addresses of the static arrays.
b2vx_status setup(int dev, char* err, size_t err_len) {
  PerDevice& d = g_dev[dev];
  std::call_once(d.once, [&d] {
    void* p = nullptr;
    d.error = cudaGetSymbolAddress(&p, g_scratch);
    if (d.error != cudaSuccess) return;
    d.scratch = static_cast<unsigned char*>(p);
    d.error = cudaGetSymbolAddress(&p, g_status);
    if (d.error != cudaSuccess) return;
    d.status = static_cast<int*>(p);
  });
  if (d.error != cudaSuccess) return fail(err, err_len, B2VX_CUDA_ERROR, cudaGetErrorString(d.error));
  return B2VX_OK;
}

}  // namespace

extern "C" b2vx_status b2vx_conv2d_first_layer_noalloc(const b2vx_conv2d_noalloc_desc* d, const void* x_whcn,
                                                       const int8_t* w8, const int32_t* bias_full, const float* acc_scale,
                                                       void* y_cl, void* cuda_stream, char* err, size_t err_len) {
  using namespace b2vx;
  if (!d || !x_whcn || !w8 || !bias_full || !acc_scale || !y_cl) return fail(err, err_len, B2VX_INVALID_ARG, "null argument");
  if (d->n == 0 || d->h == 0 || d->w == 0 || d->c == 0 || d->c >= 16 || d->kw == 0 || d->kh == 0 || d->oc == 0 || d->oc > 256)
    return fail(err, err_len, B2VX_INVALID_ARG, "need 1 <= c < 16, 1 <= oc <= 256 and non-empty shapes");
  if (!(d->out_scale > 0.0f)) return fail(err, err_len, B2VX_INVALID_ARG, "out_scale must be positive");
  // every extent is turned into an int below: refuse what would not survive that (or the sums built from it)
  const uint32_t lim = static_cast<uint32_t>(INT_MAX / 4);
  if (d->n > lim || d->h > lim || d->w > lim || d->kw > lim || d->kh > lim || d->stride[0] > lim || d->stride[1] > lim ||
      d->dilation[0] > lim || d->dilation[1] > lim || d->pad[0] > lim || d->pad[1] > lim || d->pad[2] > lim || d->pad[3] > lim)
    return fail(err, err_len, B2VX_INVALID_ARG, "an extent, stride, dilation or padding is out of range");
  if (static_cast<long long>(d->kw) * d->kh * d->c > 65536)
    return fail(err, err_len, B2VX_INVALID_ARG, "filter too large (kw*kh*c must be at most 65536)");
  if (d->in_zero_point < 0 || d->in_zero_point > 255 || d->out_zero_point < 0 || d->out_zero_point > 255)
    return fail(err, err_len, B2VX_INVALID_ARG, "zero points of uint8 tensors must lie in 0..255");
  const int sx = d->stride[0] ? d->stride[0] : 1, sy = d->stride[1] ? d->stride[1] : 1;
  const int dx = d->dilation[0] ? d->dilation[0] : 1, dy = d->dilation[1] ? d->dilation[1] : 1;
  const long long span_w = static_cast<long long>(d->w) + d->pad[0] + d->pad[1] - (static_cast<long long>(d->kw - 1) * dx + 1);
  const long long span_h = static_cast<long long>(d->h) + d->pad[2] + d->pad[3] - (static_cast<long long>(d->kh - 1) * dy + 1);
  if (span_w < 0 || span_h < 0) return fail(err, err_len, B2VX_SHAPE_MISMATCH, "kernel larger than the padded input");
  ConvGeom g;
  g.N = d->n; g.H = d->h; g.W = d->w; g.C = d->c; g.Cp = 16;
  g.Wo = static_cast<int>(span_w / sx) + 1;
  g.Ho = static_cast<int>(span_h / sy) + 1;
  g.Oc = d->oc; g.Ocp = (static_cast<int>(d->oc) + 15) & ~15;
  g.kh = d->kh; g.kw = d->kw; g.sx = sx; g.sy = sy; g.dx = dx; g.dy = dy; g.pl = d->pad[0]; g.pt = d->pad[2];
  const int K = static_cast<int>(d->c * d->kh * d->kw);
  const int Kp = (K + 15) & ~15;
  const long long M = static_cast<long long>(g.N) * g.Ho * g.Wo;
  if (M * Kp > static_cast<long long>(kScratchBytes) || M > 0x7fffffffLL) {
    char msg[200];
    std::snprintf(msg, sizeof(msg), "the im2col matrix of this problem needs %lld bytes; the built-in scratch holds %zu", M * Kp,
                  kScratchBytes);
    return fail(err, err_len, B2VX_INVALID_ARG, msg);
  }
  // staging rows of one output row must fit the im2col kernel's shared memory
  const size_t rowlen = static_cast<size_t>(g.Wo - 1) * sx + static_cast<size_t>(g.kw - 1) * dx + 1;
  if (static_cast<size_t>(g.C) * g.kh * rowlen + 4u * Kp > 40u * 1024u)
    return fail(err, err_len, B2VX_INVALID_ARG, "image rows too wide for the im2col staging buffer");

  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return fail(err, err_len, B2VX_CUDA_ERROR, "no current CUDA device");
  b2vx_status st = setup(dev, err, err_len);
  if (st != B2VX_OK) return st;
  const PerDevice& pd = g_dev[dev];
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);

  ContractEpilogue ep;
  std::memset(&ep, 0, sizeof(ep));
  ep.bias_full = bias_full;
  ep.acc_scale = acc_scale;
  ep.out.scale = d->out_scale;
  ep.out.zp = d->out_zero_point;
  ep.out.lo = 0;
  ep.out.hi = 255;
  // The scales are device memory, which this call may not read back to bound |accumulator * scale / out_scale| the
  // way the graph's planner does; the exact requantization is right for any scales.
  ep.exact_only = 1;
  alignas(64) unsigned char plan_storage[1024];
  if (gemm_tc_plan_bytes() > sizeof(plan_storage)) return fail(err, err_len, B2VX_BAD_STATE, "plan storage too small");
  char why[160] = {0};
  GemmTcPlan* plan = gemm_tc_plan_build_in(plan_storage, sizeof(plan_storage), pd.scratch, 0, w8, static_cast<int>(M), g.Ocp, Kp, y_cl,
                                           g.Ocp, ep, pd.status, why, sizeof(why));
  if (!plan) return fail(err, err_len, B2VX_UNSUPPORTED, why);

  cudaError_t e = cudaMemsetAsync(pd.status, 0, sizeof(int), stream);
  if (e == cudaSuccess) {
    launch_im2col_whcn(x_whcn, Kp, d->in_zero_point, g, pd.scratch, stream);
    e = cudaGetLastError();
  }
  if (e == cudaSuccess) e = gemm_tc_launch(plan, stream);
  int status = 0;
  if (e == cudaSuccess) e = cudaMemcpyAsync(&status, pd.status, sizeof(int), cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) return fail(err, err_len, B2VX_CUDA_ERROR, cudaGetErrorString(e));
  if (status != 0) return fail(err, err_len, B2VX_DEVICE_TIMEOUT, "the GEMM kernel gave up waiting on a barrier");
  return B2VX_OK;
}
