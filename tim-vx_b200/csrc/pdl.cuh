// Programmatic dependent launch: a kernel launched with launch_pdl() may be scheduled while the kernel
// before it in the stream is still running, so that its prologue (and its CTAs' arrival on SMs the
// predecessor has already left) overlaps the predecessor's tail.  The price is a rule: such a kernel
// must execute pdl_wait() before its first access to memory another kernel of the stream may have
// written or may still be reading.  pdl_trigger() lets the kernel after this one start the same way.
// Both are no-ops for a kernel launched normally.  B2VX_PDL=0 turns the attribute off.
#ifndef B2VX_PDL_CUH_
#define B2VX_PDL_CUH_

#include <cuda_runtime.h>

#include <cstdlib>
#include <utility>

namespace b2vx {

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

inline bool pdl_enabled() {
  static const bool on = [] { const char* e = std::getenv("B2VX_PDL"); return !(e && e[0] == '0'); }();
  return on;
}

template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(std::forward<Args>(args))...);
}

}  // namespace b2vx
#endif  // B2VX_PDL_CUH_
