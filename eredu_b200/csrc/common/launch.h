// Kernel launch with programmatic dependent launch (PDL): the next kernel of the stream may be scheduled
// while this one is still running; its prologue (barrier init, TMEM allocation, descriptor prefetch) then
// overlaps our tail. Every kernel launched through here executes `griddepcontrol.wait` before it touches
// memory another kernel may have produced (pdl_wait() in ptx.cuh). EREDU_PDL=0 turns the attribute off.
#pragma once
#include <cuda_runtime.h>

#include <cstdlib>
#include <utility>

namespace eredu {

inline bool pdl_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = std::getenv("EREDU_PDL");
    v = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args) {
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
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

}  // namespace eredu
