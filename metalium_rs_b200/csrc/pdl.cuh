// Programmatic dependent launch: a kernel launched with the attribute may have its blocks scheduled
// while the kernel before it on the stream is still running; it calls pdl_enter() before it touches
// global memory, which (1) lets the kernel after it be scheduled in turn and (2) waits until every
// kernel before it has completed and its writes are visible.  The ordering of the stream is kept; what
// is saved is the launch latency between the small kernels of a decode step or a prefill layer
// (a few microseconds each, several hundred a pass).  B200TT_PDL=0 launches without the attribute.
#pragma once
#include <cuda_runtime.h>
#include <stdlib.h>

namespace b200 {

__device__ __forceinline__ void pdl_enter() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

inline bool pdl_enabled() {
  static int v = -1;
  if (v < 0) { const char* e = getenv("B200TT_PDL"); v = (e && e[0] == '0') ? 0 : 1; }
  return v == 1;
}

template <typename... P, typename... A>
inline cudaError_t launch_pdl(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, A&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<P>(args)...);
}

}  // namespace b200
