// Kernel launch helper.  With TPB_PDL set in the environment the decode-path kernels are launched with the
// programmatic-dependent-launch attribute (the prologue of a kernel may overlap the tail of its predecessor).
// Off by default: measured on B200 it slowed the Llama-7B decode step down (6.4 -> 7.9 ms at one GPU), because
// early-scheduled successor CTAs with ~220 KB of shared memory take SMs away from the kernel they wait for.
#pragma once
#include <cuda_runtime.h>
#include <stdlib.h>

namespace tpb {

inline bool pdl_enabled() {
  static int enabled = -1;
  if (enabled < 0) enabled = getenv("TPB_PDL") ? 1 : 0;
  return enabled == 1;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
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
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace tpb
