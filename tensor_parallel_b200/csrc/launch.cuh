// Kernel launch helper.  With TPB_PDL=1 the decode-path kernels are launched with the programmatic-dependent-launch
// attribute: between two dependent kernels of a CUDA graph lie about 3.7 us on B200 (measured with %globaltimer stamps
// inside the kernels), part of it launch latency that a successor scheduled ahead of time hides.
// Off by default.  Measured on one B200 with the per-rank shapes of a Llama-2-7B decode step: 2.35 vs 2.40 ms at
// 8-way, 2.96 vs 3.09 ms at 4-way shard shapes, but 4.79 vs 3.91 ms at 2-way and 5.76 vs 5.65 ms unsharded.
// Discipline of every such kernel: do the work that does not depend on earlier kernels (barrier init, TMEM
// allocation), then griddepcontrol.wait, and only THEN griddepcontrol.launch_dependents.  A successor is scheduled
// once every CTA of this grid has passed that point, i.e. once the whole grid is resident and its predecessor has
// completed: exactly one kernel is ever scheduled ahead, and its idle CTAs cannot take an SM from a CTA of the grid
// they wait for.  (Triggering before the wait let a whole chain of future kernels pile up on the SMs and slowed the
// Llama-7B decode step from 6.4 to 7.9 ms.)  Only the GEMM kernels trigger: measured on B200 a GEMM that follows a GEMM
// gains about 1 us, whereas successors scheduled into a running attention kernel (many small CTAs, several per SM) end
// up unevenly spread over the SMs and cost more than the hidden launch latency (+1 to 2 us per attention launch).
#pragma once
#include <cuda_runtime.h>
#include <stdlib.h>

namespace tpb {

inline bool pdl_enabled() {
  static int enabled = -1;
  if (enabled < 0) {
    const char* v = getenv("TPB_PDL");
    enabled = (v && v[0] != '0' && v[0] != 0) ? 1 : 0;
  }
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
