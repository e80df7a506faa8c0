// Programmatic dependent launch: let the next kernel of a stream start its launch and prologue while this one drains.
//
// The decode step of the rollout engine is a chain of ~15 short kernels per layer; in a CUDA graph each dependency edge
// still costs a launch round trip.  A kernel launched through `launch_pdl` carries the
// programmatic-stream-serialization attribute: it may be scheduled as soon as every CTA of its predecessor has executed
// `pdl_trigger()` (or exited), and it must execute `pdl_wait()` before it reads anything the predecessor wrote —
// `griddepcontrol.wait` returns only when the predecessor grid has completed and its memory is visible.  Rules kept here:
//   * every kernel launched with `launch_pdl` calls `pdl_wait()` before its first dependent global access;
//   * `pdl_trigger()` sits at the top of the kernel (the dependent's CTAs then queue behind this grid's own CTAs: a
//     dependent is only released once ALL CTAs of this grid have been scheduled and reached the trigger);
//   * a kernel with these calls can still be launched with `<<<>>>`: both instructions are no-ops then.
#pragma once
#include <cuda_runtime.h>

extern "C" int mb_pdl_enabled();

namespace mb {

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = mb_pdl_enabled();
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace mb
