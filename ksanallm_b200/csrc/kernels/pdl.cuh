// Programmatic dependent launch (PDL): a kernel launched with the stream-serialisation attribute may start while its
// predecessor in the stream is still running; it must call pdl_wait() before it touches anything the predecessor
// (or any earlier kernel) wrote or still reads, and pdl_trigger() lets its own successor start early in turn.
// A decode step is several hundred short kernels in one stream: without this every boundary costs the full
// drain -> launch -> ramp sequence; with it the successor's CTAs are resident with their set-up done (barriers,
// TMEM, descriptor prefetch) when the predecessor's last CTA retires. Inside a CUDA graph the attribute becomes a
// programmatic dependency edge.
//
// Rules used in this library:
//   * pdl_trigger() as early as possible; pdl_wait() before the first global-memory access that is not a read of
//     weights / constants (those are never written while the engine runs);
//   * a kernel launched through launch_pdl() that lacks pdl_wait() would race: only kernels that call it are launched
//     with the attribute;
//   * both calls are no-ops in a kernel launched without the attribute.
// Off by default: in whole decode steps (CUDA graphs of 800 kernels) the measured gain of the early launches was
// within noise, while graphs of one kernel class back to back gained about a microsecond per launch. KSANA_PDL=1 in
// the environment switches the attribute on.
#pragma once
#include <cuda_runtime.h>
#include <cstdlib>
#include <utility>

namespace ksana {

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

inline bool pdl_enabled() {
  static const bool on = []() {
    const char* e = std::getenv("KSANA_PDL");
    return e && e[0] == '1';
  }();
  return on;
}

// kernel<<<grid, block, smem, st>>>(args...) with the programmatic stream-serialisation attribute (when enabled).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                              Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

}  // namespace ksana
