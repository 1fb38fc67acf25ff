// Scale rule shared by every FP8 quantiser of the library.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace ksana {

// Quantisation scale of a 128-element group with absolute maximum `amax`: the smallest power of two that maps
// the group into the e4m3 range (UE8M0 scale: the tensor cores can apply it themselves, and 1/scale is exact).
__device__ __forceinline__ float fp8_group_scale(float amax) {
  const float s = fmaxf(amax, 1e-10f) * (1.f / 448.f);
  const uint32_t bits = __float_as_uint(s);
  const uint32_t e = (bits >> 23) + ((bits & 0x7FFFFFu) ? 1u : 0u);
  return __uint_as_float(e << 23);
}

}  // namespace ksana
