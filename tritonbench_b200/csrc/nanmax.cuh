// max / min that return NaN when either argument is NaN, as torch's max, amax and clamp do
// (fmaxf and fminf return the other argument).  The quantisers reduce with these, so that a NaN
// anywhere in a row (or block) makes that row's scale and all of its codes NaN, as in torch.
#pragma once

#include <cuda_runtime.h>

namespace b200fp8 {

__device__ __forceinline__ float max_nan(float a, float b) {
  float r;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}

__device__ __forceinline__ float min_nan(float a, float b) {
  float r;
  asm("min.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}

}  // namespace b200fp8
