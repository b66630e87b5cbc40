// Router arithmetic that must give the same bits on the GPU and in a CPU checker.
//
// exp() is written out as a fixed sequence of IEEE fp32 operations (one multiply,
// round-to-nearest-even, two fused multiply-adds for the range reduction, a degree-5
// Horner polynomial in fused multiply-adds, one add, one multiply by an exact power of
// two), so any implementation that performs the same sequence in IEEE fp32 reproduces
// it exactly. The sigmoid router (modes 1 and 2) selects experts by comparing
// sigmoid(logit) + bias; with a library expf the last-ulp differences between two
// libraries flip selections at near-ties (the reference documents one such flip per
// 8192 tokens between fp32 and fp64, research_archive/ds3_acc.py:242-253). A fully
// specified exp removes that source of disagreement.
#pragma once
#include <cstdint>

namespace mono {

__device__ __forceinline__ float det_expf(float x) {
  x = fminf(fmaxf(x, -87.0f), 88.0f);
  const float t = __fmul_rn(x, 1.44269504088896341f);
  const float n = rintf(t);  // round to nearest even
  float r = __fmaf_rn(n, -0.693145751953125f, x);
  r = __fmaf_rn(n, -1.42860682030941723e-6f, r);
  float p = 1.9875691500e-4f;
  p = __fmaf_rn(p, r, 1.3981999507e-3f);
  p = __fmaf_rn(p, r, 8.3334519073e-3f);
  p = __fmaf_rn(p, r, 4.1665795894e-2f);
  p = __fmaf_rn(p, r, 1.6666665459e-1f);
  p = __fmaf_rn(p, r, 5.0000001201e-1f);
  const float z = __fmul_rn(r, r);
  float y = __fmaf_rn(p, z, r);
  y = __fadd_rn(y, 1.0f);
  const int ni = static_cast<int>(n);  // in [-126, 127] after the clamp
  const float scale = __int_as_float((ni + 127) << 23);
  return __fmul_rn(y, scale);
}

// sigmoid(v) = 1 / (1 + exp(-v)), IEEE division.
__device__ __forceinline__ float det_sigmoidf(float v) {
  return __fdiv_rn(1.0f, __fadd_rn(1.0f, det_expf(-v)));
}

}  // namespace mono
