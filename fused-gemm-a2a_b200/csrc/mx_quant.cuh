// Device helpers of the MXFP8 quantizer shared by the standalone kernels and the receive-side
// quantizer warps of the GEMM: scale rule, scale-byte layout, E4M3 conversion, and the 8-value
// lane step (4 lanes share one 32-element group).
#pragma once
#include <cstdint>
#include <cuda_runtime.h>
#include "mx_rule.cuh"

namespace fga {

// The scale rule and the scale-byte layout are plain integer functions (mx_rule.cuh), compiled for
// the host as well so that the CPU tests can sweep them against the oracle.
__device__ __forceinline__ void mx_scale(float peak, int& exponent, float& inv_scale) {
  rule::mx_scale(peak, exponent, inv_scale);
}

__device__ __forceinline__ long long mx_scale_offset(long long row, int group, int groups) {
  return rule::mx_scale_offset(row, group, groups);
}

__device__ __forceinline__ uint16_t to_e4m3x2(float lo, float hi) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}

// One lane's 8 consecutive BF16 values of a group: group maximum over the 4 lanes that share the
// group (warp-wide shuffles: call with all lanes), scale, E4M3 payload. Returns the biased E8M0
// exponent byte in `sf_byte`.
__device__ __forceinline__ uint2 mx_quantize8(const uint4 x, int& sf_byte) {
  float v[8];
  const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    v[2 * e] = __uint_as_float(w[e] << 16);
    v[2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
  }
  float peak = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) peak = fmaxf(peak, fabsf(v[j]));
  peak = fmaxf(peak, __shfl_xor_sync(0xffffffffu, peak, 1));
  peak = fmaxf(peak, __shfl_xor_sync(0xffffffffu, peak, 2));
  int e;
  float inv;
  mx_scale(peak, e, inv);
  sf_byte = e + 127;
  uint2 out;
  out.x = to_e4m3x2(v[0] * inv, v[1] * inv) | (static_cast<uint32_t>(to_e4m3x2(v[2] * inv, v[3] * inv)) << 16);
  out.y = to_e4m3x2(v[4] * inv, v[5] * inv) | (static_cast<uint32_t>(to_e4m3x2(v[6] * inv, v[7] * inv)) << 16);
  return out;
}

}  // namespace fga
