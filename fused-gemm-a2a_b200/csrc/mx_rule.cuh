// MXFP8 scale rule and scale-byte layout: integer functions shared by the device quantizers
// (mx_quant.cuh) and the CPU tests (tests/native/schedule_host.cpp builds them with g++).
#pragma once
#include <cstdint>
#include <cstring>

#if defined(__CUDACC__)
#define FGA_RULE_HD __host__ __device__ __forceinline__
#else
#define FGA_RULE_HD inline
#endif

namespace fga {
namespace rule {

FGA_RULE_HD int float_bits(float f) {
#if defined(__CUDA_ARCH__)
  return __float_as_int(f);
#else
  int i;
  memcpy(&i, &f, sizeof i);
  return i;
#endif
}

FGA_RULE_HD float bits_float(int i) {
#if defined(__CUDA_ARCH__)
  return __int_as_float(i);
#else
  float f;
  memcpy(&f, &i, sizeof f);
  return f;
#endif
}

// Scale of one 32-element group from its largest magnitude (reference _mx_scale,
// fused_gemm_a2a_kernels.py:1200-1219): exponent = ceil(log2(peak / 448)) read off the FP32 bit
// pattern - 448 = 1.75 * 2^8, so the exponent field minus 127 minus 8 is rounded up exactly when the
// mantissa exceeds that of 1.75 (0x600000) - clamped to [-126, 127]; an all-zero group scales by 1.
// inv_scale = 2^-exponent multiplies the group's values before the E4M3 conversion. A group whose
// peak is infinite gets the NaN scale (byte 255, exponent 128 here) and the multiplier 0.
FGA_RULE_HD void mx_scale(float peak, int& exponent, float& inv_scale) {
  exponent = 0;
  if (peak > 0.f) {
    const int bits = float_bits(peak);
    exponent = (bits >> 23) - 135;
    if ((bits & 0x7fffff) > 0x600000) exponent += 1;
    exponent = exponent < -126 ? -126 : (exponent > 127 ? 127 : exponent);
  }
  inv_scale = bits_float((127 - exponent) << 23);
  if (peak == bits_float(0x7f800000)) {
    exponent = 128;
    inv_scale = 0.f;
  }
}

// Byte offset of the scale of (row, 32-element group) in the tcgen05 layout: 512-byte blocks of
// 128 rows x 4 groups, rows 32 apart share a 16-byte line (reference _mx_scale_offset,
// fused_gemm_a2a_kernels.py:1195-1197). groups = padded K / 32.
FGA_RULE_HD long long mx_scale_offset(long long row, int group, int groups) {
  return ((row / 128) * (groups / 4) + group / 4) * 512 + (row % 32) * 16 + (row % 128 / 32) * 4 + group % 4;
}

}  // namespace rule
}  // namespace fga
