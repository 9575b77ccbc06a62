// Shared pieces of the basis projection kernels.
#pragma once

#include <cuda_bf16.h>

#include "common.cuh"

namespace tfgpc {

// Channels owned by one lane: with K basis functions a lane keeps CPL*K
// accumulators in registers (at most 64).
template <int K>
struct BpCfg {
  static constexpr int kCpl = (K >= 64) ? 1 : (K == 32 ? 2 : 4);
  static constexpr int kAcc = kCpl * K;
  static constexpr int kRow = kAcc + 4;  // padded staging row (floats): conflict-free 128-bit access
};

inline bool valid_basis(int K) { return K == 8 || K == 16 || K == 32 || K == 64; }
// basis_proj_ops.cpp:104-108: between 1 and 8, or a multiple of 8.
inline bool valid_features(int C) { return C > 0 && (C < 8 || C % 8 == 0); }

// Lanes cooperating on one sample: the smallest power of two covering C.
inline int bp_group_lanes(int C, int cpl) {
  int need = (C + cpl - 1) / cpl;
  int g = 1;
  while (g < need && g < 32) g <<= 1;
  return g;
}

// Split of an fp32 value into two bf16 terms, x ~= hi + mid (relative error
// about 2^-17), the operand format of the 3-pass bf16 tensor-core GEMMs.
__device__ __forceinline__ void split_bf16(float x, __nv_bfloat16& hi, __nv_bfloat16& mid) {
  hi = __float2bfloat16_rn(x);
  mid = __float2bfloat16_rn(x - __bfloat162float(hi));
}

// The same split for two values at once: packed bf16 pairs of the hi and mid
// terms (x in the low half).
__device__ __forceinline__ void split2_bf16(float x, float y, uint32_t& hi, uint32_t& mid) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
  hi = *reinterpret_cast<const uint32_t*>(&h);
  const float hx = __uint_as_float(hi << 16), hy = __uint_as_float(hi & 0xffff0000u);
  const __nv_bfloat162 m = __floats2bfloat162_rn(x - hx, y - hy);
  mid = *reinterpret_cast<const uint32_t*>(&m);
}

}  // namespace tfgpc
