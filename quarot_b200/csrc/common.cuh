// Shared host/device helpers for the quarot_b200 kernels (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>

#include "../../include/quarot_b200.h"

namespace qr {

// ---------------------------------------------------------------- host side
void set_error(const char* fmt, ...);
int fail(int code, const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);
int* kernel_status_ptr();        // device address of the per-device status word (lazy, no allocation)
int num_sms();
int tuning(const char* key, int dflt);

#define QR_CUDA(expr)                                            \
  do {                                                           \
    cudaError_t _e = (expr);                                     \
    if (_e != cudaSuccess) return ::qr::cuda_fail(_e, #expr);    \
  } while (0)

#define QR_LAUNCH_CHECK(name)                                    \
  do {                                                           \
    cudaError_t _e = cudaGetLastError();                         \
    if (_e != cudaSuccess) return ::qr::cuda_fail(_e, name);     \
  } while (0)

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
static inline bool is_pow2(int64_t v) { return v > 0 && (v & (v - 1)) == 0; }
static inline int ilog2(int64_t v) { int l = 0; while ((int64_t(1) << l) < v) ++l; return l; }

// -------------------------------------------------------------- device side
#ifdef __CUDACC__

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// Quantise two fp32 quotients that were already divided by the row scale:
// round each to fp16 (the rounding torch applies to x / s), clamp to [-8, 7],
// round half-to-even to an integer and return the two 4-bit two's-complement
// codes in bits [3:0] and [19:16].
__device__ __forceinline__ uint32_t quant_pair(float q0, float q1) {
  __half2 h = __floats2half2_rn(q0, q1);
  h = __hmax2(h, __float2half2_rn(-8.0f));   // NaN-propagation: hmax2/hmin2 return the non-NaN operand
  h = __hmin2(h, __float2half2_rn(7.0f));
  // 1536 = 1.5 * 2^10: adding it leaves the integer in the low mantissa bits with RNE rounding
  h = __hadd2(h, __float2half2_rn(1536.0f));
  uint32_t bits = *reinterpret_cast<uint32_t*>(&h);
  return bits & 0x000F000Fu;
}

// Codes for a row whose scale is zero: torch evaluates x / 0 = +-inf (or NaN for 0 / 0),
// so positive values saturate to 7, negative ones to -8 and zeros stay 0.
__device__ __forceinline__ uint32_t quant_pair_zero_scale(float a, float b) {
  const uint32_t ca = a > 0.0f ? 7u : (a < 0.0f ? 8u : 0u);
  const uint32_t cb = b > 0.0f ? 7u : (b < 0.0f ? 8u : 0u);
  return ca | (cb << 16);
}

// Correctly rounded fp32 quotient y / s given rcp = RN(1/s): the product y*rcp is
// refined by two residual (Markstein) steps, which yields the IEEE round-to-nearest
// quotient for the normal-range operands that occur here (s is a finite non-zero
// fp16 value widened to fp32, |y| <= 65504).  Costs 5 FMA-pipe instructions and no
// MUFU call per element, because the reciprocal is shared by the whole row.
__device__ __forceinline__ float div_by_scale(float y, float s, float rcp) {
  float t = y * rcp;
  float e = __fmaf_rn(-s, t, y);
  t = __fmaf_rn(e, rcp, t);
  e = __fmaf_rn(-s, t, y);
  return __fmaf_rn(e, rcp, t);
}

#endif  // __CUDACC__

}  // namespace qr
