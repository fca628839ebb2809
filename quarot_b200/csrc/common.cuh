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

// Kernel-selection knobs (qr_set_tuning); the defaults are the measured best choices.
struct Tuning {
  int gemm_bn = 256;          // N tile of the 1-CTA GEMM (256, 128 or 64)
  int gemm_bn2 = 0;           // N tile of the 2-CTA GEMM: 0 = chosen per shape, else 256, 240, 224 or 192
  int gemm_pst = 4;           // packed staging slots of the 1-CTA GEMM at BN = 256 (4 or 3)
  int gemm_grid = 0;          // cap on the number of persistent CTAs / clusters (0 = one per SM / SM pair)
  int gemm_decode_max_m = 64; // token rows up to which the weight-streaming kernels are used (decode)
  int gemm_splitk = 1;        // tcgen05 decode kernel, narrow layers: deal out (tile, stage) units through scratch memory: 0 never, 1 for K > 8192 (measured cross-over), 2 always
  int gemm_2sm = 1;           // prefill: 2-CTA kernel (cta_group::2) instead of the 1-CTA kernel
  int gemm_tma_out = 1;       // 2-CTA kernel: tiled TMA stores of the output where alignment allows
  int gemm_tail_help = 1;     // 2-CTA kernel: idle warps share the epilogue of a CTA's last tile
  int gemv_max_m = 0;         // token rows up to which the weight-streaming CUDA-core (dp4a) kernel is used (it also serves the quantiser-fused call)
  int gemv_mma_halves = 0;    // that kernel as two CTAs of eight warps per SM (1, where they fit) or one of sixteen (2); 0: the measured choice
  int hadq_heads = 1;         // heads-axis Hadamard of 8, 16 or 32 heads: two columns per thread (0: the masked warp-per-row kernel)
  int hadq_split = 1;         // up to 32 rows of n = 64 K: a cluster of four CTAs per row (0: one CTA per row)
  int gemv_mma_two_pass = 1;  // 33 .. 64 token rows of layers of at most 12 MB: two passes of that kernel instead of the tcgen05 decode kernel
  int gemv_mma_max_m = 32;    // token rows up to which the weight-streaming mma.sync kernel is used (0: never)
  int gemm_decode = 1;        // decode: the weight-streaming tcgen05 kernel (0: tokens on the MMA rows as at prefill)
  int pdl = 2;                // programmatic dependent launch: 0 never, 1 always, 2 decode-sized launches only
  int hadq_path = 0;          // 1 = always the generic Hadamard kernel (A/B checks)
  int hadq_walsh = 0;         // 1: warp-per-row register kernel also for whole-row Walsh transforms of 256 .. 4096 (measured slower)
  int hadq_tc = 1;            // tensor-core kernel for n = 64 K Kronecker shapes: 1 above 128 rows, 2 always, 0 never
};
extern Tuning g_tuning;
// programmatic dependent launch for a launch that works on `rows` token rows?
static inline bool use_pdl(int64_t rows) { return g_tuning.pdl == 1 || (g_tuning.pdl == 2 && rows <= 64); }

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

// Programmatic dependent launch.  Every kernel of the quantise -> GEMM chain is launched with the
// "programmatic stream serialization" attribute, tells the scheduler at its very start that the next kernel
// of the stream may be brought up (pdl_launch_dependents), and executes pdl_wait before its first access to
// global memory that an earlier kernel may have written or may still read.  The wait returns when the
// preceding kernel has completed and its memory is visible, so launch latency, barrier and tensor-memory
// set-up of a kernel overlap the tail of its predecessor.  Without the launch attribute both are no-ops.
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// cudaLaunchKernelEx with the programmatic-serialization attribute when `pdl` is set.
template <typename... KArgs, typename... Args>
static inline cudaError_t launch_kernel(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                        bool pdl, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}
#endif

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

// Division by the row scale as ONE multiplication with rcp = RN(1/s).
// torch computes fp16(fp32(y / s)) for fp16 y and s; t = RN(y * rcp) is not always the correctly rounded
// fp32 quotient, but it always rounds to the same fp16 value, which is all that is used:
//   * |t - y/s| <= (2^-23 + 2^-47) |y/s|  (two roundings of 2^-24 each);
//   * a tie point between neighbouring fp16 values is m = M 2^e with M an odd 12-bit integer; for y = Y 2^a,
//     s = S 2^b (Y, S < 2^11) the quotient can only be near m when y - s m is a non-zero multiple of the unit
//     of s m, so |y/s - m| >= m / (S M) > 2^-23 (1 + 2^-11) m -- further away than t can be from y/s;
//     y/s never equals a tie point (S M would need more than 11 bits in y).
// Hence fp16(t) == fp16(y / s) whenever the result is a normal fp16 number; below that every candidate
// rounds to the integer 0 anyway.  The library's self-test (qr_debug_division_check) compares the resulting
// int4 codes with those from IEEE division for every pair of finite fp16 operands.
__device__ __forceinline__ float div_by_scale(float y, float /*s*/, float rcp) { return y * rcp; }

// Two fp16 values (one 32-bit word) -> the word 0x66cc66cc whose bytes 0 and 2 hold the two int4 codes as int8.
// CLAMP = false may be used when |y / s| < 7.5 is known (clip ratio 1 and a scale in the normal fp16 range).
template <bool CLAMP>
__device__ __forceinline__ uint32_t quant2_word(uint32_t hw, float rcp) {
  const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&hw));
  __half2 h = __floats2half2_rn(f.x * rcp, f.y * rcp);
  if (CLAMP) {
    h = __hmax2(h, __float2half2_rn(-8.0f));
    h = __hmin2(h, __float2half2_rn(7.0f));
  }
  h = __hadd2(h, __float2half2_rn(1536.0f));
  return *reinterpret_cast<uint32_t*>(&h);
}

// Four such words (elements 0..7) -> 4 packed bytes: byte j = code(2j) | code(2j+1) << 4.
__device__ __forceinline__ uint32_t pack8_codes(uint32_t u0, uint32_t u1, uint32_t u2, uint32_t u3) {
  const uint32_t p01 = __byte_perm(u0, u1, 0x6240);   // [e0, e2, e1, e3]
  const uint32_t p23 = __byte_perm(u2, u3, 0x6240);   // [e4, e6, e5, e7]
  const uint32_t ev = __byte_perm(p01, p23, 0x5410);  // [e0, e2, e4, e6]
  const uint32_t od = __byte_perm(p01, p23, 0x7632);  // [e1, e3, e5, e7]
  return (ev & 0x0F0F0F0Fu) | ((od << 4) & 0xF0F0F0F0u);
}

// Eight fp16 values (four words) -> four packed bytes with torch's arithmetic.  s is the row scale
// (s == 0 follows torch's x / 0), rcp = RN(1/s); `noclamp` as for quant2_word (must be uniform per row).
__device__ __forceinline__ uint32_t quant8_words(uint32_t h0, uint32_t h1, uint32_t h2, uint32_t h3, float s, float rcp,
                                                 bool noclamp) {
  if (s == 0.0f) {
    uint32_t out = 0;
    const uint32_t hw[4] = {h0, h1, h2, h3};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&hw[e]));
      const uint32_t cd = quant_pair_zero_scale(f.x, f.y);
      out |= ((cd | (cd >> 12)) & 0xFFu) << (8 * e);
    }
    return out;
  }
  if (noclamp)
    return pack8_codes(quant2_word<false>(h0, rcp), quant2_word<false>(h1, rcp), quant2_word<false>(h2, rcp),
                       quant2_word<false>(h3, rcp));
  return pack8_codes(quant2_word<true>(h0, rcp), quant2_word<true>(h1, rcp), quant2_word<true>(h2, rcp),
                     quant2_word<true>(h3, rcp));
}

// The clamp of the codes can be skipped when the clip ratio is 1 and the scale is a normal fp16 number:
// then s >= (absmax / 7)(1 - 2^-11), so |y / s| <= 7.004 and rint gives at most 7 in magnitude.
__device__ __forceinline__ bool clamp_free(float s, float clip) { return clip == 1.0f && s >= 6.103515625e-05f; }

#endif  // __CUDACC__

}  // namespace qr
