// Kernel (a), Kronecker case with a 64-long Walsh factor (n = 64 K, e.g. LLaMA-2-7B down_proj:
// 11008 = 172 x 64): dense factor on the 5th-generation tensor cores, Walsh factor in registers.
//
//   D[k', m] = sum_k hadK[k'][k] * X[k][m]          (tcgen05.mma kind::f16, fp32 accumulate in TMEM)
//   y[k', :] = Walsh_64(D[k', :]) / sqrt(n)         (64 accumulator columns = one thread's registers)
//
// One persistent CTA per SM.  hadK (padded to 128-row tiles and 64-column swizzle atoms) is
// written once into shared memory as the K-major A operand.  A token row is 172 rows of 128 bytes,
// i.e. already the MN-major B operand [k][m]: TMA copies it with the 128-byte swizzle into a ring
// of three buffers and the MMA warp issues ceil(K/16) MMAs per 128-row tile of hadK.  Thread k' of
// the epilogue warps reads its 64 accumulators with tcgen05.ld, runs the 6 butterfly stages in
// registers (no shuffles, no shared memory), scales, rounds to fp16, joins the row-wide absmax
// (per-warp slots published through a bounded mbarrier), quantises with torch's division arithmetic and stores 32 packed bytes.
// Accumulators are double buffered and two sets of epilogue warps take alternate token rows, so the
// MMAs of row i+1 and the epilogue of row i-1 overlap the epilogue of row i.
//
// All mbarrier waits are bounded (see tc_ptx.cuh); on a timeout the CTA sets the device status
// word, leaves its loops, frees tensor memory and returns.
#include "tc_ptx.cuh"

#include <math.h>

namespace qr {

struct HadqTcParams {
  int64_t rows;
  int K;            // order of the dense factor (even, <= 256); n = 64 K
  int MT;           // 128-row tiles of hadK (1 or 2)
  int KT16;         // ceil(K / 16) MMAs per tile and row
  int KA;           // 64-column swizzle atoms of hadK
  int b_bytes;      // bytes of one token-row buffer (KT16 * 16 rows of 128 B, rounded up to 1024)
  const __half* had_k;
  float scale;      // 1 / sqrt(n)
  float clip;
  uint8_t* q;
  __half* scales;
  __half* y_out;
  int do_quant;
  int* status;
};

constexpr int kTcEpiWarps = 8;        // epilogue warps per set; two sets take alternate token rows
constexpr int kTcThreads = 32 * (2 + 2 * kTcEpiWarps);
constexpr int kTcNB = 3;              // token-row buffers
constexpr int kTcNumBars = 2 * kTcNB + 4 + 2;   // full_b, empty_b, acc_full[2], acc_empty[2], red_bar[2]

__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// MN-major operand, 128-byte swizzle: 64 contiguous elements along MN per row, rows are K;
// 8-row groups are `sbo` bytes apart; the MN-atom stride (leading byte offset) is unused for N = 64.
__device__ __forceinline__ uint64_t make_mnmajor_sw128_desc(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// kind::f16: fp16 A (K-major) and B (MN-major), fp32 accumulate.
__host__ __device__ constexpr uint32_t make_idesc_f16_kmn(int umma_m, int umma_n) {
  return (1u << 4) | (0u << 7) | (0u << 10) | (0u << 15) | (1u << 16) |
         ((uint32_t)(umma_n >> 3) << 17) | ((uint32_t)(umma_m >> 4) << 24);
}

template <int N>
__device__ __forceinline__ void fwht_regs_tc(float (&v)[N]) {
#pragma unroll
  for (int h = 1; h < N; h <<= 1) {
#pragma unroll
    for (int i = 0; i < N; ++i) {
      if ((i & h) == 0) {
        const float a = v[i], b = v[i + h];
        v[i] = a + b;
        v[i + h] = a - b;
      }
    }
  }
}

__global__ void __launch_bounds__(kTcThreads, 1)
hadq_tc_kernel(const __grid_constant__ CUtensorMap tmX, const HadqTcParams p) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ unsigned char smem_dyn[];
  const uint32_t smem_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  unsigned char* smem_gen = smem_dyn + (smem_base - smem_u32(smem_dyn));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // layout: [A: KA atoms x (MT*128 rows x 128 B)][B ring][barriers][tmem slot][abort][reduction slots]
  const int a_atom_bytes = p.MT * 128 * 128;
  const int a_bytes = p.KA * a_atom_bytes;
  const uint32_t b_off = (uint32_t)a_bytes;
  const uint32_t bar_off = b_off + kTcNB * p.b_bytes;
  const uint32_t bar_base = smem_base + bar_off;
  auto full_b = [&](int s) { return bar_base + 8u * s; };
  auto empty_b = [&](int s) { return bar_base + 8u * (kTcNB + s); };
  auto acc_full = [&](int a) { return bar_base + 8u * (2 * kTcNB + a); };
  auto acc_empty = [&](int a) { return bar_base + 8u * (2 * kTcNB + 2 + a); };
  auto red_bar = [&](int b) { return bar_base + 8u * (2 * kTcNB + 4 + b); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + bar_off + 8 * kTcNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + bar_off + 8 * kTcNumBars + 8);
  volatile float* red = reinterpret_cast<volatile float*>(smem_gen + bar_off + 8 * kTcNumBars + 16);   // [2][kTcEpiWarps]

  // ---- one-time set-up: hadK -> swizzled K-major A tiles (zero padded), zero the k padding rows of B
  {
    const int rows = p.MT * 128, K = p.K;
    const int chunks = rows * p.KA * 8;                       // 16-byte chunks of the A operand
    for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
      const int ka = c / (rows * 8);
      const int rem = c - ka * rows * 8;
      const int r = rem >> 3, ch = rem & 7;
      uint4 v = make_uint4(0, 0, 0, 0);
      const int c0 = ka * 64 + ch * 8;                        // first hadK column of this chunk
      if (r < K && c0 < K) {
        __align__(16) __half tmp[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) tmp[e] = (c0 + e < K) ? p.had_k[(size_t)r * K + c0 + e] : __float2half(0.0f);
        v = *reinterpret_cast<const uint4*>(tmp);
      }
      *reinterpret_cast<uint4*>(smem_gen + ka * a_atom_bytes + r * 128 + ((ch ^ (r & 7)) << 4)) = v;
    }
    const int pad_rows = p.KT16 * 16 - K;
    for (int c = threadIdx.x; c < kTcNB * pad_rows * 8; c += blockDim.x) {
      const int s = c / (pad_rows * 8);
      const int rem = c - s * pad_rows * 8;
      *reinterpret_cast<uint4*>(smem_gen + b_off + s * p.b_bytes + (K + (rem >> 3)) * 128 + ((rem & 7) << 4)) =
          make_uint4(0, 0, 0, 0);
    }
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < kTcNB; ++s) { mbar_init(full_b(s), 1); mbar_init(empty_b(s), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(acc_full(a), 1); mbar_init(acc_empty(a), kTcEpiWarps); mbar_init(red_bar(a), kTcEpiWarps); }
    *abort_flag = 0;
    fence_mbar_init();
  }
  constexpr uint32_t kTmemCols = 256;   // 2 row buffers x 2 tiles x 64 columns
  if (warp == 1) {
    tmem_alloc(smem_base + bar_off + 8 * kTcNumBars, kTmemCols);
    tmem_relinquish();
  }
  fence_proxy_async_smem();   // A tiles and zeroed padding were written with ordinary stores
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer: one token row per buffer
    if (lane == 0) {
      uint32_t i = 0;
      for (int64_t row = blockIdx.x; row < p.rows; row += gridDim.x, ++i) {
        const int s = i % kTcNB;
        if (!mbar_wait(empty_b(s), ((i / kTcNB) & 1) ^ 1, abort_flag, p.status, 31)) break;
        mbar_expect_tx(full_b(s), (uint32_t)p.K * 128u);
        tma_load_2d(smem_base + b_off + s * p.b_bytes, &tmX, full_b(s), 0, (int)(row * p.K));
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_f16_kmn(128, 64);
      uint32_t i = 0;
      for (int64_t row = blockIdx.x; row < p.rows; row += gridDim.x, ++i) {
        const int s = i % kTcNB, a = i & 1;
        if (!mbar_wait(full_b(s), (i / kTcNB) & 1, abort_flag, p.status, 32)) break;
        if (!mbar_wait(acc_empty(a), ((i >> 1) & 1) ^ 1, abort_flag, p.status, 33)) break;
        tc_fence_after();
        const uint32_t b_addr = smem_base + b_off + s * p.b_bytes;
        for (int mt = 0; mt < p.MT; ++mt) {
          const uint32_t d_tmem = tmem_base + a * 128 + mt * 64;
          for (int j = 0; j < p.KT16; ++j) {
            const uint32_t a_addr = smem_base + (j >> 2) * a_atom_bytes + mt * (128 * 128) + (j & 3) * 32;
            const uint64_t da = make_kmajor_sw128_desc(a_addr);
            const uint64_t db = make_mnmajor_sw128_desc(b_addr + j * 2048, (uint32_t)p.b_bytes, 1024);
            umma_f16(d_tmem, da, db, idesc, j != 0 ? 1u : 0u);
          }
        }
        umma_commit(empty_b(s));
        umma_commit(acc_full(a));
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue: thread = output row k'
    const int set = (warp - 2) >> 3;           // set 0 drains accumulator buffer 0 (even rows), set 1 buffer 1
    const int ew = (warp - 2) & 7;
    const int mt = ew >> 2, q4 = warp & 3;
    const int kprime = mt * 128 + q4 * 32 + lane;
    const bool warp_active = (mt * 128 + q4 * 32) < p.K && mt < p.MT;
    const bool active = kprime < p.K && mt < p.MT;
    const int n = p.K * 64;
    uint32_t i = set;
    for (int64_t row = blockIdx.x + (int64_t)set * gridDim.x; row < p.rows; row += 2 * (int64_t)gridDim.x, i += 2) {
      const int a = i & 1;
      __half2 h[32];
      float amax = 0.0f;
      bool ok = mbar_wait(acc_full(a), (i >> 1) & 1, abort_flag, p.status, 34);
      if (!ok) break;
      tc_fence_after();
      if (warp_active) {
        float v[64];
        {
          uint32_t r[32];
          const uint32_t taddr = tmem_base + ((uint32_t)(q4 * 32) << 16) + (uint32_t)(a * 128 + mt * 64);
          tmem_ld32(taddr, r);
#pragma unroll
          for (int e = 0; e < 32; ++e) v[e] = __uint_as_float(r[e]);
          tmem_ld32(taddr + 32, r);
#pragma unroll
          for (int e = 0; e < 32; ++e) v[32 + e] = __uint_as_float(r[e]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_empty(a));
        fwht_regs_tc<64>(v);
        __half2 mx = __float2half2_rn(0.0f);
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          h[e] = __floats2half2_rn(v[2 * e] * p.scale, v[2 * e + 1] * p.scale);
          mx = __hmax2(mx, __habs2(h[e]));
        }
        if (active) {
          const float2 mf = __half22float2(mx);
          amax = fmaxf(mf.x, mf.y);
          if (p.y_out) {
            uint4* yo = reinterpret_cast<uint4*>(p.y_out + row * (int64_t)n + kprime * 64);
#pragma unroll
            for (int e = 0; e < 8; ++e) yo[e] = *reinterpret_cast<const uint4*>(&h[4 * e]);
          }
        }
      } else {
        if (lane == 0) mbar_arrive(acc_empty(a));
      }
      if (p.do_quant) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        // row-wide absmax: one slot per warp, published through a (bounded) mbarrier
        volatile float* slots = red + (i & 1) * kTcEpiWarps;
        if (lane == 0) { slots[ew] = amax; mbar_arrive(red_bar(i & 1)); }
        if (!mbar_wait(red_bar(i & 1), (i >> 1) & 1, abort_flag, p.status, 35)) break;
        float amx = 0.0f;
#pragma unroll
        for (int w = 0; w < kTcEpiWarps; ++w) amx = fmaxf(amx, slots[w]);
        const __half s7 = __float2half_rn(__fdiv_rn(amx, 7.0f));
        const __half sh = __float2half_rn(__half2float(s7) * p.clip);
        const float s = __half2float(sh);
        if (ew == 0 && lane == 0) p.scales[row] = sh;
        if (active) {
          const float rcp = (s != 0.0f) ? __frcp_rn(s) : 0.0f;
          const bool noclamp = clamp_free(s, p.clip);
          const uint32_t* hw = reinterpret_cast<const uint32_t*>(h);
          uint32_t w4[8];
#pragma unroll
          for (int g = 0; g < 8; ++g)
            w4[g] = quant8_words(hw[4 * g], hw[4 * g + 1], hw[4 * g + 2], hw[4 * g + 3], s, rcp, noclamp);
          uint4* qo = reinterpret_cast<uint4*>(p.q + row * (int64_t)(n >> 1) + kprime * 32);
          qo[0] = make_uint4(w4[0], w4[1], w4[2], w4[3]);
          qo[1] = make_uint4(w4[4], w4[5], w4[6], w4[7]);
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

typedef CUresult (*EncodeTiledFnTc)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Launches the tensor-core Kronecker kernel.  Returns QR_EUNSUPPORTED (without setting an error
// message that matters) when the shape is outside what it covers, so the caller can fall back.
int launch_hadq_tc(const void* x, int64_t rows, int n, int K, const void* had_k, float clip, uint8_t* q,
                   void* scales, void* y_out, int do_quant, cudaStream_t st) {
  if (K < 2 || K > 256 || (K & 1) || n != 64 * K || !aligned16(x)) return QR_EUNSUPPORTED;
  if (rows * (int64_t)K > 0x7fffffffLL) return QR_EUNSUPPORTED;
  int* status = kernel_status_ptr();
  if (!status) return fail(QR_ENOTREADY, "hadamard: no CUDA device");
  static EncodeTiledFnTc encode = nullptr;
  if (!encode) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      return fail(QR_ENOTREADY, "cuTensorMapEncodeTiled is not available from this driver");
    encode = reinterpret_cast<EncodeTiledFnTc>(ptr);
  }
  CUtensorMap tm;
  cuuint64_t dims[2] = {64, (cuuint64_t)(rows * K)};
  cuuint64_t strides[1] = {128};
  cuuint32_t box[2] = {64, (cuuint32_t)K};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = encode(&tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(x), dims, strides, box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(QR_EINVAL, "hadamard: cuTensorMapEncodeTiled failed with CUresult %d", (int)r);

  HadqTcParams p;
  p.rows = rows; p.K = K; p.MT = (K + 127) / 128; p.KT16 = (K + 15) / 16; p.KA = (K + 63) / 64;
  p.had_k = reinterpret_cast<const __half*>(had_k);
  p.scale = (float)(1.0 / sqrt((double)n)); p.clip = clip; p.q = q;
  p.scales = reinterpret_cast<__half*>(scales); p.y_out = reinterpret_cast<__half*>(y_out);
  p.do_quant = do_quant; p.status = status;
  p.b_bytes = (p.KT16 * 16 * 128 + 1023) & ~1023;
  const int smem = p.KA * p.MT * 128 * 128 + kTcNB * p.b_bytes + 8 * kTcNumBars + 16 + 2 * kTcEpiWarps * 4 + 1024 + 64;
  if (smem > 227 * 1024) return QR_EUNSUPPORTED;
  static thread_local int configured[64] = {0};
  int dev = 0;
  QR_CUDA(cudaGetDevice(&dev));
  if (dev >= 64 || configured[dev] < smem) {
    QR_CUDA(cudaFuncSetAttribute(hadq_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    if (dev < 64) configured[dev] = smem;
  }
  int64_t grid = num_sms();
  if (grid > rows) grid = rows;
  QR_CUDA(launch_kernel(hadq_tc_kernel, dim3((int)grid), dim3(kTcThreads), (size_t)smem, st, tuning("pdl", 0) != 0, tm, p));
  return QR_OK;
}

}  // namespace qr
