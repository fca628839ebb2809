// Kernel (a), Kronecker case with a 64-long Walsh factor (n = 64 K, e.g. LLaMA-2-7B down_proj:
// 11008 = 172 x 64): dense factor on the 5th-generation tensor cores, Walsh factor in registers.
//
//   D[k', m] = sum_k hadK[k'][k] * X[k][m]          (tcgen05.mma kind::f16, fp32 accumulate in TMEM)
//   y[k', :] = Walsh_64(D[k', :]) / sqrt(n)         (64 accumulator columns = one thread's registers)
//
// One persistent CTA per SM.  hadK (padded to 128-row tiles and 64-column swizzle atoms) is
// written once into shared memory as the K-major A operand.  A token row is 172 rows of 128 bytes,
// i.e. already the MN-major B operand [k][m].  The unit of work is a PAIR of consecutive token rows:
// TMA copies both with the 128-byte swizzle into one stage of a two-stage ring, and the MMA warp issues
// ceil(K/16) MMAs of N = 128 (two 64-column atoms, one per token row) per 128-row tile of hadK,
// alternating between the tiles so that two independent accumulation chains are in flight (short MMAs
// chained on one accumulator run at the latency of the tensor pipe, not at its throughput).
// Thread k' of an epilogue warp reads its 64 accumulators with tcgen05.ld, runs the 6 butterfly stages in
// registers (no shuffles, no shared memory), scales, rounds to fp16, joins the row-wide absmax
// (per-warp slots published through a bounded mbarrier), quantises with torch's division arithmetic and
// stores 32 packed bytes.  Two sets of epilogue warps take the two rows of a pair; accumulators are
// double buffered, so the MMAs of pair i+1 overlap the epilogue of pair i.
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

constexpr int kTcEpiWarps = 8;        // epilogue warps per set; set r takes row r of every pair of token rows
constexpr int kTcThreads = 32 * (2 + 2 * kTcEpiWarps);
constexpr int kTcNB = 2;              // ring stages, each holding a pair of token rows
constexpr int kTcNumBars = 2 * kTcNB + 4 + 2;   // full_b, empty_b, acc_full[2], acc_empty[2], red_bar[2]

__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// The same MMA with the operand descriptors as (low word, shared high word), see tc_ptx.cuh.  ACC = 1 accumulates,
// ACC = -1 takes the decision from `accumulate` at run time.
template <int ACC>
__device__ __forceinline__ void umma_f16_w(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t hi, uint32_t idesc,
                                           uint32_t accumulate = 1u) {
  if (ACC < 0) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 da, {%1, %3};\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(hi), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 da, {%1, %3};\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(hi), "r"(idesc), "n"(ACC)
        : "memory");
  }
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

  // layout: [A: KA atoms x (MT*128 rows x 128 B)][B ring: kTcNB stages x 2 token rows][barriers][tmem slot][abort][reduction slots]
  const int a_atom_bytes = p.MT * 128 * 128;
  const int a_bytes = p.KA * a_atom_bytes;
  const uint32_t b_off = (uint32_t)a_bytes;
  const uint32_t bar_off = b_off + 2 * kTcNB * p.b_bytes;
  const uint32_t bar_base = smem_base + bar_off;
  auto full_b = [&](int s) { return bar_base + 8u * s; };
  auto empty_b = [&](int s) { return bar_base + 8u * (kTcNB + s); };
  auto acc_full = [&](int a) { return bar_base + 8u * (2 * kTcNB + a); };
  auto acc_empty = [&](int a) { return bar_base + 8u * (2 * kTcNB + 2 + a); };
  auto red_bar = [&](int b) { return bar_base + 8u * (2 * kTcNB + 4 + b); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + bar_off + 8 * kTcNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + bar_off + 8 * kTcNumBars + 8);
  volatile float* red = reinterpret_cast<volatile float*>(smem_gen + bar_off + 8 * kTcNumBars + 16);   // [2 sets][2][kTcEpiWarps]

  if (threadIdx.x == 0) {
    for (int s = 0; s < kTcNB; ++s) { mbar_init(full_b(s), 1); mbar_init(empty_b(s), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(acc_full(a), 1); mbar_init(acc_empty(a), 2 * kTcEpiWarps); mbar_init(red_bar(a), kTcEpiWarps); }
    *abort_flag = 0;
    fence_mbar_init();
  }
  constexpr uint32_t kTmemCols = 512;   // 2 pair buffers x 2 tiles x (2 rows x 64 columns)
  if (warp == 1) {
    tmem_alloc(smem_base + bar_off + 8 * kTcNumBars, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int64_t npairs = (p.rows + 1) >> 1;

  if (warp != 0) {
    // ---- one-time set-up by all warps but the producer (which already streams token rows in):
    // hadK -> swizzled K-major A tiles (zero padded), zero the k padding rows of the token-row buffers
    const int t = threadIdx.x - 32, nt = kTcThreads - 32;
    const int rows = p.MT * 128, K = p.K;
    const bool dup_rows = p.MT == 2 && K - 128 <= 64;
    const int chunks = rows * p.KA * 8;                       // 16-byte chunks of the A operand
    const bool vec = (K & 3) == 0 && ((reinterpret_cast<uintptr_t>(p.had_k) & 7) == 0);
    // twelve chunks per thread and round (one round for K <= 172): all loads of a round are issued before its
    // stores, so the set-up costs one trip to L2 instead of one per chunk
    constexpr int kU = 12;
    const int row_shift = 10 + (p.MT - 1);                    // log2(rows * 8)
    for (int c_base = t; c_base < chunks; c_base += kU * nt) {
      uint2 lo[kU], hi[kU];
      uint32_t dst[kU];
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const int c = c_base + u * nt;
        lo[u] = make_uint2(0, 0);
        hi[u] = make_uint2(0, 0);
        dst[u] = 0xFFFFFFFFu;
        if (c < chunks) {
          const int ka = c >> row_shift;
          const int rem = c - (ka << row_shift);
          const int r = rem >> 3, ch = rem & 7;
          const int c0 = ka * 64 + ch * 8;                      // first hadK column of this chunk
          dst[u] = (uint32_t)(ka * a_atom_bytes + r * 128 + ((ch ^ (r & 7)) << 4));
          // second copy of the rows of the second tile, 64 rows further down (see the epilogue)
          const int hr = (dup_rows && r >= 192) ? r - 64 : r;
          if (hr < K && c0 < K && (hr == r || hr >= 128)) {
            const __half* src = p.had_k + (size_t)hr * K + c0;
            if (vec) {      // K % 4 == 0: the chunk starts on an 8-byte boundary and holds 4 or 8 valid columns
              lo[u] = __ldg(reinterpret_cast<const uint2*>(src));
              if (c0 + 8 <= K) hi[u] = __ldg(reinterpret_cast<const uint2*>(src + 4));
            } else {
              __align__(16) __half tmp[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) tmp[e] = (c0 + e < K) ? src[e] : __float2half(0.0f);
              const uint4 v = *reinterpret_cast<const uint4*>(tmp);
              lo[u] = make_uint2(v.x, v.y);
              hi[u] = make_uint2(v.z, v.w);
            }
          }
        }
      }
#pragma unroll
      for (int u = 0; u < kU; ++u)
        if (dst[u] != 0xFFFFFFFFu)
          *reinterpret_cast<uint4*>(smem_gen + dst[u]) = make_uint4(lo[u].x, lo[u].y, hi[u].x, hi[u].y);
    }
    const int pad_rows = p.KT16 * 16 - K;
    for (int c = t; c < 2 * kTcNB * pad_rows * 8; c += nt) {
      const int s = c / (pad_rows * 8);
      const int rem = c - s * pad_rows * 8;
      *reinterpret_cast<uint4*>(smem_gen + b_off + s * p.b_bytes + (K + (rem >> 3)) * 128 + ((rem & 7) << 4)) =
          make_uint4(0, 0, 0, 0);
    }
    fence_proxy_async_smem();   // A tiles and zeroed padding were written with ordinary stores
    asm volatile("bar.sync 1, %0;" ::"n"(kTcThreads - 32) : "memory");
  }

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer: a pair of token rows per stage
    if (lane == 0) {
      uint32_t i = 0;
      for (int64_t pair = blockIdx.x; pair < npairs; pair += gridDim.x, ++i) {
        const int s = i % kTcNB;
        if (!mbar_wait(empty_b(s), ((i / kTcNB) & 1) ^ 1, abort_flag, p.status, 31)) break;
        const bool two = 2 * pair + 1 < p.rows;
        mbar_expect_tx(full_b(s), (uint32_t)p.K * 128u * (two ? 2u : 1u));
        const uint32_t dst = smem_base + b_off + (2 * s) * p.b_bytes;
        tma_load_2d(dst, &tmX, full_b(s), 0, (int)(2 * pair * p.K));
        if (two) tma_load_2d(dst + p.b_bytes, &tmX, full_b(s), 0, (int)((2 * pair + 1) * p.K));
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_f16_kmn(128, 128);
      uint32_t i = 0;
      for (int64_t pair = blockIdx.x; pair < npairs; pair += gridDim.x, ++i) {
        const int s = i % kTcNB, a = i & 1;
        if (!mbar_wait(full_b(s), (i / kTcNB) & 1, abort_flag, p.status, 32)) break;
        if (!mbar_wait(acc_empty(a), ((i >> 1) & 1) ^ 1, abort_flag, p.status, 33)) break;
        tc_fence_after();
        // Lean issue loop (one thread; every dependent integer instruction costs several cycles): descriptors are
        // (low word, constant high word) pairs advanced by 32-bit adds.  A: k step = +32 bytes inside a 64-column
        // atom, next atom a_atom_bytes further, second hadK tile 16 KB further.  B: k step = 16 rows of 128 bytes;
        // its low word also carries the distance between the two token rows (leading byte offset).
        const int kt_n = p.KT16;
        const bool two_tiles = p.MT > 1;
        const uint32_t d0 = tmem_base + a * 256;
        uint32_t a_lo = desc_lo(smem_base);
        uint32_t b_lo = desc_lo(smem_base + b_off + (2 * s) * p.b_bytes) | ((((uint32_t)p.b_bytes >> 4) & 0x3FFFu) << 16);
        const uint32_t a_atom_step = (uint32_t)a_atom_bytes >> 4;
        int j = 0;
        for (int ja = 0; ja < p.KA; ++ja, a_lo += a_atom_step, b_lo += 4 * 128) {
#pragma unroll
          for (int jj = 0; jj < 4; ++jj, ++j) {
            if (j < kt_n) {
              if (jj == 0) {
                umma_f16_w<-1>(d0, a_lo, b_lo, kDescHiKmajorSw128, idesc, ja != 0 ? 1u : 0u);
                if (two_tiles) umma_f16_w<-1>(d0 + 128, a_lo + 1024, b_lo, kDescHiKmajorSw128, idesc, ja != 0 ? 1u : 0u);
              } else {
                umma_f16_w<1>(d0, a_lo + 2 * jj, b_lo + 128 * jj, kDescHiKmajorSw128, idesc);
                if (two_tiles) umma_f16_w<1>(d0 + 128, a_lo + 2 * jj + 1024, b_lo + 128 * jj, kDescHiKmajorSw128, idesc);
              }
            }
          }
        }
        umma_commit(empty_b(s));
        umma_commit(acc_full(a));
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue: thread = output row k'
    const int set = (warp - 2) >> 3;           // set r handles row r of every pair
    const int ew = (warp - 2) & 7;
    const int mt = ew >> 2, q4 = warp & 3;
    // Scheduler balance: a warp's tensor-memory lanes (and its scheduler) follow from its id modulo 4.  When the second
    // tile of hadK holds at most 64 rows (172 = 128 + 44), the set-up wrote them twice, at rows 0 .. and 64 .. of the
    // tile, so that the warps of set 0 read them from lane quarters 0 and 1 and those of set 1 from quarters 2 and 3:
    // every scheduler then carries three busy epilogue warps per pair of token rows instead of four on two of them
    // and two on the others.
    const bool dup_rows = p.MT == 2 && p.K - 128 <= 64;
    const int q_row = (dup_rows && mt == 1 && set == 1) ? q4 - 2 : q4;      // quarter of the tile's rows this warp finishes
    const int kprime = mt * 128 + q_row * 32 + lane;
    const bool warp_active = q_row >= 0 && (mt * 128 + q_row * 32) < p.K && mt < p.MT;
    const bool active = q_row >= 0 && kprime < p.K && mt < p.MT;
    const int n = p.K * 64;
    uint32_t i = 0;
    for (int64_t pair = blockIdx.x; pair < npairs; pair += gridDim.x, ++i) {
      const int a = i & 1;
      const int64_t row = 2 * pair + set;
      __half2 h[32];
      float amax = 0.0f;
      bool ok = mbar_wait(acc_full(a), (i >> 1) & 1, abort_flag, p.status, 34);
      if (!ok) break;
      tc_fence_after();
      if (row >= p.rows) {      // odd row count: the last pair has no second row
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_empty(a));
        continue;
      }
      if (warp_active) {
        float v[64];
        {
          uint32_t r[32];
          const uint32_t taddr = tmem_base + ((uint32_t)(q4 * 32) << 16) + (uint32_t)(a * 256 + mt * 128 + set * 64);
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
        // each set has its own barrier; the slots alternate between pairs so that a fast warp cannot overwrite
        // a value that a slow warp of the same set has not read yet
        volatile float* slots = red + (set * 2 + (i & 1)) * kTcEpiWarps;
        if (lane == 0) { slots[ew] = amax; mbar_arrive(red_bar(set)); }
        if (!mbar_wait(red_bar(set), i & 1, abort_flag, p.status, 35)) break;
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

  drain_after_abort(abort_flag);
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
  const int smem = p.KA * p.MT * 128 * 128 + 2 * kTcNB * p.b_bytes + 8 * kTcNumBars + 16 + 4 * kTcEpiWarps * 4 + 1024 + 64;
  if (smem > 227 * 1024) return QR_EUNSUPPORTED;
  static thread_local int configured[64] = {0};
  int dev = 0;
  QR_CUDA(cudaGetDevice(&dev));
  if (dev >= 64 || configured[dev] < smem) {
    QR_CUDA(cudaFuncSetAttribute(hadq_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    if (dev < 64) configured[dev] = smem;
  }
  int64_t grid = num_sms();
  if (grid > (rows + 1) / 2) grid = (rows + 1) / 2;
  QR_CUDA(launch_kernel(hadq_tc_kernel, dim3((int)grid), dim3(kTcThreads), (size_t)smem, st, use_pdl(rows), tm, p));
  return QR_OK;
}

}  // namespace qr
