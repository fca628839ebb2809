// Kernel (b) for 1 .. 32 token rows: the weight-streaming GEMV with warp-level tensor-core MMAs.
//
// With this few token rows the layer is one pass over the packed weights, and what the tcgen05 kernel of
// gemm_i4_decode.cu pays per launch (tensor-memory allocation, TMA ring fill, an MMA instruction of 100+ cycles per
// 32 K values and 128 weight rows) is more than the pass itself.  The CUDA-core GEMV of gemv_i4.cu has none of that
// but runs out of dp4a throughput above four rows.  This kernel keeps its structure -- weights from global memory
// straight into registers, widened there, token rows packed in shared memory -- and replaces dp4a by
// mma.sync.m16n8k32.s8 (measured on this GPU: one per 8 cycles and scheduler, 2048 MACs per cycle and SM; the
// pass needs a fifth of that at memory speed).
//
// Mapping.  A warp owns 16 output channels (weight rows n0 .. n0 + 15).  In the m16n8k32 A fragment lane (g, t),
// g = lane / 4, t = lane % 4, holds rows g and g + 8 and, of each, eight of the 32 k values as two int8x4 registers.
// Which k values a register holds is free as long as the B fragment follows the same rule, so lane (g, t) simply
// loads the t-th 16-byte chunk of a 64-byte piece of its two weight rows, and word j of that chunk, widened with the
// x16 trick of the other kernels ((w << 4) & 0xF0F0F0F0 = the even nibbles, w & 0xF0F0F0F0 = the odd ones, as int8
// with a factor 16), is the register pair of MMA j: one 16-byte load per row feeds four MMAs.  The B fragment of
// lane (g, t) is token row g at the same chunk and word: one 16-byte shared-memory load per four MMAs (token rows are
// padded by 64 bytes so that the eight rows of a quarter-warp fall into different banks).  Further B fragments
// serve token rows 8 .. 15 and 16 .. 31.  The accumulators are 256 x the dot products, as everywhere else, and the epilogue is
// the arithmetic of the other forms of kernel (b): bit-identical results.
//
// Parallelism and balance.  Two persistent CTAs of eight warps per SM, or one of sixteen (two halves that take
// alternate groups of rows and share only the token rows); the weight rows are dealt out to the
// CTAs as contiguous ranges of N / CTAs rows (any number: every SM streams the same number of bytes), a CTA walks
// its range in groups of 16 rows (rows of the last group beyond the range are not loaded and their accumulators are
// not stored), and its eight warps split the K range of every group eight ways; their partial fragments meet in
// shared memory behind one barrier per group (two alternating areas), after which all threads add up and store one
// element each.  Every lane holds four (eight for long rows) 64-byte pieces of its two rows in a rotating register
// buffer: a slot is refilled with the piece that many pieces ahead as soon as its MMAs have been issued, also across
// groups, so three to four (seven to eight) pieces per row and lane are always in flight.  The token rows come in
// as one bulk copy per row on the TMA unit.
#include "common.cuh"
#include "tc_ptx.cuh"

namespace qr {

struct GemvMmaParams {
  const uint8_t* A;      // [M, K/2] packed token rows
  const uint8_t* B;      // [N, K/2] packed weights
  const __half* sA;      // [M] or null (int32 mode)
  const __half* sB;      // [N] or null
  const __half* bias;    // [N] or null
  void* out;             // [M, N] fp16 (ldo) or int32
  int64_t ldo;
  int M, N, K;
  int a_stride;          // bytes between token rows in shared memory (K / 2 + 64)
  int red_areas;         // reduction areas per half of the CTA: 2 (alternating, one barrier per group), or 1 where
                         // shared memory is short (a second barrier per group protects the area)
  int* status;           // device status word: a wait that ran out of time leaves its code there
};

constexpr int kGmWarps = 8;
constexpr int kGmThreads = 32 * kGmWarps;
#ifndef GM_U
#define GM_U 8
#endif
#ifndef GM_MINB
#define GM_MINB 2
#endif
constexpr int U = GM_U;    // 64-byte pieces per row that a lane keeps in flight

__device__ __forceinline__ uint4 gm_ld_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// Untiled bulk copy global -> shared memory on the TMA unit; both addresses 16-byte aligned, the size a multiple of 16.
__device__ __forceinline__ void gm_bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

__device__ __forceinline__ void mma_s8_16832(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// NF: fragments of eight token rows (1: M <= 8, 2: M <= 16, 4: M <= 32)
// U: 64-byte pieces per row that a lane keeps in flight (4, or 8 where a warp's slice of K is a multiple of eight pieces)
// H: halves of a CTA.  Where the token rows leave room for one CTA per SM only, that CTA has sixteen warps: two halves
//    of eight that take alternate groups of rows and share nothing but the token rows (own reduction areas, own
//    named barrier), so the SM keeps as many warps and as many loads in flight as with two CTAs.
template <int NF, bool F16, int U, int H>
__global__ void __launch_bounds__(kGmThreads * H, 2 / H)
gemv_mma_i4_kernel(const GemvMmaParams p) {
  constexpr int MT = 8 * NF;
  constexpr int kFrag = NF * 4 * 32;                           // ints of one warp's accumulator fragments
  extern __shared__ __align__(16) unsigned char gm_smem[];     // MT padded token rows, then two reduction areas
  __shared__ float s_scale[MT];
  __shared__ __align__(8) uint64_t s_rows_bar;                 // completes when the token rows have landed
  __shared__ int s_abort;
  const int kbytes = p.K >> 1;
  const int nchunks = kbytes >> 4;
  const int warp = (threadIdx.x >> 5) & (kGmWarps - 1), lane = threadIdx.x & 31;    // warp: index within the half
  const int half = H > 1 ? (int)(threadIdx.x / kGmThreads) : 0;
  const int htid = threadIdx.x & (kGmThreads - 1);
  const int g = lane >> 2, t = lane & 3;
  pdl_launch_dependents();   // the next kernel of the stream may be brought up; it waits for this grid to finish
  const uint32_t rows_bar = smem_u32(&s_rows_bar);
  if (threadIdx.x == 0) {
    mbar_init(rows_bar, 1);
    s_abort = 0;
    fence_mbar_init();
  }

  // this CTA's rows, this warp's slice of K (a multiple of the four chunks a warp takes per row and step)
  const int row_begin = (int)((long long)blockIdx.x * p.N / gridDim.x);
  const int row_end = (int)((long long)(blockIdx.x + 1) * p.N / gridDim.x);
  const int cps = (((nchunks + kGmWarps - 1) / kGmWarps) + 3) & ~3;
  const int c_begin = warp * cps;
  const int c_end = (c_begin + cps < nchunks) ? c_begin + cps : nchunks;
  const int steps = c_begin < c_end ? (c_end - c_begin + 3) >> 2 : 0;
  const int iters = (steps + U - 1) / U;

  // piece u of iteration it of the group of rows at rb: 16 bytes of rows rb + g and rb + g + 8
  auto load_piece = [&](int rb, int it, int u, uint4 (&w)[2]) {
    const int r0 = rb + g, r1 = r0 + 8;
    const int c = c_begin + ((it * U + u) << 2) + t;
    const bool ok = c < c_end;
    w[0] = (ok && r0 < row_end) ? gm_ld_stream16(p.B + (size_t)r0 * kbytes + (size_t)c * 16) : make_uint4(0, 0, 0, 0);
    w[1] = (ok && r1 < row_end) ? gm_ld_stream16(p.B + (size_t)r1 * kbytes + (size_t)c * 16) : make_uint4(0, 0, 0, 0);
  };

  uint4 cur[U][2];
  // The weights do not depend on the kernel in front: the first pieces are requested before the programmatic-
  // dependency wait and before the token rows are staged.
  const int first_rb = row_begin + 16 * half;
  if (first_rb < row_end && iters > 0) {
#pragma unroll
    for (int u = 0; u < U; ++u) load_piece(first_rb, 0, u, cur[u]);
  }
  pdl_wait();   // token rows, scales and the output belong to the preceding kernels
  // The token rows come in as one bulk copy each (the TMA unit moves them while the warps wait for nothing else:
  // a loop of loads and stores would pay one trip to the L2 per few chunks); rows beyond M are zero.
  if (threadIdx.x == 0) {
    mbar_expect_tx(rows_bar, (uint32_t)p.M * (uint32_t)kbytes);
    for (int m = 0; m < p.M; ++m)
      gm_bulk_load(smem_u32(gm_smem + (size_t)m * p.a_stride), p.A + (size_t)m * kbytes, (uint32_t)kbytes, rows_bar);
  }
  for (int i = threadIdx.x; i < (MT - p.M) * nchunks; i += kGmThreads * H) {
    const int m = p.M + i / nchunks, c = i % nchunks;
    *reinterpret_cast<uint4*>(gm_smem + (size_t)m * p.a_stride + (size_t)c * 16) = make_uint4(0, 0, 0, 0);
  }
  if (F16 && threadIdx.x < MT) s_scale[threadIdx.x] = threadIdx.x < p.M ? __half2float(p.sA[threadIdx.x]) : 0.0f;
  __syncthreads();
  // bounded wait; if it runs out of time the status word says so and the whole CTA leaves (nothing else is in flight)
  if (!__syncthreads_and(mbar_wait(rows_bar, 0, &s_abort, p.status, 61) ? 1 : 0)) return;
  int* red = reinterpret_cast<int*>(gm_smem + (size_t)MT * p.a_stride) + half * (p.red_areas * kGmWarps * kFrag);   // [half][area][warp][kFrag]
  auto half_barrier = [&]() {
    if (H > 1) asm volatile("bar.sync %0, %1;" ::"r"(1 + half), "r"(kGmThreads) : "memory");   // this half only
    else __syncthreads();
  };

  int parity = 0;
  for (int rb = first_rb; rb < row_end; rb += 16 * H, parity ^= (p.red_areas - 1)) {
    int acc[NF][4];
#pragma unroll
    for (int f = 0; f < NF; ++f)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[f][e] = 0;
    // channel scale and bias of the elements this thread will finish: requested now, needed behind the barrier
    constexpr int kFin = (kFrag + kGmThreads - 1) / kGmThreads;
    float fin_scale[kFin];
    __half fin_bias[kFin];
    if (F16) {
#pragma unroll
      for (int q = 0; q < kFin; ++q) {
        const int i = htid + q * kGmThreads;
        const int n = rb + ((i & 31) >> 2) + ((((i >> 5) & 3) >> 1) << 3);
        const bool live = i < kFrag && n < row_end;
        fin_scale[q] = live ? __half2float(__ldg(p.sB + n)) : 0.0f;
        fin_bias[q] = (live && p.bias) ? __ldg(p.bias + n) : __float2half(0.0f);
      }
    }
#pragma unroll 1
    for (int it = 0; it < iters; ++it) {
      const bool more = it + 1 < iters, next_group = rb + 16 * H < row_end;
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int c = c_begin + ((it * U + u) << 2) + t;
        // chunks at or beyond c_end meet zero weights; the address stays inside the padded token row
        const int cc = c < nchunks ? c : 0;
        uint4 xa[NF];
#pragma unroll
        for (int f = 0; f < NF; ++f)
          xa[f] = *reinterpret_cast<const uint4*>(gm_smem + (size_t)(8 * f + g) * p.a_stride + (size_t)cc * 16);
        const uint32_t w0[4] = {cur[u][0].x, cur[u][0].y, cur[u][0].z, cur[u][0].w};
        const uint32_t w1[4] = {cur[u][1].x, cur[u][1].y, cur[u][1].z, cur[u][1].w};
        // word j of the chunks feeds MMA j of every fragment; consecutive MMAs go to different accumulators
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint32_t a0 = (w0[j] << 4) & 0xF0F0F0F0u, a1 = (w1[j] << 4) & 0xF0F0F0F0u;
          const uint32_t a2 = w0[j] & 0xF0F0F0F0u, a3 = w1[j] & 0xF0F0F0F0u;
#pragma unroll
          for (int f = 0; f < NF; ++f) {
            const uint32_t xw = j == 0 ? xa[f].x : j == 1 ? xa[f].y : j == 2 ? xa[f].z : xa[f].w;
            mma_s8_16832(acc[f], a0, a1, a2, a3, (xw << 4) & 0xF0F0F0F0u, xw & 0xF0F0F0F0u);
          }
        }
        // the slot is free again: it takes the piece that is U pieces ahead (of this group, or the first of the next
        // group), so every lane always has U - 1 or U pieces of its two rows in flight
        if (more) load_piece(rb, it + 1, u, cur[u]);
        else if (next_group) load_piece(rb + 16 * H, 0, u, cur[u]);
      }
    }
    // the eight partial fragments meet in shared memory; the areas alternate, so one barrier per group is enough
    // (taking the sums one group later behind mbarriers instead was measured slower: 7.3 against 6.95 us for the 7B
    // qkv layer)
    int* area = red + parity * (kGmWarps * kFrag);
#pragma unroll
    for (int f = 0; f < NF; ++f)
#pragma unroll
      for (int e = 0; e < 4; ++e) area[warp * kFrag + (f * 4 + e) * 32 + lane] = acc[f][e];
    half_barrier();
    // thread i finishes element i: fragment f, register e, lane l -> channel rb + l / 4 + 8 (e / 2), token 8 f + 2 (l % 4) + e % 2
#pragma unroll
    for (int q = 0; q < kFin; ++q) {
      const int i = htid + q * kGmThreads;
      if (i >= kFrag) break;
      int v = 0;
#pragma unroll
      for (int w2 = 0; w2 < kGmWarps; ++w2) v += area[w2 * kFrag + i];
      const int l = i & 31, e = (i >> 5) & 3, f = i >> 7;
      const int n = rb + (l >> 2) + ((e >> 1) << 3);
      const int tok = 8 * f + 2 * (l & 3) + (e & 1);
      if (n < row_end && tok < p.M) {
        v >>= 8;       // the widened operands carry a factor 16 each
        if (F16) {
          __half o = __float2half_rn((float)v * (s_scale[tok] * fin_scale[q]));
          if (p.bias) o = __hadd(o, fin_bias[q]);
          reinterpret_cast<__half*>(p.out)[(size_t)tok * p.ldo + n] = o;
        } else {
          reinterpret_cast<int32_t*>(p.out)[(size_t)tok * p.ldo + n] = v;
        }
      }
    }
    if (p.red_areas == 1) half_barrier();   // the only area is rewritten by the next group
  }
}

constexpr size_t kGmSmemMax = 220 * 1024;

// Shared memory of a CTA: the padded token rows and the reduction areas.
static size_t gemv_mma_smem(int nf, int64_t K, int halves, int areas) {
  return (size_t)(8 * nf) * (size_t)((K >> 1) + 64) + (size_t)halves * areas * kGmWarps * nf * 4 * 32 * sizeof(int);
}
// Two CTAs of eight warps per SM where their token rows fit, else one CTA of sixteen.
static bool gemv_mma_two_ctas_fit(int nf, int64_t K) { return 2 * (gemv_mma_smem(nf, K, 1, 2) + 1024) <= 226 * 1024; }
// One CTA of sixteen warps also where two of eight would fit, if it was measured faster: it halves the copies of the
// token rows that the SMs pull from the L2 (32 rows of K = 4096, N = 12288: 12.2 -> 10.9 us; 16 rows of K = 11008,
// N = 4096: 9.6 -> 7.7 us; slower for up to eight rows and for 16 rows of K = 4096).
static int gemv_mma_halves(int nf, int64_t K) {
  if (g_tuning.gemv_mma_halves == 2) return 2;
  if (!gemv_mma_two_ctas_fit(nf, K)) return 2;
  if (g_tuning.gemv_mma_halves == 1) return 1;
  return (nf == 4 || (nf == 2 && K >= 8192)) ? 2 : 1;
}
static int gemv_mma_areas(int nf, int64_t K, int halves) { return gemv_mma_smem(nf, K, halves, 2) <= kGmSmemMax ? 2 : 1; }
// Does this kernel take M token rows of K values?  (The token rows have to fit into shared memory.)
bool gemv_mma_serves(int64_t M, int64_t K) {
  if (M < 1 || M > 32 || K < 32 || K % 32 != 0 || K > 65536) return false;
  const int nf = M <= 8 ? 1 : (M <= 16 ? 2 : 4);
  return gemv_mma_smem(nf, K, gemv_mma_halves(nf, K), 1) <= kGmSmemMax;
}

template <int NF, bool F16, int U, int H>
static int launch_gemv_mma_h(GemvMmaParams& p, cudaStream_t st) {
  p.a_stride = (p.K >> 1) + 64;
  p.red_areas = gemv_mma_areas(NF, p.K, H);
  const size_t smem = gemv_mma_smem(NF, p.K, H, p.red_areas);
  if (smem > kGmSmemMax) return QR_EUNSUPPORTED;
  auto kern = gemv_mma_i4_kernel<NF, F16, U, H>;
  static thread_local size_t configured[64] = {0};
  int dev = 0;
  QR_CUDA(cudaGetDevice(&dev));
  if (smem > 48 * 1024 && (dev >= 64 || configured[dev] < smem)) {
    QR_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (dev < 64) configured[dev] = smem;
  }
  int64_t grid = (int64_t)num_sms() * (2 / H);
  // every CTA gets N / grid rows, so all SMs stream the same number of bytes; only very small N shrinks the grid
  const int64_t need = ((int64_t)p.N + 8 * H - 1) / (8 * H);
  if (grid > need) grid = need;
  QR_CUDA(launch_kernel(kern, dim3((unsigned)grid), dim3(kGmThreads * H), smem, st, use_pdl(p.M), p));
  return QR_OK;
}

template <int NF, bool F16, int U>
static int launch_gemv_mma_u(GemvMmaParams& p, cudaStream_t st) {
  if (gemv_mma_halves(NF, p.K) == 2) return launch_gemv_mma_h<NF, F16, U, 2>(p, st);
  return launch_gemv_mma_h<NF, F16, U, 1>(p, st);
}

// A lane keeps eight pieces per row in flight where a warp's slice of K is a whole number of such iterations (long
// rows: K = 8192, 16384, ...; 70B gate/up with eight token rows 45.6 -> 42.4 us), else four (K = 4096: one iteration
// per group of rows; eight would idle through four pieces of zeros).
template <int NF, bool F16>
static int launch_gemv_mma_nf(GemvMmaParams& p, cudaStream_t st) {
  const int nchunks = p.K >> 5;
  const int pieces = ((((nchunks + kGmWarps - 1) / kGmWarps) + 3) & ~3) >> 2;
  if (pieces % 8 == 0) return launch_gemv_mma_u<NF, F16, 8>(p, st);
  return launch_gemv_mma_u<NF, F16, 4>(p, st);
}

// Returns QR_EUNSUPPORTED when the shape is not one this kernel serves (the caller then takes another path).
int launch_gemv_mma_i4(const uint8_t* A, const uint8_t* B, int64_t M, int64_t N, int64_t K, void* out, int64_t ldo,
                       const void* sA, const void* sB, const void* bias, bool f16, cudaStream_t st) {
  if (!gemv_mma_serves(M, K) || N < 1 || N > (1 << 30)) return QR_EUNSUPPORTED;
  if (!aligned16(A) || !aligned16(B)) return QR_EUNSUPPORTED;
  GemvMmaParams p;
  p.A = A; p.B = B; p.sA = reinterpret_cast<const __half*>(sA); p.sB = reinterpret_cast<const __half*>(sB);
  p.bias = reinterpret_cast<const __half*>(bias); p.out = out; p.ldo = ldo;
  p.M = (int)M; p.N = (int)N; p.K = (int)K; p.a_stride = 0; p.red_areas = 2;
  p.status = kernel_status_ptr();
  if (!p.status) return QR_ENOTREADY;
  if (f16) {
    if (M <= 8) return launch_gemv_mma_nf<1, true>(p, st);
    if (M <= 16) return launch_gemv_mma_nf<2, true>(p, st);
    return launch_gemv_mma_nf<4, true>(p, st);
  }
  if (M <= 8) return launch_gemv_mma_nf<1, false>(p, st);
  if (M <= 16) return launch_gemv_mma_nf<2, false>(p, st);
  return launch_gemv_mma_nf<4, false>(p, st);
}

}  // namespace qr
