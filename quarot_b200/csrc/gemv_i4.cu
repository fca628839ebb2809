// Kernel (b) for a handful of token rows (M <= 8, single-sequence decode): a weight-streaming int4 GEMV on the
// CUDA cores.  At this size the tensor-core kernel is all fixed cost (tensor-memory set-up, pipeline fill,
// split-K reduction) while the work is one pass over the packed weights, so the only thing that matters is
// keeping enough 16-byte weight loads in flight to saturate HBM.
//
// A warp owns one or two output channels at a time.  Lane l reads the 16-byte chunks l, l + 32, ... of its weight rows
// (coalesced 512 bytes per row and step, streamed past L1), widens every packed word into two int8x4 words with
// the same x16 trick as the GEMM ((w << 4) & 0xF0F0F0F0 = even elements, w & 0xF0F0F0F0 = odd elements, each
// byte = 16 x the 4-bit value with its sign) and feeds dp4a against the token rows, which sit packed in shared
// memory and are widened the same way.  The int32 sums are exactly 256 x the dot products; after a warp-shuffle
// reduction the epilogue applies the arithmetic of the GEMM epilogue (float(acc) * (s_row * s_col), rounded to
// fp16, bias added in fp16), so the results are bit-identical to the tensor-core path.
// (A variant that streamed the weights with cp.async.bulk into a shared-memory ring, one thread issuing and eight
// warps consuming, was measured at half this kernel's rate -- 1.7 TB/s -- and dropped.)
#include "common.cuh"

namespace qr {

struct GemvParams {
  const uint8_t* A;      // [M, K/2] packed token rows
  const uint8_t* B;      // [N, K/2] packed weights
  const __half* sA;      // [M] or null (int32 mode)
  const __half* sB;      // [N] or null
  const __half* bias;    // [N] or null
  void* out;             // [M, N] fp16 (ldo) or int32
  int64_t ldo;
  int M, N, K;
  // fused quantiser: when x is set, A and sA are ignored and every CTA quantises the token rows itself
  const __half* x;       // [M, K] fp16 token rows (row stride ldx), or null
  int64_t ldx;
  float clip;
};

constexpr int kGemvThreads = 256;

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// Brings the token rows into shared memory as packed int4 (MT rows of K/2 bytes, zero rows beyond M) together with
// their per-token scales: either copied from the caller's packed rows, or -- when p.x is set -- quantised here from
// fp16 (Quantizer fused in: absmax -> s = fp16(fp16(absmax / 7) * clip) -> codes, exactly as the stand-alone
// quantiser; every CTA repeats this for its few rows, which costs less than a launch).  NT = threads of the CTA.
template <int MT, bool F16, int NT>
__device__ __forceinline__ void stage_token_rows(const GemvParams& p, unsigned char* smem_a, float* s_scale, float* s_red) {
  const int kbytes = p.K >> 1;
  const int nchunks = kbytes >> 4;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (p.x == nullptr) {
    for (int i = threadIdx.x; i < MT * nchunks; i += NT) {
      const int m = i / nchunks, c = i - m * nchunks;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (m < p.M) v = *reinterpret_cast<const uint4*>(p.A + (size_t)m * kbytes + (size_t)c * 16);
      *reinterpret_cast<uint4*>(smem_a + (size_t)i * 16) = v;
    }
    if (F16 && threadIdx.x < MT) s_scale[threadIdx.x] = threadIdx.x < p.M ? __half2float(p.sA[threadIdx.x]) : 0.0f;
  } else {
    // Quantizer fused in: per token row absmax -> s = fp16(fp16(absmax / 7) * clip) -> int4 codes, exactly as the
    // stand-alone quantiser does it; every CTA repeats this for the (at most eight) rows, which costs less than a
    // launch.  A 16-byte packed chunk comes from four 16-byte groups of eight fp16 values.
    const int ngroups = p.K >> 3;
    for (int m = 0; m < MT; ++m) {
      float s = 0.0f;
      if (m < p.M) {
        const uint4* xr = reinterpret_cast<const uint4*>(p.x + (size_t)m * p.ldx);
        __half2 mx = __float2half2_rn(0.0f);
        for (int g = threadIdx.x; g < ngroups; g += NT) {
          const uint4 v = __ldg(xr + g);
          const __half2* h = reinterpret_cast<const __half2*>(&v);
          mx = __hmax2(mx, __hmax2(__hmax2(__habs2(h[0]), __habs2(h[1])), __hmax2(__habs2(h[2]), __habs2(h[3]))));
        }
        const float2 mf = __half22float2(mx);
        float a = fmaxf(mf.x, mf.y);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
        if (lane == 0) s_red[warp] = a;
        __syncthreads();
        a = (lane < NT / 32) ? s_red[lane] : 0.0f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
        __syncthreads();
        const __half s7 = __float2half_rn(__fdiv_rn(a, 7.0f));
        s = __half2float(__float2half_rn(__half2float(s7) * p.clip));
        const float rcp = (s != 0.0f) ? __frcp_rn(s) : 0.0f;
        const bool noclamp = clamp_free(s, p.clip);
        uint32_t* dst = reinterpret_cast<uint32_t*>(smem_a + (size_t)m * kbytes);
        for (int g = threadIdx.x; g < ngroups; g += NT) {
          const uint4 v = __ldg(xr + g);
          dst[g] = quant8_words(v.x, v.y, v.z, v.w, s, rcp, noclamp);
        }
      } else {
        uint32_t* dst = reinterpret_cast<uint32_t*>(smem_a + (size_t)m * kbytes);
        for (int g = threadIdx.x; g < ngroups; g += NT) dst[g] = 0u;
      }
      if (threadIdx.x == 0) s_scale[m] = s;
    }
  }
}

// MT: token rows held per warp (M rounded up), ROWS: output channels a warp works on at a time (two share the
// widening of the token rows; one gives twice as many warps when there are few output channels).
template <int MT, int ROWS, bool F16>
__global__ void __launch_bounds__(kGemvThreads)
gemv_i4_kernel(const GemvParams p) {
  constexpr int kGemvRows = ROWS;
  extern __shared__ __align__(16) unsigned char smem_a[];      // MT x K/2 packed token rows (zero rows beyond M)
  __shared__ float s_red[kGemvThreads / 32];
  __shared__ float s_scale[MT];                                // per-token scales of the token rows
  const int kbytes = p.K >> 1;
  const int nchunks = kbytes >> 4;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_launch_dependents();   // the next kernel of the stream may be brought up; it waits for this grid to finish

  // The work of a warp is the flat sequence (channel pair, k step); the weight chunks of step t + 1 are requested
  // before step t is computed, also across pair boundaries, so that every lane always has up to eight 16-byte
  // loads in flight.
  const int warps_total = gridDim.x * (kGemvThreads / 32);
  const int warp_id = blockIdx.x * (kGemvThreads / 32) + warp;
  const int npairs = (p.N + kGemvRows - 1) / kGemvRows;
  const int steps = (nchunks + 63) >> 6;                       // 64 chunks (2 per lane) per step
  const int my_pairs = warp_id < npairs ? (npairs - warp_id + warps_total - 1) / warps_total : 0;
  const int total = my_pairs * steps;

  auto row_ptr = [&](int t, int r) {
    const int pair = warp_id + (t / steps) * warps_total;
    int n = pair * kGemvRows + r;
    if (n >= p.N) n = p.N - 1;
    return p.B + (size_t)n * kbytes;
  };
  auto load_step = [&](int t, uint4 (&w)[kGemvRows][2]) {
    const int c = lane + ((t % steps) << 6);
#pragma unroll
    for (int r = 0; r < kGemvRows; ++r) {
      const uint8_t* rp = row_ptr(t, r);
      w[r][0] = (c < nchunks) ? ld_stream16(rp + (size_t)c * 16) : make_uint4(0, 0, 0, 0);
      w[r][1] = (c + 32 < nchunks) ? ld_stream16(rp + (size_t)(c + 32) * 16) : make_uint4(0, 0, 0, 0);
    }
  };

  int acc[kGemvRows][MT];
#pragma unroll
  for (int r = 0; r < kGemvRows; ++r)
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[r][m] = 0;
  // With one or two token rows the registers allow requesting step t + 1 before step t is computed; with more
  // rows (more accumulators) the extra registers cost more occupancy than the prefetch gains (measured).
  constexpr bool kPrefetch = (MT <= 2);
  uint4 cur[kGemvRows][2], nxt[kGemvRows][2];
  // The weights do not depend on the kernel in front: the first chunks are requested before the programmatic-
  // dependency wait and before the token rows are staged, so that their latency overlaps both.
  if (kPrefetch && total > 0) load_step(0, cur);
  pdl_wait();   // token rows, scales and the output belong to the preceding kernels
  stage_token_rows<MT, F16, kGemvThreads>(p, smem_a, s_scale, s_red);
  __syncthreads();
#pragma unroll 1
  for (int t = 0; t < total; ++t) {
    if (kPrefetch) {
      if (t + 1 < total) load_step(t + 1, nxt);
    } else {
      load_step(t, cur);
    }
    const int c = lane + ((t % steps) << 6);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int cc = c + 32 * h;
      if (cc < nchunks) {
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          const uint4 a = *reinterpret_cast<const uint4*>(smem_a + ((size_t)m * nchunks + cc) * 16);
          const uint32_t* ar = reinterpret_cast<const uint32_t*>(&a);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int a_lo = (int)((ar[q] << 4) & 0xF0F0F0F0u), a_hi = (int)(ar[q] & 0xF0F0F0F0u);
#pragma unroll
            for (int r = 0; r < kGemvRows; ++r) {
              const uint32_t wv = reinterpret_cast<const uint32_t*>(&cur[r][h])[q];
              acc[r][m] = __dp4a((int)((wv << 4) & 0xF0F0F0F0u), a_lo, acc[r][m]);
              acc[r][m] = __dp4a((int)(wv & 0xF0F0F0F0u), a_hi, acc[r][m]);
            }
          }
        }
      }
    }
    if ((t + 1) % steps == 0) {
      // the pair is complete: reduce over the lanes, dequantise, store, start the next pair from zero
      const int n0 = (warp_id + (t / steps) * warps_total) * kGemvRows;
      const bool two = n0 + 1 < p.N;
#pragma unroll
      for (int r = 0; r < kGemvRows; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) acc[r][m] += __shfl_xor_sync(0xffffffffu, acc[r][m], o);
      if (lane < p.M) {      // lane m writes row m of both channels
#pragma unroll
        for (int r = 0; r < kGemvRows; ++r) {
          if (r == 1 && !two) break;
          const int n = n0 + r;
          int v = 0;
#pragma unroll
          for (int m = 0; m < MT; ++m)
            if (m == lane) v = acc[r][m];
          if (F16) {
            const float sc = s_scale[lane] * __half2float(p.sB[n]);
            __half o = __float2half_rn((float)(v >> 8) * sc);
            if (p.bias) o = __hadd(o, p.bias[n]);
            reinterpret_cast<__half*>(p.out)[(size_t)lane * p.ldo + n] = o;
          } else {
            reinterpret_cast<int32_t*>(p.out)[(size_t)lane * p.ldo + n] = v >> 8;
          }
        }
      }
#pragma unroll
      for (int r = 0; r < kGemvRows; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[r][m] = 0;
    }
    if (kPrefetch) {
#pragma unroll
      for (int r = 0; r < kGemvRows; ++r) { cur[r][0] = nxt[r][0]; cur[r][1] = nxt[r][1]; }
    }
  }
}

template <int MT, int ROWS, bool F16>
static int launch_gemv_mt(const GemvParams& p, cudaStream_t st) {
  constexpr int kGemvRows = ROWS;
  const size_t smem = (size_t)MT * (p.K >> 1);
  auto kern = gemv_i4_kernel<MT, ROWS, F16>;
  static thread_local size_t configured[64] = {0};
  int dev = 0;
  QR_CUDA(cudaGetDevice(&dev));
  if (smem > 48 * 1024 && (dev >= 64 || configured[dev] < smem)) {
    QR_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (dev < 64) configured[dev] = smem;
  }
  // enough resident warps to keep HBM busy; every warp takes pairs of output channels round-robin
  int per_sm = (int)((200 * 1024) / (smem + 1024));
  if (per_sm > 4) per_sm = 4;
  if (per_sm < 1) per_sm = 1;
  int64_t grid = (int64_t)num_sms() * per_sm;
  const int64_t need = ((int64_t)(p.N + kGemvRows - 1) / kGemvRows + (kGemvThreads / 32) - 1) / (kGemvThreads / 32);
  if (grid > need) grid = need;
  QR_CUDA(launch_kernel(kern, dim3((unsigned)grid), dim3(kGemvThreads), smem, st, false, p));   // measured: no gain from a programmatic launch here
  return QR_OK;
}

// Returns QR_EUNSUPPORTED when the shape is not one this kernel serves (the caller then takes the tensor-core path).
int launch_gemv_i4(const uint8_t* A, const uint8_t* B, int64_t M, int64_t N, int64_t K, void* out, int64_t ldo,
                   const void* sA, const void* sB, const void* bias, bool f16, cudaStream_t st,
                   const void* x, int64_t ldx, float clip) {
  if (M < 1 || M > 8 || K % 32 != 0 || K > 65536 || N > (1 << 30)) return QR_EUNSUPPORTED;
  if ((size_t)8 * (K >> 1) > 200 * 1024) return QR_EUNSUPPORTED;
  GemvParams p;
  p.A = A; p.B = B; p.sA = reinterpret_cast<const __half*>(sA); p.sB = reinterpret_cast<const __half*>(sB);
  p.bias = reinterpret_cast<const __half*>(bias); p.out = out; p.ldo = ldo;
  p.M = (int)M; p.N = (int)N; p.K = (int)K;
  p.x = reinterpret_cast<const __half*>(x); p.ldx = ldx; p.clip = clip;
  if (f16) {
    if (M == 1) return launch_gemv_mt<1, 2, true>(p, st);
    if (M == 2) return launch_gemv_mt<2, 2, true>(p, st);
    if (M <= 4) return launch_gemv_mt<4, 2, true>(p, st);
    return launch_gemv_mt<8, 2, true>(p, st);
  }
  if (M == 1) return launch_gemv_mt<1, 2, false>(p, st);
  if (M == 2) return launch_gemv_mt<2, 2, false>(p, st);
  if (M <= 4) return launch_gemv_mt<4, 2, false>(p, st);
  return launch_gemv_mt<8, 2, false>(p, st);
}

}  // namespace qr

extern "C" int qr_quant_linear_i4_f16(const void* x, int64_t ldx, float clip, const uint8_t* B, const void* sB,
                                      const void* bias, int64_t M, int64_t N, int64_t K, void* out, int64_t ldo,
                                      void* stream) {
  if (M < 0 || N < 0 || K < 0) return qr::fail(QR_EINVAL, "qr_quant_linear_i4_f16: negative size");
  if (M == 0 || N == 0) return QR_OK;
  if (!x || !B || !sB || !out) return qr::fail(QR_EINVAL, "qr_quant_linear_i4_f16: null pointer");
  if (K == 0 || K % 32 != 0) return qr::fail(QR_EINVAL, "qr_quant_linear_i4_f16: K = %lld must be a positive multiple of 32", (long long)K);
  if (ldx < K || ldo < N) return qr::fail(QR_EINVAL, "qr_quant_linear_i4_f16: leading dimension too small");
  if (!qr::aligned16(x) || ldx % 8 != 0 || !qr::aligned16(B))
    return qr::fail(QR_EALIGN, "qr_quant_linear_i4_f16: x and B must be 16-byte aligned, ldx % 8 == 0");
  if (M > 8) return qr::fail(QR_EUNSUPPORTED, "qr_quant_linear_i4_f16: at most 8 token rows (use the quantiser and qr_linear_i4_f16)");
  const int rc = qr::launch_gemv_i4(nullptr, B, M, N, K, out, ldo, nullptr, sB, bias, true, (cudaStream_t)stream, x, ldx, clip);
  if (rc == QR_EUNSUPPORTED) return qr::fail(QR_EUNSUPPORTED, "qr_quant_linear_i4_f16: K = %lld is too long for this kernel", (long long)K);
  return rc;
}

