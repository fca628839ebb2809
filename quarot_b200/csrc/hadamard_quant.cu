// Kernel family (a): online Hadamard transform, per-token absmax scale, INT4
// quantise-and-pack -- fused into one pass over the activations.
//
// Operator (natural-order Sylvester-Walsh H_m on the low index bits, dense
// +-1 factor hadK on the major axis):
//     y[k', m'] = 1/sqrt(n) * sum_k sum_m hadK[k'][k] * H_m[m'][m] * x[k*m + m]
//
// hadq_fast_kernel: one persistent CTA per token row.
//   stage 1 (K > 1)  dense factor on tensor cores: D[K x m] = hadK . X[K x m] with
//                    mma.sync m16n8k16 (fp16 operands are the raw activations and
//                    +-1, fp32 accumulation, so the products are exact); B comes
//                    from shared memory with ldmatrix.trans, hadK fragments live in
//                    registers for the lifetime of the CTA.
//   low pass         index bits 0..4: each thread owns 32 consecutive values
//                    (128-bit loads from global when K == 1, from the swizzled fp32
//                    row buffer otherwise) and runs a radix-32 butterfly in registers.
//   scalar passes    index bits >= 5, up to four bits per pass, through the fp32 row
//                    buffer in shared memory; lanes always map to address bits 0..4,
//                    so every access is bank-conflict free.
//   finalise         scale, round to fp16 (the rounding OnlineHadamard applies),
//                    absmax; then the row is re-read as 8-element vectors, divided
//                    by the scale with torch's arithmetic, packed and stored.
// The fp32 row buffer is addressed through phys(i) = i ^ (((i >> 5) & 7) << 2) so
// that the float4 accesses of the low pass are conflict free as well.
//
// hadq_generic_kernel: any n = K * 2^j, fp16 or fp32 input, plain shared-memory
// butterflies and a CUDA-core dense factor.  Slow; used for shapes the fast
// kernel does not cover (tiny Walsh lengths, fp32 weights at initialisation).
#include "common.cuh"

#include <math.h>

namespace qr {

struct HadqParams {
  const void* x;
  int64_t ldx;        // elements between work items
  int64_t rows;       // work items
  int n;              // elements per work item
  int n_row;          // true transform length (n_row <= n; n is a multiple when rows are batched)
  int K;              // 0: no transform, 1: Walsh only, >1: dense factor order
  int m;              // Walsh length n_row / max(K,1)
  int wbits;          // log2(m)
  const __half* had_k;
  float scale;        // 1/sqrt(n_row)
  float clip;
  uint8_t* q;
  __half* scales;
  void* y_out;
  int do_quant;
};

__device__ __forceinline__ int phys(int i) { return i ^ (((i >> 5) & 7) << 2); }

template <int N>
__device__ __forceinline__ void fwht_regs(float (&v)[N]) {
#pragma unroll
  for (int h = 1; h < N; h <<= 1) {
#pragma unroll
    for (int i = 0; i < N; ++i) {
      if ((i & h) == 0) {
        float a = v[i], b = v[i + h];
        v[i] = a + b;
        v[i + h] = a - b;
      }
    }
  }
}

__device__ __forceinline__ float absmax8(const uint4& v) {
  const __half2* h = reinterpret_cast<const __half2*>(&v);
  __half2 m = __habs2(h[0]);
  m = __hmax2(m, __habs2(h[1]));
  m = __hmax2(m, __habs2(h[2]));
  m = __hmax2(m, __habs2(h[3]));
  float2 f = __half22float2(m);
  return fmaxf(f.x, f.y);
}

// One radix-2^R pass over index bits [b, b+R), b >= 5, in place in buf32.
// When `final`, results are scaled, rounded to fp16 and written to buf16 instead.
template <int R>
__device__ __forceinline__ void scalar_pass(float* buf32, __half* buf16, int n, int b, bool final,
                                            float scale, float& amax, int tid, int nthreads) {
  constexpr int N = 1 << R;
  const int groups = n >> R;
  for (int gid = tid; gid < groups; gid += nthreads) {
    const int low = gid & ((1 << b) - 1);
    const int base = low | ((gid >> b) << (b + R));
    float v[N];
#pragma unroll
    for (int j = 0; j < N; ++j) v[j] = buf32[phys(base + (j << b))];
    fwht_regs<N>(v);
    if (!final) {
#pragma unroll
      for (int j = 0; j < N; ++j) buf32[phys(base + (j << b))] = v[j];
    } else {
#pragma unroll
      for (int j = 0; j < N; ++j) {
        __half y = __float2half_rn(v[j] * scale);
        buf16[base + (j << b)] = y;
        amax = fmaxf(amax, fabsf(__half2float(y)));
      }
    }
  }
}

__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

// KT = number of 16-wide k tiles of the dense factor (0 when K <= 1).
template <int KT>
__global__ void __launch_bounds__(512, 1)
hadq_fast_kernel(const HadqParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int tid = threadIdx.x;
  const int nthreads = blockDim.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int nwarps = nthreads >> 5;
  const int n = p.n;
  const int m = p.m;
  const int K = p.K;

  // shared memory carve-up: [fp32 row buffer][fp16 row / raw staging][reduction scratch]
  const int buf32_bytes = (K >= 1) ? n * 4 : 0;
  const int pitch = m + 8;  // halfs; staging pitch for the dense-factor operand
  const int raw_halfs = (KT > 0) ? KT * 16 * pitch : 0;
  const int buf16_halfs = raw_halfs > n ? raw_halfs : n;
  float* buf32 = reinterpret_cast<float*>(smem_raw);
  __half* buf16 = reinterpret_cast<__half*>(smem_raw + buf32_bytes);
  float* red = reinterpret_cast<float*>(smem_raw + buf32_bytes + ((buf16_halfs * 2 + 15) & ~15));

  // dense-factor fragments: warp w owns 16 output rows (M tile w % MT) for good
  constexpr int KTT = KT > 0 ? KT : 1;
  uint32_t afrag[KTT][4];
  constexpr int MT = KT > 0 ? KT : 1;
  const int my_mt = (KT > 0) ? warp % MT : 0;
  if (KT > 0) {
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int kt = 0; kt < KTT; ++kt) {
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int row = my_mt * 16 + g + ((r & 1) ? 8 : 0);
        const int col = kt * 16 + 2 * t + ((r & 2) ? 8 : 0);
        uint32_t val = 0;
        if (row < K && col < K)  // K is even, so a pair never straddles the edge
          val = *reinterpret_cast<const uint32_t*>(p.had_k + (size_t)row * K + col);
        afrag[kt][r] = val;
      }
    }
  }

  for (int64_t row = blockIdx.x; row < p.rows; row += gridDim.x) {
    const __half* xr = reinterpret_cast<const __half*>(p.x) + row * p.ldx;
    float amax = 0.0f;

    if (K == 0) {
      for (int c = tid; c < (n >> 3); c += nthreads) {
        uint4 v = __ldg(reinterpret_cast<const uint4*>(xr) + c);
        reinterpret_cast<uint4*>(buf16)[c] = v;
        amax = fmaxf(amax, absmax8(v));
      }
    } else {
      const bool low_is_final = (p.wbits == 5);
      if (KT > 0) {
        // ---- stage 0: raw row -> padded staging, zero the padding rows
        const int vec_per_k = m >> 3;
        for (int c = tid; c < (n >> 3); c += nthreads) {
          const int k = c / vec_per_k;
          const int mm = (c - k * vec_per_k) << 3;
          uint4 v = __ldg(reinterpret_cast<const uint4*>(xr) + c);
          *reinterpret_cast<uint4*>(buf16 + k * pitch + mm) = v;
        }
        const int pad_vecs = (KT * 16 - K) * vec_per_k;
        for (int c = tid; c < pad_vecs; c += nthreads) {
          const int k = K + c / vec_per_k;
          const int mm = (c % vec_per_k) << 3;
          *reinterpret_cast<uint4*>(buf16 + k * pitch + mm) = make_uint4(0, 0, 0, 0);
        }
        __syncthreads();
        // ---- stage 1: D = hadK . X on tensor cores, 64 columns per unit
        const int nchunks = m >> 6;
        const int warps_per_mt = nwarps / MT;
        if (warp < warps_per_mt * MT) {
          const int g = lane >> 2, t = lane & 3;
          // ldmatrix lane address: matrix j = lane / 8 -> (k half j & 1, n tile j >> 1), row lane % 8
          const int lrow = (lane & 7) + ((lane >> 3) & 1) * 8;
          const int lcol = (lane >> 4) * 8;
          for (int ch = warp / MT; ch < nchunks; ch += warps_per_mt) {
            float acc[8][4];
#pragma unroll
            for (int i = 0; i < 8; ++i) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.0f; }
#pragma unroll
            for (int kt = 0; kt < KTT; ++kt) {
#pragma unroll
              for (int np = 0; np < 4; ++np) {
                uint32_t b[4];
                const __half* src = buf16 + (kt * 16 + lrow) * pitch + ch * 64 + np * 16 + lcol;
                ldmatrix_x4_trans(b, smem_u32(src));
                mma_16816(acc[2 * np], afrag[kt], b[0], b[1]);
                mma_16816(acc[2 * np + 1], afrag[kt], b[2], b[3]);
              }
            }
            const int r0 = my_mt * 16 + g;
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
              const int col = ch * 64 + nt * 8 + 2 * t;
              if (r0 < K)
                *reinterpret_cast<float2*>(buf32 + phys(r0 * m + col)) = make_float2(acc[nt][0], acc[nt][1]);
              if (r0 + 8 < K)
                *reinterpret_cast<float2*>(buf32 + phys((r0 + 8) * m + col)) = make_float2(acc[nt][2], acc[nt][3]);
            }
          }
        }
        __syncthreads();  // staging (aliased by buf16) is dead from here on
      }
      // ---- low pass: index bits 0..4
      for (int G = tid; G < (n >> 5); G += nthreads) {
        float v[32];
        if (KT > 0) {
#pragma unroll
          for (int s = 0; s < 8; ++s) {
            float4 f = *reinterpret_cast<const float4*>(buf32 + G * 32 + ((s ^ (G & 7)) << 2));
            v[4 * s] = f.x; v[4 * s + 1] = f.y; v[4 * s + 2] = f.z; v[4 * s + 3] = f.w;
          }
        } else {
#pragma unroll
          for (int s = 0; s < 4; ++s) {
            uint4 u = __ldg(reinterpret_cast<const uint4*>(xr) + G * 4 + s);
            const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              float2 f = __half22float2(h[e]);
              v[8 * s + 2 * e] = f.x;
              v[8 * s + 2 * e + 1] = f.y;
            }
          }
        }
        fwht_regs<32>(v);
        if (!low_is_final) {
#pragma unroll
          for (int s = 0; s < 8; ++s) {
            *reinterpret_cast<float4*>(buf32 + G * 32 + ((s ^ (G & 7)) << 2)) =
                make_float4(v[4 * s], v[4 * s + 1], v[4 * s + 2], v[4 * s + 3]);
          }
        } else {
#pragma unroll
          for (int s = 0; s < 4; ++s) {
            uint4 u;
            __half2* h = reinterpret_cast<__half2*>(&u);
#pragma unroll
            for (int e = 0; e < 4; ++e)
              h[e] = __floats2half2_rn(v[8 * s + 2 * e] * p.scale, v[8 * s + 2 * e + 1] * p.scale);
            reinterpret_cast<uint4*>(buf16)[G * 4 + s] = u;
            amax = fmaxf(amax, absmax8(u));
          }
        }
      }
      // ---- scalar passes: index bits 5 .. wbits-1, at most four per pass, balanced
      int rem = p.wbits - 5;
      int b = 5;
      while (rem > 0) {
        const int npass = (rem + 3) >> 2;
        const int r = (rem + npass - 1) / npass;
        const bool fin = (rem == r);
        __syncthreads();
        if (r == 4) scalar_pass<4>(buf32, buf16, n, b, fin, p.scale, amax, tid, nthreads);
        else if (r == 3) scalar_pass<3>(buf32, buf16, n, b, fin, p.scale, amax, tid, nthreads);
        else if (r == 2) scalar_pass<2>(buf32, buf16, n, b, fin, p.scale, amax, tid, nthreads);
        else scalar_pass<1>(buf32, buf16, n, b, fin, p.scale, amax, tid, nthreads);
        b += r;
        rem -= r;
      }
    }

    // ---- per-row scale
    float s = 0.0f;
    if (p.do_quant) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      if (lane == 0) red[warp] = amax;
      __syncthreads();
      float a = (lane < nwarps) ? red[lane] : 0.0f;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
      const __half s7 = __float2half_rn(__fdiv_rn(a, 7.0f));
      const __half sh = __float2half_rn(__half2float(s7) * p.clip);
      s = __half2float(sh);
      if (tid == 0) p.scales[row] = sh;
    } else {
      __syncthreads();
    }

    // ---- quantise / emit
    const float rcp = (s != 0.0f) ? __frcp_rn(s) : 0.0f;
    __half* yo = p.y_out ? reinterpret_cast<__half*>(p.y_out) + row * (int64_t)n : nullptr;
    uint8_t* qo = p.do_quant ? p.q + row * (int64_t)(n >> 1) : nullptr;
    for (int c = tid; c < (n >> 3); c += nthreads) {
      uint4 v = reinterpret_cast<const uint4*>(buf16)[c];
      if (yo) reinterpret_cast<uint4*>(yo)[c] = v;
      if (qo) {
        uint32_t packed = 0;
        const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float2 f = __half22float2(h[i]);
          uint32_t cd = (s != 0.0f) ? quant_pair(div_by_scale(f.x, s, rcp), div_by_scale(f.y, s, rcp))
                                    : quant_pair_zero_scale(f.x, f.y);
          packed |= ((cd & 0xF) | ((cd >> 12) & 0xF0)) << (8 * i);
        }
        reinterpret_cast<uint32_t*>(qo)[c] = packed;
      }
    }
    __syncthreads();  // buffers are reused by the next row
  }
}

// ------------------------------------------------------------------ generic
template <typename T> __device__ __forceinline__ float load_as_float(const T* p, int64_t i);
template <> __device__ __forceinline__ float load_as_float<__half>(const __half* p, int64_t i) { return __half2float(p[i]); }
template <> __device__ __forceinline__ float load_as_float<float>(const float* p, int64_t i) { return p[i]; }

template <typename T>
__global__ void __launch_bounds__(256)
hadq_generic_kernel(const HadqParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int tid = threadIdx.x, nthreads = blockDim.x;
  const int n = p.n, K = p.K, m = p.m;
  float* a = reinterpret_cast<float*>(smem_raw);
  float* bbuf = a + n;
  __shared__ float red[8];
  for (int64_t row = blockIdx.x; row < p.rows; row += gridDim.x) {
    const T* xr = reinterpret_cast<const T*>(p.x) + row * p.ldx;
    for (int i = tid; i < n; i += nthreads) a[i] = load_as_float<T>(xr, i);
    __syncthreads();
    float* cur = a;
    if (K >= 1) {
      for (int h = 1; h < m; h <<= 1) {
        for (int j = tid; j < (n >> 1); j += nthreads) {
          const int i = ((j / h) * 2 * h) + (j % h);
          float u = cur[i], w = cur[i + h];
          cur[i] = u + w;
          cur[i + h] = u - w;
        }
        __syncthreads();
      }
      if (K > 1) {
        for (int o = tid; o < n; o += nthreads) {
          const int kk = o / m, mm = o - kk * m;
          float acc = 0.0f;
          for (int k = 0; k < K; ++k) acc += __half2float(p.had_k[kk * K + k]) * cur[k * m + mm];
          bbuf[o] = acc;
        }
        __syncthreads();
        cur = bbuf;
      }
      for (int i = tid; i < n; i += nthreads) {
        float v = cur[i] * p.scale;
        if (sizeof(T) == 2) v = __half2float(__float2half_rn(v));
        cur[i] = v;
      }
      __syncthreads();
    }
    if (p.y_out) {
      T* yo = reinterpret_cast<T*>(p.y_out) + row * (int64_t)n;
      for (int i = tid; i < n; i += nthreads) {
        if (sizeof(T) == 2) reinterpret_cast<__half*>(yo)[i] = __float2half_rn(cur[i]);
        else reinterpret_cast<float*>(yo)[i] = cur[i];
      }
    }
    if (p.do_quant) {
      float amax = 0.0f;
      for (int i = tid; i < n; i += nthreads) amax = fmaxf(amax, fabsf(cur[i]));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      if ((tid & 31) == 0) red[tid >> 5] = amax;
      __syncthreads();
      float r = 0.0f;
      for (int w = 0; w < (nthreads >> 5); ++w) r = fmaxf(r, red[w]);
      const __half s7 = __float2half_rn(__fdiv_rn(r, 7.0f));
      const __half sh = __float2half_rn(__half2float(s7) * p.clip);
      const float s = __half2float(sh);
      if (tid == 0) p.scales[row] = sh;
      const float rcp = (s != 0.0f) ? __frcp_rn(s) : 0.0f;
      const int nb = (n + 1) >> 1;
      uint8_t* qo = p.q + row * (int64_t)nb;
      for (int j = tid; j < nb; j += nthreads) {
        const float v0 = cur[2 * j];
        const float v1 = (2 * j + 1 < n) ? cur[2 * j + 1] : 0.0f;
        const uint32_t cd = (s != 0.0f) ? quant_pair(div_by_scale(v0, s, rcp), div_by_scale(v1, s, rcp))
                                        : quant_pair_zero_scale(v0, v1);
        qo[j] = (uint8_t)((cd & 0xF) | ((cd >> 12) & 0xF0));
      }
    }
    __syncthreads();
  }
}

// ---------------------------------------------------------------- dispatch
static int kt_for(int K) { return K > 1 ? (K + 15) / 16 : 0; }

template <int KT>
static int launch_fast(const HadqParams& p, int threads, size_t smem, cudaStream_t st) {
  static thread_local size_t configured[64] = {0};
  int dev = 0;
  QR_CUDA(cudaGetDevice(&dev));
  if (dev < 64 && configured[dev] < smem) {
    QR_CUDA(cudaFuncSetAttribute(hadq_fast_kernel<KT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured[dev] = smem;
  } else if (dev >= 64) {
    QR_CUDA(cudaFuncSetAttribute(hadq_fast_kernel<KT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  }
  // persistent grid: as many CTAs as fit at once
  int per_sm = (int)(227 * 1024 / (smem + 1024));
  int by_threads = 2048 / threads;
  if (per_sm > by_threads) per_sm = by_threads;
  if (per_sm < 1) per_sm = 1;
  int64_t grid = (int64_t)num_sms() * per_sm;
  if (grid > p.rows) grid = p.rows;
  hadq_fast_kernel<KT><<<(int)grid, threads, smem, st>>>(p);
  QR_LAUNCH_CHECK("hadq_fast_kernel");
  return QR_OK;
}

template <typename T>
static int launch_generic(const HadqParams& p, cudaStream_t st) {
  const size_t smem = (size_t)p.n * 4 * (p.K > 1 ? 2 : 1);
  if (smem > 227 * 1024 - 64) return fail(QR_EUNSUPPORTED, "hadamard: row of %d elements exceeds shared memory", p.n);
  static thread_local size_t configured[64] = {0};
  int dev = 0;
  QR_CUDA(cudaGetDevice(&dev));
  if (dev >= 64 || configured[dev] < smem) {
    QR_CUDA(cudaFuncSetAttribute(hadq_generic_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (dev < 64) configured[dev] = smem;
  }
  int per_sm = (int)(227 * 1024 / (smem + 1024));
  if (per_sm > 8) per_sm = 8;
  if (per_sm < 1) per_sm = 1;
  int64_t grid = (int64_t)num_sms() * per_sm;
  if (grid > p.rows) grid = p.rows;
  hadq_generic_kernel<T><<<(int)grid, 256, smem, st>>>(p);
  QR_LAUNCH_CHECK("hadq_generic_kernel");
  return QR_OK;
}

// Decides which kernel serves (rows, n, K) and launches it.  elem_size 2 = fp16, 4 = fp32.
static int run_hadq(const char* who, const void* x, int64_t rows, int64_t n64, int64_t ldx,
                    const void* had_k, int K, float clip, uint8_t* q, void* scales, void* y_out,
                    int do_quant, int elem_size, cudaStream_t st) {
  if (rows < 0 || n64 < 0) return fail(QR_EINVAL, "%s: negative size", who);
  if (rows == 0 || n64 == 0) return QR_OK;
  if (!x) return fail(QR_EINVAL, "%s: null input", who);
  if (do_quant && (!q || !scales)) return fail(QR_EINVAL, "%s: null output", who);
  if (!do_quant && !y_out) return fail(QR_EINVAL, "%s: null output", who);
  if (n64 > (1 << 20)) return fail(QR_EUNSUPPORTED, "%s: n = %lld too large", who, (long long)n64);
  if (K < 0) return fail(QR_EINVAL, "%s: K = %d", who, K);
  const int n = (int)n64;
  int m = n;
  if (K > 1) {
    if (!had_k) return fail(QR_EINVAL, "%s: K = %d needs a table", who, K);
    if (n % K != 0 || !is_pow2(n / K)) return fail(QR_EINVAL, "%s: n = %d is not K = %d times a power of two", who, n, K);
    if (K > 176 || (K & 1)) return fail(QR_EUNSUPPORTED, "%s: table order %d not supported", who, K);
    m = n / K;
  } else if (K == 1) {
    if (!is_pow2(n)) return fail(QR_EINVAL, "%s: n = %d is not a power of two", who, n);
  }
  if (do_quant && (n & 1)) {
    if (K != 0) return fail(QR_EINVAL, "%s: odd n", who);
  }

  HadqParams p;
  p.x = x; p.ldx = ldx; p.rows = rows; p.n = n; p.n_row = n; p.K = K; p.m = m;
  p.wbits = (K >= 1) ? ilog2(m) : 0;
  p.had_k = reinterpret_cast<const __half*>(had_k);
  p.scale = (K >= 1) ? (float)(1.0 / sqrt((double)n)) : 1.0f;
  p.clip = clip; p.q = q; p.scales = reinterpret_cast<__half*>(scales); p.y_out = y_out; p.do_quant = do_quant;

  const int forced = tuning("hadq_path", 0);  // 1 = always generic (for A/B checks)
  bool fast = (elem_size == 2) && forced != 1 && aligned16(x) && (ldx % 8 == 0) && (n % 8 == 0) &&
              (!y_out || aligned16(y_out)) && (!do_quant || (((uintptr_t)q & 3) == 0));
  if (fast) {
    if (K == 0) fast = (n >= 256) && ((size_t)n * 2 <= 200 * 1024);
    else if (K == 1) fast = (n >= 1024);
    else fast = (m >= 64);
  }
  // Walsh-only with short rows and no quantisation: batch 1024/n consecutive rows per work item
  if (!fast && elem_size == 2 && forced != 1 && K == 1 && !do_quant && n >= 32 && n < 1024 && ldx == n &&
      aligned16(x) && aligned16(y_out)) {
    const int per = 1024 / n;
    if (rows % per == 0) {
      p.n = 1024; p.rows = rows / per; p.ldx = 1024; p.m = n; fast = true;
    }
  }
  if (fast) {
    const int KT = kt_for(K);
    const int pitch = p.m + 8;
    const size_t raw = KT ? (size_t)KT * 16 * pitch * 2 : 0;
    size_t b16 = (size_t)p.n * 2;
    if (raw > b16) b16 = raw;
    b16 = (b16 + 15) & ~(size_t)15;
    const size_t smem = (K >= 1 ? (size_t)p.n * 4 : 0) + b16 + 32 * 4;
    if (smem <= 227 * 1024) {
      int threads = (p.n / 32 + 31) / 32 * 32;
      if (K == 0) threads = (p.n / 8 + 31) / 32 * 32;
      if (threads < 64) threads = 64;
      if (threads > 512) threads = 512;
      if (KT > 0 && threads < KT * 32) threads = KT * 32;
      switch (KT) {
        case 0: return launch_fast<0>(p, threads, smem, st);
        case 1: return launch_fast<1>(p, threads, smem, st);
        case 2: return launch_fast<2>(p, threads, smem, st);
        case 3: return launch_fast<3>(p, threads, smem, st);
        case 4: return launch_fast<4>(p, threads, smem, st);
        case 7: return launch_fast<7>(p, threads, smem, st);
        case 9: return launch_fast<9>(p, threads, smem, st);
        case 10: return launch_fast<10>(p, threads, smem, st);
        case 11: return launch_fast<11>(p, threads, smem, st);
        default: break;  // fall through to the generic kernel
      }
    }
    // restore the unbatched description
    p.n = n; p.rows = rows; p.ldx = ldx; p.m = m;
  }
  if (elem_size == 2) return launch_generic<__half>(p, st);
  return launch_generic<float>(p, st);
}

}  // namespace qr

extern "C" {

int qr_hadamard_f16(const void* x, void* y, int64_t rows, int64_t n, const void* had_k, int K, void* stream) {
  if (K < 1) return qr::fail(QR_EINVAL, "qr_hadamard_f16: K must be >= 1");
  return qr::run_hadq("qr_hadamard_f16", x, rows, n, n, had_k, K, 1.0f, nullptr, nullptr, y, 0, 2,
                      (cudaStream_t)stream);
}

int qr_hadamard_f32(const float* x, float* y, int64_t rows, int64_t n, const void* had_k, int K, void* stream) {
  if (K < 1) return qr::fail(QR_EINVAL, "qr_hadamard_f32: K must be >= 1");
  return qr::run_hadq("qr_hadamard_f32", x, rows, n, n, had_k, K, 1.0f, nullptr, nullptr, y, 0, 4,
                      (cudaStream_t)stream);
}

int qr_hadamard_quant_i4(const void* x, int64_t rows, int64_t n, int64_t ldx, const void* had_k, int K,
                         float clip, uint8_t* q, void* scales, void* y_out, void* stream) {
  if (ldx < n) return qr::fail(QR_EINVAL, "qr_hadamard_quant_i4: ldx < n");
  return qr::run_hadq("qr_hadamard_quant_i4", x, rows, n, ldx, had_k, K, clip, q, scales, y_out, 1, 2,
                      (cudaStream_t)stream);
}

}  // extern "C"
