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

// tensor-core kernel for n = 64 K (hadamard_tc.cu); QR_EUNSUPPORTED means "not my shape"
int launch_hadq_tc(const void* x, int64_t rows, int n, int K, const void* had_k, float clip, uint8_t* q,
                   void* scales, void* y_out, int do_quant, cudaStream_t st);

// heads-axis transform of [rows, heads, head_dim] with two columns per thread (hadamard_walsh.cu); QR_EUNSUPPORTED
// means "not my shape"
int launch_hadq_heads(const void* x, void* y, int64_t rows, int heads, int head_dim, cudaStream_t st);

// warp-per-row Walsh kernel for n = 256 .. 4096 (hadamard_walsh.cu); QR_EUNSUPPORTED means "not my shape"
int launch_hadq_walsh(const void* x, int64_t rows, int n, int64_t ldx, uint32_t stage_mask, float scale, float clip,
                      uint8_t* q, void* scales, void* y_out, int64_t ldy, int do_quant, cudaStream_t st);

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
  int top_bits;       // Walsh-only kernel: 2 when the two top index bits of a work item belong to the transform
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

// Radix-2^R pass over index bits [5, 5+R), in place in the swizzled fp32 row buffer.
// Lanes map to address bits 0..4, so every access is conflict free; the swizzle term of
// element j reduces to the compile-time constant (j & 7) << 2.
template <int R>
__device__ __forceinline__ void pass_b5(float* buf32, int n, int tid, int nthreads) {
  constexpr int N = 1 << R;
  const int groups = n >> R;
  for (int gid = tid; gid < groups; gid += nthreads) {
    const int base = (gid & 31) | ((gid >> 5) << (5 + R));
    const int pb = phys(base);
    float v[N];
#pragma unroll
    for (int j = 0; j < N; ++j) v[j] = buf32[(pb ^ ((j & 7) << 2)) + (j << 5)];
    fwht_regs<N>(v);
#pragma unroll
    for (int j = 0; j < N; ++j) buf32[(pb ^ ((j & 7) << 2)) + (j << 5)] = v[j];
  }
}

// Radix-2^R pass over index bits [b, b+R) with b >= 8: the swizzle term is the same for all j.
template <int R>
__device__ __forceinline__ void pass_hi(float* buf32, int n, int b, int tid, int nthreads) {
  constexpr int N = 1 << R;
  const int groups = n >> R;
  for (int gid = tid; gid < groups; gid += nthreads) {
    const int base = (gid & ((1 << b) - 1)) | ((gid >> b) << (b + R));
    const int pb = phys(base);
    float v[N];
#pragma unroll
    for (int j = 0; j < N; ++j) v[j] = buf32[pb + (j << b)];
    fwht_regs<N>(v);
#pragma unroll
    for (int j = 0; j < N; ++j) buf32[pb + (j << b)] = v[j];
  }
}

__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void cp_async16(uint32_t dst_smem, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_smem), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

// 32 fp16 values (16 half2) -> 16 packed bytes, with torch's division arithmetic.
__device__ __forceinline__ uint4 quant32(const __half2 (&h)[16], float s, float rcp, bool noclamp) {
  const uint32_t* w = reinterpret_cast<const uint32_t*>(h);
  return make_uint4(quant8_words(w[0], w[1], w[2], w[3], s, rcp, noclamp), quant8_words(w[4], w[5], w[6], w[7], s, rcp, noclamp),
                    quant8_words(w[8], w[9], w[10], w[11], s, rcp, noclamp),
                    quant8_words(w[12], w[13], w[14], w[15], s, rcp, noclamp));
}

__device__ __forceinline__ uint32_t quant8_u4(const uint4& v, float s, float rcp, bool noclamp) {
  return quant8_words(v.x, v.y, v.z, v.w, s, rcp, noclamp);
}

// Row absmax across the CTA: warp shuffle, one slot per warp, one barrier.
__device__ __forceinline__ float block_absmax(float amax, float* red, int lane, int warp, int nwarps) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if (lane == 0) red[warp] = amax;
  __syncthreads();
  float a = (lane < nwarps) ? red[lane] : 0.0f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
  return a;
}

__device__ __forceinline__ float scale_from_absmax(float a, float clip, __half* out) {
  const __half s7 = __float2half_rn(__fdiv_rn(a, 7.0f));
  const __half sh = __float2half_rn(__half2float(s7) * clip);
  if (out) *out = sh;
  return __half2float(sh);
}

// Quantise-only kernel (no transform): the row never touches shared memory.  Thread t owns the
// 16-byte chunks t, t + T, t + 2T, t + 3T of the row (coalesced), keeps them in registers across
// the row-wide absmax reduction and stores 4 packed bytes per chunk.  The next row's loads are
// issued before the current row is reduced.
// CPT = 16-byte chunks per thread; PF = request the next row before the current one is reduced (persistent CTAs that
// walk several rows) -- without it and with eight chunks per thread a CTA is small enough that every row of a
// prefill-sized call is resident at once.
template <int CPT, bool PF>
__global__ void __launch_bounds__(PF ? 1024 : 512)
quant_rows_kernel(const HadqParams p) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[2][32];
  const int tid = threadIdx.x, T = blockDim.x, lane = tid & 31, warp = tid >> 5, nwarps = T >> 5;
  const int nchunks = p.n >> 3;
  uint4 cur[CPT], nxt[PF ? CPT : 1];
  int64_t row = blockIdx.x;
  const uint4 zero = make_uint4(0, 0, 0, 0);
  if (row < p.rows) {
    const uint4* xr = reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(p.x) + row * p.ldx);
#pragma unroll
    for (int j = 0; j < CPT; ++j) cur[j] = (tid + j * T < nchunks) ? __ldg(xr + tid + j * T) : zero;
  }
  int parity = 0;
  for (; row < p.rows; row += gridDim.x, parity ^= 1) {
    const int64_t nrow = row + gridDim.x;
    if (PF && nrow < p.rows) {
      const uint4* xn = reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(p.x) + nrow * p.ldx);
#pragma unroll
      for (int j = 0; j < CPT; ++j) nxt[j] = (tid + j * T < nchunks) ? __ldg(xn + tid + j * T) : zero;
    }
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < CPT; ++j) amax = fmaxf(amax, absmax8(cur[j]));
    const float a = block_absmax(amax, red[parity], lane, warp, nwarps);
    const float s = scale_from_absmax(a, p.clip, tid == 0 ? p.scales + row : nullptr);
    const float rcp = (s != 0.0f) ? __frcp_rn(s) : 0.0f;
    const bool noclamp = clamp_free(s, p.clip);
    uint32_t* qo = reinterpret_cast<uint32_t*>(p.q + row * (int64_t)(p.n >> 1));
    uint4* yo = p.y_out ? reinterpret_cast<uint4*>(reinterpret_cast<__half*>(p.y_out) + row * (int64_t)p.n) : nullptr;
#pragma unroll
    for (int j = 0; j < CPT; ++j) {
      const int c = tid + j * T;
      if (c < nchunks) {
        qo[c] = quant8_u4(cur[j], s, rcp, noclamp);
        if (yo) yo[c] = cur[j];
      }
    }
    if (PF) {
#pragma unroll
      for (int j = 0; j < CPT; ++j) cur[j] = nxt[j];
    } else if (nrow < p.rows) {
      const uint4* xn = reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(p.x) + nrow * p.ldx);
#pragma unroll
      for (int j = 0; j < CPT; ++j) cur[j] = (tid + j * T < nchunks) ? __ldg(xn + tid + j * T) : zero;
    }
  }
}

// RMS normalisation fused in front of the quantiser (the step directly before the path for the QKV and gate/up
// inputs): y = fp16(x * rsqrt(mean(x^2) + eps)) in fp32 as the weight-less RMSNorm of the reference computes it,
// then absmax -> scale -> int4 codes of y.  Same structure as quant_rows_kernel; the row-wide reduction carries the
// sum of squares next to the absmax, and the absmax of y is taken from the absmax of x (rounding is monotone:
// max_i fp16(|x_i| r) = fp16(max_i |x_i| r)), so one barrier serves both.
struct RmsQuantParams {
  const __half* x;
  int64_t ldx, rows;
  int n;
  float eps, mean_dim, clip;
  uint8_t* q;
  __half* scales;
  __half* y_out;     // optional copy of the normalised row, or null
};

// CPT = 16-byte chunks per thread: 4 for persistent CTAs that walk the rows, 8 for one small CTA per row where every row
// of the call can be resident at once (as in quant_rows_kernel).
template <int CPT>
__global__ void __launch_bounds__(CPT == 8 ? 512 : 1024)
rmsnorm_quant_rows_kernel(const RmsQuantParams p) {
  __shared__ float red_max[2][32];
  __shared__ float red_ss[2][32];
  const int tid = threadIdx.x, T = blockDim.x, lane = tid & 31, warp = tid >> 5, nwarps = T >> 5;
  const int nchunks = p.n >> 3;
  const uint4 zero = make_uint4(0, 0, 0, 0);
  int parity = 0;
  for (int64_t row = blockIdx.x; row < p.rows; row += gridDim.x, parity ^= 1) {
    const uint4* xr = reinterpret_cast<const uint4*>(p.x + row * p.ldx);
    uint4 cur[CPT];
#pragma unroll
    for (int j = 0; j < CPT; ++j) cur[j] = (tid + j * T < nchunks) ? __ldg(xr + tid + j * T) : zero;
    float amax = 0.0f, ss = 0.0f;
#pragma unroll
    for (int j = 0; j < CPT; ++j) {
      const __half2* h = reinterpret_cast<const __half2*>(&cur[j]);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __half22float2(h[e]);
        ss = __fmaf_rn(f.x, f.x, ss);
        ss = __fmaf_rn(f.y, f.y, ss);
      }
      amax = fmaxf(amax, absmax8(cur[j]));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      ss += __shfl_xor_sync(0xffffffffu, ss, o);
    }
    if (lane == 0) { red_max[parity][warp] = amax; red_ss[parity][warp] = ss; }
    __syncthreads();
    float a = (lane < nwarps) ? red_max[parity][lane] : 0.0f;
    float t = (lane < nwarps) ? red_ss[parity][lane] : 0.0f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
      t += __shfl_xor_sync(0xffffffffu, t, o);
    }
    const float r = rsqrtf(__fdiv_rn(t, p.mean_dim) + p.eps);
    const float ymax = __half2float(__float2half_rn(a * r));
    const float s = scale_from_absmax(ymax, p.clip, tid == 0 ? p.scales + row : nullptr);
    const float rcp = (s != 0.0f) ? __frcp_rn(s) : 0.0f;
    const bool noclamp = clamp_free(s, p.clip);
    uint32_t* qo = reinterpret_cast<uint32_t*>(p.q + row * (int64_t)(p.n >> 1));
    uint4* yo = p.y_out ? reinterpret_cast<uint4*>(p.y_out + row * (int64_t)p.n) : nullptr;
#pragma unroll
    for (int j = 0; j < CPT; ++j) {
      const int c = tid + j * T;
      if (c < nchunks) {
        const __half2* h = reinterpret_cast<const __half2*>(&cur[j]);
        uint4 y;
        uint32_t* yw = reinterpret_cast<uint32_t*>(&y);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __half22float2(h[e]);
          const __half2 yh = __floats2half2_rn(f.x * r, f.y * r);
          yw[e] = *reinterpret_cast<const uint32_t*>(&yh);
        }
        qo[c] = quant8_u4(y, s, rcp, noclamp);
        if (yo) yo[c] = y;
      }
    }
  }
}

// KT = number of 16-wide k tiles of the dense factor (0 when K == 1).  One thread per group of
// 32 consecutive outputs; blockDim.x >= n / 32 (rounded up to whole warps).
// Largest CTA each instantiation is compiled for (bounds the registers per thread).
__host__ __device__ constexpr int hadq_max_threads(int KT) {
  return KT == 0 ? 512 : KT <= 2 ? 1024 : KT <= 4 ? 512 : KT == 7 ? 448 : KT == 9 ? 576 : KT == 10 ? 640 : 384;
}

// Resident CTAs of the largest size per SM the instantiation is compiled for.  The CTAs of the Walsh-only kernel are
// small (n / 32 threads), so the registers per thread decide how many rows an SM works on at once: two CTAs of 512
// threads = 64 registers = eight rows of 4096 in flight instead of four at the 108 registers the compiler would take
// (2048 x 4096: 13.9 -> 11.7 us; 80 registers 12.1 us, 56 registers 13.9 us, 48 registers 17.0 us).
__host__ __device__ constexpr int hadq_min_blocks(int KT) { return KT == 0 ? 2 : 1; }

template <int KT>
__global__ void __launch_bounds__(hadq_max_threads(KT), hadq_min_blocks(KT))
hadq_fast_kernel(const HadqParams p) {
  pdl_launch_dependents();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int tid = threadIdx.x;
  const int nthreads = blockDim.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int nwarps = nthreads >> 5;
  const int n = p.n;
  const int m = p.m;
  const int K = p.K;
  const int ngroups = n >> 5;

  // shared memory: [fp32 row buffer (swizzled)][staging for the dense-factor operand][reduction slots]
  const int pitch = m + 8;  // halfs
  const int raw_bytes = (KT > 0) ? ((KT * 16 * pitch * 2 + 15) & ~15) : 0;
  float* buf32 = reinterpret_cast<float*>(smem_raw);
  __half* raw = reinterpret_cast<__half*>(smem_raw + (size_t)n * 4);
  float* red = reinterpret_cast<float*>(smem_raw + (size_t)n * 4 + raw_bytes);

  // dense-factor fragments: warp w owns 16 output rows (M tile w % MT) for the lifetime of the CTA
  constexpr int KTT = KT > 0 ? KT : 1;
  constexpr int MT = KT > 0 ? KT : 1;
  uint32_t afrag[KTT][4];
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
  // the table does not depend on the kernel in front, the activations do: its fragments were requested above
  pdl_wait();

  // Kronecker form: the raw row goes to the staging buffer with asynchronous 16-byte copies, so that the next row is
  // on its way from memory while the current one runs through its passes (the staging buffer is free as soon as the
  // dense factor has been applied).  The k padding rows of the buffer are zero once and for all.
  auto stage_row = [&](int64_t r) {
    const __half* xs = reinterpret_cast<const __half*>(p.x) + r * p.ldx;
    const int vec_per_k = m >> 3, vshift = p.wbits - 3;     // m is a power of two
    for (int c = tid; c < (n >> 3); c += nthreads)
      cp_async16(smem_u32(raw + (c >> vshift) * pitch + ((c & (vec_per_k - 1)) << 3)), xs + (size_t)c * 8);
  };
  if (KT > 0) {
    const int vec_per_k = m >> 3, vshift = p.wbits - 3;
    const int pad_vecs = (KT * 16 - K) * vec_per_k;
    for (int c = tid; c < pad_vecs; c += nthreads)
      *reinterpret_cast<uint4*>(raw + (K + (c >> vshift)) * pitch + ((c & (vec_per_k - 1)) << 3)) = make_uint4(0, 0, 0, 0);
    if ((int64_t)blockIdx.x < p.rows) stage_row(blockIdx.x);
  }

  int parity = 0;
  for (int64_t row = blockIdx.x; row < p.rows; row += gridDim.x, parity ^= 1) {
    const __half* xr = reinterpret_cast<const __half*>(p.x) + row * p.ldx;
    int scalar_bits = p.wbits - 5;   // index bits left for the shared-memory passes

    if (KT > 0) {
      // ---- stage 0: the raw row is in flight to the padded staging buffer (requested one row ahead, see below)
      cp_async_wait_all();
      __syncthreads();
      // ---- stage 1: D = hadK . X on tensor cores, 64 columns per unit
      const int nchunks = m >> 6;
      const int warps_per_mt = nwarps / MT;
      if (warp < warps_per_mt * MT) {
        const int g = lane >> 2, t = lane & 3;
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
              ldmatrix_x4_trans(b, smem_u32(raw + (kt * 16 + lrow) * pitch + ch * 64 + np * 16 + lcol));
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
    } else {
      // ---- stage A (Walsh only): coalesced 128-bit loads; thread t owns chunks t + j * n/32, i.e. the
      //      two top index bits are local, and transforms them when they belong to the transform
      const bool top2 = (p.top_bits == 2);
      if (top2) scalar_bits -= 2;
      if (tid < ngroups) {
        float v[4][8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint4 u = __ldg(reinterpret_cast<const uint4*>(xr) + tid + j * ngroups);
          const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = __half22float2(h[e]);
            v[j][2 * e] = f.x;
            v[j][2 * e + 1] = f.y;
          }
        }
        if (top2) {
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float t0 = v[0][e] + v[1][e], t1 = v[0][e] - v[1][e];
            const float t2 = v[2][e] + v[3][e], t3 = v[2][e] - v[3][e];
            v[0][e] = t0 + t2; v[1][e] = t1 + t3; v[2][e] = t0 - t2; v[3][e] = t1 - t3;
          }
        }
        const int sw = ((tid >> 2) & 7) << 2;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int i0 = 8 * tid + j * (n >> 2);
          *reinterpret_cast<float4*>(buf32 + (i0 ^ sw)) = make_float4(v[j][0], v[j][1], v[j][2], v[j][3]);
          *reinterpret_cast<float4*>(buf32 + ((i0 + 4) ^ sw)) = make_float4(v[j][4], v[j][5], v[j][6], v[j][7]);
        }
      }
    }

    // ---- scalar passes over index bits 5 .. 5 + scalar_bits - 1
    if (scalar_bits > 0) {
      int r1 = scalar_bits <= 5 ? scalar_bits : (scalar_bits + 1) / 2;
      if (r1 > 4 && scalar_bits > 5) r1 = 4;
      __syncthreads();
      if (KT > 0 && row + gridDim.x < p.rows) stage_row(row + gridDim.x);   // every warp is done with the staging buffer
      switch (r1) {
        case 1: pass_b5<1>(buf32, n, tid, nthreads); break;
        case 2: pass_b5<2>(buf32, n, tid, nthreads); break;
        case 3: pass_b5<3>(buf32, n, tid, nthreads); break;
        case 4: pass_b5<4>(buf32, n, tid, nthreads); break;
        default: pass_b5<5>(buf32, n, tid, nthreads); break;
      }
      int b = 5 + r1;
      int rem = scalar_bits - r1;
      while (rem > 0) {   // b >= 8 here because r1 >= 3 whenever a second pass exists
        const int r = rem > 4 ? (rem + 1) / 2 : rem;
        __syncthreads();
        switch (r) {
          case 1: pass_hi<1>(buf32, n, b, tid, nthreads); break;
          case 2: pass_hi<2>(buf32, n, b, tid, nthreads); break;
          case 3: pass_hi<3>(buf32, n, b, tid, nthreads); break;
          default: pass_hi<4>(buf32, n, b, tid, nthreads); break;
        }
        b += r < 4 ? r : 4;
        rem -= r < 4 ? r : 4;
      }
    }
    __syncthreads();

    // ---- final pass: index bits 0..4 in registers; thread t ends with outputs [32 t, 32 t + 32)
    __half2 h[16];
    float amax = 0.0f;
    if (tid < ngroups) {
      float v[32];
#pragma unroll
      for (int s = 0; s < 8; ++s) {
        const float4 f = *reinterpret_cast<const float4*>(buf32 + tid * 32 + ((s ^ (tid & 7)) << 2));
        v[4 * s] = f.x; v[4 * s + 1] = f.y; v[4 * s + 2] = f.z; v[4 * s + 3] = f.w;
      }
      fwht_regs<32>(v);
      __half2 mx = __float2half2_rn(0.0f);
#pragma unroll
      for (int e = 0; e < 16; ++e) {
        h[e] = __floats2half2_rn(v[2 * e] * p.scale, v[2 * e + 1] * p.scale);
        mx = __hmax2(mx, __habs2(h[e]));
      }
      const float2 mf = __half22float2(mx);
      amax = fmaxf(mf.x, mf.y);
      if (p.y_out) {
        uint4* yo = reinterpret_cast<uint4*>(reinterpret_cast<__half*>(p.y_out) + row * (int64_t)n + tid * 32);
#pragma unroll
        for (int s = 0; s < 4; ++s) yo[s] = *reinterpret_cast<const uint4*>(&h[4 * s]);
      }
    }
    if (p.do_quant) {
      const float a = block_absmax(amax, red + 32 * parity, lane, warp, nwarps);
      const float s = scale_from_absmax(a, p.clip, tid == 0 ? p.scales + row : nullptr);
      const float rcp = (s != 0.0f) ? __frcp_rn(s) : 0.0f;
      if (tid < ngroups)
        *reinterpret_cast<uint4*>(p.q + row * (int64_t)(n >> 1) + tid * 16) = quant32(h, s, rcp, clamp_free(s, p.clip));
    } else {
      __syncthreads();   // the row buffer is rewritten by the next row
    }
  }
}

// ------------------------------------------------------------------ generic
// ---------------------------------------------------------------------------------------------------------------
// Few rows of n = 64 K (decode: the down_proj input of a 7B model, 11008 = 172 x 64): one row per CTA leaves the
// GPU idle and the row's dense factor (K / 16 tiles x 8 x K / 16 MMAs) is what the CTA waits for.  Here a cluster of
// four CTAs shares a row: every CTA stages the whole raw row but computes only its quarter of the factor's output
// rows k', which it can finish by itself -- the Walsh transform runs along the 64 columns of each k' -- so the only
// exchange is the row's absmax, four floats through distributed shared memory behind one cluster barrier per row.
constexpr int kSplitCtas = 4;

__device__ __forceinline__ uint32_t hq_cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void hq_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float hq_peer_float(const float* p, uint32_t rank) {
  uint32_t a = smem_u32(p), ra;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(a), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(ra) : "memory");
  return v;
}

// KT = 16-wide tiles of the dense factor; TPC = tiles per CTA = ceil(KT / 4); two warps per tile (four of the eight
// 8-column MMA tiles each).  blockDim.x = 64 TPC.
template <int KT>
__global__ void __launch_bounds__(64 * ((KT + kSplitCtas - 1) / kSplitCtas))
hadq_split_kernel(const HadqParams p) {
  constexpr int TPC = (KT + kSplitCtas - 1) / kSplitCtas;
  constexpr int kLocal = TPC * 16 * 64;                  // elements of a row this CTA produces
  pdl_launch_dependents();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ float s_red[2][32];
  __shared__ float s_cmax[2];                            // this CTA's absmax of the current / the next row
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  const int K = p.K, n = p.n;
  const uint32_t rank = hq_cluster_rank();
  const int cluster_id = blockIdx.x / kSplitCtas, num_clusters = gridDim.x / kSplitCtas;
  constexpr int pitch = 64 + 8;                          // halfs per staged k row
  float* buf32 = reinterpret_cast<float*>(smem_raw);                       // [TPC * 16][64], swizzled
  __half* raw = reinterpret_cast<__half*>(smem_raw + (size_t)kLocal * 4);  // [KT * 16][pitch]

  // this warp's tile of the factor and its fragments (rows of the tile x all k)
  const int mt = (int)rank * TPC + (warp >> 1);          // global tile
  const int g = lane >> 2, t = lane & 3;
  uint32_t afrag[KT][4];
#pragma unroll
  for (int kt = 0; kt < KT; ++kt) {
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int row = mt * 16 + g + ((r & 1) ? 8 : 0);
      const int col = kt * 16 + 2 * t + ((r & 2) ? 8 : 0);
      uint32_t val = 0;
      if (row < K && col < K) val = *reinterpret_cast<const uint32_t*>(p.had_k + (size_t)row * K + col);
      afrag[kt][r] = val;
    }
  }
  auto stage_row = [&](int64_t r) {
    const __half* xs = reinterpret_cast<const __half*>(p.x) + r * p.ldx;
    for (int c = tid; c < (n >> 3); c += blockDim.x)
      cp_async16(smem_u32(raw + (c >> 3) * pitch + ((c & 7) << 3)), xs + (size_t)c * 8);
  };
  for (int c = tid; c < (KT * 16 - K) * 8; c += blockDim.x)
    *reinterpret_cast<uint4*>(raw + (K + (c >> 3)) * pitch + ((c & 7) << 3)) = make_uint4(0, 0, 0, 0);
  pdl_wait();     // the table does not depend on the kernel in front, the activations do
  if (cluster_id < p.rows) stage_row(cluster_id);

  int parity = 0;
  for (int64_t row = cluster_id; row < p.rows; row += num_clusters, parity ^= 1) {
    cp_async_wait_all();
    __syncthreads();
    // ---- dense factor: this warp's 16 rows k' x 32 of the 64 columns
    {
      const int lrow = (lane & 7) + ((lane >> 3) & 1) * 8;
      const int lcol = (lane >> 4) * 8;
      const int half = warp & 1;
      float acc[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.0f; }
#pragma unroll
      for (int kt = 0; kt < KT; ++kt) {
#pragma unroll
        for (int np = 0; np < 2; ++np) {
          uint32_t b[4];
          ldmatrix_x4_trans(b, smem_u32(raw + (kt * 16 + lrow) * pitch + (2 * half + np) * 16 + lcol));
          mma_16816(acc[2 * np], afrag[kt], b[0], b[1]);
          mma_16816(acc[2 * np + 1], afrag[kt], b[2], b[3]);
        }
      }
      const int r0 = (warp >> 1) * 16 + g;               // local row
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        const int col = half * 32 + nt * 8 + 2 * t;
        *reinterpret_cast<float2*>(buf32 + phys(r0 * 64 + col)) = make_float2(acc[nt][0], acc[nt][1]);
        *reinterpret_cast<float2*>(buf32 + phys((r0 + 8) * 64 + col)) = make_float2(acc[nt][2], acc[nt][3]);
      }
    }
    __syncthreads();
    if (row + num_clusters < p.rows) stage_row(row + num_clusters);   // every warp is done with the staging buffer
    // ---- Walsh over the 64 columns: bit 5 through shared memory, bits 0 .. 4 in registers
    pass_b5<1>(buf32, kLocal, tid, blockDim.x);
    __syncthreads();
    __half2 h[16];
    float amax = 0.0f;
    const int kprime = (int)rank * TPC * 16 + (tid >> 1);      // the factor's output row of this thread's 32 elements
    const bool live = tid < (kLocal >> 5) && kprime < K;
    if (tid < (kLocal >> 5)) {
      float v[32];
#pragma unroll
      for (int s = 0; s < 8; ++s) {
        const float4 f = *reinterpret_cast<const float4*>(buf32 + tid * 32 + ((s ^ (tid & 7)) << 2));
        v[4 * s] = f.x; v[4 * s + 1] = f.y; v[4 * s + 2] = f.z; v[4 * s + 3] = f.w;
      }
      fwht_regs<32>(v);
      __half2 mx = __float2half2_rn(0.0f);
#pragma unroll
      for (int e = 0; e < 16; ++e) {
        h[e] = __floats2half2_rn(v[2 * e] * p.scale, v[2 * e + 1] * p.scale);
        mx = __hmax2(mx, __habs2(h[e]));
      }
      const float2 mf = __half22float2(mx);
      if (live) amax = fmaxf(mf.x, mf.y);
      if (live && p.y_out) {
        uint4* yo = reinterpret_cast<uint4*>(reinterpret_cast<__half*>(p.y_out) + row * (int64_t)n + (size_t)kprime * 64 + (tid & 1) * 32);
#pragma unroll
        for (int s = 0; s < 4; ++s) yo[s] = *reinterpret_cast<const uint4*>(&h[4 * s]);
      }
    }
    // ---- the row's absmax: CTA-wide, then over the four CTAs
    const float a_cta = block_absmax(amax, s_red[parity], lane, warp, nwarps);
    if (tid == 0) s_cmax[parity] = a_cta;
    hq_cluster_sync();
    float a = 0.0f;
#pragma unroll
    for (uint32_t r = 0; r < (uint32_t)kSplitCtas; ++r) a = fmaxf(a, hq_peer_float(&s_cmax[parity], r));
    const float s = scale_from_absmax(a, p.clip, (tid == 0 && rank == 0) ? p.scales + row : nullptr);
    const float rcp = (s != 0.0f) ? __frcp_rn(s) : 0.0f;
    if (live)
      *reinterpret_cast<uint4*>(p.q + row * (int64_t)(n >> 1) + (size_t)kprime * 32 + (tid & 1) * 16) = quant32(h, s, rcp, clamp_free(s, p.clip));
  }
  hq_cluster_sync();      // nobody leaves while a peer may still read its absmax
}

template <int KT>
static int launch_split(const HadqParams& p, cudaStream_t st) {
  constexpr int TPC = (KT + kSplitCtas - 1) / kSplitCtas;
  const size_t smem = (size_t)TPC * 16 * 64 * 4 + (size_t)KT * 16 * (64 + 8) * 2;
  static thread_local size_t configured[64] = {0};
  int dev = 0;
  QR_CUDA(cudaGetDevice(&dev));
  if (smem > 48 * 1024 && (dev >= 64 || configured[dev] < smem)) {
    QR_CUDA(cudaFuncSetAttribute(hadq_split_kernel<KT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (dev < 64) configured[dev] = smem;
  }
  int64_t clusters = p.rows;
  const int64_t cap = (int64_t)num_sms() / 2; // two CTAs per SM are resident at 148 registers; more rows than clusters walk the rows
  if (clusters > cap) clusters = cap;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(clusters * kSplitCtas));
  cfg.blockDim = dim3(64 * TPC);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = kSplitCtas; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = use_pdl(p.rows) ? 2 : 1;
  QR_CUDA(cudaLaunchKernelEx(&cfg, hadq_split_kernel<KT>, p));
  return QR_OK;
}

template <typename T> __device__ __forceinline__ float load_as_float(const T* p, int64_t i);
template <> __device__ __forceinline__ float load_as_float<__half>(const __half* p, int64_t i) { return __half2float(p[i]); }
template <> __device__ __forceinline__ float load_as_float<float>(const float* p, int64_t i) { return p[i]; }

template <typename T>
__global__ void __launch_bounds__(256)
hadq_generic_kernel(const HadqParams p) {
  pdl_launch_dependents();
  pdl_wait();
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

static int persistent_grid(int64_t rows, int threads, size_t smem) {
  int per_sm = (int)(227 * 1024 / (smem + 1024));
  const int by_threads = 2048 / threads;
  if (per_sm > by_threads) per_sm = by_threads;
  if (per_sm > 16) per_sm = 16;
  if (per_sm < 1) per_sm = 1;
  int64_t grid = (int64_t)num_sms() * per_sm;
  if (grid > rows) grid = rows;
  return (int)grid;
}

template <int KT>
static int launch_fast(const HadqParams& p, int threads, size_t smem, cudaStream_t st) {
  static thread_local size_t configured[64] = {0};
  int dev = 0;
  QR_CUDA(cudaGetDevice(&dev));
  if (dev >= 64 || configured[dev] < smem) {
    QR_CUDA(cudaFuncSetAttribute(hadq_fast_kernel<KT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (dev < 64) configured[dev] = smem;
  }
  QR_CUDA(launch_kernel(hadq_fast_kernel<KT>, dim3(persistent_grid(p.rows, threads, smem)), dim3(threads), smem, st,
                        use_pdl(p.rows), p));
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
  QR_CUDA(launch_kernel(hadq_generic_kernel<T>, dim3((int)grid), dim3(256), smem, st, use_pdl(p.rows), p));
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

  p.top_bits = 0;
  const int forced = g_tuning.hadq_path;  // 1 = always generic (for A/B checks)
  const bool base_ok = (elem_size == 2) && forced != 1 && aligned16(x) && (ldx % 8 == 0) && (n % 8 == 0) &&
                       (!y_out || aligned16(y_out)) && (!do_quant || aligned16(q)) && n <= 32768;
  if (base_ok && K == 0 && do_quant && n >= 64) {
    // small CTAs of eight chunks per thread when every row can be resident at once (one wave), else persistent CTAs
    // of four chunks per thread that request their next row early
    const int threads8 = ((n / 8 + 7) / 8 + 31) / 32 * 32;
    if (rows >= 256 && rows <= (int64_t)num_sms() * 16 && threads8 <= 512 && rows * (int64_t)threads8 <= (int64_t)num_sms() * 1536) {
      QR_CUDA(launch_kernel(quant_rows_kernel<8, false>, dim3((unsigned)rows), dim3(threads8), 0, st, use_pdl(p.rows), p));
      return QR_OK;
    }
    int threads = ((n / 8 + 3) / 4 + 31) / 32 * 32;
    QR_CUDA(launch_kernel(quant_rows_kernel<4, true>, dim3(persistent_grid(rows, threads, 1024)), dim3(threads), 0, st,
                          use_pdl(p.rows), p));
    return QR_OK;
  }
  // few rows of n = 64 K with the quantiser behind: a cluster of four CTAs per row
  // (11008 = 172 x 64: 3.8 against 5.2 us for one row, 4.0 against 5.3 us for eight, 4.8 against 5.5 us for 32; from
  // 64 rows on one CTA per row is as fast, and every CTA of a cluster stages the whole row)
  if (base_ok && K > 1 && m == 64 && ldx == n && do_quant && rows <= 32 && g_tuning.hadq_split != 0) {
    switch (kt_for(K)) {
      case 7: return launch_split<7>(p, st);
      case 9: return launch_split<9>(p, st);
      case 10: return launch_split<10>(p, st);
      case 11: return launch_split<11>(p, st);
      default: break;
    }
  }
  // (below 129 rows the persistent tensor-core kernel's set-up is not amortised: 7.2 against 6.4 us at 8 rows of 11008)
  if (base_ok && K > 1 && m == 64 && ldx == n && (rows > 128 || g_tuning.hadq_tc == 2) && g_tuning.hadq_tc != 0) {
    const int rc = launch_hadq_tc(x, rows, n, K, had_k, clip, q, scales, y_out, do_quant, st);
    if (rc != QR_EUNSUPPORTED) return rc;
  }
  if (base_ok && K == 1 && n >= 256 && n <= 4096 && g_tuning.hadq_walsh != 0) {
    const int rc = launch_hadq_walsh(x, rows, n, ldx, (uint32_t)(n - 1), p.scale, clip, q, scales, y_out, n, do_quant, st);
    if (rc != QR_EUNSUPPORTED) return rc;
  }
  bool fast = base_ok && K >= 1 && (n % 32 == 0) && (!do_quant || (n % 32 == 0));
  if (fast) {
    if (K == 1) { fast = (n >= 1024); p.top_bits = 2; }
    else fast = (m >= 64);
  }
  // Walsh-only with short rows and no quantisation: batch 1024/n consecutive rows per work item
  if (!fast && base_ok && K == 1 && !do_quant && n >= 32 && n < 1024 && ldx == n) {
    const int per = 1024 / n;
    if (rows % per == 0) {
      p.n = 1024; p.rows = rows / per; p.ldx = 1024; p.m = n; p.top_bits = 0; fast = true;
    }
  }
  if (fast) {
    const int KT = kt_for(K);
    const int pitch = p.m + 8;
    const size_t raw = KT ? (((size_t)KT * 16 * pitch * 2 + 15) & ~(size_t)15) : 0;
    const size_t smem = (size_t)p.n * 4 + raw + 256;
    int threads = (p.n / 32 + 31) / 32 * 32;
    if (KT > 0 && threads < KT * 32) threads = KT * 32;
    // the dense factor is dealt out as (16-row tile, 64-column chunk) units, one per warp and round: enough warps for
    // one round where the CTA may be that large (28 x 1024: 32 warps for 2 x 16 units instead of 28)
    if (KT > 0) {
      const int one_round = KT * (p.m >> 6) * 32;
      if (one_round > threads && one_round <= hadq_max_threads(KT)) threads = one_round;
    }
    if (smem <= 227 * 1024 && threads <= hadq_max_threads(KT)) {
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
    p.n = n; p.rows = rows; p.ldx = ldx; p.m = m; p.top_bits = 0;
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

int qr_hadamard_heads_f16(const void* x, void* y, int64_t rows, int64_t heads, int64_t head_dim, void* stream) {
  if (rows < 0 || heads < 1 || head_dim < 1) return qr::fail(QR_EINVAL, "qr_hadamard_heads_f16: bad size");
  if (rows == 0) return QR_OK;
  if (!x || !y) return qr::fail(QR_EINVAL, "qr_hadamard_heads_f16: null pointer");
  const int64_t n = heads * head_dim;
  if (!qr::is_pow2(heads) || !qr::is_pow2(head_dim) || head_dim < 32 || n < 256 || n > 4096)
    return qr::fail(QR_EUNSUPPORTED, "qr_hadamard_heads_f16: heads = %lld, head_dim = %lld (powers of two, head_dim >= 32, "
                    "256 <= heads x head_dim <= 4096)", (long long)heads, (long long)head_dim);
  if (qr::g_tuning.hadq_heads != 0 && qr::aligned16(x) && qr::aligned16(y)) {
    const int rc2 = qr::launch_hadq_heads(x, y, rows, (int)heads, (int)head_dim, (cudaStream_t)stream);
    if (rc2 != QR_EUNSUPPORTED) return rc2;
  }
  const uint32_t mask = (uint32_t)((heads - 1) * head_dim);      // the index bits of the heads axis
  const int rc = qr::launch_hadq_walsh(x, rows, (int)n, n, mask, (float)(1.0 / sqrt((double)heads)), 1.0f, nullptr, nullptr,
                                       y, n, 0, (cudaStream_t)stream);
  if (rc == QR_EUNSUPPORTED) return qr::fail(QR_EALIGN, "qr_hadamard_heads_f16: x and y must be 16-byte aligned");
  return rc;
}

int qr_hadamard_quant_i4(const void* x, int64_t rows, int64_t n, int64_t ldx, const void* had_k, int K,
                         float clip, uint8_t* q, void* scales, void* y_out, void* stream) {
  if (ldx < n) return qr::fail(QR_EINVAL, "qr_hadamard_quant_i4: ldx < n");
  return qr::run_hadq("qr_hadamard_quant_i4", x, rows, n, ldx, had_k, K, clip, q, scales, y_out, 1, 2,
                      (cudaStream_t)stream);
}

int qr_rmsnorm_quant_i4(const void* x, int64_t rows, int64_t n, int64_t ldx, int64_t mean_dim, float eps, float clip,
                        uint8_t* q, void* scales, void* y_out, void* stream) {
  if (rows < 0 || n < 0) return qr::fail(QR_EINVAL, "qr_rmsnorm_quant_i4: negative size");
  if (rows == 0 || n == 0) return QR_OK;
  if (!x || !q || !scales) return qr::fail(QR_EINVAL, "qr_rmsnorm_quant_i4: null pointer");
  if (ldx < n) return qr::fail(QR_EINVAL, "qr_rmsnorm_quant_i4: ldx < n");
  if (mean_dim <= 0) return qr::fail(QR_EINVAL, "qr_rmsnorm_quant_i4: mean_dim must be positive");
  if (n % 8 != 0 || n < 64 || n > 32768) return qr::fail(QR_EUNSUPPORTED, "qr_rmsnorm_quant_i4: n = %lld (a multiple of 8 in [64, 32768])", (long long)n);
  if (!qr::aligned16(x) || ldx % 8 != 0 || !qr::aligned16(q) || (y_out && !qr::aligned16(y_out)))
    return qr::fail(QR_EALIGN, "qr_rmsnorm_quant_i4: x, q and y_out must be 16-byte aligned, ldx % 8 == 0");
  qr::RmsQuantParams p;
  p.x = reinterpret_cast<const __half*>(x); p.ldx = ldx; p.rows = rows; p.n = (int)n;
  p.eps = eps; p.mean_dim = (float)mean_dim; p.clip = clip;
  p.q = q; p.scales = reinterpret_cast<__half*>(scales); p.y_out = reinterpret_cast<__half*>(y_out);
  const int threads8 = (((int)n / 8 + 7) / 8 + 31) / 32 * 32;
  if (rows >= 256 && rows <= (int64_t)qr::num_sms() * 16 && threads8 <= 512 && rows * (int64_t)threads8 <= (int64_t)qr::num_sms() * 1536) {
    QR_CUDA(qr::launch_kernel(qr::rmsnorm_quant_rows_kernel<8>, dim3((unsigned)rows), dim3(threads8), 0, (cudaStream_t)stream, false, p));
    return QR_OK;
  }
  int threads = (((int)n / 8 + 3) / 4 + 31) / 32 * 32;
  QR_CUDA(qr::launch_kernel(qr::rmsnorm_quant_rows_kernel<4>, dim3(qr::persistent_grid(rows, threads, 1024)), dim3(threads), 0,
                            (cudaStream_t)stream, false, p));
  return QR_OK;
}

}  // extern "C"
