// Kernel (a), pure Walsh case for rows of 256 .. 4096 elements (config 0: n = 4096): one WARP per token row, the
// whole row in registers, no shared memory and no CTA-wide barrier.
//
// Lane l loads the 16-byte chunks l, l + 32, l + 64, ... of the row (coalesced 128-bit loads), so of the index
// bits of an element
//     bits 0..2   select the element inside a chunk            (registers)
//     bits 3..7   select the lane                              (lane = bits 3..7)
//     bits 8..11  select the chunk j of the lane               (registers)
// and the Walsh transform -- one butterfly stage per index bit, in any order -- splits into
//   * bits 0, 1, 3, 4: ONE mma.sync.m16n8k16 pair per chunk, straight on the raw fp16 input.  The four 32-bit words
//     of a chunk are exactly an A fragment of a 16 x 16 tile whose contraction index k is (bit 0, bits 3..4 = the
//     lane's position in its group of four, bit 1) and whose row index is (bits 5..7 = lane / 4, bit 2); B is the
//     16 x 16 Sylvester matrix, +-1 in fp16.  Products are exact, accumulation is fp32, and the D fragment puts the
//     sixteen outputs back where the inputs were: every lane ends with the same eight consecutive elements,
//     now as fp32;
//   * bit 2 and bits 8..11: butterflies between registers of one lane;
//   * bits 5, 6, 7: three warp-shuffle stages (shfl.xor with 4, 8, 16; the subtracting side is folded into one
//     fused multiply-add with a per-lane sign).
// Then 1/sqrt(n), rounding to fp16 (the rounding OnlineHadamard applies), the row absmax by warp shuffles, the
// scale, and every chunk leaves as four packed bytes (coalesced 128 bytes per warp and store).
// `stage_mask` selects the index bits that are transformed: all of them for the Hadamard of the whole row, only
// the high ones for a transform over the leading axis of a [heads, head_dim] row (the heads-axis Hadamard in front
// of o_proj, which upstream applies to a transposed view).
#include "common.cuh"

#include <math.h>

namespace qr {

struct WalshParams {
  const __half* x;
  int64_t ldx;
  int64_t rows;
  int n;
  uint32_t stage_mask;   // bit b set: butterfly stage on index bit b
  float scale;
  float clip;
  uint8_t* q;
  __half* scales;
  __half* y_out;
  int64_t ldy;
  int do_quant;
};

constexpr int kWalshWarps = 12;   // three warps per scheduler: up to 168 registers per thread, enough for a 4096-element row

__device__ __forceinline__ void mma_f16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                              uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
      : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f), "f"(0.0f), "f"(0.0f), "f"(0.0f));
}

// +-1 pair (H16[k][n], H16[k + 1][n]) as a half2 word, H16[k][n] = (-1)^popcount(k & n)
__device__ __forceinline__ uint32_t h16_pair(int k, int n) {
  const uint32_t lo = (__popc(k & n) & 1) ? 0xBC00u : 0x3C00u;
  const uint32_t hi = (__popc((k + 1) & n) & 1) ? 0xBC00u : 0x3C00u;
  return lo | (hi << 16);
}

template <int J>
__global__ void __launch_bounds__(32 * kWalshWarps, 1)
hadq_walsh_kernel(const WalshParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int warp_global = blockIdx.x * kWalshWarps + (threadIdx.x >> 5);
  const int warps_total = gridDim.x * kWalshWarps;
  const int g = lane >> 2, t = lane & 3;
  const bool mma_stage = (p.stage_mask & 0x1Bu) == 0x1Bu;     // bits 0, 1, 3, 4 (always all four or none)
  // B fragments of the two column halves of H16: column n = 8 nh + g, rows k = 2t, 2t+1 and 2t+8, 2t+9.
  // The contraction index is k = (bit 0, bits 3..4, bit 1) of the element index = (k0, t, k3).
  uint32_t bf[2][2];
#pragma unroll
  for (int nh = 0; nh < 2; ++nh) {
    // output column n = (n0 = c & 1, n1..n2 = t', n3 = nh); as a B fragment the lane holds column n = 8 nh + g
    bf[nh][0] = h16_pair(2 * t, 8 * nh + g);
    bf[nh][1] = h16_pair(2 * t + 8, 8 * nh + g);
  }
  // per-lane signs of the three shuffle stages: the lane with the bit set computes partner - own
  const float sg[3] = {(lane & 4) ? -1.0f : 1.0f, (lane & 8) ? -1.0f : 1.0f, (lane & 16) ? -1.0f : 1.0f};

  for (int64_t row = warp_global; row < p.rows; row += warps_total) {
    const uint4* xr = reinterpret_cast<const uint4*>(p.x + row * p.ldx);
    uint4 raw[J];
#pragma unroll
    for (int j = 0; j < J; ++j) raw[j] = __ldg(xr + lane + 32 * j);
    float v[J][8];
#pragma unroll
    for (int j = 0; j < J; ++j) {
      if (mma_stage) {
        // A fragment: (a0, a1, a2, a3) = words (0, 2, 1, 3) of the chunk; D of column half nh holds the elements with
        // bit 1 = nh: c0, c1 = elements (2 nh, 2 nh + 1), c2, c3 = elements (4 + 2 nh, 5 + 2 nh)
        float d0[4], d1[4];
        mma_f16_16816(d0, raw[j].x, raw[j].z, raw[j].y, raw[j].w, bf[0][0], bf[0][1]);
        mma_f16_16816(d1, raw[j].x, raw[j].z, raw[j].y, raw[j].w, bf[1][0], bf[1][1]);
        v[j][0] = d0[0]; v[j][1] = d0[1]; v[j][2] = d1[0]; v[j][3] = d1[1];
        v[j][4] = d0[2]; v[j][5] = d0[3]; v[j][6] = d1[2]; v[j][7] = d1[3];
      } else {
        const __half2* h = reinterpret_cast<const __half2*>(&raw[j]);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __half22float2(h[e]);
          v[j][2 * e] = f.x; v[j][2 * e + 1] = f.y;
        }
      }
    }
    // bit 2: elements e and e + 4 of a chunk
    if (p.stage_mask & 4u) {
#pragma unroll
      for (int j = 0; j < J; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float a = v[j][e], b = v[j][e + 4];
          v[j][e] = a + b; v[j][e + 4] = a - b;
        }
    }
    // bits 8 ..: chunks j and j + h of the lane
#pragma unroll
    for (int h = 1; h < J; h <<= 1) {
      if (p.stage_mask & (256u * h)) {
#pragma unroll
        for (int j = 0; j < J; ++j) {
          if ((j & h) == 0) {
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              const float a = v[j][e], b = v[j + h][e];
              v[j][e] = a + b; v[j + h][e] = a - b;
            }
          }
        }
      }
    }
    // bits 5, 6, 7: lanes l and l ^ 4, l ^ 8, l ^ 16
#pragma unroll
    for (int s = 0; s < 3; ++s) {
      if (p.stage_mask & (32u << s)) {
#pragma unroll
        for (int j = 0; j < J; ++j)
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float o = __shfl_xor_sync(0xffffffffu, v[j][e], 4 << s);
            v[j][e] = fmaf(v[j][e], sg[s], o);
          }
      }
    }
    // scale, round to fp16, absmax
    uint4 hq[J];
    __half2 mx = __float2half2_rn(0.0f);
#pragma unroll
    for (int j = 0; j < J; ++j) {
      __half2* hh = reinterpret_cast<__half2*>(&hq[j]);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        hh[e] = __floats2half2_rn(v[j][2 * e] * p.scale, v[j][2 * e + 1] * p.scale);
        mx = __hmax2(mx, __habs2(hh[e]));
      }
    }
    if (p.y_out) {
      uint4* yo = reinterpret_cast<uint4*>(p.y_out + row * p.ldy);
#pragma unroll
      for (int j = 0; j < J; ++j) yo[lane + 32 * j] = hq[j];
    }
    if (p.do_quant) {
      const float2 mf = __half22float2(mx);
      float amax = fmaxf(mf.x, mf.y);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      const __half s7 = __float2half_rn(__fdiv_rn(amax, 7.0f));
      const __half sh = __float2half_rn(__half2float(s7) * p.clip);
      const float s = __half2float(sh);
      if (lane == 0) p.scales[row] = sh;
      const float rcp = (s != 0.0f) ? __frcp_rn(s) : 0.0f;
      const bool noclamp = clamp_free(s, p.clip);
      uint32_t* qo = reinterpret_cast<uint32_t*>(p.q + row * (int64_t)(p.n >> 1));
#pragma unroll
      for (int j = 0; j < J; ++j) qo[lane + 32 * j] = quant8_words(hq[j].x, hq[j].y, hq[j].z, hq[j].w, s, rcp, noclamp);
    }
  }
}

template <int J>
static int launch_walsh_j(const WalshParams& p, cudaStream_t st) {
  int64_t grid = (p.rows + kWalshWarps - 1) / kWalshWarps;
  const int64_t cap = (int64_t)num_sms();
  if (grid > cap) grid = cap;
  QR_CUDA(launch_kernel(hadq_walsh_kernel<J>, dim3((unsigned)grid), dim3(32 * kWalshWarps), 0, st, use_pdl(p.rows), p));
  return QR_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// The heads-axis transform by itself: y[h'][d] = sum_h (-1)^popcount(h & h') x[h][d] / sqrt(H) for every column d of a
// [H, D] row.  Columns are independent, so a thread takes two neighbouring columns (one half2 per head: the lanes of
// a warp read 128 contiguous bytes of every head) through all H heads in registers: H loads in flight per thread,
// log2(H) butterfly stages in fp32, one rounding, H stores; no shuffles, no shared memory.  The warp-per-row kernel
// above spends 128 shuffles per lane on the same rows of 32 x 128 (16.1 us for 2048 rows against 8 us here).
struct HeadsParams {
  const __half* x;
  __half* y;
  int64_t rows;
  int D;            // head_dim (a power of two >= 32)
  int dshift;       // log2(D / 2): column pairs per row
  float scale;
};

template <int H>
__global__ void __launch_bounds__(256)
hadq_heads_kernel(const HeadsParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t row = gid >> p.dshift;
  if (row >= p.rows) return;
  const int dp = (int)(gid & ((1 << p.dshift) - 1));
  const size_t base = (size_t)row * H * p.D + 2 * dp;
  uint32_t w[H];
#pragma unroll
  for (int h = 0; h < H; ++h) w[h] = __ldg(reinterpret_cast<const uint32_t*>(p.x + base + (size_t)h * p.D));
  float a[H], b[H];
#pragma unroll
  for (int h = 0; h < H; ++h) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[h]));
    a[h] = f.x; b[h] = f.y;
  }
#pragma unroll
  for (int s = 1; s < H; s <<= 1) {
#pragma unroll
    for (int h = 0; h < H; ++h) {
      if ((h & s) == 0) {
        const float a0 = a[h], a1 = a[h + s], b0 = b[h], b1 = b[h + s];
        a[h] = a0 + a1; a[h + s] = a0 - a1;
        b[h] = b0 + b1; b[h + s] = b0 - b1;
      }
    }
  }
#pragma unroll
  for (int h = 0; h < H; ++h) {
    const __half2 o = __floats2half2_rn(a[h] * p.scale, b[h] * p.scale);
    *reinterpret_cast<uint32_t*>(p.y + base + (size_t)h * p.D) = *reinterpret_cast<const uint32_t*>(&o);
  }
}

template <int H>
static int launch_heads_h(const HeadsParams& p, cudaStream_t st) {
  const int64_t threads = p.rows << p.dshift;
  QR_CUDA(launch_kernel(hadq_heads_kernel<H>, dim3((unsigned)((threads + 255) / 256)), dim3(256), 0, st, use_pdl(p.rows), p));
  return QR_OK;
}

// Heads-axis transform of [rows, H, D] (contiguous, 4-byte aligned); QR_EUNSUPPORTED for head counts this kernel is
// not compiled for (the caller then takes the masked warp-per-row kernel).
int launch_hadq_heads(const void* x, void* y, int64_t rows, int heads, int head_dim, cudaStream_t st) {
  if (head_dim < 32 || (head_dim & (head_dim - 1)) != 0 || rows * (int64_t)head_dim > (int64_t)1 << 40) return QR_EUNSUPPORTED;
  HeadsParams p;
  p.x = reinterpret_cast<const __half*>(x); p.y = reinterpret_cast<__half*>(y); p.rows = rows; p.D = head_dim;
  p.dshift = 0;
  while ((2 << p.dshift) < head_dim) ++p.dshift;
  p.scale = (float)(1.0 / sqrt((double)heads));
  switch (heads) {
    case 8: return launch_heads_h<8>(p, st);
    case 16: return launch_heads_h<16>(p, st);
    case 32: return launch_heads_h<32>(p, st);
    default: return QR_EUNSUPPORTED;
  }
}

// Walsh transform of rows of n = 256 .. 4096 elements (a power of two) over the index bits in stage_mask, with or
// without the quantiser behind it.  Returns QR_EUNSUPPORTED when the shape is outside what the kernel covers.
int launch_hadq_walsh(const void* x, int64_t rows, int n, int64_t ldx, uint32_t stage_mask, float scale, float clip,
                      uint8_t* q, void* scales, void* y_out, int64_t ldy, int do_quant, cudaStream_t st) {
  if (n < 256 || n > 4096 || (n & (n - 1)) != 0) return QR_EUNSUPPORTED;
  if (!aligned16(x) || ldx % 8 != 0 || (y_out && (!aligned16(y_out) || ldy % 8 != 0)) || (do_quant && !aligned16(q)))
    return QR_EUNSUPPORTED;
  const uint32_t low = stage_mask & 0x1Bu;
  if (low != 0 && low != 0x1Bu) return QR_EUNSUPPORTED;     // bits 0, 1, 3, 4 go through one MMA: all or none
  WalshParams p;
  p.x = reinterpret_cast<const __half*>(x); p.ldx = ldx; p.rows = rows; p.n = n; p.stage_mask = stage_mask;
  p.scale = scale; p.clip = clip; p.q = q; p.scales = reinterpret_cast<__half*>(scales);
  p.y_out = reinterpret_cast<__half*>(y_out); p.ldy = ldy; p.do_quant = do_quant;
  switch (n >> 8) {
    case 1: return launch_walsh_j<1>(p, st);
    case 2: return launch_walsh_j<2>(p, st);
    case 4: return launch_walsh_j<4>(p, st);
    case 8: return launch_walsh_j<8>(p, st);
    default: return launch_walsh_j<16>(p, st);
  }
}

}  // namespace qr
