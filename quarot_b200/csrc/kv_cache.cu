// Paged 4-bit KV cache: quantise-and-append and single-token (decode) attention.
//
// Layout (the one the upstream cache defines): pages [num_pages, layers, 2 (k | v), heads, page_size, head_dim / 2]
// uint8 -- element 2j in the low nibble of byte j, unsigned codes 0..15 -- and parameters
// [num_pages, layers, 2, heads, page_size, 2] fp16 = (scale, zero); value = code * scale - zero.  Sequence b owns the
// pages kv_indices[kv_indptr[b] .. kv_indptr[b + 1]), the last of which holds last_page_offset[b] tokens.
//
// kv_append_kernel: one warp per (new token, head).  The lane holds four of the 128 values of the head: optional
// Walsh-Hadamard transform of the key over the head dimension (two butterfly stages in registers, five warp-shuffle
// stages, fp32, scale 1/sqrt(128), rounded to fp16), min / max by shuffles, the asymmetric quantiser in the fp16
// step-by-step arithmetic of the torch reference, two packed bytes per lane straight into the page slot, and the
// (scale, zero) pair.  Upstream runs a Hadamard kernel, about ten elementwise torch kernels and a copy kernel.
//
// kv_decode_kernel: one CTA per (sequence, head), eight warps taking chunks of 32 cached tokens.  Scores: lane =
// token, the 64-byte key row against the query in shared memory, dequantisation folded into the dot product
// (scale * <q, codes> - zero * sum(q)).  Online softmax per warp in base 2.  Values: the lane that scored a token
// also brings its 64-byte value row in (16-byte loads, requested with the key) and parks it in shared memory;
// then lane = four head dimensions, two bytes and one broadcast of p * scale per token, the zero points summed
// separately.  The eight partial states are merged
// through shared memory.  The query's Hadamard transform, which upstream applies with a separate kernel, runs at
// the start of the same kernel.
#include "common.cuh"

#include <math.h>

namespace qr {

constexpr int kHeadDim = 128;

struct KvAppendParams {
  uint8_t* data;
  __half2* param;
  const int32_t* indptr;
  const int32_t* indices;
  const int32_t* last_page_offset;
  const __half* k;              // [tokens, heads, 128]
  const __half* v;
  const int32_t* append_indptr; // [batch + 1], or null: one token per sequence
  int batch, layers, layer, heads, page_size, tokens;
  int hadamard_k;
};

// Walsh-Hadamard transform of 128 values held four per lane (element index = 4 lane + e), unscaled.
__device__ __forceinline__ void fwht128_warp(float (&x)[4], int lane) {
  {
    const float a = x[0] + x[1], b = x[0] - x[1], c = x[2] + x[3], d = x[2] - x[3];
    x[0] = a + c; x[1] = b + d; x[2] = a - c; x[3] = b - d;
  }
#pragma unroll
  for (int s = 1; s < 32; s <<= 1) {
    const float sg = (lane & s) ? -1.0f : 1.0f;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float o = __shfl_xor_sync(0xffffffffu, x[e], s);
      x[e] = fmaf(x[e], sg, o);
    }
  }
}

__device__ __forceinline__ void load4_f16(const __half* p, float (&x)[4]) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&u.x));
  const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
  x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y;
}

// Asymmetric int4 codes of one (token, head) row, four values per lane, with the fp16 arithmetic of the reference:
//   scale = fp16(max(fp16(max - min), 1e-5) / 15), zero = -min, code = clamp(rint(fp16(fp16(x + zero) / scale)), 0, 15).
__device__ __forceinline__ uint32_t asym_quant4(const __half (&h)[4], __half2* param_out, int lane) {
  float mx = fmaxf(fmaxf(__half2float(h[0]), __half2float(h[1])), fmaxf(__half2float(h[2]), __half2float(h[3])));
  float mn = fminf(fminf(__half2float(h[0]), __half2float(h[1])), fminf(__half2float(h[2]), __half2float(h[3])));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
  }
  __half range = __float2half_rn(mx - mn);
  if (__half2float(range) < 1e-5f) range = __float2half_rn(1e-5f);
  const __half scale = __float2half_rn(__fdiv_rn(__half2float(range), 15.0f));
  const __half zero = __float2half_rn(-mn);
  const float sf = __half2float(scale), zf = __half2float(zero);
  uint32_t codes = 0;
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const __half a = __float2half_rn(__half2float(h[e]) + zf);
    const __half t = __float2half_rn(__fdiv_rn(__half2float(a), sf));
    float r = rintf(__half2float(t));
    r = fminf(fmaxf(r, 0.0f), 15.0f);
    codes |= (uint32_t)r << (4 * e);
  }
  if (lane == 0) *param_out = __halves2half2(scale, zero);
  return codes;      // 16 bits: element e in bits [4e, 4e + 4)
}

__global__ void __launch_bounds__(256)
kv_append_kernel(const KvAppendParams p) {
  const int lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= (long long)p.tokens * p.heads) return;
  const int tok = (int)(item / p.heads), head = (int)(item % p.heads);
  int b = tok, j = 0, append_len = 1;
  if (p.append_indptr) {
    int lo = 0, hi = p.batch;                // largest b with append_indptr[b] <= tok
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (p.append_indptr[mid] <= tok) lo = mid; else hi = mid;
    }
    b = lo;
    j = tok - p.append_indptr[b];
    append_len = p.append_indptr[b + 1] - p.append_indptr[b];
  }
  // the page table already describes the sequence WITH the appended tokens
  const int first = p.indptr[b];
  const long long seq_len = (long long)(p.indptr[b + 1] - first - 1) * p.page_size + p.last_page_offset[b];
  const long long pos = seq_len - append_len + j;
  if (pos < 0) return;
  const long long page = p.indices[first + (int)(pos / p.page_size)];
  const int slot = (int)(pos % p.page_size);
  const size_t src = ((size_t)tok * p.heads + head) * kHeadDim + 4 * lane;
#pragma unroll
  for (int which = 0; which < 2; ++which) {
    float x[4];
    load4_f16((which == 0 ? p.k : p.v) + src, x);
    __half h[4];
    if (which == 0 && p.hadamard_k) {
      fwht128_warp(x, lane);
#pragma unroll
      for (int e = 0; e < 4; ++e) h[e] = __float2half_rn(x[e] * 0.08838834764831845f);    // 1 / sqrt(128)
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) h[e] = __float2half_rn(x[e]);
    }
    const size_t row = ((((size_t)page * p.layers + p.layer) * 2 + which) * p.heads + head) * p.page_size + slot;
    const uint32_t codes = asym_quant4(h, p.param + row, lane);
    *reinterpret_cast<uint16_t*>(p.data + row * (kHeadDim / 2) + 2 * lane) = (uint16_t)codes;
  }
}

struct KvDecodeParams {
  __half* o;                    // [batch, heads, 128]
  const __half* q;
  const uint8_t* data;
  const __half2* param;
  const int32_t* indptr;
  const int32_t* indices;
  const int32_t* last_page_offset;
  int batch, layers, layer, heads, page_size;
  int hadamard_q;
  int splits;                   // CTAs (one cluster) that share the tokens of a (sequence, head): 1, 2, 4 or 8
};

constexpr int kKvDecWarps = 8;

__device__ __forceinline__ uint32_t kv_cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void kv_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// a float of CTA `rank` of the cluster at the same shared-memory address as `local` here
__device__ __forceinline__ float kv_peer_float(const float* local, uint32_t rank) {
  uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(local)), peer;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(peer) : "r"(addr), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(peer) : "memory");
  return v;
}

// Codes as floats without a conversion instruction (those issue at a quarter of the rate of ordinary arithmetic) and
// without a subtraction: a code c moved to bits 3 .. 6 of a byte, with that byte permuted into bits 16 .. 23 of
// 0x41000000, is the float 8 + c / 2 exactly.  Sums of w * (8 + c / 2) are turned back into sums of w * c once per
// row (2 * sum - 16 * sum of w); the bias is of the size of the data, so fp32 loses a bit or two, not the result.
// `bytes` holds four codes, each already shifted to bits 3 .. 6 of its byte; k selects the byte.
template <int k>
__device__ __forceinline__ float code_to_biased_float(uint32_t bytes) {
  return __uint_as_float(__byte_perm(bytes, 0x41000000u, 0x7044 + (k << 8)));
}

__global__ void __launch_bounds__(32 * kKvDecWarps)
kv_decode_kernel(const KvDecodeParams p) {
  __shared__ __align__(16) float s_q[kHeadDim];
  __shared__ float s_qsum;
  __shared__ float s_m[kKvDecWarps], s_l[kKvDecWarps];
  __shared__ __align__(16) float s_o[kKvDecWarps][kHeadDim];
  __shared__ float s_part[2 + kHeadDim];          // this CTA's share when a cluster splits the sequence: m, l, o[128]
  // value codes of a warp's 32 tokens: lane = token brings its row in with 16-byte loads, lane = head dimensions reads
  // two bytes per token from here (rows padded to 80 bytes: the 16-byte stores of a quarter-warp hit different banks)
  __shared__ __align__(16) unsigned char s_v[kKvDecWarps][32][80];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int item = blockIdx.x / p.splits;
  const int b = item / p.heads, head = item % p.heads;
  const uint32_t crank = p.splits > 1 ? kv_cluster_rank() : 0u;
  const int first = p.indptr[b];
  const long long seq_len = (long long)(p.indptr[b + 1] - first - 1) * p.page_size + p.last_page_offset[b];

  if (warp == 0) {
    float x[4];
    load4_f16(p.q + ((size_t)b * p.heads + head) * kHeadDim + 4 * lane, x);
    if (p.hadamard_q) {
      fwht128_warp(x, lane);
      // the transformed query is an fp16 tensor upstream
#pragma unroll
      for (int e = 0; e < 4; ++e) x[e] = __half2float(__float2half_rn(x[e] * 0.08838834764831845f));
    }
    float sum = x[0] + x[1] + x[2] + x[3];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    *reinterpret_cast<float4*>(s_q + 4 * lane) = make_float4(x[0], x[1], x[2], x[3]);
    if (lane == 0) s_qsum = sum;
  }
  __syncthreads();
  const float qsum = s_qsum;
  const float sm_scale = 0.08838834764831845f * 1.4426950408889634f;   // log2(e) / sqrt(128)

  float m = -INFINITY, l = 0.0f, zacc = 0.0f, wsum = 0.0f;
  float o[4] = {0.0f, 0.0f, 0.0f, 0.0f};       // sums of w * (8 + c / 2); wsum: the sum of the weights w = p * scale
  const size_t rows_per_page_kv = (size_t)p.heads * p.page_size;      // rows between the k and the v block of a page
  // the CTAs of a cluster take contiguous ranges of whole 32-token chunks
  const long long chunks = (seq_len + 31) >> 5;
  const long long per = ((chunks + p.splits - 1) / p.splits) << 5;
  const long long tok_begin = (long long)crank * per;
  const long long tok_end = (tok_begin + per < seq_len) ? tok_begin + per : seq_len;
  for (long long base = tok_begin + (long long)warp * 32; base < tok_end; base += 32 * kKvDecWarps) {
    const long long t = base + lane;
    const bool valid = t < tok_end;
    float score = -INFINITY, vs = 0.0f, vz = 0.0f;
    if (valid) {
      const long long page = p.indices[first + (int)(t / p.page_size)];
      const int slot = (int)(t % p.page_size);
      const size_t krow = ((((size_t)page * p.layers + p.layer) * 2) * p.heads + head) * p.page_size + slot;
      const uint4* kp = reinterpret_cast<const uint4*>(p.data + krow * (kHeadDim / 2));
      const uint4* vp = reinterpret_cast<const uint4*>(p.data + (krow + rows_per_page_kv) * (kHeadDim / 2));
      uint4 kw[4], vw[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) kw[c] = __ldg(kp + c);
#pragma unroll
      for (int c = 0; c < 4; ++c) vw[c] = __ldg(vp + c);      // requested with the keys, used after the scores
      const float2 kpar = __half22float2(p.param[krow]);
      const float2 vpar = __half22float2(p.param[krow + rows_per_page_kv]);
      float dot = 0.0f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const uint32_t ww[4] = {kw[c].x, kw[c].y, kw[c].z, kw[c].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          // word i of chunk c holds elements 32 c + 8 i .. + 7, element e in bits [4e, 4e + 4)
          const float4 q0 = *reinterpret_cast<const float4*>(s_q + 32 * c + 8 * i);
          const float4 q1 = *reinterpret_cast<const float4*>(s_q + 32 * c + 8 * i + 4);
          // even elements are the low nibbles of the four bytes, odd elements the high nibbles
          const uint32_t ev = (ww[i] << 3) & 0x78787878u, od = (ww[i] >> 1) & 0x78787878u;
          dot = fmaf(q0.x, code_to_biased_float<0>(ev), dot);
          dot = fmaf(q0.y, code_to_biased_float<0>(od), dot);
          dot = fmaf(q0.z, code_to_biased_float<1>(ev), dot);
          dot = fmaf(q0.w, code_to_biased_float<1>(od), dot);
          dot = fmaf(q1.x, code_to_biased_float<2>(ev), dot);
          dot = fmaf(q1.y, code_to_biased_float<2>(od), dot);
          dot = fmaf(q1.z, code_to_biased_float<3>(ev), dot);
          dot = fmaf(q1.w, code_to_biased_float<3>(od), dot);
        }
      }
      dot = 2.0f * dot - 16.0f * qsum;            // sum of q * (8 + c / 2) -> sum of q * c
      score = (kpar.x * dot - kpar.y * qsum) * sm_scale;
      vs = vpar.x; vz = vpar.y;
#pragma unroll
      for (int c = 0; c < 4; ++c) *reinterpret_cast<uint4*>(&s_v[warp][lane][16 * c]) = vw[c];
    }
    float cmax = score;
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) cmax = fmaxf(cmax, __shfl_xor_sync(0xffffffffu, cmax, s));
    const float m_new = fmaxf(m, cmax);
    const float corr = exp2f(m - m_new);            // 0 on the first chunk (m = -inf)
    const float pr = valid ? exp2f(score - m_new) : 0.0f;
    float psum = pr, pz = pr * vz;
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
      psum += __shfl_xor_sync(0xffffffffu, psum, s);
      pz += __shfl_xor_sync(0xffffffffu, pz, s);
    }
    l = l * corr + psum;
    zacc = zacc * corr + pz;
    wsum *= corr;
#pragma unroll
    for (int e = 0; e < 4; ++e) o[e] *= corr;
    m = m_new;
    // values: lane = head dimensions 4 lane .. 4 lane + 3; token tt of the chunk broadcasts p * scale, its codes come
    // from the warp's staging rows (the shuffles above have ordered the stores of all lanes before these loads)
    const float ps = pr * vs;
    const int ntok = (int)((tok_end - base) < 32 ? (tok_end - base) : 32);
    __syncwarp();
#pragma unroll 8
    for (int tt = 0; tt < ntok; ++tt) {
      const float wv = __shfl_sync(0xffffffffu, ps, tt);
      const uint32_t cv = *reinterpret_cast<const uint16_t*>(&s_v[warp][tt][2 * lane]);
      const uint32_t ev = (cv << 3) & 0x7878u, od = (cv >> 1) & 0x7878u;
      wsum += wv;
      o[0] = fmaf(wv, code_to_biased_float<0>(ev), o[0]);
      o[1] = fmaf(wv, code_to_biased_float<0>(od), o[1]);
      o[2] = fmaf(wv, code_to_biased_float<1>(ev), o[2]);
      o[3] = fmaf(wv, code_to_biased_float<1>(od), o[3]);
    }
    __syncwarp();      // the staging rows are rewritten by the next chunk
  }
  // back from w * (8 + c / 2) to w * c; the zero points are the same for every head dimension
#pragma unroll
  for (int e = 0; e < 4; ++e) o[e] = 2.0f * o[e] - 16.0f * wsum - zacc;
  if (lane == 0) { s_m[warp] = m; s_l[warp] = l; }
  *reinterpret_cast<float4*>(&s_o[warp][4 * lane]) = make_float4(o[0], o[1], o[2], o[3]);
  __syncthreads();
  if (warp == 0) {
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < kKvDecWarps; ++w) mm = fmaxf(mm, s_m[w]);
    float ll = 0.0f, acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int w = 0; w < kKvDecWarps; ++w) {
      const float f = (s_m[w] == -INFINITY) ? 0.0f : exp2f(s_m[w] - mm);
      ll += s_l[w] * f;
      const float4 v = *reinterpret_cast<const float4*>(&s_o[w][4 * lane]);
      acc[0] = fmaf(v.x, f, acc[0]); acc[1] = fmaf(v.y, f, acc[1]); acc[2] = fmaf(v.z, f, acc[2]); acc[3] = fmaf(v.w, f, acc[3]);
    }
    if (p.splits > 1) {
      // publish this CTA's share; the first CTA of the cluster merges them below
      if (lane == 0) { s_part[0] = mm; s_part[1] = ll; }
      s_part[2 + 4 * lane + 0] = acc[0]; s_part[2 + 4 * lane + 1] = acc[1];
      s_part[2 + 4 * lane + 2] = acc[2]; s_part[2 + 4 * lane + 3] = acc[3];
    }
    if (p.splits == 1) {
    const float inv = ll > 0.0f ? 1.0f / ll : 0.0f;       // an empty sequence gives zeros
    const __half2 h0 = __floats2half2_rn(acc[0] * inv, acc[1] * inv);
    const __half2 h1 = __floats2half2_rn(acc[2] * inv, acc[3] * inv);
    uint2 out;
    out.x = *reinterpret_cast<const uint32_t*>(&h0);
    out.y = *reinterpret_cast<const uint32_t*>(&h1);
    *reinterpret_cast<uint2*>(p.o + ((size_t)b * p.heads + head) * kHeadDim + 4 * lane) = out;
    }
  }
  if (p.splits > 1) {
    kv_cluster_sync();                        // every share of the cluster is in shared memory
    if (crank == 0 && warp == 0) {
      float mm = -INFINITY;
      for (int r = 0; r < p.splits; ++r) mm = fmaxf(mm, kv_peer_float(&s_part[0], (uint32_t)r));
      float ll = 0.0f, acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      for (int r = 0; r < p.splits; ++r) {
        const float mr = kv_peer_float(&s_part[0], (uint32_t)r);
        const float f = (mr == -INFINITY) ? 0.0f : exp2f(mr - mm);
        ll += kv_peer_float(&s_part[1], (uint32_t)r) * f;
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[e] = fmaf(kv_peer_float(&s_part[2 + 4 * lane + e], (uint32_t)r), f, acc[e]);
      }
      const float inv = ll > 0.0f ? 1.0f / ll : 0.0f;       // an empty sequence gives zeros
      const __half2 h0 = __floats2half2_rn(acc[0] * inv, acc[1] * inv);
      const __half2 h1 = __floats2half2_rn(acc[2] * inv, acc[3] * inv);
      uint2 out;
      out.x = *reinterpret_cast<const uint32_t*>(&h0);
      out.y = *reinterpret_cast<const uint32_t*>(&h1);
      *reinterpret_cast<uint2*>(p.o + ((size_t)b * p.heads + head) * kHeadDim + 4 * lane) = out;
    }
    kv_cluster_sync();                        // nobody leaves while its shared memory may still be read
  }
}

}  // namespace qr

extern "C" {

int qr_kv_append_i4(void* kv_data, void* kv_param, const int32_t* kv_indptr, const int32_t* kv_indices,
                    const int32_t* last_page_offset, const void* k, const void* v, const int32_t* append_indptr,
                    int64_t tokens, int batch, int num_layers, int layer, int num_heads, int page_size, int head_dim,
                    int hadamard_k, void* stream) {
  if (tokens < 0 || batch < 0) return qr::fail(QR_EINVAL, "qr_kv_append_i4: negative size");
  if (tokens == 0 || batch == 0) return QR_OK;
  if (!kv_data || !kv_param || !kv_indptr || !kv_indices || !last_page_offset || !k || !v)
    return qr::fail(QR_EINVAL, "qr_kv_append_i4: null pointer");
  if (head_dim != qr::kHeadDim) return qr::fail(QR_EUNSUPPORTED, "qr_kv_append_i4: head_dim = %d (only 128, as upstream)", head_dim);
  if (num_layers < 1 || layer < 0 || layer >= num_layers || num_heads < 1 || page_size < 1)
    return qr::fail(QR_EINVAL, "qr_kv_append_i4: bad layer / heads / page size");
  if (!append_indptr && tokens != batch) return qr::fail(QR_EINVAL, "qr_kv_append_i4: without append_indptr every sequence appends one token");
  if (tokens * num_heads > (1ll << 40)) return qr::fail(QR_EUNSUPPORTED, "qr_kv_append_i4: too many tokens");
  if (((uintptr_t)k & 7) || ((uintptr_t)v & 7) || ((uintptr_t)kv_data & 1) || ((uintptr_t)kv_param & 3))
    return qr::fail(QR_EALIGN, "qr_kv_append_i4: k and v must be 8-byte aligned");
  qr::KvAppendParams p;
  p.data = reinterpret_cast<uint8_t*>(kv_data); p.param = reinterpret_cast<__half2*>(kv_param);
  p.indptr = kv_indptr; p.indices = kv_indices; p.last_page_offset = last_page_offset;
  p.k = reinterpret_cast<const __half*>(k); p.v = reinterpret_cast<const __half*>(v); p.append_indptr = append_indptr;
  p.batch = batch; p.layers = num_layers; p.layer = layer; p.heads = num_heads; p.page_size = page_size;
  p.tokens = (int)tokens; p.hadamard_k = hadamard_k;
  const long long items = tokens * num_heads;
  const unsigned grid = (unsigned)((items + 7) / 8);
  qr::kv_append_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(p);
  QR_LAUNCH_CHECK("kv_append_kernel");
  return QR_OK;
}

int qr_kv_decode_i4(void* o, const void* q, const void* kv_data, const void* kv_param, const int32_t* kv_indptr,
                    const int32_t* kv_indices, const int32_t* last_page_offset, int batch, int num_layers, int layer,
                    int num_heads, int page_size, int head_dim, int hadamard_q, void* stream) {
  if (batch < 0) return qr::fail(QR_EINVAL, "qr_kv_decode_i4: negative size");
  if (batch == 0) return QR_OK;
  if (!o || !q || !kv_data || !kv_param || !kv_indptr || !kv_indices || !last_page_offset)
    return qr::fail(QR_EINVAL, "qr_kv_decode_i4: null pointer");
  if (head_dim != qr::kHeadDim) return qr::fail(QR_EUNSUPPORTED, "qr_kv_decode_i4: head_dim = %d (only 128, as upstream)", head_dim);
  if (num_layers < 1 || layer < 0 || layer >= num_layers || num_heads < 1 || page_size < 1)
    return qr::fail(QR_EINVAL, "qr_kv_decode_i4: bad layer / heads / page size");
  if (((uintptr_t)q & 7) || ((uintptr_t)o & 7) || ((uintptr_t)kv_data & 15) || ((uintptr_t)kv_param & 3))
    return qr::fail(QR_EALIGN, "qr_kv_decode_i4: q and o must be 8-byte aligned, the pages 16-byte aligned");
  qr::KvDecodeParams p;
  p.o = reinterpret_cast<__half*>(o); p.q = reinterpret_cast<const __half*>(q);
  p.data = reinterpret_cast<const uint8_t*>(kv_data); p.param = reinterpret_cast<const __half2*>(kv_param);
  p.indptr = kv_indptr; p.indices = kv_indices; p.last_page_offset = last_page_offset;
  p.batch = batch; p.layers = num_layers; p.layer = layer; p.heads = num_heads; p.page_size = page_size;
  p.hadamard_q = hadamard_q;
  // few (sequence, head) pairs: a cluster of 2, 4 or 8 CTAs shares the tokens of each, so that about three CTAs per SM
  // have work; their shares are merged through distributed shared memory
  const long long items = (long long)batch * num_heads;
  int splits = 1;
  while (splits < 8 && items * splits * 2 <= 3ll * qr::num_sms()) splits *= 2;
  p.splits = splits;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)splits;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.gridDim = dim3((unsigned)(items * splits));
  cfg.blockDim = dim3(32 * qr::kKvDecWarps);
  cfg.stream = (cudaStream_t)stream;
  cfg.attrs = attr;
  cfg.numAttrs = splits > 1 ? 1 : 0;
  QR_CUDA(cudaLaunchKernelEx(&cfg, qr::kv_decode_kernel, p));
  return QR_OK;
}

}  // extern "C"
