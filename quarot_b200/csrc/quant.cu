// Standalone quantise-and-pack (caller-provided scales) and int32 -> fp16 dequantise.
// Both are pure streaming kernels: one 16-byte load -> one 4-byte store (quant),
// one 16-byte load -> one 8-byte store (dequant).
#include "common.cuh"

namespace qr {

// Eight fp16 values (one uint4) -> four packed bytes (caller-provided scale: always clamped).
__device__ __forceinline__ uint32_t quant8(const uint4& v, float s, float rcp) {
  return quant8_words(v.x, v.y, v.z, v.w, s, rcp, false);
}

__global__ void __launch_bounds__(256)
sym_quant_vec_kernel(const __half* __restrict__ x, const __half* __restrict__ scale,
                     int64_t rows, int64_t cols, uint8_t* __restrict__ q) {
  // cols % 8 == 0: every thread owns 8 consecutive elements of one row
  const int64_t vec_per_row = cols >> 3;
  const int64_t total = rows * vec_per_row;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / vec_per_row;
    const float s = __half2float(scale[row]);
    uint4 v = *reinterpret_cast<const uint4*>(x + i * 8);
    *reinterpret_cast<uint32_t*>(q + i * 4) = quant8(v, s, s != 0.0f ? __frcp_rn(s) : 0.0f);
  }
}

__global__ void __launch_bounds__(256)
sym_quant_scalar_kernel(const __half* __restrict__ x, const __half* __restrict__ scale,
                        int64_t rows, int64_t cols, int64_t cols_dst, uint8_t* __restrict__ q) {
  // any cols (also odd): one thread per output byte
  const int64_t total = rows * cols_dst;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / cols_dst;
    const int64_t c = (i - row * cols_dst) * 2;
    const float s = __half2float(scale[row]);
    const float a = __half2float(x[row * cols + c]);
    const float b = (c + 1 < cols) ? __half2float(x[row * cols + c + 1]) : 0.0f;
    uint32_t code;
    if (s != 0.0f) {
      const float rcp = __frcp_rn(s);
      code = quant_pair(div_by_scale(a, s, rcp), div_by_scale(b, s, rcp));
    } else {
      code = quant_pair_zero_scale(a, b);
    }
    q[i] = (uint8_t)((code & 0xF) | ((code >> 12) & 0xF0));
  }
}

// out = (s_row * s_col) * half(q), every product rounded to fp16, in that order.
__global__ void __launch_bounds__(256)
sym_dequant_vec_kernel(const int32_t* __restrict__ q, const __half* __restrict__ srow,
                       const __half* __restrict__ scol, int64_t rows, int64_t cols,
                       __half* __restrict__ out) {
  const int64_t vec_per_row = cols >> 2;
  const int64_t total = rows * vec_per_row;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / vec_per_row;
    const int64_t c = (i - row * vec_per_row) * 4;
    const int4 v = *reinterpret_cast<const int4*>(q + row * cols + c);
    const __half sr = srow[row];
    const __half2 sc01 = *reinterpret_cast<const __half2*>(scol + c);
    const __half2 sc23 = *reinterpret_cast<const __half2*>(scol + c + 2);
    __half2 r01 = __hmul2(__hmul2(__half2half2(sr), sc01),
                          __halves2half2(__int2half_rn(v.x), __int2half_rn(v.y)));
    __half2 r23 = __hmul2(__hmul2(__half2half2(sr), sc23),
                          __halves2half2(__int2half_rn(v.z), __int2half_rn(v.w)));
    uint2 o;
    o.x = *reinterpret_cast<uint32_t*>(&r01);
    o.y = *reinterpret_cast<uint32_t*>(&r23);
    *reinterpret_cast<uint2*>(out + row * cols + c) = o;
  }
}

__global__ void __launch_bounds__(256)
sym_dequant_scalar_kernel(const int32_t* __restrict__ q, const __half* __restrict__ srow,
                          const __half* __restrict__ scol, int64_t rows, int64_t cols,
                          __half* __restrict__ out) {
  const int64_t total = rows * cols;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / cols;
    const int64_t c = i - row * cols;
    out[i] = __hmul(__hmul(srow[row], scol[c]), __int2half_rn(q[i]));
  }
}

static int grid_for(int64_t total_threads) {
  int64_t blocks = (total_threads + 255) / 256;
  int64_t cap = (int64_t)num_sms() * 16;
  if (blocks < 1) blocks = 1;
  return (int)(blocks < cap ? blocks : cap);
}

// Self-test of the division shortcut: for every finite fp16 value x and every finite non-zero fp16 scale s,
// the int4 code obtained from x * RN(1/s) must equal the one obtained from IEEE division.
__device__ unsigned long long g_div_mismatch = 0;

__global__ void __launch_bounds__(256)
division_check_kernel(unsigned long long* mismatch) {
  // blockIdx.x enumerates the scale bit patterns 0x0001 .. 0x7BFF (positive; the sign of s only flips the quotient)
  const uint32_t sbits = blockIdx.x + 1;
  const __half sh = __ushort_as_half((unsigned short)sbits);
  const float s = __half2float(sh);
  const float rcp = __frcp_rn(s);
  unsigned int bad = 0;
  for (uint32_t xb = threadIdx.x; xb < 65536u; xb += blockDim.x) {
    if ((xb & 0x7C00u) == 0x7C00u) continue;   // inf / NaN inputs are outside the contract
    const float x = __half2float(__ushort_as_half((unsigned short)xb));
    const uint32_t fast = quant_pair(x * rcp, -x * rcp);
    const uint32_t ieee = quant_pair(__fdiv_rn(x, s), __fdiv_rn(-x, s));
    bad += (fast != ieee);
    // the unclamped form is used when |x / s| <= 7.004
    if (fabsf(__fdiv_rn(x, s)) <= 7.25f) {
      const __half2 xx = __halves2half2(__ushort_as_half((unsigned short)xb), __ushort_as_half((unsigned short)(xb ^ 0x8000u)));
      const uint32_t u = quant2_word<false>(*reinterpret_cast<const uint32_t*>(&xx), rcp);
      const uint32_t codes = (u & 0xFu) | ((u >> 12) & 0xF0u);
      bad += (codes != ((ieee & 0xFu) | ((ieee >> 12) & 0xF0u)));
    }
  }
  if (bad) atomicAdd(mismatch, (unsigned long long)bad);
}

}  // namespace qr

extern "C" {

int qr_sym_quant_i4(const void* x, const void* scale, int64_t rows, int64_t cols,
                    uint8_t* q, void* stream) {
  if (rows < 0 || cols < 0) return qr::fail(QR_EINVAL, "qr_sym_quant_i4: negative size");
  if (rows == 0 || cols == 0) return QR_OK;
  if (!x || !scale || !q) return qr::fail(QR_EINVAL, "qr_sym_quant_i4: null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  if ((cols & 7) == 0 && qr::aligned16(x) && ((uintptr_t)q & 3) == 0) {
    qr::sym_quant_vec_kernel<<<qr::grid_for(rows * (cols >> 3)), 256, 0, st>>>(
        (const __half*)x, (const __half*)scale, rows, cols, q);
  } else {
    const int64_t cd = (cols + 1) / 2;
    qr::sym_quant_scalar_kernel<<<qr::grid_for(rows * cd), 256, 0, st>>>(
        (const __half*)x, (const __half*)scale, rows, cols, cd, q);
  }
  QR_LAUNCH_CHECK("qr_sym_quant_i4");
  return QR_OK;
}

int qr_sym_dequant_i32_f16(const int32_t* q, const void* scale_row, const void* scale_col,
                           int64_t rows, int64_t cols, void* out, void* stream) {
  if (rows < 0 || cols < 0) return qr::fail(QR_EINVAL, "qr_sym_dequant_i32_f16: negative size");
  if (rows == 0 || cols == 0) return QR_OK;
  if (!q || !scale_row || !scale_col || !out)
    return qr::fail(QR_EINVAL, "qr_sym_dequant_i32_f16: null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  if ((cols & 3) == 0 && qr::aligned16(q) && ((uintptr_t)out & 7) == 0 && ((uintptr_t)scale_col & 3) == 0) {
    qr::sym_dequant_vec_kernel<<<qr::grid_for(rows * (cols >> 2)), 256, 0, st>>>(
        q, (const __half*)scale_row, (const __half*)scale_col, rows, cols, (__half*)out);
  } else {
    qr::sym_dequant_scalar_kernel<<<qr::grid_for(rows * cols), 256, 0, st>>>(
        q, (const __half*)scale_row, (const __half*)scale_col, rows, cols, (__half*)out);
  }
  QR_LAUNCH_CHECK("qr_sym_dequant_i32_f16");
  return QR_OK;
}

int qr_debug_division_check(uint64_t* mismatches_out) {
  if (!mismatches_out) return qr::fail(QR_EINVAL, "qr_debug_division_check: null output");
  unsigned long long* dptr = nullptr;
  QR_CUDA(cudaGetSymbolAddress((void**)&dptr, qr::g_div_mismatch));
  QR_CUDA(cudaMemset(dptr, 0, sizeof(unsigned long long)));
  qr::division_check_kernel<<<0x7BFF, 256>>>(dptr);
  QR_LAUNCH_CHECK("division_check_kernel");
  QR_CUDA(cudaDeviceSynchronize());
  unsigned long long v = 0;
  QR_CUDA(cudaMemcpy(&v, dptr, sizeof(v), cudaMemcpyDeviceToHost));
  *mismatches_out = (uint64_t)v;
  return QR_OK;
}

}  // extern "C"
