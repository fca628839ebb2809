// Kernel (b) at decode sizes (at most 64 token rows): a weight-streaming form of the tcgen05 int4 GEMM.
//
// With few token rows the linear layer is one pass over the N x K/2 weight bytes; what matters is that every SM
// streams its share of those bytes at memory speed.  Three things differ from the prefill kernels:
//   * Weights on the 128 MMA rows, tokens on the BN = 16 / 32 / 64 MMA columns.  The tensor core fetches its
//     operands from shared memory at about 64 bytes per cycle, (128 + BN) x 32 bytes per k-step of 32, whether or
//     not all 128 rows carry weights.
//   * Deep stages.  The pipeline TMA -> widen int4 to int8 -> tcgen05.mma has a latency of several hundred cycles
//     per stage, so a stage carries KB = 2 .. 8 k-blocks of 128 values: 16 KB and more of packed weights.
//   * All SMs busy for any N, by one of two decompositions (one CTA per SM):
//       - row split, for wide layers (more than 48 weight rows per SM): the weight rows are dealt out evenly in blocks of
//         `tile_rows` <= 96 rows (84 for N = 12288 on 148 SMs, 2 x 75 for N = 22016) and every CTA runs its blocks
//         over the whole K -- a contiguous piece of the weight matrix per SM, no partial sums, no scratch memory.
//         The MMA's operand window reads past the block into whatever follows in shared memory; the accumulator
//         rows beyond the block are never read;
//       - unit split, for narrow layers (N = 4096: 28 rows per SM would waste most of every MMA): full tiles of 128
//         rows, and the flat list of (tile, stage) units is cut into one contiguous range per CTA.  A range may
//         begin or end inside a tile; the int32 partial sums of such a piece are added into a scratch tile with
//         red.global.add (integer addition: exact and order independent), and the piece that arrives last at the
//         tile's counter reads the total, applies the epilogue and leaves scratch tile and counter at zero.
//         Nobody waits for anybody.  Without scratch memory narrow layers take the row split as well.
// The token rows (a few KB per stage, from L2) ride along in the same stages.  The weights do not depend on the
// kernel in front, so the producer requests the first ring-ful of weight tiles before the programmatic-dependency
// wait; the token tiles follow after it.
// Widening, descriptors, accumulator scaling (x 256, folded away in the epilogue) and the epilogue arithmetic are
// those of gemm_i4.cu: the results are bit-identical to every other form of kernel (b).
//
// Every mbarrier wait is bounded; on a timeout the CTA raises the device status word, every role leaves its loop,
// the CTA idles until copies and MMAs in flight have landed, frees its tensor memory and returns.
#include "tc_ptx.cuh"

#include <mutex>

namespace qr {

struct DecodeParams {
  int N, M, K;              // weight rows (output channels), token rows, K values
  int tile_rows;            // weight rows per tile (128 under the unit split)
  int tiles;                // ceil(N / tile_rows)
  int stages_per_tile;      // ceil(K / (128 KB))
  int whole_tiles;          // 1: row split, ranges are cut at tile boundaries; 0: unit split with scratch memory
  void* out;                // [M, N] fp16 or int32, row pitch ldo
  int64_t ldo;
  const __half* sW;         // [N] weight scales, or null (int32 mode)
  const __half* sX;         // [M] token scales, or null
  const __half* bias;       // [N] or null
  int* ws_counter;          // [tiles] arrival counters, zero before and after every launch
  int32_t* ws_acc;          // [tiles][BN][128] int32 sums of partial tiles, zero before and after every launch
  int* status;
};

constexpr int kDecBM = 128;                 // rows of the MMA
constexpr int kDecEpiWarps = 4;
constexpr int kDecWidenWarps = 8;
constexpr int kDecThreads = 32 * (2 + kDecEpiWarps + kDecWidenWarps);
enum { DEC_I32 = 0, DEC_F16 = 1 };

// RP: weight rows a stage has room for (tile_rows <= RP <= 128)
template <int BN, int RP, int KB, int PST, int IST>
struct DecodeSmem {
  static constexpr int kPkRow = KB * 64;                          // packed bytes per row per stage
  static constexpr int kPkStage = (RP + BN) * kPkRow;             // weight rows, then token rows
  static constexpr int kSub = (RP + BN) * 128;                    // int8 bytes of one k-block: weight rows, then token rows
  static constexpr int kI8Stage = KB * kSub;
  static constexpr int kI8Off = 0;
  static constexpr int kI8Pad = (kDecBM - RP) * 128;              // the MMA's 128-row window of the last k-block ends in here
  static constexpr int kPkOff = IST * kI8Stage + kI8Pad;
  static constexpr int kBarOff = kPkOff + PST * kPkStage;
  static constexpr int kNumBars = 2 * PST + 2 * IST + 4;
  static constexpr int kTmemSlotOff = kBarOff + kNumBars * 8;
  static constexpr int kAbortOff = kTmemSlotOff + 8;
  static constexpr int kTotal = kAbortOff + 16;                   // abort flag, last-arriver flag
  static constexpr int kDynamic = kTotal + 1024;                  // slack for manual 1024-byte alignment
  static_assert(BN % 8 == 0 && RP % 8 == 0 && RP <= kDecBM, "operand blocks start on a swizzle-atom boundary");
};

// The flat list of (tile, stage) units is cut into gridDim.x contiguous ranges; a range is walked as segments, a
// segment being the stages [st0, st1) of one tile.  Every role of the CTA walks the same segments.
struct DecodeWalk {
  long long u, u_end;
  int spt;
  __device__ DecodeWalk(const DecodeParams& p) : spt(p.stages_per_tile) {
    if (p.whole_tiles) {
      u = ((long long)blockIdx.x * p.tiles / gridDim.x) * spt;
      u_end = ((long long)(blockIdx.x + 1) * p.tiles / gridDim.x) * spt;
    } else {
      const long long total = (long long)p.tiles * spt;
      u = (long long)blockIdx.x * total / gridDim.x;
      u_end = (long long)(blockIdx.x + 1) * total / gridDim.x;
    }
  }
  __device__ bool next(int& tile, int& st0, int& st1) {
    if (u >= u_end) return false;
    tile = (int)(u / spt);
    st0 = (int)(u - (long long)tile * spt);
    const long long left = u_end - u;
    st1 = (left < (long long)(spt - st0)) ? st0 + (int)left : spt;
    u += st1 - st0;
    return true;
  }
};

template <int BN, int RP, int KB, int PST, int IST, int MODE>
__global__ void __launch_bounds__(kDecThreads, 1)
gemm_i4_decode_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, const DecodeParams p) {
  using L = DecodeSmem<BN, RP, KB, PST, IST>;
  pdl_launch_dependents();   // the next kernel of the stream may be brought up; it waits for this grid to finish
  extern __shared__ unsigned char smem_dyn[];
  const uint32_t smem_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  unsigned char* smem_gen = smem_dyn + (smem_base - smem_u32(smem_dyn));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const uint32_t bar_base = smem_base + L::kBarOff;
  auto full_p = [&](int s) { return bar_base + 8u * s; };
  auto empty_p = [&](int s) { return bar_base + 8u * (PST + s); };
  auto full_i = [&](int s) { return bar_base + 8u * (2 * PST + s); };
  auto empty_i = [&](int s) { return bar_base + 8u * (2 * PST + IST + s); };
  auto acc_full = [&](int a) { return bar_base + 8u * (2 * PST + 2 * IST + a); };
  auto acc_empty = [&](int a) { return bar_base + 8u * (2 * PST + 2 * IST + 2 + a); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + L::kTmemSlotOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + L::kAbortOff);
  volatile int* last_flag = reinterpret_cast<volatile int*>(smem_gen + L::kAbortOff + 4);
  constexpr uint32_t kTmemCols = (2 * BN) < 32 ? 32 : (2 * BN);

  if (threadIdx.x == 0) {
    for (int s = 0; s < PST; ++s) { mbar_init(full_p(s), 1); mbar_init(empty_p(s), kDecWidenWarps); }
    for (int s = 0; s < IST; ++s) { mbar_init(full_i(s), kDecWidenWarps); mbar_init(empty_i(s), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(acc_full(a), 1); mbar_init(acc_empty(a), kDecEpiWarps); }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_base + L::kTmemSlotOff, kTmemCols);
    tmem_relinquish();
  }
  if (threadIdx.x == 32) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmW) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmX) : "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t kStageTx = (uint32_t)((p.tile_rows + BN) * L::kPkRow);

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      // weights first: nothing in front of this kernel writes them
      uint32_t pre = 0;
      {
        DecodeWalk w(p);
        int tile, st0, st1;
        while (pre < (uint32_t)PST && w.next(tile, st0, st1)) {
          for (int st = st0; st < st1 && pre < (uint32_t)PST; ++st, ++pre) {
            mbar_expect_tx(full_p(pre), kStageTx);
            tma_load_2d(smem_base + L::kPkOff + pre * L::kPkStage, &tmW, full_p(pre), st * (L::kPkRow / 4), tile * p.tile_rows);
          }
        }
      }
      pdl_wait();   // the token rows come from the preceding kernel
      uint32_t it = 0;
      bool ok = true;
      DecodeWalk w(p);
      int tile, st0, st1;
      while (ok && w.next(tile, st0, st1)) {
        for (int st = st0; st < st1; ++st, ++it) {
          const int s = it % PST;
          const uint32_t dst = smem_base + L::kPkOff + s * L::kPkStage;
          if (it >= pre) {
            if (!mbar_wait(empty_p(s), ((it / PST) & 1) ^ 1, abort_flag, p.status, 51)) { ok = false; break; }
            mbar_expect_tx(full_p(s), kStageTx);
            tma_load_2d(dst, &tmW, full_p(s), st * (L::kPkRow / 4), tile * p.tile_rows);
          }
          tma_load_2d(dst + RP * L::kPkRow, &tmX, full_p(s), st * (L::kPkRow / 4), 0);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_i8(kDecBM, BN);
      uint32_t it = 0, sg = 0;
      bool ok = true;
      DecodeWalk w(p);
      int tile, st0, st1;
      while (ok && w.next(tile, st0, st1)) {
        const int a = sg & 1;
        if (!mbar_wait(acc_empty(a), ((sg >> 1) & 1) ^ 1, abort_flag, p.status, 52)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + a * BN;
        for (int st = st0; st < st1; ++st, ++it) {
          const int s = it % IST;
          if (!mbar_wait(full_i(s), (it / IST) & 1, abort_flag, p.status, 53)) { ok = false; break; }
          tc_fence_after();
          uint32_t a_lo = desc_lo(smem_base + L::kI8Off + s * L::kI8Stage);
#pragma unroll
          for (int j = 0; j < KB; ++j, a_lo += (L::kSub >> 4)) {
            const uint32_t b_lo = a_lo + ((RP * 128) >> 4);
#pragma unroll
            for (int k4 = 0; k4 < 4; ++k4) {
              // +32 bytes along K inside the swizzle atom = +2 in the (addr >> 4) field
              const uint64_t da = ((uint64_t)kDescHiKmajorSw128 << 32) | (uint64_t)(a_lo + 2 * k4);
              const uint64_t db = ((uint64_t)kDescHiKmajorSw128 << 32) | (uint64_t)(b_lo + 2 * k4);
              umma_i8(d_tmem, da, db, idesc, (st != st0 || j != 0 || k4 != 0) ? 1u : 0u);
            }
          }
          umma_commit(empty_i(s));
        }
        if (ok) umma_commit(acc_full(a));
        ++sg;
      }
    }
  } else if (warp < 2 + kDecEpiWarps) {
    // ------------------------------------------------------------ epilogue: thread = one output channel of the tile
    const int q4 = warp & 3;                 // tensor-memory lane quarter this warp may access
    const int row_in_tile = q4 * 32 + lane;
    const bool first_epi_thread = (threadIdx.x == 32 * 2);
    auto epi_sync = [&]() { asm volatile("bar.sync 1, %0;" ::"n"(32 * kDecEpiWarps) : "memory"); };
    pdl_wait();   // scales, scratch and the output belong to the preceding kernels
    uint32_t sg = 0;
    bool ok = true;
    DecodeWalk w(p);
    int tile, st0, st1;
    while (ok && w.next(tile, st0, st1)) {
      const int a = sg & 1;
      if (!mbar_wait(acc_full(a), (sg >> 1) & 1, abort_flag, p.status, 54)) { ok = false; break; }
      ++sg;
      tc_fence_after();
      int acc[BN];
#pragma unroll
      for (int c0 = 0; c0 < BN; c0 += 16) {
        uint32_t r[32];
        tmem_ld16(tmem_base + ((uint32_t)(q4 * 32) << 16) + (uint32_t)(a * BN + c0), r);
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[c0 + j] = (int)r[j];
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty(a));
      const int n = tile * p.tile_rows + row_in_tile;
      bool finish = (st0 == 0 && st1 == w.spt);       // the whole tile in one piece: no scratch involved
      if (!finish) {
        // a piece of the tile: add it into the scratch tile; whoever arrives last at the counter finishes the tile
        int32_t* wacc = p.ws_acc + (size_t)tile * BN * kDecBM + row_in_tile;      // [column][row]: coalesced per column
#pragma unroll
        for (int j = 0; j < BN; ++j)
          if (j < p.M) atomicAdd(wacc + j * kDecBM, acc[j]);
        __threadfence();
        epi_sync();
        if (first_epi_thread) {
          // number of CTAs whose range touches this tile: owner(u) = ceil((u + 1) G / U) - 1
          const long long total = (long long)p.tiles * w.spt;
          const long long ua = (long long)tile * w.spt, ub = ua + w.spt - 1;
          const int oa = (int)(((ua + 1) * gridDim.x + total - 1) / total) - 1;
          const int ob = (int)(((ub + 1) * gridDim.x + total - 1) / total) - 1;
          *last_flag = (atomicAdd(p.ws_counter + tile, 1) == ob - oa) ? 1 : 0;
        }
        epi_sync();
        finish = (*last_flag != 0);
        if (finish) {
          __threadfence();
#pragma unroll
          for (int j = 0; j < BN; ++j)
            if (j < p.M) {
              acc[j] = __ldcg(wacc + j * kDecBM);
              wacc[j * kDecBM] = 0;
            }
          if (first_epi_thread) p.ws_counter[tile] = 0;
        }
        epi_sync();      // last_flag is rewritten by the next piece
      }
      if (finish && row_in_tile < p.tile_rows && n < p.N) {
        float sw = 0.0f;
        __half bv = __float2half(0.0f);
        if (MODE == DEC_F16) {
          sw = __half2float(p.sW[n]);
          if (p.bias) bv = p.bias[n];
        }
#pragma unroll
        for (int j = 0; j < BN; ++j) {
          if (j < p.M) {
            const int v = acc[j] >> 8;       // the widened operands carry a factor 16 each
            if (MODE == DEC_I32) {
              reinterpret_cast<int32_t*>(p.out)[(int64_t)j * p.ldo + n] = v;
            } else {
              __half h = __float2half_rn((float)v * (__half2float(__ldg(p.sX + j)) * sw));
              if (p.bias) h = __hadd(h, bv);
              reinterpret_cast<__half*>(p.out)[(int64_t)j * p.ldo + n] = h;
            }
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------ widen int4 -> int8
    // Chunk c of a stage: row = c / (4 KB), k-block j = (c / 4) % KB, 16-byte piece cc = c % 4 of that row's 64 packed
    // bytes of k-block j.  Consecutive threads read consecutive 16-byte chunks (conflict free) and write two chunks of
    // the 128-byte-swizzled int8 row.
    const int wt = threadIdx.x - 32 * (2 + kDecEpiWarps);
    constexpr int kWThreads = 32 * kDecWidenWarps;
    constexpr int kRowChunks = 4 * KB;
    const int w_chunks = p.tile_rows * kRowChunks;
    const int chunks = w_chunks + BN * kRowChunks;
    const int x_shift = (RP - p.tile_rows) * kRowChunks;       // the token rows start at row RP of a stage
    uint32_t it = 0;
    bool ok = true;
    DecodeWalk w(p);
    int tile, st0, st1;
    while (ok && w.next(tile, st0, st1)) {
      for (int st = st0; st < st1; ++st, ++it) {
        const int sp_ = it % PST, si = it % IST;
        if (!mbar_wait(full_p(sp_), (it / PST) & 1, abort_flag, p.status, 55)) { ok = false; break; }
        if (!mbar_wait(empty_i(si), ((it / IST) & 1) ^ 1, abort_flag, p.status, 56)) { ok = false; break; }
        tc_fence_after();
        const unsigned char* pk = smem_gen + L::kPkOff + sp_ * L::kPkStage;
        unsigned char* i8 = smem_gen + L::kI8Off + si * L::kI8Stage;
#pragma unroll 4
        for (int c0 = wt; c0 < chunks; c0 += kWThreads) {
          const int c = c0 < w_chunks ? c0 : c0 + x_shift;
          const int row = c / kRowChunks, rem = c % kRowChunks;
          const int j = rem >> 2, cc = rem & 3;
          const uint4 q = *reinterpret_cast<const uint4*>(pk + (size_t)c * 16);
          uint4 lo, hi;
          lo.x = (q.x << 4) & 0xF0F0F0F0u; hi.x = q.x & 0xF0F0F0F0u;
          lo.y = (q.y << 4) & 0xF0F0F0F0u; hi.y = q.y & 0xF0F0F0F0u;
          lo.z = (q.z << 4) & 0xF0F0F0F0u; hi.z = q.z & 0xF0F0F0F0u;
          lo.w = (q.w << 4) & 0xF0F0F0F0u; hi.w = q.w & 0xF0F0F0F0u;
          unsigned char* drow = i8 + j * L::kSub + row * 128;
          const int sw = row & 7;
          *reinterpret_cast<uint4*>(drow + (((2 * cc) ^ sw) << 4)) = lo;
          *reinterpret_cast<uint4*>(drow + (((2 * cc + 1) ^ sw) << 4)) = hi;
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(full_i(si));
          mbar_arrive(empty_p(sp_));
        }
      }
    }
  }

  // ---------------------------------------------------------------- teardown
  drain_after_abort(abort_flag);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ------------------------------------------------------------------ host
typedef CUresult (*EncodeTiledFnDec)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                     const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                     CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFnDec decode_encode_fn() {
  static EncodeTiledFnDec fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFnDec>(ptr);
  });
  return fn;
}

// Tensor map over a packed int4 matrix [rows, kbytes] seen as 32-bit words:
// box = [box_bytes / 4 words, box_rows], no swizzle, out-of-range words read as zero.
static int make_words_map(CUtensorMap* map, const void* base, int64_t rows, int64_t kbytes, int box_rows, int box_bytes) {
  EncodeTiledFnDec fn = decode_encode_fn();
  if (!fn) return fail(QR_ENOTREADY, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[2] = {(cuuint64_t)(kbytes / 4), (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)kbytes};
  cuuint32_t box[2] = {(cuuint32_t)(box_bytes / 4), (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(QR_EINVAL, "cuTensorMapEncodeTiled (decode) failed with CUresult %d", (int)r);
  return QR_OK;
}

constexpr size_t kDecCounterRegion = 64u << 10;    // scratch: arrival counters in front (fixed size), sums behind
constexpr int kDecUnitKB = 2;                      // k-blocks per stage under the unit split

static int decode_bn(int64_t M) { return M <= 16 ? 16 : (M <= 32 ? 32 : 64); }

// Narrow layers (at most 48 weight rows per SM) take the unit split when scratch memory is there.
static bool decode_is_narrow(int64_t N, int sms) { return (N + sms - 1) / sms <= 48; }

// Scratch bytes the unit split wants for a decode-sized call (0: the shape takes the row split or another kernel).
size_t decode_stream_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  if (M < 1 || M > 64 || N < 1 || K < 256 || K % 32 != 0 || !decode_is_narrow(N, num_sms())) return 0;
  // up to K = 8192 dealing out the weight rows is as fast or faster (64 rows, N = 4096: 14.2 against 18.1 us at
  // K = 4096, 26.7 against 23.2 us at K = 11008)
  if (g_tuning.gemm_splitk == 0 || (g_tuning.gemm_splitk == 1 && K <= 8192)) return 0;
  const size_t tiles = (size_t)((N + kDecBM - 1) / kDecBM);
  if (tiles * 4 > kDecCounterRegion) return 0;
  return kDecCounterRegion + tiles * (size_t)decode_bn(M) * kDecBM * 4;
}

template <int BN, int RP, int KB, int PST, int IST, int MODE>
static int launch_decode_cfg(const uint8_t* W, const uint8_t* X, DecodeParams& p, int sms, cudaStream_t st) {
  using L = DecodeSmem<BN, RP, KB, PST, IST>;
  static_assert(L::kDynamic <= 227 * 1024, "shared memory budget exceeded");
  CUtensorMap tmW, tmX;
  int rc;
  if ((rc = make_words_map(&tmW, W, p.N, p.K / 2, p.tile_rows, L::kPkRow))) return rc;
  if ((rc = make_words_map(&tmX, X, p.M, p.K / 2, BN, L::kPkRow))) return rc;
  p.stages_per_tile = (p.K + 128 * KB - 1) / (128 * KB);
  const long long units = p.whole_tiles ? p.tiles : (long long)p.tiles * p.stages_per_tile;
  const int grid = (int)(units < sms ? units : sms);
  auto kern = gemm_i4_decode_kernel<BN, RP, KB, PST, IST, MODE>;
  static thread_local bool configured[64] = {false};
  int dev = 0;
  QR_CUDA(cudaGetDevice(&dev));
  if (dev >= 64 || !configured[dev]) {
    QR_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic));
    if (dev < 64) configured[dev] = true;
  }
  QR_CUDA(launch_kernel(kern, dim3((unsigned)grid), dim3(kDecThreads), (size_t)L::kDynamic, st, use_pdl(p.M), tmW, tmX, p));
  return QR_OK;
}

template <int MODE>
static int launch_decode_mode(const uint8_t* W, const uint8_t* X, DecodeParams& p, int bn, int sms, cudaStream_t st) {
  if (!p.whole_tiles) {      // unit split: full tiles, two k-blocks per stage
    if (bn == 16) return launch_decode_cfg<16, 128, kDecUnitKB, 4, 3, MODE>(W, X, p, sms, st);
    if (bn == 32) return launch_decode_cfg<32, 128, kDecUnitKB, 4, 3, MODE>(W, X, p, sms, st);
    return launch_decode_cfg<64, 128, kDecUnitKB, 3, 2, MODE>(W, X, p, sms, st);
  }
  if (bn == 16) {
    if (p.tile_rows <= 32) return launch_decode_cfg<16, 32, 8, 4, 2, MODE>(W, X, p, sms, st);
    return launch_decode_cfg<16, 96, 4, 3, 2, MODE>(W, X, p, sms, st);
  }
  if (bn == 32) return launch_decode_cfg<32, 96, 2, 4, 3, MODE>(W, X, p, sms, st);
  return launch_decode_cfg<64, 96, 2, 4, 3, MODE>(W, X, p, sms, st);
}

// out[M, N] = X[M, K] . W[N, K]^T for at most 64 token rows.  `ws` (optional) is zeroed scratch of at least
// decode_stream_workspace_bytes(M, N, K) bytes, 256-byte aligned; it is used by narrow layers only.
// Returns QR_EUNSUPPORTED when the shape is outside what this kernel serves (the caller then takes another path).
int launch_gemm_i4_decode(const uint8_t* X, const uint8_t* W, int64_t M, int64_t N, int64_t K, void* out, int64_t ldo,
                          const void* sX, const void* sW, const void* bias, bool f16, int grid_cap, void* ws, size_t ws_bytes,
                          cudaStream_t st) {
  if (M < 1 || M > 64 || N < 1 || N > (1 << 30) || K < 1024 || K % 32 != 0 || K > 131071) return QR_EUNSUPPORTED;
  if (!aligned16(X) || !aligned16(W)) return QR_EUNSUPPORTED;
  int* status = kernel_status_ptr();
  if (!status) return fail(QR_ENOTREADY, "decode GEMM: no CUDA device");
  int sms = num_sms();
  if (grid_cap > 0 && sms > grid_cap) sms = grid_cap;
  DecodeParams p;
  p.N = (int)N; p.M = (int)M; p.K = (int)K; p.out = out; p.ldo = ldo; p.status = status;
  p.sW = reinterpret_cast<const __half*>(sW); p.sX = reinterpret_cast<const __half*>(sX);
  p.bias = reinterpret_cast<const __half*>(bias);
  p.whole_tiles = 1; p.ws_counter = nullptr; p.ws_acc = nullptr; p.stages_per_tile = 0;
  const size_t need = decode_stream_workspace_bytes(M, N, K);
  if (ws && need > 0 && g_tuning.gemm_splitk != 0) {
    if (ws_bytes < need) return fail(QR_EINVAL, "decode GEMM: workspace of %zu bytes is too small, %zu needed", ws_bytes, need);
    if (((uintptr_t)ws & 255) != 0) return fail(QR_EALIGN, "decode GEMM: workspace must be 256-byte aligned");
    p.whole_tiles = 0;
    p.ws_counter = reinterpret_cast<int*>(ws);
    p.ws_acc = reinterpret_cast<int32_t*>(reinterpret_cast<unsigned char*>(ws) + kDecCounterRegion);
    p.tile_rows = kDecBM;
  } else {
    // weight rows per CTA, dealt out evenly in blocks of at most 96 rows
    const int64_t per_cta = (N + sms - 1) / sms;
    const int64_t tiles_per_cta = (per_cta + 95) / 96;
    p.tile_rows = (int)((N + sms * tiles_per_cta - 1) / (sms * tiles_per_cta));
  }
  p.tiles = (int)((N + p.tile_rows - 1) / p.tile_rows);
  const int bn = decode_bn(M);
  return f16 ? launch_decode_mode<DEC_F16>(W, X, p, bn, sms, st) : launch_decode_mode<DEC_I32>(W, X, p, bn, sms, st);
}

}  // namespace qr
