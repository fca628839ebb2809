// Kernel family (b): INT4 x INT4 -> INT32 GEMM on the 5th-generation tensor cores
// (tcgen05.mma kind::i8, accumulators in tensor memory), with the per-token x
// per-channel dequantisation fused into the epilogue.
//
//   D[p, q] = sum_k  P[p, k] * Q[q, k]        P: [rowsP, K/2]  Q: [rowsQ, K/2]  int4 packed
//
// Both operands are K-major packed nibbles in global memory.  tcgen05 has no
// 4-bit integer kind, so nibbles are widened to int8 in shared memory:
//   * TMA (cp.async.bulk.tensor.2d) brings [rows x 64 B] packed tiles (128 K values
//     per row) into a staging ring,
//   * eight "widen" warps turn every 32-bit word w into  (w << 4) & 0xF0F0F0F0  (the
//     four even elements) and  w & 0xF0F0F0F0  (the four odd elements): each nibble
//     lands in the HIGH half of an int8, i.e. the value times 16 with the sign for
//     free.  The accumulator is therefore exactly 256x the true dot product and the
//     epilogue shifts it right by 8.  |acc| <= 64*K*256 < 2^31 for K <= 131071.
//     Even/odd elements are written to separate 16-byte chunks: a fixed permutation of
//     K applied to both operands alike, which leaves the dot product unchanged,
//   * the int8 tiles use the canonical K-major 128-byte-swizzle layout (rows of 128 B,
//     16-byte chunk index XOR (row & 7)), are published to the async proxy with
//     fence.proxy.async and consumed by one thread issuing
//     tcgen05.mma.cta_group::1.kind::i8 (M = 128, N = BN, K = 32 per instruction),
//   * four epilogue warps read the accumulator with tcgen05.ld (32 lanes x 32 columns
//     per warp), apply >> 8 and either store int32 or the fp16 dequantised value.
// The kernel is persistent (static round-robin tile schedule) and, when ACC == 2,
// double-buffers the accumulator so the epilogue of tile i overlaps the main loop
// of tile i+1.
//
// Decode-sized M (at most 64 token rows) is served by gemm_i4_decode.cu (weights on the MMA rows,
// all SMs streaming) and, for a handful of rows, by gemv_i4.cu.
//
// Every mbarrier wait is bounded: after about two seconds of polling the waiting thread
// raises a CTA-wide abort flag and the device status word, every role leaves its
// loop, tensor memory is released and the kernel returns.
#include "tc_ptx.cuh"

#include <map>
#include <mutex>
#include <tuple>

namespace qr {

// ------------------------------------------------------------------ kernel
enum { MODE_I32 = 0, MODE_F16 = 1 };

struct GemmParams {
  int rowsP, rowsQ;      // valid rows of each operand
  int K;                 // K elements (int4 values)
  int tilesP, tilesQ;
  void* out;             // int32 or fp16
  int64_t ldo;           // elements
  const __half* sP;      // per-row scale of operand P (fp16) or null (MODE_I32)
  const __half* sQ;
  const __half* bias;    // per output channel or null
  int vec_ok;            // output rows, scales and bias are 16-byte aligned: vector epilogue allowed
  int swiglu;            // 2-CTA kernel, fp16 mode: columns [0,128) / [128,256) of a tile are gate / up channels; out = silu(gate) * up
  int bn;                // 2-CTA kernel: N of the pair tile (a multiple of 16, at most 256); 256 unless fp16 mode with one output
  int n_outs;            // 2-CTA kernel: number of output matrices that receive the result (1, or one per GPU of a column split)
  int tail_help;         // 2-CTA kernel: warps that have run out of work share the epilogue of the CTA's last tile
  int tma_out;           // 2-CTA kernel: the output has a tensor map (16-byte aligned base and row pitch): tiled stores
  int* status;
};

constexpr int kBM = 128;          // rows of operand P per tile = UMMA M
constexpr int kBKBytes = 64;      // packed bytes per row per stage = 128 K values
constexpr int kWidenWarps = 8;
constexpr int kEpiWarps = 4;
constexpr int kThreads = 32 * (2 + kEpiWarps + kWidenWarps);

template <int BN, int PST, int IST>
struct SmemLayout {
  static constexpr int kI8Stage = (kBM + BN) * 128;
  static constexpr int kPkStage = (kBM + BN) * kBKBytes;
  static constexpr int kI8Off = 0;
  static constexpr int kPkOff = IST * kI8Stage;
  static constexpr int kBarOff = kPkOff + PST * kPkStage;
  static constexpr int kNumBars = 2 * PST + 2 * IST + 4;
  static constexpr int kTmemSlotOff = kBarOff + kNumBars * 8;
  static constexpr int kAbortOff = kTmemSlotOff + 8;
  static constexpr int kTotal = kAbortOff + 8;
  static constexpr int kDynamic = kTotal + 1024;  // slack for manual 1024-byte alignment
};

template <int BN, int PST, int IST, int ACC, int MODE>
__global__ void __launch_bounds__(kThreads, 1)
gemm_i4_kernel(const __grid_constant__ CUtensorMap tmP, const __grid_constant__ CUtensorMap tmQ, const GemmParams p) {
  using L = SmemLayout<BN, PST, IST>;
  pdl_launch_dependents();   // the next kernel of the stream may be brought up; it waits for this grid to finish
  extern __shared__ unsigned char smem_dyn[];
  const uint32_t smem_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  unsigned char* smem_gen = smem_dyn + (smem_base - smem_u32(smem_dyn));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const uint32_t bar_base = smem_base + L::kBarOff;
  auto full_p = [&](int s) { return bar_base + 8u * s; };
  auto empty_p = [&](int s) { return bar_base + 8u * (PST + s); };
  auto full_i = [&](int s) { return bar_base + 8u * (2 * PST + s); };
  auto empty_i = [&](int s) { return bar_base + 8u * (2 * PST + IST + s); };
  auto acc_full = [&](int a) { return bar_base + 8u * (2 * PST + 2 * IST + a); };
  auto acc_empty = [&](int a) { return bar_base + 8u * (2 * PST + 2 * IST + 2 + a); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + L::kTmemSlotOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + L::kAbortOff);

  constexpr uint32_t kTmemCols = (ACC * BN) < 32 ? 32 : (ACC * BN);
  static_assert((kTmemCols & (kTmemCols - 1)) == 0 && kTmemCols <= 512, "TMEM columns must be a power of two <= 512");
  // The widen warps work as two groups that take alternate k-blocks when both rings have an even number of slots:
  // a group then always meets the same slots (those of its parity), one phase after the other, so its parity
  // waits stay unambiguous, and it has two MMA periods for the latency chain wait -> read -> store -> fence -> arrive.
  constexpr int kGroups = (PST % 2 == 0 && IST % 2 == 0) ? 2 : 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < PST; ++s) { mbar_init(full_p(s), 1); mbar_init(empty_p(s), kWidenWarps / kGroups); }
    for (int s = 0; s < IST; ++s) { mbar_init(full_i(s), kWidenWarps / kGroups); mbar_init(empty_i(s), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(acc_full(a), 1); mbar_init(acc_empty(a), kEpiWarps); }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_base + L::kTmemSlotOff, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int num_tiles = p.tilesP * p.tilesQ;
  const int num_kb = (p.K + 127) >> 7;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      pdl_wait();   // operands may come from the preceding kernel
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int tp = tile % p.tilesP, tq = tile / p.tilesP;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % PST;
          const uint32_t ph = (it / PST) & 1;
          if (!mbar_wait(empty_p(s), ph ^ 1, abort_flag, p.status, 1)) { ok = false; break; }
          mbar_expect_tx(full_p(s), L::kPkStage);
          const uint32_t dst = smem_base + L::kPkOff + s * L::kPkStage;
          tma_load_2d(dst, &tmP, full_p(s), kb * kBKBytes, tp * kBM);
          tma_load_2d(dst + kBM * kBKBytes, &tmQ, full_p(s), kb * kBKBytes, tq * BN);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_i8(kBM, BN);
      uint32_t it = 0, tl = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tl) {
        const int a = tl % ACC;
        const uint32_t pha = (tl / ACC) & 1;
        if (!mbar_wait(acc_empty(a), pha ^ 1, abort_flag, p.status, 2)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + a * BN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % IST;
          const uint32_t ph = (it / IST) & 1;
          if (!mbar_wait(full_i(s), ph, abort_flag, p.status, 3)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_base + L::kI8Off + s * L::kI8Stage;
          const uint64_t da = make_kmajor_sw128_desc(a_addr);
          const uint64_t db = make_kmajor_sw128_desc(a_addr + kBM * 128);
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4) {
            // +32 bytes along K inside the swizzle atom = +2 in the (addr >> 4) field
            umma_i8(d_tmem, da + 2 * k4, db + 2 * k4, idesc, (kb != 0 || k4 != 0) ? 1u : 0u);
          }
          umma_commit(empty_i(s));
        }
        if (ok) umma_commit(acc_full(a));
      }
    }
  } else if (warp < 2 + kEpiWarps) {
    // ------------------------------------------------------------ epilogue: thread = one output row (a token)
    const int q4 = warp & 3;                 // TMEM lane quarter this warp may access
    const int prow_in_tile = q4 * 32 + lane; // accumulator row owned by this thread
    pdl_wait();   // scales and output are touched only after the preceding kernel has finished
    uint32_t tl = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tl) {
      const int tp = tile % p.tilesP, tq = tile / p.tilesP;
      const int a = tl % ACC;
      const uint32_t pha = (tl / ACC) & 1;
      if (!mbar_wait(acc_full(a), pha, abort_flag, p.status, 4)) { ok = false; break; }
      tc_fence_after();
      const int prow = tp * kBM + prow_in_tile;
      const bool prow_ok = prow < p.rowsP;
      float sp = 0.0f;
      if (MODE == MODE_F16 && prow_ok) sp = __half2float(p.sP[prow]);
      constexpr int CH = BN >= 32 ? 32 : 16;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += CH) {
        uint32_t r[32];
        const uint32_t taddr = tmem_base + ((uint32_t)(q4 * 32) << 16) + (uint32_t)(a * BN + c0);
        if (CH == 32) tmem_ld32(taddr, r); else tmem_ld16(taddr, r);
        tmem_ld_wait();
        if (c0 + CH >= BN) {
          // accumulator fully read: hand the TMEM buffer back to the MMA warp
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(acc_empty(a));
        }
        const int qcol0 = tq * BN + c0;
        if (!prow_ok) continue;
        if (MODE == MODE_I32) {
          int32_t* o = reinterpret_cast<int32_t*>(p.out) + (int64_t)prow * p.ldo + qcol0;
          if (qcol0 + CH <= p.rowsQ && p.vec_ok) {
#pragma unroll
            for (int j = 0; j < CH; j += 4)
              *reinterpret_cast<int4*>(o + j) = make_int4((int32_t)r[j] >> 8, (int32_t)r[j + 1] >> 8,
                                                          (int32_t)r[j + 2] >> 8, (int32_t)r[j + 3] >> 8);
          } else {
#pragma unroll
            for (int j = 0; j < CH; ++j)
              if (qcol0 + j < p.rowsQ) o[j] = (int32_t)r[j] >> 8;
          }
        } else {
          __half* o = reinterpret_cast<__half*>(p.out) + (int64_t)prow * p.ldo + qcol0;
          const bool full = (qcol0 + CH <= p.rowsQ) && p.vec_ok;
          if (full) {
#pragma unroll
            for (int j = 0; j < CH; j += 8) {
              uint4 pk;
              __half2* h = reinterpret_cast<__half2*>(&pk);
              const uint4 sq = __ldg(reinterpret_cast<const uint4*>(p.sQ + qcol0 + j));
              const __half2* sqh = reinterpret_cast<const __half2*>(&sq);
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float2 sc = __half22float2(sqh[e]);
                const float v0 = (float)((int32_t)r[j + 2 * e] >> 8) * (sp * sc.x);
                const float v1 = (float)((int32_t)r[j + 2 * e + 1] >> 8) * (sp * sc.y);
                h[e] = __floats2half2_rn(v0, v1);
              }
              if (p.bias) {
                const uint4 bb = __ldg(reinterpret_cast<const uint4*>(p.bias + qcol0 + j));
                const __half2* bh = reinterpret_cast<const __half2*>(&bb);
#pragma unroll
                for (int e = 0; e < 4; ++e) h[e] = __hadd2(h[e], bh[e]);
              }
              *reinterpret_cast<uint4*>(o + j) = pk;
            }
          } else {
#pragma unroll
            for (int j = 0; j < CH; ++j) {
              if (qcol0 + j < p.rowsQ) {
                const float sc = __half2float(p.sQ[qcol0 + j]);
                __half v = __float2half_rn((float)((int32_t)r[j] >> 8) * (sp * sc));
                if (p.bias) v = __hadd(v, p.bias[qcol0 + j]);
                o[j] = v;
              }
            }
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------ widen int4 -> int8
    const int wt_all = threadIdx.x - 32 * (2 + kEpiWarps);  // 0 .. 255
    constexpr int kChunks = (kBM + BN) * 4;             // 16-byte packed chunks per stage
    constexpr int kWThreads = 32 * kWidenWarps / kGroups;   // threads of one group
    const int group = wt_all / kWThreads;
    const int wt = wt_all - group * kWThreads;
    uint32_t it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        if ((int)(it % kGroups) != group) continue;
        const int sp_ = it % PST, si = it % IST;
        const uint32_t php = (it / PST) & 1, phi = (it / IST) & 1;
        if (!mbar_wait(full_p(sp_), php, abort_flag, p.status, 5)) { ok = false; break; }
        if (!mbar_wait(empty_i(si), phi ^ 1, abort_flag, p.status, 6)) { ok = false; break; }
        tc_fence_after();
        const unsigned char* pk = smem_gen + L::kPkOff + sp_ * L::kPkStage;
        unsigned char* i8 = smem_gen + L::kI8Off + si * L::kI8Stage;
#pragma unroll
        for (int c = wt; c < kChunks; c += kWThreads) {
          const int row = c >> 2, cc = c & 3;
          const uint4 w = *reinterpret_cast<const uint4*>(pk + c * 16);
          uint4 lo, hi;
          lo.x = (w.x << 4) & 0xF0F0F0F0u; hi.x = w.x & 0xF0F0F0F0u;
          lo.y = (w.y << 4) & 0xF0F0F0F0u; hi.y = w.y & 0xF0F0F0F0u;
          lo.z = (w.z << 4) & 0xF0F0F0F0u; hi.z = w.z & 0xF0F0F0F0u;
          lo.w = (w.w << 4) & 0xF0F0F0F0u; hi.w = w.w & 0xF0F0F0F0u;
          unsigned char* drow = i8 + row * 128;
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

// ------------------------------------------------------------------ 2-CTA kernel (cta_group::2)
// Two CTAs of a cluster share one 256 x 256 output tile.  CTA r loads and widens rows
// [128 r, 128 r + 128) of BOTH operands; the leader CTA (rank 0) issues
// tcgen05.mma.cta_group::2 (M = 256, N = 256), which reads A from each CTA's own shared memory
// and each half of B from the CTA that holds it, so every CTA widens and feeds only half of the
// weight tile.  Accumulator rows 128 r .. 128 r + 127 live in CTA r's tensor memory and are
// drained by that CTA's epilogue warps.
//   full_i  (leader)   <- 4 local + 4 remote widen-warp arrivals (the group that owns the stage)
//   empty_i (each CTA) <- tcgen05.commit from the leader, one commit per CTA
//   acc_full (each CTA) <- tcgen05.commit from the leader, one commit per CTA
//   acc_empty (leader) <- 4 local + 4 remote epilogue-warp arrivals
// TMA loads are CTA-local (no multicast of data); the MMA-completion signal is one commit
// delivered to the same barrier in both CTAs.
constexpr int kBN2 = 256;            // largest N of the pair tile (GemmParams::bn is the one in use); each CTA holds bn / 2 rows of operand Q
constexpr int kMaxOuts = 8;          // output matrices one launch can write (the GPUs of a column split)
struct OutMaps { CUtensorMap m[kMaxOuts]; };
constexpr int kRows2 = kBM + kBN2 / 2;  // operand rows per CTA per stage (128 P + 128 Q)

template <int PST, int IST>
struct SmemLayout2 {
  static constexpr int kI8Stage = kRows2 * 128;
  static constexpr int kPkStage = kRows2 * kBKBytes;
  static constexpr int kI8Off = 0;
  static constexpr int kPkOff = IST * kI8Stage;
  static constexpr int kStageOff = kPkOff + PST * kPkStage;          // per epilogue warp: 32 rows x 128 B of output, 128B-swizzled
  static constexpr int kScaleOff = kStageOff + kEpiWarps * 4096;     // per epilogue warp: the tile's 256 column scales as fp32
  static constexpr int kBiasOff = kScaleOff + kEpiWarps * 1024;      // per epilogue warp: the tile's 256 bias values (fp16)
  static constexpr int kBarOff = kBiasOff + kEpiWarps * 512;
  static constexpr int kNumBars = 2 * PST + 2 * IST + 4 + 4;      // ..., and one "scales staged" barrier per lane quarter
  static constexpr int kTmemSlotOff = kBarOff + kNumBars * 8;
  static constexpr int kAbortOff = kTmemSlotOff + 8;
  static constexpr int kTotal = kAbortOff + 16;   // abort flag, issuer turn, scratch word
  static constexpr int kDynamic = kTotal + 1024;
};

constexpr int kWidenGroups2 = 4;                                  // widen groups of three warps; group g owns staging slot g
constexpr int kWidenWarpsPerGroup2 = 3;
constexpr int kWidenWarps2 = kWidenWarpsPerGroup2 * kWidenGroups2;
// Warp roles.  A warp is served by the warp scheduler (id modulo 4) it was born on, and a scheduler shares its
// issue slots evenly among its ready warps.  The two MMA issuers and the TMA producer are single threads whose
// instruction latency is the critical path of the main loop, so scheduler 1 carries only them (warps 1, 5, 9),
// one epilogue warp (13: the four epilogue warps must cover the four tensor-memory lane quarters, id modulo 4)
// and an idle warp (17); the twelve widen warps, which issue continuously, live on schedulers 0, 2 and 3.
constexpr int kIssuerAWarp = 1;
constexpr int kIssuerBWarp = 5;
constexpr int kProducerWarp2 = 9;
constexpr int kThreads2 = 32 * 20;
static_assert(kWidenWarps2 == 12, "widen_index2 enumerates twelve widen warps");
static_assert(kWidenGroups2 == 4, "group g owns staging slot g and int8 slot g: four of each");
__device__ __forceinline__ bool is_epilogue_warp2(int w) { return (w >= 2 && w <= 4) || w == 13; }
// 0 .. 11 for the widen warps (0, 6-8, 10-12, 14-16, 18, 19), -1 otherwise
__device__ __forceinline__ int widen_index2(int w) {
  if (w == 0) return 0;
  if (w < 6 || (w & 3) == 1) return -1;
  return w - 5 - ((w - 5) >> 2);   // 6,7,8 -> 1,2,3; 10,11,12 -> 4,5,6; 14,15,16 -> 7,8,9; 18,19 -> 10,11
}

// fp16 epilogue of 64 accumulator columns for the warps that help with the last tile of a CTA (see the end of the
// kernel): the arithmetic and the staging pattern of the epilogue warps' inline code, kept out of line so that it does
// not add to the register count of the hot loops.
__device__ __noinline__ void store_block64(uint32_t taddr, const float* sq, const __half* bias, float sp, unsigned char* stg,
                                           uint32_t stg_u32, int lane, const CUtensorMap* maps, int n_outs, int g0, int x, int y,
                                           bool in_range) {
  const uint32_t my_sw = (uint32_t)(lane & 7);
#pragma unroll 1
  for (int h = 0; h < 2; ++h) {
    uint32_t r[32];
    tmem_ld32(taddr + 32 * h, r);
    tmem_ld_wait();
    uint4 pk[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      __half2* hh = reinterpret_cast<__half2*>(&pk[e]);
      const int jc = 32 * h + 8 * e;
      const float4 s0 = *reinterpret_cast<const float4*>(sq + jc);
      const float4 s1 = *reinterpret_cast<const float4*>(sq + jc + 4);
      hh[0] = __floats2half2_rn((float)(int32_t)r[8 * e + 0] * (sp * s0.x), (float)(int32_t)r[8 * e + 1] * (sp * s0.y));
      hh[1] = __floats2half2_rn((float)(int32_t)r[8 * e + 2] * (sp * s0.z), (float)(int32_t)r[8 * e + 3] * (sp * s0.w));
      hh[2] = __floats2half2_rn((float)(int32_t)r[8 * e + 4] * (sp * s1.x), (float)(int32_t)r[8 * e + 5] * (sp * s1.y));
      hh[3] = __floats2half2_rn((float)(int32_t)r[8 * e + 6] * (sp * s1.z), (float)(int32_t)r[8 * e + 7] * (sp * s1.w));
      if (bias) {
        const uint4 bb = *reinterpret_cast<const uint4*>(bias + jc);
        const __half2* bh = reinterpret_cast<const __half2*>(&bb);
#pragma unroll
        for (int q = 0; q < 4; ++q) hh[q] = __hadd2(hh[q], bh[q]);
      }
    }
#pragma unroll
    for (int e = 0; e < 4; ++e)
      *reinterpret_cast<uint4*>(stg + lane * 128 + ((((uint32_t)(4 * h + e)) ^ my_sw) << 4)) = pk[e];
  }
  fence_proxy_async_smem();
  __syncwarp();
  if (lane == 0 && in_range) {
    for (int i = 0, g = g0 % n_outs; i < n_outs; ++i, g = (g + 1 == n_outs) ? 0 : g + 1) tma_store_2d(&maps[g], stg_u32, x, y);
    bulk_commit_group();
  }
}

// fp16 epilogue of 16 accumulator columns (tile widths that are not a multiple of 64): dequantise, stage as 32 rows x 32
// bytes and hand the piece to the TMA unit.  Kept out of line so that it does not add to the register count of the
// kernel's hot loops.
__device__ __noinline__ void store_tail_piece(uint32_t taddr, const float* sq, const __half* bias, float sp, unsigned char* stg,
                                              uint32_t stg_u32, int lane, const CUtensorMap* map, int x, int y, bool in_range) {
  uint32_t r[32];
  tmem_ld16(taddr, r);
  uint4 pk[2];
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    __half2* hh = reinterpret_cast<__half2*>(&pk[e]);
    const float4 s0 = *reinterpret_cast<const float4*>(sq + 8 * e);
    const float4 s1 = *reinterpret_cast<const float4*>(sq + 8 * e + 4);
    hh[0] = __floats2half2_rn((float)(int32_t)r[8 * e + 0] * (sp * s0.x), (float)(int32_t)r[8 * e + 1] * (sp * s0.y));
    hh[1] = __floats2half2_rn((float)(int32_t)r[8 * e + 2] * (sp * s0.z), (float)(int32_t)r[8 * e + 3] * (sp * s0.w));
    hh[2] = __floats2half2_rn((float)(int32_t)r[8 * e + 4] * (sp * s1.x), (float)(int32_t)r[8 * e + 5] * (sp * s1.y));
    hh[3] = __floats2half2_rn((float)(int32_t)r[8 * e + 6] * (sp * s1.z), (float)(int32_t)r[8 * e + 7] * (sp * s1.w));
    if (bias) {
      const uint4 bb = *reinterpret_cast<const uint4*>(bias + 8 * e);
      const __half2* bh = reinterpret_cast<const __half2*>(&bb);
#pragma unroll
      for (int q = 0; q < 4; ++q) hh[q] = __hadd2(hh[q], bh[q]);
    }
  }
  if (lane == 0) bulk_wait_read_all();   // the TMA unit has read the previous block out of the staging area
  __syncwarp();
  *reinterpret_cast<uint4*>(stg + lane * 32) = pk[0];
  *reinterpret_cast<uint4*>(stg + lane * 32 + 16) = pk[1];
  fence_proxy_async_smem();
  __syncwarp();
  if (lane == 0 && in_range) {
    tma_store_2d(map, stg_u32, x, y);
    bulk_commit_group();
  }
}

template <int PST, int IST, int MODE, int BN2>
__global__ void __launch_bounds__(kThreads2, 1)
gemm_i4_2sm_kernel(const __grid_constant__ CUtensorMap tmP, const __grid_constant__ CUtensorMap tmQ,
                   const __grid_constant__ OutMaps tmOs, const __grid_constant__ CUtensorMap tmTail, const GemmParams p) {
  using L = SmemLayout2<PST, IST>;
  constexpr int ACC = 2;
  extern __shared__ unsigned char smem_dyn[];
  const uint32_t smem_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  unsigned char* smem_gen = smem_dyn + (smem_base - smem_u32(smem_dyn));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = (rank == 0);

  const uint32_t bar_base = smem_base + L::kBarOff;
  auto full_p = [&](int s) { return bar_base + 8u * s; };
  auto empty_p = [&](int s) { return bar_base + 8u * (PST + s); };
  auto full_i = [&](int s) { return bar_base + 8u * (2 * PST + s); };
  auto empty_i = [&](int s) { return bar_base + 8u * (2 * PST + IST + s); };
  auto acc_full = [&](int a) { return bar_base + 8u * (2 * PST + 2 * IST + a); };
  auto acc_empty = [&](int a) { return bar_base + 8u * (2 * PST + 2 * IST + 2 + a); };
  auto scales_staged = [&](int q) { return bar_base + 8u * (2 * PST + 2 * IST + 4 + q); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + L::kTmemSlotOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + L::kAbortOff);
  volatile uint32_t* turn = reinterpret_cast<volatile uint32_t*>(smem_gen + L::kAbortOff + 4);   // next k-block to issue
  constexpr uint32_t kTmemCols = ACC * kBN2;  // 512
  pdl_launch_dependents();   // the next kernel of the stream may be brought up; it waits for this grid to finish
  if (threadIdx.x == 32) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmP) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmQ) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmOs.m[0]) : "memory");
  }

  if (threadIdx.x == 0) {
    for (int s = 0; s < PST; ++s) { mbar_init(full_p(s), 1); mbar_init(empty_p(s), kWidenWarpsPerGroup2); }   // the warps of the owning group
    for (int s = 0; s < IST; ++s) { mbar_init(full_i(s), 2 * kWidenWarpsPerGroup2); mbar_init(empty_i(s), 1); }      // local + remote warps of the group
    for (int a = 0; a < 2; ++a) { mbar_init(acc_full(a), 2); mbar_init(acc_empty(a), 2 * kEpiWarps); }
    for (int q = 0; q < 4; ++q) mbar_init(scales_staged(q), 1);
    *abort_flag = 0;
    *turn = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc_2sm(smem_base + L::kTmemSlotOff, kTmemCols);
    tmem_relinquish_2sm();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // both CTAs' barriers are initialised before any remote arrive
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int num_tiles = p.tilesP * p.tilesQ;     // pair tiles
  constexpr int bn = BN2;                         // columns of a pair tile; bn / 2 rows of operand Q per CTA
  static_assert(BN2 % 16 == 0 && BN2 >= 128 && BN2 <= kBN2, "pair tile width");
  const int num_kb = (p.K + 127) >> 7;
  const int cluster_id = blockIdx.x >> 1;
  const int num_clusters = gridDim.x >> 1;

  if (warp == kProducerWarp2) {
    // ------------------------------------------------------------ TMA producer (own rows only)
    if (lane == 0) {
      pdl_wait();   // operands may come from the preceding kernel
      uint32_t it = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
        const int tp = tile % p.tilesP, tq = tile / p.tilesP;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % PST;
          const uint32_t ph = (it / PST) & 1;
          if (!mbar_wait(empty_p(s), ph ^ 1, abort_flag, p.status, 11)) { ok = false; break; }
          mbar_expect_tx(full_p(s), (uint32_t)((kBM + (bn >> 1)) * kBKBytes));
          const uint32_t dst = smem_base + L::kPkOff + s * L::kPkStage;
          tma_load_2d(dst, &tmP, full_p(s), kb * kBKBytes, tp * 2 * kBM + (int)rank * kBM);
          tma_load_2d(dst + kBM * kBKBytes, &tmQ, full_p(s), kb * kBKBytes, tq * bn + (int)rank * (bn >> 1));
        }
      }
    }
  } else if (warp == kIssuerAWarp || warp == kIssuerBWarp) {
    // ------------------------------------------------------------ MMA issuers (leader CTA only)
    // Issuing is the critical path of the main loop: per k-block one thread spends several hundred cycles in
    // the barrier wait, the four tcgen05.mma and the commit, more than the MMAs take to execute.  Two threads of
    // different warps therefore take alternate k-blocks.  A shared turn counter keeps the MMAs in k order:
    // a thread issues block `it` only when turn == it, brackets the hand-over with tcgen05.fence
    // before/after_thread_sync (which orders the asynchronous MMAs of the two threads), and does its wait for
    // the next block and its commit while the other thread issues.
    if (leader && lane == 0) {
      const int me = (warp == kIssuerAWarp) ? 0 : 1;
      constexpr uint32_t idesc = make_idesc_i8(2 * kBM, bn);
      const uint32_t peer_acc_full0 = mapa_cluster(acc_full(0), 1);
      uint32_t it = 0, tl = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters, ++tl) {
        const int a = tl % ACC;
        const uint32_t pha = (tl / ACC) & 1;
        const uint32_t d_tmem = tmem_base + a * kBN2;
        bool mine_in_tile = false;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          if ((int)(it & 1u) != me) continue;
          mine_in_tile = true;
          const int s = it % IST;
          const uint32_t ph = (it / IST) & 1;
          // the operand descriptors do not depend on the hand-over: they are ready before the waits
          const uint32_t a_lo = desc_lo(smem_base + L::kI8Off + s * L::kI8Stage);
          const uint32_t b_lo = a_lo + ((kBM * 128) >> 4);
          if (kb < 2) {   // first block of this thread in the tile: the accumulator buffer must have been drained
            if (!mbar_wait(acc_empty(a), pha ^ 1, abort_flag, p.status, 12)) { ok = false; break; }
          }
          if (!mbar_wait(full_i(s), ph, abort_flag, p.status, 13)) { ok = false; break; }
          // my turn?
          {
            bool got = (*turn == it);
            if (!got) {
              const long long t0 = clock64();
              for (uint32_t spin = 1; !got; ++spin) {
                got = (*turn == it);
                if (!got && (spin & 255u) == 0u) {
                  if (*abort_flag) break;
                  if (clock64() - t0 > kWaitCycles) { *abort_flag = 1; atomicExch(p.status, 17); break; }
                }
              }
            }
            if (!got) { ok = false; break; }
          }
          // critical section of the main loop: nothing but the fences, the four MMAs and the hand-over
          tc_fence_after();
          umma_i8_2sm_w<-1>(d_tmem, a_lo, b_lo, kDescHiKmajorSw128, idesc, kb != 0 ? 1u : 0u);
          umma_i8_2sm_w<1>(d_tmem, a_lo + 2, b_lo + 2, kDescHiKmajorSw128, idesc);   // +32 bytes along K = +2 in the address field
          umma_i8_2sm_w<1>(d_tmem, a_lo + 4, b_lo + 4, kDescHiKmajorSw128, idesc);
          umma_i8_2sm_w<1>(d_tmem, a_lo + 6, b_lo + 6, kDescHiKmajorSw128, idesc);
          tc_fence_before();
          *turn = it + 1;
          umma_commit_2sm_mc(empty_i(s), 3);   // one completion signal, delivered to the same barrier in both CTAs
        }
        if (!ok) break;
        // accumulator ready: acc_full needs both issuers (a commit only tracks the MMAs of its own thread)
        if (mine_in_tile) {
          umma_commit_2sm_mc(acc_full(a), 3);
        } else {
          mbar_arrive(acc_full(a));
          mbar_arrive_cluster_relaxed(peer_acc_full0 + 8u * a);
        }
      }
    }
  } else if (is_epilogue_warp2(warp)) {
    // ------------------------------------------------------------ epilogue (own 128 accumulator rows)
    // Warp q4 owns accumulator lanes 32 q4 .. 32 q4 + 31 (one output row per thread).  With a tensor map over
    // the output the rows are written as tiled stores: the warp converts 128 bytes of every row (64 fp16 or
    // 32 int32 columns), puts them into a 128B-swizzled 4 KB staging block of shared memory (conflict-free
    // 16-byte stores) and one thread hands the block to the TMA unit, which writes whole 128-byte row segments
    // and clips what lies outside the matrix.  The load/store pipe of the SM, which the widen warps saturate,
    // then sees 16 store wavefronts per block instead of 128 scattered 16-byte global stores.
    // The tile's 256 column scales (and bias) are fetched into shared memory before the accumulator is waited for.
    // The scales are stored divided by 256: float(256 a) * (s_row * (s_col / 256)) rounds exactly like
    // float(a) * (s_row * s_col), because scaling by a power of two commutes with every rounding involved.
    const int q4 = warp & 3;
    const int prow_in_tile = q4 * 32 + lane;
    const uint32_t leader_acc_empty0 = mapa_cluster(acc_empty(0), 0);
    constexpr int CW = (MODE == MODE_I32) ? 32 : 64;     // columns per staged block (128 bytes per row)
    unsigned char* stg = smem_gen + L::kStageOff + q4 * 4096;
    const uint32_t stg_u32 = smem_base + L::kStageOff + q4 * 4096;
    float* sqf = reinterpret_cast<float*>(smem_gen + L::kScaleOff + q4 * 1024);
    __half* bsh = reinterpret_cast<__half*>(smem_gen + L::kBiasOff + q4 * 512);
    const uint32_t my_sw = (uint32_t)(lane & 7);
    pdl_wait();   // scales and output are touched only after the preceding kernel has finished
    uint32_t tl = 0;
    bool ok = true;
    for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters, ++tl) {
      const int tp = tile % p.tilesP, tq = tile / p.tilesP;
      const int a = tl % ACC;
      const uint32_t pha = (tl / ACC) & 1;
      if (MODE == MODE_F16 && p.tma_out) {
        __syncwarp();   // the previous tile's reads of the scale block are done
#pragma unroll
        for (int j = lane; j < bn; j += 32) {
          const int col = tq * bn + j;
          sqf[j] = col < p.rowsQ ? __half2float(p.sQ[col]) * 0.00390625f : 0.0f;   // 1/256: the accumulator is 256 x the dot product
          if (p.bias) bsh[j] = col < p.rowsQ ? p.bias[col] : __float2half(0.0f);
        }
        __syncwarp();
      }
      // The last tile of this CTA has no main loop behind it to hide its epilogue: the warps that have run out of work
      // take three quarters of it (end of the kernel); they read the scales this warp has just staged.
      const bool shared_tile = MODE == MODE_F16 && p.tma_out && !p.swiglu && p.tail_help && tile + num_clusters >= num_tiles;
      if (shared_tile && lane == 0) mbar_arrive(scales_staged(q4));
      if (!mbar_wait(acc_full(a), pha, abort_flag, p.status, 14)) { ok = false; break; }
      tc_fence_after();
      const int prow = tp * 2 * kBM + (int)rank * kBM + prow_in_tile;
      const bool prow_ok = prow < p.rowsP;
      float sp = 0.0f;
      if (MODE == MODE_F16 && prow_ok) sp = __half2float(p.sP[prow]);
      auto release_acc = [&]() {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive_cluster_relaxed(leader_acc_empty0 + 8u * a);
        }
      };
      if (MODE == MODE_F16 && p.swiglu) {
        // Gate and up projections computed as ONE GEMM over row-interleaved weights: columns [0,128) of the tile are
        // 128 gate channels, columns [128,256) the same 128 up channels.  The epilogue applies the fp16 arithmetic
        // of  act_fn(gate_proj(x)) * up_proj(x)  (both products rounded to fp16, SiLU evaluated in fp32 and rounded,
        // product rounded) and stores 128 columns of the [M, N/2] result: neither projection is ever written out.
        const int row0 = tp * 2 * kBM + (int)rank * kBM + q4 * 32;
#pragma unroll 1
        for (int c0 = 0; c0 < kBN2 / 2; c0 += 64) {
#pragma unroll 1
          for (int q16 = 0; q16 < 4; ++q16) {
            uint32_t rg[32], ru[32];
            const uint32_t tcol = (uint32_t)(a * kBN2 + c0 + 16 * q16);
            tmem_ld16(tmem_base + ((uint32_t)(q4 * 32) << 16) + tcol, rg);
            tmem_ld16(tmem_base + ((uint32_t)(q4 * 32) << 16) + tcol + kBN2 / 2, ru);
            if (c0 + 64 >= kBN2 / 2 && q16 == 3) release_acc();
            uint4 pk[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              __half2* hh = reinterpret_cast<__half2*>(&pk[e]);
#pragma unroll
              for (int j2 = 0; j2 < 4; ++j2) {
                float hv[2];
#pragma unroll
                for (int t = 0; t < 2; ++t) {
                  const int j = 8 * e + 2 * j2 + t;
                  const int jc = c0 + 16 * q16 + j;
                  const __half g = __float2half_rn((float)(int32_t)rg[j] * (sp * sqf[jc]));
                  const __half u = __float2half_rn((float)(int32_t)ru[j] * (sp * sqf[kBN2 / 2 + jc]));
                  const float gf = __half2float(g);
                  const __half act = __float2half_rn(__fdiv_rn(gf, 1.0f + expf(-gf)));
                  hv[t] = __half2float(act) * __half2float(u);
                }
                hh[j2] = __floats2half2_rn(hv[0], hv[1]);
              }
            }
            if (q16 == 0) {
              if (lane == 0) bulk_wait_read_all();
              __syncwarp();
            }
#pragma unroll
            for (int e = 0; e < 2; ++e)
              *reinterpret_cast<uint4*>(stg + lane * 128 + ((((uint32_t)(2 * q16 + e)) ^ my_sw) << 4)) = pk[e];
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0 && row0 < p.rowsP) {
            // the destinations are visited in an order that differs from warp to warp and tile to tile, so that the
            // ranks of a column split do not all write to the same peer at the same time
            for (int i = 0, g = (int)((tl + warp) % (uint32_t)p.n_outs); i < p.n_outs; ++i, g = (g + 1 == p.n_outs) ? 0 : g + 1)
              tma_store_2d(&tmOs.m[g], stg_u32, tq * (kBN2 / 2) + c0, row0);
            bulk_commit_group();
          }
        }
      } else if (p.tma_out) {
        const int row0 = tp * 2 * kBM + (int)rank * kBM + q4 * 32;
        constexpr int full_cols = (MODE == MODE_I32) ? bn : (bn & ~63);    // fp16: whole 64-column blocks, then 16-column pieces
#pragma unroll 1
        for (int c0 = 0; c0 < full_cols; c0 += CW) {
          if (shared_tile && c0 > 0) break;      // the helpers take the other blocks
#pragma unroll
          for (int h = 0; h < CW / 32; ++h) {
            uint32_t r[32];
            tmem_ld32(tmem_base + ((uint32_t)(q4 * 32) << 16) + (uint32_t)(a * kBN2 + c0 + 32 * h), r);
            tmem_ld_wait();
            if (c0 + CW >= bn && h == CW / 32 - 1) release_acc();
            if (MODE == MODE_I32) {
              if (lane == 0) bulk_wait_read_all();   // the TMA unit has read the previous block out of the staging area
              __syncwarp();
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                const uint4 v = make_uint4((uint32_t)((int32_t)r[4 * e] >> 8), (uint32_t)((int32_t)r[4 * e + 1] >> 8),
                                           (uint32_t)((int32_t)r[4 * e + 2] >> 8), (uint32_t)((int32_t)r[4 * e + 3] >> 8));
                *reinterpret_cast<uint4*>(stg + lane * 128 + ((((uint32_t)e) ^ my_sw) << 4)) = v;
              }
            } else {
              uint4 pk[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                __half2* hh = reinterpret_cast<__half2*>(&pk[e]);
                const int jc = c0 + 32 * h + 8 * e;     // column inside the tile
                const float4 s0 = *reinterpret_cast<const float4*>(sqf + jc);
                const float4 s1 = *reinterpret_cast<const float4*>(sqf + jc + 4);
                hh[0] = __floats2half2_rn((float)(int32_t)r[8 * e + 0] * (sp * s0.x),
                                          (float)(int32_t)r[8 * e + 1] * (sp * s0.y));
                hh[1] = __floats2half2_rn((float)(int32_t)r[8 * e + 2] * (sp * s0.z),
                                          (float)(int32_t)r[8 * e + 3] * (sp * s0.w));
                hh[2] = __floats2half2_rn((float)(int32_t)r[8 * e + 4] * (sp * s1.x),
                                          (float)(int32_t)r[8 * e + 5] * (sp * s1.y));
                hh[3] = __floats2half2_rn((float)(int32_t)r[8 * e + 6] * (sp * s1.z),
                                          (float)(int32_t)r[8 * e + 7] * (sp * s1.w));
                if (p.bias) {
                  const uint4 bb = *reinterpret_cast<const uint4*>(bsh + jc);
                  const __half2* bh = reinterpret_cast<const __half2*>(&bb);
#pragma unroll
                  for (int q = 0; q < 4; ++q) hh[q] = __hadd2(hh[q], bh[q]);
                }
              }
              if (h == 0) {
                if (lane == 0) bulk_wait_read_all();
                __syncwarp();
              }
#pragma unroll
              for (int e = 0; e < 4; ++e)
                *reinterpret_cast<uint4*>(stg + lane * 128 + ((((uint32_t)(4 * h + e)) ^ my_sw) << 4)) = pk[e];
            }
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0 && row0 < p.rowsP && tq * bn + c0 < p.rowsQ) {
            // one tiled store per destination: the block goes to this GPU's output and, in a column split, straight
            // into the peers' copies of the full matrix over NVLink; the destinations are visited in an order that differs
            // from warp to warp and tile to tile, so that the ranks do not all write to the same peer at the same time
            for (int i = 0, g = (int)((tl + warp) % (uint32_t)p.n_outs); i < p.n_outs; ++i, g = (g + 1 == p.n_outs) ? 0 : g + 1)
              tma_store_2d(&tmOs.m[g], stg_u32, tq * bn + c0, row0);
            bulk_commit_group();
          }
        }
        if (MODE == MODE_F16 && (bn & 63) != 0 && !shared_tile) {
          // tile widths that are not a multiple of 64 (chosen so that the tiles fill whole waves of clusters): the
          // remaining columns leave as 16-column pieces through a second tensor map (32 rows x 32 bytes, unswizzled)
#pragma unroll 1
          for (int c0 = full_cols; c0 < bn; c0 += 16) {
            store_tail_piece(tmem_base + ((uint32_t)(q4 * 32) << 16) + (uint32_t)(a * kBN2 + c0), sqf + c0,
                             p.bias ? bsh + c0 : nullptr, sp, stg, stg_u32, lane, &tmTail, tq * bn + c0, row0,
                             row0 < p.rowsP && tq * bn + c0 < p.rowsQ);
            if (c0 + 16 >= bn) release_acc();
          }
        }
      } else {
        // output without a tensor map (unaligned base or row pitch): element-wise stores
#pragma unroll 1
        for (int c0 = 0; c0 < bn; c0 += 32) {      // bn is 256 on this path
          uint32_t r[32];
          tmem_ld32(tmem_base + ((uint32_t)(q4 * 32) << 16) + (uint32_t)(a * kBN2 + c0), r);
          tmem_ld_wait();
          if (c0 + 32 >= bn) release_acc();
          const int qcol0 = tq * bn + c0;
          if (prow_ok) {
            if (MODE == MODE_I32) {
              int32_t* o = reinterpret_cast<int32_t*>(p.out) + (int64_t)prow * p.ldo + qcol0;
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (qcol0 + j < p.rowsQ) o[j] = (int32_t)r[j] >> 8;
            } else {
              __half* o = reinterpret_cast<__half*>(p.out) + (int64_t)prow * p.ldo + qcol0;
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                if (qcol0 + j < p.rowsQ) {
                  const float sc = __half2float(p.sQ[qcol0 + j]);
                  __half v = __float2half_rn((float)((int32_t)r[j] >> 8) * (sp * sc));
                  if (p.bias) v = __hadd(v, p.bias[qcol0 + j]);
                  o[j] = v;
                }
              }
            }
          }
        }
      }
    }
    if (lane == 0) bulk_wait_read_all();   // the staging block must outlive the TMA unit's reads of it
  } else if (widen_index2(warp) >= 0) {
    // ------------------------------------------------------------ widen int4 -> int8 (own rows)
    // Groups of three warps take the k-blocks round-robin, so that a group has kWidenGroups2 MMA periods
    // per stage (its stores and the proxy fence take more than one).  Packed data is read into registers
    // before the int8 slot is waited for, which keeps the shared-memory read off the slot-reuse path.
    const int wi = widen_index2(warp);
    const int group = wi / kWidenWarpsPerGroup2;                               // three warps per group
    const int gt = (wi % kWidenWarpsPerGroup2) * 32 + lane;                    // 0 .. 95 inside the group
    constexpr int kChunks = (kBM + (bn >> 1)) * 4;      // packed 16-byte chunks per stage (1024 at bn = 256)
    constexpr int kGThreads = 32 * kWidenWarpsPerGroup2;
    constexpr int kPer = (kChunks + kGThreads - 1) / kGThreads;   // 11 chunks per thread at bn = 256 (the last round is partial)
    const uint32_t leader_full_i0 = mapa_cluster(full_i(0), 0);
    uint32_t it = 0;
    bool ok = true;
    for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        if ((int)(it % kWidenGroups2) != group) continue;
        const int sp_ = it % PST, si = it % IST;
        const uint32_t php = (it / PST) & 1, phi = (it / IST) & 1;
        // Group g is the only reader of staging slot g (four groups, four slots), so it sees every phase of that
        // slot's barrier in turn and a parity wait is unambiguous even when TMA loads complete out of order.  (With
        // three groups a group came back to a slot only every third use; a load of the previous use still in flight
        // then looked like "this phase complete" and deadlocked the pipeline.)
        if (!mbar_wait(full_p(sp_), php, abort_flag, p.status, 15)) { ok = false; break; }
        const unsigned char* pk = smem_gen + L::kPkOff + sp_ * L::kPkStage;
        uint4 w[kPer];
#pragma unroll
        for (int j = 0; j < kPer; ++j)
          w[j] = (gt + j * kGThreads < kChunks) ? *reinterpret_cast<const uint4*>(pk + (gt + j * kGThreads) * 16)
                                                : make_uint4(0, 0, 0, 0);
        // Hand the staging slot back to the TMA producer as soon as the packed data is in registers.  The
        // arrive must not overtake the loads, so it is made to depend on every loaded word: the words are
        // folded into one value that feeds a (practically never taken) predicated store.
        {
          uint32_t fold = 0;
#pragma unroll
          for (int j = 0; j < kPer; ++j) fold ^= w[j].x ^ w[j].y ^ w[j].z ^ w[j].w;
          asm volatile(
              "{\n\t.reg .pred p;\n\t"
              "setp.eq.u32 p, %0, 0xC0FFEE11;\n\t"
              "@p st.volatile.shared.u32 [%1], %0;\n\t}"
              ::"r"(fold), "r"(smem_base + L::kAbortOff + 8)
              : "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive(empty_p(sp_));
        }
        if (!mbar_wait(empty_i(si), phi ^ 1, abort_flag, p.status, 16)) { ok = false; break; }
        tc_fence_after();
        unsigned char* i8 = smem_gen + L::kI8Off + si * L::kI8Stage;
#pragma unroll
        for (int j = 0; j < kPer; ++j) {
          const int c = gt + j * kGThreads;
          if (c >= kChunks) break;
          const int row = c >> 2, cc = c & 3;
          uint4 lo, hi;
          lo.x = (w[j].x << 4) & 0xF0F0F0F0u; hi.x = w[j].x & 0xF0F0F0F0u;
          lo.y = (w[j].y << 4) & 0xF0F0F0F0u; hi.y = w[j].y & 0xF0F0F0F0u;
          lo.z = (w[j].z << 4) & 0xF0F0F0F0u; hi.z = w[j].z & 0xF0F0F0F0u;
          lo.w = (w[j].w << 4) & 0xF0F0F0F0u; hi.w = w[j].w & 0xF0F0F0F0u;
          unsigned char* drow = i8 + row * 128;
          const int sw = row & 7;
          *reinterpret_cast<uint4*>(drow + (((2 * cc) ^ sw) << 4)) = lo;
          *reinterpret_cast<uint4*>(drow + (((2 * cc + 1) ^ sw) << 4)) = hi;
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive_cluster_relaxed(leader_full_i0 + 8u * si);
        }
      }
    }
  }

  // ---------------------------------------------------------------- the last tile's epilogue, shared
  // After the last MMA of a CTA only its four epilogue warps would still have work (a quarter of the accumulator each,
  // four 64-column blocks one after the other) while sixteen warps idle, and nothing hides that time.  Three more
  // warps per tensor-memory lane quarter (warp id modulo 4: the widen warps on quarters 0, 2, 3; the idle warp, the
  // producer and one issuer on quarter 1) therefore take the blocks behind the first; their staging blocks lie in the
  // int8 operand ring, which nothing reads once the accumulator is complete.
  if (MODE == MODE_F16 && p.tma_out && !p.swiglu && p.tail_help) {
    __syncwarp();                       // single-thread roles: the rest of the warp has waited here
    const int q4 = warp & 3;
    int hr = -1;
    if (!is_epilogue_warp2(warp)) {
      if (q4 == 1) hr = warp == 17 ? 0 : warp == kProducerWarp2 ? 1 : warp == kIssuerBWarp ? 2 : -1;
      else hr = warp == 0 ? 0 : (warp >> 2) - 1;
      if (hr > 2) hr = -1;
    }
    const int my_tiles = cluster_id < num_tiles ? (num_tiles - cluster_id + num_clusters - 1) / num_clusters : 0;
    if (hr >= 0 && my_tiles > 0 && !*abort_flag) {
      const uint32_t tl = (uint32_t)(my_tiles - 1);
      const int tile = cluster_id + (int)tl * num_clusters;
      const int tp = tile % p.tilesP, tq = tile / p.tilesP;
      const int a = tl % ACC;
      const uint32_t pha = (tl / ACC) & 1;
      pdl_wait();   // the output belongs to the preceding kernels
      if (mbar_wait(scales_staged(q4), 0, abort_flag, p.status, 18) && mbar_wait(acc_full(a), pha, abort_flag, p.status, 19)) {
        tc_fence_after();
        const float* sqf = reinterpret_cast<const float*>(smem_gen + L::kScaleOff + q4 * 1024);
        const __half* bsh = reinterpret_cast<const __half*>(smem_gen + L::kBiasOff + q4 * 512);
        const int prow = tp * 2 * kBM + (int)rank * kBM + q4 * 32 + lane;
        const float sp = prow < p.rowsP ? __half2float(p.sP[prow]) : 0.0f;
        const int row0 = tp * 2 * kBM + (int)rank * kBM + q4 * 32;
        unsigned char* stg = smem_gen + L::kI8Off + (q4 * 3 + hr) * 4096;
        const uint32_t stg_u32 = smem_base + L::kI8Off + (q4 * 3 + hr) * 4096;
        constexpr int full_cols = bn & ~63;
        const int c0 = 64 * (hr + 1);
        const uint32_t taddr = tmem_base + ((uint32_t)(q4 * 32) << 16) + (uint32_t)(a * kBN2);
        if (c0 < full_cols) {
          store_block64(taddr + c0, sqf + c0, p.bias ? bsh + c0 : nullptr, sp, stg, stg_u32, lane, &tmOs.m[0], p.n_outs,
                        (int)tl + warp, tq * bn + c0, row0, row0 < p.rowsP && tq * bn + c0 < p.rowsQ);
        } else if (c0 == full_cols) {
#pragma unroll 1
          for (int c1 = full_cols; c1 < bn; c1 += 16)
            store_tail_piece(taddr + c1, sqf + c1, p.bias ? bsh + c1 : nullptr, sp, stg, stg_u32, lane, &tmTail, tq * bn + c1, row0,
                             row0 < p.rowsP && tq * bn + c1 < p.rowsQ);
        }
        if (lane == 0) bulk_wait_read_all();   // the staging block must outlive the TMA unit's reads of it
      }
    }
  }

  // ---------------------------------------------------------------- teardown
  drain_after_abort(abort_flag);
  tc_fence_before();
  __syncthreads();
  __syncwarp();
  cluster_sync_all();   // the peer may still read this CTA's shared memory or arrive on its barriers
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc_2sm(tmem_base, kTmemCols);
  }
}

// ------------------------------------------------------------------ host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

// Tensor map over a packed int4 matrix [rows, kbytes] (uint8), box = [64 bytes, box_rows], no swizzle.
static int make_packed_map(CUtensorMap* map, const void* base, int64_t rows, int64_t kbytes, int box_rows,
                           int box_bytes = kBKBytes) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return fail(QR_ENOTREADY, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[2] = {(cuuint64_t)kbytes, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)kbytes};
  cuuint32_t box[2] = {(cuuint32_t)box_bytes, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(QR_EINVAL, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return QR_OK;
}

// Tensor map over the output matrix [rows, cols] with a row pitch of ldo elements (fp16 or int32), box = 128 bytes
// of a row x 32 rows, 128-byte swizzle: what one epilogue warp of the 2-CTA kernel stores at a time.
// (tail = true: 16 fp16 columns x 32 rows, unswizzled, for tile widths that are not a multiple of 64.)
static int make_out_map(CUtensorMap* map, void* base, int64_t rows, int64_t cols, int64_t ldo, bool is_i32, bool tail = false) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return fail(QR_ENOTREADY, "cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t esz = is_i32 ? 4 : 2;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ldo * esz};
  cuuint32_t box[2] = {(cuuint32_t)(tail ? 16 : 128 / esz), 32};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, is_i32 ? CU_TENSOR_MAP_DATA_TYPE_INT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, base, dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, tail ? CU_TENSOR_MAP_SWIZZLE_NONE : CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(QR_EINVAL, "cuTensorMapEncodeTiled (output) failed with CUresult %d", (int)r);
  return QR_OK;
}

template <int BN, int PST, int IST, int ACC, int MODE>
static int launch_gemm(const CUtensorMap& tmP, const CUtensorMap& tmQ, const GemmParams& p, int grid_cap, cudaStream_t st) {
  using L = SmemLayout<BN, PST, IST>;
  static_assert(L::kDynamic <= 227 * 1024, "shared memory budget exceeded");
  auto kern = gemm_i4_kernel<BN, PST, IST, ACC, MODE>;
  static thread_local bool configured[64] = {false};
  int dev = 0;
  QR_CUDA(cudaGetDevice(&dev));
  if (dev >= 64 || !configured[dev]) {
    QR_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic));
    if (dev < 64) configured[dev] = true;
  }
  int grid = p.tilesP * p.tilesQ;
  int cap = grid_cap > 0 ? grid_cap : num_sms();
  if (grid > cap) grid = cap;
  QR_CUDA(launch_kernel(kern, dim3(grid), dim3(kThreads), (size_t)L::kDynamic, st, use_pdl(p.rowsP), tmP, tmQ, p));
  return QR_OK;
}

template <typename Kern, typename... Maps>
static int launch_cluster2(Kern kern, int threads, int smem_bytes, int* max_clusters, const GemmParams& p, int grid_cap,
                           cudaStream_t st, bool pdl, const Maps&... maps);

template <int PST, int IST, int MODE, int BN2>
static int launch_gemm_2sm_bn(const CUtensorMap& tmP, const CUtensorMap& tmQ, const OutMaps& tmO, const CUtensorMap& tmTail,
                              const GemmParams& p, int grid_cap, cudaStream_t st) {
  using L = SmemLayout2<PST, IST>;
  static_assert(L::kDynamic <= 227 * 1024, "shared memory budget exceeded");
  static_assert(L::kStageOff % 1024 == 0, "staging blocks must be 1024-byte aligned for the 128-byte swizzle");
  static thread_local int max_clusters[64] = {0};
  return launch_cluster2(gemm_i4_2sm_kernel<PST, IST, MODE, BN2>, kThreads2, L::kDynamic, max_clusters, p, grid_cap, st,
                         use_pdl(p.rowsP), tmP, tmQ, tmO, tmTail);
}

// pair-tile widths the fp16 epilogue is compiled for (the int32 path always uses 256)
constexpr int kPairWidths[] = {256, 240, 224, 192};

template <int PST, int IST, int MODE>
static int launch_gemm_2sm(const CUtensorMap& tmP, const CUtensorMap& tmQ, const OutMaps& tmO, const CUtensorMap& tmTail,
                           const GemmParams& p, int grid_cap, cudaStream_t st) {
  if (MODE == MODE_F16) {
    if (p.bn == 240) return launch_gemm_2sm_bn<PST, IST, MODE_F16, 240>(tmP, tmQ, tmO, tmTail, p, grid_cap, st);
    if (p.bn == 224) return launch_gemm_2sm_bn<PST, IST, MODE_F16, 224>(tmP, tmQ, tmO, tmTail, p, grid_cap, st);
    if (p.bn == 192) return launch_gemm_2sm_bn<PST, IST, MODE_F16, 192>(tmP, tmQ, tmO, tmTail, p, grid_cap, st);
  }
  return launch_gemm_2sm_bn<PST, IST, MODE, kBN2>(tmP, tmQ, tmO, tmTail, p, grid_cap, st);
}

template <typename Kern, typename... Maps>
static int launch_cluster2(Kern kern, int threads, int smem_bytes, int* max_clusters, const GemmParams& p, int grid_cap,
                           cudaStream_t st, bool pdl, const Maps&... maps) {
  int dev = 0;
  QR_CUDA(cudaGetDevice(&dev));
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.blockDim = dim3(threads);
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = st;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int nclusters = (dev < 64) ? max_clusters[dev] : 0;
  if (nclusters == 0) {
    QR_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
    cfg.gridDim = dim3(2 * (num_sms() / 2));
    QR_CUDA(cudaOccupancyMaxActiveClusters(&nclusters, kern, &cfg));
    if (nclusters < 1) return fail(QR_EUNSUPPORTED, "2-CTA GEMM: no cluster of 2 CTAs fits on this device");
    if (dev < 64) max_clusters[dev] = nclusters;
  }
  int clusters = p.tilesP * p.tilesQ;
  if (clusters > nclusters) clusters = nclusters;
  if (grid_cap > 0 && clusters > grid_cap) clusters = grid_cap;
  cfg.gridDim = dim3(2 * clusters);
  cfg.numAttrs = pdl ? 2 : 1;
  QR_CUDA(cudaLaunchKernelEx(&cfg, kern, maps..., p));
  return QR_OK;
}

// weight-streaming tcgen05 kernel for M <= 64 (gemm_i4_decode.cu)
int launch_gemm_i4_decode(const uint8_t* X, const uint8_t* W, int64_t M, int64_t N, int64_t K, void* out, int64_t ldo,
                          const void* sX, const void* sW, const void* bias, bool f16, int grid_cap, void* ws, size_t ws_bytes,
                          cudaStream_t st);
size_t decode_stream_workspace_bytes(int64_t M, int64_t N, int64_t K);
// weight-streaming mma.sync kernel for M <= 32 (gemv_mma_i4.cu)
bool gemv_mma_serves(int64_t M, int64_t K);
// 33 .. 64 token rows of a layer small enough that two passes of that kernel are the fastest form
static bool gemv_two_pass(int64_t M, int64_t N, int64_t K) {
  return g_tuning.gemv_mma_two_pass != 0 && g_tuning.gemv_mma_max_m >= 32 && M > 32 && M <= 64 &&
         N * (K / 2) <= (int64_t)12 * 1024 * 1024 && gemv_mma_serves(32, K);
}
int launch_gemv_mma_i4(const uint8_t* A, const uint8_t* B, int64_t M, int64_t N, int64_t K, void* out, int64_t ldo,
                       const void* sA, const void* sB, const void* bias, bool f16, cudaStream_t st);
// weight-streaming CUDA-core kernel for M <= 8 (gemv_i4.cu)
int launch_gemv_i4(const uint8_t* A, const uint8_t* B, int64_t M, int64_t N, int64_t K, void* out, int64_t ldo,
                   const void* sA, const void* sB, const void* bias, bool f16, cudaStream_t st,
                   const void* x = nullptr, int64_t ldx = 0, float clip = 1.0f);

template <int MODE>
static int run_gemm(const char* who, const uint8_t* A, const uint8_t* B, int64_t M, int64_t N, int64_t K,
                    void* out, int64_t ldo, const void* sA, const void* sB, const void* bias, cudaStream_t st,
                    void* ws = nullptr, size_t ws_bytes = 0,
                    void* const* more_outs = nullptr, int n_more = 0, bool swiglu = false) {
  if (M < 0 || N < 0 || K < 0) return fail(QR_EINVAL, "%s: negative size", who);
  if (M == 0 || N == 0) return QR_OK;
  if (!A || !B || !out) return fail(QR_EINVAL, "%s: null pointer", who);
  if (MODE == MODE_F16 && (!sA || !sB)) return fail(QR_EINVAL, "%s: null scale pointer", who);
  if (K == 0 || (K % 32) != 0) return fail(QR_EINVAL, "%s: K = %lld must be a positive multiple of 32", who, (long long)K);
  if (K > 131071) return fail(QR_EUNSUPPORTED, "%s: K = %lld exceeds the int32 headroom of the x256 accumulator", who, (long long)K);
  if (M > (1 << 30) || N > (1 << 30)) return fail(QR_EUNSUPPORTED, "%s: dimension too large", who);
  if (!aligned16(A) || !aligned16(B)) return fail(QR_EALIGN, "%s: operands must be 16-byte aligned", who);
  if (!swiglu && ldo < N) return fail(QR_EINVAL, "%s: ldo < N", who);
  int* status = kernel_status_ptr();
  if (!status) return fail(QR_ENOTREADY, "%s: no CUDA device", who);

  GemmParams p;
  p.K = (int)K; p.out = out; p.ldo = ldo; p.status = status;
  p.bias = reinterpret_cast<const __half*>(bias);
  p.tma_out = 0; p.n_outs = 1; p.swiglu = 0; p.bn = kBN2; p.tail_help = g_tuning.gemm_tail_help;
  if (swiglu) {
    if (M <= kBM || g_tuning.gemm_2sm == 0)
      return fail(QR_EUNSUPPORTED, "%s: served by the prefill kernel only (more than %d rows)", who, kBM);
    if (N % kBN2 != 0) return fail(QR_EINVAL, "%s: N = %lld must be a multiple of %d (interleaved gate/up rows)", who, (long long)N, kBN2);
    if (bias) return fail(QR_EUNSUPPORTED, "%s: bias is not supported", who);
    if (!aligned16(out) || ldo % 8 != 0) return fail(QR_EALIGN, "%s: output must be 16-byte aligned with ldo %% 8 == 0", who);
    if (ldo < N / 2) return fail(QR_EINVAL, "%s: ldo < N / 2", who);
  }
  if (n_more > 0 && (M <= kBM || g_tuning.gemm_2sm == 0))
    return fail(QR_EUNSUPPORTED, "%s: several outputs are served by the prefill kernel only (more than %d rows)", who, kBM);
  p.vec_ok = aligned16(out) && (ldo % (MODE == MODE_I32 ? 4 : 8) == 0) &&
             (MODE == MODE_I32 || (aligned16(sB) && (!bias || aligned16(bias))));
  CUtensorMap tmP, tmQ;
  int rc;
  const int grid_cap = g_tuning.gemm_grid;
  if (M > kBM && g_tuning.gemm_2sm != 0) {
    p.rowsP = (int)M; p.rowsQ = (int)N;
    p.tilesP = (int)((M + 2 * kBM - 1) / (2 * kBM));
    p.sP = reinterpret_cast<const __half*>(sA); p.sQ = reinterpret_cast<const __half*>(sB);
    // tiled stores need a 16-byte aligned base and row pitch; otherwise the epilogue stores element-wise
    OutMaps tmO;
    CUtensorMap tmTail;
    p.tma_out = aligned16(out) && (ldo % (MODE == MODE_I32 ? 4 : 8) == 0) && g_tuning.gemm_tma_out != 0;
    p.n_outs = 1;
    // Tile width.  The persistent clusters take the pair tiles in waves, and a last wave that is half empty costs as
    // much as a full one; a slightly narrower tile often fills the waves (4096 x 12288 on 74 clusters: 384 tiles of
    // 256 columns = 6 waves of 256, 440 tiles of 224 columns = 6 waves of 224).  The width that minimises
    // waves x (width + a fixed per-tile cost) is taken; widths other than 256 need the fp16 epilogue with tiled stores.
    p.bn = kBN2;
    if (MODE == MODE_F16 && !swiglu && n_more == 0 && p.tma_out && g_tuning.gemm_bn2 != 256) {
      int clusters = num_sms() / 2;
      if (grid_cap > 0 && clusters > grid_cap) clusters = grid_cap;
      long long best = -1;
      for (int bn : kPairWidths) {
        if (g_tuning.gemm_bn2 != 0 && g_tuning.gemm_bn2 != bn) continue;     // a width forced through the knob
        const long long tiles = (long long)p.tilesP * ((N + bn - 1) / bn);
        const long long cost = ((tiles + clusters - 1) / clusters) * (bn + 8);
        if (best < 0 || cost < best) { best = cost; p.bn = bn; }
      }
    }
    p.tilesQ = (int)((N + p.bn - 1) / p.bn);
    if ((rc = make_packed_map(&tmP, A, M, K / 2, kBM))) return rc;
    if ((rc = make_packed_map(&tmQ, B, N, K / 2, p.bn / 2))) return rc;
    if (swiglu) {
      p.swiglu = 1; p.tma_out = 1;
      if ((rc = make_out_map(&tmO.m[0], out, M, N / 2, ldo, false))) return rc;
    } else if (p.tma_out) {
      if ((rc = make_out_map(&tmO.m[0], out, M, N, ldo, MODE == MODE_I32))) return rc;
      if (p.bn % 64 != 0 && (rc = make_out_map(&tmTail, out, M, N, ldo, false, true))) return rc;
      for (int g = 0; g < n_more; ++g) {
        if (!aligned16(more_outs[g])) return fail(QR_EALIGN, "%s: every output must be 16-byte aligned", who);
        if ((rc = make_out_map(&tmO.m[1 + g], more_outs[g], M, N, ldo, MODE == MODE_I32))) return rc;
      }
      p.n_outs = 1 + n_more;
    } else {
      if (n_more > 0) return fail(QR_EALIGN, "%s: several outputs need a 16-byte aligned base and row pitch", who);
      tmO.m[0] = tmP;   // never dereferenced
    }
    for (int g = p.n_outs; g < kMaxOuts; ++g) tmO.m[g] = tmO.m[0];
    if (p.bn % 64 == 0) tmTail = tmO.m[0];   // never dereferenced
    return launch_gemm_2sm<4, 4, MODE>(tmP, tmQ, tmO, tmTail, p, grid_cap, st);
  }
  if (M <= g_tuning.gemm_decode_max_m && !swiglu && n_more == 0) {
    // a handful of token rows: one pass over the weights on the CUDA cores, no tensor-core fixed costs
    if (M <= g_tuning.gemv_max_m) {
      rc = launch_gemv_i4(A, B, M, N, K, out, ldo, sA, sB, bias, MODE == MODE_F16, st);
      if (rc != QR_EUNSUPPORTED) return rc;
    }
    // a few more rows: the same streaming structure with warp-level MMAs (gemv_mma_i4.cu)
    if (M <= g_tuning.gemv_mma_max_m) {
      rc = launch_gemv_mma_i4(A, B, M, N, K, out, ldo, sA, sB, bias, MODE == MODE_F16, st);
      if (rc != QR_EUNSUPPORTED) return rc;
    }
    // 33 .. 64 rows of a small layer (o_proj of a 7B model: 8 MB of weights): two passes of that kernel over the
    // weights, 32 token rows each, beat the tcgen05 kernel below, whose MMA instruction count does not shrink with
    // the layer (4096 x 4096 at 64 rows: 10.6 against 14.0 us; from about 12 MB on the single pass wins)
    if (gemv_two_pass(M, N, K)) {
      const size_t esz = MODE == MODE_F16 ? 2 : 4;
      rc = launch_gemv_mma_i4(A, B, 32, N, K, out, ldo, sA, sB, bias, MODE == MODE_F16, st);
      if (rc == QR_OK)
        rc = launch_gemv_mma_i4(A + (size_t)32 * (K / 2), B, M - 32, N, K, reinterpret_cast<char*>(out) + (size_t)32 * ldo * esz, ldo,
                                sA ? reinterpret_cast<const char*>(sA) + 64 : nullptr, sB, bias, MODE == MODE_F16, st);
      if (rc != QR_EUNSUPPORTED) return rc;
    }
    // decode-sized M on the tensor cores: weights on the MMA rows, all SMs streaming (gemm_i4_decode.cu)
    if (g_tuning.gemm_decode != 0) {
      rc = launch_gemm_i4_decode(A, B, M, N, K, out, ldo, sA, sB, bias, MODE == MODE_F16, grid_cap, ws, ws_bytes, st);
      if (rc != QR_EUNSUPPORTED) return rc;
    }
  }
  // everything else (up to 128 token rows, or the 2-CTA kernel switched off): tokens on the 128 MMA rows of one CTA
  int bn = g_tuning.gemm_bn;
  if (bn != 256 && bn != 128 && bn != 64) bn = 256;
  p.rowsP = (int)M; p.rowsQ = (int)N;
  p.tilesP = (int)((M + kBM - 1) / kBM); p.tilesQ = (int)((N + bn - 1) / bn);
  p.sP = reinterpret_cast<const __half*>(sA); p.sQ = reinterpret_cast<const __half*>(sB);
  if ((rc = make_packed_map(&tmP, A, M, K / 2, kBM))) return rc;
  if ((rc = make_packed_map(&tmQ, B, N, K / 2, bn))) return rc;
  const int pst = g_tuning.gemm_pst;
  if (bn == 256) {
    if (pst == 3) return launch_gemm<256, 3, 3, 2, MODE>(tmP, tmQ, p, grid_cap, st);
    return launch_gemm<256, 4, 2, 2, MODE>(tmP, tmQ, p, grid_cap, st);
  }
  if (bn == 128) return launch_gemm<128, 4, 4, 2, MODE>(tmP, tmQ, p, grid_cap, st);
  return launch_gemm<64, 6, 4, 2, MODE>(tmP, tmQ, p, grid_cap, st);
}

}  // namespace qr

extern "C" {

int qr_matmul_i4_i32(const uint8_t* A, const uint8_t* B, int64_t M, int64_t N, int64_t K, int32_t* C, void* stream) {
  return qr::run_gemm<qr::MODE_I32>("qr_matmul_i4_i32", A, B, M, N, K, C, N, nullptr, nullptr, nullptr,
                                    (cudaStream_t)stream);
}

int qr_linear_i4_f16(const uint8_t* A, const void* sA, const uint8_t* B, const void* sB, const void* bias,
                     int64_t M, int64_t N, int64_t K, void* out, int64_t ldo, void* stream) {
  return qr::run_gemm<qr::MODE_F16>("qr_linear_i4_f16", A, B, M, N, K, out, ldo, sA, sB, bias,
                                    (cudaStream_t)stream);
}

int qr_linear_i4_f16_outs(const uint8_t* A, const void* sA, const uint8_t* B, const void* sB, const void* bias,
                          int64_t M, int64_t N, int64_t K, void* const* outs, int n_outs, int64_t ldo, void* stream) {
  if (!outs || n_outs < 1 || n_outs > qr::kMaxOuts)
    return qr::fail(QR_EINVAL, "qr_linear_i4_f16_outs: between 1 and %d outputs", qr::kMaxOuts);
  for (int g = 0; g < n_outs; ++g)
    if (!outs[g]) return qr::fail(QR_EINVAL, "qr_linear_i4_f16_outs: null output %d", g);
  return qr::run_gemm<qr::MODE_F16>("qr_linear_i4_f16_outs", A, B, M, N, K, outs[0], ldo, sA, sB, bias,
                                    (cudaStream_t)stream, nullptr, 0, outs + 1, n_outs - 1);
}

int qr_linear_i4_swiglu_f16(const uint8_t* A, const void* sA, const uint8_t* B, const void* sB,
                            int64_t M, int64_t N2, int64_t K, void* out, int64_t ldo, void* stream) {
  return qr::run_gemm<qr::MODE_F16>("qr_linear_i4_swiglu_f16", A, B, M, N2, K, out, ldo, sA, sB, nullptr,
                                    (cudaStream_t)stream, nullptr, 0, nullptr, 0, true);
}

// Scratch bytes a decode-sized call wants: narrow layers only (their (tile, stage) units are dealt out to the
// SMs and pieces of a tile meet in scratch memory); everything else runs without scratch.
size_t qr_linear_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  if (M <= qr::g_tuning.gemv_max_m || M > qr::g_tuning.gemm_decode_max_m || qr::g_tuning.gemm_decode == 0) return 0;
  if (M <= qr::g_tuning.gemv_mma_max_m && qr::gemv_mma_serves(M, K)) return 0;      // the mma.sync GEMV needs no scratch
  if (qr::gemv_two_pass(M, N, K)) return 0;                                           // nor do two passes of it
  return qr::decode_stream_workspace_bytes(M, N, K);
}

// ---- scratch that lives inside the library image (see qr_linear_i4_f16_static) -----------------
// In host code the array's name is only a handle: the device address has to be asked for with
// cudaGetSymbolAddress, once per device and with that device current.
namespace qr {
constexpr size_t kStaticScratchBytes = (1u << 20) + (64u << 10);   // 64 KiB of arrival counters + 1 MiB of int32 sums
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

static int static_scratch_ptr(void** out) {
  static std::mutex mu;
  static std::map<int, void*> per_device;
  int dev = 0;
  QR_CUDA(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lk(mu);
  auto it = per_device.find(dev);
  if (it == per_device.end()) {
    void* ptr = nullptr;
    QR_CUDA(cudaGetSymbolAddress(&ptr, g_static_scratch));
    it = per_device.emplace(dev, ptr).first;
  }
  *out = it->second;
  return QR_OK;
}
}  // namespace qr

int qr_linear_i4_f16_static(const uint8_t* A, const void* sA, const uint8_t* B, const void* sB, const void* bias,
                            int64_t M, int64_t N, int64_t K, void* out, int64_t ldo, void* stream) {
  const size_t need = qr_linear_workspace_bytes(M, N, K);
  if (need > qr::kStaticScratchBytes)
    return qr::fail(QR_EUNSUPPORTED,
                    "qr_linear_i4_f16_static: this shape needs %zu bytes of scratch, the built-in scratch holds %zu; "
                    "use qr_linear_i4_f16_ws with a caller-provided workspace", need, qr::kStaticScratchBytes);
  if (need == 0)   // shape runs without scratch
    return qr::run_gemm<qr::MODE_F16>("qr_linear_i4_f16_static", A, B, M, N, K, out, ldo, sA, sB, bias,
                                      (cudaStream_t)stream);
  void* scratch = nullptr;
  const int rc = qr::static_scratch_ptr(&scratch);
  if (rc != QR_OK) return rc;
  // Every call shares the array and finds the previous call's contents in it.  A call that ran to its end leaves
  // the part it used at zero, but nothing says that the previous call did (a different shape, a kernel that gave
  // up on a wait): the counters and sums this shape uses are cleared on the caller's stream first.
  const size_t tiles = (size_t)((N + 127) / 128);
  const size_t counters = 64u << 10;
  QR_CUDA(cudaMemsetAsync(scratch, 0, tiles * sizeof(int), (cudaStream_t)stream));
  QR_CUDA(cudaMemsetAsync(static_cast<unsigned char*>(scratch) + counters, 0, need - counters, (cudaStream_t)stream));
  return qr::run_gemm<qr::MODE_F16>("qr_linear_i4_f16_static", A, B, M, N, K, out, ldo, sA, sB, bias,
                                    (cudaStream_t)stream, scratch, qr::kStaticScratchBytes);
}

int qr_linear_i4_f16_ws(const uint8_t* A, const void* sA, const uint8_t* B, const void* sB, const void* bias,
                        int64_t M, int64_t N, int64_t K, void* out, int64_t ldo,
                        void* workspace, size_t workspace_bytes, void* stream) {
  return qr::run_gemm<qr::MODE_F16>("qr_linear_i4_f16_ws", A, B, M, N, K, out, ldo, sA, sB, bias,
                                    (cudaStream_t)stream, workspace, workspace_bytes);
}

}  // extern "C"
