/*
 * quarot_b200 -- C ABI of the B200 (sm_100a) quantized-linear kernels.
 *
 * Every entry point takes raw device pointers and sizes, enqueues work on the
 * given CUDA stream of the CURRENT device, never allocates device memory,
 * never synchronises the device and never throws.  Return value: 0 on success,
 * a negative QR_E* code for an argument error, or a positive cudaError_t value
 * if a CUDA call failed.  qr_last_error() returns a human-readable message for
 * the most recent failure on the calling thread.
 *
 * Buffers are borrowed for the duration of the enqueued work; all matrices are
 * row-major and densely packed unless a leading dimension is given.
 * "int4 packed" means two signed 4-bit codes per byte, element 2j in the low
 * nibble and element 2j+1 in the high nibble of byte j (the layout of
 * pack_i4, quarot/functional/quantization.py:42-49, and of the upstream CUDA
 * kernel, quarot/kernels/quant.cu:36-44 + quarot/kernels/include/int4.h:86-98).
 *
 * Each declaration cites the upstream interface it stands in for (paths are
 * relative to the upstream QuaRot project).
 */
#ifndef QUAROT_B200_H
#define QUAROT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define QR_VERSION 100

enum {
  QR_OK = 0,
  QR_EINVAL = -1,      /* bad size / null pointer */
  QR_EALIGN = -2,      /* pointer or leading dimension not aligned as documented */
  QR_EUNSUPPORTED = -3,/* shape outside what the kernels implement */
  QR_ENOTREADY = -4,   /* driver entry point missing (needs an sm_100 device + CUDA >= 12.8 driver) */
  QR_EKERNEL = -5      /* a kernel reported a bounded-wait timeout (see qr_kernel_status) */
};

/* Library version (QR_VERSION) -- no upstream counterpart. */
int qr_version(void);

/* Message of the last failure on this thread ("" if none). Stands in for the
 * C++ exceptions raised by TORCH_CHECK / ensure() upstream
 * (quarot/kernels/bindings.cpp:11-16, quarot/kernels/include/common.h:16-23). */
const char* qr_last_error(void);

/* Reads (and clears) the device-side status word of the current device.
 * Kernels with mbarrier waits give up after a bounded number of polls and set
 * it instead of hanging; 0 means no kernel ever timed out.  Synchronises the
 * device.  No upstream counterpart (upstream never checks launches). */
int qr_kernel_status(int* status_out);

/* Kernel-selection knobs, process-wide: "gemm_bn", "gemm_bn2", "gemm_pst", "gemm_grid", "gemm_decode_max_m",
 * "gemm_decode", "gemm_splitk", "gemm_2sm", "gemm_tma_out", "gemm_tail_help", "gemv_max_m", "gemv_mma_max_m", "gemv_mma_halves", "gemv_mma_two_pass", "pdl", "hadq_path",
 * "hadq_tc", "hadq_split", "hadq_heads", "hadq_walsh".  The "gemm_*", "gemv_*" and "pdl" settings never change a bit of a
 * result; the "hadq_*" settings choose between Hadamard kernels that add in different orders, whose fp16 outputs agree
 * within the rounding of the transform (codes and scales are always exact for the output that was produced).  The
 * defaults are the measured best choices.  Unknown keys
 * return QR_EINVAL.  No upstream counterpart. */
int qr_set_tuning(const char* key, int value);

/* Self-test: the quantisers divide by the row scale with one multiplication by the rounded reciprocal.  This
 * runs every finite fp16 value against every finite non-zero fp16 scale on the current device and counts the
 * pairs whose int4 code differs from the one IEEE division gives (expected: 0).  Synchronises the device;
 * uses the legacy default stream.  No upstream counterpart (upstream divides with the `/` operator,
 * quarot/kernels/quant.cu:38-39). */
int qr_debug_division_check(uint64_t* mismatches_out);

/* ------------------------------------------------------------------ (a) ---
 * Online Hadamard transform over the last axis, y = x (hadK (x) H_{n/K})^T/sqrt(n).
 * Replaces fast_hadamard_transform.hadamard_transform + `hadK @` as called by
 * matmul_hadU_cuda (quarot/functional/hadamard.py:92-101) and
 * OnlineHadamard.forward (quarot/nn/hadamard.py:17-23).
 *   x, y      : [rows, n] fp16 (f16 variant) or fp32 (f32 variant); y may alias x
 *   had_k     : K x K row-major table of +-1 in fp16 on the device, or NULL when K == 1
 *   K         : 1, or one of the table orders; n / K must be a power of two
 * Internal arithmetic is fp32 in both variants; the result is rounded once. */
int qr_hadamard_f16(const void* x, void* y, int64_t rows, int64_t n,
                    const void* had_k, int K, void* stream);
int qr_hadamard_f32(const float* x, float* y, int64_t rows, int64_t n,
                    const void* had_k, int K, void* stream);

/* Walsh-Hadamard transform over the LEADING axis of rows that are [heads, head_dim] matrices:
 *   y[h', d] = sum_h (-1)^popcount(h & h') x[h, d] / sqrt(heads)        for every row and every d.
 * This is OnlineHadamard(num_heads) applied to the transposed view attn_output.transpose(-1, -2) and transposed
 * back, as the attention block does in front of o_proj (e2e/quantized_llama/modeling_llama.py:82 with
 * quarot/nn/hadamard.py:17-23), without materialising the transposed tensor: one read and one write of the data.
 *   x, y : [rows, heads, head_dim] fp16, contiguous, 16-byte aligned; y may alias x
 *   heads and head_dim powers of two, head_dim >= 32, 256 <= heads * head_dim <= 4096 (QR_EUNSUPPORTED otherwise:
 *   transform a contiguous copy of the transposed view with qr_hadamard_f16). */
int qr_hadamard_heads_f16(const void* x, void* y, int64_t rows, int64_t heads, int64_t head_dim, void* stream);

/* Fused [online Hadamard ->] per-token absmax scale -> INT4 quantise -> pack.
 * Replaces OnlineHadamard.forward + Quantizer.forward
 * (quarot/nn/hadamard.py:17-23, quarot/nn/quantization.py:9-13) including the
 * sym_quant kernel (quarot/kernels/quant.cu:11-61).
 *   x        : [rows, n] fp16, row stride ldx elements (ldx % 8 == 0, 16-byte aligned)
 *   K        : 0 = no Hadamard (quantiser only); 1 = Walsh; >1 = Kronecker with had_k
 *   clip     : Quantizer.input_clip_ratio
 *   q        : [rows, n/2] uint8 int4 packed          (n % 2 == 0)
 *   scales   : [rows] fp16,  s = fp16(fp16(absmax/7) * clip)
 *   y_out    : optional [rows, n] fp16 copy of the (rounded) Hadamard output that
 *              was quantised, or NULL
 * Codes are clamp(rint(fp16(y / s)), -8, 7) with the division in fp32, exactly
 * the torch arithmetic of sym_quant (quarot/functional/quantization.py:29-32).
 * A row whose scale underflows to 0 follows torch's x / 0 arithmetic: zeros give code 0,
 * positive values 7, negative values -8 (an all-zero row therefore gets all-zero codes). */
int qr_hadamard_quant_i4(const void* x, int64_t rows, int64_t n, int64_t ldx,
                         const void* had_k, int K, float clip,
                         uint8_t* q, void* scales, void* y_out, void* stream);

/* Weight-less RMS normalisation fused in front of the quantiser: the step directly before the path for the
 * inputs of the q/k/v and gate/up projections.  Replaces RMSNorm.forward (quarot/nn/normalization.py:15-21)
 * followed by Quantizer.forward (quarot/nn/quantization.py:9-13):
 *   y = fp16( float(x) * rsqrt(sum(float(x)^2) / mean_dim + eps) ),  then scales and codes of y as in
 *   qr_hadamard_quant_i4 with K = 0.  One pass over x instead of the eight elementwise / reduction kernels
 *   (and their fp32 temporaries) of the unfused modules.
 *   x [rows, n] fp16 with row stride ldx (ldx % 8 == 0, 16-byte aligned), n % 8 == 0, 64 <= n <= 32768;
 *   q [rows, n/2], scales [rows] fp16, y_out optional [rows, n] fp16 copy of the normalised rows. */
int qr_rmsnorm_quant_i4(const void* x, int64_t rows, int64_t n, int64_t ldx, int64_t mean_dim, float eps, float clip,
                        uint8_t* q, void* scales, void* y_out, void* stream);

/* Standalone quantise-and-pack with caller-provided per-row scales.
 * Replaces sym_quant_host (quarot/kernels/include/quant.h:6-13,
 * quarot/kernels/quant.cu:48-61) behind quarot.sym_quant (quarot/__init__.py:43-46).
 *   x [rows, cols] fp16, scale [rows] fp16, q [rows, ceil(cols/2)] uint8. */
int qr_sym_quant_i4(const void* x, const void* scale, int64_t rows, int64_t cols,
                    uint8_t* q, void* stream);

/* ------------------------------------------------------------------ (b) ---
 * C[M,N] int32 = unpack(A)[M,K] . unpack(B)[N,K]^T, exact.
 * Replaces matmul_host (quarot/kernels/include/gemm.h:6-13,
 * quarot/kernels/gemm.cu:7-46) behind quarot.matmul (quarot/__init__.py:37-41).
 *   A [M, K/2], B [N, K/2] uint8 int4 packed, 16-byte aligned; K % 32 == 0. */
int qr_matmul_i4_i32(const uint8_t* A, const uint8_t* B, int64_t M, int64_t N, int64_t K,
                     int32_t* C, void* stream);

/* out[M,N] fp16 = s_row[m] * s_col[n] * half(q[m,n]), all products in fp16 in
 * that order -- the arithmetic of sym_dequant_host
 * (quarot/kernels/include/quant.h:15-23, quarot/kernels/quant.cu:64-97) behind
 * quarot.sym_dequant (quarot/__init__.py:48-52). */
int qr_sym_dequant_i32_f16(const int32_t* q, const void* scale_row, const void* scale_col,
                           int64_t rows, int64_t cols, void* out, void* stream);

/* Fused Linear4bit.forward (quarot/nn/linear.py:42-56): int4 GEMM with the
 * dequantisation (and optional bias) applied in the epilogue, no int32 round
 * trip through memory.
 *   out[m,n] = fp16( float(acc[m,n]) * (float(sA[m]) * float(sB[n])) ) (+ bias[n] in fp16)
 *   A [M,K/2], B [N,K/2] int4 packed; sA [M], sB [N], bias [N] or NULL: fp16;
 *   out [M, N] fp16 with row stride ldo elements. */
int qr_linear_i4_f16(const uint8_t* A, const void* sA, const uint8_t* B, const void* sB,
                     const void* bias, int64_t M, int64_t N, int64_t K,
                     void* out, int64_t ldo, void* stream);

/* qr_linear_i4_f16 whose result lands in several matrices at once: outs[0 .. n_outs) (n_outs <= 8) each point
 * to an [M, N] block with row pitch ldo, in the memory of this GPU or of a peer GPU that this process can
 * address (peer access enabled, or a mapped symmetric allocation).  The epilogue issues one tiled TMA store per
 * destination, so in a column split over G GPUs (rank r owns output channels [r N/G, (r+1) N/G) of a linear, every
 * rank sees all token rows) each rank passes the address of its column block inside every rank's full [M, N_total]
 * matrix and no all-gather is needed afterwards: the slabs cross NVLink while the tensor cores work on the next
 * tile.  The caller orders the launches of the ranks around the buffers (a barrier before the matrices are
 * overwritten and one before they are read).  Needs M > 128, 16-byte aligned outputs and ldo % 8 == 0
 * (QR_EUNSUPPORTED / QR_EALIGN otherwise).  No upstream counterpart: upstream has no multi-GPU code on this path
 * (quarot/nn/linear.py:42-56 runs on one device). */
int qr_linear_i4_f16_outs(const uint8_t* A, const void* sA, const uint8_t* B, const void* sB,
                          const void* bias, int64_t M, int64_t N, int64_t K,
                          void* const* outs, int n_outs, int64_t ldo, void* stream);

/* Gate and up projection of a LLaMA MLP as one GEMM with the SwiGLU product applied in the epilogue:
 *   out[m, c] = fp16( fp16(silu(g)) * u ),  g = fp16(acc_gate[m,c] * (sA[m] * s_gate[c])),  u likewise,
 * silu(g) = g / (1 + exp(-g)) evaluated in fp32 -- the fp16 arithmetic of
 * act_fn(gate_proj(x)) * up_proj(x) in the MLP that upstream subclasses
 * (e2e/quantized_llama/modeling_llama.py:105-119 with Linear4bit.forward, quarot/nn/linear.py:42-56).
 *   B  [N2, K/2], sB [N2]: gate and up weights (and scales) interleaved in groups of 128 output channels:
 *       rows [256 t, 256 t + 128) = gate channels [128 t, 128 t + 128), rows [256 t + 128, 256 t + 256) = the
 *       same up channels; N2 = 2 x intermediate size, a multiple of 256;
 *   out [M, N2/2] fp16 with row pitch ldo (ldo % 8 == 0, 16-byte aligned).
 * Neither projection is written to memory.  Needs M > 128 (QR_EUNSUPPORTED otherwise: run qr_linear_i4_f16 on
 * the interleaved weights and apply the product separately).  No upstream counterpart: upstream launches the two
 * Linear4bit modules and two elementwise kernels. */
int qr_linear_i4_swiglu_f16(const uint8_t* A, const void* sA, const uint8_t* B, const void* sB,
                            int64_t M, int64_t N2, int64_t K, void* out, int64_t ldo, void* stream);

/* Quantizer.forward + Linear4bit.forward (quarot/nn/quantization.py:9-13, quarot/nn/linear.py:42-56) in one
 * launch for at most 8 token rows (single-sequence decode): every CTA of the weight-streaming kernel quantises the
 * rows itself (same scales and codes as qr_hadamard_quant_i4 with K = 0), so the separate quantiser launch and
 * the packed activations disappear.  Same result, bit for bit, as the two calls.
 *   x [M, K] fp16 with row stride ldx (ldx % 8 == 0, 16-byte aligned), clip = Quantizer.input_clip_ratio,
 *   B [N, K/2] int4 packed, sB [N] fp16, bias [N] fp16 or NULL, out [M, N] fp16 with row stride ldo.
 * M > 8: QR_EUNSUPPORTED.  No upstream counterpart. */
int qr_quant_linear_i4_f16(const void* x, int64_t ldx, float clip, const uint8_t* B, const void* sB,
                           const void* bias, int64_t M, int64_t N, int64_t K, void* out, int64_t ldo,
                           void* stream);

/* Decode-sized M (M <= 64) is bound by streaming the weights, so every SM has to stream its share.  Up to 32 token
 * rows a kernel without scratch does that (weights from global memory straight into warp-level MMAs), as long as the
 * token rows fit into shared memory (K up to about 54 000 / 26 000 / 12 000 values for up to 8 / 16 / 32 rows).  What is
 * left -- 33 to 64 rows, or longer rows -- runs on a tcgen05 kernel.  There wide layers
 * get there by dealing the weight rows out to the SMs, which needs no scratch.  A narrow layer (at most 48 weight rows
 * per SM, e.g. N = 4096) with long rows (K above 8192) would leave most of every 128-row MMA idle that way; its (128-row tile, k stage) units are
 * dealt out instead, a tile may then be shared by several CTAs, and its pieces meet in a caller-provided scratch
 * buffer: int32 partial sums added with integer atomics (exact, order independent) plus one arrival counter per
 * tile; the piece that arrives last finishes the tile, nobody waits.  qr_linear_workspace_bytes returns the bytes
 * needed for a shape (0 when the shape runs without scratch).  The workspace must be 256-byte aligned device memory
 * that was zeroed once before its first use -- a kernel that ran to its end leaves what it used at zero; after a
 * non-zero qr_kernel_status zero it again -- and must not be shared by launches that may overlap on the GPU.  Its
 * first 64 KiB hold the arrival counters whatever the shape and the sums follow, so calls of different shapes may
 * share one workspace.  Same result as qr_linear_i4_f16, bit for bit.
 * No upstream counterpart: upstream runs one CUTLASS GEMM (quarot/kernels/gemm.cu:16-41). */
size_t qr_linear_workspace_bytes(int64_t M, int64_t N, int64_t K);
int qr_linear_i4_f16_ws(const uint8_t* A, const void* sA, const uint8_t* B, const void* sB,
                        const void* bias, int64_t M, int64_t N, int64_t K,
                        void* out, int64_t ldo, void* workspace, size_t workspace_bytes, void* stream);

/* qr_linear_i4_f16 for callers that cannot allocate device memory.  This entry point has no
 * counterpart in the upstream project.
 *
 * Who needs it: a host that gave all of its device memory to one arena at start-up (an inference
 * server with a fixed HBM budget, a framework whose caching allocator owns the rest of the card)
 * has nowhere to take the scratch buffer of qr_linear_i4_f16_ws from -- a late cudaMalloc can
 * fail there, and where it succeeds it synchronises the whole device in the middle of the decode
 * loop; a plain C caller in that loop may not own an allocator at all.  For them the scratch of the
 * decode kernel lives inside the library image: a fixed array of 1 MiB + 64 KiB in device memory, held by
 * every GPU that loads the library until the process exits.
 *
 * Same arguments and the same result, bit for bit, as qr_linear_i4_f16.  The call allocates nothing
 * (no cudaMalloc / cudaFree, no allocating library routine).  Limits and rules:
 *   - shapes whose scratch (qr_linear_workspace_bytes: 64 KiB of counters + 128 x BN x 4 bytes per tile of 128
 *     output channels, BN = 16 / 32 / 64 for up to 16 / 32 / 64 token rows) exceeds that size are refused with
 *     QR_EUNSUPPORTED and a message: N <= 4096 fits at every M <= 64, N <= 7104 at M <= 32; shapes that need no
 *     scratch (wide layers, prefill sizes, and up to 32 token rows whose length the scratch-free kernel takes) are
 *     simply run;
 *   - the first call on each device looks up the array's device address (once per device, with
 *     that device current); make that first call before any stream capture begins;
 *   - all calls share the one array and find the previous call's contents in it; the entry point
 *     clears the counters and sums it relies on at the start of every call (on the given stream), but two calls that may
 *     overlap on the GPU (different streams without an ordering between them) race on the array --
 *     order them, or give one of them its own workspace through qr_linear_i4_f16_ws. */
int qr_linear_i4_f16_static(const uint8_t* A, const void* sA, const uint8_t* B, const void* sB,
                            const void* bias, int64_t M, int64_t N, int64_t K,
                            void* out, int64_t ldo, void* stream);

/* ------------------------------------------------------------- KV cache ---
 * Paged 4-bit KV cache of the upstream decoder (quarot/transformers/kv_cache.py:130-289).  Layout, as upstream
 * (quarot/kernels/include/flashinfer/page.cuh:76-103): kv_data [pages, layers, 2 (k | v), heads, page_size, head_dim/2]
 * uint8, unsigned int4 codes with element 2j in the low nibble of byte j; kv_param [pages, layers, 2, heads,
 * page_size, 2] fp16 = (scale, zero), value = code * scale - zero.  Sequence b owns the pages
 * kv_indices[kv_indptr[b] .. kv_indptr[b+1]), the last of which holds last_page_offset[b] tokens (int32 arrays on the
 * device).  head_dim must be 128, as in the upstream kernels.
 *
 * qr_kv_append_i4: [Walsh-Hadamard transform of the keys over head_dim, scale 1/sqrt(head_dim) ->] per-(token, head)
 * asymmetric int4 quantisation (scale = clamp(max - min, 1e-5) / 15, zero = -min, code = clamp(round((x + zero) /
 * scale), 0, 15), every step rounded to fp16 as the torch reference does) -> pack -> write into the page slots, for k
 * and v [tokens, heads, head_dim] fp16.  The page table must already describe the sequences WITH the new tokens;
 * append_indptr [batch + 1] gives the new tokens per sequence (a prompt), NULL means one token per sequence
 * (tokens == batch).  One kernel for matmul_had_cuda + asym_quantize_and_pack_i4 (quarot/transformers/kv_cache.py:10-35)
 * + init_kv_i4 / append_kv_i4 (quarot/kernels/bindings.cpp:140-260, flashinfer/page.cuh:120,167). */
int qr_kv_append_i4(void* kv_data, void* kv_param, const int32_t* kv_indptr, const int32_t* kv_indices,
                    const int32_t* last_page_offset, const void* k, const void* v, const int32_t* append_indptr,
                    int64_t tokens, int batch, int num_layers, int layer, int num_heads, int page_size, int head_dim,
                    int hadamard_k, void* stream);

/* qr_kv_decode_i4: o[b, h, :] = softmax(q[b, h, :] . K^T / sqrt(head_dim)) V over the cached tokens of sequence b, one
 * new token per sequence, keys and values dequantised on the fly; q, o [batch, heads, head_dim] fp16.  With
 * hadamard_q the query is Walsh-Hadamard transformed (and rounded to fp16) first.  Replaces batch_decode_i4
 * (quarot/kernels/bindings.cpp:115-138, flashinfer/decode.cuh:492) and the query transform of _AttentionStub.forward
 * (quarot/transformers/kv_cache.py:113-114).  Query heads and KV heads coincide, as upstream. */
int qr_kv_decode_i4(void* o, const void* q, const void* kv_data, const void* kv_param, const int32_t* kv_indptr,
                    const int32_t* kv_indices, const int32_t* last_page_offset, int batch, int num_layers, int layer,
                    int num_heads, int page_size, int head_dim, int hadamard_q, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* QUAROT_B200_H */
