/*
 * gnk.h - C ABI of libgnk.so: hand-written sm_100a kernels behind the gn_kernels Python API.
 *
 * Every entry point takes plain device pointers and sizes, launches on the given CUDA
 * stream, allocates no device memory, never throws and never exits; it returns GNK_OK (0)
 * or a negative GNK_ERR_* code (gnk_strerror gives the text).  Outputs are caller-allocated.
 * Entry points may be called from several host threads; encoded TMA descriptors are kept in a
 * small mutex-guarded host cache.  Only the gnk_debug_* hooks at the end are process-wide.
 * Kernels whose warps wait on hardware barriers bound every wait; a wait that runs out
 * is recorded in a sticky device status word readable with gnk_device_status().
 *
 * "Replaces" comments name the upstream gn_kernels interface (file:line in the upstream
 * tree) that a maintainer would rebind to the entry point.
 *
 * Conventions: matrices are row-major with the reduction dimension contiguous
 * (A is [M,K], "Bt" is [N,K]; the product is A * Bt^T); ld* are row strides in ELEMENTS
 * of the stored type (bytes for packed FP4).  stream is a cudaStream_t.
 */
#ifndef GNK_H_
#define GNK_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GNK_VERSION 100

typedef void* gnk_stream_t; /* cudaStream_t */

enum gnk_status {
  GNK_OK = 0,
  GNK_ERR_BAD_ARG = -1,      /* null pointer, non-positive size, unknown enum */
  GNK_ERR_BAD_SHAPE = -2,    /* divisibility rule of the op violated */
  GNK_ERR_BAD_ALIGN = -3,    /* pointer or stride not aligned as the op needs */
  GNK_ERR_ARCH = -4,         /* current device is not compute capability 10.x */
  GNK_ERR_CUDA = -5,         /* a CUDA runtime / driver call failed (see gnk_last_cuda_error) */
  GNK_ERR_TIMEOUT = -6,      /* a bounded device-side wait ran out (from gnk_device_status) */
  GNK_ERR_TOO_LARGE = -7,    /* size beyond a documented maximum */
  GNK_ERR_UNSUPPORTED = -8   /* valid request this build has no kernel for */
};

enum gnk_dtype { GNK_BF16 = 0, GNK_F16 = 1, GNK_F32 = 2 };
enum gnk_qkind { GNK_Q_INT8 = 0, GNK_Q_E4M3 = 1, GNK_Q_E5M2 = 2, GNK_Q_E2M1 = 3, GNK_Q_BF16 = 4, GNK_Q_F16 = 5 };
enum gnk_mx_rule { GNK_MX_OCP = 0, GNK_MX_NV = 1 };
enum gnk_out { GNK_OUT_BF16 = 0, GNK_OUT_I32 = 1 };

int gnk_version(void);
const char* gnk_strerror(int status);
/* Text of the last CUDA error seen by this library on the calling thread ("" if none). */
const char* gnk_last_cuda_error(void);
/* Reads (and optionally clears) the sticky device status word of the current device.
 * Synchronises the device.  *status is GNK_OK or GNK_ERR_TIMEOUT; *detail identifies the
 * kernel role and barrier that gave up (0 if none). */
int gnk_device_status(int* status, uint32_t* detail, int clear);

/* ------------------------------------------------------------------ quantizers ---- */

/* Bytes of device scratch gnk_absmax needs for n elements. */
size_t gnk_absmax_scratch_bytes(int64_t n);
/* out[0] = max |x[i]| / divisor as fp32 (IEEE division; divisor 1 gives the plain maximum,
 * 2688 = 448*6 gives the NVFP4 tensor scale).  x: contiguous n elements of `dtype`.  scratch: device
 * memory of gnk_absmax_scratch_bytes(n) bytes, its first 4 bytes zero on entry (the
 * kernel restores that before it ends, so one zero-initialised buffer can be reused by
 * calls that do not overlap).
 * Replaces: the torch reduction `x.abs().amax()` callers run before
 * gn_kernels/quant_utils.py:162 / tests/test_quant_utils.py:10. */
int gnk_absmax(const void* x, int dtype, int64_t n, float divisor, float* out, void* scratch,
               gnk_stream_t stream);

/* gnk_absmax without caller-provided scratch.  No counterpart in the reference: it exists for
 * hosts that cannot allocate on the library's behalf - a runtime whose arena already owns all
 * device memory, or a binding that passes nothing but input/output pointers - and for which a
 * cudaMalloc inside the call would be impossible or would stall a serving loop.  The scratch is a
 * fixed 8 KB array inside the library image (each GPU that loads the library carries it until
 * exit); the call allocates nothing.  Limit: n <= gnk_absmax_static_max_elems() (2^32), larger n
 * returns GNK_ERR_TOO_LARGE.  The first call on a device looks up the array's device address;
 * make that first call before any stream capture begins.  All calls share the one array, so two
 * calls that overlap on the GPU (different streams, or different host threads) race: serialise them.
 * Same result as gnk_absmax. */
int64_t gnk_absmax_static_max_elems(void);
int gnk_absmax_static(const void* x, int dtype, int64_t n, float divisor, float* out, gnk_stream_t stream);

/* Row-wise absmax quantizer: one fp32 scale per row of `cols` contiguous elements.
 * scale = amax/qmax (127 for INT8, 448 for E4M3); q = x / max(scale, 1e-6); INT8 rounds
 * half-to-even and clips to [-128,127]; E4M3 clips to +-448 then rounds to nearest even.
 * q: rows x cols bytes, contiguous.  scale: `rows` floats; when perm_h > 0 the row index
 * r = (b*perm_l + l)*perm_h + h is stored at (b*perm_h + h)*perm_l + l instead (the
 * [B,L,H] -> [B,H,L] transpose attention wants).  cols % 8 == 0, x 16-byte aligned rows.
 * Replaces: benchmark_attn.py:39-51 `quantize` (+ the transpose at :77-80). */
int gnk_quant_rowwise(const void* x, int dtype, int64_t rows, int64_t cols, int64_t ldx, int qkind,
                      void* q, float* scale, int64_t perm_h, int64_t perm_l, gnk_stream_t stream);

/* MX quantizer: one E8M0 exponent per 32 contiguous K elements (OCP floor rule or the
 * cuBLAS round-up rule), elements E4M3 / E5M2 (1 byte each) or E2M1 (two per byte, even
 * element in the high nibble).  sf: [M, K/32] bytes row-major, or (sf_swizzled != 0) the
 * 128x4-atom layout with rows padded to 128 and K/32 padded to 4 (padding written as 0).
 * K % 32 == 0.  Replaces: gn_kernels/quant_utils.py:93-117 `quantize_mx` (+ :21-30). */
int gnk_quant_mx(const void* x, int dtype, int64_t M, int64_t K, int64_t ldx, int qkind, int rule,
                 void* q, uint8_t* sf, int sf_swizzled, gnk_stream_t stream);

/* NVFP4 quantizer: E2M1 pairs (even element in the high nibble), one E4M3 scale per 16
 * K elements, fp32 per-tensor scale read from DEVICE memory (tensor_scale[0]).
 *   s = e4m3(clip(amax16 / max(6*ts, 1e-12), +-448));  q = e2m1(x / max(ts*f32(s), eps))
 * with IEEE fp32 divisions, so bytes and scales equal the torch reference bit for bit.
 * sf layout as in gnk_quant_mx with K/16 columns.  K % 16 == 0.
 * Replaces: gn_kernels/quant_utils.py:156-171 `quantize_nvfp4` (row-major scales) and
 * :242-252 `quantize_nvfp4_triton` (swizzled scales). */
int gnk_quant_nvfp4(const void* x, int dtype, int64_t M, int64_t K, int64_t ldx, const float* tensor_scale,
                    float eps, void* q, uint8_t* sf, int sf_swizzled, gnk_stream_t stream);

/* Scale-factor layout conversion between row-major [M, Ks] bytes and the swizzled
 * 128x4-atom layout [ceil128(M), ceil4(Ks)].  to_swizzled: pads with zeros.
 * Replaces: gn_kernels/quant_utils.py:21-36 `permute_nv_sf` / `unpermute_nv_sf`. */
int gnk_sf_swizzle(const uint8_t* src, uint8_t* dst, int64_t M, int64_t Ks, int to_swizzled, gnk_stream_t stream);

/* MX / NVFP4 dequantizer to fp32 (test and debugging aid; inverse of the two above with
 * row-major scales).  tensor_scale may be NULL (treated as 1).
 * Replaces: gn_kernels/quant_utils.py:120-152 `dequantize_mx`. */
int gnk_dequant_block(const void* q, const uint8_t* sf, int64_t M, int64_t K, int qkind, int block,
                      const float* tensor_scale, float* out, gnk_stream_t stream);

/* ------------------------------------------------------------------ matmuls ------- */

/* C[M,N] bf16 = A[M,K] bf16 * Bt[N,K]^T, fp32 accumulate.  K % 8 == 0 (16-byte rows).
 * Replaces: gn_kernels/cutedsl/sm100/sm100_mm_bf16.py:252-255 `mm`. */
int gnk_mm_bf16(const void* A, int64_t lda, const void* Bt, int64_t ldb, void* C, int64_t ldc,
                int64_t M, int64_t N, int64_t K, gnk_stream_t stream);

/* C[M,N] fp16 = A[M,K] fp16 * Bt[N,K]^T; acc_f16 = 0: fp32 accumulate, != 0: the tensor core's fp16
 * accumulator (kind::f16 with an F16 destination).  K % 8 == 0.
 * Replaces: gn_kernels/triton_mm.py:128-171 `triton_mm` for float16 inputs, `acc_dtype=torch.float16`
 * (:164-165) included. */
int gnk_mm_f16(const void* A, int64_t lda, const void* Bt, int64_t ldb, void* C, int64_t ldc,
               int64_t M, int64_t N, int64_t K, int acc_f16, gnk_stream_t stream);

/* INT8 x INT8 -> exact INT32 accumulate.  out_kind GNK_OUT_I32: C int32 = acc (scales and
 * bias must be NULL).  GNK_OUT_BF16: C = bf16(f32(acc) * scale_A[m] * scale_B[n] + bias[n])
 * evaluated in that order in fp32; any of scale_A / scale_B / bias may be NULL.
 * K % 16 == 0.  Replaces: gn_kernels/triton_mm.py:128-171 `triton_mm` for int8 inputs. */
int gnk_mm_i8(const void* A, int64_t lda, const void* Bt, int64_t ldb, void* C, int64_t ldc,
              int64_t M, int64_t N, int64_t K, const float* scale_A, const float* scale_B,
              const float* bias, int out_kind, gnk_stream_t stream);

/* E4M3 x E4M3, fp32 accumulate, same row-scaled epilogue, bf16 output.  K % 16 == 0.
 * Replaces: gn_kernels/triton_mm.py:128-171 `triton_mm` for float8_e4m3fn inputs. */
int gnk_mm_f8(const void* A, int64_t lda, const void* Bt, int64_t ldb, void* C, int64_t ldc,
              int64_t M, int64_t N, int64_t K, const float* scale_A, const float* scale_B,
              const float* bias, gnk_stream_t stream);

/* MXFP8: C bf16 = (A .* 2^(SFA-127)) * (Bt .* 2^(SFB-127))^T.  A, Bt E4M3; SFA, SFB E8M0
 * in the swizzled 128x4-atom layout ([ceil128(rows), ceil4(K/32)] bytes).  K % 32 == 0 (a K that is
 * not a multiple of 128 ends in a partly filled stage: TMA reads zeros beyond K).
 * Replaces: gn_kernels/cutedsl/sm100/sm100_mm_mxfp8.py:380-383 `mm`. */
int gnk_mm_mxfp8(const void* A, int64_t lda, const void* Bt, int64_t ldb, const uint8_t* SFA,
                 const uint8_t* SFB, void* C, int64_t ldc, int64_t M, int64_t N, int64_t K,
                 gnk_stream_t stream);

/* NVFP4: A, Bt packed E2M1 ([rows, K/2] bytes, ld in bytes), SFA/SFB E4M3 per 16, swizzled
 * ([ceil128(rows), K/16] bytes); alpha (host value, = tensor_scale_A * tensor_scale_B)
 * multiplies the fp32 accumulator before the bf16 rounding.  K % 32 == 0 (16-byte rows of packed codes).
 * Replaces: gn_kernels/cutedsl/sm100/sm100_mm_nvfp4.py:383-386 `mm` (upstream has no
 * alpha; gn_kernels/cutedsl/sm120/sm120_gated_gemm_nvfp4.py:317-319 shows where it goes). */
int gnk_mm_nvfp4(const void* A, int64_t lda, const void* Bt, int64_t ldb, const uint8_t* SFA,
                 const uint8_t* SFB, float alpha, void* C, int64_t ldc, int64_t M, int64_t N,
                 int64_t K, gnk_stream_t stream);

/* SwiGLU-gated dual NVFP4 GEMM:  out[M,N] = silu(o1) * o3,  o1 = (X W1^T) * (ts_w1 * ts_x),
 * o3 = (X W3^T) * (ts_w3 * ts_x), evaluated in fp32 as (o1 * o3) * sigmoid(o1).  X [M, K/2], W1 / W3
 * [N, K/2] packed E2M1 (ld in bytes), SFX / SFW1 / SFW3 E4M3 block scales in the swizzled layout, ts_*
 * fp32 per-tensor scales in DEVICE memory.  One tcgen05 tile holds 128 rows of W1 and the same 128
 * rows of W3, so X is read once for both products.
 *   ts_out == NULL: C is bf16 [M, N] (ldc in elements), SFC must be NULL.
 *   ts_out != NULL: the bf16 result is quantised to NVFP4 with per-tensor scale ts_out[0] in the
 *     epilogue: C = packed E2M1 [M, N/2] (ldc in bytes), SFC = E4M3 scales, swizzled layout
 *     [ceil128(M), N/16]; rows >= M of SFC are not written.  Bytes and scales equal
 *     gnk_quant_nvfp4 applied to the bf16 output of the ts_out == NULL call.
 * N % 128 == 0, K % 32 == 0.
 * Replaces: gn_kernels/cutedsl/sm120/sm120_gated_gemm_nvfp4.py:513-555 `mm` (epilogue :374-464). */
int gnk_gated_mm_nvfp4(const void* X, int64_t ldx, const uint8_t* SFX, const float* ts_x, const void* W1,
                       const uint8_t* SFW1, const float* ts_w1, const void* W3, const uint8_t* SFW3,
                       const float* ts_w3, int64_t ldw, const float* ts_out, void* C, int64_t ldc, uint8_t* SFC,
                       int64_t M, int64_t N, int64_t K, gnk_stream_t stream);

/* FP8 with DeepSeek-style scales: SFA fp32 [M, K/128] stored M-major (element (m,kb) at
 * SFA[kb*ld_sfa + m]), SFB fp32 [N/128, K/128] row-major (ld_sfb).  Each 128-deep partial
 * product is scaled by SFA[m,kb]*SFB[n/128,kb] and summed in fp32; then + add[m,n] (bf16,
 * optional) + bias[n] (bf16, optional); bf16 output.  K % 128 == 0, N % 128 == 0.
 * Replaces: gn_kernels/cutedsl/sm120/sm120_mm_fp8_1d2d.py:307-333 `mm`. */
int gnk_mm_f8_block128(const void* A, int64_t lda, const float* SFA, int64_t ld_sfa, const void* Bt,
                       int64_t ldb, const float* SFB, int64_t ld_sfb, const void* bias, const void* add,
                       int64_t ld_add, void* C, int64_t ldc, int64_t M, int64_t N, int64_t K,
                       gnk_stream_t stream);

/* ------------------------------------------------------------------ attention ----- */

/* Causal / full GQA attention forward, [B, L, H, D] layouts with D = 128 contiguous and
 * element strides given per tensor (batch, seq, head).
 *   qk_kind GNK_Q_E4M3 / GNK_Q_INT8: 8-bit codes for Q and K, with fp32 scales scale_q [B,Hq,Lq] and
 *     scale_k [B,Hkv,Lk] (both or neither; INT8 accumulates exactly in int32);
 *   qk_kind GNK_Q_BF16 / GNK_Q_F16: plain 16-bit Q and K, no scales, v_dtype must be the same type.
 *   v_dtype GNK_BF16 / GNK_F16: type of V, of P (rounded before P*V) and of O.
 *   acc16: bit 0 = Q*K^T accumulates in fp16, bit 1 = P*V accumulates in fp16 (fp16 operands only;
 *     0 = fp32 accumulation).
 *   S = (q.k) * scale_q * scale_k * D^-1/2;  causal mask j <= i + (Lk - Lq);
 *   O = softmax(S) V, softmax in fp32 with exp2; rows that see no key give 0.
 * Replaces: gn_kernels/triton_attn.py:268-325 `triton_attn` (scaled path :316-320, unscaled :322,
 * qk_fp16_acc / pv_fp16_acc :276-277,311-312). */
int gnk_attn_fwd(const void* q, const void* k, const void* v, void* o, const float* scale_q,
                 const float* scale_k, int qk_kind, int v_dtype, int acc16, int64_t B, int64_t Lq, int64_t Lk,
                 int64_t Hq, int64_t Hkv, int64_t D, const int64_t* q_strides, const int64_t* k_strides,
                 const int64_t* v_strides, const int64_t* o_strides, int causal, gnk_stream_t stream);

/* Same attention over packed variable-length sequences: q [Lq_total, Hq, D], k / v [Lk_total, Hkv, D],
 * o [Lq_total, Hq, D], all bf16 or all fp16 (qk_kind GNK_Q_BF16 / GNK_Q_F16), D = 128 contiguous,
 * strides (seq, head) in elements.  q_offsets / kv_offsets: int32 [B + 1] on the device, sequence b
 * owns rows [offsets[b], offsets[b+1]); max_q_len bounds the longest query sequence (it sizes the
 * grid).  The causal mask is lower-right aligned per sequence.  Tiles are loaded 128 rows at a time,
 * so the last tile of a sequence also reads rows of its successor: they are masked out of the
 * softmax, but a non-finite value in V there would still reach this sequence's output as NaN.
 * Replaces: gn_kernels/triton_attn.py:462-517 `triton_varlen_attn`. */
int gnk_attn_varlen_fwd(const void* q, const void* k, const void* v, void* o, const int32_t* q_offsets,
                        const int32_t* kv_offsets, int qk_kind, int acc16, int64_t B, int64_t max_q_len,
                        int64_t Lq_total, int64_t Lk_total, int64_t Hq, int64_t Hkv, int64_t D,
                        const int64_t* q_strides, const int64_t* k_strides, const int64_t* v_strides,
                        const int64_t* o_strides, int causal, gnk_stream_t stream);

/* ------------------------------------------------------------------ GEMM + RS ----- */

/* Number of int32 words the flags buffer of gnk_gemm_rs_bf16 must hold (-1 for a shape the op rejects). */
int64_t gnk_gemm_rs_flag_words(int64_t M, int64_t N, int world);

/* Host-side restatement of the device tile order (for tests of the ownership / flag arithmetic):
 * for sequence index i of `rank`, out[0..4] = {owner rank, tile row, tile column, first flag word
 * signalled, number of 128-row units signalled}.  Returns the number of tiles, -1 for a bad shape. */
int64_t gnk_gemm_rs_plan(int64_t M, int64_t N, int world, int rank, int64_t i, int32_t* out);

/* K-sharded bf16 GEMM fused with a reduce-scatter along M over NVLink peer memory.
 * x [M, K_local], w [N, K_local] (this rank's K shard).  staging[r] / flags[r]: device
 * pointers, valid on THIS GPU, to rank r's staging buffer (M * N bf16: `world` slots of
 * [M/world, N]) and flag words (zero before the first call; a call that completes leaves them zero).
 * Every rank stores each finished bf16 tile into the owner's staging slot for this rank and
 * bumps the owner's flag; the owner sums the `world` slots from its own memory in fp32 and
 * writes output [M/world, N] bf16; an exit barrier across ranks ends the call.
 * lagged_exit = 0: the call signals its peers and waits for theirs before it returns, so on return
 *   every buffer may be reused for anything, and the flag words are zero again.
 * lagged_exit = 1 (calls issued back to back on the same buffers): the call signals its peers and
 *   returns; the NEXT gnk_gemm_rs_bf16* call on the same flags waits for those signals before its
 *   first store, while its first tiles are already being computed.  `output` is complete on return
 *   as before, but staging / partial must not be written by anything else, and the last two flag words
 *   stay non-zero, until a later call with lagged_exit = 0 (or a host barrier across the ranks followed
 *   by zeroing the flags) has ended the sequence.
 * Shapes: M % (128*world) == 0 and N % 128 == 0, K_local % 8 == 0, world <= 8.  When M/world % 256 == 0 and
 * N % 256 == 0 the 2-CTA 256 x 256 tile with bulk-store epilogue runs, otherwise a 128 x 128 tile with
 * plain peer stores.  world == 1 degenerates to gnk_mm_bf16 into `output`.
 * Failure: all device-side waits are bounded by timeout_ms (0 = 20 s).  When a peer never signals, the
 * first wait of a CTA that runs out records GNK_ERR_TIMEOUT (gnk_device_status; detail = role 4,
 * barrier 6 = unit flag, 7 = exit barrier; role 3, barrier 8 = the deferred exit wait of the previous call) and every later wait of the call returns at once, so a
 * call costs at most about 2 x timeout_ms; the rows it could not reduce are left unwritten.  After
 * GNK_ERR_TIMEOUT the flag words are NOT zero: before the buffers are used again every rank must
 * finish or abandon its call, clear the status (gnk_device_status(..., clear = 1)), zero its flags
 * buffer, and meet the other ranks in a host barrier.  While the status word is set, further calls
 * skip their reductions.
 * Replaces: gn_kernels/cutedsl/sm100/sm100_gemm_rs.py:458-496 `gemm_rs`. */
int gnk_gemm_rs_bf16(const void* x, int64_t ldx, const void* w, int64_t ldw, void* const* staging,
                     int32_t* const* flags, void* output, int64_t ldo, int64_t M, int64_t N,
                     int64_t K_local, int rank, int world, uint32_t timeout_ms, int lagged_exit,
                     gnk_stream_t stream);

/* Same operation for buffers that also have an NVLink multicast address (NVSwitch systems):
 * partial[r] are the ranks' [M, N] bf16 buffers (only partial[rank] is written, by this rank),
 * partial_multicast the multicast address of the same allocation.  A finished tile stays in the
 * rank's own buffer; the owner reads every 16-byte piece once with multimem.ld_reduce (fp32 adds in
 * the switch), as upstream does (sm100_gemm_rs.py:27-60, 283-327).  flags and lagged_exit as above.
 * Replaces: gn_kernels/cutedsl/sm100/sm100_gemm_rs.py:458-496 `gemm_rs`. */
int gnk_gemm_rs_bf16_pull(const void* x, int64_t ldx, const void* w, int64_t ldw, void* const* partial,
                          const void* partial_multicast, int32_t* const* flags, void* output, int64_t ldo,
                          int64_t M, int64_t N, int64_t K_local, int rank, int world, uint32_t timeout_ms,
                          int lagged_exit, gnk_stream_t stream);

/* The reduce-scatter for E4M3 operands with tensor-wise scales (no counterpart upstream, whose gemm_rs is
 * BF16 only): x [M, K_local], w [N, K_local] float8_e4m3fn codes, alpha = scale_x * scale_w of this rank;
 * partial_r = bf16(alpha * (x_r w_r^T)), summed over the ranks in fp32.  K_local % 16 == 0, world >= 2;
 * partial_multicast NULL selects the push variant (partial[r] are then the staging buffers); everything
 * else as for gnk_gemm_rs_bf16 / gnk_gemm_rs_bf16_pull. */
int gnk_gemm_rs_f8(const void* x, int64_t ldx, const void* w, int64_t ldw, float alpha, void* const* partial,
                   const void* partial_multicast, int32_t* const* flags, void* output, int64_t ldo, int64_t M,
                   int64_t N, int64_t K_local, int rank, int world, uint32_t timeout_ms, int lagged_exit,
                   gnk_stream_t stream);

/* GEMM + all-reduce (no counterpart upstream, whose only fused collective is the reduce-scatter above): the
 * same kernel and buffers as gnk_gemm_rs_bf16_pull, but the owner of a block of rows stores each reduced
 * 16-byte piece through output_multicast, the NVLink multicast address of the ranks' [M, N] bf16 outputs
 * (row pitch ldo), so after the call every rank holds all M rows of the sum.  `output` is this rank's own
 * address of that buffer (world == 1: the plain GEMM writes there).  The exit barrier always waits. */
int gnk_gemm_ar_bf16(const void* x, int64_t ldx, const void* w, int64_t ldw, void* const* partial,
                     const void* partial_multicast, int32_t* const* flags, void* output, void* output_multicast,
                     int64_t ldo, int64_t M, int64_t N, int64_t K_local, int rank, int world, uint32_t timeout_ms,
                     gnk_stream_t stream);

/* ------------------------------------------------------------------ test hooks ---- */
/* Process-wide switches for tests and profiling; none of them changes a result.
 * Force a GEMM tile configuration (0: 2-CTA 256x256, 1: 128x256, 2: 128x128, 3: 128x64, 4: 2-CTA 256x192 for
 * the block-scaled kinds (256x256 for the others), -1: automatic),
 * cap the persistent grid (0 = no cap), record per-stage clock stamps of CTAs 0 and 1 into a
 * caller-owned device buffer of 2*2*256*3 + 4 int64 (NULL = off); the last four words are clock64 and
 * globaltimer (ns) at entry and at exit of CTA 0, whose ratio is the SM clock the launch ran at. */
int gnk_debug_force_tile(int sel);
int gnk_debug_staged(int mode); /* pair-tile epilogue: -1 default (staged), 0 direct stores from registers, 1 bulk tensor stores through shared-memory staging */
int gnk_debug_max_clusters(int n);
/* Host-side pipeline plan of a GEMM configuration (no GPU needed): kind 0 bf16/fp16, 1 int8, 2 fp8, 3 mxfp8,
 * 4 nvfp4; tile as in gnk_debug_force_tile; kd = 128-byte K slices per stage (1, or 2 / 4 with tile 3); a_rows =
 * rows of A kept per stage (8..128).  out[0] = stages, out[1] = bytes per stage, out[2] = bytes the stages may use,
 * out[3] = bytes from the start of the last stage to the end of the 128-row operand read of its last A slice. */
int gnk_debug_stage_plan(int kind, int tile, int kd, int a_rows, int32_t* out);
int gnk_debug_deep_stage(int on); /* 64-wide GEMM tile: bit 0: 1 (default) = four 128-byte K slices per pipeline stage where the shape qualifies (one tile per CTA, K bytes a multiple of 128 and >= 1024), 0 = always one; bit 1 set: launch those kernels without programmatic stream serialization */
int gnk_debug_trace(void* device_buffer);
int gnk_debug_attn_trace(void* device_buffer); /* attention: clock stamps of CTA 0, 2 tiles x 32 key tiles x 8 int64 (NULL = off) */
/* GEMM + reduce-scatter: per-CTA timeline into a caller-owned, caller-zeroed device buffer of 160 x 8
 * uint64 (globaltimer ns: start, epilogue end, reducer end, reducer wait total, MMA end, epilogue
 * store+signal total, epilogue wait total); NULL = off. */
int gnk_debug_rs_trace(void* device_buffer);

#ifdef __cplusplus
}
#endif
#endif /* GNK_H_ */
