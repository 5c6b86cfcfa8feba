/*
 * rk_mx_attn.h -- C ABI of the B200 (sm_100a) MX flash-attention path.
 *
 * Drop-in boundary for the MXFP8 attention path of radiance-kernels: the MX
 * block quantizer, the tiled prefill attention (MHA / GQA / Gemma soft-cap /
 * sliding window / MXFP6 operands) and single-token decode attention over an
 * MX KV cache.  The reference exposes this path as bare-metal kernel entry
 * points whose operands are link-time arrays; every entry point below names the
 * reference interface it stands in for (file:line inside the reference tree).
 *
 * Conventions
 *   - plain C, no C++/torch types; every pointer is a DEVICE pointer unless the
 *     parameter name ends in `_host`; the caller owns all memory, nothing is
 *     retained or freed.
 *   - `stream` is a cudaStream_t passed as void* (NULL = default stream).  Calls
 *     are asynchronous on that stream.
 *   - return value: 0 = RK_OK, negative = argument error (nothing launched),
 *     positive = a cudaError_t reported by the runtime.
 *   - element codes are one byte each (6-bit formats use the low 6 bits);
 *     E8M0 scale codes are one byte per 32-element block, value 2^(code-127);
 *     callers must not pass E4M3 codes 0x7F/0xFF or scale code 0xFF (NaN in
 *     hardware, a number in the reference's decoder -- lib/golden/mx_fp_math.h
 *     :227-236,249-252); the quantizer never emits them.
 */
#ifndef RK_MX_ATTN_H_
#define RK_MX_ATTN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define RK_API __attribute__((visibility("default")))
#else
#define RK_API
#endif

#define RK_OK 0
#define RK_ERR_NULL_POINTER (-1)
#define RK_ERR_BAD_SHAPE (-2)       /* d not in {64,128,256}, H % H_kv != 0, sizes <= 0 ... */
#define RK_ERR_BAD_FORMAT (-3)      /* unknown / unsupported element format or layout */
#define RK_ERR_WORKSPACE (-4)       /* workspace missing, too small or misaligned */
#define RK_ERR_MISALIGNED (-5)      /* a tensor pointer breaks the 16-byte alignment TMA needs */
#define RK_ERR_UNSUPPORTED (-6)     /* valid request this build does not implement */
#define RK_ERR_NO_DEVICE (-7)       /* no sm_100 device / driver entry point missing */
#define RK_ERR_KERNEL_TIMEOUT (-8)  /* a bounded device-side wait gave up (see rk_last_device_status) */
#define RK_ERR_TOO_LARGE (-9)       /* request exceeds a fixed capacity (no-allocation entry points) */

/* Element formats (codes as in OCP MX; E4M3 and E3M2 decode exactly as
 * lib/golden/mx_fp_math.h:227-236,256-264). */
enum { RK_FMT_E4M3 = 0, RK_FMT_E5M2 = 1, RK_FMT_E2M3 = 2, RK_FMT_E3M2 = 3,
       RK_FMT_E2M1 = 4 /* FP4: lib/golden/mx_fp_math.h:238-246 (fp4_e2m1_decode), kernels/flash_attention_mx_gqa/fp6_attn_relerr.py:31-36 */ };

/* Where V's block-32 scales run.
 * KEYS: scales [B][H_kv][ceil(S_kv/32)][d], the reference's own V layout
 *       (kernels/flash_attention_mx_gqa/fa_gen_data.py:106-117: V_scales[Bk/32][d]).
 * D   : scales [B][H_kv][S_kv][d/32], what a KV cache quantized "along d" holds;
 *       V is re-blocked along the keys into the workspace before the kernel runs. */
enum { RK_V_SCALES_ALONG_KEYS = 0, RK_V_SCALES_ALONG_D = 1 };

/* Where the block scales of a [S][d] matrix (blocks of 32 along d) sit in memory.
 * ROWMAJOR  : [batch][S][d/32].
 * GROUPMAJOR: [batch][d/32][S], the reference's own order for Q (QK_A_scales_row[FA_GK][FA_SQ] per head,
 *             kernels/flash_attention_mx/gen_data.py:82-83; kernels/flash_attention_mx_gqa/fa_gen_data.py:101-104).
 * SF_ATOMS  : [batch][ceil(S/128)][ceil(d/128)][512]: the scale-factor atoms the tensor core reads.  The atom of
 *             row tile t and 128-column chunk c holds, at byte (r%32)*16 + (r/32)*4 + kb, the scale of row
 *             128t + r, columns 128c + 32kb .. +31.  rk_mx_quantize_ex writes it; passing it to rk_attn_prefill
 *             saves the two re-tiling launches of every call.  For V scaled along the keys the atom of key tile t
 *             and chunk c holds, at byte (n%32)*16 + (n/32)*4 + kb, the scale of column 128c + n, keys
 *             128t + 32kb .. +31 (rk_mx_quantize_keys_ex writes it).  Bytes that belong to rows or columns past
 *             the matrix edge must hold a finite scale code (the quantizers write 0x7F there). */
enum { RK_SCALES_ROWMAJOR = 0, RK_SCALES_GROUPMAJOR = 1, RK_SCALES_SF_ATOMS = 2 };

RK_API const char* rk_error_string(int code);
RK_API int rk_version(void);

/* ---------------------------------------------------------------------------
 * MX block quantizer.  Replaces kernel_body/quantize_one_block of
 * kernels/simt_quant/kernel.cpp:95-137 (KernelArgs{X,out,nblocks} :83-87) and
 * its golden lib/golden/golden.py:118-170.  Bit-exact with both.
 *   x      fp32 [rows][cols] row-major
 *   codes  u8   [rows][cols]
 *   scales u8   [rows][cols/32]           (rk_mx_quantize: blocks along cols)
 *          u8   [batch][ceil(rows/32)][cols]  (rk_mx_quantize_keys: blocks run
 *               down the rows of each [rows][cols] matrix of the batch -- how
 *               the reference quantizes V, kernels/flash_attention_mx/gen_data.py:77)
 * cols must be a multiple of 32 for rk_mx_quantize.
 * ------------------------------------------------------------------------- */
RK_API int rk_mx_quantize(const float* x, int64_t rows, int64_t cols, int fmt,
                   uint8_t* codes, uint8_t* scales, void* stream);
/* Same as rk_mx_quantize with a bf16 input [rows][cols] (the dtype projections usually produce): each value is
 * widened exactly to fp32 and takes the same path, at 2 instead of 4 input bytes per element. */
RK_API int rk_mx_quantize_bf16(const void* x_bf16, int64_t rows, int64_t cols, int fmt,
                               uint8_t* codes, uint8_t* scales, void* stream);
RK_API int rk_mx_quantize_keys(const float* x, int64_t batch, int64_t rows, int64_t cols, int fmt,
                        uint8_t* codes, uint8_t* scales, void* stream);
/* The same two quantizers with a choice of scale layout (RK_SCALES_*), per matrix of a batch:
 *   rk_mx_quantize_ex      x fp32 (x_is_bf16 = 0) or bf16 (1) [batch][S][d], blocks along d; codes [batch][S][d];
 *                          scales in `scale_layout` (all three).  d a multiple of 32.
 *   rk_mx_quantize_keys_ex x fp32 [batch][rows][cols], blocks down the rows; scales ROWMAJOR
 *                          ([batch][ceil(rows/32)][cols]) or SF_ATOMS.
 * SF_ATOMS output is 16-byte aligned atoms of 512 bytes; the call first fills bytes of ragged edges with 0x7F. */
RK_API int rk_mx_quantize_ex(const void* x, int x_is_bf16, int64_t batch, int64_t S, int64_t d, int fmt,
                             uint8_t* codes, uint8_t* scales, int scale_layout, void* stream);
RK_API int rk_mx_quantize_keys_ex(const float* x, int64_t batch, int64_t rows, int64_t cols, int fmt,
                                  uint8_t* codes, uint8_t* scales, int scale_layout, void* stream);

/* Import of the reference's streaming K operand.  Its generator emits K per KV head and key block j as a
 * transposed tile K^T [d][Bk] (QK_B_blocks[(kv*NBU + j)*FA_D][FA_BK]) with group-major scales
 * (QK_B_scales_blocks[(kv*NBU + j)*FA_GK][FA_BK]) -- kernels/flash_attention_mx_gqa/fa_gen_data.py:110-117 -- a
 * layout made for the Gemmini DMA.  This call turns `heads` x `n_blocks` such tiles into the natural layout
 * rk_attn_prefill takes: k codes [heads][n_blocks*Bk][d], k scales [heads][n_blocks*Bk][d/32] (row-major).
 * Bk and d multiples of 32. */
RK_API int rk_import_kt_blocks(const uint8_t* kt_blocks, const uint8_t* kt_scale_blocks, int64_t heads,
                               int32_t n_blocks, int32_t Bk, int32_t d, uint8_t* k_codes, uint8_t* k_scales,
                               void* stream);

/* Re-block V from scales along d to scales along the keys (decode exactly, then
 * the same block rule down each column).  No reference counterpart: the
 * reference generates V already blocked along the keys.
 *   codes [batch][S][d], scales [batch][S][d/32] -> out_codes [batch][S][d],
 *   out_scales [batch][ceil(S/32)][d]. */
RK_API int rk_mx_rebase_v(const uint8_t* codes, const uint8_t* scales, int64_t batch, int64_t S, int64_t d,
                   int fmt, uint8_t* out_codes, uint8_t* out_scales, void* stream);

/* Dense 6-bit / 4-bit operands, the form the tensor maps of the attention kernel read (a KV cache
 * kept in E2M3, E3M2 or E2M1 is prepared once and used by many calls).  No reference counterpart: the
 * reference's FP6 kernels keep one code per byte (kernels/flash_attention_mx_fp6/README.md:14-18).
 *   rows form (Q, K): codes [rows][d] one per byte -> [rows][dp * bits / 8] bytes, dp = d rounded up to
 *     128, codes little-endian bit-packed in order (code i of a row at bits [i*bits, (i+1)*bits)),
 *     padding codes 0;
 *   transposed form (V, blocked along the keys): codes [batch][S][d] -> [batch][d][Sp * bits / 8] bytes,
 *     Sp = S rounded up to 128, the keys of one column packed the same way.
 * d must be a multiple of 16; fmt one of RK_FMT_E2M3, RK_FMT_E3M2 (bits = 6), RK_FMT_E2M1 (bits = 4). */
RK_API size_t rk_mx_packed_rows_bytes(int64_t rows, int64_t d, int fmt);
RK_API int rk_mx_pack_rows(const uint8_t* codes, int64_t rows, int64_t d, int fmt, uint8_t* out, void* stream);
RK_API size_t rk_mx_packed_vt_bytes(int64_t batch, int64_t S, int64_t d, int fmt);
RK_API int rk_mx_pack_vt(const uint8_t* v_codes, int64_t batch, int64_t S, int64_t d, int fmt, uint8_t* out, void* stream);

/* ---------------------------------------------------------------------------
 * Prefill attention.  Replaces fa_entry(void*, tid, threads, block_id) of
 * kernels/flash_attention_mx_gqa/kernel.cpp:91-184 (GQA + causal),
 * kernels/flash_attention_mx/kernel.cpp:3768 (single head) and
 * kernels/flash_attention_mx_gemma/kernel.cpp (soft-cap, sliding window); the
 * fields carry what those kernels read from include/fa_data.h
 * (QK_A_in, QK_A_scales_row, QK_B_blocks, QK_B_scales_blocks, V_in, V_scales,
 * FA_SQ FA_SK FA_D FA_NQ FA_NKV FA_QPOS0 FA_SOFTMAX_SCALE FA_ATTN_SOFTCAP
 * FA_WINDOW -- kernels/flash_attention_mx_gemma/fa_gen_data.py:148-192),
 * generalised by a batch dimension.
 * ------------------------------------------------------------------------- */
typedef struct rk_prefill_args {
  const uint8_t* q;        /* codes [B][H][S_q][d]      (QK_A_in) */
  const uint8_t* k;        /* codes [B][H_kv][S_kv][d]  (QK_B_blocks, natural [key][d] order) */
  const uint8_t* v;        /* codes [B][H_kv][S_kv][d]  (V_in) */
  const uint8_t* q_scale;  /* E8M0, [B*H] matrices [S_q][d] in q_scale_layout (QK_A_scales_row as it lies = GROUPMAJOR) */
  const uint8_t* k_scale;  /* E8M0, [B*H_kv] matrices [S_kv][d] in k_scale_layout */
  const uint8_t* v_scale;  /* E8M0, axis chosen by v_scale_axis, layout by v_scale_layout */
  void* o;                 /* bf16 [B][H][S_q][d]  (O_GMEM, kernels/flash_attention_mx_gqa/kernel.cpp:50,115) */
  float* lse;              /* optional fp32 [B][H][S_q]: running max + log(l), natural log */
  int32_t B, H, H_kv, S_q, S_kv, d;   /* d in {64,128,256}; H % H_kv == 0 */
  int32_t q_pos0;          /* global position of query row 0 (FA_QPOS0) */
  int32_t causal;          /* mask key_pos > q_pos0 + row */
  int32_t window;          /* >0: also mask key_pos <= q_pos - window (FA_WINDOW); 0 = off */
  float softcap;           /* >0: s <- cap*tanh(s/cap) after the softmax scale, before mask/max; 0 = off */
  float softmax_scale;     /* FA_SOFTMAX_SCALE; 0 selects 1/sqrt(d) */
  int32_t q_fmt, kv_fmt;   /* RK_FMT_*; 6-bit (E2M3 / E3M2) and 4-bit (E2M1) codes come one per byte and are packed into the
                              workspace for the tensor core, unless q_packed / kv_packed say that they are dense
                              already; P is always E4M3 as in the reference */
  int32_t v_scale_axis;    /* RK_V_SCALES_ALONG_KEYS | RK_V_SCALES_ALONG_D */
  int32_t block_n;         /* keys per online-softmax step; 0 = default.  On return from
                              rk_attn_prefill_block_n() the value the kernel uses (128). */
  int32_t q_scale_layout;  /* RK_SCALES_ROWMAJOR (0) | RK_SCALES_GROUPMAJOR | RK_SCALES_SF_ATOMS */
  int32_t k_scale_layout;  /* same three */
  int32_t v_scale_layout;  /* RK_SCALES_ROWMAJOR (0), or RK_SCALES_SF_ATOMS with v_scale_axis = RK_V_SCALES_ALONG_KEYS */
  void* workspace;         /* >= rk_attn_prefill_workspace_bytes(), 256-byte aligned */
  size_t workspace_bytes;
  int32_t q_packed;        /* 1: q is the dense form written by rk_mx_pack_rows (6- and 4-bit formats only) */
  int32_t kv_packed;       /* 1: k is the dense form of rk_mx_pack_rows and v the dense transposed form of
                              rk_mx_pack_vt (6- and 4-bit formats only; V blocked along the keys,
                              v_scale_axis = RK_V_SCALES_ALONG_KEYS).  With scale-factor atoms for all three
                              scale tensors such a call launches the attention kernel alone.  Not taken by
                              rk_attn_prefill_host. */
} rk_prefill_args;

/* Keys per online-softmax step the kernel uses (results depend on it; an oracle
 * must be run with the same value). */
RK_API int rk_attn_prefill_block_n(const rk_prefill_args* a);
RK_API size_t rk_attn_prefill_workspace_bytes(const rk_prefill_args* a);
RK_API int rk_attn_prefill(const rk_prefill_args* a, void* stream);

/* Same call with HOST buffers: copies q/k/v and their scales to the device arena
 * (256-byte aligned, at least rk_attn_prefill_host_arena_bytes()), runs rk_attn_prefill and
 * copies O (and lse) back.  The reference's counterpart is the host stub that
 * releases the kernel and waits for it (kernels/flash_attention_mx_gqa/host.cpp:5-18).
 * The (batch, KV head) units are independent, so the call is cut into a few (five) chunks of whole
 * units and pipelined: while one chunk is computed on `stream`, the next one crosses the bus on
 * a copy stream of the library and the previous one's output goes back on a second one (host
 * buffers should be pinned for the copies to overlap).  Results are those of rk_attn_prefill.
 * Synchronises the stream before returning; calls from several host threads take turns. */
RK_API size_t rk_attn_prefill_host_arena_bytes(const rk_prefill_args* a_host);
RK_API int rk_attn_prefill_host(const rk_prefill_args* a_host, void* device_arena, size_t arena_bytes, void* stream);

/* ---------------------------------------------------------------------------
 * Decode attention over an MX KV cache (one query token per sequence), split
 * over the keys with an fp32 log-sum-exp combine.  The reference has no decode
 * attention kernel (its nearest is the batched projection GEMV
 * kernels/gemv_batched_fp8_m128/kernel.cpp:1-33); semantics are the prefill
 * path at S_q = 1, q_pos = kv_len-1, GQA head map of
 * kernels/flash_attention_mx_gqa/kernel.cpp:109-115, no P requant.
 * ------------------------------------------------------------------------- */
typedef struct rk_decode_args {
  const void* q;           /* bf16 [B][H][d] */
  const uint8_t* k;        /* codes [B][H_kv][L][d] */
  const uint8_t* v;        /* codes [B][H_kv][L][d] */
  const uint8_t* k_scale;  /* E8M0 [B][H_kv][L][d/32] */
  const uint8_t* v_scale;  /* E8M0 [B][H_kv][L][d/32] */
  const int32_t* kv_len;   /* [B] valid keys per sequence, or NULL for L everywhere */
  void* o;                 /* bf16 [B][H][d] */
  float* lse;              /* optional fp32 [B][H] */
  int32_t B, H, H_kv, L, d;   /* d == 128; H / H_kv in {1,2,4,8} */
  float softmax_scale;     /* 0 selects 1/sqrt(d) */
  int32_t kv_fmt;          /* RK_FMT_*: what rk_kv_cache_append writes, one code per byte.  E4M3 and E5M2 go through the
                              tensor-core kernel; E2M3, E3M2 and E2M1 caches are converted by the threads of the
                              mma.sync kernel (about two thirds of its speed).  rk_attn_decode_noalloc: E4M3 only */
  int32_t num_splits;      /* 0 = choose; otherwise 1..64 */
  void* workspace;         /* >= rk_attn_decode_workspace_bytes(), 16-byte aligned */
  size_t workspace_bytes;
} rk_decode_args;

RK_API int rk_attn_decode_num_splits(const rk_decode_args* a);
RK_API size_t rk_attn_decode_workspace_bytes(const rk_decode_args* a);
RK_API int rk_attn_decode(const rk_decode_args* a, void* stream);

/* RoPE fused with the block quantizer: the producer step right before attention, without the fp32 round trip of
 * the rotated tensor through HBM.  x is fp32 [rows][d] (rows = any flattening of batch, head, token; d a
 * multiple of 64); row r is rotated with row pos[r] of the half-width caches cos_half / sin_half [n_pos][d/2]
 * (pos a device array, entries in [0, n_pos)), or with row pos0 + r % seq_len when pos is NULL (the layout
 * [batch][head][seq_len][d]).  Rotation is the rotate-half form of lib/golden/golden.py:229-236 (rope_apply, the
 * golden of kernels/rope_qkv_fused), every product and sum rounded to fp32 on its own; quantization as
 * rk_mx_quantize.  Outputs: codes [rows][d], scales [rows][d/32]. */
RK_API int rk_rope_mx_quantize(const float* x, int64_t rows, int32_t d, const int32_t* pos, int32_t seq_len, int32_t pos0,
                               const float* cos_half, const float* sin_half, int32_t n_pos, int32_t fmt,
                               uint8_t* codes, uint8_t* scales, void* stream);

/* RMSNorm fused with the block quantizer: the prologue of the QKV projection, without the fp32 round trip of the
 * normalized activation through HBM.  Replaces phase 0 of kernels/rmsnorm_qkv_fused/kernel.cpp:96-110 (golden:
 * rmsnorm, lib/golden/golden.py:203-216) and is bit-exact with that golden: sum of squares in index order, every
 * product and sum rounded to fp32 on its own, rms = 1 / sqrt(ss / K + eps), y = (x * rms) * gamma.
 *   x fp32 (x_is_bf16 = 0) or bf16 (1) [rows][K], K a multiple of 32; gamma fp32 [K]; codes [rows][K] (16-byte aligned);
 *   scales [rows][K/32].  unit_scale = 0: y is MX-quantized along K as rk_mx_quantize does; unit_scale = 1: no block
 *   scale, code = E4M3(y) and every scale byte 0x7F -- what the reference kernel writes (gen_data.py:33-41). */
RK_API int rk_rmsnorm_mx_quantize(const void* x, int x_is_bf16, int64_t rows, int32_t K, const float* gamma, float eps,
                                  int32_t fmt, int32_t unit_scale, uint8_t* codes, uint8_t* scales, void* stream);

/* MX matmul in the accumulate semantics of the MX-Gemmini mesh: C = A . B with E8M0 scales per 32-element K group,
 * rounded where the hardware rounds.  Replaces the mesh call of the reference's GEMM and batched-decode projection
 * kernels (the kernels/gemm_mxgemmini family, kernels/gemv_batched_fp8_m128/kernel.cpp:1-33) and is bit-exact with their
 * golden program lib/golden/mx_golden.cpp:114-144 (16 accumulator stages per 16-deep K step, products truncated to 3
 * fraction bits and saturated at 448, bf16 accumulation across K steps), overflow to inf / NaN included.
 *   a E4M3 codes [M][K] (A_in), b E4M3 codes [K][N] (B_in), a_scales E8M0 [K/32][M] (A_scales_row),
 *   b_scales E8M0 [K/32][N] (B_scales_col), c_bf16 [M][N] (C_out_bf16).  M, N multiples of 16, K of 32; a 16-byte aligned.
 * Only the fp8 form of the golden is provided (its LUT-indexed fp6 and nibble-packed fp4 forms are mesh-specific). */
RK_API int rk_mx_gemm_hw(const uint8_t* a, const uint8_t* b, const uint8_t* a_scales, const uint8_t* b_scales, int32_t M,
                         int32_t N, int32_t K, void* c_bf16, void* stream);

/* Append one token to an MXFP8 / MXFP6 KV cache so that decode can run in a loop: for every batch b and KV
 * head, the new K row and the new V row (fp32 [B][H_kv][d], device memory) are quantized in blocks of 32
 * along d with the rule of rk_mx_quantize and stored as row pos[b] of the cache (codes [B][H_kv][L][d],
 * scales [B][H_kv][L][d/32]; pos is a device array of B int32).  A position outside [0, L) leaves that
 * sequence untouched.  The reference has no KV cache (its attention kernels read link-time arrays,
 * kernels/flash_attention_mx_gemma/fa_gen_data.py:148-192); the quantization is that of
 * kernels/simt_quant/kernel.cpp:95-129 applied to one row. */
RK_API int rk_kv_cache_append(const float* k_new, const float* v_new, int32_t B, int32_t H_kv, int32_t L, int32_t d,
                              const int32_t* pos, int32_t fmt, uint8_t* k_codes, uint8_t* k_scales,
                              uint8_t* v_codes, uint8_t* v_scales, void* stream);

/* Decode for callers that cannot allocate device memory at the call site -- a plugin running inside a
 * memory pool it does not own, a serving loop whose allocator is locked while a step is in flight, a
 * host that must leave a caching allocator's bookkeeping untouched.  It has no counterpart in the
 * reference.  Same arguments and results as rk_attn_decode, except that `workspace` / `workspace_bytes`
 * are ignored: the split partials go to a fixed array of RK_DECODE_NOALLOC_SCRATCH_BYTES (5 MiB) inside
 * the library image (every GPU that loads the library holds it until exit).
 * The call allocates nothing, neither directly nor through a library.
 *   - B * H * splits * 130 floats must fit the array.  With num_splits == 0 the split count is lowered
 *     until it fits; if even one split does not fit, or a requested num_splits does not, the call
 *     returns RK_ERR_TOO_LARGE and launches nothing.
 *   - The first call on each device looks up the array's device address (no allocation, but a runtime
 *     query): make that first call outside any stream capture.
 *   - All calls on a device share the array.  Nothing in it has to start at zero (every slot a launch
 *     reads it has written first), but two calls that overlap on the GPU (different streams) would
 *     overwrite each other's partials: serialise them.
 *   - A bounded wait that gives up is recorded in a status word of its own inside the library image
 *     (rk_last_device_status() does not see it); it is sticky: later no-allocation launches on that
 *     device return without computing until rk_attn_decode_noalloc_status() has read and cleared it. */
#define RK_DECODE_NOALLOC_SCRATCH_BYTES (5u << 20)
RK_API int rk_attn_decode_noalloc(const rk_decode_args* a, void* stream);
/* Status word of the no-allocation decode path on the current device: 0 = clean, otherwise the code of the
 * wait that gave up (the output of that call and of every later one is not valid).  Synchronises the device,
 * clears the word, allocates nothing.  No counterpart in the reference. */
RK_API int rk_attn_decode_noalloc_status(void);

/* ---------------------------------------------------------------------------
 * Sharding over GPUs (one process per GPU).  The path has no exchange step: (batch, KV head) units are
 * independent (the head map of kernels/flash_attention_mx_gqa/kernel.cpp:109-115 keeps a KV head and its query
 * heads together).  rk_shard_units gives rank `rank` of `world` its contiguous block [*begin, *end) of
 * n_units = B * H_kv units (the first n_units % world ranks get one unit more).  A block of n units is a problem
 * of its own for rk_attn_prefill / rk_attn_decode: B = n, H = H / H_kv, H_kv = 1, pointers advanced to the block's
 * first unit (query heads [begin * H/H_kv, end * H/H_kv) of the flattened [B*H] axis).  Gathering O on one
 * device, where a caller wants that, is the caller's collective (the blocks are contiguous in [B][H][S][d]).
 * ------------------------------------------------------------------------- */
RK_API int rk_shard_units(int64_t n_units, int32_t rank, int32_t world, int64_t* begin, int64_t* end);

/* Profiling aid (no reference counterpart): when both are non-NULL, the next rk_attn_prefill /
 * rk_attn_decode calls record cudaEvent_t `before` right before their main kernel (the tiled
 * attention kernel / the split-KV kernel) and `after` right after it, on the call's stream, so a
 * caller can time that kernel apart from the preparation passes.  Pass NULLs to switch it off. */
RK_API void rk_profile_set_events(void* before, void* after);   /* process-wide: set it while no other thread is in a call */

/* Status word of the last kernel that ran on the current device: 0 = clean;
 * non-zero = a bounded wait inside a kernel gave up (the code says which) and
 * the output of that launch is not valid.  Synchronises the device. */
RK_API int rk_last_device_status(void);

#ifdef __cplusplus
}
#endif
#endif /* RK_MX_ATTN_H_ */
