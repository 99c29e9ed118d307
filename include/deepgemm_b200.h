/*
 * deepgemm_b200.h -- C ABI of libdeepgemm_b200.so
 *
 * Grouped MoE GEMM for NVIDIA B200 (sm_100a): D = bf16( a_scale * (A . B^T) * b_scale )
 * over groups ("experts"), in the row layouts the HYGON-AI/deepgemm-das library exposes
 * (masked, contiguous, compact page), for INT8, FP8-e4m3, W4A8 and BF16 operands; the same
 * kernels as a plain batched GEMM on unpacked weights (dg_dense_gemm); and the memory-bound
 * steps of an MoE layer around them: quantise + group + pad (dg_quant_group_rows, also for a
 * vLLM-style routing list: dg_group_sorted_rows), SiLU * up + requantise
 * (dg_silu_mul_quant_rows), weighted top-k sum (dg_combine_rows), weight packing.
 *
 * The reference library has no C ABI of its own: its shared object is a PyTorch
 * extension whose C++ entry points take at::Tensor.  Each function below names the
 * reference C++ entry point(s) it stands in for (path inside the reference tree:line).
 *
 * Conventions
 *   - Every pointer is a device pointer unless stated otherwise; all buffers are
 *     caller-owned; nothing is allocated, freed or synchronised inside any call,
 *     except where a function's comment says so.
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream).
 *     Work is enqueued on it and the call returns immediately.
 *   - Return value: DG_OK (0) or a negative dg_status code; dg_strerror() maps it to
 *     text.  No call prints, exits the process or launches partially.
 *   - The device that owns the buffers must be current (cudaSetDevice) in the calling
 *     thread.  Calls are thread-safe.
 */
#ifndef DEEPGEMM_B200_H_
#define DEEPGEMM_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DG_ABI_VERSION 2

/* Exported-symbol marker: the library is built with hidden default visibility. */
#if defined(__GNUC__)
#define DG_API __attribute__((visibility("default")))
#else
#define DG_API
#endif

/* Operand kinds.  The arithmetic type the tensor cores run in is given in brackets. */
typedef enum dg_kind {
  DG_KIND_I8   = 0, /* A int8,  B int8           [s8 x s8 -> s32]                    */
  DG_KIND_E4M3 = 1, /* A e4m3,  B e4m3           [e4m3 x e4m3 -> f32]                */
  DG_KIND_W4A8 = 2, /* A int8,  B packed int4    [s8 x s8 -> s32, B = nibble << 4]   */
  DG_KIND_BF16 = 3  /* A bf16,  B bf16           [bf16 x bf16 -> f32], no scales     */
} dg_kind;

typedef enum dg_scale_mode {
  DG_SCALE_PER_CHANNEL = 0, /* a_scale per row, b_scale[g][n] per output channel   */
  DG_SCALE_TENSOR_WISE = 1, /* a_scale per row, b_scale[g] one value per group     */
  DG_SCALE_NONE        = 2  /* no scales (BF16)                                    */
} dg_scale_mode;

typedef enum dg_status {
  DG_OK                 = 0,
  DG_ERR_NULL_POINTER   = -1,
  DG_ERR_BAD_KIND       = -2,
  DG_ERR_BAD_SHAPE      = -3, /* N, K, group count or row count outside what the kernels take */
  DG_ERR_BAD_ALIGNMENT  = -4, /* a base pointer is not 16-byte aligned                       */
  DG_ERR_BAD_SCALE_MODE = -5,
  DG_ERR_NO_DEVICE      = -6, /* no CUDA device, or the device is not compute capability 10.x */
  DG_ERR_CUDA           = -7, /* a CUDA runtime/driver call failed; dg_last_cuda_error() has it */
  DG_ERR_TOO_LARGE      = -8, /* a size exceeds a stated maximum                              */
  DG_ERR_BAD_ARGUMENT   = -9
} dg_status;

/* Output element types (F32: dg_dense_gemm only). */
#define DG_OUT_BF16 0
#define DG_OUT_F16  1
#define DG_OUT_F32  2

/* Words of the optional device-side status buffer (`status`, int32[DG_STATUS_WORDS]).
 * The kernels never trap: a wait that runs out records {code, block, role, detail} here,
 * the block leaves cleanly, and the host reads the words after synchronising the stream.
 * status[0] == 0 means no device-side problem was seen. */
#define DG_STATUS_WORDS 4
#define DG_DEV_OK              0
#define DG_DEV_WAIT_EXPIRED    1  /* a bounded mbarrier wait gave up */
#define DG_DEV_BAD_GROUP_INDEX 2  /* an m_indices entry was >= num_groups (row block skipped) */

/*
 * Packed weight layout ("k-block-major tiles"), produced by dg_pack_weight():
 *
 *   packed[g][kb][n][0..127]  =  the 128 bytes of row n of group g that cover
 *                                K-range [kb*BK, (kb+1)*BK)
 *
 * BK = 128 elements for 8-bit kinds, 64 for bf16, 256 int4 values for W4A8: every packed
 * row is 128 bytes.  Each (kb, n-range) tile a thread block needs is one contiguous span, so
 * a single TMA box fetches it.  Same byte count as the row-major [G][N][K] source.
 * INT8 / FP8 with K % 128 == 64 (the reference's packers take K % 64,
 * deepgemm/m_group_gemm.py:815-818): the GEMM entry points take the true K, b_packed holds
 * ceil(K / 128) blocks and the last 64 bytes of every row of the last block must be zero
 * (pack a source padded to K + 64 columns of zeros; the Python packers do that).
 * For W4A8 each 16-byte chunk j (of 8) of a 128-byte row holds, in byte i, value
 * w[32j+i] in the high nibble and w[32j+16+i] in the low nibble (two's-complement
 * nibbles), so that `x & 0xF0` and `(x << 4) & 0xF0` each yield 16 consecutive int8
 * values equal to 16*w.  Replaces the reference's W6 / marlin / HIPC-N32 layouts
 * (deepgemm/m_group_gemm.py:826-863, deepgemm/group_gemm_weight_pack.py:167-331,594-714).
 */

/* Arguments of the masked-layout grouped GEMM.
 *   for g in [0,num_groups), m in [0, masked_m[g]), n in [0,N):
 *     acc      = sum_k A[g][m][k] * B[g][n][k]            (s32 or f32)
 *     D[g][m][n] = bf16_rne( (float(acc) * a_scale[g][m]) * b_scale[g][n] )
 *   Rows m >= masked_m[g] of D are never written.  masked_m[g] is clamped to [0,max_m]. */
typedef struct dg_masked_args {
  int32_t kind;               /* dg_kind */
  int32_t scale_mode;         /* dg_scale_mode */
  const void*    a;           /* [G][max_m][K] row-major; int8 / e4m3 / bf16 */
  const void*    b_packed;    /* packed layout above */
  void*          d;           /* [G][max_m][N] bf16 */
  const float*   a_scale;     /* [G][max_m]          (NULL iff DG_SCALE_NONE) */
  const float*   b_scale;     /* [G][N] or [G]       (NULL iff DG_SCALE_NONE) */
  const int32_t* masked_m;    /* [G] valid rows per group */
  int32_t num_groups;         /* G, 1..DG_MAX_GROUPS */
  int32_t max_m;              /* rows allocated per group */
  int32_t n;                  /* N, multiple of 16 */
  int32_t k;                  /* K, multiple of 64 (256 for W4A8) */
  int32_t expected_m;         /* hint only: typical masked_m; never limits the rows computed */
  int32_t block_n;            /* 0 = choose; 128 / 256 = one-CTA tile width; 512 = two-CTA 256x256 tiles;
                                 32 / 64 = 128-wide kernel narrowed to that width (sparse routing) */
  void*          debug_acc;   /* NULL, or [G][max_m][N] of raw 32-bit accumulators (s32 / f32) */
  int32_t*       status;      /* NULL, or int32[DG_STATUS_WORDS] device status words */
  int32_t out_kind;           /* DG_OUT_BF16 (0) or DG_OUT_F16: element type of d.  The reference's W4A8 ops
                                 take half outputs (m_grouped_w4a8_gemm_nt_masked_hipc.cu:1148) */
  int32_t reserved;
  int32_t*       signal;      /* NULL, or int32 [G][ceil(max_m / 128)] completion counters, zeroed by the
                                 caller: when a tile of row block mb of group g has been stored,
                                 signal[g][mb] grows by the number of output columns the tile covers, so
                                 the rows of that block are complete once it reads N (release ordering:
                                 a consumer that acquires the value sees the rows).  The overlap hook of
                                 m_grouped_fp8_gemm_nt_maksed_low_latency.cu:1022-1029 (there +1 per tile,
                                 and switched off at run time, :1148).  INT8 / FP8 / BF16 kinds. */
} dg_masked_args;

/* Arguments of the contiguous-layout grouped GEMM.
 *   for every row i with e = m_indices[i] >= 0:
 *     D[i][n] = bf16_rne( (float(sum_k A[i][k]*B[e][n][k]) * a_scale[i]) * b_scale[e][n] )
 *   Rows are processed in blocks of 128; a block's group is m_indices of its FIRST row
 *   and the block is skipped when that is negative, so each group's rows must start on
 *   a multiple of 128 (callers pad to 256).  Rows with m_indices[i] < 0 are never written. */
typedef struct dg_contig_args {
  int32_t kind;
  int32_t scale_mode;
  const void*    a;           /* [M_total][K] */
  const void*    b_packed;
  void*          d;           /* [M_total][N] bf16 */
  const float*   a_scale;     /* [M_total] */
  const float*   b_scale;     /* [G][N] or [G] */
  const int32_t* m_indices;   /* [M_total] group id per row, -1 = padding row */
  int32_t num_groups;
  int32_t m_total;            /* <= DG_MAX_CONTIG_ROWS */
  int32_t n;
  int32_t k;
  int32_t block_n;            /* 0 = choose; 128 / 256 = one-CTA tile width; 512 = two-CTA 256x256 tiles */
  int32_t out_kind;           /* DG_OUT_BF16 (0) or DG_OUT_F16 (m_grouped_w4a8_gemm_nt_contiguous_hipc.cu:880,909) */
  void*          debug_acc;   /* NULL, or [M_total][N] raw accumulators */
  int32_t*       status;
  /* Scattered output (expert-parallel layers): when scatter_tag is not NULL, the result row i
   * is written to row (scatter_tag[i] & 0xFFFFFF) of the bf16 [.][N] buffer
   * scatter_base[scatter_tag[i] >> 24] instead of d[i]; the buffers may live on peer GPUs that
   * this GPU has mapped (plain 16-byte stores; see dg_ep_push for the tag).  `d` is then unused
   * but must still be a valid pointer.  bf16 output, N % 8 == 0. */
  const int32_t* scatter_tag;   /* NULL, or [M_total] device array */
  void* const*   scatter_base;  /* HOST array of scatter_world device pointers */
  int32_t        scatter_world; /* 1..DG_EP_MAX_WORLD */
  int32_t        group_window;  /* 0: m_indices holds group ids of this call.  w > 0: it holds ids of a wider
                                   numbering and this call covers ids [w - 1, w - 1 + num_groups) of it
                                   (b_packed / b_scale start at id w - 1): rows with other ids are skipped
                                   without a report -- one m_indices array serves several calls that each
                                   take a slice of the experts (INT8 / FP8 / BF16 kinds) */
} dg_contig_args;

/* Arguments of the compact-layout grouped GEMM: rows of all groups in one flat tensor, group g
 * owning rows [offsets[g], offsets[g] + counts[g]) with no alignment or padding between groups.
 *   D[offsets[g] + m][n] = bf16_rne((float(sum_k A[offsets[g] + m][k] * B[g][n][k]) * a_scale[.]) * b_scale[g][n])
 * for m < counts[g]; no other row of D is written.  INT8, FP8 and BF16 kinds. */
typedef struct dg_compact_args {
  int32_t kind;
  int32_t scale_mode;
  const void*    a;           /* [capacity][K] */
  const void*    b_packed;
  void*          d;           /* [capacity][N] bf16 */
  const float*   a_scale;     /* [capacity] */
  const float*   b_scale;     /* [G][N] or [G] */
  const int32_t* counts;      /* [G] rows per group */
  const int32_t* offsets;     /* [G] first row of each group */
  int32_t num_groups;
  int32_t capacity;           /* rows of a / d, <= DG_MAX_CONTIG_ROWS */
  int32_t n;
  int32_t k;
  int32_t expected_m;         /* hint only */
  int32_t block_n;            /* 0 = choose; 128 / 256; 32 / 64 as in dg_masked_args */
  void*          debug_acc;
  int32_t*       status;
} dg_compact_args;

#define DG_MAX_GROUPS      1024
#define DG_MAX_CONTIG_ROWS (4096 * 128)

/* Masked grouped GEMM.  Stands in for, in the reference:
 *   m_grouped_marlin_w8a8_gemm_nt_masked   csrc/arch/gfx936_gfx938_shared/m_grouped_w8a8_gemm_nt_masked.cu:1699-1765
 *   group_gemm_fp8_masked / masked_fp8_gemm_impl<false|true>
 *                                          csrc/arch/gfx936_gfx938_shared/low_latency_grouped_gemm.cu:5-26,
 *                                          csrc/arch/gfx936_gfx938_shared/m_grouped_fp8_gemm_nt_maksed_low_latency.cu:1037-1199
 *   m_grouped_marlin_w4a8_gemm_nt_masked[_hipc]
 *                                          csrc/arch/gfx936_gfx938_shared/m_grouped_w4a8_gemm_nt_masked.cu:214-241,
 *                                          csrc/arch/gfx936_gfx938_shared/m_grouped_w4a8_gemm_nt_masked_hipc.cu:1158-1213
 *   m_grouped_bf16_gemm_nt_masked          csrc/arch/gfx936_gfx938_shared/m_grouped_bf16_gemm_nt_masked.cu:222-262 */
DG_API int dg_masked_gemm(const dg_masked_args* args, void* stream);

/* Contiguous grouped GEMM.  Stands in for, in the reference:
 *   m_grouped_i8_contiguous::m_grouped_i8_gemm_nt_contiguous
 *                                          csrc/include/m_grouped_i8_gemm_nt_contiguous/dispatch.inc.cuh:9-27
 *   m_grouped_fp8_gemm_nt_contiguous       csrc/arch/gfx938/m_grouped_fp8_gemm_nt_contiguous/dispatch.inc.cuh:8-32
 *   m_grouped_fp8_gemm_nt_contiguous_marlin_tensor_wise
 *                                          csrc/arch/gfx938/m_grouped_fp8_gemm_nt_contiguous.cu:199-266
 *   m_grouped_marlin_w4a8_gemm_nt_contiguous_hipc
 *                                          csrc/arch/gfx936_gfx938_shared/m_grouped_w4a8_gemm_nt_contiguous_hipc.cu:861-915 */
DG_API int dg_contig_gemm(const dg_contig_args* args, void* stream);

/* Compact grouped GEMM.  Stands in for, in the reference:
 *   m_grouped_marlin_w8a8_gemm_nt_compact_masked   csrc/arch/gfx936_gfx938_shared/m_grouped_w8a8_gemm_nt_masked.cu:1767-1838
 *   m_grouped_w8a8_gemm_nt_nopad_contiguous        csrc/arch/gfx936_gfx938_shared/asm_m_grouped_w8a8_gemm_nt_contiguous.cu:595-607
 *     (rows per group given as token_per_expert; the caller passes their running sum as offsets) */
DG_API int dg_compact_gemm(const dg_compact_args* args, void* stream);

/* Arguments of the plain (batched) GEMM  d[b] = (a[b] * a_scale[b][:,None]) @ (w[b] *
 * b_scale[b][:,None])^T  with weights in their natural row-major [n][k] order (no packing),
 * computed as  out((float(acc) * a_scale[row]) * b_scale[col]). */
typedef struct dg_dense_args {
  int32_t kind;               /* DG_KIND_I8, DG_KIND_E4M3 or DG_KIND_BF16 */
  int32_t out_kind;           /* DG_OUT_BF16 / DG_OUT_F16 / DG_OUT_F32 */
  const void*  a;             /* [batch][m][k] */
  const void*  b;             /* [batch][n][k] */
  void*        d;             /* [batch][m][n] */
  const float* a_scale;       /* [batch][m], or NULL together with b_scale: no scaling */
  const float* b_scale;       /* [batch][n] */
  int32_t batch;              /* 1..DG_MAX_GROUPS */
  int32_t m;
  int32_t n;                  /* any n >= 1; n % 8 != 0 and non-bf16 outputs use scalar stores */
  int32_t k;                  /* multiple of 64 */
  int32_t block_n;            /* 0 = choose; 128 / 256 / 512 as in dg_masked_args */
  int32_t reserved;           /* must be 0 */
  void*        debug_acc;     /* NULL, or [batch][m][n] raw 32-bit accumulators */
  int32_t*     status;        /* NULL, or int32[DG_STATUS_WORDS] */
} dg_dense_args;

/* Dense GEMM on the grouped kernels (a batch entry is a group whose rows are all valid).
 * Stands in for deepgemm::fp8_gemm / fp8_gemm_hipc behind deepgemm/gemm.py:8-42 and :44-83
 * (hipBLASLt and csrc/arch/gfx938/fp8_gemm_hipc.cu there): same operands, alpha = 1, beta = 0,
 * no bias. */
DG_API int dg_dense_gemm(const dg_dense_args* args, void* stream);

/* Nibble order of a row-major int4 source [G][N][K/2]:
 *   DG_NIBBLE_HIGH_FIRST: byte j holds w[2j] in its high nibble (the reference's
 *     framework layout, deepgemm/group_gemm_weight_pack.py:594-602)
 *   DG_NIBBLE_LOW_FIRST:  byte j holds w[2j] in its low nibble. */
#define DG_NIBBLE_HIGH_FIRST 0
#define DG_NIBBLE_LOW_FIRST  1

/* Grouped GEMM on a routing list (the second-stage op of a MoE layer whose rows are named by a
 * vLLM-style sorted_token_ids / expert_ids pair): replaces the launcher behind
 * moe_w8a8_marlin_prefill_down_fp8 (csrc/arch/gfx938/moe_w8a8_marlin_prefill_down_fp8.cu:27-110,
 * device code csrc/include/moe_marlin/moe_marlin_prefill_down_fp8_device.inc.h:58-64,262-272).
 *   entry i of sorted_token_ids = (slot << 24 | token) names row = token * real_topk + slot;
 *   blocks of block_m entries share expert e = expert_ids[i / block_m];
 *   entries at or beyond *num_tokens_post_pad, with slot >= real_topk or row >= size_m are padding.
 *   e >= 0:  D[row][n] = bf16_rne( (float(sum_k A[row][k]*B[e][n][k]) * (row_weight[row]*a_scale[row])) * b_scale[e][n] )
 *   e <  0:  D[row][:] = 0          (the expert lives on another rank)
 *   rows the list never names are not written.
 * One launch: the kernel's producer fetches the rows of a tile by index and its epilogue writes
 * each result row to its place; nothing is regrouped or allocated.  Blocks of one expert should
 * follow one another (they do in a list sorted by expert): every run of blocks is tiled on its
 * own, and more than 2 * num_groups + 2 runs are refused on the device (DG_DEV_BAD_GROUP_INDEX in
 * `status`, nothing computed).  INT8 / FP8, per-channel weight scales, bf16 output, N % 8 == 0. */
typedef struct dg_sorted_args {
  int32_t kind;                        /* DG_KIND_I8 or DG_KIND_E4M3 */
  int32_t num_groups;                  /* experts held in b_packed */
  const void*    a;                    /* [size_m][K] quantised activations */
  const void*    b_packed;             /* packed layout, num_groups experts */
  void*          d;                    /* [size_m][N] bf16 */
  const float*   a_scale;              /* [size_m] */
  const float*   row_weight;           /* NULL, or [size_m]: multiplies a_scale (top-k weights) */
  const float*   b_scale;              /* [num_groups][N] */
  const int32_t* sorted_token_ids;     /* [num_sorted] */
  const int32_t* expert_ids;           /* [num_blocks] */
  const int32_t* num_tokens_post_pad;  /* device scalar: entries of the list in use */
  int32_t num_sorted;
  int32_t num_blocks;
  int32_t block_m;                     /* entries per block; num_blocks * block_m >= num_sorted */
  int32_t size_m;                      /* rows of a and d */
  int32_t real_topk;
  int32_t n;
  int32_t k;
  int32_t reserved;
  int32_t*       status;               /* NULL, or int32[DG_STATUS_WORDS] */
} dg_sorted_args;
DG_API int dg_sorted_gemm(const dg_sorted_args* args, void* stream);

/* Re-lays a row-major weight [G][N][K] (W4A8: [G][N][K/2] bytes) into the packed layout.
 * src and dst must not overlap (the Python packers pass a per-group temporary to get the
 * reference's in-place behaviour).  Stands in for the torch re-layout code of
 * pack_int8_weight_enk_to_w6_low_latency_inplace (deepgemm/m_group_gemm.py:826-863) and
 * pack_w4a8_moe_hipc_weight_inplace (deepgemm/group_gemm_weight_pack.py:691-714). */
DG_API int dg_pack_weight(int32_t kind, const void* src, void* dst, int32_t num_groups, int32_t n,
                   int32_t k, int32_t nibble_order, void* stream);

/* Inverse of dg_pack_weight (packed -> row-major, W4A8 in the given nibble order).
 * No counterpart in the reference, which never unpacks; used to verify packers. */
DG_API int dg_unpack_weight(int32_t kind, const void* src, void* dst, int32_t num_groups, int32_t n,
                     int32_t k, int32_t nibble_order, void* stream);

/* Arguments of the producer that feeds dg_contig_gemm: per-token quantisation of bf16 rows
 * fused with grouping the rows by expert, each expert's block padded to `align` rows.
 *   a_out[dest[r]][:] = quantise(rows[r][:]),  a_scale_out[dest[r]] = absmax(rows[r]) / qmax,
 *   m_indices_out[i]  = expert of the row stored at i, -1 for every other i in [0, m_cap)
 * Rows keep their input order inside an expert.  Rows with expert[r] outside [0, num_groups)
 * or that would land beyond m_cap are dropped (dest -1).  m_cap >= num_rows + num_groups *
 * (align - 1) always fits everything.  Nothing is returned to the host: launch the GEMM on
 * m_cap rows, it skips blocks whose first m_indices entry is -1. */
typedef struct dg_quant_group_args {
  int32_t kind;              /* element type of a_out: DG_KIND_E4M3 (qmax 448) or DG_KIND_I8 (qmax 127) */
  int32_t num_rows;          /* R */
  int32_t hidden;            /* H, multiple of 8, <= DG_MAX_QUANT_HIDDEN */
  int32_t num_groups;        /* 1..DG_MAX_GROUPS */
  int32_t align;             /* block alignment of each expert's rows, e.g. 256 */
  int32_t m_cap;             /* rows allocated in a_out / a_scale_out / m_indices_out */
  const void*    rows;       /* [R][H] bf16 */
  const int32_t* expert;     /* [R] group of each row */
  void*          a_out;      /* [m_cap][H] e4m3 or int8 */
  float*         a_scale_out;   /* [m_cap] */
  int32_t*       m_indices_out; /* [m_cap] */
  int32_t*       dest_out;      /* NULL, or [R] output row of each input row (-1 = dropped) */
  int32_t*       m_total_out;   /* NULL, or one int: rows in use (multiple of align, <= m_cap) */
  void*          scratch;       /* device scratch of dg_quant_group_scratch_bytes() bytes */
  size_t         scratch_bytes;
  const int32_t* src_index;     /* NULL, or [R]: input row r is rows[src_index[r]] (entries must be
                                   valid rows of `rows`), so that the top-k copies of a token can
                                   all read the token's one row */
  const float*   row_scale;     /* NULL, or [rows of `rows`]: the rows are quantised already (`rows`
                                   holds `hidden` one-byte elements of type `kind` per row, hidden a
                                   multiple of 16); they are copied and a_scale_out gets row_scale of
                                   the row read -- grouping only, e.g. after a dispatch that moved
                                   quantised rows */
} dg_quant_group_args;

#define DG_MAX_QUANT_HIDDEN 16384

/* Scratch bytes dg_quant_group_rows needs for the given problem (0 on bad arguments). */
DG_API size_t dg_quant_group_scratch_bytes(int32_t num_rows, int32_t num_groups);

/* Quantise + group + pad (four small launches on `stream`).  The reference has no kernel for
 * this step: its callers and tests do it with framework tensor ops
 * (op_test/contiguous_w8a8_int8_common.py:38-62 builds the layout, op_test/quant_utils.py:4-19
 * quantises); the arithmetic of the latter is reproduced bit for bit. */
DG_API int dg_quant_group_rows(const dg_quant_group_args* args, void* stream);

/* Arguments of the grouping step for callers that hold a vLLM-style routing list instead of an
 * expert id per row (the operands of the reference's second-stage op, see below):
 *   sorted_token_ids[i] = (top-k slot << 24) | token, in blocks of block_m entries that share
 *   the expert expert_ids[i / block_m] (-1 = expert not on this rank); entries at or beyond
 *   num_tokens_post_pad[0], with slot >= real_topk, or whose row token * real_topk + slot is
 *   >= size_m, are padding.
 * Row token * real_topk + slot of `rows` (already quantised, one byte per element) is copied to
 * a_out[dest], a_scale_out[dest] = row_scale[row] * row_weight[row], m_indices_out[dest] = its
 * expert, each expert's block padded to `align` rows as in dg_quant_group_rows;
 * dest_out[row] = dest for every row copied and -1 for every other row of `rows`. */
typedef struct dg_group_sorted_args {
  int32_t num_sorted;        /* entries of sorted_token_ids */
  int32_t block_m;           /* entries per expert_ids entry (32 in the reference) */
  int32_t size_m;            /* rows of `rows` */
  int32_t hidden;            /* bytes per row, multiple of 16 */
  int32_t num_groups;        /* 1..DG_MAX_GROUPS */
  int32_t align;
  int32_t m_cap;
  int32_t real_topk;
  const void*    rows;                /* [size_m][hidden] int8 / e4m3 */
  const float*   row_scale;           /* [size_m] */
  const float*   row_weight;          /* NULL, or [size_m] routing weights */
  const int32_t* sorted_token_ids;    /* [num_sorted] */
  const int32_t* expert_ids;          /* [ceil(num_sorted / block_m)] */
  const int32_t* num_tokens_post_pad; /* [1] */
  void*          a_out;               /* [m_cap][hidden] */
  float*         a_scale_out;         /* [m_cap] */
  int32_t*       m_indices_out;       /* [m_cap] */
  int32_t*       dest_out;            /* NULL, or [size_m] */
  int32_t*       m_total_out;         /* NULL, or one int */
  void*          scratch;             /* dg_quant_group_scratch_bytes(num_sorted, num_groups) bytes */
  size_t         scratch_bytes;
  int32_t*       src_out;             /* NULL, or [m_cap]: src_out[dest] = the row of `rows` stored at dest
                                         (the scatter_tag of dg_contig_gemm with one output buffer) */
  void*          zero_rows;           /* NULL, or a [size_m][zero_row_bytes] buffer: every row named by a
                                         block whose expert_ids entry is -1 is set to zero in it, as the
                                         reference's kernel stores zeros for such rows */
  int32_t        zero_row_bytes;      /* multiple of 16 */
  int32_t        reserved;
} dg_group_sorted_args;

/* Regroups the rows named by a sorted routing list into the contiguous layout of
 * dg_contig_gemm (four small launches).  With dg_contig_gemm and dg_combine_rows (top_k = 1,
 * src_row = dest_out) this is the reference's second-stage MoE GEMM
 * moe_marlin_w8a8_gemm2_prefill_down_fp8 (csrc/arch/gfx938/moe_w8a8_marlin_prefill_down_fp8.cu:27-110;
 * gather and routing-weight multiply at csrc/include/moe_marlin/
 * moe_marlin_prefill_down_fp8_device.inc.h:58-64,114-119, scatter at :262-272), whose kernel
 * gathers 32-row blocks itself; tcgen05 tiles want 128 rows of one expert, hence the regroup. */
DG_API int dg_group_sorted_rows(const dg_group_sorted_args* args, void* stream);

/* Arguments of the step between the gate/up GEMM and the down GEMM of an MoE layer:
 *   act[r][c]   = bf16( bf16(silu(x[r][c])) * x[r][H + c] )      (gate | up halves of a row)
 *   scale_out[r] = absmax(act[r]) / qmax,   q_out[r][c] = quantise(act[r][c] * qmax / absmax)
 * with the same per-row quantiser as dg_quant_group_rows.  Rows marked unused are skipped and
 * their outputs left untouched: m_indices[r] < 0 (contiguous layout), or row (r % max_m) >=
 * masked_m[r / max_m] (masked layout, num_rows = groups * max_m). */
typedef struct dg_act_quant_args {
  int32_t kind;              /* element type of q_out: DG_KIND_E4M3 or DG_KIND_I8 */
  int32_t num_rows;
  int32_t hidden;            /* H (columns of q_out), multiple of 8, <= DG_MAX_QUANT_HIDDEN */
  int32_t max_m;             /* rows per group when masked_m is given, else ignored */
  const void*    x;          /* [num_rows][2H] bf16 */
  const int32_t* m_indices;  /* NULL, or [num_rows] */
  const int32_t* masked_m;   /* NULL, or [num_rows / max_m] */
  void*          q_out;      /* [num_rows][H] */
  float*         scale_out;  /* [num_rows] */
} dg_act_quant_args;

/* SiLU(gate) * up fused with the per-row requantisation that feeds the down GEMM (one launch).
 * No kernel of the reference does this step: its second-stage op
 * (deepgemm/moe_marlin_prefill.py:15-56) takes activations that the serving framework has
 * already activated and quantised; the quantiser formula is op_test/quant_utils.py:4-19. */
DG_API int dg_silu_mul_quant_rows(const dg_act_quant_args* args, void* stream);

/* Arguments of the top-k reduction after the down GEMM:
 *   out[t][:] = bf16( sum_j weights[t][j] * y[src_row[t][j]][:] ),  j = 0..top_k-1 in order,
 * fp32 accumulation; entries of src_row outside [0, num_rows) contribute nothing. */
typedef struct dg_combine_args {
  int32_t num_tokens;
  int32_t top_k;
  int32_t n;                 /* columns, multiple of 8 */
  int32_t num_rows;          /* rows of y */
  const void*    y;          /* [num_rows][n] bf16 */
  const int32_t* src_row;    /* [num_tokens][top_k] */
  const float*   weights;    /* NULL (all ones), or [num_tokens][top_k] */
  void*          out;        /* [num_tokens][n] bf16 */
} dg_combine_args;

/* Weighted sum of each token's top-k expert outputs (one launch).  The reference folds the
 * routing weight into its second-stage GEMM's row scale
 * (csrc/include/moe_marlin/moe_marlin_prefill_down_fp8_device.inc.h:114-119) and leaves the
 * sum over the top-k rows to the caller; here both happen in this reduction. */
DG_API int dg_combine_rows(const dg_combine_args* args, void* stream);

/* Same operation as dg_quant_group_rows, for callers that may not allocate device memory at
 * all: code that runs inside a serving engine after its memory pool has been frozen, plugins
 * that are handed fixed buffers by a host framework, or anything that must not disturb a
 * caching allocator.  Such callers cannot provide the scratch buffer either, so this entry
 * point keeps it inside the library: a fixed array that lives in every GPU that loads the
 * library, for as long as the process runs.  `scratch` and `scratch_bytes` of the argument
 * struct are ignored; inputs and outputs are still the caller's.  The call itself never
 * allocates or frees anything, on the host or on the device.
 *
 * Limit: ceil(num_rows / 32) * num_groups + num_groups <= DG_NOALLOC_MAX_SCRATCH_INTS
 * (about 1 MiB of scratch; e.g. 32768 rows x 256 groups, or 65536 rows x 127 groups).
 * Larger problems return DG_ERR_TOO_LARGE and launch nothing.
 * The first call on each device looks up the array's device address (once, with that device
 * current); make that first call outside any CUDA stream capture.
 * All calls on a device share the one array: two calls whose kernels may overlap on the GPU
 * (different streams without an ordering between them) race on it.  Calls on one stream are
 * safe; the kernels re-initialise every scratch word they read, so nothing needs clearing
 * between calls.
 * This function has no counterpart in the reference. */
#define DG_NOALLOC_MAX_SCRATCH_INTS (262144 + 1024)
DG_API int dg_quant_group_rows_noalloc(const dg_quant_group_args* args, void* stream);

/*
 * Expert-parallel exchange over peer memory.  The reference is a single-GPU library and has no
 * counterpart for these three calls: serving frameworks shard its experts over the GPUs of a box
 * and move the routed rows themselves (all-to-all dispatch before the first grouped GEMM, the
 * reverse after the second).  Here the exchange is done by kernels of this library with plain
 * peer-to-peer stores into buffers that every rank has mapped into its address space (for
 * example with torch.distributed's symmetric memory, or CUDA IPC); no call synchronises with the
 * host, so a whole layer is enqueued without a round trip.
 *
 * Ranks 0..world-1 own num_experts / world consecutive experts each.  Per layer every rank calls,
 * on one stream: dg_ep_plan, dg_ep_push, dg_ep_barrier, its grouped GEMMs (the second with
 * scatter_tag / scatter_base so that result rows go straight home), dg_ep_barrier,
 * dg_combine_rows.  `epoch` must grow by one with every dg_ep_plan / dg_ep_barrier call of a
 * rank and be the same on all ranks for the same call.  All waits on peers are bounded (2 s): on
 * expiry status[0] = DG_DEV_WAIT_EXPIRED and the stream carries on.
 * Every peer_* argument is a HOST array of `world` device pointers, entry r being rank r's copy
 * of the buffer (entry `rank` is this rank's own).
 */
#define DG_EP_MAX_WORLD 16
/* dg_ep_plan and dg_ep_barrier consist of a posting half (publish, signal) and a waiting half
 * (wait for every rank's signal, then the rest).  With `phases` = 0 a call does both.  A test
 * that plays several ranks on ONE GPU must enqueue the posting half of every rank before any
 * waiting half (two launches per rank): kernels that wait for one another cannot be relied on to
 * run at the same time on one GPU. */
#define DG_EP_PHASE_POST 1
#define DG_EP_PHASE_WAIT 2
#define DG_EP_QUANT_E4M3 1
#define DG_EP_QUANT_I8   2

typedef struct dg_ep_plan_args {
  int32_t world;              /* ranks, 1..DG_EP_MAX_WORLD */
  int32_t rank;               /* this rank */
  int32_t num_experts;        /* E, multiple of world, <= DG_MAX_GROUPS */
  int32_t num_pairs;          /* tokens * top_k of this rank */
  int32_t align;              /* rows each expert's block is padded to in the receive buffers (e.g. 256) */
  int32_t m_cap;              /* rows of every rank's receive buffer */
  int32_t epoch;
  int32_t phases;             /* 0 = the whole call; DG_EP_PHASE_POST / DG_EP_PHASE_WAIT: one half of it */
  const int32_t* topk_ids;    /* [num_pairs] expert of each (token, slot) pair */
  void* const*   peer_counts; /* int32 [world][E] on every rank (scratch, written by all ranks) */
  void* const*   peer_flags;  /* int32 [world] on every rank, zero before the first call */
  int32_t* my_base;           /* [E] out: first row, in the owning rank's buffer, of this rank's rows of expert e */
  int32_t* cursor;            /* [E] out: zeroed */
  int32_t* m_indices;         /* [m_cap] out: m_indices of the buffer this rank receives into */
  int32_t* m_total;           /* [1] out: rows in use in it */
  int32_t* status;            /* NULL, or int32[DG_STATUS_WORDS] */
} dg_ep_plan_args;

/* Counts this rank's routed pairs per expert, exchanges the counts with every rank and derives
 * the layout of all receive buffers (one small kernel per rank; waits for every peer's counts). */
DG_API int dg_ep_plan(const dg_ep_plan_args* args, void* stream);

typedef struct dg_ep_push_args {
  int32_t world;              /* ranks, 1..DG_EP_MAX_WORLD */
  int32_t rank;               /* this rank */
  int32_t num_experts;
  int32_t num_tokens;         /* T */
  int32_t top_k;              /* <= 32 */
  int32_t row_bytes;          /* bytes per quantised row, multiple of 16, <= DG_MAX_QUANT_HIDDEN */
  int32_t m_cap;
  int32_t quantise;           /* 0: `rows` holds quantised bytes and row_scale their scales;
                                 DG_EP_QUANT_E4M3 / DG_EP_QUANT_I8: `rows` holds bf16 [T][row_bytes]
                                 elements (row_bytes % 8 == 0, <= 8192) and each token is quantised
                                 on the way out exactly as dg_quant_group_rows would (row_scale unused) */
  const void*    rows;        /* [T][row_bytes] this rank's tokens, quantised once per token */
  const float*   row_scale;   /* [T] */
  const int32_t* topk_ids;    /* [T][top_k] */
  const int32_t* my_base;     /* [E] from dg_ep_plan */
  int32_t*       cursor;      /* [E] from dg_ep_plan */
  void* const*   peer_a;      /* [m_cap][row_bytes] receive buffer of every rank */
  void* const*   peer_scale;  /* float [m_cap] of every rank */
  void* const*   peer_tag;    /* int32 [m_cap] of every rank: rank << 24 | (token * top_k + slot) */
  int32_t*       pair_dest;   /* NULL, or [T][top_k] out: row each pair was written to, -1 = dropped */
  int32_t*       status;      /* DG_DEV_BAD_GROUP_INDEX when a pair did not fit (m_cap) and was dropped */
  int32_t        local_lo;    /* with local_hi > 0: only pairs whose expert is number [local_lo, local_hi) */
  int32_t        local_hi;    /* among its owner's experts are sent (a layer pushed in several slices, so that
                                 the owner's GEMM on the first slice overlaps the push of the next); 0 = all */
  int32_t        max_blocks;  /* 0 = 8 per SM.  A push that runs beside a GEMM on another stream takes fewer
                                 (NVLink, not the grid, bounds a push: one block per SM is as fast) */
  int32_t        reserved;
} dg_ep_push_args;

/* Writes every routed row of this rank into the owning rank's receive buffer (the grouped,
 * padded A operand of that rank's dg_contig_gemm), with its scale and its return tag.  The rows
 * of one expert from one source rank are contiguous; their order within that range is not
 * fixed, which no result depends on (every output row is a function of its own row only). */
DG_API int dg_ep_push(const dg_ep_push_args* args, void* stream);

typedef struct dg_ep_barrier_args {
  int32_t world;              /* ranks, 1..DG_EP_MAX_WORLD */
  int32_t rank;               /* this rank */
  int32_t epoch;
  int32_t phases;             /* as in dg_ep_plan_args */
  void* const* peer_flags;
  int32_t*     status;
} dg_ep_barrier_args;

/* All stores this rank enqueued before the call are visible to every rank that has passed its
 * own call with the same epoch (system-scope fence, signal, bounded wait; one tiny kernel). */
DG_API int dg_ep_barrier(const dg_ep_barrier_args* args, void* stream);

/* dg_query() selectors. */
#define DG_QUERY_ABI_VERSION   0
#define DG_QUERY_SM_COUNT      1 /* multiprocessors of the current device (cached per device) */
#define DG_QUERY_MAX_SMEM      2 /* opt-in shared memory per block, bytes */
#define DG_QUERY_CC            3 /* compute capability major*10+minor of the current device */
#define DG_QUERY_LAUNCH_COUNT  4 /* kernels this library has launched in this process */
#define DG_QUERY_MAP_ENCODES   5 /* tensor maps encoded through the driver so far (a repeated call finds its
                                   maps in the calling thread's table and encodes none) */
#define DG_QUERY_MAP_REUSES    6 /* tensor maps taken from that table instead */

/* Returns the queried value (>= 0) or a negative dg_status.  Replaces the reference's
 * per-call hipGetDeviceProperties (m_grouped_w8a8_gemm_nt_masked.cu:85-89) and rocminfo
 * parsing (deepgemm/utils.py:15-50). */
DG_API int64_t dg_query(int32_t what);

/* Text for a dg_status code; never NULL.  Replaces TORCH_CHECK message strings. */
DG_API const char* dg_strerror(int code);

/* The cudaError_t (as int) behind the calling thread's most recent DG_ERR_CUDA. */
DG_API int dg_last_cuda_error(void);

#ifdef __cplusplus
}
#endif
#endif /* DEEPGEMM_B200_H_ */
