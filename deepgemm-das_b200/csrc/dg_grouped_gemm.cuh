// Persistent, warp-specialised grouped GEMM kernel for sm_100a.
//
//   D[row][n] = bf16( (float(sum_k A[row][k] * B[g][n][k]) * a_scale[row]) * b_scale[g][n] )
//
// One thread block per SM walks a list of work items (group g, 128-row block, BN-column
// tile) derived on the device from masked_m (masked layout) or m_indices (contiguous
// layout), so groups without rows and padding row blocks produce no items at all.
//
// Roles inside a block
//   warp 0      TMA producer: one lane issues cp.async.bulk.tensor loads of the A tile
//               (128 rows x 128 bytes of K) and the weight tile (BN rows x 128 bytes of K,
//               one contiguous span of the packed weight) into a STAGES-deep ring.  Only the
//               32-row slices of A with valid rows are fetched.  With few items (sparse
//               routing) the BN = 128 instantiation narrows its tiles to 64 or 32 columns so
//               that every SM streams weights; a stage then holds several K blocks.
//   warp 1      UMMA issuer: one lane issues four tcgen05.mma (K = 32 bytes each) per
//               ring stage into one of two TMEM accumulators (128 lanes x BN columns),
//               and owns TMEM allocation.
//   warps 2..5  epilogue: tcgen05.ld of the accumulator, scale, bf16 convert, predicated
//               16-byte stores; overlaps the next item's main loop through the second
//               TMEM accumulator.
// (W4A8 has its own kernel, dg_grouped_gemm_w4.cuh.)
//
// Every wait on an mbarrier is bounded; on expiry the block records a status word and
// leaves through the common tear-down path (TMEM is always released).
//
// Semantics follow the reference kernels
//   csrc/arch/gfx936_gfx938_shared/m_grouped_fp8_gemm_nt_maksed_low_latency.cu:272-604 (masked)
//   csrc/include/m_grouped_i8_gemm_nt_contiguous/bm128_bn256_bk64_nloop4.inc.cuh:206-652 (contiguous)
// but none of their structure: those stream operands through registers on wave64 hardware.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "deepgemm_b200.h"
#include "dg_ptx.cuh"

namespace dg {

constexpr int kBM = 128;         // rows of A per tile = UMMA M
constexpr int kRowBytes = 128;   // bytes of K per shared-memory row (one swizzle span)
constexpr int kATileBytes = kBM * kRowBytes;
constexpr int kMaxSmem = 232448;  // 227 KB opt-in limit per block on sm_100

enum : int { MODE_MASKED = 0, MODE_CONTIG = 1, MODE_COMPACT = 2, MODE_SORTED = 3 };

// Where a bounded wait gave up (reported in status[2]).
enum : int {
  SITE_PRODUCER_EMPTY = 1,
  SITE_MMA_ACC_EMPTY = 2,
  SITE_MMA_FULL = 3,
  SITE_MMA_UNPACKED = 4,
  SITE_EPI_ACC_FULL = 5,
  SITE_UNPACK_FULL = 6,
  SITE_PRODUCER_DRAIN = 7
};

struct KernelParams {
  int mode;        // MODE_MASKED / MODE_CONTIG
  int scale_mode;  // dg_scale_mode
  int G;           // groups
  int M;           // max_m (masked) or M_total (contiguous)
  int N;
  int K;
  int kblocks;     // K / (elements per 128 bytes)
  int n_tiles;     // ceil(N / BN)
  int m_blocks;    // masked: ceil(max_m/128); contiguous: ceil(M_total/128)
  const int32_t* sched;  // masked_m[G], m_indices[M_total], or (compact) rows per group [G]
  const int32_t* offsets;  // compact layout only: first row of each group in the flat [M][K] tensor
  const float* a_scale;
  const float* b_scale;
  __nv_bfloat16* d;
  uint32_t* debug_acc;
  int32_t* status;
  int b_rowmajor;  // 1: weights are plain [G][N][K] rows (dense GEMM), 0: the packed layout
  int out_kind;    // 0 = bf16 output; 1 = fp16, 2 = fp32 (dense GEMM only, scalar stores)
  int split_tail;  // masked / compact: 1 = the items of a last round that is at most half full are
                   // split into two halves of BN / 2 columns
  int pack_stages;  // W4A8: stages of the packed-weight ring
  int pack_off;     // W4A8: offset of that ring in the block's shared memory
  // Contiguous layout only: when scatter_tag is given, output row i is written to row
  // (scatter_tag[i] & 0xFFFFFF) of the buffer scatter_base[scatter_tag[i] >> 24] (bf16 [.][N], on
  // this or a peer GPU) instead of d[i] -- the result rows of an expert-parallel layer go straight
  // back to the ranks their tokens came from, tile by tile, while the GEMM is still running.
  const int32_t* scatter_tag;
  void* scatter_base[16];
  // Masked layout only: per (group, 128-row block) completion counters; a finished tile adds the
  // number of columns it covers, a quarter per epilogue warp (the block is done at N).
  int32_t* signal;
  int group_window;  // contiguous layout: 0, or 1 + the id (in m_indices' numbering) of this call's group 0;
                     // entries that name a group outside the call are then skipped silently
  int wide_off;  // 0, or offset in shared memory of four 32-row x 128-byte store strips (scattered output)
  // MODE_SORTED (one-CTA kernel): the rows are named by a routing list instead of lying in place.
  // Entry i of sorted_ids packs (top-k slot << 24 | token) and names row token * real_topk + slot
  // of the [size_m][K] activation and of the [size_m][N] output; entries come in blocks of
  // block_m that share expert_ids[i / block_m] (-1: the expert lives on another rank, its rows
  // are written as zeros); entries at or beyond *num_post_pad, with slot >= real_topk or a row
  // >= size_m are padding.  A tile is 128 consecutive entries of a run of blocks with one expert:
  // the producer warp fetches the rows one by one (a one-row TMA box each, the swizzle is a
  // function of the shared-memory address, so 128 of them make the tile a 128-row box would),
  // the epilogue writes each result row to its place.  a_scale is per activation row, row_weight
  // (nullable) multiplies it.
  const int32_t* sorted_ids;
  const int32_t* expert_ids;
  const int32_t* num_post_pad;
  const float* row_weight;
  const void* gather_a;  // the [size_m][K] activation the rows are gathered from
  int block_m, num_blocks, num_sorted, real_topk, size_m;
  int tbl_groups;  // MODE_SORTED: entries per array of the schedule table (the most runs it holds)
  int narrow;  // masked / compact: 0 = tiles stay BN columns wide, 1 = the kernel may narrow them
               // (down to 32 columns) when few groups have rows, 128 / 64 / 32 = forced width
};

// Shape of one pipeline stage for a tile with `rows_valid` rows and `bn_eff` columns.  A tile
// with at most 8 / 32 / 64 valid rows (decode steps mostly have one or two rows per active
// expert) fetches only an 8 / 32 / 64-row slice of A with one TMA box of that height (the UMMA still reads 128 rows; what it reads beyond the slice is stale shared
// memory that only reaches accumulator rows nobody stores).  Several 32-row copies per tile
// were measured 18 % slower on the decode workload than one copy, so there is one box per
// height.  When both operands
// are narrow, several K blocks share one stage slot so the bytes in flight per stage stay
// near 32 KB.
struct StageShape {
  int a_rows;         // rows of A fetched per K block: 8, 32, 64 or 128 (one TMA box each)
  int kps;            // K blocks per stage
  uint32_t a_stride;  // bytes between the A sub-tiles of consecutive K blocks in a slot
  uint32_t b_stride;  // same for the weight sub-tiles
  uint32_t bytes;     // bytes fetched per K block
};
__device__ __forceinline__ StageShape stage_shape(int rows_valid, int bn_eff, int bn) {
  StageShape sh;
  sh.a_rows = rows_valid <= 8 ? 8 : (rows_valid <= 32 ? 32 : (rows_valid <= 64 ? 64 : kBM));
  sh.kps = min(bn / bn_eff, kBM / sh.a_rows);
  sh.a_stride = static_cast<uint32_t>(sh.a_rows) * kRowBytes;
  sh.b_stride = static_cast<uint32_t>(bn_eff) * kRowBytes;
  sh.bytes = static_cast<uint32_t>(sh.a_rows + bn_eff) * kRowBytes;
  return sh;
}

template <int KIND, int BN, int STAGES>
struct SmemLayout {
  static_assert(KIND != DG_KIND_W4A8, "W4A8 uses grouped_gemm_w4_kernel");
  static constexpr int kBBytes = BN * kRowBytes;  // weight tile of one K block
  static constexpr int kAStage = kATileBytes;
  static constexpr int kBStage = kBBytes;
  static constexpr int off_a = 0;
  static constexpr int off_b = off_a + STAGES * kAStage;
  static constexpr int off_bar = off_b + STAGES * kBStage;
  // full[S], empty[S], acc_full[2], acc_empty[2], drain
  static constexpr int kNumBars = 2 * STAGES + 5;
  static constexpr int off_misc = off_bar + kNumBars * 8;  // tmem slot, abort, n_items, pad
  static constexpr int off_bs = (off_misc + 32 + 15) & ~15;  // a tile's weight scales, one strip per epilogue warp; read as float4
  static constexpr int off_epi = off_bs + 4 * BN * 4;        // store strips: 32 rows x 64 B per epilogue warp
  static constexpr int off_table = off_epi + 4 * 2048;
  static_assert(off_bs % 16 == 0 && off_epi % 16 == 0 && off_table % 4 == 0,
                "scale and store strips are accessed with 16-byte loads and stores");
  static constexpr int kThreads = 192;
  static constexpr int kTmemCols = 2 * BN;
  __host__ __device__ static constexpr int total(int table_bytes) {
    return off_table + table_bytes + 1024;  // + slack to align the base to 1024 bytes
  }
};

// Per-thread output-row context of the epilogue.
struct EpiRow {
  float as;              // a_scale of this row (1 when unscaled)
  float bs_g;            // per-group weight scale (TENSOR_WISE)
  const float* bs_row;   // the tile's weight scales (PER_CHANNEL), staged in shared memory
  __nv_bfloat16* d_row;  // &D[row][n0]
  uint32_t* dbg_row;     // &debug_acc[row][n0] or nullptr
  bool f16 = false;      // 16-bit outputs are fp16 instead of bf16 (warp-uniform)
};

// Scales and converts 8 accumulator columns (j .. j+7 of the chunk that starts at column
// `col` of the tile) of one row: out = bf16_rne((float(acc) * a_scale) * b_scale), two separate
// fp32 multiplications in the reference's order (m_grouped_fp8_gemm_nt_maksed_low_latency.cu:584).
template <bool kIntAcc>
__device__ __forceinline__ uint4 epilogue_pack8(const uint32_t (&r)[32], int j, const EpiRow& e,
                                                int scale_mode, int col) {
  float v[8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
    v[i] = kIntAcc ? __int2float_rn(static_cast<int>(r[j + i])) : __uint_as_float(r[j + i]);
  if (scale_mode == DG_SCALE_PER_CHANNEL) {
    const float4 b0 = *reinterpret_cast<const float4*>(e.bs_row + col + j);
    const float4 b1 = *reinterpret_cast<const float4*>(e.bs_row + col + j + 4);
    v[0] = (v[0] * e.as) * b0.x;
    v[1] = (v[1] * e.as) * b0.y;
    v[2] = (v[2] * e.as) * b0.z;
    v[3] = (v[3] * e.as) * b0.w;
    v[4] = (v[4] * e.as) * b1.x;
    v[5] = (v[5] * e.as) * b1.y;
    v[6] = (v[6] * e.as) * b1.z;
    v[7] = (v[7] * e.as) * b1.w;
  } else if (scale_mode == DG_SCALE_TENSOR_WISE) {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = (v[i] * e.as) * e.bs_g;
  }
  uint4 o;
  if (e.f16) {
    __half2 h;
    h = __floats2half2_rn(v[0], v[1]);
    o.x = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2half2_rn(v[2], v[3]);
    o.y = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2half2_rn(v[4], v[5]);
    o.z = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2half2_rn(v[6], v[7]);
    o.w = *reinterpret_cast<uint32_t*>(&h);
    return o;
  }
  __nv_bfloat162 h;
  h = __floats2bfloat162_rn(v[0], v[1]);
  o.x = *reinterpret_cast<uint32_t*>(&h);
  h = __floats2bfloat162_rn(v[2], v[3]);
  o.y = *reinterpret_cast<uint32_t*>(&h);
  h = __floats2bfloat162_rn(v[4], v[5]);
  o.z = *reinterpret_cast<uint32_t*>(&h);
  h = __floats2bfloat162_rn(v[6], v[7]);
  o.w = *reinterpret_cast<uint32_t*>(&h);
  return o;
}

// Stores 32 accumulator columns of this lane's row straight from registers: 16-byte stores,
// columns >= N skipped.  (Every lane of a warp writes a different row, so one store
// instruction touches 32 rows; epilogue_store32_staged is the coalesced form.)
template <bool kIntAcc>
__device__ __forceinline__ void epilogue_store32(const uint32_t (&r)[32], const EpiRow& e,
                                                 int scale_mode, int col, int cols_left) {
#pragma unroll
  for (int j = 0; j < 32; j += 8) {
    if (j + 8 <= cols_left) {
      *reinterpret_cast<uint4*>(e.d_row + col + j) = epilogue_pack8<kIntAcc>(r, j, e, scale_mode, col);
      if (e.dbg_row != nullptr) {
        *reinterpret_cast<uint4*>(e.dbg_row + col + j) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
        *reinterpret_cast<uint4*>(e.dbg_row + col + j + 4) =
            make_uint4(r[j + 4], r[j + 5], r[j + 6], r[j + 7]);
      }
    }
  }
}

// What a warp needs to store its 32 consecutive rows through shared memory.
struct EpiWarp {
  uint8_t* strip;         // 32 rows x 64 bytes of shared memory private to the warp
  __nv_bfloat16* d_warp;  // &D[first row of the warp][n0]
  size_t ld;              // elements between consecutive rows of D (= N)
  unsigned rv_mask;       // bit r: row r of the warp may be stored
  int lane;
  __nv_bfloat16* lane_row = nullptr;  // scattered output: where this lane's row goes (&dst[row][n0])
  bool scatter = false;               // warp-uniform
  uint8_t* wide_strip = nullptr;      // optional 32 rows x 128 bytes: 64 columns per pass (see epilogue_store64_staged)
};

// Coalesced form of epilogue_store32: every lane converts its row's 32 columns into the warp's
// strip (four 16-byte pieces per row, piece index XOR-swizzled with the row so that neither the
// writes nor the reads conflict), then lane l stores piece l % 4 of rows l / 4, l / 4 + 8, ...:
// a store instruction covers 8 rows x 64 contiguous bytes instead of 32 rows x 16 bytes.
template <bool kIntAcc>
__device__ __forceinline__ void epilogue_store32_staged(const uint32_t (&r)[32], const EpiRow& e,
                                                        const EpiWarp& w, int scale_mode, int col,
                                                        int cols_left) {
  const int swz = (w.lane >> 1) & 3;
#pragma unroll
  for (int p = 0; p < 4; ++p)
    *reinterpret_cast<uint4*>(w.strip + w.lane * 64 + ((p ^ swz) << 4)) =
        epilogue_pack8<kIntAcc>(r, 8 * p, e, scale_mode, col);
  __syncwarp();
  const int p = w.lane & 3;
#pragma unroll
  for (int h = 0; h < 4; ++h) {
    const int row = (w.lane >> 2) + 8 * h;
    __nv_bfloat16* dst = w.d_warp + row * w.ld;
    if (w.scatter)  // the row's destination is known to the lane that owns the row
      dst = reinterpret_cast<__nv_bfloat16*>(
          __shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(w.lane_row), row));
    if (8 * p + 8 <= cols_left && ((w.rv_mask >> row) & 1u))
      *reinterpret_cast<uint4*>(dst + col + 8 * p) =
          *reinterpret_cast<const uint4*>(w.strip + row * 64 + ((p ^ ((row >> 1) & 3)) << 4));
  }
  __syncwarp();  // the strip is rewritten by the next chunk
}

// Two chunks (64 columns) at once through a 32-row x 128-byte strip: a store instruction then
// covers 4 rows x 128 contiguous bytes.  Used when the rows go to peer GPUs (scattered output):
// a 128-byte write carries half the per-packet overhead of a 64-byte one over NVLink.  Piece
// index XOR row % 8 keeps writes and reads free of bank conflicts.
template <bool kIntAcc>
__device__ __forceinline__ void epilogue_store64_staged(const uint32_t (&ra)[32], const uint32_t (&rb)[32],
                                                        const EpiRow& e, const EpiWarp& w, int scale_mode,
                                                        int col, int cols_left) {
  const int swz = w.lane & 7;
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    *reinterpret_cast<uint4*>(w.wide_strip + w.lane * 128 + ((p ^ swz) << 4)) =
        epilogue_pack8<kIntAcc>(ra, 8 * p, e, scale_mode, col);
    *reinterpret_cast<uint4*>(w.wide_strip + w.lane * 128 + (((4 + p) ^ swz) << 4)) =
        epilogue_pack8<kIntAcc>(rb, 8 * p, e, scale_mode, col + 32);
  }
  __syncwarp();
  const int p = w.lane & 7;
#pragma unroll
  for (int h = 0; h < 8; ++h) {
    const int row = (w.lane >> 3) + 4 * h;
    __nv_bfloat16* dst = w.d_warp + row * w.ld;
    if (w.scatter)
      dst = reinterpret_cast<__nv_bfloat16*>(
          __shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(w.lane_row), row));
    if (8 * p + 8 <= cols_left && ((w.rv_mask >> row) & 1u))
      *reinterpret_cast<uint4*>(dst + col + 8 * p) =
          *reinterpret_cast<const uint4*>(w.wide_strip + row * 128 + ((p ^ (row & 7)) << 4));
  }
  __syncwarp();  // the strip is rewritten by the next pass
}

// TMA coordinates of the weight tile of K block kb: packed layout = flat list of 128-byte rows
// ordered [g][kb][n]; row-major = rows [g][n] of K elements.
__device__ __forceinline__ void weight_coords(const KernelParams& p, int g, int n0, int kb,
                                              int elems_per_row, int& x, int& y) {
  if (p.b_rowmajor) {
    x = kb * elems_per_row;
    y = g * p.N + n0;
  } else {
    x = 0;
    y = (g * p.kblocks + kb) * p.N + n0;
  }
}

// Slow twin of epilogue_store32 for what the grouped entry points never produce: fp32
// output or an N that is not a multiple of 8 (rows of D then start at unaligned addresses).
// Same arithmetic, one scalar store per element.
template <bool kIntAcc>
__device__ __forceinline__ void epilogue_store32_scalar(const uint32_t (&r)[32], const EpiRow& e,
                                                        int scale_mode, int col, int cols_left,
                                                        int out_kind) {
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    if (j < cols_left) {
      float v = kIntAcc ? __int2float_rn(static_cast<int>(r[j])) : __uint_as_float(r[j]);
      if (scale_mode == DG_SCALE_PER_CHANNEL)
        v = (v * e.as) * e.bs_row[col + j];
      else if (scale_mode == DG_SCALE_TENSOR_WISE)
        v = (v * e.as) * e.bs_g;
      if (out_kind == 0)
        e.d_row[col + j] = __float2bfloat16_rn(v);
      else if (out_kind == 1)
        reinterpret_cast<__half*>(e.d_row)[col + j] = __float2half_rn(v);
      else
        reinterpret_cast<float*>(e.d_row)[col + j] = v;
      if (e.dbg_row != nullptr) e.dbg_row[col + j] = r[j];
    }
  }
}

// Each epilogue warp copies the weight scales of a tile's `width` columns into its own strip of
// shared memory before it waits for the accumulator, so that the global-load latency hides
// behind the main loop and the per-column reads in epilogue_store32 are shared-memory
// broadcasts (read from global memory there, eight columns at a time, they cost more than
// the stores).  Columns at or beyond N get 0.  Strips are private to a warp, so a
// __syncwarp() is all the ordering needed and no warp ever waits for another.
__device__ __forceinline__ void stage_tile_scales(float* dst, const float* b_scale_group, int n0,
                                                  int width, int n, int lane, bool per_channel) {
  __syncwarp();  // the previous tile's reads of the strip are done
  if (per_channel) {
    for (int c = lane; c < width; c += 32) dst[c] = (n0 + c < n) ? __ldg(b_scale_group + n0 + c) : 0.0f;
  }
  __syncwarp();
}

// Drains `nchunks` 32-column chunks of one accumulator row block: the TMEM load of chunk c + 1
// is in flight while chunk c is scaled, converted and stored.  `cols_left0` = N - first column
// of the tile.  Every lane of the warp takes part in the loads (and in the staged stores); in
// the direct forms only lanes with `rv` store.
template <bool kIntAcc>
__device__ __forceinline__ void epilogue_drain(uint32_t t_row, int nchunks, bool rv, const EpiRow& row,
                                               const EpiWarp& ew, int scale_mode, int cols_left0,
                                               bool scalar_out, int out_kind) {
  const bool staged = !scalar_out && row.dbg_row == nullptr && ew.strip != nullptr;  // warp-uniform
  auto store = [&](const uint32_t (&r)[32], int c) {
    if (staged) {
      epilogue_store32_staged<kIntAcc>(r, row, ew, scale_mode, c * 32, cols_left0 - c * 32);
      return;
    }
    if (!rv) return;
    if (!scalar_out)
      epilogue_store32<kIntAcc>(r, row, scale_mode, c * 32, cols_left0 - c * 32);
    else
      epilogue_store32_scalar<kIntAcc>(r, row, scale_mode, c * 32, cols_left0 - c * 32, out_kind);
  };
  uint32_t ra[32], rb[32];
  if (staged && ew.wide_strip != nullptr) {  // warp-uniform: 64 columns per pass
    int c = 0;
#pragma unroll 1
    for (; c + 1 < nchunks; c += 2) {
      tmem_ld_32x32(t_row + c * 32, ra);
      tmem_ld_32x32(t_row + (c + 1) * 32, rb);
      tmem_ld_wait();
      epilogue_store64_staged<kIntAcc>(ra, rb, row, ew, scale_mode, c * 32, cols_left0 - c * 32);
    }
    if (c < nchunks) {
      tmem_ld_32x32(t_row + c * 32, ra);
      tmem_ld_wait();
      store(ra, c);
    }
    return;
  }
  if (nchunks > 0) tmem_ld_32x32(t_row, ra);
#pragma unroll 1
  for (int c = 0; c < nchunks; c += 2) {
    tmem_ld_wait();
    if (c + 1 < nchunks) tmem_ld_32x32(t_row + (c + 1) * 32, rb);
    store(ra, c);
    if (c + 1 < nchunks) {
      tmem_ld_wait();
      if (c + 2 < nchunks) tmem_ld_32x32(t_row + (c + 2) * 32, ra);
      store(rb, c + 1);
    }
  }
}

struct FalseTag { static constexpr bool value = false; };
struct TrueTag { static constexpr bool value = true; };

struct TileCoord {
  int g;           // group
  int row0;        // first row: within the group (masked) or global (contiguous)
  int n0;          // first output column
  int width;       // columns of this item
  int rows_valid;  // rows of this tile that may be stored (before the m_indices check)
};

// Maps a work-item number to its tile using the block's shared-memory schedule table.
// Masked / compact table: cnt[G], pref[G+1] = running number of 128-row blocks, (compact)
// off[G]; item = (global row block) * n_tiles + column tile.  Contiguous table: list of row
// blocks as (group << 16 | block).  `bn` / `n_tiles` are the tile width in use and the number
// of column tiles at that width.
// MODE_SORTED: activation / output row named by entry `pos` of the routing list, -1 for padding.
__device__ __forceinline__ int sorted_row(const KernelParams& p, int pos, int post_pad) {
  if (pos >= post_pad) return -1;
  const uint32_t id = static_cast<uint32_t>(p.sorted_ids[pos]);
  const int slot = static_cast<int>(id >> 24);
  const long long row = static_cast<long long>(id & 0x00FFFFFFu) * p.real_topk + slot;
  return (slot >= p.real_topk || row >= p.size_m) ? -1 : static_cast<int>(row);
}

struct ItemDecoder {
  const KernelParams& p;
  const int32_t* tbl;
  int bn;
  int n_tiles;
  int cursor;
  int split_from;  // items from this one on are halves of tiles: item = split_from + 2 * k + half
  __device__ ItemDecoder(const KernelParams& p_, const int32_t* tbl_, int bn_, int n_tiles_,
                         int split_from_ = 0x7fffffff)
      : p(p_), tbl(tbl_), bn(bn_), n_tiles(n_tiles_), cursor(0), split_from(split_from_) {}
  __device__ __forceinline__ TileCoord get(int item) {
    TileCoord t;
    t.width = bn;
    int sub = 0;
    if (item >= split_from) {
      const int j = item - split_from;
      item = split_from + (j >> 1);
      t.width = bn >> 1;
      sub = (j & 1) * t.width;
    }
    if (p.mode != MODE_CONTIG) {
      const int tg = p.mode == MODE_SORTED ? p.tbl_groups : p.G;  // entries per array of the table
      const int32_t* cnt = tbl;
      const int32_t* pref = tbl + tg;
      const int blk = item / n_tiles;
      while (blk >= pref[cursor + 1]) ++cursor;  // items only grow, so the cursor persists
      const int mt = blk - pref[cursor];
      t.g = cursor;
      t.row0 = mt * kBM;
      t.n0 = (item - blk * n_tiles) * bn + sub;
      t.rows_valid = min(kBM, cnt[cursor] - t.row0);
      if (p.mode == MODE_COMPACT) {  // rows of group g start at offsets[g] in the flat tensor
        t.row0 += tbl[2 * p.G + 1 + cursor];
        t.rows_valid = min(t.rows_valid, p.M - t.row0);
      } else if (p.mode == MODE_SORTED) {  // the cursor counts runs: expert (-1: zeros) and first list entry
        t.g = tbl[2 * tg + 1 + cursor];
        t.row0 += tbl[3 * tg + 1 + cursor];
      }
    } else {
      const int bi = item / n_tiles;
      const int e = tbl[bi];
      t.g = e >> 16;
      t.row0 = (e & 0xFFFF) * kBM;
      t.n0 = (item - bi * n_tiles) * bn + sub;
      t.rows_valid = min(kBM, p.M - t.row0);
    }
    return t;
  }
};

// kGather: the instantiation behind MODE_SORTED, with four more warps that fetch the rows of a
// tile by index (the other instantiations carry none of that code).
constexpr int kGatherThreads = 128;
constexpr int kGatherDepth = 2;  // K blocks a gathering thread keeps in flight behind the one it issues
template <int KIND, int BN, int STAGES, bool kGather = false>
__global__ void __launch_bounds__(SmemLayout<KIND, BN, STAGES>::kThreads + (kGather ? kGatherThreads : 0), 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tm_a,
                    const __grid_constant__ CUtensorMap tm_a64,
                    const __grid_constant__ CUtensorMap tm_a32,
                    const __grid_constant__ CUtensorMap tm_a8,
                    const __grid_constant__ CUtensorMap tm_b,
                    const __grid_constant__ CUtensorMap tm_b128,
                    const __grid_constant__ CUtensorMap tm_b64,
                    const __grid_constant__ CUtensorMap tm_b32, const KernelParams p) {
  using L = SmemLayout<KIND, BN, STAGES>;
  constexpr int kUmmaKind =
      (KIND == DG_KIND_E4M3) ? UMMA_F8F6F4 : (KIND == DG_KIND_BF16 ? UMMA_F16 : UMMA_I8);
  constexpr bool kIntAcc = (KIND == DG_KIND_I8);
  constexpr int kElemsPerRow = (KIND == DG_KIND_BF16) ? 64 : 128;  // A elements per 128 bytes
  constexpr uint32_t kIdesc =
      umma_idesc(kIntAcc ? 2u : 1u, (KIND == DG_KIND_E4M3) ? 0u : 1u, kBM, BN);

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw_addr);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  auto bar_full = [&](int s) { return base + L::off_bar + 8u * s; };
  auto bar_empty = [&](int s) { return base + L::off_bar + 8u * (STAGES + s); };
  auto bar_acc_full = [&](int b) { return base + L::off_bar + 8u * (2 * STAGES + b); };
  auto bar_acc_empty = [&](int b) { return base + L::off_bar + 8u * (2 * STAGES + 2 + b); };
  const uint32_t bar_drain = base + L::off_bar + 8u * (2 * STAGES + 4);

  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::off_misc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::off_misc + 4);
  volatile int* n_items_s = reinterpret_cast<volatile int*>(smem + L::off_misc + 8);
  volatile int* bn_eff_s = reinterpret_cast<volatile int*>(smem + L::off_misc + 12);
  volatile int* split_from_s = reinterpret_cast<volatile int*>(smem + L::off_misc + 16);
  volatile int* post_pad_s = reinterpret_cast<volatile int*>(smem + L::off_misc + 20);  // MODE_SORTED
  int32_t* tbl = reinterpret_cast<int32_t*>(smem + L::off_table);

  // ------------------------------------------------------------------ one-time set-up
  if (tid == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full(s), kGather ? 5 : 1);  // the producer thread (+ the four gathering warps)
      mbar_init(bar_empty(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_acc_full(b), 1);
      mbar_init(bar_acc_empty(b), 4);
    }
    mbar_init(bar_drain, 1);
    fence_mbar_init();
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_b);
  }

  // Schedule table.  Masked / compact: cnt[G] (clamped rows per group), pref[G+1] (running
  // number of work items) and, compact, off[G] (first row of each group).  Contiguous: the
  // list of 128-row blocks whose first row belongs to a group, as (group << 16 | block).
  if (p.mode == MODE_SORTED) {
    // Runs of list blocks with one expert: cnt[r] entries, pref[r + 1] running 128-entry tiles,
    // run_e[r] the expert (-1: rows to be written as zeros), run_p0[r] the first list entry.
    const int RM = p.tbl_groups;
    int32_t* cnt = tbl;
    int32_t* pref = tbl + RM;
    int32_t* run_e = tbl + 2 * RM + 1;
    int32_t* run_p0 = tbl + 3 * RM + 1;
    if (warp == 0) {
      const int post = max(0, min(*p.num_post_pad, p.num_sorted));
      const int nb = min(p.num_blocks, (post + p.block_m - 1) / p.block_m);
      int runs = 0;
      bool bad = false;
      for (int b0 = 0; b0 < nb; b0 += 32) {
        const int b = b0 + lane;
        const int e = (b < nb) ? p.expert_ids[b] : 0;
        const bool start = b < nb && (b == 0 || p.expert_ids[b - 1] != e);
        const unsigned mask = __ballot_sync(0xffffffffu, start);
        const int r = runs + __popc(mask & ((1u << lane) - 1u));
        if (start && r < RM) {
          run_e[r] = e >= p.G ? -2 : (e < 0 ? -1 : e);  // -2: no such expert, nothing is computed
          run_p0[r] = b * p.block_m;
          bad |= e >= p.G;
        }
        runs += __popc(mask);
      }
      __syncwarp();
      const bool overflow = runs > RM;  // more runs than the table holds: compute nothing, say so
      if (overflow) runs = 0;
      int running = 0;
      for (int r0 = 0; r0 < runs; r0 += 32) {
        const int r = r0 + lane;
        int x = 0;
        if (r < runs) {
          const int end = (r + 1 < runs) ? run_p0[r + 1] : nb * p.block_m;
          const int rows = run_e[r] == -2 ? 0 : end - run_p0[r];
          cnt[r] = rows;
          x = (rows + kBM - 1) / kBM;
        }
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int y = __shfl_up_sync(0xffffffffu, x, o);
          if (lane >= o) x += y;
        }
        if (r < runs) pref[r + 1] = running + x;
        running += __shfl_sync(0xffffffffu, x, 31);
      }
      if (lane == 0) {
        pref[0] = 0;
        *bn_eff_s = BN;
        *split_from_s = 0x7fffffff;
        *n_items_s = running * p.n_tiles;
        *post_pad_s = post;
      }
      if ((__any_sync(0xffffffffu, bad) || overflow) && lane == 0 && blockIdx.x == 0 && p.status != nullptr)
        atomicCAS(p.status, DG_DEV_OK, DG_DEV_BAD_GROUP_INDEX);
    }
  } else if (p.mode != MODE_CONTIG) {
    int32_t* cnt = tbl;
    int32_t* pref = tbl + p.G;
    for (int g = tid; g < p.G; g += blockDim.x) {
      cnt[g] = p.sched ? max(0, min(p.sched[g], p.M)) : p.M;  // no masked_m: every row (dense GEMM)
      if (p.mode == MODE_COMPACT) tbl[2 * p.G + 1 + g] = max(0, min(p.offsets[g], p.M));
    }
    __syncthreads();
    if (warp == 0) {
      int running = 0;
      for (int g0 = 0; g0 < p.G; g0 += 32) {
        const int g = g0 + lane;
        int x = (g < p.G) ? (cnt[g] + kBM - 1) / kBM : 0;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int y = __shfl_up_sync(0xffffffffu, x, o);
          if (lane >= o) x += y;
        }
        if (g < p.G) pref[g + 1] = running + x;
        running += __shfl_sync(0xffffffffu, x, 31);
      }
      if (lane == 0) {
        pref[0] = 0;
        // Sparse routing (few groups with rows): narrow the tiles until there is an item for
        // every block, so that all SMs take part in streaming the few weight panels.
        int bn_eff = BN;
        if (p.narrow > 1 && p.narrow < BN) {
          bn_eff = p.narrow;
        } else if (p.narrow == 1) {
          // Narrow only while every item still finds a block of its own: with more items
          // than blocks the wide tiles win (measured: a second round of narrow items costs
          // more than idle SMs do, as each item pays the same UMMA issue time).
          for (int bn = BN / 2; bn >= 32; bn >>= 1)
            if (running * ((p.N + bn - 1) / bn) <= static_cast<int>(gridDim.x)) bn_eff = bn;
        }
        *bn_eff_s = bn_eff;
        int items = running * ((p.N + bn_eff - 1) / bn_eff);
        int split_from = 0x7fffffff;
        if (bn_eff == BN && p.split_tail) {
          // Items go round-robin to the blocks, so a last round with few items leaves most SMs
          // idle for a whole item.  If that round is at most half full, its tiles are split in
          // two: one more round of half the length, on twice as many blocks.
          const int tail = items % static_cast<int>(gridDim.x);
          if (items > static_cast<int>(gridDim.x) && tail > 0 && 2 * tail <= static_cast<int>(gridDim.x)) {
            split_from = items - tail;
            items += tail;
          }
        }
        *split_from_s = split_from;
        *n_items_s = items;
      }
    }
  } else {
    const int window0 = p.group_window ? p.group_window - 1 : 0;
    for (int b = tid; b < p.m_blocks; b += blockDim.x) {
      const int e = p.sched[(size_t)b * kBM];
      tbl[b] = e < 0 ? -1 : e - window0;
    }
    __syncthreads();
    if (warp == 0) {
      int count = 0;
      bool bad = false;
      for (int b0 = 0; b0 < p.m_blocks; b0 += 32) {
        const int b = b0 + lane;
        const int e = (b < p.m_blocks) ? tbl[b] : -1;
        const bool ok = (e >= 0) && (e < p.G);
        bad |= (e >= p.G) && !p.group_window;
        const unsigned mask = __ballot_sync(0xffffffffu, ok);
        __syncwarp();
        if (ok) tbl[count + __popc(mask & ((1u << lane) - 1u))] = (e << 16) | b;
        count += __popc(mask);
        __syncwarp();
      }
      if (lane == 0) {
        *bn_eff_s = BN;
        *split_from_s = 0x7fffffff;
        *n_items_s = count * p.n_tiles;
      }
      if (__any_sync(0xffffffffu, bad) && lane == 0 && blockIdx.x == 0 && p.status != nullptr)
        atomicCAS(p.status, DG_DEV_OK, DG_DEV_BAD_GROUP_INDEX);
    }
  }

  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), L::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();

  const uint32_t tmem_base = *tmem_slot;
  const int n_items = *n_items_s;
  const int split_from = *split_from_s;
  const int bn_eff = *bn_eff_s;                      // tile width in use: BN, or 64 / 32 when narrowed
  const int nt_eff = (p.N + bn_eff - 1) / bn_eff;    // column tiles at that width

  // ------------------------------------------------------------------ roles
  if (kGather && warp >= 6) {
    if constexpr (kGather) {
      // ---- gathering warps (MODE_SORTED): thread g copies the 16-byte piece g % 8 of rows g / 8,
      // g / 8 + 16, ... of the tile, so that eight neighbouring lanes read one row's 128 bytes.
      // A thread keeps kGatherDepth K blocks in flight: after issuing block i it waits for block
      // i - kGatherDepth, makes it visible to the tensor core's proxy and its warp signals the
      // stage.
      const int g = tid - L::kThreads;
      const int piece = g & 7, rsub = g >> 3;
      const int post = *post_pad_s;
      const uint8_t* a_bytes = static_cast<const uint8_t*>(p.gather_a);
      const size_t row_bytes = static_cast<size_t>(p.K) * (KIND == DG_KIND_BF16 ? 2 : 1);
      ItemDecoder dec(p, tbl, BN, p.n_tiles);
      uint32_t it = 0;
      bool ok = true;
      auto signal_done = [&](uint32_t j) {  // K block j of this block's sequence has landed
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_full(j % STAGES));
      };
      for (int item = blockIdx.x; ok && item < n_items; item += gridDim.x) {
        const TileCoord t = dec.get(item);
        if (t.g < 0) continue;  // rows of an absent expert: nothing to load
        int src[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int r = rsub + 16 * i;
          src[i] = r < t.rows_valid ? sorted_row(p, t.row0 + r, post) : -1;
        }
        for (int kb = 0; kb < p.kblocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          if (!mbar_wait_warp(bar_empty(s), ph ^ 1u, abort_flag, SITE_PRODUCER_EMPTY)) {
            ok = false;
            break;
          }
          const size_t col = static_cast<size_t>(kb) * kRowBytes + piece * 16;
          const uint32_t in_row = col < row_bytes ? 16u : 0u;  // last half block of K % 128 == 64: zeros
          const uint32_t a_dst = base + L::off_a + s * L::kAStage;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int r = rsub + 16 * i;
            if (src[i] >= 0)
              cp_async_16(a_dst + r * kRowBytes + ((piece ^ (r & 7)) << 4),
                          a_bytes + static_cast<size_t>(src[i]) * row_bytes + (in_row ? col : 0), in_row);
          }
          cp_async_commit();
          if (it >= kGatherDepth) {
            cp_async_wait_group<kGatherDepth>();
            signal_done(it - kGatherDepth);
          }
        }
      }
      cp_async_wait_group<0>();
      if (ok)
        for (uint32_t j = it > kGatherDepth ? it - kGatherDepth : 0; j < it; ++j) signal_done(j);
    }
  } else if (warp == 0 && p.mode == MODE_SORTED) {
    if (lane == 0) {
      // ---- weight producer of MODE_SORTED (the activation rows come from the gathering warps)
      const uint64_t pol_b = l2_policy_evict_first();
      ItemDecoder dec(p, tbl, BN, p.n_tiles);
      uint32_t it = 0;
      bool ok = true;
      for (int item = blockIdx.x; ok && item < n_items; item += gridDim.x) {
        const TileCoord t = dec.get(item);
        if (t.g < 0) continue;
        for (int kb = 0; kb < p.kblocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          if (!mbar_wait_bounded(bar_empty(s), ph ^ 1u, abort_flag, SITE_PRODUCER_EMPTY)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(bar_full(s), static_cast<uint32_t>(BN) * kRowBytes);
          int bx, by;
          weight_coords(p, t.g, t.n0, kb, kElemsPerRow, bx, by);
          tma_load_2d(base + L::off_b + s * L::kBStage, &tm_b, bar_full(s), bx, by, pol_b);
        }
      }
      if (*abort_flag) {  // the stage barriers also count the gathering warps: just let copies land
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) {
        }
      }
    }
  } else if (warp == 0) {
    if (lane == 0) {
      // ---- TMA producer.  kNarrow = false is the straight-line loop for full-width tiles
      // (one K block per stage); kNarrow = true handles 64 / 32-column tiles.
      const uint64_t pol_a = l2_policy_evict_last();   // A tiles are re-read by other n-tiles
      const uint64_t pol_b = l2_policy_evict_first();  // weights stream through once
      uint32_t it = 0;
      auto produce = [&](auto narrow_tag) {
        constexpr bool kNarrow = decltype(narrow_tag)::value;
        ItemDecoder dec(p, tbl, bn_eff, nt_eff, split_from);
        for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
          const TileCoord t = dec.get(item);
          // weight box of the item's width
          const CUtensorMap* tm_w = t.width == BN ? &tm_b
                                    : (t.width == 128 ? &tm_b128 : (t.width == 64 ? &tm_b64 : &tm_b32));
          const StageShape sh = stage_shape(t.rows_valid, t.width, BN);
          const CUtensorMap* tm_act = (sh.a_rows == kBM) ? &tm_a
                                      : (sh.a_rows == 64 ? &tm_a64 : (sh.a_rows == 32 ? &tm_a32 : &tm_a8));
          const int kps = kNarrow ? sh.kps : 1;
          for (int kb0 = 0; kb0 < p.kblocks; kb0 += kps, ++it) {
            const int s = it % STAGES;
            const uint32_t ph = (it / STAGES) & 1u;
            if (!mbar_wait_bounded(bar_empty(s), ph ^ 1u, abort_flag, SITE_PRODUCER_EMPTY)) return;
            const int nb = kNarrow ? min(kps, p.kblocks - kb0) : 1;
            mbar_arrive_expect_tx(bar_full(s), nb * sh.bytes);
            for (int j = 0; j < nb; ++j) {
              const int kb = kb0 + j;
              const uint32_t a_dst = base + L::off_a + s * L::kAStage + j * sh.a_stride;
              if (p.mode == MODE_MASKED)
                tma_load_3d(a_dst, tm_act, bar_full(s), kb * kElemsPerRow, t.row0, t.g, pol_a);
              else
                tma_load_2d(a_dst, tm_act, bar_full(s), kb * kElemsPerRow, t.row0, pol_a);
              int bx, by;
              weight_coords(p, t.g, t.n0, kb, kElemsPerRow, bx, by);
              tma_load_2d(base + L::off_b + s * L::kBStage + j * sh.b_stride, tm_w, bar_full(s), bx,
                          by, pol_b);
            }
          }
        }
      };
      if (bn_eff == BN)
        produce(FalseTag{});
      else
        produce(TrueTag{});
      // Do not leave while a copy into this block's shared memory is still in flight:
      // wait (bounded) for the last fill of every stage.
      int local_abort = 0;
      for (int s = 0; s < STAGES; ++s) {
        const uint32_t fills = (it + STAGES - 1 - s) / STAGES;
        if (fills > 0 && !mbar_wait_bounded(bar_full(s), (fills - 1) & 1u, &local_abort,
                                            SITE_PRODUCER_DRAIN))
          *abort_flag = SITE_PRODUCER_DRAIN;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- UMMA issuer (same two variants as the producer)
      auto issue = [&](auto narrow_tag) {
        constexpr bool kNarrow = decltype(narrow_tag)::value;
        ItemDecoder dec(p, tbl, bn_eff, nt_eff, split_from);
        uint32_t it = 0, tile = 0;
        for (int item = blockIdx.x; item < n_items; item += gridDim.x, ++tile) {
          const TileCoord t = dec.get(item);
          const StageShape sh = stage_shape(t.rows_valid, t.width, BN);
          // N = the tile's width; M = 64 when the item has no more than 64 rows: the tensor
          // cores then work on half the rows, which on a GPU held back by its power cap buys SM
          // clock (decode workload, all items at M = 64 for the comparison: 152-156 us at
          // 1.3-1.9 GHz against 168-178 us at 0.86-1.05 GHz).  With M = 64 row r of the tile is
          // TMEM lane 32 * (r / 16) + r % 16.
          const uint32_t idesc = (kIdesc & ~(0x3Fu << 17) & ~(0x1Fu << 24)) |
                                 (static_cast<uint32_t>(t.width >> 3) << 17) |
                                 ((t.rows_valid <= 64 ? 4u : 8u) << 24);
          const int kps = kNarrow ? sh.kps : 1;
          const uint32_t buf = tile & 1u;
          const uint32_t aph = (tile >> 1) & 1u;
          if (!mbar_wait_bounded(bar_acc_empty(buf), aph ^ 1u, abort_flag, SITE_MMA_ACC_EMPTY)) return;
          tc_fence_after_sync();
          const uint32_t d_tmem = tmem_base + buf * BN;
          const int k_end = (p.mode == MODE_SORTED && t.g < 0) ? 0 : p.kblocks;  // zero rows: no products
          for (int kb0 = 0; kb0 < k_end; kb0 += kps, ++it) {
            const int s = it % STAGES;
            const uint32_t ph = (it / STAGES) & 1u;
            if (!mbar_wait_bounded(bar_full(s), ph, abort_flag, SITE_MMA_FULL)) return;
            tc_fence_after_sync();
            const int nb = kNarrow ? min(kps, p.kblocks - kb0) : 1;
            for (int j = 0; j < nb; ++j) {
              const uint64_t a_desc = umma_desc_sw128(base + L::off_a + s * L::kAStage +
                                                      (kNarrow ? j * sh.a_stride : 0u));
              const uint64_t b_desc = umma_desc_sw128(base + L::off_b + s * L::kBStage +
                                                      (kNarrow ? j * sh.b_stride : 0u));
#pragma unroll
              for (int k = 0; k < kRowBytes / 32; ++k) {
                // +2 in the start-address field = +32 bytes along K inside the swizzled row
                umma_ss<kUmmaKind>(d_tmem, a_desc + 2u * k, b_desc + 2u * k, idesc,
                                   (kb0 | j | k) != 0 ? 1u : 0u);
              }
            }
            umma_commit(bar_empty(s));  // frees the stage once these UMMAs have read it
          }
          umma_commit(bar_acc_full(buf));
        }
      };
      if (bn_eff == BN)
        issue(FalseTag{});
      else
        issue(TrueTag{});
      if (*abort_flag) {
        // Abnormal exit: make sure no UMMA is still running before TMEM is released.
        int local_abort = 0;
        umma_commit(bar_drain);
        mbar_wait_bounded(bar_drain, 0, &local_abort, 0);
      }
    }
  } else if (warp < 6) {
    // ---- epilogue: this warp may touch TMEM lanes [32q, 32q+32)
    const int q = warp & 3;
    ItemDecoder dec(p, tbl, bn_eff, nt_eff, split_from);
    uint32_t tile = 0;
    for (int item = blockIdx.x; item < n_items; item += gridDim.x, ++tile) {
      const TileCoord t = dec.get(item);
      // M = 128: this warp's lanes hold rows 32q .. 32q+31.  M = 64 (items of at most 64 rows):
      // its lanes 0..15 hold rows 16q .. 16q+15 and the other lanes nothing.
      const bool m64 = t.rows_valid <= 64;
      const int rows_per_warp = m64 ? 16 : 32;
      const int row_in_tile = q * rows_per_warp + lane;
      const uint32_t buf = tile & 1u;
      const uint32_t aph = (tile >> 1) & 1u;
      // Everything that depends only on the tile's coordinates is fetched before the wait for
      // the accumulator, so that the global-load latency hides behind the main loop.
      float* bs_s = reinterpret_cast<float*>(smem + L::off_bs) + q * BN;
      const bool warp_has_rows = t.rows_valid > q * rows_per_warp;  // warp-uniform
      bool rv = false;
      size_t grow = 0;
      EpiRow row;
      row.as = 1.0f;
      row.bs_g = 1.0f;
      const bool sorted = p.mode == MODE_SORTED;
      if (warp_has_rows && sorted) {
        // the list entry of this lane's row names the activation / output row
        if (t.g >= 0)
          stage_tile_scales(bs_s, p.b_scale + (size_t)t.g * p.N, t.n0, t.width, p.N, lane,
                            p.scale_mode == DG_SCALE_PER_CHANNEL);
        const int srow = (lane < rows_per_warp && row_in_tile < t.rows_valid)
                             ? sorted_row(p, t.row0 + row_in_tile, *post_pad_s) : -1;
        rv = srow >= 0;
        grow = rv ? static_cast<size_t>(srow) : 0;
        if (rv) row.as = p.row_weight ? __fmul_rn(p.row_weight[grow], p.a_scale[grow]) : p.a_scale[grow];
        if (p.scale_mode == DG_SCALE_TENSOR_WISE && t.g >= 0) row.bs_g = p.b_scale[t.g];
      } else if (warp_has_rows) {
        stage_tile_scales(bs_s, p.b_scale + (size_t)t.g * p.N, t.n0, t.width, p.N, lane,
                          p.scale_mode == DG_SCALE_PER_CHANNEL);
        rv = lane < rows_per_warp && row_in_tile < t.rows_valid;
        grow = (p.mode == MODE_MASKED ? (size_t)t.g * p.M : (size_t)0) + t.row0 + row_in_tile;
        if (p.mode == MODE_CONTIG && rv) rv = p.sched[grow] >= 0;
        if (rv && p.scale_mode != DG_SCALE_NONE) row.as = p.a_scale[grow];
        if (p.scale_mode == DG_SCALE_TENSOR_WISE) row.bs_g = p.b_scale[t.g];
      }
      if (!mbar_wait_warp(bar_acc_full(buf), aph, abort_flag, SITE_EPI_ACC_FULL)) break;
      tc_fence_after_sync();
      if (warp_has_rows && sorted && t.g < 0) {
        // rows of an expert that lives elsewhere: zeros (one 16-byte store per lane and row
        // covers up to 256 columns; the accumulator was never written and is not read)
        const unsigned rows_mask = __ballot_sync(0xffffffffu, rv);
        const int cols = min(t.width, p.N - t.n0);
        for (int r = 0; r < 32; ++r) {
          if (!((rows_mask >> r) & 1u)) continue;
          const size_t zr = __shfl_sync(0xffffffffu, grow, r);
          __nv_bfloat16* dst = p.d + zr * p.N + t.n0;
          for (int c = lane * 8; c < cols; c += 256) {
            if (c + 8 <= cols && (p.N & 7) == 0)
              *reinterpret_cast<uint4*>(dst + c) = make_uint4(0u, 0u, 0u, 0u);
            else
              for (int i = c; i < min(c + 8, cols); ++i) dst[i] = __float2bfloat16_rn(0.0f);
          }
        }
      } else if (warp_has_rows) {
        row.bs_row = bs_s;  // PER_CHANNEL only
        const size_t d_off = grow * p.N + t.n0;  // in output elements
        row.d_row = p.out_kind == 2 ? reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<float*>(p.d) + d_off)
                                    : p.d + d_off;
        const bool scatter = sorted || (p.mode == MODE_CONTIG && p.scatter_tag != nullptr);
        if (scatter && rv && !sorted) {
          const int tag = p.scatter_tag[grow];
          row.d_row = static_cast<__nv_bfloat16*>(p.scatter_base[(tag >> 24) & 15]) +
                      (size_t)(tag & 0xFFFFFF) * p.N + t.n0;
        }
        row.dbg_row = p.debug_acc ? p.debug_acc + grow * p.N + t.n0 : nullptr;
        row.f16 = p.out_kind == 1;
        const bool scalar_out = p.out_kind == 2 || (p.N & 7) != 0;
        const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN;
        const int cols_left0 = p.N - t.n0;
        EpiWarp ew;
        ew.strip = smem + L::off_epi + q * 2048;
        ew.d_warp = p.d + (grow - lane) * p.N + t.n0;  // rows of a warp are consecutive in D
        ew.ld = static_cast<size_t>(p.N);
        ew.rv_mask = __ballot_sync(0xffffffffu, rv);
        ew.lane = lane;
        ew.scatter = scatter;
        ew.lane_row = row.d_row;
        if (p.wide_off) ew.wide_strip = smem + p.wide_off + q * 4096;
        epilogue_drain<kIntAcc>(t_row, min(t.width / 32, (cols_left0 + 31) / 32), rv, row, ew, p.scale_mode,
                                cols_left0, scalar_out, p.out_kind);
      }
      // hand the accumulator back to the UMMA issuer
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(bar_acc_empty(buf));
        if (p.signal != nullptr && p.mode == MODE_MASKED) {
          __threadfence();  // this warp's stores (ordered before by __syncwarp) before the count
          atomicAdd(p.signal + (size_t)t.g * p.m_blocks + t.row0 / kBM, min(t.width, p.N - t.n0) / 4);
        }
      }
    }
  }

  // ------------------------------------------------------------------ tear-down
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, L::kTmemCols);
  }
  if (tid == 0 && *abort_flag != 0 && p.status != nullptr) {
    if (atomicCAS(p.status, DG_DEV_OK, DG_DEV_WAIT_EXPIRED) == DG_DEV_OK) {
      p.status[1] = blockIdx.x;
      p.status[2] = *abort_flag;
      p.status[3] = n_items;
    }
  }
}

}  // namespace dg
