// W4A8 grouped GEMM kernel: int8 activations x int4 weights, the int4 -> int8 unpack done in
// shared memory.
//
// Same orientation as the 8-bit kernels: the tokens of a work item are the UMMA M dimension
// (128 rows, or 64 for items of at most 64 rows), 256 output channels are the UMMA N dimension,
// accumulators live in TMEM (two buffers of 256 columns) and the epilogue is the one of
// grouped_gemm_kernel (rows on TMEM lanes, coalesced 16-byte stores).  One tcgen05.mma covers
// 32 K values of 256 channels = 4 KB of packed weights.
//
// Pipeline per K block of 128 values:
//   packed ring (P stages x 16 KB)   TMA loads of [256 channels][64 bytes]: the half of every
//            128-byte packed row that holds this K block (a packed row is 256 int4 values:
//            chunks 0..3 = first K block, 4..7 = second).  No swizzle: the tile is read
//            linearly, one 16-byte chunk per lane, which is conflict-free.
//   token ring (TOKS x 16 KB)        [128 tokens][128 B] int8 activations by TMA (SWIZZLE_128B),
//            fetched ahead of their use like the weights (a tile requested only when its
//            weight slot frees would put the L2 latency into every K block).
//   weight slots (SLOTS x 32 KB)     [256 channels][128 B] int8 weights written by the unpack
//            warps in the same swizzled K-major layout.  Chunk j of a packed row, `x`, becomes two 16-byte
//            chunks: `x & 0xF0F0F0F0` (K values 32j .. 32j+15) and `(x << 4) & 0xF0F0F0F0`
//            (32j+16 .. 32j+31), every nibble turning into the int8 value 16*w -- the
//            reference's rule (csrc/arch/gfx936_gfx938_shared/m_grouped_w4a8_gemm_nt_masked_hipc.cu:378-381).
//            A warp instruction covers 8 rows x 4 chunks; rows r and r+1 of a pair differ in
//            bit 0 of the swizzle, so the eight lanes of a quarter warp hit eight different
//            16-byte columns on the store side too.  fence.proxy.async orders the stores
//            before the tensor core's reads.
//   The UMMA thread's instruction stream is the scarce resource (a wait on an mbarrier costs it
//   about 200 cycles, a commit 60, an issue 50): it touches no barrier.  A watcher warp waits for
//   the token tile and the weight slot of each K block (and for a free accumulator per item) and
//   posts counters in plain shared-memory words; the UMMA thread issues four tcgen05.mma per K
//   block and one commit to the K block's "consumed" barrier, which frees the weight slot and
//   the token tile together (a ring of barriers, so that a waiter can name the K block whose
//   resources it re-uses).
//
// Accumulators carry sum a * (16 w); the caller's weight scale carries the 1/16
// (op_test/test_deepgemm_masked_w4a8_hipc.py:67,89).
#pragma once

#include "dg_grouped_gemm.cuh"

namespace dg {

constexpr int kWsBN = 256;                            // output channels per work item
constexpr int kWsUnpackWarps = 8;
constexpr int kWsPackStageBytes = kWsBN * 64;         // packed weights of one K block
constexpr int kWsTokBytes = kATileBytes;              // 128 tokens x 128 B
constexpr int kWsSlotBytes = kWsBN * kRowBytes;       // 256 channels x 128 B, unpacked
constexpr int kWsMaxPackStages = 8;
constexpr int kWsEpiWarp0 = 2;                        // warps 2..5
constexpr int kWsTokWarp = 6;
constexpr int kWsUnpWarp0 = 7;                        // warps 7..14
constexpr int kWsChkWarp = kWsUnpWarp0 + kWsUnpackWarps;  // warp 15: barrier watcher
// Ring of "K block consumed" barriers: K block i commits to barrier i % kWsCons.  A waiter names
// the K block j it needs (barrier j % kWsCons, phase j / kWsCons); the ring must be at least as
// long as the unpack groups' stride and the slot / token rings, so that a waiter is never two
// phases away from the barrier's current one.
constexpr int kWsCons = 8;

enum : int { SITE_WS_PACK_EMPTY = 8, SITE_WS_TOK_EMPTY = 9, SITE_WS_SLOT_EMPTY = 10,
             SITE_WS_PACK_FULL = 11, SITE_WS_TOK_FULL = 12 };

template <int SLOTS, int TOKS>
struct WsSmem {
  static constexpr int off_slot = 0;
  static constexpr int off_tok = off_slot + SLOTS * kWsSlotBytes;
  static constexpr int off_bar = off_tok + TOKS * kWsTokBytes;
  static constexpr int kCons = kWsCons;
  static_assert(kCons >= SLOTS && kCons >= TOKS, "consumed ring too short");
  // pack_full[8], pack_empty[8], slot_full[SLOTS], tok_full[TOKS], consumed[kCons],
  // acc_full[2], acc_empty[2], drain
  static constexpr int kNumBars = 2 * kWsMaxPackStages + SLOTS + TOKS + kCons + 5;
  // misc: tmem slot, abort, n_items, split_from, K blocks ready, items ready, 8 instruction descriptors
  static constexpr int off_misc = off_bar + kNumBars * 8;
  static constexpr int off_bs = (off_misc + 64 + 15) & ~15;  // weight scales of a tile, one strip per epilogue warp
  static constexpr int off_epi = off_bs + 4 * kWsBN * 4;     // store strips: 32 rows x 64 B per epilogue warp
  static constexpr int off_table = off_epi + 4 * 2048;
  static_assert(off_bs % 16 == 0 && off_epi % 16 == 0 && off_table % 4 == 0, "16-byte accesses");
  static constexpr int kThreads = 32 * (kWsChkWarp + 1);
  // the packed ring follows the schedule table
  __host__ __device__ static constexpr int pack_offset(int table_bytes) {
    return (off_table + table_bytes + 127) & ~127;
  }
  __host__ __device__ static constexpr int total(int table_bytes, int pack_stages) {
    return pack_offset(table_bytes) + pack_stages * kWsPackStageBytes + 1024;  // + alignment slack
  }
};

template <int SLOTS, int TOKS, int NG>
__global__ void __launch_bounds__(WsSmem<SLOTS, TOKS>::kThreads, 1)
grouped_gemm_w4_smem_kernel(const __grid_constant__ CUtensorMap tm_tok,
                            const __grid_constant__ CUtensorMap tm_tok64,
                            const __grid_constant__ CUtensorMap tm_tok32,
                            const __grid_constant__ CUtensorMap tm_tok8,
                            const __grid_constant__ CUtensorMap tm_w,
                            const __grid_constant__ CUtensorMap tm_w128, const KernelParams p) {
  using L = WsSmem<SLOTS, TOKS>;
  constexpr uint32_t kIdescBase = umma_idesc(2u, 1u, kBM, kWsBN);  // s8 x s8 -> s32

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw_addr);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int P = p.pack_stages;
  const uint32_t pack_base = base + p.pack_off;

  auto bar_pfull = [&](int s) { return base + L::off_bar + 8u * s; };
  auto bar_pempty = [&](int s) { return base + L::off_bar + 8u * (kWsMaxPackStages + s); };
  auto bar_sfull = [&](int u) { return base + L::off_bar + 8u * (2 * kWsMaxPackStages + u); };
  constexpr int kCons = L::kCons;
  constexpr int kBar0 = 2 * kWsMaxPackStages + SLOTS;
  auto bar_tfull = [&](int a) { return base + L::off_bar + 8u * (kBar0 + a); };
  auto bar_cons = [&](int c) { return base + L::off_bar + 8u * (kBar0 + TOKS + c); };
  auto bar_acc_full = [&](int b) { return base + L::off_bar + 8u * (kBar0 + TOKS + kCons + b); };
  auto bar_acc_empty = [&](int b) { return base + L::off_bar + 8u * (kBar0 + TOKS + kCons + 2 + b); };
  const uint32_t bar_drain = base + L::off_bar + 8u * (kBar0 + TOKS + kCons + 4);

  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::off_misc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::off_misc + 4);
  volatile int* n_items_s = reinterpret_cast<volatile int*>(smem + L::off_misc + 8);
  volatile int* split_from_s = reinterpret_cast<volatile int*>(smem + L::off_misc + 12);
  const uint32_t ready_addr = base + L::off_misc + 16;  // K blocks whose tokens and weights were seen in place
  const uint32_t items_addr = base + L::off_misc + 20;  // items whose accumulator is free and whose descriptor is posted
  volatile uint32_t* idesc_ring = reinterpret_cast<volatile uint32_t*>(smem + L::off_misc + 24);
  int32_t* tbl = reinterpret_cast<int32_t*>(smem + L::off_table);
  // Waits until K block `it - lag` of this block has been consumed by the tensor core, i.e. until
  // the resource that K block `it` re-uses is free (nothing to wait for during the first `lag`).
  auto wait_consumed = [&](uint32_t it, uint32_t lag, int site) -> bool {
    if (it < lag) return true;
    const uint32_t j = it - lag;
    return mbar_wait_bounded(bar_cons(j % kCons), (j / kCons) & 1u, abort_flag, site);
  };

  if (tid == 0) {
    *abort_flag = 0;
    *reinterpret_cast<volatile uint32_t*>(smem + L::off_misc + 16) = 0;
    *reinterpret_cast<volatile uint32_t*>(smem + L::off_misc + 20) = 0;
    for (int s = 0; s < kWsMaxPackStages; ++s) {
      mbar_init(bar_pfull(s), 1);
      mbar_init(bar_pempty(s), kWsUnpackWarps / NG);  // the warps of the unpack group that owns the K block
    }
    for (int u = 0; u < SLOTS; ++u) {
      mbar_init(bar_sfull(u), kWsUnpackWarps / NG);  // one arrival per warp of the owning unpack group
    }
    for (int a = 0; a < TOKS; ++a) mbar_init(bar_tfull(a), 1);
    for (int c = 0; c < kCons; ++c) mbar_init(bar_cons(c), 1);  // one commit of the UMMA thread
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_acc_full(b), 1);
      mbar_init(bar_acc_empty(b), 4);
    }
    mbar_init(bar_drain, 1);
    fence_mbar_init();
    tma_prefetch_desc(&tm_tok);
    tma_prefetch_desc(&tm_w);
  }

  // Schedule table, as in grouped_gemm_kernel (p.n_tiles = ceil(N / 256) channel tiles).
  if (p.mode == MODE_MASKED) {
    int32_t* cnt = tbl;
    int32_t* pref = tbl + p.G;
    for (int g = tid; g < p.G; g += blockDim.x) cnt[g] = max(0, min(p.sched[g], p.M));
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
        int items = running * p.n_tiles;
        int split_from = 0x7fffffff;
        if (p.split_tail) {
          // a last round that is at most half full: its tiles are split into two 128-channel halves
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
    for (int b = tid; b < p.m_blocks; b += blockDim.x) tbl[b] = p.sched[(size_t)b * kBM];
    __syncthreads();
    if (warp == 0) {
      int count = 0;
      bool bad = false;
      for (int b0 = 0; b0 < p.m_blocks; b0 += 32) {
        const int b = b0 + lane;
        const int e = (b < p.m_blocks) ? tbl[b] : -1;
        const bool ok = (e >= 0) && (e < p.G);
        bad |= (e >= p.G);
        const unsigned mask = __ballot_sync(0xffffffffu, ok);
        __syncwarp();
        if (ok) tbl[count + __popc(mask & ((1u << lane) - 1u))] = (e << 16) | b;
        count += __popc(mask);
        __syncwarp();
      }
      if (lane == 0) {
        *split_from_s = 0x7fffffff;
        *n_items_s = count * p.n_tiles;
      }
      if (__any_sync(0xffffffffu, bad) && lane == 0 && blockIdx.x == 0 && p.status != nullptr)
        atomicCAS(p.status, DG_DEV_OK, DG_DEV_BAD_GROUP_INDEX);
    }
  }

  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();

  const uint32_t tmem_base = *tmem_slot;
  const int n_items = *n_items_s;
  const int split_from = *split_from_s;
  const int kblocks = p.kblocks;  // K / 128

  if (warp == 0) {
    if (lane == 0) {
      // ---- weight producer: the packed half rows of one K block per stage, streamed once
      const uint64_t pol_w = l2_policy_evict_first();
      ItemDecoder dec(p, tbl, kWsBN, p.n_tiles, split_from);
      int ps = 0;
      uint32_t pph = 0;
      bool ok = true;
      for (int item = blockIdx.x; ok && item < n_items; item += gridDim.x) {
        const TileCoord t = dec.get(item);
        const CUtensorMap* tm = t.width == kWsBN ? &tm_w : &tm_w128;
        const uint32_t bytes = static_cast<uint32_t>(t.width) * 64u;
        const int row0 = t.g * (kblocks >> 1) * p.N + t.n0;  // packed row of K block 0
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait_bounded(bar_pempty(ps), pph ^ 1u, abort_flag, SITE_WS_PACK_EMPTY)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(bar_pfull(ps), bytes);
          tma_load_2d(pack_base + ps * kWsPackStageBytes, tm, bar_pfull(ps), (kb & 1) * 64,
                      row0 + (kb >> 1) * p.N, pol_w);
          if (++ps == P) {
            ps = 0;
            pph ^= 1u;
          }
        }
      }
    }
  } else if (warp == kWsTokWarp) {
    if (lane == 0) {
      // ---- token producer: one [rows][128 B] activation tile per K block (L2 resident)
      const uint64_t pol_tok = l2_policy_evict_last();
      ItemDecoder dec(p, tbl, kWsBN, p.n_tiles, split_from);
      int u = 0;
      uint32_t it = 0;
      bool ok = true;
      for (int item = blockIdx.x; ok && item < n_items; item += gridDim.x) {
        const TileCoord t = dec.get(item);
        const int a_rows = t.rows_valid <= 8 ? 8 : (t.rows_valid <= 32 ? 32 : (t.rows_valid <= 64 ? 64 : kBM));
        const CUtensorMap* tm = a_rows == kBM ? &tm_tok
                                : (a_rows == 64 ? &tm_tok64 : (a_rows == 32 ? &tm_tok32 : &tm_tok8));
        const uint32_t bytes = static_cast<uint32_t>(a_rows) * kRowBytes;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          if (!wait_consumed(it, TOKS, SITE_WS_TOK_EMPTY)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(bar_tfull(u), bytes);
          const uint32_t dst = base + L::off_tok + u * kWsTokBytes;
          if (p.mode == MODE_MASKED)
            tma_load_3d(dst, tm, bar_tfull(u), kb * 128, t.row0, t.g, pol_tok);
          else
            tma_load_2d(dst, tm, bar_tfull(u), kb * 128, t.row0, pol_tok);
          if (++u == TOKS) u = 0;
        }
      }
    }
  } else if (warp == kWsChkWarp) {
    if (lane == 0) {
      // ---- barrier watcher: waits in the UMMA thread's place and publishes, in plain
      // shared-memory words, how many items (accumulator free, instruction descriptor posted)
      // and K blocks (tokens and unpacked weights in place) may be issued
      ItemDecoder dec(p, tbl, kWsBN, p.n_tiles, split_from);
      int u = 0, a = 0;
      uint32_t uph = 0, tph = 0, it = 0, tile = 0;
      bool ok = true;
      for (int item = blockIdx.x; ok && item < n_items; item += gridDim.x, ++tile) {
        const TileCoord t = dec.get(item);
        // N = the item's width; M = 64 for items of at most 64 rows (row r then sits in TMEM lane
        // 32 * (r / 16) + r % 16)
        const uint32_t idesc = (kIdescBase & ~(0x3Fu << 17) & ~(0x1Fu << 24)) |
                               (static_cast<uint32_t>(t.width >> 3) << 17) |
                               ((t.rows_valid <= 64 ? 4u : 8u) << 24);
        if (!mbar_wait_bounded(bar_acc_empty(tile & 1u), ((tile >> 1) & 1u) ^ 1u, abort_flag,
                               SITE_MMA_ACC_EMPTY))
          break;
        idesc_ring[tile & 7u] = idesc;
        asm volatile("st.release.cta.shared::cta.u32 [%0], %1;" ::"r"(items_addr), "r"(tile + 1u) : "memory");
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait_bounded(bar_tfull(a), tph, abort_flag, SITE_WS_TOK_FULL)) {
            ok = false;
            break;
          }
          if (!mbar_wait_bounded(bar_sfull(u), uph, abort_flag, SITE_MMA_FULL)) {
            ok = false;
            break;
          }
          ++it;
          asm volatile("st.release.cta.shared::cta.u32 [%0], %1;" ::"r"(ready_addr), "r"(it) : "memory");
          if (++u == SLOTS) {
            u = 0;
            uph ^= 1u;
          }
          if (++a == TOKS) {
            a = 0;
            tph ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- UMMA issuer: A = token tile a, B = unpacked weights of slot u.  Ordering: the watcher
      // observes the mbarriers (acquire), then publishes with st.release; this thread's volatile
      // loads of one shared-memory word after another are performed in program order, and
      // tcgen05.fence::after_thread_sync orders the UMMAs after the load that saw the new count.
      auto poll_above = [&](uint32_t addr, uint32_t have, int site) -> uint32_t {
        // returns a value > have, or 0 after giving up (abort flag set); the timer is only read
        // once the word has been found unchanged a few times
        uint32_t v;
#pragma unroll 1
        for (int i = 0; i < 16; ++i) {
          asm volatile("ld.volatile.shared::cta.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
          if (v > have) return v;
        }
        const uint64_t t0 = global_timer_ns();
        uint32_t spins = 0;
        while (true) {
          asm volatile("ld.volatile.shared::cta.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
          if (v > have) return v;
          if ((++spins & 63u) == 0 && (*abort_flag || global_timer_ns() - t0 > 1500000000ull)) {
            if (!*abort_flag) *abort_flag = site;
            return 0;
          }
        }
      };
      int u = 0, a = 0;
      uint32_t it = 0, tile = 0, ready_known = 0, items_known = 0;
      bool ok = true;
      for (int item = blockIdx.x; ok && item < n_items; item += gridDim.x, ++tile) {
        if (items_known <= tile && (items_known = poll_above(items_addr, tile, SITE_MMA_ACC_EMPTY)) == 0) {
          ok = false;
          break;
        }
        const uint32_t idesc = idesc_ring[tile & 7u];
        const uint32_t buf = tile & 1u;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * kWsBN;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          if (ready_known <= it) {
            if ((ready_known = poll_above(ready_addr, it, SITE_MMA_FULL)) == 0) {
              ok = false;
              break;
            }
            tc_fence_after_sync();
          }
          const uint64_t a_desc = umma_desc_sw128(base + L::off_tok + a * kWsTokBytes);
          const uint64_t b_desc = umma_desc_sw128(base + L::off_slot + u * kWsSlotBytes);
#pragma unroll
          for (int k = 0; k < kRowBytes / 32; ++k)
            umma_ss<UMMA_I8>(d_tmem, a_desc + 2u * k, b_desc + 2u * k, idesc, (kb | k) != 0 ? 1u : 0u);
          umma_commit(bar_cons(it % kCons));  // frees the slot and the token tile once these UMMAs have read them
          if (++u == SLOTS) u = 0;
          if (++a == TOKS) a = 0;
        }
        if (ok) umma_commit(bar_acc_full(buf));
      }
      if (*abort_flag) {
        int local_abort = 0;
        umma_commit(bar_drain);
        mbar_wait_bounded(bar_drain, 0, &local_abort, 0);
      }
    }
  } else if (warp < kWsTokWarp) {
    // ---- epilogue: this warp may touch TMEM lanes [32q, 32q+32); same as grouped_gemm_kernel
    const int q = warp & 3;
    ItemDecoder dec(p, tbl, kWsBN, p.n_tiles, split_from);
    uint32_t tile = 0;
    for (int item = blockIdx.x; item < n_items; item += gridDim.x, ++tile) {
      const TileCoord t = dec.get(item);
      const bool m64 = t.rows_valid <= 64;
      const int rows_per_warp = m64 ? 16 : 32;
      const int row_in_tile = q * rows_per_warp + lane;
      const uint32_t buf = tile & 1u;
      const uint32_t aph = (tile >> 1) & 1u;
      float* bs_s = reinterpret_cast<float*>(smem + L::off_bs) + q * kWsBN;
      const bool warp_has_rows = t.rows_valid > q * rows_per_warp;  // warp-uniform
      bool rv = false;
      size_t grow = 0;
      EpiRow row;
      row.as = 1.0f;
      row.bs_g = 1.0f;
      if (warp_has_rows) {
        stage_tile_scales(bs_s, p.b_scale + (size_t)t.g * p.N, t.n0, t.width, p.N, lane,
                          p.scale_mode == DG_SCALE_PER_CHANNEL);
        rv = lane < rows_per_warp && row_in_tile < t.rows_valid;
        grow = (p.mode == MODE_MASKED ? (size_t)t.g * p.M : (size_t)0) + t.row0 + row_in_tile;
        if (p.mode == MODE_CONTIG && rv) rv = p.sched[grow] >= 0;
        if (rv) row.as = p.a_scale[grow];
        if (p.scale_mode == DG_SCALE_TENSOR_WISE) row.bs_g = p.b_scale[t.g];
      }
      if (!mbar_wait_warp(bar_acc_full(buf), aph, abort_flag, SITE_EPI_ACC_FULL)) break;
      tc_fence_after_sync();
      if (warp_has_rows) {
        row.bs_row = bs_s;
        row.f16 = p.out_kind == 1;
        const size_t d_off = grow * p.N + t.n0;
        row.d_row = p.d + d_off;
        row.dbg_row = p.debug_acc ? p.debug_acc + d_off : nullptr;
        const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * kWsBN;
        const int cols_left0 = p.N - t.n0;
        EpiWarp ew;
        ew.strip = smem + L::off_epi + q * 2048;
        ew.d_warp = p.d + (grow - lane) * p.N + t.n0;
        ew.ld = static_cast<size_t>(p.N);
        ew.rv_mask = __ballot_sync(0xffffffffu, rv);
        ew.lane = lane;
        epilogue_drain<true>(t_row, min(t.width / 32, (cols_left0 + 31) / 32), rv, row, ew, p.scale_mode,
                             cols_left0, (p.N & 7) != 0, p.out_kind);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_acc_empty(buf));
    }
  } else if (warp >= kWsUnpWarp0 && warp < kWsChkWarp) {
    // ---- unpack.  The NG groups of warps take the K blocks in turn, so that a warp's own chain
    // (wait for the packed stage, load, wait for the slot, store, fence, arrive) may take NG K
    // block periods; its registers double as a staging buffer (the packed stage is handed back
    // as soon as it has been read).  Within a group, warp wi handles the 8-row groups wi,
    // wi + WPG, ... of the weight tile.  Lane l reads 16-byte chunk l of its row group's 512
    // packed bytes: row l / 4 of the group, chunk j = l % 4 of that row's 64 bytes, and writes
    // chunks 2j and 2j + 1 of the same row in the 128-byte-swizzled tile (physical chunk =
    // logical chunk ^ row % 8).
    constexpr int WPG = kWsUnpackWarps / NG;
    static_assert(kWsCons >= NG && kWsUnpackWarps % NG == 0, "unpack groups");
    const int w = warp - kWsUnpWarp0;
    const uint32_t g = static_cast<uint32_t>(w / WPG);
    const int wi = w % WPG;
    const int r = lane >> 2;
    const uint32_t src_off = static_cast<uint32_t>(lane) * 16u;
    const uint32_t hi_off = static_cast<uint32_t>(r * 128 + (((2 * (lane & 3)) ^ r) << 4));
    const uint32_t lo_off = static_cast<uint32_t>(r * 128 + (((2 * (lane & 3) + 1) ^ r) << 4));
    constexpr int kMaxIters = kWsBN / 8 / WPG;  // row groups per warp and K block
    ItemDecoder dec(p, tbl, kWsBN, p.n_tiles, split_from);
    int ps = 0, u = 0;
    uint32_t pph = 0, it = 0;
    bool ok = true;
    for (int item = blockIdx.x; ok && item < n_items; item += gridDim.x) {
      const TileCoord t = dec.get(item);
      const int groups = t.width >> 3;
      for (int kb = 0; kb < kblocks; ++kb, ++it) {
        if (it % NG == g) {
          if (!mbar_wait_warp(bar_pfull(ps), pph, abort_flag, SITE_WS_PACK_FULL)) {
            ok = false;
            break;
          }
          const uint32_t src = pack_base + ps * kWsPackStageBytes + src_off;
          uint4 v[kMaxIters];
#pragma unroll
          for (int j = 0; j < kMaxIters; ++j) {
            const int grp = wi + WPG * j;
            if (grp < groups)
              asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                           : "=r"(v[j].x), "=r"(v[j].y), "=r"(v[j].z), "=r"(v[j].w)
                           : "r"(src + grp * 512u)
                           : "memory");
          }
          __syncwarp();  // the packed rows are in registers: hand the stage back
          if (lane == 0) mbar_arrive(bar_pempty(ps));
          if (!__all_sync(0xffffffffu, wait_consumed(it, SLOTS, SITE_WS_SLOT_EMPTY))) {
            ok = false;
            break;
          }
          const uint32_t dst = base + L::off_slot + u * kWsSlotBytes;
#pragma unroll
          for (int j = 0; j < kMaxIters; ++j) {
            const int grp = wi + WPG * j;
            if (grp < groups) {
              const uint32_t d0 = dst + grp * 1024u;
              asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(d0 + hi_off),
                           "r"(v[j].x & 0xF0F0F0F0u), "r"(v[j].y & 0xF0F0F0F0u),
                           "r"(v[j].z & 0xF0F0F0F0u), "r"(v[j].w & 0xF0F0F0F0u)
                           : "memory");
              asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(d0 + lo_off),
                           "r"((v[j].x << 4) & 0xF0F0F0F0u), "r"((v[j].y << 4) & 0xF0F0F0F0u),
                           "r"((v[j].z << 4) & 0xF0F0F0F0u), "r"((v[j].w << 4) & 0xF0F0F0F0u)
                           : "memory");
            }
          }
          fence_proxy_async_smem();  // generic-proxy stores before the tensor core's reads
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_sfull(u));
        }
        if (++ps == P) {
          ps = 0;
          pph ^= 1u;
        }
        if (++u == SLOTS) u = 0;
      }
    }
  }

  // ---- tear-down
  if (*abort_flag != 0 && tid == 0) {
    // abnormal exit: give copies still in flight into this block's shared memory time to land
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) {
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
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
