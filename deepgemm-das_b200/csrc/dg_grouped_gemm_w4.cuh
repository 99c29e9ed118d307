// W4A8 grouped GEMM kernel: int8 activations x int4 weights, weights fed to the tensor cores
// through tensor memory.
//
// Orientation is swapped relative to the other kernels: the 128 output channels of a weight
// tile are the UMMA M dimension (= TMEM lanes), the tokens are the UMMA N dimension (16..128,
// chosen per work item from the number of valid rows).  The unit of pipelining is a "round"
// of 256 K values:
//   weight ring (kW4WStages x 16 KB)  TMA loads of packed weight tiles [128 channels][128 B]
//            = 256 int4 values per channel, one contiguous 16 KB span per tile.  The unpack
//            warps (one thread per channel) read their 128-byte row into registers and
//            release the stage at once.
//   round slots (kW4Rounds)  each = a 32 KB token stage (two [128 tokens][128 B] tiles, UMMA B
//            operand, TMA from L2; only the first 32 / 64 rows are fetched when the item has
//            no more valid rows than that) + 64 TMEM columns holding the unpacked weights of the same
//            256 K values, stored by the unpack warps with tcgen05.st: each packed word `x`
//            becomes `x & 0xF0F0F0F0` and `(x << 4) & 0xF0F0F0F0`, i.e. every nibble becomes
//            the int8 value 16*w -- the reference's rule
//            (csrc/arch/gfx936_gfx938_shared/m_grouped_w4a8_gemm_nt_masked_hipc.cu:378-381).
//            One mbarrier per slot collects the token bytes and the four unpack-warp arrivals.
//            The UMMA thread's instruction stream is what bounds the kernel (about 50 cycles per
//            tcgen05.mma whatever N is, plus everything else it executes between them), so it
//            does nothing but issue: per round eight tcgen05.mma (A from TMEM, B from shared
//            memory) and one tcgen05.commit.  A watcher warp waits on the round-full and
//            accumulator-empty barriers in its place, decodes the work items, and posts the
//            number of rounds / items that may be issued (and each item's instruction
//            descriptor) in plain shared-memory words.
// Unpacked weights never touch shared memory.
//
// TMEM: columns [0,256) two accumulators (128 channels x 128 tokens), columns [256,512) the
// four 64-column weight slots.  Accumulator lanes are channels and columns are tokens, so the
// epilogue thread of channel c writes D[token][c] per token: a warp writes 64 contiguous
// bytes per row.
#pragma once

#include "dg_grouped_gemm.cuh"

namespace dg {

constexpr int kW4WStages = 4;   // packed-weight ring, one stage per round
constexpr int kW4Rounds = 4;    // token stages = TMEM weight slots
constexpr int kW4TmemCols = 512;
constexpr int kW4AccCols = 128;
constexpr int kW4SlotBase = 256;
// The unpack and epilogue roles are instruction-latency bound with one warp per scheduler, so
// each has two groups of four warps: unpack groups alternate rounds, epilogue groups alternate
// work items (group e owns accumulator e).
constexpr int kW4Groups = 2;
// A group finds "its" stage of the weight ring by the parity of the stage's barrier, which only
// tells neighbouring fills apart: the fill before the one it waits for must be one it consumed
// itself, or it could take the barrier's initial state for its fill, read a stage that has not
// landed and arrive on the stage-empty barrier a phase early.
static_assert(kW4WStages % kW4Groups == 0, "the weight ring must be a multiple of the unpack groups");
constexpr int kW4EpiWarp0 = 2;                            // warps 2..9
constexpr int kW4UnpWarp0 = kW4EpiWarp0 + 4 * kW4Groups;  // warps 10..17
constexpr int kW4TokWarp = kW4UnpWarp0 + 4 * kW4Groups;   // warp 18
constexpr int kW4ChkWarp = kW4TokWarp + 1;                // warp 19

enum : int { SITE_W4_WEMPTY = 8, SITE_W4_TEMPTY = 9, SITE_W4_SLOT_EMPTY = 10 };

struct W4Smem {
  static constexpr int kTokBytes = 2 * 128 * kRowBytes;  // token stage of a round: two tiles
  static constexpr int kPackBytes = 128 * kRowBytes;     // packed int4 weight tile (256 values/row)
  static constexpr int off_tok = 0;
  static constexpr int off_pack = off_tok + kW4Rounds * kTokBytes;
  static constexpr int off_bar = off_pack + kW4WStages * kPackBytes;
  // wfull[W], wempty[W], rfull[R], cons[R], acc_full[2], acc_empty[2], drain
  static constexpr int kNumBars = 2 * kW4WStages + 2 * kW4Rounds + 5;
  static constexpr int off_misc = off_bar + kNumBars * 8;
  // epilogue transposition strips: [16 tokens][32 channels] bf16 per epilogue warp
  static constexpr int kEpiStripBytes = 16 * 32 * 2;
  // misc: tmem slot, abort, n_items, rounds ready, items ready, 8 instruction descriptors
  static constexpr int off_epi = (off_misc + 64 + 15) & ~15;
  static constexpr int off_table = off_epi + 4 * kW4Groups * kEpiStripBytes;
  static_assert(off_epi % 16 == 0 && off_table % 4 == 0, "strips are read with 16-byte loads");
  static constexpr int kThreads = 32 * (kW4ChkWarp + 1);
  __host__ __device__ static constexpr int total(int table_bytes) {
    return off_table + table_bytes + 1024;
  }
};

__global__ void __launch_bounds__(W4Smem::kThreads, 1)
grouped_gemm_w4_kernel(const __grid_constant__ CUtensorMap tm_tok,
                       const __grid_constant__ CUtensorMap tm_tok64,
                       const __grid_constant__ CUtensorMap tm_tok32,
                       const __grid_constant__ CUtensorMap tm_w, const KernelParams p) {
  using L = W4Smem;
  constexpr int WS = kW4WStages, RS = kW4Rounds;
  // s8 x s8 -> s32, M = 128; N (tokens) is filled in per work item
  constexpr uint32_t kIdescBase = umma_idesc(2u, 1u, 128, 0);

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw_addr);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  auto bar_wfull = [&](int s) { return base + L::off_bar + 8u * s; };
  auto bar_wempty = [&](int s) { return base + L::off_bar + 8u * (WS + s); };
  auto bar_rfull = [&](int s) { return base + L::off_bar + 8u * (2 * WS + s); };
  auto bar_cons = [&](int s) { return base + L::off_bar + 8u * (2 * WS + RS + s); };
  auto bar_acc_full = [&](int b) { return base + L::off_bar + 8u * (2 * WS + 2 * RS + b); };
  auto bar_acc_empty = [&](int b) { return base + L::off_bar + 8u * (2 * WS + 2 * RS + 2 + b); };
  const uint32_t bar_drain = base + L::off_bar + 8u * (2 * WS + 2 * RS + 4);

  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::off_misc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::off_misc + 4);
  volatile int* n_items_s = reinterpret_cast<volatile int*>(smem + L::off_misc + 8);
  const uint32_t ready_addr = base + L::off_misc + 12;  // rounds whose round-full barrier was seen complete
  const uint32_t items_addr = base + L::off_misc + 16;  // items whose accumulator is free and whose descriptor is posted
  volatile uint32_t* idesc_ring = reinterpret_cast<volatile uint32_t*>(smem + L::off_misc + 20);
  int32_t* tbl = reinterpret_cast<int32_t*>(smem + L::off_table);

  if (tid == 0) {
    *abort_flag = 0;
    *reinterpret_cast<volatile uint32_t*>(smem + L::off_misc + 12) = 0;
    *reinterpret_cast<volatile uint32_t*>(smem + L::off_misc + 16) = 0;
    for (int s = 0; s < WS; ++s) {
      mbar_init(bar_wfull(s), 1);
      mbar_init(bar_wempty(s), 4);  // the four warps of the unpack group that owns the stage
    }
    for (int s = 0; s < RS; ++s) {
      mbar_init(bar_rfull(s), 5);  // token producer (with the byte count) + four unpack warps
      mbar_init(bar_cons(s), 1);   // one commit of the UMMA thread
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_acc_full(b), 1);
      mbar_init(bar_acc_empty(b), 4);
    }
    mbar_init(bar_drain, 1);
    fence_mbar_init();
    tma_prefetch_desc(&tm_tok);
    tma_prefetch_desc(&tm_tok64);
    tma_prefetch_desc(&tm_tok32);
    tma_prefetch_desc(&tm_w);
  }

  // Schedule table, as in grouped_gemm_kernel (p.n_tiles = ceil(N / 128) channel tiles).
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
        *n_items_s = running * p.n_tiles;
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
      if (lane == 0) *n_items_s = count * p.n_tiles;
      if (__any_sync(0xffffffffu, bad) && lane == 0 && blockIdx.x == 0 && p.status != nullptr)
        atomicCAS(p.status, DG_DEV_OK, DG_DEV_BAD_GROUP_INDEX);
    }
  }

  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), kW4TmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();

  const uint32_t tmem_base = *tmem_slot;
  const int n_items = *n_items_s;
  const int wblocks = p.kblocks;  // weight stages per item: K / 256

  if (warp == 0) {
    if (lane == 0) {
      // ---- weight producer: one 16 KB packed tile (256 K values) per stage, streamed once
      const uint64_t pol_w = l2_policy_evict_first();
      ItemDecoder dec(p, tbl, 128, p.n_tiles);
      uint32_t it = 0;
      bool ok = true;
      for (int item = blockIdx.x; ok && item < n_items; item += gridDim.x) {
        const TileCoord t = dec.get(item);
        const int w_row0 = t.g * wblocks * p.N + t.n0;
        for (int wb = 0; wb < wblocks; ++wb, ++it) {
          const int s = it % WS;
          const uint32_t ph = (it / WS) & 1u;
          if (!mbar_wait_bounded(bar_wempty(s), ph ^ 1u, abort_flag, SITE_W4_WEMPTY)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(bar_wfull(s), L::kPackBytes);
          tma_load_2d(base + L::off_pack + s * L::kPackBytes, &tm_w, bar_wfull(s), 0,
                      w_row0 + wb * p.N, pol_w);
        }
      }
      int local_abort = 0;
      for (int s = 0; s < WS; ++s) {
        const uint32_t fills = (it + WS - 1 - s) / WS;
        if (fills > 0 && !mbar_wait_bounded(bar_wfull(s), (fills - 1) & 1u, &local_abort,
                                            SITE_PRODUCER_DRAIN))
          *abort_flag = SITE_PRODUCER_DRAIN;
      }
    }
  } else if (warp == kW4TokWarp) {
    if (lane == 0) {
      // ---- token producer: two [128 tokens][128 B] tiles per round (L2 resident)
      const uint64_t pol_tok = l2_policy_evict_last();
      ItemDecoder dec(p, tbl, 128, p.n_tiles);
      uint32_t it = 0;
      bool ok = true;
      for (int item = blockIdx.x; ok && item < n_items; item += gridDim.x) {
        const TileCoord t = dec.get(item);
        // fetch 32, 64 or 128 token rows: what the UMMA reads is rows_valid rounded up to 16
        const int box_rows = t.rows_valid <= 32 ? 32 : (t.rows_valid <= 64 ? 64 : 128);
        const CUtensorMap* tm = box_rows == 128 ? &tm_tok : (box_rows == 64 ? &tm_tok64 : &tm_tok32);
        const uint32_t round_bytes = 2u * static_cast<uint32_t>(box_rows) * kRowBytes;
        for (int wb = 0; wb < wblocks; ++wb, ++it) {
          const int s = it % RS;
          const uint32_t ph = (it / RS) & 1u;
          if (!mbar_wait_bounded(bar_cons(s), ph ^ 1u, abort_flag, SITE_W4_TEMPTY)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(bar_rfull(s), round_bytes);
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint32_t dst = base + L::off_tok + s * L::kTokBytes + h * (L::kTokBytes / 2);
            if (p.mode == MODE_MASKED)
              tma_load_3d(dst, tm, bar_rfull(s), (2 * wb + h) * 128, t.row0, t.g, pol_tok);
            else
              tma_load_2d(dst, tm, bar_rfull(s), (2 * wb + h) * 128, t.row0, pol_tok);
          }
        }
      }
      // the round-full barriers also need the unpack warps; only wait for this thread's copies
      // through the consumer: every issued round is consumed unless the block is aborting
      if (*abort_flag) {
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) {
        }
      }
    }
  } else if (warp == kW4ChkWarp) {
    if (lane == 0) {
      // ---- barrier watcher: waits for the round-full barriers in order and publishes the
      // number of complete rounds in a plain shared-memory word, which is all the UMMA thread
      // reads
      ItemDecoder dec(p, tbl, 128, p.n_tiles);
      uint32_t it = 0, tile = 0;
      bool ok = true;
      for (int item = blockIdx.x; ok && item < n_items; item += gridDim.x, ++tile) {
        // the item's instruction descriptor (s8 x s8 -> s32, M = 128, N = its tokens rounded up
        // to 16) and its accumulator, posted before its rounds
        const TileCoord t = dec.get(item);
        const uint32_t n_tok = static_cast<uint32_t>((max(t.rows_valid, 1) + 15) & ~15);
        if (!mbar_wait_bounded(bar_acc_empty(tile & 1u), ((tile >> 1) & 1u) ^ 1u, abort_flag,
                               SITE_MMA_ACC_EMPTY))
          break;
        idesc_ring[tile & 7u] = kIdescBase | ((n_tok >> 3) << 17);
        asm volatile("st.release.cta.shared::cta.u32 [%0], %1;" ::"r"(items_addr), "r"(tile + 1u) : "memory");
        for (int wb = 0; wb < wblocks; ++wb) {
          if (!mbar_wait_bounded(bar_rfull(it % RS), (it / RS) & 1u, abort_flag, SITE_MMA_FULL)) {
            ok = false;
            break;
          }
          ++it;
          asm volatile("st.release.cta.shared::cta.u32 [%0], %1;" ::"r"(ready_addr), "r"(it) : "memory");
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- UMMA issuer: per round, A (weights) from TMEM slot s, B (tokens) from token stage s.
      // This thread's instruction stream bounds the kernel, so it neither decodes work items
      // nor touches an mbarrier: the watcher warp posts, in plain shared-memory words, how
      // many items (descriptor ready, accumulator free) and rounds (weights and tokens in
      // place) may be issued, and this thread re-reads a word only when its last copy is used up.
      // Ordering: the watcher observes the mbarrier (acquire), then publishes with st.release;
      // this thread's volatile loads of one shared-memory word after another are performed in
      // program order, and tcgen05.fence::after_thread_sync orders the UMMAs after the load
      // that saw the new count.  The operands themselves are read by the tensor core only.
      auto poll_above = [&](uint32_t addr, uint32_t have, int site) -> uint32_t {
        // returns a value > have, or 0 after giving up (abort flag set); the timer is only read
        // once the word has been found unchanged a few times (reading it costs ~100 cycles)
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
      uint32_t it = 0, tile = 0, rounds_known = 0, items_known = 0;
      bool ok = true;
      for (int item = blockIdx.x; ok && item < n_items; item += gridDim.x, ++tile) {
        if (items_known <= tile && (items_known = poll_above(items_addr, tile, SITE_MMA_ACC_EMPTY)) == 0) {
          ok = false;
          break;
        }
        const uint32_t idesc = idesc_ring[tile & 7u];
        const uint32_t buf = tile & 1u;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * kW4AccCols;
        for (int wb = 0; wb < wblocks; ++wb, ++it) {
          const int s = it % RS;
          if (rounds_known <= it) {
            if ((rounds_known = poll_above(ready_addr, it, SITE_MMA_FULL)) == 0) {
              ok = false;
              break;
            }
            tc_fence_after_sync();  // orders the UMMAs of every round learnt of here after the unpack warps' stores
          }
          const uint32_t a_tmem = tmem_base + kW4SlotBase + s * 64;
          const uint64_t b_desc = umma_desc_sw128(base + L::off_tok + s * L::kTokBytes);
#pragma unroll
          for (int k = 0; k < 8; ++k)  // k / 4 selects the 128-value half: +16 KB of tokens
            umma_ts_i8(d_tmem, a_tmem + 8u * k, b_desc + (k >= 4 ? 1024u : 0u) + 2u * (k & 3), idesc,
                       (wb | k) != 0 ? 1u : 0u);
          umma_commit(bar_cons(s));  // frees token stage s and weight slot s
        }
        if (ok) umma_commit(bar_acc_full(buf));
      }
      if (*abort_flag) {
        int local_abort = 0;
        umma_commit(bar_drain);
        mbar_wait_bounded(bar_drain, 0, &local_abort, 0);
      }
    }
  } else if (warp < kW4UnpWarp0) {
    // ---- epilogue: thread = one output channel (TMEM lane), columns = tokens; this warp's
    // group handles every second item of the block (the ones accumulated in its buffer)
    const int q = warp & 3;
    const uint32_t group = static_cast<uint32_t>(warp - kW4EpiWarp0) >> 2;
    ItemDecoder dec(p, tbl, 128, p.n_tiles);
    uint32_t tile = 0;
    for (int item = blockIdx.x; item < n_items; item += gridDim.x, ++tile) {
      const uint32_t buf = tile & 1u;
      if (buf != group) continue;
      const TileCoord t = dec.get(item);
      const uint32_t aph = (tile >> 1) & 1u;
      // Everything that depends only on the item's coordinates is fetched before waiting for
      // the accumulator, so that the global-load latency hides behind the main loop: this
      // channel's weight scale, and (lane l) the activation scale and validity of tokens
      // l, 32+l, 64+l, 96+l.
      const int chan = t.n0 + q * 32 + lane;
      const bool chan_ok = chan < p.N;
      const float bs = !chan_ok ? 0.0f
                       : (p.scale_mode == DG_SCALE_TENSOR_WISE ? p.b_scale[t.g]
                                                                : p.b_scale[(size_t)t.g * p.N + chan]);
      const size_t row_base = (p.mode == MODE_MASKED ? (size_t)t.g * p.M : (size_t)0) + t.row0;
      float as_l[4];
      unsigned tok_mask[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        bool okl = false;
        as_l[c] = 0.0f;
        if (c * 32 + lane < t.rows_valid) {
          const size_t row = row_base + c * 32 + lane;
          okl = (p.mode == MODE_MASKED) || (p.sched[row] >= 0);
          as_l[c] = p.a_scale[row];
        }
        tok_mask[c] = __ballot_sync(0xffffffffu, okl);
      }
      if (!mbar_wait_warp(bar_acc_full(buf), aph, abort_flag, SITE_EPI_ACC_FULL)) break;
      tc_fence_after_sync();
      const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * kW4AccCols;
      // 16 tokens per step.  A lane holds one channel of 16 tokens, but D is token-major, so the
      // step goes through a [16 tokens][32 channels] strip of shared memory: 16 two-byte
      // writes per lane, then every lane stores two 16-byte pieces (8 channels of one token),
      // 2 global store instructions per lane and step instead of 16.  The step loop stays
      // rolled to keep the code small (the fully unrolled form stalled on instruction fetch).
      __nv_bfloat16* strip = reinterpret_cast<__nv_bfloat16*>(
          smem + L::off_epi + (warp - kW4EpiWarp0) * L::kEpiStripBytes);
      const int piece_chan = t.n0 + q * 32 + (lane & 3) * 8;   // first channel of this lane's pieces
#pragma unroll 1
      for (int c = 0; c * 16 < t.rows_valid; ++c) {
        const int w = c >> 1;  // which of the four prefetched 32-token groups
        const float as_w = w == 0 ? as_l[0] : (w == 1 ? as_l[1] : (w == 2 ? as_l[2] : as_l[3]));
        const unsigned m_w =
            (w == 0 ? tok_mask[0] : (w == 1 ? tok_mask[1] : (w == 2 ? tok_mask[2] : tok_mask[3]))) >>
            ((c & 1) * 16);
        uint32_t r[16];
        tmem_ld_32x16(t_lane + c * 16, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float as_j = __shfl_sync(0xffffffffu, as_w, (c & 1) * 16 + j);
          const float v = (__int2float_rn(static_cast<int>(r[j])) * as_j) * bs;
          if (p.out_kind == 1)  // fp16 output: same 16-bit slots
            reinterpret_cast<__half*>(strip)[j * 32 + lane] = __float2half_rn(v);
          else
            strip[j * 32 + lane] = __float2bfloat16_rn(v);
        }
        if (p.debug_acc != nullptr && chan_ok) {  // raw accumulators (tests only): direct stores
          uint32_t* dbg_col = p.debug_acc + (row_base + c * 16) * p.N + chan;
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if ((m_w >> j) & 1u) dbg_col[(size_t)j * p.N] = r[j];
        }
        __syncwarp();
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int tok = (lane >> 2) + 8 * h;  // token of the step this lane stores a piece of
          if (((m_w >> tok) & 1u) && piece_chan < p.N) {
            const uint4 v16 = *reinterpret_cast<const uint4*>(strip + tok * 32 + (lane & 3) * 8);
            *reinterpret_cast<uint4*>(p.d + (row_base + c * 16 + tok) * p.N + piece_chan) = v16;
          }
        }
        __syncwarp();  // the strip is rewritten by the next step
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_acc_empty(buf));
    }
  } else {
    // ---- unpack: thread = one weight row (channel) of the tile = one TMEM lane; this warp's
    // group handles every second round
    const int q = warp & 3;
    const uint32_t group = static_cast<uint32_t>(warp - kW4UnpWarp0) >> 2;
    const int r_row = q * 32 + lane;
    const int sw = r_row & 7;  // 128-byte swizzle: 16-byte chunk index ^= row % 8
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + kW4SlotBase;
    uint32_t it = 0;
    bool ok = true;
    for (int item = blockIdx.x; ok && item < n_items; item += gridDim.x) {
      for (int wb = 0; ok && wb < wblocks; ++wb, ++it) {
        if (it % kW4Groups != group) continue;
        const int ws = it % WS;
        const uint32_t wph = (it / WS) & 1u;
        if (!mbar_wait_warp(bar_wfull(ws), wph, abort_flag, SITE_UNPACK_FULL)) {
          ok = false;
          break;
        }
        // chunk j of the row: byte i = w[32j+i] (high nibble) | w[32j+16+i] (low nibble)
        const uint8_t* src = smem + L::off_pack + ws * L::kPackBytes + r_row * kRowBytes;
        uint32_t lo[32], hi[32];  // K values [0,128) and [128,256) of the round, 4 per word
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint4 c = *reinterpret_cast<const uint4*>(src + ((j ^ sw) << 4));
          const uint32_t w[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const uint32_t a = w[u] & 0xF0F0F0F0u;         // k = 32j + 4u .. +3
            const uint32_t b = (w[u] << 4) & 0xF0F0F0F0u;  // k = 32j + 16 + 4u .. +3
            if (j < 4) {
              lo[8 * j + u] = a;
              lo[8 * j + 4 + u] = b;
            } else {
              hi[8 * (j - 4) + u] = a;
              hi[8 * (j - 4) + 4 + u] = b;
            }
          }
        }
        __syncwarp();  // the row is in registers: hand the shared-memory stage back
        if (lane == 0) mbar_arrive(bar_wempty(ws));
        const int s = it % RS;
        const uint32_t ph = (it / RS) & 1u;
        if (!mbar_wait_warp(bar_cons(s), ph ^ 1u, abort_flag, SITE_W4_SLOT_EMPTY)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        tmem_st_32x32(lane_addr + s * 64, lo);
        tmem_st_32x32(lane_addr + s * 64 + 32, hi);
        tmem_st_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_rfull(s));
      }
    }
  }

  // ---- tear-down
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kW4TmemCols);
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
