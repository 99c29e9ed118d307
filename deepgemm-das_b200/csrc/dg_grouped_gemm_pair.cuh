// Two-CTA variant of the grouped GEMM kernel for compute-bound shapes (prefill).
//
// A cluster of two thread blocks on the two SMs of one TPC computes a 256-row x 256-column
// tile with tcgen05.mma.cta_group::2: block r of the pair owns rows [128r, 128r+128) of the
// tile (its A tile, its TMEM accumulator, its epilogue) and holds columns [128r, 128r+128)
// of the weight tile, which the tensor cores of both SMs read.  Per SM and K block this
// moves 32 KB into shared memory instead of the 48 KB of the one-CTA 128x256 tile, and
// leaves room for a six-stage ring.
//
// Protocol.  Each block's producer waits on its own stage-empty barrier and issues its own
// plain TMA loads (one destination each) whose byte counts complete on the LEADER's
// stage-full barrier; the leader's producer posts the expected bytes of both blocks.  The
// leader's UMMA thread issues the MMAs for the pair and commits to the stage-empty and
// accumulator-full barriers of both blocks; the epilogue warps of both blocks arrive on
// the leader's accumulator-empty barrier.  The leader's UMMA thread itself touches no barrier:
// a watcher warp waits on stage-full and accumulator-empty in its place and posts counters in
// plain shared-memory words (0.745 -> 0.740 ms on the INT8 prefill workload).  All waits are
// bounded as in the one-CTA kernel.
//
// Work unit = (group, 256-row super block, which halves may be stored).  Contiguous layout:
// a super block whose halves belong to two different groups (callers that pad groups to 128
// instead of 256 rows) becomes two units, each computing the super block with one group's
// weights and storing only that group's half.
#pragma once

#include "dg_grouped_gemm.cuh"

namespace dg {

constexpr int kPairBN = 256;
constexpr int kPairStages = 6;
constexpr int kPairTmemCols = 512;

struct PairSmem {
  static constexpr int kBHalfBytes = 128 * kRowBytes;
  static constexpr int off_a = 0;
  static constexpr int off_b = off_a + kPairStages * kATileBytes;
  static constexpr int off_bar = off_b + kPairStages * kBHalfBytes;
  // full[S], empty[S], acc_full[2], acc_empty[2], drain
  static constexpr int kNumBars = 2 * kPairStages + 5;
  static constexpr int off_misc = off_bar + kNumBars * 8;
  // misc: tmem slot, abort, n_items, stages ready, items ready
  static constexpr int off_bs = (off_misc + 32 + 15) & ~15;  // a tile's weight scales, one strip per epilogue warp; read as float4
  static constexpr int off_epi = off_bs + 4 * kPairBN * 4;  // store strips: 32 rows x 64 B per epilogue warp
  static constexpr int off_table = off_epi + 4 * 2048;
  static_assert(off_bs % 16 == 0 && off_epi % 16 == 0 && off_table % 4 == 0,
                "scale and store strips are accessed with 16-byte loads and stores");
  static constexpr int kThreads = 224;  // producer, UMMA issuer, four epilogue warps, barrier watcher
  __host__ __device__ static constexpr int total(int table_bytes) {
    return off_table + table_bytes + 1024;
  }
};

struct PairTile {
  int g;
  int row0;        // first row of the 256-row super block (within the group if masked)
  int n0;
  int rows_valid;  // rows of the super block that exist / are below masked_m
  int half_mask;   // bit r set: rows of half r may be stored
};

struct PairDecoder {
  const KernelParams& p;
  const int32_t* tbl;
  int cursor;
  __device__ PairDecoder(const KernelParams& p_, const int32_t* tbl_) : p(p_), tbl(tbl_), cursor(0) {}
  __device__ __forceinline__ PairTile get(int item) {
    PairTile t;
    if (p.mode == MODE_MASKED) {
      const int32_t* cnt = tbl;
      const int32_t* pref = tbl + p.G;
      while (item >= pref[cursor + 1]) ++cursor;
      const int local = item - pref[cursor];
      const int sb = local / p.n_tiles;
      t.g = cursor;
      t.row0 = sb * 256;
      t.n0 = (local - sb * p.n_tiles) * kPairBN;
      t.rows_valid = min(256, cnt[cursor] - t.row0);
      t.half_mask = 3;
    } else {
      const int ui = item / p.n_tiles;
      const int e = tbl[ui];
      t.g = e >> 16;
      t.half_mask = (e >> 12) & 3;
      t.row0 = (e & 0xFFF) * 256;
      t.n0 = (item - ui * p.n_tiles) * kPairBN;
      t.rows_valid = min(256, p.M - t.row0);
    }
    return t;
  }
};

template <int KIND>
__global__ void __launch_bounds__(PairSmem::kThreads, 1)
grouped_gemm_pair_kernel(const __grid_constant__ CUtensorMap tm_a,
                         const __grid_constant__ CUtensorMap tm_b, const KernelParams p) {
  using L = PairSmem;
  constexpr int STAGES = kPairStages;
  constexpr int kUmmaKind =
      (KIND == DG_KIND_E4M3) ? UMMA_F8F6F4 : (KIND == DG_KIND_BF16 ? UMMA_F16 : UMMA_I8);
  constexpr bool kIntAcc = (KIND == DG_KIND_I8);
  constexpr int kElemsPerRow = (KIND == DG_KIND_BF16) ? 64 : 128;
  constexpr uint32_t kIdesc =
      umma_idesc(kIntAcc ? 2u : 1u, (KIND == DG_KIND_E4M3) ? 0u : 1u, 256, kPairBN);
  constexpr uint32_t kStageBytes = kATileBytes + L::kBHalfBytes;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw_addr);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  auto bar_full = [&](int s) { return base + L::off_bar + 8u * s; };
  auto bar_empty = [&](int s) { return base + L::off_bar + 8u * (STAGES + s); };
  auto bar_acc_full = [&](int b) { return base + L::off_bar + 8u * (2 * STAGES + b); };
  auto bar_acc_empty = [&](int b) { return base + L::off_bar + 8u * (2 * STAGES + 2 + b); };
  const uint32_t bar_drain = base + L::off_bar + 8u * (2 * STAGES + 4);

  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::off_misc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::off_misc + 4);
  volatile int* n_items_s = reinterpret_cast<volatile int*>(smem + L::off_misc + 8);
  const uint32_t stages_addr = base + L::off_misc + 12;  // stages whose full barrier was seen complete (leader)
  const uint32_t items_addr = base + L::off_misc + 16;   // work items whose accumulator is free (leader)
  int32_t* tbl = reinterpret_cast<int32_t*>(smem + L::off_table);

  if (tid == 0) {
    *abort_flag = 0;
    *reinterpret_cast<volatile uint32_t*>(smem + L::off_misc + 12) = 0;
    *reinterpret_cast<volatile uint32_t*>(smem + L::off_misc + 16) = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full(s), 1);   // leader's producer (the peer's barrier stays unused)
      mbar_init(bar_empty(s), 1);  // one commit from the leader's UMMA thread
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_acc_full(b), 1);
      mbar_init(bar_acc_empty(b), 8);  // four epilogue warps of each block
    }
    mbar_init(bar_drain, 1);
    fence_mbar_init();
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_b);
  }

  // Schedule table (identical in both blocks of a pair).
  if (p.mode == MODE_MASKED) {
    int32_t* cnt = tbl;
    int32_t* pref = tbl + p.G;
    for (int g = tid; g < p.G; g += blockDim.x) cnt[g] = p.sched ? max(0, min(p.sched[g], p.M)) : p.M;
    __syncthreads();
    if (warp == 0) {
      int running = 0;
      for (int g0 = 0; g0 < p.G; g0 += 32) {
        const int g = g0 + lane;
        int x = (g < p.G) ? ((cnt[g] + 255) / 256) * p.n_tiles : 0;
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
        *n_items_s = running;
      }
    }
  } else {
    // two slots per super block: slot 0 = unit of the first half's group (covering both
    // halves when they agree), slot 1 = unit of the second half's group when it differs
    const int sbs = (p.M + 255) / 256;
    const int window0 = p.group_window ? p.group_window - 1 : 0;
    for (int sb = tid; sb < sbs; sb += blockDim.x) {
      int e0 = p.sched[(size_t)sb * 256];
      int e1 = ((size_t)sb * 256 + 128 < (size_t)p.M) ? p.sched[(size_t)sb * 256 + 128] : -1;
      e0 = e0 < 0 ? -1 : e0 - window0;
      e1 = e1 < 0 ? -1 : e1 - window0;
      if (p.group_window) {  // groups of other calls: not this call's business
        if (e0 >= p.G) e0 = -1;
        if (e1 >= p.G) e1 = -1;
      }
      const bool v0 = e0 >= 0 && e0 < p.G, v1 = e1 >= 0 && e1 < p.G;
      int u0 = -1, u1 = -1;
      if (v0) {
        u0 = (e0 << 16) | ((1 | ((v1 && e1 == e0) ? 2 : 0)) << 12) | sb;
        if (v1 && e1 != e0) u1 = (e1 << 16) | (2 << 12) | sb;
      } else if (v1) {
        u0 = (e1 << 16) | (2 << 12) | sb;
      }
      tbl[2 * sb] = u0;
      tbl[2 * sb + 1] = u1;
      if ((e0 >= p.G || e1 >= p.G) && blockIdx.x == 0 && p.status != nullptr)
        atomicCAS(p.status, DG_DEV_OK, DG_DEV_BAD_GROUP_INDEX);
    }
    __syncthreads();
    if (warp == 0) {
      int count = 0;
      for (int b0 = 0; b0 < 2 * sbs; b0 += 32) {
        const int b = b0 + lane;
        const int u = (b < 2 * sbs) ? tbl[b] : -1;
        const bool ok = u >= 0;
        const unsigned mask = __ballot_sync(0xffffffffu, ok);
        __syncwarp();
        if (ok) tbl[count + __popc(mask & ((1u << lane) - 1u))] = u;
        count += __popc(mask);
        __syncwarp();
      }
      if (lane == 0) *n_items_s = count * p.n_tiles;
    }
  }

  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_slot), kPairTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers are initialised before anything signals them
  tc_fence_after_sync();

  const uint32_t tmem_base = *tmem_slot;
  const int n_items = *n_items_s;

  if (warp == 0) {
    if (lane == 0) {
      // ---- TMA producer (both blocks)
      const uint64_t pol_a = l2_policy_evict_last();
      const uint64_t pol_b = l2_policy_evict_last();  // prefill re-reads weight panels from L2
      PairDecoder dec(p, tbl);
      uint32_t it = 0;
      bool ok = true;
      for (int item = pair; ok && item < n_items; item += num_pairs) {
        const PairTile t = dec.get(item);
        const int a_row = t.row0 + static_cast<int>(rank) * 128;
        const int b_n0 = t.n0 + static_cast<int>(rank) * 128;
        for (int kb = 0; kb < p.kblocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          if (!mbar_wait_bounded(bar_empty(s), ph ^ 1u, abort_flag, SITE_PRODUCER_EMPTY)) {
            ok = false;
            break;
          }
          if (rank == 0) mbar_arrive_expect_tx(bar_full(s), 2u * kStageBytes);
          const uint32_t full_leader = mapa_shared(bar_full(s), 0);
          const uint32_t a_dst = base + L::off_a + s * kATileBytes;
          const uint32_t b_dst = base + L::off_b + s * L::kBHalfBytes;
          if (p.mode == MODE_MASKED)
            tma_load_3d_pair(a_dst, &tm_a, full_leader, kb * kElemsPerRow, a_row, t.g, pol_a);
          else
            tma_load_2d_pair(a_dst, &tm_a, full_leader, kb * kElemsPerRow, a_row, pol_a);
          int bx, by;
          weight_coords(p, t.g, b_n0, kb, kElemsPerRow, bx, by);
          tma_load_2d_pair(b_dst, &tm_b, full_leader, bx, by, pol_b);
        }
      }
      if (rank == 0) {
        // The leader's stage-full barriers count the copies of both blocks.
        int local_abort = 0;
        for (int s = 0; s < STAGES; ++s) {
          const uint32_t fills = (it + STAGES - 1 - s) / STAGES;
          if (fills > 0 && !mbar_wait_bounded(bar_full(s), (fills - 1) & 1u, &local_abort,
                                              SITE_PRODUCER_DRAIN))
            *abort_flag = SITE_PRODUCER_DRAIN;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      // ---- UMMA issuer (leader only).  The first look at a barrier whose phase completed
      // long ago costs this thread about 200 cycles, comparable with the four UMMAs of a
      // stage: the watcher warp does the waits and posts "stages ready" / "items ready" in
      // plain shared-memory words, which this thread re-reads only when its copy is used up.
      // Ordering: the watcher observes the mbarrier (acquire), then publishes with st.release;
      // this thread's volatile loads of one shared-memory word after another are performed in
      // program order, and tcgen05.fence::after_thread_sync orders the UMMAs after the load
      // that saw the new count.  The operands themselves are read by the tensor core only.
      auto poll_above = [&](uint32_t addr, uint32_t have, int site) -> uint32_t {
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
      uint32_t it = 0, tile = 0, stages_known = 0, items_known = 0;
      bool ok = true;
      for (int item = pair; ok && item < n_items; item += num_pairs, ++tile) {
        const uint32_t buf = tile & 1u;
        if (items_known <= tile && (items_known = poll_above(items_addr, tile, SITE_MMA_ACC_EMPTY)) == 0) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * kPairBN;
        for (int kb = 0; kb < p.kblocks; ++kb, ++it) {
          const int s = it % STAGES;
          if (stages_known <= it) {
            if ((stages_known = poll_above(stages_addr, it, SITE_MMA_FULL)) == 0) {
              ok = false;
              break;
            }
            tc_fence_after_sync();
          }
          const uint64_t a_desc = umma_desc_sw128(base + L::off_a + s * kATileBytes);
          const uint64_t b_desc = umma_desc_sw128(base + L::off_b + s * L::kBHalfBytes);
#pragma unroll
          for (int k = 0; k < kRowBytes / 32; ++k)
            umma_ss_pair<kUmmaKind>(d_tmem, a_desc + 2u * k, b_desc + 2u * k, kIdesc,
                                    (kb | k) != 0 ? 1u : 0u);
          umma_commit_pair(bar_empty(s), 3);
        }
        if (ok) umma_commit_pair(bar_acc_full(buf), 3);
      }
      if (*abort_flag) {
        int local_abort = 0;
        umma_commit_pair(bar_drain, 1);
        mbar_wait_bounded(bar_drain, 0, &local_abort, 0);
      }
    }
  } else if (warp == 6) {
    if (lane == 0 && rank == 0) {
      // ---- barrier watcher (leader only): waits in the UMMA thread's place
      uint32_t it = 0, tile = 0;
      bool ok = true;
      for (int item = pair; ok && item < n_items; item += num_pairs, ++tile) {
        if (!mbar_wait_bounded(bar_acc_empty(tile & 1u), ((tile >> 1) & 1u) ^ 1u, abort_flag,
                               SITE_MMA_ACC_EMPTY))
          break;
        asm volatile("st.release.cta.shared::cta.u32 [%0], %1;" ::"r"(items_addr), "r"(tile + 1u) : "memory");
        for (int kb = 0; kb < p.kblocks; ++kb) {
          if (!mbar_wait_bounded(bar_full(it % STAGES), (it / STAGES) & 1u, abort_flag, SITE_MMA_FULL)) {
            ok = false;
            break;
          }
          ++it;
          asm volatile("st.release.cta.shared::cta.u32 [%0], %1;" ::"r"(stages_addr), "r"(it) : "memory");
        }
      }
    }
  } else {
    // ---- epilogue (both blocks): rows [128*rank, 128*rank+128) of the super block
    const int q = warp & 3;
    const int row_in_half = q * 32 + lane;
    const uint32_t acc_empty_leader[2] = {mapa_shared(bar_acc_empty(0), 0),
                                          mapa_shared(bar_acc_empty(1), 0)};
    PairDecoder dec(p, tbl);
    uint32_t tile = 0;
    for (int item = pair; item < n_items; item += num_pairs, ++tile) {
      const PairTile t = dec.get(item);
      const uint32_t buf = tile & 1u;
      const uint32_t aph = (tile >> 1) & 1u;
      // Everything that depends only on the tile's coordinates is fetched before the wait for
      // the accumulator, so that the global-load latency hides behind the main loop.
      float* bs_s = reinterpret_cast<float*>(smem + L::off_bs) + q * kPairBN;
      const int half_rows = t.rows_valid - static_cast<int>(rank) * 128;           // rows of my half
      const bool warp_has_rows = ((t.half_mask >> rank) & 1) && half_rows > q * 32;  // warp-uniform
      bool rv = false;
      size_t grow = 0;
      EpiRow row;
      row.as = 1.0f;
      row.bs_g = 1.0f;
      if (warp_has_rows) {
        stage_tile_scales(bs_s, p.b_scale + (size_t)t.g * p.N, t.n0, kPairBN, p.N, lane,
                          p.scale_mode == DG_SCALE_PER_CHANNEL);
        rv = row_in_half < half_rows;
        grow = (p.mode == MODE_MASKED ? (size_t)t.g * p.M : (size_t)0) + t.row0 + rank * 128 + row_in_half;
        if (p.mode == MODE_CONTIG && rv) rv = p.sched[grow] >= 0;
        if (rv && p.scale_mode != DG_SCALE_NONE) row.as = p.a_scale[grow];
        if (p.scale_mode == DG_SCALE_TENSOR_WISE) row.bs_g = p.b_scale[t.g];
      }
      if (!mbar_wait_warp(bar_acc_full(buf), aph, abort_flag, SITE_EPI_ACC_FULL)) break;
      tc_fence_after_sync();
      if (warp_has_rows) {
        row.bs_row = bs_s;
        row.f16 = p.out_kind == 1;
        row.d_row = p.d + grow * p.N + t.n0;
        const bool scatter = p.mode == MODE_CONTIG && p.scatter_tag != nullptr;
        if (scatter && rv) {
          const int tag = p.scatter_tag[grow];
          row.d_row = static_cast<__nv_bfloat16*>(p.scatter_base[(tag >> 24) & 15]) +
                      (size_t)(tag & 0xFFFFFF) * p.N + t.n0;
        }
        row.dbg_row = p.debug_acc ? p.debug_acc + grow * p.N + t.n0 : nullptr;
        const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * kPairBN;
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
        epilogue_drain<kIntAcc>(t_row, min(kPairBN / 32, (cols_left0 + 31) / 32), rv, row, ew, p.scale_mode,
                                cols_left0, false, 0);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(acc_empty_leader[buf]);
    }
  }

  // ---- tear-down: nobody leaves while the peer may still read this block's shared memory
  // or signal its barriers
  if (*abort_flag != 0 && tid == 0) {
    // abnormal exit: give copies still in flight into this block time to land
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) {
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, kPairTmemCols);
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
