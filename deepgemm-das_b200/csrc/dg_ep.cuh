// Expert-parallel token exchange over peer memory (NVLink / NVSwitch), without host round trips.
//
// The reference library is single-GPU; serving frameworks shard its experts over GPUs and move
// the routed rows themselves.  These kernels are that exchange for one box, built on plain
// peer-to-peer loads and stores into buffers every rank has mapped (no TMA on peer memory, no
// multicast): a rank writes each routed row straight into the owning rank's grouped, padded
// activation buffer -- the A operand of that rank's contiguous grouped GEMM -- so nothing has to
// be regrouped after the transfer.
//
//   ep_plan_kernel     one block per rank: histogram of this rank's routed pairs per expert ->
//                      written into every rank's counts table -> signal -> wait for every rank's
//                      signal -> from the full table, the layout of every destination buffer:
//                      where this rank's rows of each expert start (`my_base`), and for this
//                      rank's own experts the m_indices array of the buffer it receives into.
//   ep_push_kernel     a block per token: the token's quantised row is read once and stored to
//                      the destination row of each of its top-k experts (16-byte stores to peer
//                      memory), with its scale and a tag (source rank << 24 | pair index) that
//                      the second GEMM's epilogue uses to send the result row home.
//   ep_push_quant_kernel  the same with the per-token quantisation fused in: the token's bf16 row
//                      is read once, quantised in registers (the arithmetic of qg_quantise_kernel)
//                      and its e4m3 / int8 bytes go to the top-k destinations.
//   ep_barrier_kernel  fence + signal + wait: every rank's earlier stores have landed.
//
// Signals are monotonically increasing epoch numbers in one int per (rank, peer), so a signal
// that arrives early is not lost and nothing needs resetting.  Every wait is bounded
// (kEpWaitLimitNs); on expiry the kernel records DG_DEV_WAIT_EXPIRED in the status words and
// carries on, so a missing peer cannot hang the device.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "deepgemm_b200.h"
#include "dg_moe_chain.cuh"
#include "dg_ptx.cuh"

namespace dg {

constexpr int kEpMaxWorld = 16;
constexpr int kEpPlanThreads = 1024;
constexpr int kEpPushThreads = 256;
constexpr uint64_t kEpWaitLimitNs = 2000000000ull;

struct EpPeers {
  void* ptr[kEpMaxWorld];
};

__device__ __forceinline__ void ep_signal(int32_t* flag, int32_t value) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(flag), "r"(value) : "memory");
}
__device__ __forceinline__ int32_t ep_peek(const int32_t* flag) {
  int32_t v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
  return v;
}
// Waits until *flag >= value; false after kEpWaitLimitNs.
__device__ __forceinline__ bool ep_wait(const int32_t* flag, int32_t value) {
  if (ep_peek(flag) - value >= 0) return true;
  const uint64_t t0 = global_timer_ns();
  while (true) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i)
      if (ep_peek(flag) - value >= 0) return true;
    if (global_timer_ns() - t0 > kEpWaitLimitNs) return false;
  }
}

// Threads 0..world-1 of a block: make the block's earlier stores visible system-wide, tell every
// rank that this rank has reached `epoch`, and wait until every rank has.  Call with all threads
// of the block (it synchronises them before and after).
// `phases`: bit 0 = signal, bit 1 = wait.
__device__ __forceinline__ void ep_block_barrier(const EpPeers& peer_flags, int32_t* flags, int world,
                                                 int me, int32_t epoch, int32_t* status, int phases) {
  __syncthreads();
  if (threadIdx.x < world) {
    if (phases & 1) {
      __threadfence_system();
      ep_signal(static_cast<int32_t*>(peer_flags.ptr[threadIdx.x]) + me, epoch);
    }
    if ((phases & 2) && !ep_wait(flags + threadIdx.x, epoch) && status != nullptr) {
      if (atomicCAS(status, DG_DEV_OK, DG_DEV_WAIT_EXPIRED) == DG_DEV_OK) {
        status[1] = me;
        status[2] = 100 + static_cast<int>(threadIdx.x);  // which peer never signalled
        status[3] = epoch;
      }
    }
  }
  __syncthreads();
}

struct EpPlanParams {
  const int32_t* topk_ids;  // [pairs] expert of each (token, slot) pair of this rank
  int pairs;
  int E, world, me, e_local, align, m_cap;
  EpPeers peer_counts;  // every rank's counts table [world][E]
  EpPeers peer_flags;   // every rank's flags [world]
  int32_t* counts;      // this rank's counts table
  int32_t* flags;       // this rank's flags
  int32_t epoch;
  int phases;           // bit 0: count, publish, signal; bit 1: wait, lay out
  int32_t* my_base;     // [E] out: row, in the owning rank's buffer, of this rank's first row of expert e
  int32_t* cursor;      // [E] out: zeroed (ep_push_kernel hands out rows with it)
  int32_t* m_indices;   // [m_cap] out: layout of the buffer this rank receives into
  int32_t* m_total;     // [1] out: rows in use in that buffer (multiple of align)
  int32_t* status;
};

__global__ void __launch_bounds__(kEpPlanThreads, 1) ep_plan_kernel(const EpPlanParams p) {
  extern __shared__ int32_t ep_sm[];  // hist[E], padded[E], start[E]
  int32_t* hist = ep_sm;
  int32_t* padded = ep_sm + p.E;
  int32_t* start = ep_sm + 2 * p.E;
  const int tid = threadIdx.x;
  if (p.phases & 1) {
    for (int e = tid; e < p.E; e += blockDim.x) hist[e] = 0;
    __syncthreads();
    for (int i = tid; i < p.pairs; i += blockDim.x) {
      const int e = p.topk_ids[i];
      if (e >= 0 && e < p.E) atomicAdd(&hist[e], 1);
    }
    __syncthreads();
    // this rank's row of every rank's counts table
    for (int r = 0; r < p.world; ++r) {
      int32_t* dst = static_cast<int32_t*>(p.peer_counts.ptr[r]) + (size_t)p.me * p.E;
      for (int e = tid; e < p.E; e += blockDim.x) dst[e] = hist[e];
    }
  }
  ep_block_barrier(p.peer_flags, p.flags, p.world, p.me, p.epoch, p.status, p.phases);
  if (!(p.phases & 2)) return;

  // layout of every destination buffer: expert e holds the rows of rank 0, then rank 1, ...;
  // each expert's block is padded to `align` rows; experts of a rank follow one another
  for (int e = tid; e < p.E; e += blockDim.x) {
    int tot = 0, before = 0;
    for (int s = 0; s < p.world; ++s) {
      const int c = __ldcg(p.counts + (size_t)s * p.E + e);  // written by rank s
      tot += c;
      if (s < p.me) before += c;
    }
    padded[e] = (tot + p.align - 1) / p.align * p.align;
    hist[e] = tot;      // re-used: total rows of expert e
    start[e] = before;  // re-used below
  }
  __syncthreads();
  for (int e = tid; e < p.E; e += blockDim.x) {
    const int first = e / p.e_local * p.e_local;
    int s0 = 0;
    for (int x = first; x < e; ++x) s0 += padded[x];
    p.my_base[e] = s0 + start[e];
    p.cursor[e] = 0;
  }
  __syncthreads();
  // m_indices of this rank's receive buffer
  int row0 = 0;
  for (int el = 0; el < p.e_local; ++el) {
    const int e = p.me * p.e_local + el;
    const int tot = hist[e], pad = padded[e];
    for (int i = tid; i < pad; i += blockDim.x)
      if (row0 + i < p.m_cap) p.m_indices[row0 + i] = i < tot ? el : -1;
    row0 += pad;
  }
  for (int i = row0 + tid; i < p.m_cap; i += blockDim.x) p.m_indices[i] = -1;
  if (tid == 0) {
    *p.m_total = row0 < p.m_cap ? row0 : p.m_cap / p.align * p.align;
    if (row0 > p.m_cap && p.status != nullptr) atomicCAS(p.status, DG_DEV_OK, DG_DEV_BAD_GROUP_INDEX);
  }
}

struct EpPushParams {
  const uint8_t* rows;       // [T][row_bytes] quantised rows of this rank's tokens
  const float* row_scale;    // [T]
  const int32_t* topk_ids;   // [T][top_k]
  int T, top_k, row_bytes;   // row_bytes a multiple of 16
  int E, e_local, me, m_cap;
  const int32_t* my_base;    // [E] from ep_plan_kernel
  int32_t* cursor;           // [E]
  EpPeers peer_a;            // every rank's receive buffer [m_cap][row_bytes]
  EpPeers peer_scale;        // every rank's [m_cap] scales
  EpPeers peer_tag;          // every rank's [m_cap] tags: source rank << 24 | pair index
  int32_t* pair_dest;        // NULL, or [T][top_k] out: destination row of each pair (-1 = dropped)
  int32_t* status;
  int local_lo, local_hi;    // only pairs whose expert is number [local_lo, local_hi) of its owner's are sent
};

constexpr int kEpMaxChunksPerThread = 4;  // row_bytes <= 16 * 256 * 4 = 16384
constexpr int kEpMaxTopK = 32;

__global__ void __launch_bounds__(kEpPushThreads) ep_push_kernel(const EpPushParams p) {
  __shared__ int32_t dest_s[kEpMaxTopK];
  const int tid = threadIdx.x;
  const int chunks = p.row_bytes >> 4;
  for (int t = blockIdx.x; t < p.T; t += gridDim.x) {
    uint4 v[kEpMaxChunksPerThread];
    const uint4* src = reinterpret_cast<const uint4*>(p.rows + (size_t)t * p.row_bytes);
#pragma unroll
    for (int c = 0; c < kEpMaxChunksPerThread; ++c)
      if (tid + c * kEpPushThreads < chunks) v[c] = __ldg(src + tid + c * kEpPushThreads);
    if (tid < p.top_k) {
      const int e = p.topk_ids[(size_t)t * p.top_k + tid];
      int dest = -1;
      const int el = e % p.e_local;
      const bool mine = e >= 0 && e < p.E && el >= p.local_lo && el < p.local_hi;  // this slice's pair
      if (mine) {
        dest = p.my_base[e] + atomicAdd(&p.cursor[e], 1);
        if (dest >= p.m_cap) {  // the owning rank's buffer is full: the pair is dropped and reported
          dest = -1;
          if (p.status != nullptr) atomicCAS(p.status, DG_DEV_OK, DG_DEV_BAD_GROUP_INDEX);
        }
      }
      dest_s[tid] = dest;
      if (p.pair_dest != nullptr && (mine || e < 0 || e >= p.E)) p.pair_dest[(size_t)t * p.top_k + tid] = dest;
      if (dest >= 0) {
        const int r = e / p.e_local;
        static_cast<float*>(p.peer_scale.ptr[r])[dest] = p.row_scale[t];
        static_cast<int32_t*>(p.peer_tag.ptr[r])[dest] = (p.me << 24) | (t * p.top_k + tid);
      }
    }
    __syncthreads();
    for (int j = 0; j < p.top_k; ++j) {
      const int dest = dest_s[j];
      if (dest < 0) continue;
      const int r = p.topk_ids[(size_t)t * p.top_k + j] / p.e_local;
      uint4* dst = reinterpret_cast<uint4*>(static_cast<uint8_t*>(p.peer_a.ptr[r]) + (size_t)dest * p.row_bytes);
#pragma unroll
      for (int c = 0; c < kEpMaxChunksPerThread; ++c)
        if (tid + c * kEpPushThreads < chunks) dst[tid + c * kEpPushThreads] = v[c];
    }
    __syncthreads();  // dest_s is rewritten for the next token
  }
}

// bf16 rows in, quantised rows out.  p.rows holds bf16 [T][row_bytes] (row_bytes = elements per
// row = bytes per quantised row, a multiple of 8, at most 8 * 256 * kEpMaxVec); p.row_scale is
// not read.
constexpr int kEpMaxVec = 4;
template <int KIND>
__global__ void __launch_bounds__(kEpPushThreads) ep_push_quant_kernel(const EpPushParams p) {
  static_assert(kEpPushThreads == kQgThreads, "qg_block_max reduces over kQgThreads threads");
  __shared__ float red[kEpPushThreads / 32];
  __shared__ int32_t dest_s[kEpMaxTopK];
  const int tid = threadIdx.x;
  const int nvec = p.row_bytes >> 3;  // 16-byte vectors of 8 bf16
  constexpr float kQmax = (KIND == DG_KIND_E4M3) ? 448.0f : 127.0f;
  for (int t = blockIdx.x; t < p.T; t += gridDim.x) {
    const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.rows) +
                                                      (size_t)t * p.row_bytes);
    uint4 v[kEpMaxVec];
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < kEpMaxVec; ++i) {
      const int idx = tid + i * kEpPushThreads;
      if (idx < nvec) {
        v[i] = __ldg(src + idx);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[i]);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 f = __bfloat1622float2(h[k]);
          amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
        }
      }
    }
    amax = fmaxf(qg_block_max(amax, red), 1e-10f);
    const float inv = __fmul_rn(__frcp_rn(amax), kQmax);  // as torch evaluates qmax / absmax
    if (tid < p.top_k) {
      const int e = p.topk_ids[(size_t)t * p.top_k + tid];
      int dest = -1;
      const int el = e % p.e_local;
      const bool mine = e >= 0 && e < p.E && el >= p.local_lo && el < p.local_hi;  // this slice's pair
      if (mine) {
        dest = p.my_base[e] + atomicAdd(&p.cursor[e], 1);
        if (dest >= p.m_cap) {
          dest = -1;
          if (p.status != nullptr) atomicCAS(p.status, DG_DEV_OK, DG_DEV_BAD_GROUP_INDEX);
        }
      }
      dest_s[tid] = dest;
      if (p.pair_dest != nullptr && (mine || e < 0 || e >= p.E)) p.pair_dest[(size_t)t * p.top_k + tid] = dest;
      if (dest >= 0) {
        const int r = e / p.e_local;
        static_cast<float*>(p.peer_scale.ptr[r])[dest] = __fdiv_rn(amax, kQmax);
        static_cast<int32_t*>(p.peer_tag.ptr[r])[dest] = (p.me << 24) | (t * p.top_k + tid);
      }
    }
    uint2 q[kEpMaxVec];
#pragma unroll
    for (int i = 0; i < kEpMaxVec; ++i) {
      if (tid + i * kEpPushThreads < nvec) {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[i]);
        float x[8];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 f = __bfloat1622float2(h[k]);
          x[2 * k] = f.x * inv;
          x[2 * k + 1] = f.y * inv;
        }
        q[i] = quantise8<KIND>(x);
      }
    }
    __syncthreads();
    for (int j = 0; j < p.top_k; ++j) {
      const int dest = dest_s[j];
      if (dest < 0) continue;
      const int r = p.topk_ids[(size_t)t * p.top_k + j] / p.e_local;
      uint2* dst = reinterpret_cast<uint2*>(static_cast<uint8_t*>(p.peer_a.ptr[r]) + (size_t)dest * p.row_bytes);
#pragma unroll
      for (int i = 0; i < kEpMaxVec; ++i)
        if (tid + i * kEpPushThreads < nvec) dst[tid + i * kEpPushThreads] = q[i];
    }
    __syncthreads();  // dest_s and red are rewritten for the next token
  }
}

struct EpBarrierParams {
  EpPeers peer_flags;
  int32_t* flags;
  int world, me;
  int32_t epoch;
  int phases;
  int32_t* status;
};

__global__ void ep_barrier_kernel(const EpBarrierParams p) {
  ep_block_barrier(p.peer_flags, p.flags, p.world, p.me, p.epoch, p.status, p.phases);
}

}  // namespace dg
