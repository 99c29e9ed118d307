// Producer for the contiguous grouped GEMM: per-token quantisation fused with the
// group-by-expert / pad-to-alignment re-layout.
//
//   in : rows[R][H] bf16 (tokens as they arrive from dispatch), expert[R] int32 (< 0 = drop)
//   out: a[m_cap][H] e4m3 or int8 (rows of one expert contiguous, each expert's block starting
//        at a multiple of `align`), a_scale[m_cap], m_indices[m_cap] (-1 on every row that
//        holds no token, up to m_cap), dest[R] (where each input row went, -1 if dropped),
//        m_total (rows in use, a multiple of align)
//
// Nothing is read back by the host: the GEMM is launched on m_cap rows and skips the blocks
// whose first m_indices entry is -1.  The order of rows inside an expert is the input order
// (stable), so results do not depend on scheduling.
//
// Four launches on the caller's stream, using caller-provided scratch (dg_quant_group_scratch_bytes):
//   1. histogram   one warp per chunk of 32 input rows counts rows per expert into
//                  hist[expert][chunk] with __match_any_sync; the same grid fills m_indices with -1
//   2. scan        one block per expert: exclusive scan of its histogram row (rows of that expert
//                  in earlier chunks) and its total
//   3. starts      one block: scan of the totals padded to `align` -> first row of each expert, m_total
//   4. quantise    one block per input row: 16-byte loads of the row into registers, block-wide
//                  absmax, scale = absmax / 448 (or / 127), convert, 16- or 8-byte stores to the
//                  row's destination.  HBM-bound: 2 bytes read + 1 byte written per element.
//
// The reference has no kernel for this step; its tests build the layout with torch ops
// (op_test/contiguous_w8a8_int8_common.py:38-62) and quantise with op_test/quant_utils.py:4-19,
// whose arithmetic (fp32 absmax, x * (qmax / absmax), round to nearest even) is kept bit for bit.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "deepgemm_b200.h"

namespace dg {

constexpr int kQgChunk = 32;        // input rows per histogram chunk (one warp)
constexpr int kQgThreads = 256;     // quantise block
constexpr int kQgMaxVec = 8;        // 16-byte vectors per thread -> H <= 256 * 8 * 8 = 16384

struct QuantGroupParams {
  const __nv_bfloat16* rows;
  const int32_t* expert;
  const int32_t* src_index;  // nullable: input row r is rows[src_index[r]] instead of rows[r]
  // "sorted ids" input (all null / 0 otherwise): row r is entry r of a routing list in which
  // every entry packs (top-k slot << 24 | token), entries come in blocks of block_m that share
  // one expert (expert_ids[r / block_m], -1 = not on this rank), and entries at or beyond
  // *num_post_pad, with a slot >= real_topk or a row index >= size_m are padding.  The row
  // read is token * real_topk + slot; it is already quantised (1 byte per element, scale
  // row_scale[row], optionally times row_weight[row]) and is copied, not quantised.
  const int32_t* sorted_ids;
  const int32_t* expert_ids;
  const int32_t* num_post_pad;
  const float* row_scale;
  const float* row_weight;
  int block_m, real_topk, size_m;
  void* a_out;
  float* a_scale_out;
  int32_t* m_indices_out;
  int32_t* dest_out;     // nullable
  int32_t* src_out;      // nullable, sorted-ids input: src_out[dest] = row of `rows` stored at dest
  void* zero_rows;       // nullable, sorted-ids input: rows named by blocks whose expert is -1 are
  int zero_row_bytes;    //   zeroed in this [size_m][zero_row_bytes] buffer (multiple of 16 bytes)
  int32_t* m_total_out;  // nullable
  int32_t* hist;         // scratch: [G][chunks] rows per (expert, chunk); exclusive-scanned in place
  int32_t* starts;       // scratch: [G] totals, then first output row of each expert
  int R, H, G, align, m_cap, chunks, kind;
};

// Expert of input row r (-1 = drop) and the row of `rows` it reads.
__device__ __forceinline__ int qg_expert_of(const QuantGroupParams& p, int r, int* src) {
  if (p.sorted_ids == nullptr) {
    *src = p.src_index ? p.src_index[r] : r;
    return p.expert[r];
  }
  *src = 0;
  if (r >= *p.num_post_pad) return -1;
  const uint32_t id = static_cast<uint32_t>(p.sorted_ids[r]);
  const int slot = static_cast<int>(id >> 24);
  const long long row = static_cast<long long>(id & 0x00FFFFFFu) * p.real_topk + slot;
  if (slot >= p.real_topk || row >= p.size_m) return -1;
  *src = static_cast<int>(row);
  return p.expert_ids[r / p.block_m];
}

__global__ void qg_histogram_kernel(const QuantGroupParams p) {
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const int gwarp = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  const int nwarps = gridDim.x * warps_per_block;
  for (int c = gwarp; c < p.chunks; c += nwarps) {
    for (int e = lane; e < p.G; e += 32) p.hist[(size_t)e * p.chunks + c] = 0;
    __syncwarp();
    const int r = c * kQgChunk + lane;
    int src;
    int e = (r < p.R) ? qg_expert_of(p, r, &src) : -1;
    if (e >= p.G) e = -1;
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    if (e >= 0 && (peers & ((1u << lane) - 1u)) == 0)  // first lane of each distinct expert
      p.hist[(size_t)e * p.chunks + c] = __popc(peers);
  }
  const int tid = blockIdx.x * blockDim.x + threadIdx.x;
  for (int i = tid; i < p.m_cap; i += gridDim.x * blockDim.x) p.m_indices_out[i] = -1;
  if (p.sorted_ids != nullptr && p.dest_out != nullptr)  // dest is indexed by source row there
    for (int i = tid; i < p.size_m; i += gridDim.x * blockDim.x) p.dest_out[i] = -1;
}

// Block e: exclusive scan of hist[e][0..chunks) in place, total to starts[e].
__global__ void __launch_bounds__(256) qg_scan_kernel(const QuantGroupParams p) {
  __shared__ int warp_sums[8];
  __shared__ int carry_s;
  const int e = blockIdx.x;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  int32_t* h = p.hist + (size_t)e * p.chunks;
  if (threadIdx.x == 0) carry_s = 0;
  __syncthreads();
  for (int c0 = 0; c0 < p.chunks; c0 += 256) {
    const int c = c0 + threadIdx.x;
    const int v = (c < p.chunks) ? h[c] : 0;
    int x = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int y = __shfl_up_sync(0xffffffffu, x, o);
      if (lane >= o) x += y;
    }
    if (lane == 31) warp_sums[w] = x;
    __syncthreads();
    int before = carry_s;
    for (int i = 0; i < w; ++i) before += warp_sums[i];
    if (c < p.chunks) h[c] = before + x - v;
    __syncthreads();
    if (threadIdx.x == 255) carry_s = before + x;
    __syncthreads();
  }
  if (threadIdx.x == 0) p.starts[e] = carry_s;
}

// One block: totals padded to `align` -> exclusive scan -> first output row of each expert.
__global__ void qg_starts_kernel(const QuantGroupParams p) {
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < p.G; ++e) {
      const int padded = (p.starts[e] + p.align - 1) / p.align * p.align;
      p.starts[e] = run;
      run += padded;
    }
    if (p.m_total_out != nullptr) *p.m_total_out = run < p.m_cap ? run : p.m_cap / p.align * p.align;
  }
}

__device__ __forceinline__ float qg_block_max(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float m = red[0];
#pragma unroll
  for (int w = 1; w < kQgThreads / 32; ++w) m = fmaxf(m, red[w]);
  return m;
}

// Output row of input row r (-1 = dropped), its expert and the row it reads.  One thread.
__device__ __forceinline__ int qg_dest_of(const QuantGroupParams& p, int r, int* expert, int* src) {
  const int e = qg_expert_of(p, r, src);
  *expert = e;
  if (e < 0 || e >= p.G) return -1;
  // stable rank inside the chunk: earlier rows of the same chunk with the same expert
  const int c = r / kQgChunk;
  int rank = 0, other;
  for (int j = c * kQgChunk; j < r; ++j) rank += (qg_expert_of(p, j, &other) == e);
  const int dest = p.starts[e] + p.hist[(size_t)e * p.chunks + c] + rank;
  return dest < p.m_cap ? dest : -1;
}

// MAXVEC = 16-byte vectors of the row per thread (rows up to 256 * 8 * MAXVEC elements); the
// smaller instantiation needs fewer registers, so more rows are resident per SM.
template <int KIND, int MAXVEC>
__global__ void __launch_bounds__(kQgThreads) qg_quantise_kernel(const QuantGroupParams p) {
  __shared__ float red[kQgThreads / 32];
  __shared__ int s_dest, s_src, s_expert;
  const int r = blockIdx.x;
  // Every thread can tell a dropped row and find the source row by itself; the row's loads
  // are issued before thread 0 works out the destination (a chain of dependent global loads)
  // so that the two latencies overlap.
  int src_row;
  const int e_all = qg_expert_of(p, r, &src_row);
  if (e_all < 0 || e_all >= p.G) {
    if (threadIdx.x == 0 && p.dest_out != nullptr) p.dest_out[r] = -1;
    return;
  }
  const int nvec = p.H / 8;  // 16-byte vectors of 8 bf16
  const uint4* src = reinterpret_cast<const uint4*>(p.rows + static_cast<size_t>(src_row) * p.H);
  uint4 v[MAXVEC];
#pragma unroll
  for (int i = 0; i < MAXVEC; ++i) {
    const int idx = threadIdx.x + i * kQgThreads;
    if (idx < nvec) v[i] = __ldg(src + idx);
  }
  if (threadIdx.x == 0) {
    s_dest = qg_dest_of(p, r, &s_expert, &s_src);
    if (p.dest_out != nullptr) p.dest_out[r] = s_dest;
  }
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < MAXVEC; ++i) {
    const int idx = threadIdx.x + i * kQgThreads;
    if (idx < nvec) {
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[i]);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __bfloat1622float2(h[k]);
        amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
      }
    }
  }
  amax = fmaxf(qg_block_max(amax, red), 1e-10f);  // its barrier also publishes s_dest
  const int dest = s_dest;
  if (dest < 0) return;
  constexpr float kQmax = (KIND == DG_KIND_E4M3) ? 448.0f : 127.0f;
  // torch evaluates `qmax / absmax` (scalar / tensor) as reciprocal(absmax) * qmax: two
  // roundings, reproduced here so that ties fall the same way
  const float inv = __fmul_rn(__frcp_rn(amax), kQmax);
  if (threadIdx.x == 0) {
    p.a_scale_out[dest] = __fdiv_rn(amax, kQmax);
    p.m_indices_out[dest] = s_expert;
  }
  uint2* dst = reinterpret_cast<uint2*>(static_cast<uint8_t*>(p.a_out) + (size_t)dest * p.H);
#pragma unroll
  for (int i = 0; i < MAXVEC; ++i) {
    const int idx = threadIdx.x + i * kQgThreads;
    if (idx < nvec) {
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[i]);
      uint32_t out[2];
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const float2 f0 = __bfloat1622float2(h[2 * half]);
        const float2 f1 = __bfloat1622float2(h[2 * half + 1]);
        const float x0 = f0.x * inv, x1 = f0.y * inv, x2 = f1.x * inv, x3 = f1.y * inv;
        if constexpr (KIND == DG_KIND_E4M3) {
          const float lim = 448.0f;
          const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(
              make_float2(fminf(fmaxf(x0, -lim), lim), fminf(fmaxf(x1, -lim), lim)), __NV_SATFINITE,
              __NV_E4M3);
          const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(
              make_float2(fminf(fmaxf(x2, -lim), lim), fminf(fmaxf(x3, -lim), lim)), __NV_SATFINITE,
              __NV_E4M3);
          out[half] = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
        } else {
          const int q0 = max(-128, min(127, __float2int_rn(x0)));
          const int q1 = max(-128, min(127, __float2int_rn(x1)));
          const int q2 = max(-128, min(127, __float2int_rn(x2)));
          const int q3 = max(-128, min(127, __float2int_rn(x3)));
          out[half] = (q0 & 0xFF) | ((q1 & 0xFF) << 8) | ((q2 & 0xFF) << 16) |
                      (static_cast<uint32_t>(q3 & 0xFF) << 24);
        }
      }
      dst[idx] = make_uint2(out[0], out[1]);
    }
  }
}

// Rows that are quantised already (row_scale given; always so for sorted-ids input): copy H
// bytes and the (weighted) scale.
constexpr int kQgCopyThreads = 64;
__global__ void __launch_bounds__(kQgCopyThreads) qg_copy_kernel(const QuantGroupParams p) {
  __shared__ int s_dest, s_src, s_expert, s_zero;
  const int r = blockIdx.x;
  if (threadIdx.x == 0) {
    s_dest = qg_dest_of(p, r, &s_expert, &s_src);
    s_zero = -1;
    if (p.dest_out != nullptr && p.sorted_ids == nullptr) p.dest_out[r] = s_dest;
    if (p.sorted_ids != nullptr && p.zero_rows != nullptr && r < *p.num_post_pad &&
        p.expert_ids[r / p.block_m] < 0) {
      // a row of an expert that does not live here: the reference's kernel stores zeros for it
      const uint32_t id = static_cast<uint32_t>(p.sorted_ids[r]);
      const int slot = static_cast<int>(id >> 24);
      const long long row = static_cast<long long>(id & 0x00FFFFFFu) * p.real_topk + slot;
      if (slot < p.real_topk && row < p.size_m) s_zero = static_cast<int>(row);
    }
    if (s_dest >= 0) {
      // sorted-ids input: dest is indexed by the source row (one entry per row of `rows`)
      if (p.dest_out != nullptr && p.sorted_ids != nullptr) p.dest_out[s_src] = s_dest;
      if (p.src_out != nullptr) p.src_out[s_dest] = s_src;
      const float w = p.row_weight ? p.row_weight[s_src] : 1.0f;
      p.a_scale_out[s_dest] = p.row_weight ? __fmul_rn(w, p.row_scale[s_src]) : p.row_scale[s_src];
      p.m_indices_out[s_dest] = s_expert;
    }
  }
  __syncthreads();
  if (s_zero >= 0) {
    uint4* z = reinterpret_cast<uint4*>(static_cast<uint8_t*>(p.zero_rows) +
                                        static_cast<size_t>(s_zero) * p.zero_row_bytes);
    for (int i = threadIdx.x; i < p.zero_row_bytes / 16; i += kQgCopyThreads) z[i] = make_uint4(0, 0, 0, 0);
  }
  if (s_dest < 0) return;
  const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(p.rows) +
                                                    static_cast<size_t>(s_src) * p.H);
  uint4* dst = reinterpret_cast<uint4*>(static_cast<uint8_t*>(p.a_out) + static_cast<size_t>(s_dest) * p.H);
  for (int i = threadIdx.x; i < p.H / 16; i += kQgCopyThreads) dst[i] = __ldg(src + i);
}

// `sms`: multiprocessors of the current device (sizes the histogram grid).
inline cudaError_t launch_quant_group(const QuantGroupParams& p, int sms, cudaStream_t stream) {
  if (p.R == 0) {
    // still mark every row unused
    QuantGroupParams q = p;
    q.chunks = 0;
    qg_histogram_kernel<<<sms, 256, 0, stream>>>(q);
    if (p.m_total_out != nullptr) cudaMemsetAsync(p.m_total_out, 0, sizeof(int32_t), stream);
    return cudaGetLastError();
  }
  int hblocks = (p.chunks + 7) / 8;
  if (hblocks < sms) hblocks = sms;
  if (hblocks > sms * 8) hblocks = sms * 8;
  qg_histogram_kernel<<<hblocks, 256, 0, stream>>>(p);
  qg_scan_kernel<<<p.G, 256, 0, stream>>>(p);
  qg_starts_kernel<<<1, 32, 0, stream>>>(p);
  if (p.row_scale != nullptr)  // rows are quantised already
    qg_copy_kernel<<<p.R, kQgCopyThreads, 0, stream>>>(p);
  else if (p.H <= kQgThreads * 8 * 4) {
    if (p.kind == DG_KIND_E4M3)
      qg_quantise_kernel<DG_KIND_E4M3, 4><<<p.R, kQgThreads, 0, stream>>>(p);
    else
      qg_quantise_kernel<DG_KIND_I8, 4><<<p.R, kQgThreads, 0, stream>>>(p);
  } else {
    if (p.kind == DG_KIND_E4M3)
      qg_quantise_kernel<DG_KIND_E4M3, kQgMaxVec><<<p.R, kQgThreads, 0, stream>>>(p);
    else
      qg_quantise_kernel<DG_KIND_I8, kQgMaxVec><<<p.R, kQgThreads, 0, stream>>>(p);
  }
  return cudaGetLastError();
}

}  // namespace dg
