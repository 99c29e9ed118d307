// Weight re-layout kernels: row-major [G][N][K] <-> packed [G][K/BK][N][128 bytes]
// (plus a nibble re-pairing inside every 16-byte chunk for int4).  One thread moves one 16-byte
// chunk; the work is a pure byte permutation bound by HBM bandwidth and runs once at
// model-load time, like the torch re-layout code it replaces
// (deepgemm/m_group_gemm.py:826-863, deepgemm/group_gemm_weight_pack.py:594-714).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "deepgemm_b200.h"

namespace dg {

// 16 source bytes holding 32 consecutive int4 values w[0..31] of one row (two per byte, in
// `nibble_order`) -> 16 packed bytes with w[i] in the high and w[16+i] in the low nibble.
__device__ __forceinline__ uint4 w4_pair_for_kernel(uint4 s, int nibble_order) {
  uint8_t in[16], w[32], out[16];
  *reinterpret_cast<uint4*>(in) = s;
#pragma unroll
  for (int t = 0; t < 16; ++t) {
    const uint8_t hi = in[t] >> 4, lo = in[t] & 0xF;
    w[2 * t] = (nibble_order == DG_NIBBLE_HIGH_FIRST) ? hi : lo;
    w[2 * t + 1] = (nibble_order == DG_NIBBLE_HIGH_FIRST) ? lo : hi;
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) out[i] = static_cast<uint8_t>((w[i] << 4) | w[16 + i]);
  return *reinterpret_cast<uint4*>(out);
}

__device__ __forceinline__ uint4 w4_pair_for_framework(uint4 s, int nibble_order) {
  uint8_t in[16], w[32], out[16];
  *reinterpret_cast<uint4*>(in) = s;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    w[i] = in[i] >> 4;
    w[16 + i] = in[i] & 0xF;
  }
#pragma unroll
  for (int t = 0; t < 16; ++t) {
    const uint8_t first = w[2 * t], second = w[2 * t + 1];
    out[t] = (nibble_order == DG_NIBBLE_HIGH_FIRST) ? static_cast<uint8_t>((first << 4) | second)
                                                    : static_cast<uint8_t>((second << 4) | first);
  }
  return *reinterpret_cast<uint4*>(out);
}

// row_bytes: bytes per row-major source row; every packed row is 128 bytes = 8 chunks.
template <bool UNPACK, bool W4>
__global__ void relayout_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst,
                                long long total_chunks, int n, int kblocks, int row_bytes,
                                int nibble_order) {
  constexpr int CPR = 8;
  for (long long c = blockIdx.x * (long long)blockDim.x + threadIdx.x; c < total_chunks;
       c += (long long)gridDim.x * blockDim.x) {
    const int j = static_cast<int>(c % CPR);
    long long r = c / CPR;
    const int row = static_cast<int>(r % n);
    r /= n;
    const int kb = static_cast<int>(r % kblocks);
    const long long g = r / kblocks;
    const long long rm = ((g * n + row) * (long long)row_bytes + (long long)kb * (CPR * 16) +
                          j * 16) >> 4;  // chunk index in the row-major tensor
    if (!UNPACK) {
      uint4 v = src[rm];
      if (W4) v = w4_pair_for_kernel(v, nibble_order);
      dst[c] = v;
    } else {
      uint4 v = src[c];
      if (W4) v = w4_pair_for_framework(v, nibble_order);
      dst[rm] = v;
    }
  }
}

inline cudaError_t launch_pack(bool unpack, int kind, const void* src, void* dst, int G, int n,
                               int k, int nibble_order, cudaStream_t stream) {
  const bool w4 = (kind == DG_KIND_W4A8);
  const int row_bytes = (kind == DG_KIND_BF16) ? k * 2 : (w4 ? k / 2 : k);
  const int kblocks = row_bytes / 128;
  const long long total = (long long)G * n * row_bytes / 16;
  const int threads = 256;
  long long blocks = (total + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (blocks < 1) blocks = 1;
  const uint4* s = static_cast<const uint4*>(src);
  uint4* d = static_cast<uint4*>(dst);
  if (w4) {
    if (unpack)
      relayout_kernel<true, true><<<(int)blocks, threads, 0, stream>>>(s, d, total, n, kblocks,
                                                                      row_bytes, nibble_order);
    else
      relayout_kernel<false, true><<<(int)blocks, threads, 0, stream>>>(s, d, total, n, kblocks,
                                                                       row_bytes, nibble_order);
  } else {
    if (unpack)
      relayout_kernel<true, false><<<(int)blocks, threads, 0, stream>>>(s, d, total, n, kblocks,
                                                                       row_bytes, nibble_order);
    else
      relayout_kernel<false, false><<<(int)blocks, threads, 0, stream>>>(s, d, total, n, kblocks,
                                                                        row_bytes, nibble_order);
  }
  return cudaGetLastError();
}

}  // namespace dg
