// Memory-bound steps between the two grouped GEMMs of an MoE layer and after the second one.
//
//   act_quant_kernel   x bf16 [rows][2H] (gate | up)  ->  q [rows][H] int8 / e4m3, scale [rows]
//                      act = bf16(bf16(silu(gate)) * up), quantised per row like
//                      qg_quantise_kernel; rows named unused by m_indices / masked_m are skipped.
//   combine_kernel     out[t][:] = bf16( sum_j weights[t][j] * y[src_row[t][j]][:] )
//
// The reference has no kernels for these steps; its second-GEMM op multiplies the routing
// weight into the activation scale (csrc/include/moe_marlin/
// moe_marlin_prefill_down_fp8_device.inc.h:114-119) and leaves the reduction over the top-k
// rows to the caller.  One thread block per row (token), 16-byte accesses, a row is read from
// HBM once and kept in registers between the absmax pass and the store.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "deepgemm_b200.h"
#include "dg_quant_group.cuh"

namespace dg {

struct ActQuantParams {
  int kind, rows, H, max_m;
  const __nv_bfloat16* x;
  const int32_t* m_indices;
  const int32_t* masked_m;
  void* q_out;
  float* scale_out;
};

// 8 floats, already multiplied by qmax / absmax, to 8 bytes of int8 (round to nearest even,
// clamped to [-128, 127]) or e4m3 (saturating).
template <int KIND>
__device__ __forceinline__ uint2 quantise8(const float (&x)[8]) {
  uint32_t out[2];
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const float x0 = x[4 * half], x1 = x[4 * half + 1], x2 = x[4 * half + 2], x3 = x[4 * half + 3];
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
  return make_uint2(out[0], out[1]);
}

// silu(g) * u with the roundings of the unfused bf16 computation: silu is rounded to bf16,
// then the product is.  exp and the division use the fast hardware approximations (relative
// error about 2^-21): the result is rounded to bf16 (2^-9) right after, so this moves an
// output only when the exact value lies within that error of a rounding boundary.
__device__ __forceinline__ float silu_mul_bf16(float g, float u) {
  const float s = __bfloat162float(__float2bfloat16_rn(__fdividef(g, 1.0f + __expf(-g))));
  return __bfloat162float(__float2bfloat16_rn(s * u));
}

template <int THREADS>
__device__ __forceinline__ float block_max(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  if (THREADS == 32) return v;
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float m = red[0];
#pragma unroll
  for (int w = 1; w < THREADS / 32; ++w) m = fmaxf(m, red[w]);
  return m;
}

// One block of THREADS threads per row, at most MAXVEC 16-byte vectors of the output row per
// thread.  Short rows use small blocks so that each thread keeps several loads in flight and
// many rows are resident per SM.
template <int KIND, int THREADS, int MAXVEC>
__global__ void __launch_bounds__(THREADS) act_quant_kernel(const ActQuantParams p) {
  __shared__ float red[THREADS / 32];
  const int r = blockIdx.x;
  if (p.m_indices != nullptr && p.m_indices[r] < 0) return;
  if (p.masked_m != nullptr && (r % p.max_m) >= p.masked_m[r / p.max_m]) return;

  const int nvec = p.H / 8;
  const uint4* gate = reinterpret_cast<const uint4*>(p.x + (size_t)r * 2 * p.H);
  const uint4* up = gate + nvec;
  uint4 gv[MAXVEC], uv[MAXVEC];
#pragma unroll
  for (int i = 0; i < MAXVEC; ++i) {
    const int idx = threadIdx.x + i * THREADS;
    if (idx < nvec) {
      gv[i] = __ldg(gate + idx);
      uv[i] = __ldg(up + idx);
    }
  }
  float act[MAXVEC][8];
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < MAXVEC; ++i) {
    const int idx = threadIdx.x + i * THREADS;
    if (idx < nvec) {
      const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&gv[i]);
      const __nv_bfloat162* uh = reinterpret_cast<const __nv_bfloat162*>(&uv[i]);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 g = __bfloat1622float2(gh[k]);
        const float2 u = __bfloat1622float2(uh[k]);
        act[i][2 * k] = silu_mul_bf16(g.x, u.x);
        act[i][2 * k + 1] = silu_mul_bf16(g.y, u.y);
        amax = fmaxf(amax, fmaxf(fabsf(act[i][2 * k]), fabsf(act[i][2 * k + 1])));
      }
    }
  }
  amax = fmaxf(block_max<THREADS>(amax, red), 1e-10f);
  constexpr float kQmax = (KIND == DG_KIND_E4M3) ? 448.0f : 127.0f;
  const float inv = __fmul_rn(__frcp_rn(amax), kQmax);  // as in qg_quantise_kernel
  if (threadIdx.x == 0) p.scale_out[r] = __fdiv_rn(amax, kQmax);
  uint2* dst = reinterpret_cast<uint2*>(static_cast<uint8_t*>(p.q_out) + (size_t)r * p.H);
#pragma unroll
  for (int i = 0; i < MAXVEC; ++i) {
    const int idx = threadIdx.x + i * THREADS;
    if (idx < nvec) {
      float x[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) x[k] = act[i][k] * inv;
      dst[idx] = quantise8<KIND>(x);
    }
  }
}

template <int KIND>
inline void launch_act_quant_kind(const ActQuantParams& p, cudaStream_t stream) {
  if (p.H <= 1024)
    act_quant_kernel<KIND, 32, 4><<<p.rows, 32, 0, stream>>>(p);
  else if (p.H <= 2048)
    act_quant_kernel<KIND, 64, 4><<<p.rows, 64, 0, stream>>>(p);
  else if (p.H <= 4096)
    act_quant_kernel<KIND, 128, 4><<<p.rows, 128, 0, stream>>>(p);
  else
    act_quant_kernel<KIND, 256, DG_MAX_QUANT_HIDDEN / 8 / 256><<<p.rows, 256, 0, stream>>>(p);
}

inline cudaError_t launch_act_quant(const ActQuantParams& p, cudaStream_t stream) {
  if (p.rows == 0) return cudaSuccess;
  if (p.kind == DG_KIND_E4M3)
    launch_act_quant_kind<DG_KIND_E4M3>(p, stream);
  else
    launch_act_quant_kind<DG_KIND_I8>(p, stream);
  return cudaGetLastError();
}

struct CombineParams {
  int tokens, top_k, n, rows;
  const __nv_bfloat16* y;
  const int32_t* src_row;
  const float* weights;
  __nv_bfloat16* out;
};

constexpr int kCombineThreads = 128;

// One block per token; each thread owns 8 columns at a time and adds the top-k rows in order
// j = 0, 1, ... in fp32, so the result does not depend on the launch shape.
__global__ void __launch_bounds__(kCombineThreads) combine_kernel(const CombineParams p) {
  const int t = blockIdx.x;
  const int32_t* src = p.src_row + (size_t)t * p.top_k;
  const float* w = p.weights ? p.weights + (size_t)t * p.top_k : nullptr;
  const int nvec = p.n / 8;
  for (int v = threadIdx.x; v < nvec; v += kCombineThreads) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < p.top_k; ++j) {
      const int row = src[j];
      if (row < 0 || row >= p.rows) continue;
      const float wj = w ? w[j] : 1.0f;
      const uint4 yv = __ldg(reinterpret_cast<const uint4*>(p.y + (size_t)row * p.n) + v);
      const __nv_bfloat162* yh = reinterpret_cast<const __nv_bfloat162*>(&yv);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __bfloat1622float2(yh[k]);
        acc[2 * k] = fmaf(wj, f.x, acc[2 * k]);
        acc[2 * k + 1] = fmaf(wj, f.y, acc[2 * k + 1]);
      }
    }
    uint4 o;
    __nv_bfloat162 h;
    h = __floats2bfloat162_rn(acc[0], acc[1]);
    o.x = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2bfloat162_rn(acc[2], acc[3]);
    o.y = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2bfloat162_rn(acc[4], acc[5]);
    o.z = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2bfloat162_rn(acc[6], acc[7]);
    o.w = *reinterpret_cast<uint32_t*>(&h);
    reinterpret_cast<uint4*>(p.out + (size_t)t * p.n)[v] = o;
  }
}

inline cudaError_t launch_combine(const CombineParams& p, cudaStream_t stream) {
  if (p.tokens == 0) return cudaSuccess;
  combine_kernel<<<p.tokens, kCombineThreads, 0, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace dg
