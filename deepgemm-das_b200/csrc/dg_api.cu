// C ABI of libdeepgemm_b200.so: argument validation, TMA descriptor encoding, kernel
// selection and launch.  No torch types, no allocation, no stream synchronisation.
#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstring>
#include <mutex>

#include "deepgemm_b200.h"
#include "dg_grouped_gemm.cuh"
#include "dg_grouped_gemm_pair.cuh"
#include "dg_grouped_gemm_w4.cuh"
#include "dg_grouped_gemm_w4s.cuh"
#include "dg_pack.cuh"
#include "dg_moe_chain.cuh"
#include "dg_quant_group.cuh"
#include "dg_ep.cuh"

namespace {

using namespace dg;

thread_local int tl_last_cuda_error = 0;
std::atomic<long long> g_launch_count{0};

int cuda_fail(cudaError_t e) {
  tl_last_cuda_error = static_cast<int>(e);
  return DG_ERR_CUDA;
}

// ---- per-device cache (filled once; the reference queries device properties per call,
//      csrc/arch/gfx936_gfx938_shared/m_grouped_w8a8_gemm_nt_masked.cu:85-89)
constexpr int kMaxDevices = 64;
struct DeviceInfo {
  std::once_flag once;
  int status = DG_ERR_NO_DEVICE;
  int sm_count = 0;
  int max_smem = 0;
  int cc = 0;
};
DeviceInfo g_dev[kMaxDevices];

int device_info(const DeviceInfo** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    tl_last_cuda_error = static_cast<int>(e);
    (void)cudaGetLastError();
    return DG_ERR_NO_DEVICE;
  }
  if (dev < 0 || dev >= kMaxDevices) return DG_ERR_NO_DEVICE;
  DeviceInfo& d = g_dev[dev];
  std::call_once(d.once, [&]() {
    int major = 0, minor = 0;
    if (cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&d.max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) !=
            cudaSuccess ||
        cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev) != cudaSuccess) {
      d.status = DG_ERR_NO_DEVICE;
      return;
    }
    d.cc = major * 10 + minor;
    d.status = (major == 10) ? DG_OK : DG_ERR_NO_DEVICE;
  });
  *out = &d;
  return d.status;
}

// ---- cuTensorMapEncodeTiled through the runtime's driver entry point (no libcuda link)
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
std::once_flag g_encode_once;

EncodeTiledFn get_encode() {
  std::call_once(g_encode_once, []() {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    else
      (void)cudaGetLastError();
  });
  return g_encode;
}

// A tensor map is a pure function of (address, type, extents, strides, box, swizzle), and a
// serving loop calls with the same weights and the same activation buffers step after step:
// each host thread keeps the maps it encoded last in a small direct-mapped table, so a repeated
// call copies 128 bytes instead of entering the driver (about 0.4 us per map, up to eight a call).
struct MapKey {
  const void* base;
  uint64_t dims[3];
  uint64_t strides[2];
  uint32_t box[3];
  int32_t dt, rank, swizzle;
  bool operator==(const MapKey& o) const { return std::memcmp(this, &o, sizeof(MapKey)) == 0; }
};
struct MapSlot {
  MapKey key;
  CUtensorMap map;
  bool used;
};
constexpr int kMapSlots = 256;
std::atomic<unsigned long long> g_map_hits{0}, g_map_misses{0};

// rank-2 or rank-3 tiled map; dims/strides innermost first, strides in bytes for dims 1..
int encode_map(CUtensorMap* map, CUtensorMapDataType dt, int rank, const void* base,
               const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
               CUtensorMapSwizzle swizzle) {
  EncodeTiledFn enc = get_encode();
  if (enc == nullptr) return DG_ERR_CUDA;
  cuuint64_t gdim[3] = {1, 1, 1};
  cuuint64_t gstr[2] = {0, 0};
  cuuint32_t bdim[3] = {1, 1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bdim[i] = box[i];
  }
  for (int i = 0; i + 1 < rank; ++i) gstr[i] = strides_bytes[i];
  thread_local MapSlot slots[kMapSlots] = {};
  MapKey key;
  std::memset(&key, 0, sizeof(key));  // padding bytes take part in the comparison
  key.base = base;
  for (int i = 0; i < 3; ++i) key.dims[i] = gdim[i], key.box[i] = bdim[i];
  key.strides[0] = gstr[0];
  key.strides[1] = gstr[1];
  key.dt = static_cast<int32_t>(dt);
  key.rank = rank;
  key.swizzle = static_cast<int32_t>(swizzle);
  uint64_t h = reinterpret_cast<uint64_t>(base) * 0x9E3779B97F4A7C15ull;
  h ^= (key.dims[1] + 0x632BE59BD9B4E019ull * key.box[1] + (key.dims[0] << 20) + key.dims[2]) * 0xD6E8FEB86659FD93ull;
  MapSlot& slot = slots[(h >> 40) & (kMapSlots - 1)];
  if (slot.used && slot.key == key) {
    *map = slot.map;
    g_map_hits.fetch_add(1, std::memory_order_relaxed);
    return DG_OK;
  }
  g_map_misses.fetch_add(1, std::memory_order_relaxed);
  struct Store {  // fills the slot when the encode below succeeded
    MapSlot& s; const MapKey& k; CUtensorMap* m; bool ok;
    ~Store() { if (ok) { s.key = k; s.map = *m; s.used = true; } }
  } store{slot, key, map, false};
  bool& encoded_ok = store.ok;
  CUresult r = enc(map, dt, static_cast<cuuint32_t>(rank), const_cast<void*>(base), gdim, gstr,
                   bdim, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r == CUDA_ERROR_INVALID_CONTEXT) {
    // A host thread that has made no runtime call of its own yet (a worker thread of the
    // caller) has no context bound for the driver entry point above: bind the device's
    // primary context (cudaFree(nullptr) does nothing else) and try once more.
    cudaFree(nullptr);
    r = enc(map, dt, static_cast<cuuint32_t>(rank), const_cast<void*>(base), gdim, gstr, bdim, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  if (r != CUDA_SUCCESS) {
    tl_last_cuda_error = 10000 + static_cast<int>(r);
    return DG_ERR_CUDA;
  }
  encoded_ok = true;
  return DG_OK;
}

// ---- kernel instantiations: (kind, BN) -> stages so the ring holds ~192-200 KB
template <int KIND, int BN>
struct StagesFor {
  // One K block per stage: two per stage (three 64 KB stages for BN = 128) measured 7 % slower
  // on the decode workload at full SM clock than six 32 KB stages.
  static constexpr int per_stage = kATileBytes + BN * kRowBytes;
  static constexpr int value = (200 * 1024) / per_stage;
};

#ifndef DG_WIDE_STRIPS_ALWAYS
#define DG_WIDE_STRIPS_ALWAYS 0
#endif
constexpr bool kWideStripsAlways = DG_WIDE_STRIPS_ALWAYS != 0;

struct Problem {
  int kind, scale_mode, mode;
  const void* a;
  const void* b;
  void* d;
  const float* a_scale;
  const float* b_scale;
  const int32_t* sched;
  const int32_t* offsets;
  int G, M, N, K, block_n, expected_m;
  int narrow;  // filled by validate_and_launch: KernelParams::narrow
  int dense;     // 1: dg_dense_gemm (row-major weights, no masked_m, any N, out_kind honoured)
  int out_kind;  // DG_OUT_BF16 / DG_OUT_F16 / DG_OUT_F32
  void* debug_acc;
  int32_t* status;
  const int32_t* scatter_tag;
  void* const* scatter_base;  // host array
  int scatter_world;
  int32_t* signal;
  int group_window;
  // MODE_SORTED
  const int32_t* sorted_ids;
  const int32_t* expert_ids;
  const int32_t* num_post_pad;
  const float* row_weight;
  int block_m, num_blocks, num_sorted, real_topk, max_runs;
};

template <int KIND, int BN, bool kGather = false>
int launch(const Problem& pr, const DeviceInfo& dev, cudaStream_t stream) {
  constexpr int STAGES = StagesFor<KIND, BN>::value;
  using L = SmemLayout<KIND, BN, STAGES>;
  static_assert(STAGES >= 2, "ring too shallow");
  static_assert(kGatherDepth < STAGES, "the gathering warps would wait for stages they have not signalled");
  auto kernel = grouped_gemm_kernel<KIND, BN, STAGES, kGather>;

  const int esize = (KIND == DG_KIND_BF16) ? 2 : 1;
  const int elems_per_row = kRowBytes / esize;  // A elements per 128-byte K block
  KernelParams p{};
  p.mode = pr.mode;
  p.scale_mode = pr.scale_mode;
  p.G = pr.G;
  p.M = pr.M;
  p.N = pr.N;
  p.K = pr.K;
  p.kblocks = (pr.K + elems_per_row - 1) / elems_per_row;  // 8-bit kinds: a last half block reads zeros
  p.n_tiles = (pr.N + BN - 1) / BN;
  p.m_blocks = (pr.M + kBM - 1) / kBM;
  p.sched = pr.sched;
  p.offsets = pr.offsets;
  p.a_scale = pr.a_scale;
  p.b_scale = pr.b_scale;
  p.d = static_cast<__nv_bfloat16*>(pr.d);
  p.debug_acc = static_cast<uint32_t*>(pr.debug_acc);
  p.status = pr.status;
  p.b_rowmajor = pr.dense;
  p.out_kind = pr.out_kind;
  p.signal = pr.signal;
  p.group_window = pr.group_window;
  p.scatter_tag = pr.scatter_tag;
  for (int r = 0; r < pr.scatter_world && pr.scatter_tag != nullptr; ++r) p.scatter_base[r] = pr.scatter_base[r];
  p.tbl_groups = pr.mode == MODE_SORTED ? pr.max_runs : pr.G;
  p.sorted_ids = pr.sorted_ids;
  p.expert_ids = pr.expert_ids;
  p.num_post_pad = pr.num_post_pad;
  p.row_weight = pr.row_weight;
  p.gather_a = pr.a;
  p.block_m = pr.block_m;
  p.num_blocks = pr.num_blocks;
  p.num_sorted = pr.num_sorted;
  p.real_topk = pr.real_topk;
  p.size_m = pr.M;

  // MODE_SORTED: 128-entry tiles of the routing list; every run of blocks may end in a partial one
  const long long max_blocks = pr.mode == MODE_MASKED    ? (long long)pr.G * p.m_blocks
                               : pr.mode == MODE_COMPACT ? (long long)p.m_blocks + pr.G
                               : pr.mode == MODE_SORTED  ? (long long)(pr.num_sorted + kBM - 1) / kBM + pr.max_runs
                                                         : (long long)p.m_blocks;
  const long long max_items = max_blocks * p.n_tiles;
  if (max_items <= 0) return DG_OK;
  const int table_bytes = pr.mode == MODE_MASKED    ? (2 * pr.G + 1) * 4
                          : pr.mode == MODE_COMPACT ? (3 * pr.G + 1) * 4
                          : pr.mode == MODE_SORTED  ? (4 * pr.max_runs + 2) * 4
                                                    : p.m_blocks * 4;
  int smem_bytes = L::total(table_bytes);
  if (smem_bytes > dev.max_smem || smem_bytes > kMaxSmem) return DG_ERR_TOO_LARGE;
  // scattered output: wider store strips behind the table when they fit
  if (pr.scatter_tag != nullptr || pr.mode == MODE_SORTED || kWideStripsAlways) {
    const int off = (L::off_table + table_bytes + 15) & ~15;
    if (off + 4 * 4096 + 1024 <= dev.max_smem && off + 4 * 4096 + 1024 <= kMaxSmem) {
      p.wide_off = off;
      smem_bytes = off + 4 * 4096 + 1024;
    }
  }

  // A: rows of K elements.  Masked: (K, max_m, G) so a box never crosses into the next
  // group; contiguous: (K, M_total).  Rows past the extent read as zero.
  const CUtensorMapDataType dt_a =
      (KIND == DG_KIND_BF16) ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  // tm_a64 / tm_a32 fetch the first 64 / 32 rows of it, for tiles with no more valid rows.
  CUtensorMap tm_a, tm_a64, tm_a32, tm_a8, tm_b;
  int rc;
  if (pr.mode == MODE_MASKED) {
    const uint64_t dims[3] = {(uint64_t)pr.K, (uint64_t)pr.M, (uint64_t)pr.G};
    const uint64_t strides[2] = {(uint64_t)pr.K * esize, (uint64_t)pr.M * pr.K * esize};
    const uint32_t box[3] = {(uint32_t)elems_per_row, (uint32_t)kBM, 1u};
    const uint32_t box64[3] = {(uint32_t)elems_per_row, 64u, 1u};
    const uint32_t box32[3] = {(uint32_t)elems_per_row, 32u, 1u};
    const uint32_t box8[3] = {(uint32_t)elems_per_row, 8u, 1u};
    rc = encode_map(&tm_a8, dt_a, 3, pr.a, dims, strides, box8, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc == DG_OK)
      rc = encode_map(&tm_a, dt_a, 3, pr.a, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc == DG_OK)
      rc = encode_map(&tm_a64, dt_a, 3, pr.a, dims, strides, box64, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc == DG_OK)
      rc = encode_map(&tm_a32, dt_a, 3, pr.a, dims, strides, box32, CU_TENSOR_MAP_SWIZZLE_128B);
  } else {
    const uint64_t dims[2] = {(uint64_t)pr.K, (uint64_t)pr.M};
    const uint64_t strides[1] = {(uint64_t)pr.K * esize};
    const uint32_t box[2] = {(uint32_t)elems_per_row, (uint32_t)kBM};
    const uint32_t box64[2] = {(uint32_t)elems_per_row, 64u};
    const uint32_t box32[2] = {(uint32_t)elems_per_row, 32u};
    const uint32_t box8[2] = {(uint32_t)elems_per_row, 8u};
    rc = encode_map(&tm_a8, dt_a, 2, pr.a, dims, strides, box8, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc == DG_OK)
      rc = encode_map(&tm_a, dt_a, 2, pr.a, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc == DG_OK)
      rc = encode_map(&tm_a64, dt_a, 2, pr.a, dims, strides, box64, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc == DG_OK)
      rc = encode_map(&tm_a32, dt_a, 2, pr.a, dims, strides, box32, CU_TENSOR_MAP_SWIZZLE_128B);
  }
  if (rc != DG_OK) return rc;
  // B (packed): a flat list of G*kblocks*N rows of 128 bytes, so a BN-row box is one
  // contiguous span.  Dense GEMM: plain [G*N][K] rows, the box walks along K.
  const uint64_t b_dims[2] = {pr.dense ? (uint64_t)pr.K : (uint64_t)elems_per_row,
                              pr.dense ? (uint64_t)pr.G * pr.N : (uint64_t)pr.G * p.kblocks * pr.N};
  const uint64_t b_strides[1] = {pr.dense ? (uint64_t)pr.K * esize : (uint64_t)kRowBytes};
  {
    const uint32_t box[2] = {(uint32_t)elems_per_row, (uint32_t)BN};
    rc = encode_map(&tm_b, dt_a, 2, pr.b, b_dims, b_strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
  }
  if (rc != DG_OK) return rc;
  // Weight boxes of 128, 64 and 32 rows: narrowed tiles (sparse routing) and the half items of a
  // split last round.
  CUtensorMap tm_b128 = tm_b, tm_b64 = tm_b, tm_b32 = tm_b;
  const bool fixed_tiles = pr.mode == MODE_CONTIG || pr.mode == MODE_SORTED;
  p.narrow = fixed_tiles ? 0 : pr.narrow;
  p.split_tail = fixed_tiles ? 0 : 1;
  if (p.narrow || p.split_tail) {
    const uint32_t box128[2] = {(uint32_t)elems_per_row, 128u};
    const uint32_t box64[2] = {(uint32_t)elems_per_row, 64u};
    const uint32_t box32[2] = {(uint32_t)elems_per_row, 32u};
    rc = encode_map(&tm_b128, dt_a, 2, pr.b, b_dims, b_strides, box128, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc == DG_OK)
      rc = encode_map(&tm_b64, dt_a, 2, pr.b, b_dims, b_strides, box64, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc == DG_OK && p.narrow)
      rc = encode_map(&tm_b32, dt_a, 2, pr.b, b_dims, b_strides, box32, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != DG_OK) return rc;
  }

  // Opt in to the large shared-memory carve-out once per device and instantiation.
  static std::atomic<unsigned long long> configured{0};
  int devid = 0;
  cudaGetDevice(&devid);
  const unsigned long long bit = 1ull << (devid & 63);
  if ((configured.load(std::memory_order_acquire) & bit) == 0) {
    cudaError_t e =
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem);
    if (e != cudaSuccess) return cuda_fail(e);
    configured.fetch_or(bit, std::memory_order_release);
  }

  // With narrowing allowed the item count can reach max_blocks * ceil(N / 32).
  const long long grid_items = p.narrow ? max_blocks * ((pr.N + 31) / 32) : max_items;  // split tails need no more
  const int grid = static_cast<int>(grid_items < dev.sm_count ? grid_items : dev.sm_count);
  kernel<<<grid, L::kThreads + (kGather ? kGatherThreads : 0), smem_bytes, stream>>>(tm_a, tm_a64, tm_a32, tm_a8, tm_b,
                                                                                    tm_b128, tm_b64, tm_b32, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e);
  g_launch_count.fetch_add(1, std::memory_order_relaxed);
  return DG_OK;
}

// Two-CTA (cta_group::2) 256x256 tiles for compute-bound shapes; one cluster per TPC.
template <int KIND>
int launch_pair(const Problem& pr, const DeviceInfo& dev, cudaStream_t stream) {
  using L = PairSmem;
  auto kernel = grouped_gemm_pair_kernel<KIND>;
  const int esize = (KIND == DG_KIND_BF16) ? 2 : 1;
  const int elems_per_row = kRowBytes / esize;
  KernelParams p{};
  p.mode = pr.mode;
  p.scale_mode = pr.scale_mode;
  p.G = pr.G;
  p.M = pr.M;
  p.N = pr.N;
  p.K = pr.K;
  p.kblocks = (pr.K + elems_per_row - 1) / elems_per_row;  // 8-bit kinds: a last half block reads zeros
  p.n_tiles = (pr.N + kPairBN - 1) / kPairBN;
  p.m_blocks = (pr.M + 255) / 256;  // super blocks of 256 rows
  p.sched = pr.sched;
  p.a_scale = pr.a_scale;
  p.b_scale = pr.b_scale;
  p.d = static_cast<__nv_bfloat16*>(pr.d);
  p.debug_acc = static_cast<uint32_t*>(pr.debug_acc);
  p.status = pr.status;
  p.b_rowmajor = pr.dense;
  p.out_kind = pr.out_kind;
  p.group_window = pr.group_window;
  p.scatter_tag = pr.scatter_tag;
  for (int r = 0; r < pr.scatter_world && pr.scatter_tag != nullptr; ++r) p.scatter_base[r] = pr.scatter_base[r];

  const long long max_items =
      (pr.mode == MODE_MASKED ? (long long)pr.G * p.m_blocks : 2LL * p.m_blocks) * p.n_tiles;
  if (max_items <= 0) return DG_OK;
  const int table_bytes = (pr.mode == MODE_MASKED) ? (2 * pr.G + 1) * 4 : 2 * p.m_blocks * 4;
  int smem_bytes = L::total(table_bytes);
  if (smem_bytes > dev.max_smem || smem_bytes > kMaxSmem) return DG_ERR_TOO_LARGE;
  if (pr.scatter_tag != nullptr || kWideStripsAlways) {
    const int off = (L::off_table + table_bytes + 15) & ~15;
    if (off + 4 * 4096 + 1024 <= dev.max_smem && off + 4 * 4096 + 1024 <= kMaxSmem) {
      p.wide_off = off;
      smem_bytes = off + 4 * 4096 + 1024;
    }
  }

  const CUtensorMapDataType dt_a =
      (KIND == DG_KIND_BF16) ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  CUtensorMap tm_a, tm_b;
  int rc;
  if (pr.mode == MODE_MASKED) {
    const uint64_t dims[3] = {(uint64_t)pr.K, (uint64_t)pr.M, (uint64_t)pr.G};
    const uint64_t strides[2] = {(uint64_t)pr.K * esize, (uint64_t)pr.M * pr.K * esize};
    const uint32_t box[3] = {(uint32_t)elems_per_row, 128u, 1u};
    rc = encode_map(&tm_a, dt_a, 3, pr.a, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
  } else {
    const uint64_t dims[2] = {(uint64_t)pr.K, (uint64_t)pr.M};
    const uint64_t strides[1] = {(uint64_t)pr.K * esize};
    const uint32_t box[2] = {(uint32_t)elems_per_row, 128u};
    rc = encode_map(&tm_a, dt_a, 2, pr.a, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
  }
  if (rc != DG_OK) return rc;
  {
    const uint64_t dims[2] = {pr.dense ? (uint64_t)pr.K : (uint64_t)elems_per_row,
                              pr.dense ? (uint64_t)pr.G * pr.N : (uint64_t)pr.G * p.kblocks * pr.N};
    const uint64_t strides[1] = {pr.dense ? (uint64_t)pr.K * esize : (uint64_t)kRowBytes};
    const uint32_t box[2] = {(uint32_t)elems_per_row, 128u};  // each block loads half the tile
    rc = encode_map(&tm_b, dt_a, 2, pr.b, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
  }
  if (rc != DG_OK) return rc;

  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cudaLaunchConfig_t cfg{};
  cfg.blockDim = dim3(L::kThreads, 1, 1);
  cfg.dynamicSmemBytes = static_cast<size_t>(smem_bytes);
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;

  // Once per device: opt in to the shared-memory size and ask how many pairs fit at once
  // (a persistent kernel must not be given more clusters than can be resident together).
  static std::mutex mu;
  static int max_pairs[kMaxDevices] = {0};
  int devid = 0;
  cudaGetDevice(&devid);
  {
    std::lock_guard<std::mutex> lock(mu);
    if (max_pairs[devid] == 0) {
      cudaError_t e =
          cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem);
      if (e != cudaSuccess) return cuda_fail(e);
      cudaLaunchConfig_t q = cfg;
      q.gridDim = dim3(dev.sm_count & ~1, 1, 1);
      q.dynamicSmemBytes = kMaxSmem;
      int n = 0;
      e = cudaOccupancyMaxActiveClusters(&n, kernel, &q);
      if (e != cudaSuccess) return cuda_fail(e);
      if (n < 1) return DG_ERR_TOO_LARGE;
      max_pairs[devid] = n < dev.sm_count / 2 ? n : dev.sm_count / 2;
    }
  }
  long long pairs = max_items < max_pairs[devid] ? max_items : max_pairs[devid];
  cfg.gridDim = dim3(static_cast<unsigned>(2 * pairs), 1, 1);
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, tm_a, tm_b, p);
  if (e != cudaSuccess) return cuda_fail(e);
  g_launch_count.fetch_add(1, std::memory_order_relaxed);
  return DG_OK;
}

// W4A8: swapped orientation, unpacked weights handed to the UMMA through tensor memory.
int launch_w4(const Problem& pr, const DeviceInfo& dev, cudaStream_t stream) {
  using L = W4Smem;
  auto kernel = grouped_gemm_w4_kernel;
  KernelParams p{};
  p.mode = pr.mode;
  p.scale_mode = pr.scale_mode;
  p.G = pr.G;
  p.M = pr.M;
  p.N = pr.N;
  p.K = pr.K;
  p.out_kind = pr.out_kind;
  p.kblocks = pr.K / 256;  // packed-weight stages per item (two 128-value K blocks each)
  p.n_tiles = (pr.N + 127) / 128;
  p.m_blocks = (pr.M + kBM - 1) / kBM;
  p.sched = pr.sched;
  p.a_scale = pr.a_scale;
  p.b_scale = pr.b_scale;
  p.d = static_cast<__nv_bfloat16*>(pr.d);
  p.debug_acc = static_cast<uint32_t*>(pr.debug_acc);
  p.status = pr.status;
  const long long max_items =
      (pr.mode == MODE_MASKED ? (long long)pr.G * p.m_blocks : (long long)p.m_blocks) * p.n_tiles;
  if (max_items <= 0) return DG_OK;
  const int table_bytes = (pr.mode == MODE_MASKED) ? (2 * pr.G + 1) * 4 : p.m_blocks * 4;
  const int smem_bytes = L::total(table_bytes);
  if (smem_bytes > dev.max_smem || smem_bytes > kMaxSmem) return DG_ERR_TOO_LARGE;

  // Token tiles: three boxes (128, 64, 32 rows) so an item fetches no more rows than the next
  // power of two above its valid rows.
  CUtensorMap tm_tok[3], tm_w;
  int rc = DG_OK;
  for (int i = 0; i < 3 && rc == DG_OK; ++i) {
    const uint32_t rows = 128u >> i;
    if (pr.mode == MODE_MASKED) {
      const uint64_t dims[3] = {(uint64_t)pr.K, (uint64_t)pr.M, (uint64_t)pr.G};
      const uint64_t strides[2] = {(uint64_t)pr.K, (uint64_t)pr.M * pr.K};
      const uint32_t box[3] = {128u, rows, 1u};
      rc = encode_map(&tm_tok[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, pr.a, dims, strides, box,
                      CU_TENSOR_MAP_SWIZZLE_128B);
    } else {
      const uint64_t dims[2] = {(uint64_t)pr.K, (uint64_t)pr.M};
      const uint64_t strides[1] = {(uint64_t)pr.K};
      const uint32_t box[2] = {128u, rows};
      rc = encode_map(&tm_tok[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, pr.a, dims, strides, box,
                      CU_TENSOR_MAP_SWIZZLE_128B);
    }
  }
  if (rc != DG_OK) return rc;
  {
    // packed weights: G*(K/256)*N rows of 128 bytes (256 int4 values); a 128-row box is one
    // contiguous 16 KB span
    const uint64_t dims[2] = {128, (uint64_t)pr.G * p.kblocks * pr.N};
    const uint64_t strides[1] = {128};
    const uint32_t box[2] = {128u, 128u};
    rc = encode_map(&tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, pr.b, dims, strides, box,
                    CU_TENSOR_MAP_SWIZZLE_128B);
  }
  if (rc != DG_OK) return rc;

  static std::atomic<unsigned long long> configured{0};
  int devid = 0;
  cudaGetDevice(&devid);
  const unsigned long long bit = 1ull << (devid & 63);
  if ((configured.load(std::memory_order_acquire) & bit) == 0) {
    cudaError_t e =
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem);
    if (e != cudaSuccess) return cuda_fail(e);
    configured.fetch_or(bit, std::memory_order_release);
  }
  const int grid = static_cast<int>(max_items < dev.sm_count ? max_items : dev.sm_count);
  kernel<<<grid, L::kThreads, smem_bytes, stream>>>(tm_tok[0], tm_tok[1], tm_tok[2], tm_w, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e);
  g_launch_count.fetch_add(1, std::memory_order_relaxed);
  return DG_OK;
}

// W4A8, tokens on UMMA M, 256 channels on N, int4 -> int8 unpack in shared memory.
template <int SLOTS, int TOKS, int NG>
int launch_w4_smem(const Problem& pr, const DeviceInfo& dev, cudaStream_t stream) {
  using L = WsSmem<SLOTS, TOKS>;
  auto kernel = grouped_gemm_w4_smem_kernel<SLOTS, TOKS, NG>;
  KernelParams p{};
  p.mode = pr.mode;
  p.scale_mode = pr.scale_mode;
  p.G = pr.G;
  p.M = pr.M;
  p.N = pr.N;
  p.K = pr.K;
  p.kblocks = pr.K / 128;  // K blocks of 128 values; a packed row covers two of them
  p.n_tiles = (pr.N + kWsBN - 1) / kWsBN;
  p.m_blocks = (pr.M + kBM - 1) / kBM;
  p.sched = pr.sched;
  p.a_scale = pr.a_scale;
  p.b_scale = pr.b_scale;
  p.d = static_cast<__nv_bfloat16*>(pr.d);
  p.debug_acc = static_cast<uint32_t*>(pr.debug_acc);
  p.status = pr.status;
  p.out_kind = pr.out_kind;
  p.split_tail = (pr.mode == MODE_MASKED) ? 1 : 0;
  const long long max_items =
      (pr.mode == MODE_MASKED ? (long long)pr.G * p.m_blocks : (long long)p.m_blocks) * p.n_tiles;
  if (max_items <= 0) return DG_OK;
  const int table_bytes = (pr.mode == MODE_MASKED) ? (2 * pr.G + 1) * 4 : p.m_blocks * 4;
  // the packed ring takes what the opt-in shared-memory limit leaves after the slots and the table
  const int limit = dev.max_smem < kMaxSmem ? dev.max_smem : kMaxSmem;
  int stages = (limit - L::total(table_bytes, 0)) / kWsPackStageBytes;
  if (stages > kWsMaxPackStages) stages = kWsMaxPackStages;
  if (stages < 2) return DG_ERR_TOO_LARGE;
  p.pack_stages = stages;
  p.pack_off = L::pack_offset(table_bytes);
  const int smem_bytes = L::total(table_bytes, stages);

  // Token tiles: boxes of 128, 64, 32 and 8 rows, so an item fetches little more than its rows.
  CUtensorMap tm_tok[4], tm_w, tm_w128;
  int rc = DG_OK;
  const uint32_t tok_rows[4] = {128u, 64u, 32u, 8u};
  for (int i = 0; i < 4 && rc == DG_OK; ++i) {
    if (pr.mode == MODE_MASKED) {
      const uint64_t dims[3] = {(uint64_t)pr.K, (uint64_t)pr.M, (uint64_t)pr.G};
      const uint64_t strides[2] = {(uint64_t)pr.K, (uint64_t)pr.M * pr.K};
      const uint32_t box[3] = {128u, tok_rows[i], 1u};
      rc = encode_map(&tm_tok[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, pr.a, dims, strides, box,
                      CU_TENSOR_MAP_SWIZZLE_128B);
    } else {
      const uint64_t dims[2] = {(uint64_t)pr.K, (uint64_t)pr.M};
      const uint64_t strides[1] = {(uint64_t)pr.K};
      const uint32_t box[2] = {128u, tok_rows[i]};
      rc = encode_map(&tm_tok[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, pr.a, dims, strides, box,
                      CU_TENSOR_MAP_SWIZZLE_128B);
    }
  }
  if (rc != DG_OK) return rc;
  {
    // packed weights: G*(K/256)*N rows of 128 bytes (256 int4 values); a box is the 64-byte half
    // of 256 (or 128) consecutive rows that holds one K block, stored linearly in shared memory
    const uint64_t dims[2] = {128, (uint64_t)pr.G * (pr.K / 256) * pr.N};
    const uint64_t strides[1] = {128};
    const uint32_t box[2] = {64u, (uint32_t)kWsBN};
    const uint32_t box128[2] = {64u, 128u};
    rc = encode_map(&tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, pr.b, dims, strides, box,
                    CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc == DG_OK)
      rc = encode_map(&tm_w128, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, pr.b, dims, strides, box128,
                      CU_TENSOR_MAP_SWIZZLE_NONE);
  }
  if (rc != DG_OK) return rc;

  static std::atomic<unsigned long long> configured{0};
  int devid = 0;
  cudaGetDevice(&devid);
  const unsigned long long bit = 1ull << (devid & 63);
  if ((configured.load(std::memory_order_acquire) & bit) == 0) {
    cudaError_t e =
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem);
    if (e != cudaSuccess) return cuda_fail(e);
    configured.fetch_or(bit, std::memory_order_release);
  }
  const int grid = static_cast<int>(max_items < dev.sm_count ? max_items : dev.sm_count);
  kernel<<<grid, L::kThreads, smem_bytes, stream>>>(tm_tok[0], tm_tok[1], tm_tok[2], tm_tok[3], tm_w,
                                                    tm_w128, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e);
  g_launch_count.fetch_add(1, std::memory_order_relaxed);
  return DG_OK;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int validate_and_launch(Problem& pr, cudaStream_t stream) {
  if (pr.kind < DG_KIND_I8 || pr.kind > DG_KIND_BF16) return DG_ERR_BAD_KIND;
  if (pr.scale_mode < DG_SCALE_PER_CHANNEL || pr.scale_mode > DG_SCALE_NONE)
    return DG_ERR_BAD_SCALE_MODE;
  if (!pr.dense && (pr.kind == DG_KIND_BF16) != (pr.scale_mode == DG_SCALE_NONE))
    return DG_ERR_BAD_SCALE_MODE;
  if (pr.G < 1 || pr.M < 0 || pr.N < (pr.dense ? 1 : 16) || pr.K < 1) return DG_ERR_BAD_SHAPE;
  if (pr.out_kind < DG_OUT_BF16 || pr.out_kind > DG_OUT_F32) return DG_ERR_BAD_ARGUMENT;
  if (pr.dense && pr.kind == DG_KIND_W4A8) return DG_ERR_BAD_KIND;
  if (pr.G > DG_MAX_GROUPS) return DG_ERR_TOO_LARGE;
  if (pr.mode != MODE_MASKED && pr.M > DG_MAX_CONTIG_ROWS) return DG_ERR_TOO_LARGE;
  if (pr.mode == MODE_COMPACT && pr.kind == DG_KIND_W4A8) return DG_ERR_BAD_KIND;
  if (!pr.dense && pr.N % 16 != 0) return DG_ERR_BAD_SHAPE;
  // INT8 / FP8: K % 64 (the reference's W6 block, deepgemm/m_group_gemm.py:815-818).  The kernels step K
  // in 128-byte blocks: the packed weight then carries ceil(K / 128) blocks whose tail is zero
  // (the packers pad it) and TMA fills the activation's last half block with zeros.
  const int kq = (pr.kind == DG_KIND_W4A8) ? 256 : 64;
  if (pr.K % kq != 0) return DG_ERR_BAD_SHAPE;
  const int kstep = (pr.kind == DG_KIND_BF16) ? 64 : (pr.kind == DG_KIND_W4A8 ? 256 : 128);
  if ((long long)pr.G * ((pr.K + kstep - 1) / kstep) * pr.N > 0x7fffffffLL) return DG_ERR_TOO_LARGE;
  if (pr.M == 0) return DG_OK;
  if (!pr.a || !pr.b || !pr.d || (!pr.sched && !pr.dense && pr.mode != MODE_SORTED)) return DG_ERR_NULL_POINTER;
  if (pr.mode == MODE_COMPACT && !pr.offsets) return DG_ERR_NULL_POINTER;
  if (pr.scale_mode != DG_SCALE_NONE && (!pr.a_scale || !pr.b_scale)) return DG_ERR_NULL_POINTER;
  if (!aligned16(pr.a) || !aligned16(pr.b) || !aligned16(pr.d)) return DG_ERR_BAD_ALIGNMENT;
  if (pr.scale_mode == DG_SCALE_PER_CHANNEL && !aligned16(pr.b_scale)) return DG_ERR_BAD_ALIGNMENT;
  // fp32 output and rows of D that start unaligned exist only in the one-CTA kernel
  const bool scalar_out = pr.out_kind == DG_OUT_F32 || (pr.N % 8) != 0;
  if (!pr.dense && pr.out_kind == DG_OUT_F32) return DG_ERR_BAD_ARGUMENT;  // grouped outputs are 16-bit
  if (pr.debug_acc && !aligned16(pr.debug_acc)) return DG_ERR_BAD_ALIGNMENT;
  if (pr.block_n != 0 && pr.block_n != 32 && pr.block_n != 64 && pr.block_n != 128 &&
      pr.block_n != 256 && pr.block_n != 512)
    return DG_ERR_BAD_ARGUMENT;
  if ((pr.block_n == 32 || pr.block_n == 64) && (pr.mode == MODE_CONTIG || pr.kind == DG_KIND_W4A8))
    return DG_ERR_BAD_ARGUMENT;

  const DeviceInfo* dev = nullptr;
  int rc = device_info(&dev);
  if (rc != DG_OK) return rc;

  // Tile choice.  Weight-streaming shapes (few rows per group) want many equal items so the
  // 148 SMs stay balanced: one-CTA tiles, BN = 128.  Compute-bound shapes want the least
  // operand traffic per flop: two-CTA 256x256 tiles when there are enough of them to fill
  // every SM pair twice, else one-CTA 128x256 tiles.
  int bn = pr.block_n;
  // Tiles may narrow on the device when few groups have rows: always when the library chooses,
  // never when the caller asked for an exact width (128 / 256), to a fixed width for 32 / 64.
  pr.narrow = (bn == 0) ? 1 : ((bn == 32 || bn == 64) ? bn : 0);
  if (bn == 32 || bn == 64) bn = 128;
  if (bn == 0) {
    const long long rows = (pr.mode != MODE_MASKED) ? (long long)pr.M
                                                    : (long long)pr.G * (pr.expected_m > 0 ? pr.expected_m : 0);
    // rows per group (padding included) decide whether 256-row super blocks are mostly real
    // rows; measured on 32768 routed rows over 256 / 128 / 64 / 32 groups the two-CTA tiles win
    // from about 380 allocated rows per group upwards and lose at 256
    const bool big_groups = (pr.mode == MODE_CONTIG) ? (rows / pr.G >= 320) : (pr.expected_m >= 256);
    const long long pair_items = (rows / 256) * (pr.N / 256);
    if (pr.mode == MODE_COMPACT)
      bn = (pr.N >= 256 && (rows / 128) * (pr.N / 256) >= dev->sm_count) ? 256 : 128;
    else if (pr.mode == MODE_SORTED)  // the gathering producer lives in the one-CTA kernel
      bn = (pr.N >= 256 && ((long long)pr.num_sorted / 128) * (pr.N / 256) >= dev->sm_count) ? 256 : 128;
    else if (big_groups && pr.N >= 256 && pair_items >= 2LL * (dev->sm_count / 2))
      bn = 512;
    else if (pr.mode == MODE_CONTIG)
      bn = (pr.N >= 256 && (rows / 128) * (pr.N / 256) >= dev->sm_count) ? 256 : 128;
    else {
      // Weight-streaming (decode) shapes.  256-column tiles move half the activation bytes from
      // L2, issue half the UMMAs per weight byte and keep more weight bytes in flight per SM
      // (4 x 32 KB against 6 x 16 KB): within 1 % of 128-column tiles at the full SM clock on
      // the 32 x 4096 x 7168 decode shape, 10-15 % faster on a power-capped GPU, 27 % faster
      // with 8 rows in every expert.  With few active experts the kernel narrows them on the
      // device, so they serve every row count.
      bn = (pr.N % 256 == 0) ? 256 : 128;
    }
  }
  if (bn == 512 && (pr.N < 256 || pr.mode == MODE_COMPACT)) bn = 128;
  if (bn == 512 && pr.mode == MODE_SORTED) bn = 256;
  if (bn == 512 && pr.signal != nullptr) bn = 256;  // completion counters live in the one-CTA kernel
  if (bn == 512 && scalar_out) bn = 256;
  if (pr.kind == DG_KIND_W4A8) {
    if (pr.block_n == 512) return launch_w4_smem<3, 3, 4>(pr, *dev, stream);
    return launch_w4(pr, *dev, stream);
  }

  if (bn == 512) {  // two-CTA 256x256 tiles
    switch (pr.kind) {
      case DG_KIND_I8: return launch_pair<DG_KIND_I8>(pr, *dev, stream);
      case DG_KIND_E4M3: return launch_pair<DG_KIND_E4M3>(pr, *dev, stream);
      case DG_KIND_BF16: return launch_pair<DG_KIND_BF16>(pr, *dev, stream);
      default: return DG_ERR_BAD_KIND;
    }
  }
  if (pr.mode == MODE_SORTED) {
    if (pr.kind == DG_KIND_I8)
      return bn == 256 ? launch<DG_KIND_I8, 256, true>(pr, *dev, stream) : launch<DG_KIND_I8, 128, true>(pr, *dev, stream);
    return bn == 256 ? launch<DG_KIND_E4M3, 256, true>(pr, *dev, stream)
                     : launch<DG_KIND_E4M3, 128, true>(pr, *dev, stream);
  }
  switch (pr.kind) {
    case DG_KIND_I8:
      return bn == 256 ? launch<DG_KIND_I8, 256>(pr, *dev, stream)
                       : launch<DG_KIND_I8, 128>(pr, *dev, stream);
    case DG_KIND_E4M3:
      return bn == 256 ? launch<DG_KIND_E4M3, 256>(pr, *dev, stream)
                       : launch<DG_KIND_E4M3, 128>(pr, *dev, stream);
    case DG_KIND_BF16:
      return bn == 256 ? launch<DG_KIND_BF16, 256>(pr, *dev, stream)
                       : launch<DG_KIND_BF16, 128>(pr, *dev, stream);
    default:
      break;
  }
  return DG_ERR_BAD_KIND;
}

}  // namespace

extern "C" {

int dg_masked_gemm(const dg_masked_args* a, void* stream) {
  if (a == nullptr) return DG_ERR_NULL_POINTER;
  Problem pr{};
  pr.kind = a->kind;
  pr.scale_mode = a->scale_mode;
  pr.mode = MODE_MASKED;
  pr.a = a->a;
  pr.b = a->b_packed;
  pr.d = a->d;
  pr.a_scale = a->a_scale;
  pr.b_scale = a->b_scale;
  pr.sched = a->masked_m;
  pr.G = a->num_groups;
  pr.M = a->max_m;
  pr.N = a->n;
  pr.K = a->k;
  pr.block_n = a->block_n;
  pr.expected_m = a->expected_m;
  pr.debug_acc = a->debug_acc;
  pr.status = a->status;
  pr.out_kind = a->out_kind;
  if (a->signal != nullptr) {
    // a tile's columns are credited in four equal parts: N % 32 == 0 keeps them whole numbers
    if (a->kind == DG_KIND_W4A8 || a->n % 32 != 0) return DG_ERR_BAD_ARGUMENT;
    pr.signal = a->signal;
  }
  return validate_and_launch(pr, static_cast<cudaStream_t>(stream));
}

int dg_compact_gemm(const dg_compact_args* a, void* stream) {
  if (a == nullptr) return DG_ERR_NULL_POINTER;
  Problem pr{};
  pr.kind = a->kind;
  pr.scale_mode = a->scale_mode;
  pr.mode = MODE_COMPACT;
  pr.a = a->a;
  pr.b = a->b_packed;
  pr.d = a->d;
  pr.a_scale = a->a_scale;
  pr.b_scale = a->b_scale;
  pr.sched = a->counts;
  pr.offsets = a->offsets;
  pr.G = a->num_groups;
  pr.M = a->capacity;
  pr.N = a->n;
  pr.K = a->k;
  pr.block_n = a->block_n;
  pr.expected_m = a->expected_m;
  pr.debug_acc = a->debug_acc;
  pr.status = a->status;
  return validate_and_launch(pr, static_cast<cudaStream_t>(stream));
}

int dg_dense_gemm(const dg_dense_args* a, void* stream) {
  if (a == nullptr) return DG_ERR_NULL_POINTER;
  if ((a->a_scale == nullptr) != (a->b_scale == nullptr)) return DG_ERR_BAD_ARGUMENT;
  Problem pr{};
  pr.kind = a->kind;
  pr.scale_mode = a->a_scale ? DG_SCALE_PER_CHANNEL : DG_SCALE_NONE;
  if (a->kind == DG_KIND_BF16 && a->a_scale) return DG_ERR_BAD_SCALE_MODE;
  pr.mode = MODE_MASKED;  // batch = groups, every row valid
  pr.dense = 1;
  pr.out_kind = a->out_kind;
  pr.a = a->a;
  pr.b = a->b;
  pr.d = a->d;
  pr.a_scale = a->a_scale;
  pr.b_scale = a->b_scale;
  pr.sched = nullptr;
  pr.G = a->batch;
  pr.M = a->m;
  pr.N = a->n;
  pr.K = a->k;
  pr.block_n = a->block_n;
  pr.expected_m = a->m;
  pr.debug_acc = a->debug_acc;
  pr.status = a->status;
  return validate_and_launch(pr, static_cast<cudaStream_t>(stream));
}

int dg_contig_gemm(const dg_contig_args* a, void* stream) {
  if (a == nullptr) return DG_ERR_NULL_POINTER;
  Problem pr{};
  pr.kind = a->kind;
  pr.scale_mode = a->scale_mode;
  pr.mode = MODE_CONTIG;
  pr.a = a->a;
  pr.b = a->b_packed;
  pr.d = a->d;
  pr.a_scale = a->a_scale;
  pr.b_scale = a->b_scale;
  pr.sched = a->m_indices;
  pr.G = a->num_groups;
  pr.M = a->m_total;
  pr.N = a->n;
  pr.K = a->k;
  pr.block_n = a->block_n;
  pr.expected_m = 0;
  pr.debug_acc = a->debug_acc;
  pr.status = a->status;
  pr.out_kind = a->out_kind;
  if (a->group_window < 0 || (a->group_window > 0 && a->kind == DG_KIND_W4A8)) return DG_ERR_BAD_ARGUMENT;
  pr.group_window = a->group_window;
  if (a->scatter_tag != nullptr) {
    if (a->scatter_base == nullptr) return DG_ERR_NULL_POINTER;
    if (a->scatter_world < 1 || a->scatter_world > DG_EP_MAX_WORLD) return DG_ERR_BAD_ARGUMENT;
    if (a->kind == DG_KIND_W4A8 || a->n % 8 != 0 || a->debug_acc != nullptr || a->out_kind != DG_OUT_BF16)
      return DG_ERR_BAD_ARGUMENT;
    for (int r = 0; r < a->scatter_world; ++r)
      if (a->scatter_base[r] == nullptr || !aligned16(a->scatter_base[r])) return DG_ERR_BAD_ALIGNMENT;
    pr.scatter_tag = a->scatter_tag;
    pr.scatter_base = a->scatter_base;
    pr.scatter_world = a->scatter_world;
  }
  return validate_and_launch(pr, static_cast<cudaStream_t>(stream));
}

int dg_sorted_gemm(const dg_sorted_args* a, void* stream) {
  if (a == nullptr) return DG_ERR_NULL_POINTER;
  if (a->kind != DG_KIND_I8 && a->kind != DG_KIND_E4M3) return DG_ERR_BAD_KIND;
  if (a->num_sorted < 0 || a->block_m < 1 || a->num_blocks < 0 || a->real_topk < 1 || a->size_m < 0)
    return DG_ERR_BAD_ARGUMENT;
  if ((long long)a->num_blocks * a->block_m < a->num_sorted) return DG_ERR_BAD_ARGUMENT;
  if (a->size_m > 0x00FFFFFF * (long long)a->real_topk || a->num_sorted > DG_MAX_CONTIG_ROWS) return DG_ERR_TOO_LARGE;
  if (a->num_sorted == 0 || a->num_blocks == 0 || a->size_m == 0) return DG_OK;
  if (!a->sorted_token_ids || !a->expert_ids || !a->num_tokens_post_pad) return DG_ERR_NULL_POINTER;
  Problem pr{};
  pr.kind = a->kind;
  pr.scale_mode = DG_SCALE_PER_CHANNEL;
  pr.mode = MODE_SORTED;
  pr.a = a->a;
  pr.b = a->b_packed;
  pr.d = a->d;
  pr.a_scale = a->a_scale;
  pr.b_scale = a->b_scale;
  pr.row_weight = a->row_weight;
  pr.sorted_ids = a->sorted_token_ids;
  pr.expert_ids = a->expert_ids;
  pr.num_post_pad = a->num_tokens_post_pad;
  pr.G = a->num_groups;
  pr.M = a->size_m;
  pr.N = a->n;
  pr.K = a->k;
  pr.block_m = a->block_m;
  pr.num_blocks = a->num_blocks;
  pr.num_sorted = a->num_sorted;
  pr.real_topk = a->real_topk;
  // runs of blocks with one expert: one per expert in a sorted list, some more for the blocks of
  // experts that live elsewhere; more than this many and the launch reports DG_DEV_BAD_GROUP_INDEX
  const long long runs = 2LL * a->num_groups + 2;
  pr.max_runs = static_cast<int>(runs < a->num_blocks ? runs : a->num_blocks);
  pr.out_kind = DG_OUT_BF16;
  pr.status = a->status;
  if (a->n % 8 != 0) return DG_ERR_BAD_SHAPE;  // result rows leave through 16-byte stores
  return validate_and_launch(pr, static_cast<cudaStream_t>(stream));
}

static int pack_common(bool unpack, int32_t kind, const void* src, void* dst, int32_t G,
                       int32_t n, int32_t k, int32_t nibble_order, void* stream) {
  if (kind < DG_KIND_I8 || kind > DG_KIND_BF16) return DG_ERR_BAD_KIND;
  if (!src || !dst) return DG_ERR_NULL_POINTER;
  if (G < 1 || n < 1 || k < 1) return DG_ERR_BAD_SHAPE;
  const int kq = (kind == DG_KIND_BF16) ? 64 : (kind == DG_KIND_W4A8 ? 256 : 128);
  if (k % kq != 0) return DG_ERR_BAD_SHAPE;
  if (!aligned16(src) || !aligned16(dst)) return DG_ERR_BAD_ALIGNMENT;
  if (nibble_order != DG_NIBBLE_HIGH_FIRST && nibble_order != DG_NIBBLE_LOW_FIRST)
    return DG_ERR_BAD_ARGUMENT;
  const DeviceInfo* dev = nullptr;
  int rc = device_info(&dev);
  if (rc != DG_OK) return rc;
  cudaError_t e = dg::launch_pack(unpack, kind, src, dst, G, n, k, nibble_order,
                                  static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e);
  g_launch_count.fetch_add(1, std::memory_order_relaxed);
  return DG_OK;
}

int dg_pack_weight(int32_t kind, const void* src, void* dst, int32_t G, int32_t n, int32_t k,
                   int32_t nibble_order, void* stream) {
  return pack_common(false, kind, src, dst, G, n, k, nibble_order, stream);
}

int dg_unpack_weight(int32_t kind, const void* src, void* dst, int32_t G, int32_t n, int32_t k,
                     int32_t nibble_order, void* stream) {
  return pack_common(true, kind, src, dst, G, n, k, nibble_order, stream);
}

size_t dg_quant_group_scratch_bytes(int32_t num_rows, int32_t num_groups) {
  if (num_rows < 0 || num_groups < 1 || num_groups > DG_MAX_GROUPS) return 0;
  const size_t chunks = (static_cast<size_t>(num_rows) + dg::kQgChunk - 1) / dg::kQgChunk;
  return (chunks * num_groups + num_groups) * sizeof(int32_t) + 256;
}

// Shared by dg_quant_group_rows and its variant with library-owned scratch.
static int quant_group_common(const dg_quant_group_args* a, int32_t* scratch, void* stream) {
  if (a->kind != DG_KIND_E4M3 && a->kind != DG_KIND_I8) return DG_ERR_BAD_KIND;
  if (a->num_rows < 0 || a->hidden < 8 || a->hidden % 8 != 0 || a->num_groups < 1 ||
      a->align < 1 || a->m_cap < 0)
    return DG_ERR_BAD_SHAPE;
  if (a->row_scale != nullptr && a->hidden % 16 != 0) return DG_ERR_BAD_SHAPE;  // 16-byte copies
  if (a->num_groups > DG_MAX_GROUPS || a->hidden > DG_MAX_QUANT_HIDDEN) return DG_ERR_TOO_LARGE;
  if (!a->a_out || !a->a_scale_out || !a->m_indices_out || !scratch) return DG_ERR_NULL_POINTER;
  if (a->num_rows > 0 && (!a->rows || !a->expert)) return DG_ERR_NULL_POINTER;
  if (!aligned16(a->rows) || !aligned16(a->a_out) || !aligned16(scratch)) return DG_ERR_BAD_ALIGNMENT;
  const DeviceInfo* dev = nullptr;
  int rc = device_info(&dev);
  if (rc != DG_OK) return rc;
  dg::QuantGroupParams p{};
  p.rows = static_cast<const __nv_bfloat16*>(a->rows);
  p.expert = a->expert;
  p.src_index = a->src_index;
  p.row_scale = a->row_scale;
  p.a_out = a->a_out;
  p.a_scale_out = a->a_scale_out;
  p.m_indices_out = a->m_indices_out;
  p.dest_out = a->dest_out;
  p.m_total_out = a->m_total_out;
  p.R = a->num_rows;
  p.H = a->hidden;
  p.G = a->num_groups;
  p.align = a->align;
  p.m_cap = a->m_cap;
  p.chunks = (a->num_rows + dg::kQgChunk - 1) / dg::kQgChunk;
  p.kind = a->kind;
  p.hist = scratch;
  p.starts = scratch + static_cast<size_t>(p.chunks) * p.G;
  cudaError_t e = dg::launch_quant_group(p, dev->sm_count, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e);
  g_launch_count.fetch_add(a->num_rows > 0 ? 4 : 1, std::memory_order_relaxed);
  return DG_OK;
}

int dg_quant_group_rows(const dg_quant_group_args* a, void* stream) {
  if (a == nullptr) return DG_ERR_NULL_POINTER;
  if (a->num_groups >= 1 && a->num_groups <= DG_MAX_GROUPS && a->num_rows >= 0 &&
      a->scratch_bytes < dg_quant_group_scratch_bytes(a->num_rows, a->num_groups))
    return DG_ERR_BAD_ARGUMENT;
  return quant_group_common(a, static_cast<int32_t*>(a->scratch), stream);
}

int dg_group_sorted_rows(const dg_group_sorted_args* a, void* stream) {
  if (a == nullptr) return DG_ERR_NULL_POINTER;
  if (a->num_sorted < 0 || a->block_m < 1 || a->size_m < 0 || a->hidden < 16 || a->hidden % 16 != 0 ||
      a->num_groups < 1 || a->align < 1 || a->m_cap < 0 || a->real_topk < 1 || a->real_topk > 255)
    return DG_ERR_BAD_SHAPE;
  if (a->num_groups > DG_MAX_GROUPS) return DG_ERR_TOO_LARGE;
  if (!a->a_out || !a->a_scale_out || !a->m_indices_out || !a->scratch) return DG_ERR_NULL_POINTER;
  if (a->num_sorted > 0 && (!a->rows || !a->row_scale || !a->sorted_token_ids || !a->expert_ids ||
                            !a->num_tokens_post_pad))
    return DG_ERR_NULL_POINTER;
  if (!aligned16(a->rows) || !aligned16(a->a_out) || !aligned16(a->scratch)) return DG_ERR_BAD_ALIGNMENT;
  if (a->scratch_bytes < dg_quant_group_scratch_bytes(a->num_sorted, a->num_groups))
    return DG_ERR_BAD_ARGUMENT;
  dg::QuantGroupParams p{};
  p.rows = static_cast<const __nv_bfloat16*>(a->rows);
  p.sorted_ids = a->sorted_token_ids;
  p.expert_ids = a->expert_ids;
  p.num_post_pad = a->num_tokens_post_pad;
  p.row_scale = a->row_scale;
  p.row_weight = a->row_weight;
  p.block_m = a->block_m;
  p.real_topk = a->real_topk;
  p.size_m = a->size_m;
  p.a_out = a->a_out;
  p.a_scale_out = a->a_scale_out;
  p.m_indices_out = a->m_indices_out;
  p.dest_out = a->dest_out;
  p.src_out = a->src_out;
  if (a->zero_rows != nullptr && (a->zero_row_bytes < 16 || a->zero_row_bytes % 16 != 0 || !aligned16(a->zero_rows)))
    return DG_ERR_BAD_ARGUMENT;
  p.zero_rows = a->zero_rows;
  p.zero_row_bytes = a->zero_row_bytes;
  p.m_total_out = a->m_total_out;
  p.R = a->num_sorted;
  p.H = a->hidden;
  p.G = a->num_groups;
  p.align = a->align;
  p.m_cap = a->m_cap;
  p.chunks = (a->num_sorted + dg::kQgChunk - 1) / dg::kQgChunk;
  p.kind = DG_KIND_I8;
  p.hist = static_cast<int32_t*>(a->scratch);
  p.starts = p.hist + static_cast<size_t>(p.chunks) * p.G;
  const DeviceInfo* dev = nullptr;
  const int rc = device_info(&dev);
  if (rc != DG_OK) return rc;
  cudaError_t e = dg::launch_quant_group(p, dev->sm_count, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e);
  g_launch_count.fetch_add(a->num_sorted > 0 ? 4 : 1, std::memory_order_relaxed);
  return DG_OK;
}

int dg_silu_mul_quant_rows(const dg_act_quant_args* a, void* stream) {
  if (a == nullptr) return DG_ERR_NULL_POINTER;
  if (a->kind != DG_KIND_E4M3 && a->kind != DG_KIND_I8) return DG_ERR_BAD_KIND;
  if (a->num_rows < 0 || a->hidden <= 0 || a->hidden % 8 != 0) return DG_ERR_BAD_SHAPE;
  if (a->hidden > DG_MAX_QUANT_HIDDEN) return DG_ERR_TOO_LARGE;
  if (a->masked_m != nullptr && (a->max_m <= 0 || a->num_rows % a->max_m != 0)) return DG_ERR_BAD_SHAPE;
  if (a->num_rows == 0) return DG_OK;
  if (!a->x || !a->q_out || !a->scale_out) return DG_ERR_NULL_POINTER;
  if (!aligned16(a->x) || ((uintptr_t)a->q_out & 7) != 0) return DG_ERR_BAD_ALIGNMENT;
  ActQuantParams p{};
  p.kind = a->kind;
  p.rows = a->num_rows;
  p.H = a->hidden;
  p.max_m = a->max_m;
  p.x = static_cast<const __nv_bfloat16*>(a->x);
  p.m_indices = a->m_indices;
  p.masked_m = a->masked_m;
  p.q_out = a->q_out;
  p.scale_out = a->scale_out;
  cudaError_t e = launch_act_quant(p, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e);
  g_launch_count.fetch_add(1, std::memory_order_relaxed);
  return DG_OK;
}

int dg_combine_rows(const dg_combine_args* a, void* stream) {
  if (a == nullptr) return DG_ERR_NULL_POINTER;
  if (a->num_tokens < 0 || a->top_k <= 0 || a->n <= 0 || a->n % 8 != 0 || a->num_rows < 0)
    return DG_ERR_BAD_SHAPE;
  if (a->num_tokens == 0) return DG_OK;
  if (!a->y || !a->src_row || !a->out) return DG_ERR_NULL_POINTER;
  if (!aligned16(a->y) || !aligned16(a->out)) return DG_ERR_BAD_ALIGNMENT;
  CombineParams p{};
  p.tokens = a->num_tokens;
  p.top_k = a->top_k;
  p.n = a->n;
  p.rows = a->num_rows;
  p.y = static_cast<const __nv_bfloat16*>(a->y);
  p.src_row = a->src_row;
  p.weights = a->weights;
  p.out = static_cast<__nv_bfloat16*>(a->out);
  cudaError_t e = launch_combine(p, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e);
  g_launch_count.fetch_add(1, std::memory_order_relaxed);
  return DG_OK;
}

// ---- library-owned scratch for dg_quant_group_rows_noalloc.  In host code the array's name
// is only a handle: its device address is looked up once per device with
// cudaGetSymbolAddress and that pointer is what the kernels receive.
static __device__ __align__(256) int32_t g_noalloc_scratch[DG_NOALLOC_MAX_SCRATCH_INTS];
static std::mutex g_noalloc_mu;
static int32_t* g_noalloc_ptr[kMaxDevices] = {nullptr};

int dg_quant_group_rows_noalloc(const dg_quant_group_args* a, void* stream) {
  if (a == nullptr) return DG_ERR_NULL_POINTER;
  if (a->num_rows < 0 || a->num_groups < 1) return DG_ERR_BAD_SHAPE;
  if (a->num_groups > DG_MAX_GROUPS) return DG_ERR_TOO_LARGE;
  const long long chunks = (static_cast<long long>(a->num_rows) + dg::kQgChunk - 1) / dg::kQgChunk;
  if (chunks * a->num_groups + a->num_groups > static_cast<long long>(DG_NOALLOC_MAX_SCRATCH_INTS))
    return DG_ERR_TOO_LARGE;  // does not fit the built-in scratch array
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    tl_last_cuda_error = static_cast<int>(e);
    (void)cudaGetLastError();
    return DG_ERR_NO_DEVICE;
  }
  if (dev < 0 || dev >= kMaxDevices) return DG_ERR_NO_DEVICE;
  int32_t* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_noalloc_mu);
    if (g_noalloc_ptr[dev] == nullptr) {  // first call on this device (which is current)
      void* ptr = nullptr;
      e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
      if (e != cudaSuccess) return cuda_fail(e);
      g_noalloc_ptr[dev] = static_cast<int32_t*>(ptr);
    }
    scratch = g_noalloc_ptr[dev];
  }
  return quant_group_common(a, scratch, stream);
}

// ---- expert-parallel exchange over peer memory (dg_ep.cuh)
static int ep_copy_peers(dg::EpPeers* dst, void* const* src, int world) {
  if (src == nullptr) return DG_ERR_NULL_POINTER;
  for (int r = 0; r < dg::kEpMaxWorld; ++r) dst->ptr[r] = nullptr;
  for (int r = 0; r < world; ++r) {
    if (src[r] == nullptr) return DG_ERR_NULL_POINTER;
    dst->ptr[r] = src[r];
  }
  return DG_OK;
}

int dg_ep_plan(const dg_ep_plan_args* a, void* stream) {
  if (a == nullptr) return DG_ERR_NULL_POINTER;
  if (a->world < 1 || a->world > DG_EP_MAX_WORLD || a->rank < 0 || a->rank >= a->world)
    return DG_ERR_BAD_ARGUMENT;
  if (a->num_experts < a->world || a->num_experts % a->world != 0 || a->num_pairs < 0 || a->align < 1 ||
      a->m_cap < a->align)
    return DG_ERR_BAD_SHAPE;
  if (a->num_experts > DG_MAX_GROUPS) return DG_ERR_TOO_LARGE;
  if (!a->my_base || !a->cursor || !a->m_indices || !a->m_total || (a->num_pairs > 0 && !a->topk_ids))
    return DG_ERR_NULL_POINTER;
  dg::EpPlanParams p{};
  int rc = ep_copy_peers(&p.peer_counts, a->peer_counts, a->world);
  if (rc == DG_OK) rc = ep_copy_peers(&p.peer_flags, a->peer_flags, a->world);
  if (rc != DG_OK) return rc;
  p.topk_ids = a->topk_ids;
  p.pairs = a->num_pairs;
  p.E = a->num_experts;
  p.world = a->world;
  p.me = a->rank;
  p.e_local = a->num_experts / a->world;
  p.align = a->align;
  p.m_cap = a->m_cap;
  p.counts = static_cast<int32_t*>(p.peer_counts.ptr[a->rank]);
  p.flags = static_cast<int32_t*>(p.peer_flags.ptr[a->rank]);
  p.epoch = a->epoch;
  if (a->phases < 0 || a->phases > 3) return DG_ERR_BAD_ARGUMENT;
  p.phases = a->phases == 0 ? 3 : a->phases;
  p.my_base = a->my_base;
  p.cursor = a->cursor;
  p.m_indices = a->m_indices;
  p.m_total = a->m_total;
  p.status = a->status;
  dg::ep_plan_kernel<<<1, dg::kEpPlanThreads, 3 * a->num_experts * sizeof(int32_t),
                       static_cast<cudaStream_t>(stream)>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e);
  g_launch_count.fetch_add(1, std::memory_order_relaxed);
  return DG_OK;
}

int dg_ep_push(const dg_ep_push_args* a, void* stream) {
  if (a == nullptr) return DG_ERR_NULL_POINTER;
  if (a->world < 1 || a->world > DG_EP_MAX_WORLD || a->rank < 0 || a->rank >= a->world)
    return DG_ERR_BAD_ARGUMENT;
  if (a->num_experts < a->world || a->num_experts % a->world != 0 || a->num_tokens < 0 || a->top_k < 1 ||
      a->top_k > dg::kEpMaxTopK || a->row_bytes < 16 || a->row_bytes % 16 != 0 || a->m_cap < 1)
    return DG_ERR_BAD_SHAPE;
  if (a->row_bytes > 16 * dg::kEpPushThreads * dg::kEpMaxChunksPerThread || a->num_experts > DG_MAX_GROUPS ||
      (long long)a->num_tokens * a->top_k >= (1 << 24))
    return DG_ERR_TOO_LARGE;
  if (a->quantise < 0 || a->quantise > DG_EP_QUANT_I8) return DG_ERR_BAD_ARGUMENT;
  if (a->quantise != 0 && (a->row_bytes % 8 != 0 || a->row_bytes > 8 * dg::kEpPushThreads * dg::kEpMaxVec))
    return DG_ERR_BAD_SHAPE;
  if (a->num_tokens == 0) return DG_OK;
  if (!a->rows || (!a->row_scale && a->quantise == 0) || !a->topk_ids || !a->my_base || !a->cursor)
    return DG_ERR_NULL_POINTER;
  if (!aligned16(a->rows)) return DG_ERR_BAD_ALIGNMENT;
  const DeviceInfo* dev = nullptr;
  int rc = device_info(&dev);
  if (rc != DG_OK) return rc;
  dg::EpPushParams p{};
  rc = ep_copy_peers(&p.peer_a, a->peer_a, a->world);
  if (rc == DG_OK) rc = ep_copy_peers(&p.peer_scale, a->peer_scale, a->world);
  if (rc == DG_OK) rc = ep_copy_peers(&p.peer_tag, a->peer_tag, a->world);
  if (rc != DG_OK) return rc;
  for (int r = 0; r < a->world; ++r)
    if (!aligned16(a->peer_a[r])) return DG_ERR_BAD_ALIGNMENT;
  p.rows = static_cast<const uint8_t*>(a->rows);
  p.row_scale = a->row_scale;
  p.topk_ids = a->topk_ids;
  p.T = a->num_tokens;
  p.top_k = a->top_k;
  p.row_bytes = a->row_bytes;
  p.E = a->num_experts;
  p.e_local = a->num_experts / a->world;
  p.me = a->rank;
  p.m_cap = a->m_cap;
  p.my_base = a->my_base;
  p.cursor = a->cursor;
  p.pair_dest = a->pair_dest;
  p.status = a->status;
  if (a->local_lo < 0 || a->local_hi < 0 || (a->local_hi > 0 && a->local_lo >= a->local_hi)) return DG_ERR_BAD_ARGUMENT;
  p.local_lo = a->local_lo;
  p.local_hi = a->local_hi > 0 ? a->local_hi : p.e_local;
  if (a->max_blocks < 0) return DG_ERR_BAD_ARGUMENT;
  const int max_blocks = (a->max_blocks > 0 && a->max_blocks < dev->sm_count * 8) ? a->max_blocks : dev->sm_count * 8;
  const int grid = a->num_tokens < max_blocks ? a->num_tokens : max_blocks;
  if (a->quantise == DG_EP_QUANT_E4M3)
    dg::ep_push_quant_kernel<DG_KIND_E4M3><<<grid, dg::kEpPushThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  else if (a->quantise == DG_EP_QUANT_I8)
    dg::ep_push_quant_kernel<DG_KIND_I8><<<grid, dg::kEpPushThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  else
    dg::ep_push_kernel<<<grid, dg::kEpPushThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e);
  g_launch_count.fetch_add(1, std::memory_order_relaxed);
  return DG_OK;
}

int dg_ep_barrier(const dg_ep_barrier_args* a, void* stream) {
  if (a == nullptr) return DG_ERR_NULL_POINTER;
  if (a->world < 1 || a->world > DG_EP_MAX_WORLD || a->rank < 0 || a->rank >= a->world)
    return DG_ERR_BAD_ARGUMENT;
  dg::EpBarrierParams p{};
  int rc = ep_copy_peers(&p.peer_flags, a->peer_flags, a->world);
  if (rc != DG_OK) return rc;
  p.flags = static_cast<int32_t*>(p.peer_flags.ptr[a->rank]);
  p.world = a->world;
  p.me = a->rank;
  p.epoch = a->epoch;
  if (a->phases < 0 || a->phases > 3) return DG_ERR_BAD_ARGUMENT;
  p.phases = a->phases == 0 ? 3 : a->phases;
  p.status = a->status;
  dg::ep_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e);
  g_launch_count.fetch_add(1, std::memory_order_relaxed);
  return DG_OK;
}

int64_t dg_query(int32_t what) {
  if (what == DG_QUERY_ABI_VERSION) return DG_ABI_VERSION;
  if (what == DG_QUERY_LAUNCH_COUNT) return g_launch_count.load(std::memory_order_relaxed);
  if (what == DG_QUERY_MAP_ENCODES) return static_cast<int64_t>(g_map_misses.load(std::memory_order_relaxed));
  if (what == DG_QUERY_MAP_REUSES) return static_cast<int64_t>(g_map_hits.load(std::memory_order_relaxed));
  const DeviceInfo* dev = nullptr;
  int rc = device_info(&dev);
  if (what == DG_QUERY_CC && dev != nullptr && dev->cc > 0) return dev->cc;
  if (rc != DG_OK) return rc;
  switch (what) {
    case DG_QUERY_SM_COUNT: return dev->sm_count;
    case DG_QUERY_MAX_SMEM: return dev->max_smem;
    case DG_QUERY_CC: return dev->cc;
    default: return DG_ERR_BAD_ARGUMENT;
  }
}

const char* dg_strerror(int code) {
  switch (code) {
    case DG_OK: return "ok";
    case DG_ERR_NULL_POINTER: return "a required pointer is NULL";
    case DG_ERR_BAD_KIND: return "unknown operand kind";
    case DG_ERR_BAD_SHAPE:
      return "bad shape: need N % 16 == 0, K % 64 == 0 (K % 256 for W4A8), groups >= 1";
    case DG_ERR_BAD_ALIGNMENT: return "a base pointer is not 16-byte aligned";
    case DG_ERR_BAD_SCALE_MODE: return "scale mode does not fit the operand kind";
    case DG_ERR_NO_DEVICE: return "no current CUDA device of compute capability 10.x (B200)";
    case DG_ERR_CUDA: return "a CUDA call failed (see dg_last_cuda_error)";
    case DG_ERR_TOO_LARGE: return "a size exceeds the library maximum";
    case DG_ERR_BAD_ARGUMENT: return "bad argument value";
    default: return "unknown status code";
  }
}

int dg_last_cuda_error(void) { return tl_last_cuda_error; }

}  // extern "C"
