// Host fast path between torch tensors and the C ABI of libdeepgemm_b200.so.
//
// The reference binds its launchers to Python from C++ (csrc/common/deepgemm_ops.cpp:127-144), so
// a call costs a pybind argument conversion and the TORCH_CHECKs.  The Python marshalling in
// deepgemm/_core.py does the same checks with tensor attribute reads, about 7 us a call; for a
// sparse decode step that is half of what the kernel takes.  This module does them natively.
//
// It is deliberately only the accepting half: each function returns true when the arguments
// passed every check and the launch was enqueued, false when anything at all is unusual (a
// check failed, a layout this file does not know, a device that is not current, a launch error).
// On false nothing was enqueued and the caller runs the Python marshalling, which either raises
// the error with its full message or handles the unusual case.  No message text lives here.
//
// It is not part of the C ABI boundary (include/deepgemm_b200.h has no torch types); it is a
// client of it, like the ctypes marshalling.
#include <c10/cuda/CUDAFunctions.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/extension.h>

#include <array>

#include "deepgemm_b200.h"

namespace {

using at::Tensor;
using OptTensor = c10::optional<Tensor>;

constexpr int kMaxDevices = 64;
std::array<Tensor, kMaxDevices> g_status;  // int32[DG_STATUS_WORDS] per device, registered from Python
int64_t g_accepted = 0, g_declined = 0;     // calls enqueued here / handed back (under the GIL)

inline bool on(const Tensor& t, int dev) { return t.is_cuda() && t.get_device() == dev && t.is_contiguous(); }

// activation / weight / output element types per kind (deepgemm/_core.py: _A_DTYPES, _B_DTYPES)
inline bool a_dtype_ok(int kind, at::ScalarType t) {
  switch (kind) {
    case DG_KIND_I8: case DG_KIND_W4A8: return t == at::kChar;
    case DG_KIND_E4M3: return t == at::kFloat8_e4m3fn;
    case DG_KIND_BF16: return t == at::kBFloat16;
  }
  return false;
}
inline bool b_dtype_ok(int kind, at::ScalarType t) {
  switch (kind) {
    case DG_KIND_I8: case DG_KIND_W4A8: return t == at::kChar || t == at::kByte;
    case DG_KIND_E4M3: return t == at::kFloat8_e4m3fn || t == at::kChar || t == at::kByte;
    case DG_KIND_BF16: return t == at::kBFloat16;
  }
  return false;
}
// the packed weight of an INT8 / FP8 problem with K % 128 == 64 carries one zero-padded block more
inline bool k_matches(int kind, int64_t packed_k, int64_t k) {
  return packed_k == k || ((kind == DG_KIND_I8 || kind == DG_KIND_E4M3) && k % 128 == 64 && packed_k == k + 64);
}
inline bool d_dtype_ok(int kind, at::ScalarType t) {
  return t == at::kBFloat16 || (kind == DG_KIND_W4A8 && t == at::kHalf);
}

// 4-D packed weight [G, K / block, N, row]; the 3-D W4A8 form needs the Python side's registry
inline bool weight_dims(const Tensor& b, int kind, int64_t* g, int64_t* n, int64_t* k) {
  if (b.dim() != 4) return false;
  const int64_t row = (kind == DG_KIND_BF16) ? 64 : 128;
  const int64_t k_per_block = (kind == DG_KIND_BF16) ? 64 : (kind == DG_KIND_W4A8 ? 256 : 128);
  if (b.size(3) != row) return false;
  *g = b.size(0);
  *n = b.size(2);
  *k = b.size(1) * k_per_block;
  return true;
}

// fp32, contiguous, 16-byte aligned, shape (s0[, s1]) optionally followed by a 1
inline const float* scale_ptr(const OptTensor& t, int dev, int64_t s0, int64_t s1) {
  if (!t.has_value()) return nullptr;
  const Tensor& x = *t;
  if (!on(x, dev) || x.scalar_type() != at::kFloat) return nullptr;
  const int64_t want = s1 < 0 ? 1 : 2;
  const int64_t nd = x.dim();
  if (!(nd == want || (nd == want + 1 && x.size(nd - 1) == 1))) return nullptr;
  if (x.size(0) != s0 || (s1 >= 0 && x.size(1) != s1)) return nullptr;
  const float* p = x.data_ptr<float>();
  return (reinterpret_cast<uintptr_t>(p) % 16 == 0) ? p : nullptr;
}

inline int32_t* status_ptr(const OptTensor& status, int dev) {
  const Tensor& s = status.has_value() ? *status : g_status[dev];
  if (!s.defined() || !on(s, dev) || s.scalar_type() != at::kInt || s.numel() < DG_STATUS_WORDS) return nullptr;
  return s.data_ptr<int32_t>();
}

bool masked_impl(int64_t kind, int64_t scale_mode, const Tensor& a, const Tensor& b, const Tensor& d,
            const OptTensor& a_scale, const OptTensor& b_scale, const Tensor& masked_m, int64_t expected_m,
            int64_t block_n, const OptTensor& status, const OptTensor& signal) {
  if (!a.is_cuda()) return false;
  const int dev = static_cast<int>(a.get_device());
  if (dev < 0 || dev >= kMaxDevices || dev != c10::cuda::current_device()) return false;
  if (a.dim() != 3 || d.dim() != 3) return false;
  if (!on(a, dev) || !on(b, dev) || !on(d, dev) || !on(masked_m, dev)) return false;
  const int ki = static_cast<int>(kind);
  if (!a_dtype_ok(ki, a.scalar_type()) || !b_dtype_ok(ki, b.scalar_type()) || !d_dtype_ok(ki, d.scalar_type()))
    return false;
  if (masked_m.scalar_type() != at::kInt) return false;
  int64_t bg, n, bk;
  if (!weight_dims(b, ki, &bg, &n, &bk)) return false;
  const int64_t g = a.size(0), max_m = a.size(1), k = a.size(2);
  if (bg != g || !k_matches(ki, bk, k) || d.size(0) != g || d.size(1) != max_m || d.size(2) != n || masked_m.numel() != g)
    return false;
  if (g > INT32_MAX || max_m > INT32_MAX || n > INT32_MAX || k > INT32_MAX) return false;

  dg_masked_args args{};
  args.kind = ki;
  args.scale_mode = static_cast<int32_t>(scale_mode);
  if (scale_mode != DG_SCALE_NONE) {
    args.a_scale = scale_ptr(a_scale, dev, g, max_m);
    args.b_scale = scale_ptr(b_scale, dev, g, scale_mode == DG_SCALE_PER_CHANNEL ? n : -1);
    if (args.a_scale == nullptr || args.b_scale == nullptr) return false;
  }
  args.status = status_ptr(status, dev);
  if (args.status == nullptr) return false;
  if (signal.has_value()) {
    const Tensor& s = *signal;
    if (!on(s, dev) || s.scalar_type() != at::kInt || s.numel() != g * ((max_m + 127) / 128)) return false;
    if (ki == DG_KIND_W4A8 || n % 32 != 0) return false;
    args.signal = s.data_ptr<int32_t>();
  }
  args.a = a.data_ptr();
  args.b_packed = b.data_ptr();
  args.d = d.data_ptr();
  args.masked_m = masked_m.data_ptr<int32_t>();
  args.num_groups = static_cast<int32_t>(g);
  args.max_m = static_cast<int32_t>(max_m);
  args.n = static_cast<int32_t>(n);
  args.k = static_cast<int32_t>(k);
  args.expected_m = static_cast<int32_t>(expected_m);
  args.block_n = static_cast<int32_t>(block_n);
  args.out_kind = d.scalar_type() == at::kHalf ? DG_OUT_F16 : DG_OUT_BF16;
  return dg_masked_gemm(&args, c10::cuda::getCurrentCUDAStream(dev).stream()) == DG_OK;
}

bool contiguous_impl(int64_t kind, int64_t scale_mode, const Tensor& a, const Tensor& b, const Tensor& d,
                const OptTensor& a_scale, const OptTensor& b_scale, const Tensor& m_indices, int64_t block_n,
                const OptTensor& status) {
  if (!a.is_cuda()) return false;
  const int dev = static_cast<int>(a.get_device());
  if (dev < 0 || dev >= kMaxDevices || dev != c10::cuda::current_device()) return false;
  if (a.dim() != 2 || d.dim() != 2) return false;
  if (!on(a, dev) || !on(b, dev) || !on(d, dev) || !on(m_indices, dev)) return false;
  const int ki = static_cast<int>(kind);
  if (!a_dtype_ok(ki, a.scalar_type()) || !b_dtype_ok(ki, b.scalar_type()) || !d_dtype_ok(ki, d.scalar_type()))
    return false;
  if (m_indices.scalar_type() != at::kInt) return false;
  int64_t g, n, bk;
  if (!weight_dims(b, ki, &g, &n, &bk)) return false;
  const int64_t m_total = a.size(0), k = a.size(1);
  if (!k_matches(ki, bk, k) || d.size(0) != m_total || d.size(1) != n || m_indices.numel() != m_total) return false;
  if (g > INT32_MAX || m_total > INT32_MAX || n > INT32_MAX || k > INT32_MAX) return false;

  dg_contig_args args{};
  args.kind = ki;
  args.scale_mode = static_cast<int32_t>(scale_mode);
  if (scale_mode != DG_SCALE_NONE) {
    args.a_scale = scale_ptr(a_scale, dev, m_total, -1);
    args.b_scale = scale_ptr(b_scale, dev, g, scale_mode == DG_SCALE_PER_CHANNEL ? n : -1);
    if (args.a_scale == nullptr || args.b_scale == nullptr) return false;
  }
  args.status = status_ptr(status, dev);
  if (args.status == nullptr) return false;
  args.a = a.data_ptr();
  args.b_packed = b.data_ptr();
  args.d = d.data_ptr();
  args.m_indices = m_indices.data_ptr<int32_t>();
  args.num_groups = static_cast<int32_t>(g);
  args.m_total = static_cast<int32_t>(m_total);
  args.n = static_cast<int32_t>(n);
  args.k = static_cast<int32_t>(k);
  args.block_n = static_cast<int32_t>(block_n);
  args.out_kind = d.scalar_type() == at::kHalf ? DG_OUT_F16 : DG_OUT_BF16;
  return dg_contig_gemm(&args, c10::cuda::getCurrentCUDAStream(dev).stream()) == DG_OK;
}

inline bool count(bool ok) {
  ++(ok ? g_accepted : g_declined);
  return ok;
}

bool masked(int64_t kind, int64_t scale_mode, const Tensor& a, const Tensor& b, const Tensor& d,
            const OptTensor& a_scale, const OptTensor& b_scale, const Tensor& masked_m, int64_t expected_m,
            int64_t block_n, const OptTensor& status, const OptTensor& signal) {
  return count(masked_impl(kind, scale_mode, a, b, d, a_scale, b_scale, masked_m, expected_m, block_n, status, signal));
}

bool contiguous(int64_t kind, int64_t scale_mode, const Tensor& a, const Tensor& b, const Tensor& d,
                const OptTensor& a_scale, const OptTensor& b_scale, const Tensor& m_indices, int64_t block_n,
                const OptTensor& status) {
  return count(contiguous_impl(kind, scale_mode, a, b, d, a_scale, b_scale, m_indices, block_n, status));
}

void set_status_words(int64_t device, const Tensor& words) {
  TORCH_CHECK(device >= 0 && device < kMaxDevices, "device index out of range");
  TORCH_CHECK(words.is_cuda() && words.get_device() == device && words.scalar_type() == at::kInt &&
                  words.is_contiguous() && words.numel() >= DG_STATUS_WORDS,
              "status words must be a contiguous int32 CUDA tensor on that device");
  g_status[device] = words;
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "native argument checks and launch for the grouped GEMM entry points (accepting half only)";
  m.def("masked", &masked, "enqueue dg_masked_gemm if every check passes; False otherwise");
  m.def("contiguous", &contiguous, "enqueue dg_contig_gemm if every check passes; False otherwise");
  m.def("set_status_words", &set_status_words);
  m.def("stats", []() { return std::make_pair(g_accepted, g_declined); }, "(calls enqueued here, calls handed back)");
  // the header this file was compiled against; the caller compares it with the library's own
  m.def("abi_version", []() { return static_cast<int64_t>(DG_ABI_VERSION); });
}
