"""ctypes binding of libdeepgemm_b200.so (declared in include/deepgemm_b200.h).

The library is the only compute path: there is no CPU or PyTorch fallback.  Importing this
module raises ImportError when the shared object has not been built.
"""
from __future__ import annotations

import ctypes as C
import os

_LIB_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib")
LIB_PATH = os.environ.get("DEEP_GEMM_LIB_PATH") or os.path.join(_LIB_DIR, "libdeepgemm_b200.so")

# enum dg_kind / dg_scale_mode
KIND_I8, KIND_E4M3, KIND_W4A8, KIND_BF16 = 0, 1, 2, 3
SCALE_PER_CHANNEL, SCALE_TENSOR_WISE, SCALE_NONE = 0, 1, 2
NIBBLE_HIGH_FIRST, NIBBLE_LOW_FIRST = 0, 1
STATUS_WORDS = 4
OUT_BF16, OUT_F16, OUT_F32 = 0, 1, 2
NOALLOC_MAX_SCRATCH_INTS = 262144 + 1024
QUERY_ABI_VERSION, QUERY_SM_COUNT, QUERY_MAX_SMEM, QUERY_CC, QUERY_LAUNCH_COUNT = 0, 1, 2, 3, 4
QUERY_MAP_ENCODES, QUERY_MAP_REUSES = 5, 6
ERR_CUDA = -7

EXPORTED_SYMBOLS = (
    "dg_masked_gemm",
    "dg_contig_gemm",
    "dg_compact_gemm",
    "dg_sorted_gemm",
    "dg_dense_gemm",
    "dg_quant_group_rows",
    "dg_quant_group_scratch_bytes",
    "dg_quant_group_rows_noalloc",
    "dg_group_sorted_rows",
    "dg_silu_mul_quant_rows",
    "dg_combine_rows",
    "dg_ep_plan",
    "dg_ep_push",
    "dg_ep_barrier",
    "dg_pack_weight",
    "dg_unpack_weight",
    "dg_query",
    "dg_strerror",
    "dg_last_cuda_error",
)


class MaskedArgs(C.Structure):
    _fields_ = [
        ("kind", C.c_int32),
        ("scale_mode", C.c_int32),
        ("a", C.c_void_p),
        ("b_packed", C.c_void_p),
        ("d", C.c_void_p),
        ("a_scale", C.c_void_p),
        ("b_scale", C.c_void_p),
        ("masked_m", C.c_void_p),
        ("num_groups", C.c_int32),
        ("max_m", C.c_int32),
        ("n", C.c_int32),
        ("k", C.c_int32),
        ("expected_m", C.c_int32),
        ("block_n", C.c_int32),
        ("debug_acc", C.c_void_p),
        ("status", C.c_void_p),
        ("out_kind", C.c_int32),
        ("reserved", C.c_int32),
        ("signal", C.c_void_p),
    ]


class ContigArgs(C.Structure):
    _fields_ = [
        ("kind", C.c_int32),
        ("scale_mode", C.c_int32),
        ("a", C.c_void_p),
        ("b_packed", C.c_void_p),
        ("d", C.c_void_p),
        ("a_scale", C.c_void_p),
        ("b_scale", C.c_void_p),
        ("m_indices", C.c_void_p),
        ("num_groups", C.c_int32),
        ("m_total", C.c_int32),
        ("n", C.c_int32),
        ("k", C.c_int32),
        ("block_n", C.c_int32),
        ("out_kind", C.c_int32),
        ("debug_acc", C.c_void_p),
        ("status", C.c_void_p),
        ("scatter_tag", C.c_void_p),
        ("scatter_base", C.POINTER(C.c_void_p)),
        ("scatter_world", C.c_int32),
        ("group_window", C.c_int32),
    ]


class CompactArgs(C.Structure):
    _fields_ = [
        ("kind", C.c_int32),
        ("scale_mode", C.c_int32),
        ("a", C.c_void_p),
        ("b_packed", C.c_void_p),
        ("d", C.c_void_p),
        ("a_scale", C.c_void_p),
        ("b_scale", C.c_void_p),
        ("counts", C.c_void_p),
        ("offsets", C.c_void_p),
        ("num_groups", C.c_int32),
        ("capacity", C.c_int32),
        ("n", C.c_int32),
        ("k", C.c_int32),
        ("expected_m", C.c_int32),
        ("block_n", C.c_int32),
        ("debug_acc", C.c_void_p),
        ("status", C.c_void_p),
    ]


class SortedGemmArgs(C.Structure):
    _fields_ = [
        ("kind", C.c_int32),
        ("num_groups", C.c_int32),
        ("a", C.c_void_p),
        ("b_packed", C.c_void_p),
        ("d", C.c_void_p),
        ("a_scale", C.c_void_p),
        ("row_weight", C.c_void_p),
        ("b_scale", C.c_void_p),
        ("sorted_token_ids", C.c_void_p),
        ("expert_ids", C.c_void_p),
        ("num_tokens_post_pad", C.c_void_p),
        ("num_sorted", C.c_int32),
        ("num_blocks", C.c_int32),
        ("block_m", C.c_int32),
        ("size_m", C.c_int32),
        ("real_topk", C.c_int32),
        ("n", C.c_int32),
        ("k", C.c_int32),
        ("reserved", C.c_int32),
        ("status", C.c_void_p),
    ]


class QuantGroupArgs(C.Structure):
    _fields_ = [
        ("kind", C.c_int32),
        ("num_rows", C.c_int32),
        ("hidden", C.c_int32),
        ("num_groups", C.c_int32),
        ("align", C.c_int32),
        ("m_cap", C.c_int32),
        ("rows", C.c_void_p),
        ("expert", C.c_void_p),
        ("a_out", C.c_void_p),
        ("a_scale_out", C.c_void_p),
        ("m_indices_out", C.c_void_p),
        ("dest_out", C.c_void_p),
        ("m_total_out", C.c_void_p),
        ("scratch", C.c_void_p),
        ("scratch_bytes", C.c_size_t),
        ("src_index", C.c_void_p),
        ("row_scale", C.c_void_p),
    ]


class DenseArgs(C.Structure):
    _fields_ = [
        ("kind", C.c_int32),
        ("out_kind", C.c_int32),
        ("a", C.c_void_p),
        ("b", C.c_void_p),
        ("d", C.c_void_p),
        ("a_scale", C.c_void_p),
        ("b_scale", C.c_void_p),
        ("batch", C.c_int32),
        ("m", C.c_int32),
        ("n", C.c_int32),
        ("k", C.c_int32),
        ("block_n", C.c_int32),
        ("reserved", C.c_int32),
        ("debug_acc", C.c_void_p),
        ("status", C.c_void_p),
    ]


class GroupSortedArgs(C.Structure):
    _fields_ = [
        ("num_sorted", C.c_int32),
        ("block_m", C.c_int32),
        ("size_m", C.c_int32),
        ("hidden", C.c_int32),
        ("num_groups", C.c_int32),
        ("align", C.c_int32),
        ("m_cap", C.c_int32),
        ("real_topk", C.c_int32),
        ("rows", C.c_void_p),
        ("row_scale", C.c_void_p),
        ("row_weight", C.c_void_p),
        ("sorted_token_ids", C.c_void_p),
        ("expert_ids", C.c_void_p),
        ("num_tokens_post_pad", C.c_void_p),
        ("a_out", C.c_void_p),
        ("a_scale_out", C.c_void_p),
        ("m_indices_out", C.c_void_p),
        ("dest_out", C.c_void_p),
        ("m_total_out", C.c_void_p),
        ("scratch", C.c_void_p),
        ("scratch_bytes", C.c_size_t),
        ("src_out", C.c_void_p),
        ("zero_rows", C.c_void_p),
        ("zero_row_bytes", C.c_int32),
        ("reserved", C.c_int32),
    ]


class ActQuantArgs(C.Structure):
    _fields_ = [
        ("kind", C.c_int32),
        ("num_rows", C.c_int32),
        ("hidden", C.c_int32),
        ("max_m", C.c_int32),
        ("x", C.c_void_p),
        ("m_indices", C.c_void_p),
        ("masked_m", C.c_void_p),
        ("q_out", C.c_void_p),
        ("scale_out", C.c_void_p),
    ]


class CombineArgs(C.Structure):
    _fields_ = [
        ("num_tokens", C.c_int32),
        ("top_k", C.c_int32),
        ("n", C.c_int32),
        ("num_rows", C.c_int32),
        ("y", C.c_void_p),
        ("src_row", C.c_void_p),
        ("weights", C.c_void_p),
        ("out", C.c_void_p),
    ]


EP_MAX_WORLD = 16
EP_PHASE_POST, EP_PHASE_WAIT = 1, 2
EP_QUANT_NONE, EP_QUANT_E4M3, EP_QUANT_I8 = 0, 1, 2


class EpPlanArgs(C.Structure):
    _fields_ = [
        ("world", C.c_int32),
        ("rank", C.c_int32),
        ("num_experts", C.c_int32),
        ("num_pairs", C.c_int32),
        ("align", C.c_int32),
        ("m_cap", C.c_int32),
        ("epoch", C.c_int32),
        ("phases", C.c_int32),
        ("topk_ids", C.c_void_p),
        ("peer_counts", C.POINTER(C.c_void_p)),
        ("peer_flags", C.POINTER(C.c_void_p)),
        ("my_base", C.c_void_p),
        ("cursor", C.c_void_p),
        ("m_indices", C.c_void_p),
        ("m_total", C.c_void_p),
        ("status", C.c_void_p),
    ]


class EpPushArgs(C.Structure):
    _fields_ = [
        ("world", C.c_int32),
        ("rank", C.c_int32),
        ("num_experts", C.c_int32),
        ("num_tokens", C.c_int32),
        ("top_k", C.c_int32),
        ("row_bytes", C.c_int32),
        ("m_cap", C.c_int32),
        ("quantise", C.c_int32),
        ("rows", C.c_void_p),
        ("row_scale", C.c_void_p),
        ("topk_ids", C.c_void_p),
        ("my_base", C.c_void_p),
        ("cursor", C.c_void_p),
        ("peer_a", C.POINTER(C.c_void_p)),
        ("peer_scale", C.POINTER(C.c_void_p)),
        ("peer_tag", C.POINTER(C.c_void_p)),
        ("pair_dest", C.c_void_p),
        ("status", C.c_void_p),
        ("local_lo", C.c_int32),
        ("local_hi", C.c_int32),
        ("max_blocks", C.c_int32),
        ("reserved", C.c_int32),
    ]


class EpBarrierArgs(C.Structure):
    _fields_ = [
        ("world", C.c_int32),
        ("rank", C.c_int32),
        ("epoch", C.c_int32),
        ("phases", C.c_int32),
        ("peer_flags", C.POINTER(C.c_void_p)),
        ("status", C.c_void_p),
    ]


def pointer_array(ptrs):
    """ctypes array of device pointers (a HOST array, as the dg_ep_* calls take)."""
    return (C.c_void_p * len(ptrs))(*[int(x) for x in ptrs])


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"libdeepgemm_b200.so not found at {LIB_PATH}. Build it with "
            "`python deepgemm-das_b200/build.py` (needs nvcc with sm_100a support). "
            "There is no fallback implementation."
        )
    lib = C.CDLL(LIB_PATH)
    lib.dg_masked_gemm.argtypes = [C.POINTER(MaskedArgs), C.c_void_p]
    lib.dg_masked_gemm.restype = C.c_int
    lib.dg_contig_gemm.argtypes = [C.POINTER(ContigArgs), C.c_void_p]
    lib.dg_contig_gemm.restype = C.c_int
    lib.dg_compact_gemm.argtypes = [C.POINTER(CompactArgs), C.c_void_p]
    lib.dg_compact_gemm.restype = C.c_int
    for fn in (lib.dg_pack_weight, lib.dg_unpack_weight):
        fn.argtypes = [C.c_int32, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32,
                       C.c_int32, C.c_void_p]
        fn.restype = C.c_int
    lib.dg_quant_group_rows.argtypes = [C.POINTER(QuantGroupArgs), C.c_void_p]
    lib.dg_quant_group_rows.restype = C.c_int
    lib.dg_quant_group_rows_noalloc.argtypes = [C.POINTER(QuantGroupArgs), C.c_void_p]
    lib.dg_quant_group_rows_noalloc.restype = C.c_int
    lib.dg_quant_group_scratch_bytes.argtypes = [C.c_int32, C.c_int32]
    lib.dg_quant_group_scratch_bytes.restype = C.c_size_t
    lib.dg_sorted_gemm.argtypes = [C.POINTER(SortedGemmArgs), C.c_void_p]
    lib.dg_sorted_gemm.restype = C.c_int
    lib.dg_dense_gemm.argtypes = [C.POINTER(DenseArgs), C.c_void_p]
    lib.dg_dense_gemm.restype = C.c_int
    lib.dg_group_sorted_rows.argtypes = [C.POINTER(GroupSortedArgs), C.c_void_p]
    lib.dg_group_sorted_rows.restype = C.c_int
    lib.dg_silu_mul_quant_rows.argtypes = [C.POINTER(ActQuantArgs), C.c_void_p]
    lib.dg_silu_mul_quant_rows.restype = C.c_int
    lib.dg_combine_rows.argtypes = [C.POINTER(CombineArgs), C.c_void_p]
    lib.dg_combine_rows.restype = C.c_int
    lib.dg_ep_plan.argtypes = [C.POINTER(EpPlanArgs), C.c_void_p]
    lib.dg_ep_plan.restype = C.c_int
    lib.dg_ep_push.argtypes = [C.POINTER(EpPushArgs), C.c_void_p]
    lib.dg_ep_push.restype = C.c_int
    lib.dg_ep_barrier.argtypes = [C.POINTER(EpBarrierArgs), C.c_void_p]
    lib.dg_ep_barrier.restype = C.c_int
    lib.dg_query.argtypes = [C.c_int32]
    lib.dg_query.restype = C.c_int64
    lib.dg_strerror.argtypes = [C.c_int]
    lib.dg_strerror.restype = C.c_char_p
    lib.dg_last_cuda_error.argtypes = []
    lib.dg_last_cuda_error.restype = C.c_int
    return lib


lib = _load()


class DeepGemmError(RuntimeError):
    """A non-zero dg_status from the library (RuntimeError, like the reference's TORCH_CHECK)."""

    def __init__(self, code: int, where: str):
        self.code = code
        msg = lib.dg_strerror(code).decode()
        if code == ERR_CUDA:
            msg += f" [cuda error {lib.dg_last_cuda_error()}]"
        super().__init__(f"{where}: {msg} (dg_status {code})")


def check(code: int, where: str) -> None:
    if code != 0:
        raise DeepGemmError(code, where)


def query(what: int) -> int:
    return int(lib.dg_query(what))
