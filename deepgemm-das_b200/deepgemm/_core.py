"""Tensor-level marshalling from torch tensors to the C ABI.

Every public grouped-GEMM entry point of the package ends here (through the
``torch.ops.deep_gemm.*`` custom ops of ``deepgemm.op``).  Checks mirror the reference's
host-side TORCH_CHECKs (csrc/arch/gfx936_gfx938_shared/m_grouped_fp8_gemm_nt_maksed_low_latency.cu:1053-1126,
csrc/include/m_grouped_i8_gemm_nt_contiguous/bm128_bn256_bk64_nloop4.inc.cuh:729-791) and
raise RuntimeError like they do; nothing here computes on the CPU.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional, Tuple

import torch

from . import _cabi
from ._cabi import (KIND_BF16, KIND_E4M3, KIND_I8, KIND_W4A8, SCALE_NONE, SCALE_PER_CHANNEL,
                    SCALE_TENSOR_WISE)

try:                                   # native argument checks + launch (csrc/dg_torch_glue.cpp)
    from . import _glue
    if _glue.abi_version() != _cabi.query(_cabi.QUERY_ABI_VERSION):
        _glue = None                   # built against another header: the ctypes path below still works
except ImportError:
    _glue = None
if os.environ.get("DEEPGEMM_NO_GLUE"):
    _glue = None

_FP8 = torch.float8_e4m3fn
# (device type, index, data pointer) of every [E, N, K/2] int4 tensor a packer of this package has
# put into the kernel layout: that shape is shared with the unpacked framework layout
PACKED_W4A8_STORAGES = set()

# bytes of K per packed row, and elements per row, by kind
_ROW_ELEMS = {KIND_I8: 128, KIND_E4M3: 128, KIND_BF16: 64, KIND_W4A8: 128}
_K_PER_BLOCK = {KIND_I8: 128, KIND_E4M3: 128, KIND_BF16: 64, KIND_W4A8: 256}
_A_DTYPES = {KIND_I8: (torch.int8,), KIND_E4M3: (_FP8,), KIND_W4A8: (torch.int8,),
             KIND_BF16: (torch.bfloat16,)}
_B_DTYPES = {KIND_I8: (torch.int8, torch.uint8), KIND_E4M3: (_FP8, torch.int8, torch.uint8),
             KIND_W4A8: (torch.int8, torch.uint8), KIND_BF16: (torch.bfloat16,)}
KIND_NAMES = {KIND_I8: "int8", KIND_E4M3: "fp8_e4m3", KIND_W4A8: "w4a8", KIND_BF16: "bf16"}


def packed_weight_dims(b: torch.Tensor, kind: int, k_hint: Optional[int] = None
                       ) -> Tuple[int, int, int]:
    """(G, N, K) of a packed weight tensor; rejects tensors that do not carry the packed shape.

    Packed weights are 4-D ``[G, K/BK, N, row]`` with row = 128 (8-bit elements, or int4 bytes
    holding 256 values) or 64 (bf16 elements).  W4A8 weights may also be the 3-D ``[G, N, K/2]`` tensor that the reference's
    in-place packer returns (deepgemm/group_gemm_weight_pack.py:691-714); since that shape is also
    the unpacked one, such a tensor is accepted only if a packer of this package marked its storage.
    """
    if kind == KIND_W4A8 and b.dim() == 3:
        if (b.device.type, b.device.index, b.data_ptr()) not in PACKED_W4A8_STORAGES \
                and not os.environ.get("DEEPGEMM_TRUST_W4A8_LAYOUT"):
            raise ValueError(
                "w4a8 grouped GEMM: this [E, N, K/2] weight has not been through pack_w4a8_moe_hipc_weight "
                "(the framework layout would be silently mis-read); pack it, or mark a weight packed "
                "elsewhere with group_gemm_weight_pack.register_packed_w4a8_weight")
        g, n, kh = b.shape
        return int(g), int(n), int(kh) * 2
    if b.dim() != 4 or int(b.shape[3]) != _ROW_ELEMS[kind]:
        raise ValueError(
            f"{KIND_NAMES[kind]} grouped GEMM expects a packed weight [G, K/{_K_PER_BLOCK[kind]}, N, "
            f"{_ROW_ELEMS[kind]}] from the deepgemm.group_gemm_weight_pack packers, got shape "
            f"{tuple(b.shape)}"
        )
    g, kb, n, _ = b.shape
    return int(g), int(n), int(kb) * _K_PER_BLOCK[kind]


def _k_matches(kind: int, packed_k: int, k: int) -> bool:
    """The packed weight of an INT8 / FP8 problem whose K is an odd multiple of 64 carries one
    more, zero-padded, half block (the kernels step K in 128-byte blocks)."""
    return packed_k == k or (kind in (KIND_I8, KIND_E4M3) and k % 128 == 64 and packed_k == k + 64)


def _common_checks(kind, a, b, d, sched, what):
    if not (a.is_cuda and b.is_cuda and d.is_cuda and sched.is_cuda):
        raise RuntimeError(f"{what}: all tensors must be CUDA tensors (there is no CPU implementation)")
    if not (a.device == b.device == d.device == sched.device):
        raise RuntimeError(f"{what}: tensors on different devices")
    if not (a.dtype in _A_DTYPES[kind]):
        raise RuntimeError(f"{what}: activation dtype {a.dtype} does not fit {KIND_NAMES[kind]}")
    if not (b.dtype in _B_DTYPES[kind]):
        raise RuntimeError(f"{what}: weight dtype {b.dtype} does not fit {KIND_NAMES[kind]}")
    if not (d.dtype == torch.bfloat16 or (kind == KIND_W4A8 and d.dtype == torch.float16)):
        # half outputs exist for the W4A8 ops only, as in the reference
        # (csrc/arch/gfx936_gfx938_shared/m_grouped_w4a8_gemm_nt_contiguous_hipc.cu:880,909)
        raise RuntimeError(f"{what}: output must be torch.bfloat16"
                           f"{' or torch.float16' if kind == KIND_W4A8 else ''}, got {d.dtype}")
    if not (a.is_contiguous()):
        raise RuntimeError(f"{what}: activation must be contiguous")
    if not (b.is_contiguous()):
        raise RuntimeError(f"{what}: packed weight must be contiguous")
    if not (d.is_contiguous()):
        raise RuntimeError(f"{what}: output must be contiguous")
    if not (sched.dtype == torch.int32 and sched.is_contiguous()):
        raise RuntimeError(f"{what}: masked_m / m_indices must be contiguous torch.int32")


def _scale(t: torch.Tensor, shape: Tuple[int, ...], name: str, what: str) -> torch.Tensor:
    if not (t.is_cuda):
        raise RuntimeError(f"{what}: {name} must be a CUDA tensor")
    if not (t.dtype == torch.float32):
        raise RuntimeError(f"{what}: {name} must be torch.float32, got {t.dtype}")
    if t.dim() == len(shape) + 1 and t.shape[-1] == 1:
        t = t.squeeze(-1)  # a view: same storage
    if not (tuple(t.shape) == tuple(shape)):
        raise RuntimeError(f"{what}: {name} must have shape {tuple(shape)} "
                       f"(optionally with a trailing 1), got {tuple(t.shape)}")
    # no copy is made on the caller's behalf: the ops allocate nothing
    if not t.is_contiguous():
        raise RuntimeError(f"{what}: {name} must be contiguous (got strides {tuple(t.stride())})")
    if t.data_ptr() % 16 != 0:  # a sliced view can be misaligned for the kernels' 16-byte loads
        raise RuntimeError(f"{what}: {name} must start on a 16-byte boundary")
    return t


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _launch(entry, args, device: torch.device, what: str) -> None:
    """Calls a C-ABI entry point on the current stream of `device`.  The common case (the
    tensors live on the current device) avoids the device context manager and the Stream
    object: together they cost more host time than the library call itself."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    if index == torch.cuda.current_device():
        stream = _raw_stream(index) if _raw_stream is not None else torch.cuda.current_stream(device).cuda_stream
        _cabi.check(entry(C.byref(args), C.c_void_p(stream)), what)
        return
    with torch.cuda.device(device):
        stream = torch.cuda.current_stream(device).cuda_stream
        _cabi.check(entry(C.byref(args), C.c_void_p(stream)), what)


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


# ---- device status words ------------------------------------------------------------------
# The kernels never trap.  A bounded wait that ran out, or an m_indices entry outside the group
# range, is recorded in four int32 words that the launch was given.  Callers of the public entry
# points pass none, so every launch gets the words of its device from here and the caller asks
# for them with check_device_status() whenever it synchronises anyway.
_status_words = {}
_STATUS_TEXT = {1: "a bounded wait inside a kernel ran out (thread block {1}, wait site {2}, {3} work items): "
                   "the launch left part of its output unwritten",
                2: "an expert index was outside [0, num_groups) (m_indices entry, routed pair or block of a "
                   "routing list): the rows it names were skipped; or a routing list had more runs of "
                   "blocks than 2 * experts + 2 and nothing was computed"}


def device_status_words(device: torch.device) -> torch.Tensor:
    """The int32[4] status words every launch on `device` reports into (allocated on first use)."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    words = _status_words.get(index)
    if words is None:
        words = torch.zeros(_cabi.STATUS_WORDS, dtype=torch.int32, device=torch.device("cuda", index))
        _status_words[index] = words
        if _glue is not None:
            _glue.set_status_words(index, words)
    return words


def check_device_status(device=None, *, clear: bool = True) -> None:
    """Raises RuntimeError if a kernel of this library reported a problem on `device` (default:
    the current device) since the last call.  Reads four ints from the device, i.e. waits for the
    work enqueued so far: call it where the caller synchronises anyway.  No launch of the public
    API fails silently: a wait that ran out or a skipped row block always shows up here."""
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    device = torch.device(device)
    index = device.index if device.index is not None else torch.cuda.current_device()
    words = _status_words.get(index)
    if words is None:
        return
    st = words.tolist()
    if st[0] == 0:
        return
    if clear:
        words.zero_()
    text = _STATUS_TEXT.get(st[0], "unknown device status {0}").format(*st)
    raise RuntimeError(f"deepgemm device status on cuda:{index}: {text}")


def _debug_and_status(debug_acc, status, rows, n, dev, what):
    if debug_acc is not None:
        if not (debug_acc.is_cuda and debug_acc.device == dev and debug_acc.is_contiguous() and debug_acc.element_size() == 4 and debug_acc.numel() == rows * n):
            raise RuntimeError(f"{what}: debug_acc must be a contiguous 32-bit tensor of {rows}x{n} on the same device")
    if status is not None:
        if not (status.is_cuda and status.device == dev and status.dtype == torch.int32 and status.is_contiguous() and status.numel() >= _cabi.STATUS_WORDS):
            raise RuntimeError(f"{what}: status must be int32[{_cabi.STATUS_WORDS}] on the same device")


def grouped_gemm_masked(kind: int, scale_mode: int, a: torch.Tensor, b: torch.Tensor,
                        d: torch.Tensor, a_scale: Optional[torch.Tensor],
                        b_scale: Optional[torch.Tensor], masked_m: torch.Tensor,
                        expected_m: int, *, block_n: int = 0,
                        debug_acc: Optional[torch.Tensor] = None,
                        status: Optional[torch.Tensor] = None,
                        signal: Optional[torch.Tensor] = None) -> torch.Tensor:
    """d[g, :masked_m[g]] = bf16((A[g] @ B[g]^T) * a_scale[g] * b_scale[g]) via dg_masked_gemm.
    ``signal``: int32 [G, ceil(max_m / 128)] completion counters (zeroed by the caller); entry
    (g, mb) reaches N when rows [128 mb, 128 mb + 128) of group g are complete."""
    # The native glue enqueues the call if every check below would pass; otherwise it enqueues
    # nothing and the checks run here, for the message or for the case it does not know.
    if _glue is not None and debug_acc is None and _glue.masked(
            kind, scale_mode, a, b, d, a_scale, b_scale, masked_m, expected_m, block_n, status, signal):
        return d
    what = f"masked {KIND_NAMES[kind]} grouped GEMM"
    if not (a.dim() == 3):
        raise RuntimeError(f"{what}: activation must be [G, max_m, K], got {tuple(a.shape)}")
    if not (d.dim() == 3):
        raise RuntimeError(f"{what}: output must be [G, max_m, N], got {tuple(d.shape)}")
    g, max_m, k = (int(x) for x in a.shape)
    bg, n, bk = packed_weight_dims(b, kind)
    _common_checks(kind, a, b, d, masked_m, what)
    if not (bg == g):
        raise RuntimeError(f"{what}: weight has {bg} groups, activation has {g}")
    if not _k_matches(kind, bk, k):
        raise RuntimeError(f"{what}: weight K={bk} does not match activation K={k}")
    if not (tuple(d.shape) == (g, max_m, n)):
        raise RuntimeError(f"{what}: output must be {(g, max_m, n)}, got {tuple(d.shape)}")
    if not (masked_m.numel() == g):
        raise RuntimeError(f"{what}: masked_m must have {g} entries, got {masked_m.numel()}")
    if scale_mode == SCALE_NONE:
        a_s = b_s = None
    else:
        if not (a_scale is not None and b_scale is not None):
            raise RuntimeError(f"{what}: scales are required")
        a_s = _scale(a_scale, (g, max_m), "a_scale", what)
        b_s = _scale(b_scale, (g, n) if scale_mode == SCALE_PER_CHANNEL else (g,), "b_scale", what)
    _debug_and_status(debug_acc, status, g * max_m, n, a.device, what)
    if status is None:
        status = device_status_words(a.device)
    if signal is not None:
        if not (signal.is_cuda and signal.device == a.device and signal.dtype == torch.int32
                and signal.is_contiguous() and signal.numel() == g * ((max_m + 127) // 128)):
            raise RuntimeError(f"{what}: signal must be contiguous CUDA int32 [{g}, {(max_m + 127) // 128}]")
        if kind == KIND_W4A8 or n % 32 != 0:
            raise RuntimeError(f"{what}: completion counters need an INT8 / FP8 / BF16 kind and N % 32 == 0")

    args = _cabi.MaskedArgs(
        kind=kind, scale_mode=scale_mode, a=a.data_ptr(), b_packed=b.data_ptr(), d=d.data_ptr(),
        a_scale=_ptr(a_s), b_scale=_ptr(b_s), masked_m=masked_m.data_ptr(), num_groups=g,
        max_m=max_m, n=n, k=k, expected_m=int(expected_m), block_n=int(block_n),
        debug_acc=_ptr(debug_acc), status=_ptr(status),
        out_kind=_cabi.OUT_F16 if d.dtype == torch.float16 else _cabi.OUT_BF16, signal=_ptr(signal))
    _launch(_cabi.lib.dg_masked_gemm, args, a.device, what)
    return d


def grouped_gemm_contiguous(kind: int, scale_mode: int, a: torch.Tensor, b: torch.Tensor,
                            d: torch.Tensor, a_scale: Optional[torch.Tensor],
                            b_scale: Optional[torch.Tensor], m_indices: torch.Tensor, *,
                            block_n: int = 0, debug_acc: Optional[torch.Tensor] = None,
                            status: Optional[torch.Tensor] = None, scatter=None,
                            group_window: Optional[int] = None) -> torch.Tensor:
    """d[i] = bf16((A[i] @ B[m_indices[i]]^T) * a_scale[i] * b_scale[m_indices[i]]) via dg_contig_gemm.
    ``group_window`` = w: ``m_indices`` numbers the groups of a wider set and ``b`` holds groups
    w .. w + G - 1 of it; rows of other groups are skipped (their output rows stay as they were).
    ``scatter`` = (tag int32 [M] CUDA tensor, ctypes array of buffer pointers, count): result row i
    goes to row ``tag[i] & 0xFFFFFF`` of buffer ``tag[i] >> 24`` instead of ``d[i]`` (``d`` is then
    only checked for dtype and device)."""
    what = f"contiguous {KIND_NAMES[kind]} grouped GEMM"
    if not (a.dim() == 2):
        raise RuntimeError(f"{what}: activation must be [M, K], got {tuple(a.shape)}")
    if not (d.dim() == 2):
        raise RuntimeError(f"{what}: output must be [M, N], got {tuple(d.shape)}")
    m_total, k = (int(x) for x in a.shape)
    g, n, bk = packed_weight_dims(b, kind)
    _common_checks(kind, a, b, d, m_indices, what)
    if not _k_matches(kind, bk, k):
        raise RuntimeError(f"{what}: weight K={bk} does not match activation K={k}")
    if scatter is None and not (tuple(d.shape) == (m_total, n)):
        raise RuntimeError(f"{what}: output must be {(m_total, n)}, got {tuple(d.shape)}")
    if scatter is not None:
        tag, bases, count = scatter
        if not (tag.is_cuda and tag.device == a.device and tag.dtype == torch.int32 and tag.is_contiguous()
                and tag.numel() == m_total):
            raise RuntimeError(f"{what}: scatter tag must be contiguous CUDA int32 [{m_total}]")
        if not (d.shape[-1] == n):
            raise RuntimeError(f"{what}: scattered rows have {n} columns, the buffers {d.shape[-1]}")
    if not (m_indices.numel() == m_total):
        raise RuntimeError(f"{what}: m_indices must have {m_total} entries")
    if scale_mode == SCALE_NONE:
        a_s = b_s = None
    else:
        if not (a_scale is not None and b_scale is not None):
            raise RuntimeError(f"{what}: scales are required")
        a_s = _scale(a_scale, (m_total,), "a_scale", what)
        b_s = _scale(b_scale, (g, n) if scale_mode == SCALE_PER_CHANNEL else (g,), "b_scale", what)
    _debug_and_status(debug_acc, status, m_total, n, a.device, what)
    if status is None:
        status = device_status_words(a.device)

    args = _cabi.ContigArgs(
        kind=kind, scale_mode=scale_mode, a=a.data_ptr(), b_packed=b.data_ptr(), d=d.data_ptr(),
        a_scale=_ptr(a_s), b_scale=_ptr(b_s), m_indices=m_indices.data_ptr(), num_groups=g,
        m_total=m_total, n=n, k=k, block_n=int(block_n),
        out_kind=_cabi.OUT_F16 if d.dtype == torch.float16 else _cabi.OUT_BF16,
        debug_acc=_ptr(debug_acc), status=_ptr(status))
    if scatter is not None:
        args.scatter_tag, args.scatter_base, args.scatter_world = scatter[0].data_ptr(), scatter[1], int(scatter[2])
    if group_window is not None:
        if group_window < 0:
            raise RuntimeError(f"{what}: group_window must not be negative")
        args.group_window = int(group_window) + 1
    _launch(_cabi.lib.dg_contig_gemm, args, a.device, what)
    return d


def grouped_gemm_compact(kind: int, scale_mode: int, a: torch.Tensor, b: torch.Tensor,
                         d: torch.Tensor, a_scale: Optional[torch.Tensor],
                         b_scale: Optional[torch.Tensor], counts: torch.Tensor,
                         offsets: torch.Tensor, expected_m: int, *, block_n: int = 0,
                         debug_acc: Optional[torch.Tensor] = None,
                         status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """d[offsets[g] + m] = bf16((A[offsets[g] + m] @ B[g]^T) * a_scale * b_scale[g]) for
    m < counts[g], via dg_compact_gemm; checks follow the reference's
    (csrc/arch/gfx936_gfx938_shared/m_grouped_w8a8_gemm_nt_masked.cu:1778-1838)."""
    what = f"compact {KIND_NAMES[kind]} grouped GEMM"
    if not (a.dim() == 2):
        raise RuntimeError(f"{what}: input must be [capacity, K], got {tuple(a.shape)}")
    if not (d.dim() == 2):
        raise RuntimeError(f"{what}: output must be [capacity, N], got {tuple(d.shape)}")
    cap, k = (int(x) for x in a.shape)
    g, n, bk = packed_weight_dims(b, kind)
    _common_checks(kind, a, b, d, counts, what)
    if not _k_matches(kind, bk, k):
        raise RuntimeError(f"{what}: weight K={bk} does not match activation K={k}")
    if not (tuple(d.shape) == (cap, n)):
        raise RuntimeError(f"{what}: output must be {(cap, n)}, got {tuple(d.shape)}")
    if not (counts.dim() == 1 and counts.numel() == g):
        raise RuntimeError(f"{what}: masked_m must be int32 [{g}]")
    if not (offsets.is_cuda and offsets.dtype == torch.int32 and offsets.is_contiguous() and offsets.shape == counts.shape):
        raise RuntimeError(f"{what}: expert_offsets must be contiguous CUDA int32 [{g}]")
    if scale_mode == SCALE_NONE:
        a_s = b_s = None
    else:
        if not (a_scale is not None and b_scale is not None):
            raise RuntimeError(f"{what}: scales are required")
        a_s = _scale(a_scale, (cap,), "a_scale", what)
        b_s = _scale(b_scale, (g, n) if scale_mode == SCALE_PER_CHANNEL else (g,), "b_scale", what)
    _debug_and_status(debug_acc, status, cap, n, a.device, what)
    if status is None:
        status = device_status_words(a.device)
    args = _cabi.CompactArgs(
        kind=kind, scale_mode=scale_mode, a=a.data_ptr(), b_packed=b.data_ptr(), d=d.data_ptr(),
        a_scale=_ptr(a_s), b_scale=_ptr(b_s), counts=counts.data_ptr(), offsets=offsets.data_ptr(),
        num_groups=g, capacity=cap, n=n, k=k, expected_m=int(expected_m), block_n=int(block_n),
        debug_acc=_ptr(debug_acc), status=_ptr(status))
    _launch(_cabi.lib.dg_compact_gemm, args, a.device, what)
    return d


def kind_of_activation(a: torch.Tensor) -> int:
    """INT8 or FP8 from the activation dtype, as the reference's low-latency op does
    (m_grouped_fp8_gemm_nt_maksed_low_latency.cu:1150-1161)."""
    if a.dtype == torch.int8:
        return KIND_I8
    if a.dtype == _FP8:
        return KIND_E4M3
    raise RuntimeError(f"activation must be torch.int8 or torch.float8_e4m3fn, got {a.dtype}")


__all__ = [
    "grouped_gemm_masked", "grouped_gemm_contiguous", "grouped_gemm_compact", "packed_weight_dims", "kind_of_activation",
    "check_device_status", "device_status_words",
    "KIND_I8", "KIND_E4M3", "KIND_W4A8", "KIND_BF16",
    "SCALE_PER_CHANNEL", "SCALE_TENSOR_WISE", "SCALE_NONE",
]
