"""Producer for the contiguous grouped GEMM: per-token quantisation fused with grouping the
rows by expert and padding each expert's block (``dg_quant_group_rows`` of the C ABI).

The reference leaves this step to its callers; its tests do it with torch tensor ops
(op_test/contiguous_w8a8_int8_common.py:38-62, op_test/quant_utils.py:4-19).  The fused
kernels read every activation row once and write the quantised row straight to its place in
the ``[M, K]`` operand, with ``m_indices`` and the per-row scales, without a host round trip.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _cabi
from ._core import _launch
from ._cabi import KIND_E4M3, KIND_I8


def quant_group_capacity(num_rows: int, num_groups: int, align: int = 256) -> int:
    """Rows that always hold every grouped, padded row: R + G * (align - 1), rounded up to align."""
    cap = int(num_rows) + int(num_groups) * (int(align) - 1)
    return (cap + align - 1) // align * align


def quantize_group_rows(rows: torch.Tensor, expert: torch.Tensor, num_groups: int, *,
                        kind: str = "fp8", align: int = 256, m_cap: Optional[int] = None,
                        scratch: Optional[torch.Tensor] = None,
                        src_index: Optional[torch.Tensor] = None,
                        row_scale: Optional[torch.Tensor] = None
                        ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """rows bf16 [R, H] (CUDA), expert int32 [R] -> (a [m_cap, H] e4m3 / int8, a_scale fp32
    [m_cap], m_indices int32 [m_cap], dest int32 [R], m_total int32 [1]); all on the device,
    no synchronisation.  Pass the results to the contiguous grouped GEMM as they are.  With
    ``src_index`` (int32 [R], entries in [0, rows.shape[0])) row r is read from
    ``rows[src_index[r]]``, so the top-k copies of a token need not be materialised.  With
    ``row_scale`` (fp32, one per row of ``rows``) the rows are e4m3 / int8 already and are only
    grouped: bytes copied, scales carried along."""
    if not rows.is_cuda:
        raise RuntimeError("quantize_group_rows: rows must be a CUDA tensor (there is no CPU implementation)")
    if kind not in ("fp8", "int8"):
        raise ValueError(f"kind must be 'fp8' or 'int8', got {kind!r}")
    if row_scale is not None:
        want = torch.float8_e4m3fn if kind == "fp8" else torch.int8
        if rows.dim() != 2 or rows.dtype != want or not rows.is_contiguous():
            raise ValueError(f"with row_scale, rows must be a contiguous {want} [R, H] tensor")
        if row_scale.dtype != torch.float32 or row_scale.numel() != rows.shape[0]:
            raise ValueError("row_scale must be fp32 with one entry per row")
        row_scale = row_scale.contiguous()
    elif rows.dim() != 2 or rows.dtype != torch.bfloat16 or not rows.is_contiguous():
        raise ValueError(f"rows must be a contiguous bf16 [R, H] tensor, got {rows.dtype} {tuple(rows.shape)}")
    r, h = (int(v) for v in rows.shape)
    if src_index is not None:
        if src_index.dtype != torch.int32 or src_index.dim() != 1:
            raise ValueError("src_index must be an int32 vector")
        src_index = src_index.contiguous()
        r = int(src_index.numel())
    if expert.numel() != r:
        raise ValueError(f"expert must have {r} entries, got {expert.numel()}")
    if expert.dtype != torch.int32:
        expert = expert.to(torch.int32)
    expert = expert.contiguous()
    k = KIND_E4M3 if kind == "fp8" else KIND_I8
    if m_cap is None:
        m_cap = quant_group_capacity(r, num_groups, align)
    dev = rows.device
    a = torch.empty((m_cap, h), dtype=torch.float8_e4m3fn if kind == "fp8" else torch.int8, device=dev)
    a_scale = torch.zeros((m_cap,), dtype=torch.float32, device=dev)
    m_indices = torch.empty((m_cap,), dtype=torch.int32, device=dev)
    dest = torch.empty((r,), dtype=torch.int32, device=dev)
    m_total = torch.empty((1,), dtype=torch.int32, device=dev)
    need = int(_cabi.lib.dg_quant_group_scratch_bytes(r, int(num_groups)))
    if need == 0:
        raise ValueError(f"bad problem size: rows={r} groups={num_groups}")
    if scratch is None or scratch.numel() * scratch.element_size() < need or scratch.device != dev:
        scratch = torch.empty((need,), dtype=torch.uint8, device=dev)
    args = _cabi.QuantGroupArgs(
        kind=k, num_rows=r, hidden=h, num_groups=int(num_groups), align=int(align), m_cap=int(m_cap),
        rows=rows.data_ptr(), expert=expert.data_ptr(), a_out=a.data_ptr(),
        a_scale_out=a_scale.data_ptr(), m_indices_out=m_indices.data_ptr(), dest_out=dest.data_ptr(),
        m_total_out=m_total.data_ptr(), scratch=scratch.data_ptr(),
        scratch_bytes=scratch.numel() * scratch.element_size(),
        src_index=src_index.data_ptr() if src_index is not None else None,
        row_scale=row_scale.data_ptr() if row_scale is not None else None)
    _launch(_cabi.lib.dg_quant_group_rows, args, dev, "dg_quant_group_rows")
    return a, a_scale, m_indices, dest, m_total


def quantize_rows(rows: torch.Tensor, *, kind: str = "fp8") -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-row quantisation only: bf16 [R, H] -> (q [R, H] e4m3 / int8, scale fp32 [R]), rows in
    place (the producer with a single group and no padding)."""
    r = rows.shape[0]
    expert = torch.zeros((r,), dtype=torch.int32, device=rows.device)
    a, a_scale, _, _, _ = quantize_group_rows(rows, expert, 1, kind=kind, align=1, m_cap=max(r, 1))
    return a[:r], a_scale[:r]
