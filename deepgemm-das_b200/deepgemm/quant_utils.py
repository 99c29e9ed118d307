"""Activation / weight quantisers and workload builders used by callers, the benchmark and
the expert-parallel harness.  Plain torch ops on whatever device the input lives on; these
run before the GEMM, they are not part of it.

``per_token_quant_int8`` follows the reference's test helper (op_test/quant_utils.py:4-19);
``per_token_quant_fp8`` is its e4m3 analogue with scale = absmax / 448.
"""
from __future__ import annotations

from typing import Sequence, Tuple

import torch

FP8 = torch.float8_e4m3fn
FP8_MAX = 448.0


def per_token_quant_int8(x: torch.Tensor, eps: float = 1e-10) -> Tuple[torch.Tensor, torch.Tensor]:
    """Symmetric int8 quantisation along the last dimension: (q int8, scale fp32 [...,1])."""
    if not x.is_floating_point():
        raise TypeError(f"x must be floating point, got {x.dtype}")
    xf = x.float()
    absmax = xf.abs().amax(dim=-1, keepdim=True).clamp_min(eps)
    q = torch.round(xf * (127.0 / absmax)).clamp(-128, 127).to(torch.int8)
    return q.contiguous(), (absmax / 127.0).contiguous()


def per_token_quant_fp8(x: torch.Tensor, eps: float = 1e-10) -> Tuple[torch.Tensor, torch.Tensor]:
    """Symmetric e4m3 quantisation along the last dimension: (q e4m3, scale fp32 [...,1])."""
    if not x.is_floating_point():
        raise TypeError(f"x must be floating point, got {x.dtype}")
    xf = x.float()
    absmax = xf.abs().amax(dim=-1, keepdim=True).clamp_min(eps)
    q = (xf * (FP8_MAX / absmax)).clamp(-FP8_MAX, FP8_MAX).to(FP8)
    return q.contiguous(), (absmax / FP8_MAX).contiguous()


def per_channel_quant_int4(w: torch.Tensor, eps: float = 1e-10) -> Tuple[torch.Tensor, torch.Tensor]:
    """Symmetric int4 quantisation to [-7,7] along the last dimension:
    (values int8 in [-7,7], scale fp32 [...,1])."""
    wf = w.float()
    absmax = wf.abs().amax(dim=-1, keepdim=True).clamp_min(eps)
    q = torch.round(wf * (7.0 / absmax)).clamp(-7, 7).to(torch.int8)
    return q.contiguous(), (absmax / 7.0).contiguous()


def pack_int4_pairs(w4: torch.Tensor, nibble_order: str = "high_first") -> torch.Tensor:
    """Signed int4 values [..., K] -> bytes [..., K/2], two per byte, even-k value in the high
    (``high_first``) or low (``low_first``) nibble."""
    nib = (w4.to(torch.int16) & 0xF).view(*w4.shape[:-1], w4.shape[-1] // 2, 2)
    first, second = (nib[..., 0], nib[..., 1]) if nibble_order == "high_first" else (nib[..., 1], nib[..., 0])
    packed = (first << 4) | second
    return torch.where(packed > 127, packed - 256, packed).to(torch.int8)


def contiguous_layout(rows_per_group: Sequence[int], align: int = 256, device="cpu"
                      ) -> Tuple[torch.Tensor, torch.Tensor, int]:
    """Row layout of the contiguous grouped GEMM: every group's rows padded up to a multiple
    of ``align``.  Returns (m_indices int32 [M_total] with -1 on padding rows,
    group_starts int64 [G], M_total)."""
    rows = torch.as_tensor(rows_per_group, dtype=torch.int64)
    padded = (rows + align - 1) // align * align
    starts = torch.cumsum(padded, 0) - padded
    m_total = int(padded.sum())
    m_indices = torch.full((m_total,), -1, dtype=torch.int32)
    for g, (s, r) in enumerate(zip(starts.tolist(), rows.tolist())):
        m_indices[s:s + r] = g
    return m_indices.to(device), starts.to(device), m_total


def algorithmic_bytes(valid_rows: int, groups_with_rows: int, groups: int, n: int, k: int,
                      a_bytes: float, b_bytes: float, tensor_wise: bool = False,
                      index_entries: int = 0) -> float:
    """Bytes a grouped GEMM must move at minimum: activations and outputs of valid rows,
    weights of groups that have rows, scales, and the masked_m / m_indices array.  The
    reference's own accounting (op_test/test_deepgemm_masked_w8a8_fp8.py:270-274) plus scales."""
    v, gp = valid_rows, groups_with_rows
    return (v * k * a_bytes + gp * n * k * b_bytes + v * n * 2 + 4 * v +
            (4 * gp if tensor_wise else 4 * gp * n) + 4 * (index_entries or groups))
