"""The steps around the two grouped GEMMs of an MoE layer, and the layer itself.

gate/up GEMM -> SiLU(gate) * up + per-row requantisation -> down GEMM -> weighted sum of every
token's top-k rows.  The reference ships only the GEMMs (its second-stage op
``moe_w8a8_marlin_prefill_down_fp8``, deepgemm/moe_marlin_prefill.py:15-56, expects activated,
quantised rows and folds the routing weight into the row scale); the two memory-bound steps
here are ``dg_silu_mul_quant_rows`` and ``dg_combine_rows`` of the C ABI.  CUDA tensors only.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _cabi
from ._core import _launch
from ._cabi import KIND_E4M3, KIND_I8


def silu_mul_quant(x: torch.Tensor, *, kind: str = "fp8", m_indices: Optional[torch.Tensor] = None,
                   masked_m: Optional[torch.Tensor] = None,
                   out: Optional[Tuple[torch.Tensor, torch.Tensor]] = None
                   ) -> Tuple[torch.Tensor, torch.Tensor]:
    """x bf16 ``[M, 2H]`` (contiguous layout; rows with ``m_indices < 0`` are skipped) or
    ``[G, max_m, 2H]`` (masked layout; rows ``>= masked_m[g]`` are skipped), gate in the first H
    columns -> ``(q [.., H] e4m3 / int8, scale fp32 [..])``.  Skipped rows keep whatever ``out``
    held (zeros when this function allocates)."""
    if not x.is_cuda:
        raise RuntimeError("silu_mul_quant: x must be a CUDA tensor (there is no CPU implementation)")
    if x.dtype != torch.bfloat16 or not x.is_contiguous() or x.dim() not in (2, 3):
        raise ValueError(f"x must be a contiguous bf16 [M,2H] or [G,max_m,2H] tensor, got {x.dtype} {tuple(x.shape)}")
    if kind not in ("fp8", "int8"):
        raise ValueError(f"kind must be 'fp8' or 'int8', got {kind!r}")
    if x.shape[-1] % 2:
        raise ValueError("last dimension must hold the gate and the up half")
    h = x.shape[-1] // 2
    lead = tuple(x.shape[:-1])
    rows = 1
    for v in lead:
        rows *= int(v)
    if masked_m is not None:
        if x.dim() != 3 or masked_m.numel() != x.shape[0] or masked_m.dtype != torch.int32:
            raise ValueError("masked_m must be int32 [G] and x [G,max_m,2H]")
    if m_indices is not None:
        if x.dim() != 2 or m_indices.numel() != rows or m_indices.dtype != torch.int32:
            raise ValueError("m_indices must be int32 [M] and x [M,2H]")
    qdtype = torch.float8_e4m3fn if kind == "fp8" else torch.int8
    if out is None:
        q = torch.zeros(lead + (h,), dtype=qdtype, device=x.device)
        scale = torch.zeros(lead, dtype=torch.float32, device=x.device)
    else:
        q, scale = out
        if q.dtype != qdtype or tuple(q.shape) != lead + (h,) or not q.is_contiguous():
            raise ValueError("out[0] has the wrong dtype or shape")
        if scale.dtype != torch.float32 or scale.numel() != rows or not scale.is_contiguous():
            raise ValueError("out[1] must be a contiguous fp32 tensor with one entry per row")
    args = _cabi.ActQuantArgs(
        kind=KIND_E4M3 if kind == "fp8" else KIND_I8, num_rows=rows, hidden=h,
        max_m=int(x.shape[1]) if x.dim() == 3 else 0, x=x.data_ptr(),
        m_indices=m_indices.contiguous().data_ptr() if m_indices is not None else None,
        masked_m=masked_m.contiguous().data_ptr() if masked_m is not None else None,
        q_out=q.data_ptr(), scale_out=scale.data_ptr())
    _launch(_cabi.lib.dg_silu_mul_quant_rows, args, x.device, "dg_silu_mul_quant_rows")
    return q, scale


def combine_rows(y: torch.Tensor, src_row: torch.Tensor, weights: Optional[torch.Tensor] = None,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[t] = bf16(sum_j weights[t, j] * y[src_row[t, j]])``; y bf16 ``[R, N]``, src_row int32
    ``[T, top_k]`` (negative entries contribute nothing), weights fp32 ``[T, top_k]`` or None."""
    if not y.is_cuda:
        raise RuntimeError("combine_rows: y must be a CUDA tensor (there is no CPU implementation)")
    if y.dtype != torch.bfloat16 or y.dim() != 2 or not y.is_contiguous():
        raise ValueError("y must be a contiguous bf16 [R, N] tensor")
    if src_row.dim() != 2 or src_row.dtype != torch.int32:
        raise ValueError("src_row must be int32 [T, top_k]")
    t, k = (int(v) for v in src_row.shape)
    if weights is not None and (tuple(weights.shape) != (t, k) or weights.dtype != torch.float32):
        raise ValueError("weights must be fp32 [T, top_k]")
    if out is None:
        out = torch.empty((t, y.shape[1]), dtype=torch.bfloat16, device=y.device)
    elif out.dtype != torch.bfloat16 or tuple(out.shape) != (t, y.shape[1]) or not out.is_contiguous():
        raise ValueError("out must be a contiguous bf16 [T, N] tensor")
    args = _cabi.CombineArgs(
        num_tokens=t, top_k=k, n=int(y.shape[1]), num_rows=int(y.shape[0]), y=y.data_ptr(),
        src_row=src_row.contiguous().data_ptr(),
        weights=weights.contiguous().data_ptr() if weights is not None else None, out=out.data_ptr())
    _launch(_cabi.lib.dg_combine_rows, args, y.device, "dg_combine_rows")
    return out


def expert_mlp_contiguous(a: torch.Tensor, a_scale: torch.Tensor, m_indices: torch.Tensor,
                          w13: Tuple[torch.Tensor, torch.Tensor], w2: Tuple[torch.Tensor, torch.Tensor],
                          *, kind: str = "fp8") -> torch.Tensor:
    """Both GEMMs of the experts on rows already quantised and grouped (the outputs of
    ``quantize_group_rows``): ``w13`` = (packed ``[E, 2I, K]`` gate|up weight, scale ``[E, 2I]``),
    ``w2`` = (packed ``[E, K_out, I]``, scale ``[E, K_out]``).  Returns bf16 ``[M, K_out]``; padding
    rows (``m_indices < 0``) are not written and hold whatever the allocator returned."""
    from .m_group_gemm_nt_contiguous import m_grouped_fp8_gemm_nt_contiguous, m_grouped_i8_gemm_nt_contiguous
    gemm = m_grouped_fp8_gemm_nt_contiguous if kind == "fp8" else m_grouped_i8_gemm_nt_contiguous
    m = a.shape[0]
    h13 = torch.empty((m, w13[1].shape[1]), dtype=torch.bfloat16, device=a.device)
    gemm((a, a_scale), w13, h13, m_indices)
    # padding rows of the activation operand are never stored by the GEMM: no need to clear them
    qdtype = torch.float8_e4m3fn if kind == "fp8" else torch.int8
    q, s = silu_mul_quant(h13, kind=kind, m_indices=m_indices,
                          out=(torch.empty((m, h13.shape[1] // 2), dtype=qdtype, device=a.device),
                               torch.empty((m,), dtype=torch.float32, device=a.device)))
    y = torch.empty((m, w2[1].shape[1]), dtype=torch.bfloat16, device=a.device)
    gemm((q, s), w2, y, m_indices)
    return y


def moe_forward(hidden: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor,
                w13: Tuple[torch.Tensor, torch.Tensor], w2: Tuple[torch.Tensor, torch.Tensor],
                *, kind: str = "fp8") -> torch.Tensor:
    """A whole MoE layer on one GPU: hidden bf16 ``[T, K]``, topk_ids ``[T, top_k]`` (distinct
    experts per token), topk_weights fp32 ``[T, top_k]`` -> bf16 ``[T, K_out]``.  Six launches
    after the routing: quantise+group (4), gate/up GEMM, activation, down GEMM, combine."""
    from .quant_group import quantize_group_rows
    t, k = topk_ids.shape
    num_experts = w13[1].shape[0]
    token = torch.arange(t, dtype=torch.int32, device=hidden.device).repeat_interleave(k)
    expert = topk_ids.reshape(-1).to(torch.int32)                   # pair t*k + j = (token t, j)
    a, a_scale, m_indices, dest, _ = quantize_group_rows(hidden, expert, num_experts, kind=kind,
                                                         src_index=token)
    y = expert_mlp_contiguous(a, a_scale, m_indices, w13, w2, kind=kind)
    return combine_rows(y, dest.view(t, k), topk_weights.to(torch.float32))
