"""Contiguous grouped GEMM front-ends: INT8, FP8 (per-channel and per-expert scales), W4A8.

Same names, argument order, return values and exception types as the reference's
``deepgemm/m_group_gemm_nt_contiguous.py`` (:60-109, :172-222, :330-426).  Rows of all
experts are stacked in one ``[M_total, K]`` tensor, ``m_indices[i]`` names row i's expert
and -1 marks padding rows; each expert's rows must start at a multiple of 128 (callers pad
every expert to a multiple of 256, README.md:115 of the reference).  ``config`` keys
(``MODE`` / ``BLOCK_M`` / ``BLOCK_N`` / ``N_LOOP_NUM``) selected Hygon tiles; they are
parsed for type errors and ignored.
"""
from __future__ import annotations

from typing import Any, Dict, Optional

import torch

from . import op
from .group_gemm_weight_pack import _resolve_shuffle_unique


def _int_cfg(config: Optional[Dict[str, Any]], key: str, default: int) -> int:
    return int(config.get(key, default)) if config is not None else default


def _normalize_contiguous_w4a8_a_scale(a_scale: torch.Tensor) -> torch.Tensor:
    if a_scale.dim() == 2:
        if a_scale.size(1) != 1:
            raise ValueError(
                f"contiguous W4A8 a_scale must be [M] or [M,1], got {tuple(a_scale.shape)}")
        return a_scale
    if a_scale.dim() != 1:
        raise ValueError(
            f"contiguous W4A8 a_scale must be [M] or [M,1], got {tuple(a_scale.shape)}")
    return a_scale


def _normalize_contiguous_b_scale(b_scale: torch.Tensor, what: str) -> torch.Tensor:
    if b_scale.dim() == 3:
        if b_scale.size(-1) != 1:
            raise ValueError(
                f"contiguous {what} b_scale must be [E,N] or [E,N,1], got {tuple(b_scale.shape)}")
        b_scale = b_scale.squeeze(-1)
    if b_scale.dim() != 2:
        raise ValueError(
            f"contiguous {what} b_scale must be [E,N] or [E,N,1], got {tuple(b_scale.shape)}")
    return b_scale


def m_grouped_w4a8_gemm_nt_contiguous_hipc(
    a: tuple[torch.Tensor, torch.Tensor],
    b: tuple[torch.Tensor, torch.Tensor],
    output: torch.Tensor,
    m_indices: torch.Tensor,
    config: Optional[Dict[str, Any]] = None,
) -> torch.Tensor:
    """INT8 activations x int4 weights, contiguous layout (reference :60-109).  ``b[0]`` is the
    ``[E,N,K/2]`` tensor rewritten by ``pack_w4a8_moe_hipc_weight``; ``b_scale`` carries 1/16."""
    input, a_scale = a
    b_qweight, b_scale = b
    mode = _int_cfg(config, "MODE", 1002)
    a_scale = _normalize_contiguous_w4a8_a_scale(a_scale)
    b_scale = _normalize_contiguous_b_scale(b_scale, "W4A8")
    if input.dim() != 2:
        raise ValueError(f"contiguous W4A8 input must be [M,K], got {tuple(input.shape)}")
    if output.dim() != 2:
        raise ValueError(f"contiguous W4A8 output must be [M,N], got {tuple(output.shape)}")
    if b_qweight.dim() not in (3, 4):
        raise ValueError(
            "contiguous W4A8 packed weight must be [E,N,K/2] from pack_w4a8_moe_hipc_weight")
    if output.size(0) != input.size(0):
        raise ValueError("contiguous W4A8 output M must match input M")
    if m_indices.numel() != input.size(0):
        raise ValueError("contiguous W4A8 m_indices length must match input M")
    if m_indices.dtype != torch.int32:
        m_indices = m_indices.to(torch.int32)
    return op.m_grouped_marlin_w4a8_gemm_nt_contiguous_hipc(
        input, b_qweight, output, a_scale.contiguous(), b_scale.contiguous(),
        m_indices.contiguous(), mode)


def m_grouped_i8_gemm_nt_contiguous(
    a: tuple[torch.Tensor, torch.Tensor],
    b: tuple[torch.Tensor, torch.Tensor],
    output: torch.Tensor,
    m_indices: torch.Tensor,
    config: Optional[Dict[str, Any]] = None,
    *,
    shuffle_unique: int = 1,
) -> torch.Tensor:
    """INT8 contiguous grouped GEMM (reference :172-222 -> :126-169)."""
    _resolve_shuffle_unique(shuffle_unique)
    input, a_scale = a
    b_qweight, b_scale = b
    b_scale = _normalize_contiguous_b_scale(b_scale, "int8")
    block_m = _int_cfg(config, "BLOCK_M", _int_cfg(config, "MODE", 128))
    block_n = _int_cfg(config, "BLOCK_N", 256)
    n_loop_num = _int_cfg(config, "N_LOOP_NUM", 4)
    if b_qweight.dim() != 4:
        raise ValueError(
            "m_grouped_i8_gemm_nt_contiguous expects a packed weight [E,K/128,N,128] "
            "from marlin_i8_contiguous_weight")
    if m_indices.dtype != torch.int32:
        m_indices = m_indices.to(torch.int32)
    torch.ops.deep_gemm.m_grouped_i8_gemm_nt_contiguous(
        input, b_qweight, output, a_scale.contiguous(), b_scale.contiguous(),
        m_indices.contiguous(), block_m, block_n, n_loop_num)
    return output


def m_grouped_i8_gemm_nt_contiguous_nopad(
    a: tuple[torch.Tensor, torch.Tensor],
    b: tuple[torch.Tensor, torch.Tensor],
    output: torch.Tensor,
    m_indices: torch.Tensor,
    token_per_expert: torch.Tensor,
) -> torch.Tensor:
    """INT8 contiguous grouped GEMM without padding rows (reference :312-323): the rows of
    expert e follow those of expert e-1 directly, ``token_per_expert[e]`` of them."""
    input, a_scale = a
    b_qweight, b_scale = b
    b_scale = _normalize_contiguous_b_scale(b_scale, "int8")
    return op.m_grouped_w8a8_gemm_nt_nopad_contiguous(
        input, b_qweight, output, a_scale, b_scale, m_indices, token_per_expert)


def m_grouped_bf16_gemm_nt_contiguous(
    a: torch.Tensor,
    b: torch.Tensor,
    output: torch.Tensor,
    m_indices: torch.Tensor,
    config: Optional[Dict[str, Any]] = {"MODE": 1000},
) -> torch.Tensor:
    """BF16 contiguous grouped GEMM, no scales (reference :504-518); ``b`` from
    ``pack_bf16_masked_weight``."""
    mode = config["MODE"]
    if b.dim() != 4:
        raise ValueError("BF16 contiguous kernels require weights packed by pack_bf16_masked_weight")
    if m_indices.dtype != torch.int32:
        m_indices = m_indices.to(torch.int32)
    ones = torch.empty(0, device=a.device)      # the reference passed unit scales; none are needed
    return op.m_grouped_w16a16_gemm_nt_contiguous(a, b, output, ones, ones, m_indices.contiguous(), mode)


def m_grouped_fp8_gemm_nt_contiguous(
    a: tuple[torch.Tensor, torch.Tensor],
    b: tuple[torch.Tensor, torch.Tensor],
    output: torch.Tensor,
    m_indices: torch.Tensor,
    config: Optional[Dict[str, Any]] = None,
) -> torch.Tensor:
    """FP8-e4m3 contiguous grouped GEMM, per-token x per-channel scales (reference :330-377)."""
    input, a_scale = a
    b_qweight, b_scale = b
    block_m = _int_cfg(config, "BLOCK_M", _int_cfg(config, "MODE", 128))
    block_n = _int_cfg(config, "BLOCK_N", 256)
    n_loop_num = _int_cfg(config, "N_LOOP_NUM", 4)
    if m_indices.dtype != torch.int32:
        m_indices = m_indices.to(torch.int32)
    torch.ops.deep_gemm.m_grouped_fp8_gemm_nt_contiguous(
        input, b_qweight, output, a_scale.contiguous(), b_scale.contiguous(),
        m_indices.contiguous(), block_m, block_n, n_loop_num)
    return output


def m_grouped_fp8_gemm_nt_contiguous_tensor_wise(
    a: tuple[torch.Tensor, torch.Tensor],
    b: tuple[torch.Tensor, torch.Tensor],
    output: torch.Tensor,
    m_indices: torch.Tensor,
    config: Optional[Dict[str, Any]] = None,
) -> torch.Tensor:
    """FP8 contiguous grouped GEMM with one weight scale per expert, ``b_scale`` ``[E]`` or
    ``[E,1]`` (reference :380-426)."""
    input, a_scale = a
    b_qweight, b_scale = b
    mode = _int_cfg(config, "MODE", 128)
    n_loop_num = _int_cfg(config, "N_LOOP_NUM", 4)
    if m_indices.dtype != torch.int32:
        m_indices = m_indices.to(torch.int32)
    if not (b_scale.dim() == 1 or (b_scale.dim() == 2 and b_scale.size(1) == 1)):
        raise ValueError(
            f"tensor-wise contiguous B scale must have shape [E] or [E, 1], got {tuple(b_scale.shape)}")
    torch.ops.deep_gemm.m_grouped_fp8_gemm_nt_contiguous_marlin_tensor_wise(
        input, b_qweight, output, a_scale.contiguous(), b_scale.contiguous(),
        m_indices.contiguous(), mode, n_loop_num)
    return output


def get_m_grouped_fp8_contiguous_config(size_m: int, size_n: int) -> Dict[str, int]:
    """Kept for callers that pass its result back as ``config`` (reference
    deepgemm/configs/contiguous.py:13-84 looked up Hygon tiles); the values are not used."""
    return {"MODE": 128, "N_LOOP_NUM": 4}
