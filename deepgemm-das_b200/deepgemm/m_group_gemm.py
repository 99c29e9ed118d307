"""Low-latency masked grouped GEMM front-ends (FP8 and INT8, per-channel or per-expert
weight scales).  Signatures, argument handling and error behaviour follow the reference's
``deepgemm/m_group_gemm.py`` (:111-197, :200-288, :291-370, :867-882); the ``cu`` argument
chose a persistent grid size on Hygon parts and is accepted and ignored here (the library
launches one block per SM).
"""
from __future__ import annotations

from typing import Any, Dict, Optional

import torch

from . import op
from .group_gemm_weight_pack import (pack_int8_weight_enk_to_w6_low_latency,
                                     pack_int8_weight_enk_to_w6_low_latency_inplace)


def _resolve_masked_ll_cu(cu: Optional[int]) -> int:
    return 0 if cu is None else int(cu)


def _check_expert_counts(a, b, masked_m) -> int:
    experts = int(a[0].shape[0])
    if int(masked_m.numel()) != experts:
        raise ValueError(
            f"masked_m length {masked_m.numel()} != expert count from a[0] ({experts})")
    if int(b[0].shape[0]) != experts:
        raise ValueError(f"b[0].shape[0] ({b[0].shape[0]}) != expert count ({experts})")
    return experts


def m_grouped_w8a8_gemm_nt_masked_ll(
    a: tuple[torch.Tensor, torch.Tensor],
    b: tuple[torch.Tensor, torch.Tensor],
    d: torch.Tensor,
    masked_m: torch.Tensor,
    expected_m_per_group: int,
    config: Optional[Dict[str, Any]] = None,
    *,
    block_wise: bool = False,
    cu: Optional[int] = None,
) -> torch.Tensor:
    """INT8 masked grouped GEMM, per-token x per-channel scales (reference :111-197).

    ``b[0]`` must come from ``pack_int8_weight_enk_to_w6_low_latency`` / ``marlin_i8_masked_weight``.
    """
    cu = _resolve_masked_ll_cu(cu)
    experts = _check_expert_counts(a, b, masked_m)
    matrix_a, a_scale = a
    matrix_b, b_scale = b
    if block_wise:
        raise RuntimeError("m_grouped_w8a8_gemm_nt_masked_ll only supports channel-wise scales")
    if a_scale.dim() == 3:
        if a_scale.size(-1) != 1:
            raise ValueError(
                f"channel-wise a_scale must have shape [E,M] or [E,M,1], got {tuple(a_scale.shape)}")
        a_scale = a_scale.squeeze(-1)
    if b_scale.dim() == 3:
        if b_scale.size(-1) != 1:
            raise ValueError(
                f"channel-wise b_scale must have shape [E,N] or [E,N,1], got {tuple(b_scale.shape)}")
        b_scale = b_scale.squeeze(-1)
    if not a_scale.is_contiguous():
        raise ValueError("a_scale must be contiguous")
    if not b_scale.is_contiguous():
        raise ValueError("b_scale must be contiguous")
    if masked_m.dtype != torch.int32:
        raise ValueError(f"masked_m must be torch.int32, got {masked_m.dtype}")
    op.low_latency_grouped_gemm(matrix_a, matrix_b, a_scale, b_scale, masked_m, d,
                                int(expected_m_per_group), experts, cu, False, False, None)
    return d


def m_grouped_fp8_gemm_nt_masked_ll(
    a: tuple[torch.Tensor, torch.Tensor],
    b: tuple[torch.Tensor, torch.Tensor],
    d: torch.Tensor,
    masked_m: torch.Tensor,
    expected_m_per_group: int,
    enable_overlap: bool = False,
    signal: Optional[torch.Tensor] = None,
    config: Optional[Dict[str, Any]] = None,
    *,
    block_wise: bool = False,
    cu: Optional[int] = None,
) -> torch.Tensor:
    """FP8-e4m3 masked grouped GEMM, per-token x per-channel scales (reference :200-260)."""
    del config
    if block_wise:
        raise RuntimeError(
            "m_grouped_fp8_gemm_nt_masked only supports channel-wise non-block-wise scales")
    cu = _resolve_masked_ll_cu(cu)
    matrix_a, a_scale = a
    matrix_b, b_scale = b
    if a_scale.dim() == 3:
        a_scale = a_scale.squeeze(-1)
    if b_scale.dim() == 3:
        b_scale = b_scale.squeeze(-1)
    experts = int(matrix_a.shape[0])
    op.low_latency_grouped_gemm(matrix_a, matrix_b, a_scale, b_scale, masked_m, d,
                                int(expected_m_per_group), experts, cu, False,
                                bool(enable_overlap), signal)
    return d


def m_grouped_fp8_gemm_nt_masked(
    a: tuple[torch.Tensor, torch.Tensor],
    b: tuple[torch.Tensor, torch.Tensor],
    d: torch.Tensor,
    masked_m: torch.Tensor,
    expected_m_per_group: int,
    enable_overlap: bool = False,
    signal: Optional[torch.Tensor] = None,
    config: Optional[Dict[str, Any]] = None,
    *,
    block_wise: bool = False,
    cu: Optional[int] = None,
) -> torch.Tensor:
    """Reference :264-288."""
    return m_grouped_fp8_gemm_nt_masked_ll(a, b, d, masked_m, expected_m_per_group,
                                           enable_overlap=enable_overlap, signal=signal,
                                           config=config, block_wise=block_wise, cu=cu)


def m_grouped_fp8_gemm_nt_masked_ll_tensor_wise(
    a: tuple[torch.Tensor, torch.Tensor],
    b: tuple[torch.Tensor, torch.Tensor],
    d: torch.Tensor,
    masked_m: torch.Tensor,
    expected_m_per_group: int,
    enable_overlap: bool = False,
    signal: Optional[torch.Tensor] = None,
    config: Optional[Dict[str, Any]] = None,
    *,
    cu: Optional[int] = None,
) -> torch.Tensor:
    """FP8 masked grouped GEMM with one weight scale per expert, ``b_scale`` of shape ``[E]`` or
    ``[E,1]``; activations stay per-token (reference :291-370)."""
    del config
    cu = _resolve_masked_ll_cu(cu)
    experts = _check_expert_counts(a, b, masked_m)
    matrix_a, a_scale = a
    matrix_b, b_scale = b
    if a_scale.dim() == 3 and a_scale.size(-1) == 1:
        a_scale = a_scale.squeeze(-1)
    if not (b_scale.dim() == 1 or (b_scale.dim() == 2 and b_scale.size(1) == 1)):
        raise ValueError(
            f"tensor-wise B scale must have shape [E] or [E, 1], got {tuple(b_scale.shape)}")
    if not a_scale.is_contiguous():
        raise ValueError("a_scale must be contiguous")
    if not b_scale.is_contiguous():
        raise ValueError("b_scale must be contiguous")
    if masked_m.dtype != torch.int32:
        raise ValueError(f"masked_m must be torch.int32, got {masked_m.dtype}")
    op.low_latency_grouped_gemm_tensor_wise(matrix_a, matrix_b, a_scale, b_scale, masked_m, d,
                                            int(expected_m_per_group), experts, cu,
                                            bool(enable_overlap), signal)
    return d


def m_grouped_fp8_gemm_nt_masked_tensor_wise(
    a: tuple[torch.Tensor, torch.Tensor],
    b: tuple[torch.Tensor, torch.Tensor],
    d: torch.Tensor,
    masked_m: torch.Tensor,
    expected_m_per_group: int,
    enable_overlap: bool = False,
    signal: Optional[torch.Tensor] = None,
    config: Optional[Dict[str, Any]] = None,
    *,
    cu: Optional[int] = None,
) -> torch.Tensor:
    """Reference :867-882."""
    return m_grouped_fp8_gemm_nt_masked_ll_tensor_wise(
        a, b, d, masked_m, expected_m_per_group, enable_overlap=enable_overlap, signal=signal,
        config=config, cu=cu)


__all__ = [
    "m_grouped_w8a8_gemm_nt_masked_ll",
    "m_grouped_fp8_gemm_nt_masked_ll",
    "m_grouped_fp8_gemm_nt_masked",
    "m_grouped_fp8_gemm_nt_masked_ll_tensor_wise",
    "m_grouped_fp8_gemm_nt_masked_tensor_wise",
    "pack_int8_weight_enk_to_w6_low_latency",
    "pack_int8_weight_enk_to_w6_low_latency_inplace",
]
