"""Dense (batched) FP8 / INT8 GEMM front-ends.

Same names and argument order as the reference's ``deepgemm/gemm.py`` (:8-42 ``fp8_gemm`` on
hipBLASLt, :44-83 ``fp8_gemm_hipc`` on its own kernel): ``a = (A, scale_a)`` with A ``[M, K]`` or
``[batch, M, K]`` and scale_a fp32 ``[M]``; ``b = (B, scale_b)`` with B ``[N, K]`` or
``[batch, N, K]`` and scale_b fp32 ``[N]``; ``d`` is written in place:
``d = (A * scale_a[:, None]) @ (B * scale_b[:, None]).T``.  Empty scale tensors mean no scaling.
Both run the grouped kernels of this library with the batch as groups and the weights read in
their natural row-major order (``dg_dense_gemm``); ``c``, ``recipe``, ``compiled_dims`` and
``disable_ue8m0_cast`` are accepted and ignored as in the reference.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _cabi
from ._core import _launch, device_status_words

_OUT_KIND = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}


def _dense(a, b, d, where: str, allowed) -> torch.Tensor:
    mat_a, scale_a = a
    mat_b, scale_b = b
    if mat_a.dtype not in allowed:
        raise ValueError(f"{where} expects {' or '.join(str(t) for t in allowed)} inputs, got {mat_a.dtype}")
    if mat_b.dtype != mat_a.dtype:
        raise ValueError(f"{where}: A is {mat_a.dtype} but B is {mat_b.dtype}")
    if not mat_a.is_cuda:
        raise RuntimeError(f"{where}: tensors must be on a CUDA device (there is no CPU implementation)")
    if mat_a.dtype == torch.bfloat16 and ((scale_a is not None and scale_a.numel()) or
                                          (scale_b is not None and scale_b.numel())):
        raise ValueError(f"{where}: bf16 operands take no scales")
    if mat_a.dim() not in (2, 3) or mat_b.dim() != mat_a.dim():
        raise ValueError(f"{where}: A and B must both be 2-D or both 3-D")
    batch = mat_b.shape[0] if mat_b.dim() == 3 else 1
    m, k = int(mat_a.shape[-2]), int(mat_a.shape[-1])
    n = int(mat_b.shape[-2])
    if int(mat_b.shape[-1]) != k:
        raise ValueError(f"{where}: B must be [N, K] with K={k}, got {tuple(mat_b.shape)}")
    if mat_a.dim() == 3 and mat_a.shape[0] != batch:
        raise ValueError(f"{where}: batch of A and B differ")
    if d.dtype not in _OUT_KIND:
        raise ValueError(f"{where}: output must be bf16, fp16 or fp32, got {d.dtype}")
    if tuple(d.shape[-2:]) != (m, n) or d.numel() != batch * m * n:
        raise ValueError(f"{where}: output must be [{m}, {n}] per batch entry, got {tuple(d.shape)}")
    for t, what in ((mat_a, "A"), (mat_b, "B"), (d, "output")):
        if not t.is_contiguous():
            raise ValueError(f"{where}: {what} must be contiguous")
    has_a = scale_a is not None and scale_a.numel() > 0
    has_b = scale_b is not None and scale_b.numel() > 0
    if has_a or has_b:                                   # one-sided scaling: the other side is 1
        scale_a = (scale_a.to(torch.float32).contiguous() if has_a
                   else torch.ones(batch * m, dtype=torch.float32, device=mat_a.device))
        scale_b = (scale_b.to(torch.float32).contiguous() if has_b
                   else torch.ones(batch * n, dtype=torch.float32, device=mat_a.device))
        if scale_a.numel() != batch * m or scale_b.numel() != batch * n:
            raise ValueError(f"{where}: scales must have one entry per row of A ({batch * m}) and of B ({batch * n})")
    kind = {torch.int8: _cabi.KIND_I8, torch.float8_e4m3fn: _cabi.KIND_E4M3,
            torch.bfloat16: _cabi.KIND_BF16}[mat_a.dtype]
    args = _cabi.DenseArgs(
        kind=kind, out_kind=_OUT_KIND[d.dtype], a=mat_a.data_ptr(), b=mat_b.data_ptr(), d=d.data_ptr(),
        a_scale=scale_a.data_ptr() if (has_a or has_b) else None,
        b_scale=scale_b.data_ptr() if (has_a or has_b) else None,
        batch=batch, m=m, n=n, k=k, block_n=0, reserved=0, debug_acc=None,
        status=device_status_words(mat_a.device).data_ptr())
    _launch(_cabi.lib.dg_dense_gemm, args, mat_a.device, where)
    return d


def fp8_gemm(a: Tuple[torch.Tensor, torch.Tensor],
             b: Tuple[torch.Tensor, torch.Tensor],
             d: torch.Tensor,
             c: Optional[torch.Tensor] = None,
             recipe: Optional[Tuple[int, int, int]] = None,
             compiled_dims: str = "nk",
             disable_ue8m0_cast: bool = False):
    """e4m3 or int8 operands (reference :8-42, which raises for anything else)."""
    _dense(a, b, d, "fp8_gemm", (torch.float8_e4m3fn, torch.int8))


def fp8_gemm_hipc(a: Tuple[torch.Tensor, torch.Tensor],
                  b: Tuple[torch.Tensor, torch.Tensor],
                  d: torch.Tensor,
                  c: Optional[torch.Tensor] = None,
                  recipe: Optional[Tuple[int, int, int]] = None,
                  compiled_dims: str = "nk",
                  disable_ue8m0_cast: bool = False):
    """e4m3 operands only (reference :44-83)."""
    _dense(a, b, d, "fp8_gemm_hipc", (torch.float8_e4m3fn,))
