"""einsum / fp8_einsum for the three attention-projection contractions of the reference.

Same names, argument order and expressions as the reference's C++ ops
(csrc/arch/gfx938/einsum.cu:157-222): ``einsum(expr, a, b, d, c=None)`` on bf16 tensors with
``"bmk,bnk->mn"``, ``"bhr,hdr->bhd"``, ``"bhd,hdr->bhr"`` and ``fp8_einsum(expr, a, b, d, c=None,
recipe=...)`` on ``(e4m3 tensor, fp32 scale)`` pairs with ``"bhr,hdr->bhd"`` (scales ``[b,h]`` /
``[h,d]``), ``"bhd,hdr->bhr"`` (``[b,h]`` / ``[h,r]``), ``"bhd,bhr->hdr"`` (``[h,d]`` / ``[h,r]``).
Every one is a batched GEMM over the head dimension once the operands are laid out
``[batch, rows, K]``; the reference permutes and calls ``at::bmm`` / its fp8 GEMM (:64-147), here
the GEMM is ``dg_dense_gemm`` on the grouped kernels.  ``d`` is written in place; with ``c`` the
result is ``c + contraction`` (fp32 ``d`` only, as the reference asserts).  K is padded with
zeros to the kernel's granularity (128 for e4m3, 64 for bf16) where needed.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .gemm import _dense

__all__ = ["einsum", "fp8_einsum"]


def _pad_k(x: torch.Tensor, mult: int) -> torch.Tensor:
    k = x.shape[-1]
    if k % mult == 0:
        return x.contiguous()
    out = torch.zeros(x.shape[:-1] + ((k + mult - 1) // mult * mult,), dtype=torch.uint8 if x.element_size() == 1
                      else x.dtype, device=x.device)
    out = out.view(x.dtype) if x.element_size() == 1 else out
    out[..., :k] = x
    return out


def _batched(a, sa, b, sb, out_dtype, where):
    """a [B,M,K], b [B,N,K] (+ per-row scales [B,M] / [B,N] or None) -> [B,M,N]."""
    mult = 64 if a.dtype == torch.bfloat16 else 128
    a, b = _pad_k(a, mult), _pad_k(b, mult)
    out = torch.empty((a.shape[0], a.shape[1], b.shape[1]), dtype=out_dtype, device=a.device)
    empty = torch.empty(0, device=a.device)
    _dense((a, sa.contiguous() if sa is not None else empty), (b, sb.contiguous() if sb is not None else empty),
           out, where, (torch.float8_e4m3fn, torch.bfloat16))
    return out


def _finish(d: torch.Tensor, result: torch.Tensor, c: Optional[torch.Tensor]) -> None:
    if c is not None:
        if d.dtype != torch.float32 or c.dtype != torch.float32:
            raise ValueError("an accumulator c needs fp32 c and d")
        d.copy_(c + result.float())
    else:
        d.copy_(result)


def einsum(expr: str, a: torch.Tensor, b: torch.Tensor, d: torch.Tensor,
           c: Optional[torch.Tensor] = None) -> None:
    """bf16 contractions (reference einsum.cu:157-183)."""
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
        raise ValueError("einsum expects bf16 operands")
    if d.dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("einsum writes bf16 or fp32")
    if 0 in a.shape or 0 in b.shape:
        return
    out_dtype = torch.float32 if d.dtype == torch.float32 else torch.bfloat16
    if expr == "bmk,bnk->mn":
        # sum over the batch of a[b] @ b[b]^T = one GEMM with the batch folded into K
        if (d.dtype == torch.float32) != (c is not None):
            raise ValueError("bmk,bnk->mn: fp32 d needs c, bf16 d takes none (reference einsum.cu:38-43)")
        s, m, k = a.shape
        a2 = a.permute(1, 0, 2).reshape(1, m, s * k)
        b2 = b.permute(1, 0, 2).reshape(1, b.shape[1], s * k)
        _finish(d, _batched(a2, None, b2, None, out_dtype, "einsum")[0], c)
    elif expr == "bhr,hdr->bhd":
        if c is not None:
            raise ValueError("bhr,hdr->bhd takes no accumulator")
        out = _batched(a.permute(1, 0, 2), None, b, None, out_dtype, "einsum")      # [h,b,d]
        d.copy_(out.permute(1, 0, 2))
    elif expr == "bhd,hdr->bhr":
        if c is not None:
            raise ValueError("bhd,hdr->bhr takes no accumulator")
        out = _batched(a.permute(1, 0, 2), None, b.transpose(1, 2), None, out_dtype, "einsum")   # [h,b,r]
        d.copy_(out.permute(1, 0, 2))
    else:
        raise RuntimeError(f"Unsupported einsum expression: {expr}")


def fp8_einsum(expr: str, a: Tuple[torch.Tensor, torch.Tensor], b: Tuple[torch.Tensor, torch.Tensor],
               d: torch.Tensor, c: Optional[torch.Tensor] = None,
               recipe: Tuple[int, int, int] = (1, 128, 128)) -> None:
    """e4m3 contractions with per-row scales (reference einsum.cu:185-222)."""
    (qa, sa), (qb, sb) = a, b
    if qa.dtype != torch.float8_e4m3fn or qb.dtype != torch.float8_e4m3fn:
        raise ValueError("fp8_einsum expects e4m3 operands")
    if d.dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("fp8_einsum writes bf16 or fp32")
    if 0 in qa.shape or 0 in qb.shape:
        return
    out_dtype = torch.float32 if d.dtype == torch.float32 else torch.bfloat16
    if expr == "bhr,hdr->bhd":      # A [h,b,r] scale [h,b]; B [h,d,r] scale [h,d]
        out = _batched(qa.permute(1, 0, 2), sa.permute(1, 0), qb, sb, out_dtype, "fp8_einsum")
        _finish(d, out.permute(1, 0, 2), c)
    elif expr == "bhd,hdr->bhr":    # A [h,b,d] scale [h,b]; B [h,r,d] scale [h,r]
        out = _batched(qa.permute(1, 0, 2), sa.permute(1, 0), qb.permute(0, 2, 1), sb, out_dtype,
                       "fp8_einsum")
        _finish(d, out.permute(1, 0, 2), c)
    elif expr == "bhd,bhr->hdr":    # A [h,d,b] scale [h,d]; B [h,r,b] scale [h,r]; K = b
        out = _batched(qa.permute(1, 2, 0), sa, qb.permute(1, 2, 0), sb, out_dtype, "fp8_einsum")
        _finish(d, out, c)
    else:
        raise RuntimeError(f"Unsupported einsum expression: {expr}")
