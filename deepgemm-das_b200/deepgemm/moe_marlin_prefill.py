"""Second-stage MoE GEMM on a vLLM-style routing list.

Same name, argument order and checks as the reference's ``deepgemm/moe_marlin_prefill.py``
(:15-56, C++ side csrc/arch/gfx938/moe_w8a8_marlin_prefill_down_fp8.cu:27-110):

    output[row] = bf16( (input[row] @ W[e]^T) * (topk_weights[row] * a_scale[row]) * b_scale[e] )

for every ``row = token * real_topk + slot`` named by ``sorted_token_ids`` (``slot << 24 | token``,
blocks of ``len(sorted_token_ids) / len(expert_ids)`` entries per expert), zeros for rows whose
block has ``expert_ids == -1``; rows the list never names are left untouched, as in the
reference.  Like the reference's kernel, which gathers its 32-row blocks itself, the GEMM does the
gathering: ``dg_sorted_gemm`` tiles every expert's run of the list into 128 entries, its producer
warp fetches the rows of a tile by index and its epilogue writes each result row to its place
(and zeros for absent experts): one launch, no allocation, no pass over the operands or the
result.  Large problems with many rows per expert (where two-CTA 256 x 256 tiles pay) take two
steps instead: ``dg_group_sorted_rows`` regroups the rows into 128-row blocks per expert in a
workspace kept per problem size, and the contiguous grouped GEMM scatters the result rows from
its epilogue (``scatter_tag``).  Both give the same bytes.  ``b_qweight`` must come from
``marlin_fp8_contiguous_weight`` / ``marlin_i8_contiguous_weight`` of this package.
"""
from __future__ import annotations


import torch

from . import _cabi, _core
from .print_size import PRINT_SIZE_ENABLED, describe
from .quant_group import quant_group_capacity

__all__ = ["moe_w8a8_marlin_prefill_down_fp8", "assert_moe_prefill_down_fp8_shapes"]

_MOE_N_ALIGN = 512  # the reference's tile needs it; kept so that callers' checks behave the same


def _impl(input, b_qweight, output, a_scale, b_scale, topk_weights, sorted_token_ids, expert_ids,
          num_tokens_post_pad, top_k, real_topk):
    if input.element_size() != 1 or b_qweight.element_size() != 1:
        raise RuntimeError("input and weight must be 1-byte (fp8_e4m3 or int8)")
    if output.dtype != torch.bfloat16:
        raise RuntimeError("output bf16")
    if a_scale.dtype != torch.float32 or b_scale.dtype != torch.float32:
        raise RuntimeError("scales float32")
    if topk_weights.dtype != torch.float32:
        raise RuntimeError("topk_weights float32")
    for t, name in ((sorted_token_ids, "sorted_token_ids"), (expert_ids, "expert_ids"),
                    (num_tokens_post_pad, "num_tokens_post_pad")):
        if t.dtype != torch.int32:
            raise RuntimeError(f"{name} int32")
    if b_qweight.dim() != 4:
        raise RuntimeError("b_qweight must be the packed [E, K/128, N, 128] weight of this package")
    if a_scale.dim() not in (1, 2):
        raise RuntimeError("a_scale must be 1-D [M] or 2-D [M, 1]")
    if b_scale.dim() not in (2, 3):
        raise RuntimeError("b_scale must be 2-D [E, N] or 3-D [E, N, 1]")
    size_m, size_k = int(input.shape[0]), int(input.shape[1])
    size_n = int(output.shape[-1])
    if size_k % 64 != 0:
        raise RuntimeError(f"moe_marlin_prefill_down_fp8: size_k={size_k} must be a multiple of 64")
    experts = int(b_scale.shape[0])
    em, blocks = int(sorted_token_ids.numel()), int(expert_ids.numel())
    if blocks == 0 or em % blocks != 0:
        raise RuntimeError("sorted_token_ids must hold a whole number of blocks per expert_ids entry")
    if output.numel() != size_m * size_n or topk_weights.numel() < size_m or a_scale.numel() < size_m:
        raise RuntimeError("output, topk_weights and a_scale must have one row per row of input")
    dev = input.device
    kind = _cabi.KIND_E4M3 if input.dtype == torch.float8_e4m3fn else _cabi.KIND_I8
    path = FORCE_PATH or ("regroup" if _two_cta_tiles_pay(em, experts, size_n) else "gather")
    if path == "gather":
        if not (input.is_contiguous() and output.is_contiguous()):
            raise RuntimeError("input and output must be contiguous")
        args = _cabi.SortedGemmArgs(
            kind=kind, num_groups=experts, a=input.data_ptr(), b_packed=b_qweight.data_ptr(),
            d=output.data_ptr(), a_scale=a_scale.contiguous().data_ptr(),
            row_weight=topk_weights.contiguous().data_ptr(),
            b_scale=b_scale.reshape(experts, size_n).contiguous().data_ptr(),
            sorted_token_ids=sorted_token_ids.contiguous().data_ptr(),
            expert_ids=expert_ids.contiguous().data_ptr(),
            num_tokens_post_pad=num_tokens_post_pad.contiguous().data_ptr(),
            num_sorted=em, num_blocks=blocks, block_m=em // blocks, size_m=size_m, real_topk=int(real_topk),
            n=size_n, k=size_k, reserved=0, status=_core.device_status_words(dev).data_ptr())
        _core._launch(_cabi.lib.dg_sorted_gemm, args, dev, "dg_sorted_gemm")
        return output
    m_cap = quant_group_capacity(em, experts, 128)
    ws = _workspace(dev, m_cap, size_k, em, experts, input.dtype)
    out2d = output.view(size_m, size_n)
    args = _cabi.GroupSortedArgs(
        num_sorted=em, block_m=em // blocks, size_m=size_m, hidden=size_k, num_groups=experts, align=128,
        m_cap=m_cap, real_topk=int(real_topk), rows=input.data_ptr(),
        row_scale=a_scale.contiguous().data_ptr(), row_weight=topk_weights.contiguous().data_ptr(),
        sorted_token_ids=sorted_token_ids.contiguous().data_ptr(),
        expert_ids=expert_ids.contiguous().data_ptr(),
        num_tokens_post_pad=num_tokens_post_pad.contiguous().data_ptr(),
        a_out=ws["a"].data_ptr(), a_scale_out=ws["a_s"].data_ptr(), m_indices_out=ws["m_idx"].data_ptr(),
        dest_out=None, m_total_out=None, scratch=ws["scratch"].data_ptr(),
        scratch_bytes=ws["scratch"].numel(), src_out=ws["src"].data_ptr(),
        zero_rows=out2d.data_ptr(), zero_row_bytes=size_n * 2, reserved=0)
    _core._launch(_cabi.lib.dg_group_sorted_rows, args, dev, "dg_group_sorted_rows")
    # the GEMM's epilogue writes result row i straight to output[src[i]] (tag = buffer 0, row src[i])
    _core.grouped_gemm_contiguous(kind, _cabi.SCALE_PER_CHANNEL, ws["a"], b_qweight, out2d, ws["a_s"],
                                  b_scale.reshape(experts, size_n), ws["m_idx"],
                                  scatter=(ws["src"], _cabi.pointer_array([out2d.data_ptr()]), 1))
    return output


# None: choose by size; "gather" / "regroup": tests pin one of the two paths
FORCE_PATH = None


def _two_cta_tiles_pay(em: int, experts: int, size_n: int) -> bool:
    """The rule of the contiguous GEMM's tile choice: 256 x 256 two-CTA tiles from about 320
    routed rows per expert upwards, when there are at least two of them for every SM pair."""
    return em // max(experts, 1) >= 320 and (em // 256) * (size_n // 256) >= 148


_WORKSPACES = {}


def _workspace(dev, m_cap, size_k, em, experts, dtype):
    """The regrouped operand, its scales and index arrays: allocated on the first call for a
    problem size and kept, so that steady-state calls allocate nothing."""
    key = (dev.index, m_cap, size_k, em, experts, dtype)
    ws = _WORKSPACES.get(key)
    if ws is None:
        need = int(_cabi.lib.dg_quant_group_scratch_bytes(em, experts))
        ws = {"a": torch.empty((m_cap, size_k), dtype=dtype, device=dev),
              "a_s": torch.empty((m_cap,), dtype=torch.float32, device=dev),
              "m_idx": torch.empty((m_cap,), dtype=torch.int32, device=dev),
              "src": torch.zeros((m_cap,), dtype=torch.int32, device=dev),
              "scratch": torch.empty((max(need, 16),), dtype=torch.uint8, device=dev)}
        if len(_WORKSPACES) >= 8:          # a handful of layer shapes at most; drop the oldest
            _WORKSPACES.pop(next(iter(_WORKSPACES)))
        _WORKSPACES[key] = ws
    return ws


_lib = torch.library.Library("deep_gemm", "FRAGMENT")
_lib.define("moe_w8a8_marlin_prefill_down_fp8(Tensor input, Tensor b_qweight, Tensor(a!) output, "
            "Tensor a_scale, Tensor b_scale, Tensor topk_weights, Tensor sorted_token_ids, "
            "Tensor expert_ids, Tensor num_tokens_post_pad, int top_k, int real_topk) -> Tensor(a!)")
_lib.impl("moe_w8a8_marlin_prefill_down_fp8", _impl, "CUDA")


def moe_w8a8_marlin_prefill_down_fp8(
    input: torch.Tensor,
    b_qweight: torch.Tensor,
    output: torch.Tensor,
    a_scale: torch.Tensor,
    b_scale: torch.Tensor,
    topk_weights: torch.Tensor,
    sorted_token_ids: torch.Tensor,
    expert_ids: torch.Tensor,
    num_tokens_post_pad: torch.Tensor,
    top_k: int,
    real_topk: int,
) -> torch.Tensor:
    """MoE second-stage GEMM (activations x packed expert weights -> bf16), reference :15-56."""
    if PRINT_SIZE_ENABLED:
        print("[DeepGEMM][size]", "moe_w8a8_marlin_prefill_down_fp8",
              *(f"{n}={describe(v)}" for n, v in (
                  ("input", input), ("b_qweight", b_qweight), ("output", output), ("a_scale", a_scale),
                  ("b_scale", b_scale), ("topk_weights", topk_weights),
                  ("sorted_token_ids", sorted_token_ids), ("expert_ids", expert_ids),
                  ("num_tokens_post_pad", num_tokens_post_pad), ("top_k", top_k), ("real_topk", real_topk))))
    return torch.ops.deep_gemm.moe_w8a8_marlin_prefill_down_fp8(
        input, b_qweight, output, a_scale, b_scale, topk_weights, sorted_token_ids, expert_ids,
        num_tokens_post_pad, top_k, real_topk)


def assert_moe_prefill_down_fp8_shapes(*, k: int, n: int) -> None:
    """Reference :59-66 (kept: callers use it to validate model shapes)."""
    if k % 64 != 0:
        raise ValueError(f"K={k} must be a multiple of 64 for prefill-down FP8")
    if n % _MOE_N_ALIGN != 0:
        raise ValueError(f"N={n} must be divisible by {_MOE_N_ALIGN} for tile <32,128,64,32,32,64,2>")
