"""CPU oracle for the grouped MoE GEMM path -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.

A restatement, in plain torch CPU ops, of the dequant-matmul references that the
HYGON-AI/deepgemm-das test scripts compare their GPU kernels with.  Only tests/,
__graft_entry__.smoke() and bench.py's CPU-baseline / reference arm may import this module;
the shipped package never does.

Parity pin: tests/golden/*.npz holds inputs and outputs produced by the reference's own
helper functions (imported from its op_test/ directory by tests/golden/make_golden.py);
tests/test_oracle.py checks every function here against them bit for bit.

Every function names the reference lines it follows (paths inside the reference tree).
"""
from __future__ import annotations

from typing import Optional, Tuple

import numpy as np
import torch

FP8 = torch.float8_e4m3fn
FP8_MAX = 448.0


# ----------------------------------------------------------------------------- quantisers
def per_token_quant_int8(x: torch.Tensor, eps: float = 1e-10) -> Tuple[torch.Tensor, torch.Tensor]:
    """Symmetric per-row int8 quantisation; op_test/quant_utils.py:4-19.
    scale = absmax/127 (keepdim), q = round(x * (127/absmax)) clamped to [-128,127]."""
    xf = x.float()
    absmax = xf.abs().amax(dim=-1, keepdim=True).clamp_min(eps)
    scale = absmax / 127.0
    q = torch.round(xf * (127.0 / absmax)).clamp(-128, 127).to(torch.int8)
    return q.contiguous(), scale.contiguous()


def per_token_quant_fp8(x: torch.Tensor, eps: float = 1e-10) -> Tuple[torch.Tensor, torch.Tensor]:
    """Symmetric per-row e4m3 quantisation with scale = absmax/448.  The reference has no such
    helper (its FP8 tests cast small integers); this mirrors per_token_quant_int8's structure
    with the e4m3 maximum, as the benchmark configurations specify."""
    xf = x.float()
    absmax = xf.abs().amax(dim=-1, keepdim=True).clamp_min(eps)
    scale = absmax / FP8_MAX
    q = (xf * (FP8_MAX / absmax)).clamp(-FP8_MAX, FP8_MAX).to(FP8)
    return q.contiguous(), scale.contiguous()


def to_int8(t: torch.Tensor) -> torch.Tensor:
    """op_test/masked_w8a8_int8_common.py:25-26."""
    return torch.round(t.clamp(min=-128, max=127)).to(torch.int8)


# ----------------------------------------------------------------------------- int4
def unpack_int4_to_int8_x16(packed: torch.Tensor, nibble_order: str = "high_first") -> torch.Tensor:
    """Framework int4 bytes [E,N,K/2] -> int8 [E,N,K] holding 16 * (signed nibble): the value
    the W4A8 kernels multiply by.  op_test/test_deepgemm_masked_w4a8.py:19-30 (high nibble =
    even k).  `low_first` swaps the two nibbles of each byte first."""
    p = packed.view(torch.uint8).to(torch.int16)
    high = (p & 0xF0)
    low = ((p << 4) & 0xF0)
    first, second = (high, low) if nibble_order == "high_first" else (low, high)
    e, n, kh = packed.shape
    out = torch.empty((e, n, kh * 2), dtype=torch.int16)
    out[..., 0::2] = first
    out[..., 1::2] = second
    out = torch.where(out > 127, out - 256, out)  # reinterpret the byte as int8
    return out.to(torch.int8)


def signed_int4(u4: torch.Tensor) -> torch.Tensor:
    """Unsigned nibble 0..15 -> signed -8..7; op_test/test_deepgemm_masked_w4a8_hipc.py:77."""
    u = u4.to(torch.int16) & 0xF
    return torch.where(u > 7, u - 16, u).to(torch.int8)


# ----------------------------------------------------------------------------- masked references
def _f32(t: torch.Tensor) -> torch.Tensor:
    return t.detach().cpu().to(torch.float32)


def ref_masked_scaled(a: torch.Tensor, b: torch.Tensor, a_scale: torch.Tensor,
                      b_scale: torch.Tensor, out_dtype=torch.bfloat16) -> torch.Tensor:
    """Per-token x per-channel masked reference, all rows computed (callers compare rows below
    masked_m only).  a [E,M,K], b [E,N,K] (int8 or e4m3, row-major), a_scale [E,M,1],
    b_scale [E,N,1].  op_test/masked_w8a8_int8_common.py:55-69,
    op_test/test_deepgemm_masked_w8a8_fp8.py:15-34: fp32 bmm, then a_scale * c * b_scale^T."""
    c = torch.bmm(_f32(a), _f32(b).transpose(1, 2))
    e, m, _ = a.shape
    n = b.shape[1]
    c = _f32(a_scale).reshape(e, m, 1) * c * _f32(b_scale).reshape(e, n, 1).transpose(1, 2)
    return c.to(out_dtype)


def ref_masked_tensor_wise(a: torch.Tensor, b: torch.Tensor, a_scale: torch.Tensor,
                           b_scale: torch.Tensor, out_dtype=torch.bfloat16) -> torch.Tensor:
    """One weight scale per expert; op_test/test_deepgemm_masked_w8a8_fp8_tensor_wise.py:15-33:
    input_scale * C * weight_scale.view(-1,1,1)."""
    c = torch.bmm(_f32(a), _f32(b).transpose(1, 2))
    e, m, _ = a.shape
    c = _f32(a_scale).reshape(e, m, 1) * c * _f32(b_scale).reshape(-1, 1, 1)
    return c.to(out_dtype)


def ref_masked_bf16(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """op_test/test_deepgemm_masked_w16a16_bf16.py:74: fp32 matmul per expert -> bf16."""
    return torch.bmm(_f32(a), _f32(b).transpose(1, 2)).to(torch.bfloat16)


def ref_masked_w4a8(a: torch.Tensor, packed_b: torch.Tensor, a_scale: torch.Tensor,
                    b_scale: torch.Tensor, nibble_order: str = "high_first") -> torch.Tensor:
    """op_test/test_deepgemm_masked_w4a8.py:19-45: weights unpacked with the nibble in the high
    4 bits (16 x value), then the per-channel reference; b_scale already carries the 1/16."""
    return ref_masked_scaled(a, unpack_int4_to_int8_x16(packed_b, nibble_order), a_scale, b_scale)


def ref_masked_w4a8_hipc(a: torch.Tensor, packed_b: torch.Tensor, a_scale: torch.Tensor,
                         w_scale: torch.Tensor, out_dtype=torch.bfloat16,
                         nibble_order: str = "high_first") -> torch.Tensor:
    """op_test/test_deepgemm_masked_w4a8_hipc.py:63-82: nibbles read as two's complement
    (`where(u4 > 7, u4 - 16, u4)`), `ref = bmm(a.float(), w.float()^T) * a_scale * w_scale^T`; the
    kernel under test receives `w_scale / 16` and multiplies by 16 x the nibble.  `packed_b` is
    the framework layout [E, N, K/2]; a_scale [E, M, 1], w_scale [E, N, 1]."""
    w = (unpack_int4_to_int8_x16(packed_b, nibble_order).to(torch.int16) // 16).to(torch.float32)
    ref = torch.bmm(_f32(a), w.transpose(1, 2))
    return (ref * a_scale * w_scale.transpose(1, 2)).to(out_dtype)


def ref_contiguous_w4a8_hipc(a: torch.Tensor, packed_b: torch.Tensor, a_scale: torch.Tensor,
                             w_scale: torch.Tensor, m_indices: torch.Tensor, out_dtype=torch.bfloat16,
                             nibble_order: str = "high_first") -> torch.Tensor:
    """op_test/test_deepgemm_contiguous_w4a8_hipc.py:70-76: per expert `acc = a[rows].float() @
    w.float().t(); acc * a_scale[rows] * w_scale[e].t()`, rows with m_indices < 0 left zero."""
    w = (unpack_int4_to_int8_x16(packed_b, nibble_order).to(torch.int16) // 16).to(torch.float32)
    ref = torch.zeros((a.shape[0], w.shape[1]), dtype=torch.float32)
    for e in range(w.shape[0]):
        rows = m_indices == e
        acc = _f32(a[rows]) @ w[e].t()
        ref[rows] = acc * _f32(a_scale[rows]) * _f32(w_scale[e]).t()
    return ref.to(out_dtype)


# ----------------------------------------------------------------------------- contiguous references
def ref_contiguous(a: torch.Tensor, b: torch.Tensor, a_scale: torch.Tensor, b_scale: torch.Tensor,
                   m_indices: torch.Tensor, out_dtype=torch.bfloat16,
                   tensor_wise: bool = False) -> torch.Tensor:
    """a [M,K], b [E,N,K], a_scale [M] or [M,1], b_scale [E,N(,1)] or (tensor-wise) [E(,1)],
    m_indices [M] (-1 = padding row, left zero).  op_test/contiguous_w8a8_int8_common.py:73-109,
    op_test/test_deepgemm_contiguous_w8a8_fp8.py:77-112: per expert fp32 matmul, times the row
    scale, times the column scale; tensor-wise form
    op_test/test_deepgemm_contiguous_w8a8_fp8_tensor_wise.py:72-99."""
    af, bf = _f32(a), _f32(b)
    sa = _f32(a_scale).reshape(-1)
    sb = _f32(b_scale)
    idx = m_indices.detach().cpu().to(torch.long)
    m, n = a.shape[0], b.shape[1]
    out = torch.zeros((m, n), dtype=out_dtype)
    for e in range(b.shape[0]):
        rows = torch.nonzero(idx == e, as_tuple=False).flatten()
        if rows.numel() == 0:
            continue
        o = af.index_select(0, rows).matmul(bf[e].t())
        o = o * sa.index_select(0, rows).view(-1, 1)
        o = o * (sb.reshape(-1)[e] if tensor_wise else sb[e].reshape(1, -1))
        out[rows] = o.to(out_dtype)
    return out


# ----------------------------------------------------------------------------- exact accumulators
def exact_int_acc(a_rows: torch.Tensor, b_rows: torch.Tensor) -> torch.Tensor:
    """Exact sum_k a[m,k]*b[n,k] for int8 operands as int32 [M,N] (float64 matmul is exact:
    |acc| <= K*128*128 << 2^53).  The fp32 matmul of the references above is only exact while
    partial sums stay below 2^24, so bit-exactness of the kernels' int32 accumulators is
    checked against this function instead."""
    acc = a_rows.detach().cpu().to(torch.float64).matmul(b_rows.detach().cpu().to(torch.float64).t())
    return acc.to(torch.int64).to(torch.int32)


def epilogue_from_acc(acc: torch.Tensor, a_scale_rows: torch.Tensor, b_scale_cols) -> torch.Tensor:
    """bf16( (float32(acc) * a_scale[row]) * b_scale[col] ), the order every reference uses
    (a_scale * c * w_scale^T evaluates left to right).  acc int32 or float32 [M,N]."""
    c = acc.to(torch.float32)
    c = c * _f32(a_scale_rows).reshape(-1, 1)
    if torch.is_tensor(b_scale_cols):
        c = c * _f32(b_scale_cols).reshape(1, -1)
    else:
        c = c * torch.tensor(float(b_scale_cols), dtype=torch.float32)
    return c.to(torch.bfloat16)


# ----------------------------------------------------------------------------- comparison helpers
def calc_diff(x: torch.Tensor, y: torch.Tensor) -> float:
    """1 - 2*sum(x*y)/sum(x^2+y^2) (DeepGEMM's similarity measure), in float64."""
    xd, yd = x.detach().cpu().double(), y.detach().cpu().double()
    denom = (xd * xd + yd * yd).sum()
    if float(denom) == 0.0:
        return 0.0
    return float(1.0 - 2.0 * (xd * yd).sum() / denom)


def bf16_ulp_distance(x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """Distance in units of bf16 representable steps between two bf16 tensors (int64)."""
    def ordered(t):
        bits = t.detach().cpu().contiguous().view(torch.int16).to(torch.int64) & 0xFFFF
        return torch.where(bits >= 0x8000, 0x8000 - bits, bits)  # sign-magnitude -> ordered
    return (ordered(x) - ordered(y)).abs()


# ----------------------------------------------------------------------------- layout helpers
def build_contiguous_layout(rows_per_group, align: int = 256) -> Tuple[torch.Tensor, int]:
    """m_indices for groups padded to `align` rows with -1 on padding rows
    (op_test/contiguous_w8a8_int8_common.py:38-62).  Returns (m_indices int32 [M_total], M_total)."""
    chunks = []
    for g, m in enumerate(rows_per_group):
        m = int(m)
        padded = ((m + align - 1) // align) * align
        chunks.append(torch.full((m,), g, dtype=torch.int32))
        chunks.append(torch.full((padded - m,), -1, dtype=torch.int32))
    idx = torch.cat(chunks) if chunks else torch.zeros((0,), dtype=torch.int32)
    return idx, int(idx.numel())


def topk_routing_counts(num_tokens: int, num_experts: int, top_k: int,
                        gen: torch.Generator, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Tokens per expert when each token picks top_k distinct experts by random score."""
    scores = torch.rand(num_tokens, num_experts, generator=gen) if bias is None else \
        torch.randn(num_tokens, num_experts, generator=gen) + bias
    picks = scores.topk(top_k, dim=1).indices.flatten()
    return torch.bincount(picks, minlength=num_experts)


# ----------------------------------------------------------------------------- MoE layer chain
def ref_silu_mul(x: torch.Tensor) -> torch.Tensor:
    """bf16 [.., 2H] (gate | up) -> bf16 [.., H], the unfused bf16 computation
    ``silu(gate) * up``: silu evaluated in fp32 and rounded to bf16, then the product rounded to
    bf16.  The reference has no such function (its second-stage op takes activated rows,
    deepgemm/moe_marlin_prefill.py:15-56); this defines what the fused kernel must produce."""
    h = x.shape[-1] // 2
    g, u = x[..., :h].float(), x[..., h:].float()
    s = (g / (1.0 + torch.exp(-g))).bfloat16().float()
    return (s * u).bfloat16()


def ref_combine(y: torch.Tensor, src_row: torch.Tensor, weights: Optional[torch.Tensor]) -> torch.Tensor:
    """out[t] = sum_j weights[t, j] * y[src_row[t, j]] in float64 (rounded to bf16 by the caller's
    comparison); negative / out-of-range rows contribute nothing.  The routing-weight multiply is
    the one at csrc/include/moe_marlin/moe_marlin_prefill_down_fp8_device.inc.h:114-119."""
    t, k = src_row.shape
    out = torch.zeros(t, y.shape[1], dtype=torch.float64)
    for j in range(k):
        ok = (src_row[:, j] >= 0) & (src_row[:, j] < y.shape[0])
        rows = y[src_row[:, j].clamp(0, max(y.shape[0] - 1, 0)).long()].double()
        w = weights[:, j].double() if weights is not None else torch.ones(t, dtype=torch.float64)
        out += torch.where(ok[:, None], rows * w[:, None], torch.zeros_like(rows))
    return out


def ref_moe_layer(hidden: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor,
                  w13: torch.Tensor, w13_scale: torch.Tensor, w2: torch.Tensor, w2_scale: torch.Tensor,
                  kind: str = "fp8") -> torch.Tensor:
    """One MoE layer with quantised experts, step by step with the reference formulas: per-token
    quantise (op_test/quant_utils.py:4-19) -> dequant-matmul (masked_w8a8_int8_common.py:55-69)
    -> silu*mul -> per-token quantise -> dequant-matmul -> weighted top-k sum.  float64 result."""
    quant = per_token_quant_fp8 if kind == "fp8" else per_token_quant_int8
    qa, sa = quant(hidden)
    t, k = topk_ids.shape
    y = torch.zeros(t * k, w2.shape[1], dtype=torch.bfloat16)
    for e in range(w13.shape[0]):
        pairs = torch.nonzero(topk_ids.reshape(-1) == e).flatten()
        if pairs.numel() == 0:
            continue
        tok = pairs // k
        h13 = ((qa[tok].float() @ w13[e].float().t()) * sa[tok].reshape(-1, 1) * w13_scale[e].reshape(1, -1)).bfloat16()
        q, s = quant(ref_silu_mul(h13))
        y[pairs] = ((q.float() @ w2[e].float().t()) * s.reshape(-1, 1) * w2_scale[e].reshape(1, -1)).bfloat16()
    src = torch.arange(t * k, dtype=torch.int32).view(t, k)
    return ref_combine(y, src, topk_weights)


# ----------------------------------------------------------------------------- dense GEMM
def ref_dense_scaled(a: torch.Tensor, b: torch.Tensor, scale_a: Optional[torch.Tensor],
                     scale_b: Optional[torch.Tensor], out_dtype=torch.bfloat16) -> torch.Tensor:
    """a [M,K], b [N,K], scale_a [M], scale_b [N] -> [M,N]; op_test/test_fp8_gemm.py:31-39
    (operands are scaled first, then one fp32 matmul); identity scales as in
    op_test/test_fp8_gemm_hipc.py:96-101 when a scale is None."""
    a_fp = a.to(torch.float32)
    b_fp = b.to(torch.float32).t()
    if scale_a is not None:
        a_fp = a_fp * scale_a.view(-1, 1)
    if scale_b is not None:
        b_fp = b_fp * scale_b.view(1, -1)
    return torch.matmul(a_fp, b_fp).to(out_dtype)


# ----------------------------------------------------------------------------- second-stage MoE GEMM
def build_sorted_routing(topk_ids: torch.Tensor, num_experts: int, block_m: int,
                         local_experts=None, extra_blocks: int = 0):
    """The routing list the reference's second-stage op consumes (what aiter / vLLM's
    moe_align_block_size produces): entries ``slot << 24 | token`` sorted by expert, each
    expert's run padded to a multiple of block_m with ``top_k << 24 | T`` (an invalid slot),
    one expert id per block (-1 for experts outside ``local_experts``), the number of entries
    in use, plus ``extra_blocks`` unused blocks of padding at the end."""
    t, k = topk_ids.shape
    ids, experts = [], []
    pad = (k << 24) | t
    for e in range(num_experts):
        pairs = torch.nonzero(topk_ids == e)
        if pairs.numel() == 0:
            continue
        run = [(int(s) << 24) | int(tok) for tok, s in pairs.tolist()]
        run += [pad] * (-len(run) % block_m)
        ids += run
        local = local_experts is None or e in local_experts
        experts += [e if local else -1] * (len(run) // block_m)
    used = len(ids)
    ids += [pad] * (extra_blocks * block_m)
    experts += [0] * extra_blocks
    return (torch.tensor(ids, dtype=torch.int32), torch.tensor(experts, dtype=torch.int32),
            torch.tensor([used], dtype=torch.int32))


def ref_prefill_down(inp: torch.Tensor, w: torch.Tensor, a_scale: torch.Tensor, b_scale: torch.Tensor,
                     topk_weights: torch.Tensor, sorted_token_ids: torch.Tensor, expert_ids: torch.Tensor,
                     num_tokens_post_pad: torch.Tensor, real_topk: int, out: torch.Tensor) -> torch.Tensor:
    """Block by block as the reference kernel walks the list
    (csrc/include/moe_marlin/moe_marlin_prefill_down_fp8_device.inc.h): a block is skipped when
    it starts at or beyond num_tokens_post_pad or its first entry has slot >= real_topk (:58-59);
    expert -1 writes zeros (:137-156); otherwise row = token * real_topk + slot gets
    bf16(acc * (topk_weight[row] * a_scale[row]) * b_scale[e][n]) (:114-119, :262-272).
    inp [size_m, K] int8 / e4m3, w [E, N, K], out bf16 [size_m, N] updated in place."""
    block_m = sorted_token_ids.numel() // expert_ids.numel()
    size_m = inp.shape[0]
    for blk in range(expert_ids.numel()):
        ids = sorted_token_ids[blk * block_m:(blk + 1) * block_m].to(torch.int64) & 0xFFFFFFFF
        if blk * block_m >= int(num_tokens_post_pad[0]) or int(ids[0] >> 24) >= real_topk:
            continue
        slot, tok = ids >> 24, ids & 0xFFFFFF
        row = tok * real_topk + slot
        keep = (slot < real_topk) & (row < size_m)
        row = row[keep]
        e = int(expert_ids[blk])
        if e < 0:
            out[row] = 0
            continue
        acc = inp[row].float().double() @ w[e].float().double().t()
        scale = (topk_weights.reshape(-1)[row] * a_scale.reshape(-1)[row]).float()
        out[row] = ((acc.float() * scale[:, None]) * b_scale[e].reshape(1, -1).float()).bfloat16()
    return out
