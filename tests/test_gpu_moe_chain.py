"""The memory-bound steps between and after the two grouped GEMMs (SiLU*up + requantise,
weighted top-k combine) and the whole MoE layer, against the CPU oracle.

Tolerances (floating point): the activation is rounded to bf16 twice exactly as the oracle
does, but expf on the GPU and exp on the CPU may differ in the last fp32 bit, which can move a
bf16 rounding; so scales must agree to 2^-7 relative and dequantised values to 1.01 quantisation
steps, with at least 99.9 % of the quantised bytes identical.  The combine result must be within
1 bf16 ulp of the float64 sum.  The layer is judged by calc_diff < 1e-3."""
import pytest
import torch

import deepgemm
from deepgemm.moe_chain import combine_rows, moe_forward, silu_mul_quant

import dg_oracle as O
from helpers import assert_bf16_within_ulp, assert_calc_diff

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _check_act_rows(q, s, x_rows, kind):
    act = O.ref_silu_mul(x_rows).float()
    want_q, want_s = (O.per_token_quant_fp8 if kind == "fp8" else O.per_token_quant_int8)(act)
    want_s = want_s.reshape(-1)
    assert torch.all((s - want_s).abs() <= want_s * 2.0 ** -7), "row scales differ"
    got = q.float() * s[:, None]
    want = want_q.float() * want_s[:, None]
    step = want_s[:, None] * (1.0 if kind == "int8" else 32.0)       # e4m3 spacing near 448 is 32
    assert torch.all((got - want).abs() <= 1.01 * step), "dequantised activations differ by more than a step"
    same = (q.view(torch.uint8) == want_q.view(torch.uint8)).float().mean().item()
    assert same >= 0.999, f"only {same:.5f} of the quantised bytes match the oracle"


@pytest.mark.parametrize("kind", ["fp8", "int8"])
@pytest.mark.parametrize("rows,h", [(300, 2048), (64, 16384), (17, 8)])
def test_silu_mul_quant_contiguous(kind, rows, h):
    gen = torch.Generator().manual_seed(rows + h)
    x = (torch.randn(rows, 2 * h, generator=gen) * 2).bfloat16()
    x[3] = 0                                                      # all-zero row: absmax clamps to eps
    m_idx = torch.randint(0, 4, (rows,), generator=gen).to(torch.int32)
    m_idx[::7] = -1                                               # padding rows are skipped
    q, s = silu_mul_quant(x.to(DEV), kind=kind, m_indices=m_idx.to(DEV))
    torch.cuda.synchronize()
    q, s = q.cpu(), s.cpu()
    keep = m_idx >= 0
    _check_act_rows(q[keep], s[keep], x[keep], kind)
    assert torch.all(q[~keep].view(torch.uint8) == 0) and torch.all(s[~keep] == 0), "skipped rows were written"


def test_silu_mul_quant_masked_layout_and_given_outputs():
    gen = torch.Generator().manual_seed(9)
    g, max_m, h = 5, 24, 512
    x = torch.randn(g, max_m, 2 * h, generator=gen).bfloat16()
    mm = torch.tensor([0, 24, 7, 1, 13], dtype=torch.int32)
    q = torch.full((g, max_m, h), 77, dtype=torch.int8, device=DEV)
    s = torch.full((g, max_m), -1.0, dtype=torch.float32, device=DEV)
    rq, rs = silu_mul_quant(x.to(DEV), kind="int8", masked_m=mm.to(DEV), out=(q, s))
    assert rq is q and rs is s
    q, s = q.cpu(), s.cpu()
    for e in range(g):
        m = int(mm[e])
        if m:
            _check_act_rows(q[e, :m], s[e, :m], x[e, :m], "int8")
        assert torch.all(q[e, m:] == 77) and torch.all(s[e, m:] == -1.0)


def test_silu_mul_quant_rejects_bad_arguments():
    x = torch.zeros(4, 64, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(ValueError):
        silu_mul_quant(x.float())
    with pytest.raises(ValueError):
        silu_mul_quant(x, kind="int4")
    with pytest.raises(ValueError):
        silu_mul_quant(x, m_indices=torch.zeros(3, dtype=torch.int32, device=DEV))
    with pytest.raises(RuntimeError):
        silu_mul_quant(x.cpu())
    with pytest.raises(RuntimeError):                         # H = 20 is not a multiple of 8
        silu_mul_quant(torch.zeros(4, 40, dtype=torch.bfloat16, device=DEV))


@pytest.mark.parametrize("t,k,n,weighted", [(100, 8, 512, True), (33, 2, 7168, True), (5, 1, 8, False)])
def test_combine_rows(t, k, n, weighted):
    gen = torch.Generator().manual_seed(t + n)
    rows = t * k + 9
    y = torch.randn(rows, n, generator=gen).bfloat16()
    src = torch.randperm(rows, generator=gen)[: t * k].view(t, k).to(torch.int32)
    src[0, 0] = -1                                            # a dropped pair
    if k > 1:
        src[1, 1] = rows + 5                                  # out of range counts as dropped
    w = torch.rand(t, k, generator=gen) if weighted else None
    out = combine_rows(y.to(DEV), src.to(DEV), w.to(DEV) if weighted else None).cpu()
    ref = O.ref_combine(y, src, w)
    assert_bf16_within_ulp(out, ref.float().bfloat16(), 1, "combine")


@pytest.mark.parametrize("kind", ["fp8", "int8"])
def test_whole_layer_matches_the_oracle(kind):
    gen = torch.Generator().manual_seed(21)
    t, k, e, hid, inter = 96, 4, 6, 512, 256
    hidden = torch.randn(t, hid, generator=gen).bfloat16()
    topk_ids = torch.rand(t, e, generator=gen).topk(k, dim=1).indices
    topk_w = torch.softmax(torch.randn(t, k, generator=gen), dim=1)
    quant = O.per_token_quant_fp8 if kind == "fp8" else O.per_token_quant_int8
    w13, s13 = quant(torch.randn(e, 2 * inter, hid, generator=gen) * 0.05)
    w2, s2 = quant(torch.randn(e, hid, inter, generator=gen) * 0.05)
    s13, s2 = s13.reshape(e, -1), s2.reshape(e, -1)
    pack = deepgemm.marlin_fp8_contiguous_weight if kind == "fp8" else deepgemm.marlin_i8_contiguous_weight
    out = moe_forward(hidden.to(DEV), topk_ids.to(DEV), topk_w.to(DEV),
                      (pack(w13.clone().to(DEV)), s13.to(DEV)), (pack(w2.clone().to(DEV)), s2.to(DEV)),
                      kind=kind).cpu()
    ref = O.ref_moe_layer(hidden, topk_ids, topk_w, w13, s13, w2, s2, kind=kind)
    assert_calc_diff(out, ref.float(), 1e-3, f"{kind} MoE layer")      # tolerance: calc_diff < 1e-3
