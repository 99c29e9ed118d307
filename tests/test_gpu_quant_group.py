"""The fused quantise + group + pad producer against its torch definition
(deepgemm.quant_utils quantisers + deepgemm.expert_parallel.group_and_pad): bit-exact
quantised bytes and scales, identical layout, and the contiguous GEMM on its output."""
import pytest
import torch

import deepgemm
from deepgemm import expert_parallel as ep
from deepgemm.quant_group import quant_group_capacity, quantize_group_rows
from deepgemm.quant_utils import per_token_quant_fp8, per_token_quant_int8

import dg_oracle as O
from helpers import assert_calc_diff

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("kind", ["fp8", "int8"])
@pytest.mark.parametrize("R,H,G,align", [(1000, 512, 7, 256), (37, 7168, 4, 128), (4096, 2048, 64, 256)])
def test_matches_torch_definition(kind, R, H, G, align):
    gen = torch.Generator().manual_seed(R + H)
    rows = (torch.randn(R, H, generator=gen) * 3).bfloat16()
    rows[5] = 0                                               # an all-zero row (absmax clamps to eps)
    expert = torch.randint(0, G, (R,), generator=gen).to(torch.int32)
    expert[expert == 2] = 3                                   # leave a group empty
    expert[11] = -1                                           # a dropped row
    a, a_s, m_idx, dest, m_total = quantize_group_rows(rows.to(DEV), expert.to(DEV), G, kind=kind, align=align)
    torch.cuda.synchronize()
    a, a_s, m_idx, dest = a.cpu(), a_s.cpu(), m_idx.cpu(), dest.cpu()
    keep = expert >= 0
    want_rows, want_idx, want_dest = ep.group_and_pad(rows[keep], expert[keep].long(), G, align=align)
    m = want_rows.shape[0]
    assert int(m_total) == m and a.shape[0] == quant_group_capacity(R, G, align)
    assert torch.equal(m_idx[:m], want_idx) and torch.all(m_idx[m:] == -1)
    assert torch.equal(dest[keep], want_dest.to(torch.int32)) and int(dest[11]) == -1
    quant = per_token_quant_fp8 if kind == "fp8" else per_token_quant_int8
    q, s = quant(rows[keep])
    pos = want_dest
    got_q = a[pos].view(torch.uint8) if kind == "fp8" else a[pos]
    want_q = q.view(torch.uint8) if kind == "fp8" else q
    assert torch.equal(got_q, want_q), "quantised bytes differ from the torch quantiser"
    assert torch.equal(a_s[pos], s.reshape(-1)), "scales differ from the torch quantiser"


def test_feeds_the_contiguous_gemm():
    gen = torch.Generator().manual_seed(3)
    R, H, G, N = 700, 512, 5, 256
    rows = torch.randn(R, H, generator=gen).bfloat16()
    expert = torch.randint(0, G, (R,), generator=gen).to(torch.int32)
    b, b_s = O.per_token_quant_fp8(torch.randn(G, N, H, generator=gen))
    bp = deepgemm.marlin_fp8_contiguous_weight(b.clone().to(DEV))
    a, a_s, m_idx, dest, _ = quantize_group_rows(rows.to(DEV), expert.to(DEV), G)
    out = torch.zeros(a.shape[0], N, dtype=torch.bfloat16, device=DEV)
    deepgemm.m_grouped_fp8_gemm_nt_contiguous((a, a_s), (bp, b_s.reshape(G, N).to(DEV)), out, m_idx)
    out, dest = out.cpu(), dest.cpu().long()
    qa, sa = O.per_token_quant_fp8(rows)
    for g in range(G):
        r = torch.nonzero(expert == g).flatten()
        ref = O.ref_masked_scaled(qa[r][None], b[g][None], sa[r][None], b_s[g][None])[0]
        assert_calc_diff(out[dest[r]], ref, 1e-3, f"group {g}")                  # calc_diff < 1e-3


def test_argument_errors():
    rows = torch.zeros(8, 64, dtype=torch.bfloat16, device=DEV)
    e = torch.zeros(8, dtype=torch.int32, device=DEV)
    with pytest.raises(ValueError):
        quantize_group_rows(rows.float(), e, 2)
    with pytest.raises(ValueError):
        quantize_group_rows(rows, e[:4], 2)
    with pytest.raises(ValueError):
        quantize_group_rows(rows, e, 2, kind="fp4")
    with pytest.raises(RuntimeError):
        quantize_group_rows(torch.zeros(8, 20, dtype=torch.bfloat16, device=DEV), e, 2)   # H % 8
    with pytest.raises(RuntimeError):
        quantize_group_rows(rows.cpu(), e.cpu(), 2)


@pytest.mark.parametrize("kind", ["fp8", "int8"])
def test_grouping_rows_quantised_elsewhere_gives_the_same_operands(kind):
    """quantize_rows + grouping with row_scale (what a rank does with rows that were quantised
    before the dispatch) must produce exactly what quantise+group in one go does."""
    from deepgemm.quant_group import quantize_rows
    gen = torch.Generator().manual_seed(11)
    R, H, G = 777, 1024, 9
    rows = (torch.randn(R, H, generator=gen) * 2).bfloat16().to(DEV)
    expert = torch.randint(-1, G, (R,), generator=gen).to(torch.int32).to(DEV)
    want = quantize_group_rows(rows, expert, G, kind=kind, align=128)
    q, s = quantize_rows(rows, kind=kind)
    quant = per_token_quant_fp8 if kind == "fp8" else per_token_quant_int8
    q_ref, s_ref = quant(rows.cpu())
    assert torch.equal(q.cpu().view(torch.uint8), q_ref.view(torch.uint8)) and torch.equal(s.cpu(), s_ref.reshape(-1))
    got = quantize_group_rows(q, expert, G, kind=kind, align=128, row_scale=s)
    torch.cuda.synchronize()
    m = int(want[4])
    assert int(got[4]) == m
    assert torch.equal(got[2], want[2]) and torch.equal(got[3], want[3])          # m_indices, dest
    valid = (want[2][:m] >= 0).cpu()
    assert torch.equal(got[0][:m].cpu().view(torch.uint8)[valid], want[0][:m].cpu().view(torch.uint8)[valid])
    assert torch.equal(got[1][:m].cpu()[valid], want[1][:m].cpu()[valid])
