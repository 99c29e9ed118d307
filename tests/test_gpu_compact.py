"""Compact page layout (expert_offsets + counts), the no-padding contiguous entry and the BF16
contiguous entry against the CPU oracle.  The compact cases follow the reference's own test
(op_test/test_deepgemm_compact_masked_w8a8.py:42-163): counts [300, 0, 511, 101] on a 1024-row
page, NaN-filled output that must stay untouched outside the valid rows, and an empty page."""
import pytest
import torch

import deepgemm
from deepgemm import _cabi, _core

import dg_oracle as O
from helpers import assert_bf16_within_ulp, assert_calc_diff

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _page(counts, offsets, capacity, K, N, seed):
    g = torch.Generator().manual_seed(seed)
    q_x, x_s = O.per_token_quant_int8(torch.randn(capacity, K, generator=g))
    w = torch.randint(-8, 8, (len(counts), N, K), generator=g).to(torch.int8)
    w_s = torch.rand(len(counts), N, 1, generator=g)
    return q_x, x_s, w, w_s


@pytest.mark.parametrize("bn", [0, 128, 256])
def test_compact_masked_matches_oracle_and_leaves_other_rows_alone(bn):
    counts, offsets, cap, K, N = [300, 0, 511, 101], [0, 300, 300, 811], 1024, 2048, 256
    q_x, x_s, w, w_s = _page(counts, offsets, cap, K, N, 7)
    bp = deepgemm.marlin_i8_masked_weight(w.clone().to(DEV))
    out = torch.full((cap, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    acc = torch.full((cap, N), -9, dtype=torch.int32, device=DEV)
    c_t = torch.tensor(counts, dtype=torch.int32, device=DEV)
    o_t = torch.tensor(offsets, dtype=torch.int32, device=DEV)
    if bn == 0:
        r = deepgemm.m_grouped_w8a8_gemm_nt_compact_masked((q_x.to(DEV), x_s.to(DEV)), (bp, w_s.to(DEV)),
                                                           out, c_t, o_t, expected_m_per_group=512)
        assert r is out
    else:
        _core.grouped_gemm_compact(_cabi.KIND_I8, 0, q_x.to(DEV), bp, out, x_s.to(DEV), w_s.to(DEV), c_t, o_t,
                                   512, block_n=bn, debug_acc=acc)
    out = out.cpu()
    written = torch.zeros(cap, dtype=torch.bool)
    for e, (c, o) in enumerate(zip(counts, offsets)):
        if c == 0:
            continue
        rows = slice(o, o + c)
        want_acc = O.exact_int_acc(q_x[rows], w[e])
        want = O.epilogue_from_acc(want_acc, x_s[rows], w_s[e].reshape(-1))
        assert_bf16_within_ulp(out[rows], want, 0, f"compact expert {e}")
        if bn:
            assert torch.equal(acc.cpu()[rows], want_acc)
        written[rows] = True
    assert torch.isnan(out[~written].float()).all(), "rows outside every expert's range were written"


def test_compact_page_with_more_items_than_sms_and_a_split_last_round():
    """44 experts x 4 column tiles of 256 = 176 items: the 28 of the second round run as 56 half
    tiles (on a 148-SM GPU).  Result rows and untouched rows as above."""
    gen = torch.Generator().manual_seed(9)
    counts = torch.randint(0, 25, (44,), generator=gen).clamp_min(1).tolist()
    offsets, run = [], 0
    for c in counts:
        offsets.append(run)
        run += c + 3                                           # gaps between experts stay untouched
    cap, K, N = run + 5, 256, 1024
    q_x, x_s, w, w_s = _page(counts, offsets, cap, K, N, 11)
    bp = deepgemm.marlin_i8_masked_weight(w.clone().to(DEV))
    out = torch.full((cap, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    _core.grouped_gemm_compact(_cabi.KIND_I8, 0, q_x.to(DEV), bp, out, x_s.to(DEV), w_s.to(DEV),
                               torch.tensor(counts, dtype=torch.int32, device=DEV),
                               torch.tensor(offsets, dtype=torch.int32, device=DEV), 24, block_n=256)
    out = out.cpu()
    written = torch.zeros(cap, dtype=torch.bool)
    for e, (c, o) in enumerate(zip(counts, offsets)):
        rows = slice(o, o + c)
        want = O.epilogue_from_acc(O.exact_int_acc(q_x[rows], w[e]), x_s[rows], w_s[e].reshape(-1))
        assert_bf16_within_ulp(out[rows], want, 0, f"compact expert {e}")
        written[rows] = True
    assert torch.isnan(out[~written].float()).all()


def test_compact_masked_empty_page_is_untouched():
    q_x = torch.zeros(256, 2048, dtype=torch.int8, device=DEV)
    x_s = torch.ones(256, 1, device=DEV)
    bp = deepgemm.marlin_i8_masked_weight(torch.zeros(4, 256, 2048, dtype=torch.int8, device=DEV))
    out = torch.full((256, 256), 17, dtype=torch.bfloat16, device=DEV)
    z = torch.zeros(4, dtype=torch.int32, device=DEV)
    deepgemm.m_grouped_w8a8_gemm_nt_compact_masked((q_x, x_s), (bp, torch.ones(4, 256, 1, device=DEV)), out, z, z,
                                                   expected_m_per_group=1)
    torch.cuda.synchronize()
    assert torch.all(out == 17)


def test_contiguous_nopad():
    counts = [37, 0, 200, 129, 1]
    M, K, N = sum(counts), 512, 384
    g = torch.Generator().manual_seed(11)
    a, a_s = O.per_token_quant_int8(torch.randn(M, K, generator=g))
    w, w_s = O.per_token_quant_int8(torch.randn(len(counts), N, K, generator=g))
    m_indices = torch.repeat_interleave(torch.arange(len(counts)), torch.tensor(counts)).to(torch.int32)
    bp = deepgemm.marlin_i8_contiguous_weight(w.clone().to(DEV))
    out = torch.zeros(M, N, dtype=torch.bfloat16, device=DEV)
    r = deepgemm.m_grouped_i8_gemm_nt_contiguous_nopad(
        (a.to(DEV), a_s.to(DEV)), (bp, w_s.to(DEV)), out, m_indices.to(DEV),
        torch.tensor(counts, dtype=torch.int32, device=DEV))
    assert r is out
    ref = O.ref_contiguous(a, w, a_s, w_s, m_indices)
    assert_bf16_within_ulp(out.cpu(), ref, 1, "nopad contiguous")


def test_contiguous_bf16():
    rows = [130, 0, 256]
    idx, M = O.build_contiguous_layout(rows, 128)
    g = torch.Generator().manual_seed(12)
    a = (torch.randn(M, 512, generator=g) * 0.1).bfloat16()
    w = (torch.randn(len(rows), 256, 512, generator=g) * 0.1).bfloat16()
    packed, _ = deepgemm.pack_bf16_masked_weight(w.clone().to(DEV))
    out = torch.full((M, 256), 3.0, dtype=torch.bfloat16, device=DEV)
    r = deepgemm.m_grouped_bf16_gemm_nt_contiguous(a.to(DEV), packed, out, idx.to(DEV))
    assert r is out
    out = out.cpu()
    for e in range(len(rows)):
        r_ = torch.nonzero(idx == e).flatten()
        if r_.numel():
            ref = (a[r_].float() @ w[e].float().t()).bfloat16()
            assert_calc_diff(out[r_], ref, 1e-3, f"bf16 contiguous expert {e}")      # calc_diff < 1e-3
    assert torch.all(out[idx < 0] == 3.0)


def test_legacy_names_pack_like_the_current_ones():
    w = torch.randint(-128, 128, (2, 32, 256), dtype=torch.int8, device=DEV)
    assert torch.equal(deepgemm.weight8bit_nt_kpack2_marlin2(w.clone()), deepgemm.marlin_i8_masked_weight(w.clone()))
    assert torch.equal(deepgemm.weight8bit_nt_kpack2_marlin(w.clone()), deepgemm.marlin_i8_contiguous_weight(w.clone()))
