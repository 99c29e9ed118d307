"""GPU parity of the contiguous grouped GEMM entry points against the CPU oracle
(same criteria as tests/test_gpu_masked.py)."""
import pytest
import torch

import deepgemm
from deepgemm import _cabi, _core
from deepgemm import group_gemm_weight_pack as P

import dg_oracle as O
from helpers import assert_bf16_within_ulp, assert_calc_diff, gen_contig, gen_masked_w4a8, load_golden

pytestmark = pytest.mark.gpu
DEV = "cuda"
SENTINEL = 17.0


def _check_int8_contig(c, rows_per_group, block_n=0, what=""):
    M, K = c["a"].shape
    G, N, _ = c["b"].shape
    bp = P.marlin_i8_contiguous_weight(c["b"].clone())
    d = torch.full((M, N), SENTINEL, dtype=torch.bfloat16, device=DEV)
    acc = torch.full((M, N), -12345, dtype=torch.int32, device=DEV)
    st = torch.zeros(_cabi.STATUS_WORDS, dtype=torch.int32, device=DEV)
    _core.grouped_gemm_contiguous(_cabi.KIND_I8, _cabi.SCALE_PER_CHANNEL, c["a"].to(DEV), bp.to(DEV),
                                  d, c["a_scale"].to(DEV), c["b_scale"].to(DEV),
                                  c["m_indices"].to(DEV), block_n=block_n, debug_acc=acc, status=st)
    torch.cuda.synchronize()
    assert st.tolist() == [0, 0, 0, 0], f"{what}: device status {st.tolist()}"
    d, acc = d.cpu(), acc.cpu()
    idx = c["m_indices"]
    for g in range(G):
        rows = torch.nonzero(idx == g).flatten()
        if rows.numel() == 0:
            continue
        want_acc = O.exact_int_acc(c["a"][rows], c["b"][g])
        assert torch.equal(acc[rows], want_acc), f"{what}: accumulators differ in group {g}"
        want = O.epilogue_from_acc(want_acc, c["a_scale"][rows], c["b_scale"][g])
        assert_bf16_within_ulp(d[rows], want, 0, f"{what} group {g}")
    pad = idx < 0
    assert torch.all(d[pad].float() == SENTINEL), f"{what}: padding rows were written"
    ref = O.ref_contiguous(c["a"], c["b"], c["a_scale"], c["b_scale"], idx)
    assert_bf16_within_ulp(d[~pad], ref[~pad], 1, f"{what} vs reference formula")


@pytest.mark.parametrize("bn", [0, 128, 256, 512])
def test_contiguous_int8_ragged_groups(bn):
    rows = [300, 0, 511, 101, 256, 1]
    c = gen_contig("int8", rows, 512, 512, seed=20)
    _check_int8_contig(c, rows, block_n=bn, what=f"contig int8 BN={bn}")


def test_contiguous_int8_align_128_and_ragged_tail():
    """Groups padded to 128 only, and a total row count that is not a multiple of 128."""
    rows = [128, 5, 200]
    c = gen_contig("int8", rows, 256, 256, seed=21, align=128)
    cut = c["a"].shape[0] - 40               # drop 40 trailing padding rows -> ragged last block
    assert int(c["m_indices"][cut - 1]) < 0
    c = dict(a=c["a"][:cut].contiguous(), a_scale=c["a_scale"][:cut].contiguous(), b=c["b"],
             b_scale=c["b_scale"], m_indices=c["m_indices"][:cut].contiguous())
    for bn in (0, 512):      # 512: super blocks whose halves belong to different groups
        _check_int8_contig(c, rows, block_n=bn, what=f"align 128 BN={bn}")


def test_contiguous_pair_kernel_many_super_blocks():
    """Two-CTA tiles: more work items than SM pairs, several column tiles, ragged N."""
    rows = [700, 256, 1, 0, 900, 130, 512, 255, 257, 64, 300, 1024]
    c = gen_contig("int8", rows, 1312, 256, seed=27)
    _check_int8_contig(c, rows, block_n=512, what="pair kernel")


def test_contiguous_public_api_int64_indices_and_golden():
    g = load_golden("contig_int8")
    M, K = g["a"].shape
    N = g["b"].shape[1]
    bp = P.marlin_i8_contiguous_weight(g["b"].clone().to(DEV))
    out = torch.zeros(M, N, dtype=torch.bfloat16, device=DEV)
    r = deepgemm.m_grouped_i8_gemm_nt_contiguous([g["a"].to(DEV), g["a_scale"].to(DEV)],
                                                 [bp, g["b_scale"].to(DEV)], out,
                                                 g["m_indices"].long().to(DEV))   # cast like the reference
    assert r is out
    assert_bf16_within_ulp(out.cpu(), g["out"], 1, "golden contig int8")        # padding rows: zeros on both sides


def test_contiguous_fp8_golden_and_random():
    g = load_golden("contig_fp8")
    M, K = g["a"].shape
    N = g["b"].shape[1]
    bp = P.marlin_fp8_contiguous_weight(g["b"].clone().to(DEV))
    out = torch.zeros(M, N, dtype=torch.bfloat16, device=DEV)
    deepgemm.m_grouped_fp8_gemm_nt_contiguous((g["a"].to(DEV), g["a_scale"].to(DEV)),
                                              (bp, g["b_scale"].to(DEV)), out, g["m_indices"].to(DEV))
    assert_bf16_within_ulp(out.cpu(), g["out"], 0, "golden contig fp8")          # integer inputs: exact

    rows = [256, 40, 0, 300]
    c = gen_contig("fp8", rows, 512, 1024, seed=22)
    bp = P.marlin_fp8_contiguous_weight(c["b"].clone().to(DEV))
    out = torch.full((c["a"].shape[0], 512), SENTINEL, dtype=torch.bfloat16, device=DEV)
    deepgemm.m_grouped_fp8_gemm_nt_contiguous((c["a"].to(DEV), c["a_scale"].to(DEV)),
                                              (bp, c["b_scale"].to(DEV)), out, c["m_indices"].to(DEV))
    out2 = torch.full_like(out, SENTINEL)
    _core.grouped_gemm_contiguous(_cabi.KIND_E4M3, _cabi.SCALE_PER_CHANNEL, c["a"].to(DEV), bp, out2,
                                  c["a_scale"].to(DEV), c["b_scale"].to(DEV), c["m_indices"].to(DEV),
                                  block_n=512)
    ref = O.ref_contiguous(c["a"], c["b"], c["a_scale"], c["b_scale"], c["m_indices"])
    pad = c["m_indices"] < 0
    for o, name in ((out.cpu(), "contig fp8"), (out2.cpu(), "contig fp8 two-CTA")):
        assert_calc_diff(o[~pad], ref[~pad], 1e-3, name)                          # calc_diff < 1e-3
        assert torch.all(o[pad].float() == SENTINEL)


def test_contiguous_fp8_tensor_wise():
    rows = [130, 256, 7]
    c = gen_contig("fp8", rows, 256, 512, seed=23, tensor_wise=True)
    bp = P.marlin_fp8_contiguous_weight(c["b"].clone().to(DEV))
    out = torch.zeros(c["a"].shape[0], 256, dtype=torch.bfloat16, device=DEV)
    deepgemm.m_grouped_fp8_gemm_nt_contiguous_tensor_wise(
        (c["a"].to(DEV), c["a_scale"].to(DEV)), (bp, c["b_scale"].reshape(-1, 1).to(DEV)), out,
        c["m_indices"].to(DEV))
    ref = O.ref_contiguous(c["a"], c["b"], c["a_scale"], c["b_scale"], c["m_indices"], tensor_wise=True)
    pad = c["m_indices"] < 0
    assert_calc_diff(out.cpu()[~pad], ref[~pad], 1e-3, "contig fp8 tensor-wise")


def test_contiguous_w4a8():
    rows = [128, 60, 256]
    idx, M = O.build_contiguous_layout(rows, 128)
    cw = gen_masked_w4a8(len(rows), 1, 256, 512, [1] * len(rows), seed=24)      # weights only
    gen = torch.Generator().manual_seed(25)
    a, a_s = O.per_token_quant_int8(torch.randn(M, 512, generator=gen))
    bp = P.pack_w4a8_moe_hipc_weight(cw["b_framework"].clone().to(DEV))
    out = torch.full((M, 256), SENTINEL, dtype=torch.bfloat16, device=DEV)
    r = deepgemm.m_grouped_w4a8_gemm_nt_contiguous_hipc(
        (a.to(DEV), a_s.to(DEV)), (bp, (cw["b_scale"] / 16.0).unsqueeze(-1).to(DEV)), out, idx.to(DEV))
    assert r is out
    out = out.cpu()
    w_x16 = (cw["w4"].to(torch.int16) * 16).to(torch.int8)
    for g in range(len(rows)):
        r_ = torch.nonzero(idx == g).flatten()
        want = O.epilogue_from_acc(O.exact_int_acc(a[r_], w_x16[g]), a_s.reshape(-1)[r_], cw["b_scale"][g] / 16.0)
        assert_bf16_within_ulp(out[r_], want, 0, f"contig w4a8 group {g}")
    assert torch.all(out[idx < 0].float() == SENTINEL)


def test_out_of_range_group_index_is_reported_not_read():
    """An m_indices entry >= num_groups must never index the weights: the block is skipped and
    the device status word says so."""
    rows = [128, 128]
    c = gen_contig("int8", rows, 128, 128, seed=26, align=128)
    bad = c["m_indices"].clone()
    bad[128:] = 7                                   # only groups 0..1 exist
    bp = P.marlin_i8_contiguous_weight(c["b"].clone())
    d = torch.full((256, 128), SENTINEL, dtype=torch.bfloat16, device=DEV)
    st = torch.zeros(_cabi.STATUS_WORDS, dtype=torch.int32, device=DEV)
    _core.grouped_gemm_contiguous(_cabi.KIND_I8, _cabi.SCALE_PER_CHANNEL, c["a"].to(DEV), bp.to(DEV), d,
                                  c["a_scale"].to(DEV), c["b_scale"].to(DEV), bad.to(DEV), status=st)
    torch.cuda.synchronize()
    assert int(st[0]) == 2
    d = d.cpu()
    assert torch.all(d[128:].float() == SENTINEL)
    ref = O.ref_contiguous(c["a"], c["b"], c["a_scale"], c["b_scale"], c["m_indices"])
    assert_bf16_within_ulp(d[:128], ref[:128], 1, "valid block next to a bad one")


@pytest.mark.parametrize("seed", range(16))
def test_random_group_sizes_and_tile_choices_bit_exact(seed):
    """Seeded random group counts, ragged group sizes (empty groups included), N and K, each
    with one of the tile options and one of the two paddings; a random cut of the trailing
    padding makes the last row block ragged."""
    gen = torch.Generator().manual_seed(3000 + seed)
    r = lambda lo, hi: int(torch.randint(lo, hi + 1, (1,), generator=gen))
    G = r(1, 10)
    rows = [0 if r(0, 3) == 0 else r(1, 600) for _ in range(G)]
    if sum(rows) == 0:
        rows[0] = r(1, 600)
    n, k = 16 * r(1, 48), 128 * r(1, 5)
    align = (128, 256)[r(0, 1)]
    bn = (0, 128, 256, 512)[seed % 4]
    c = gen_contig("int8", rows, n, k, seed=4000 + seed, align=align)
    idx = c["m_indices"]
    trailing = 0
    while trailing < idx.numel() and int(idx[idx.numel() - 1 - trailing]) < 0:
        trailing += 1
    cut = idx.numel() - (r(0, trailing) if trailing else 0)
    c = dict(a=c["a"][:cut].contiguous(), a_scale=c["a_scale"][:cut].contiguous(), b=c["b"],
             b_scale=c["b_scale"], m_indices=idx[:cut].contiguous())
    _check_int8_contig(c, rows, block_n=bn,
                       what=f"seed {seed}: rows={rows} N={n} K={k} align={align} BN={bn} cut={cut}")


@pytest.mark.parametrize("block_n", [0, 512])
@pytest.mark.parametrize("seed", range(6))
def test_contiguous_w4a8_random_group_sizes(seed, block_n):
    """Seeded random contiguous W4A8 cases: ragged groups (empty ones included) padded to 128
    rows, N not a multiple of the channel tile, one to four 256-value rounds of K; with the default
    kernel (block_n 0) and with the one that unpacks in shared memory (512)."""
    gen = torch.Generator().manual_seed(7000 + seed)
    r = lambda lo, hi: int(torch.randint(lo, hi + 1, (1,), generator=gen))
    G = r(1, 8)
    rows = [0 if r(0, 3) == 0 else r(1, 400) for _ in range(G)]
    if sum(rows) == 0:
        rows[0] = r(1, 400)
    n, k = 16 * r(1, 30), 256 * r(1, 4)
    idx, M = O.build_contiguous_layout(rows, 128)
    cw = gen_masked_w4a8(G, 1, n, k, [1] * G, seed=7100 + seed)                 # weights only
    a, a_s = O.per_token_quant_int8(torch.randn(M, k, generator=gen))
    bp = P.pack_w4a8_moe_hipc_weight(cw["b_framework"].clone().to(DEV))
    out = torch.full((M, n), SENTINEL, dtype=torch.bfloat16, device=DEV)
    if block_n == 0:
        deepgemm.m_grouped_w4a8_gemm_nt_contiguous_hipc(
            (a.to(DEV), a_s.to(DEV)), (bp, (cw["b_scale"] / 16.0).unsqueeze(-1).to(DEV)), out, idx.to(DEV))
    else:
        _core.grouped_gemm_contiguous(_cabi.KIND_W4A8, _cabi.SCALE_PER_CHANNEL, a.to(DEV), bp, out,
                                      a_s.reshape(-1).to(DEV), (cw["b_scale"] / 16.0).to(DEV), idx.to(DEV),
                                      block_n=block_n)
    out = out.cpu()
    w_x16 = (cw["w4"].to(torch.int16) * 16).to(torch.int8)
    for g in range(G):
        r_ = torch.nonzero(idx == g).flatten()
        if r_.numel() == 0:
            continue
        want = O.epilogue_from_acc(O.exact_int_acc(a[r_], w_x16[g]), a_s.reshape(-1)[r_], cw["b_scale"][g] / 16.0)
        assert_bf16_within_ulp(out[r_], want, 0, f"seed {seed}: rows={rows} N={n} K={k} group {g}")
    assert torch.all(out[idx < 0].float() == SENTINEL), f"seed {seed}: padding rows were written"


@pytest.mark.parametrize("bn", [0, 128, 512])
def test_group_window_calls_cover_the_same_rows_as_one_call(bn):
    """Three calls, each with a slice of the groups and the whole m_indices array (group_window),
    write exactly the rows of their groups and, together, the bytes of the single call; a window
    is not an out-of-range report."""
    rows = [300, 0, 511, 101, 256, 1, 77]
    c = gen_contig("int8", rows, 512, 512, seed=61)
    M, N = c["a"].shape[0], c["b"].shape[1]
    bp = P.marlin_i8_contiguous_weight(c["b"].clone()).to(DEV)
    a, sa, sb, idx = c["a"].to(DEV), c["a_scale"].to(DEV), c["b_scale"].to(DEV), c["m_indices"].to(DEV)
    whole = torch.full((M, N), SENTINEL, dtype=torch.bfloat16, device=DEV)
    _core.grouped_gemm_contiguous(_cabi.KIND_I8, _cabi.SCALE_PER_CHANNEL, a, bp, whole, sa, sb, idx, block_n=bn)
    parts = torch.full((M, N), SENTINEL, dtype=torch.bfloat16, device=DEV)
    st = torch.zeros(_cabi.STATUS_WORDS, dtype=torch.int32, device=DEV)
    for lo, hi in ((0, 3), (3, 4), (4, 7)):
        before = parts.clone()
        _core.grouped_gemm_contiguous(_cabi.KIND_I8, _cabi.SCALE_PER_CHANNEL, a, bp[lo:hi], parts, sa, sb[lo:hi],
                                      idx, block_n=bn, status=st, group_window=lo)
        outside = ~((idx >= lo) & (idx < hi))
        assert torch.equal(parts[outside].view(torch.int16), before[outside].view(torch.int16)), \
            f"window {lo}..{hi} wrote rows of other groups"
    torch.cuda.synchronize()
    assert st.tolist() == [0, 0, 0, 0]
    assert torch.equal(parts.view(torch.int16), whole.view(torch.int16))
    # without a window the same slice call reports the foreign ids
    _core.grouped_gemm_contiguous(_cabi.KIND_I8, _cabi.SCALE_PER_CHANNEL, a, bp[0:3], parts, sa, sb[0:3], idx,
                                  block_n=bn, status=st)
    torch.cuda.synchronize()
    assert st.tolist()[0] == 2       # DG_DEV_BAD_GROUP_INDEX


@pytest.mark.parametrize("K", [192, 1088])
def test_contiguous_k_an_odd_multiple_of_64(K):
    rows = [300, 0, 511, 101]
    c = gen_contig("int8", rows, 512, K, seed=K)
    for bn in (0, 256, 512):
        _check_int8_contig(c, rows, block_n=bn, what=f"contig int8 K={K} BN={bn}")
