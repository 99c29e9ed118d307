"""GPU parity of the masked grouped GEMM entry points (through the Python API -> custom op
-> C ABI) against the CPU oracle.

Criteria: INT8 / W4A8 -- raw int32 accumulators bit-exact and bf16 output within 1 bf16 ulp
of the reference formula; FP8 / BF16 -- calc_diff (1 - 2*sum(xy)/sum(x^2+y^2)) < 1e-3, and
bit-exact where inputs are small integers (sums are then order independent)."""
import pytest
import torch

import deepgemm
from deepgemm import _cabi, _core
from deepgemm import group_gemm_weight_pack as P

import dg_oracle as O
from helpers import (assert_bf16_within_ulp, assert_calc_diff, gen_masked_fp8, gen_masked_int8,
                     gen_masked_w4a8, load_golden)

pytestmark = pytest.mark.gpu
DEV = "cuda"
SENTINEL = 17.0


def _status():
    return torch.zeros(_cabi.STATUS_WORDS, dtype=torch.int32, device=DEV)


def _check_int_case(c, kind, b_rows_int8, b_packed, b_scale_kernel, block_n=0, what=""):
    """Runs the kernel with the accumulator dump on and checks acc bit-exact, output <= 1 ulp,
    rows >= masked_m untouched."""
    G, max_m, K = c["a"].shape
    N = b_rows_int8.shape[1]
    d = torch.full((G, max_m, N), SENTINEL, dtype=torch.bfloat16, device=DEV)
    acc = torch.full((G, max_m, N), -12345, dtype=torch.int32, device=DEV)
    st = _status()
    _core.grouped_gemm_masked(kind, _cabi.SCALE_PER_CHANNEL, c["a"].to(DEV), b_packed.to(DEV), d,
                              c["a_scale"].to(DEV), b_scale_kernel.to(DEV), c["masked_m"].to(DEV),
                              int(c["masked_m"].max()), block_n=block_n, debug_acc=acc, status=st)
    torch.cuda.synchronize()
    assert st.tolist() == [0, 0, 0, 0], f"{what}: device status {st.tolist()}"
    d, acc = d.cpu(), acc.cpu()
    for g in range(G):
        m = int(c["masked_m"][g])
        want_acc = O.exact_int_acc(c["a"][g, :m], b_rows_int8[g])
        assert torch.equal(acc[g, :m], want_acc), f"{what}: int32 accumulators differ in group {g}"
        want = O.epilogue_from_acc(want_acc, c["a_scale"][g, :m], b_scale_kernel[g])
        assert_bf16_within_ulp(d[g, :m], want, 0, f"{what} group {g} vs exact epilogue")
        assert torch.all(d[g, m:].float() == SENTINEL), f"{what}: rows >= masked_m written (group {g})"
        assert torch.all(acc[g, m:] == -12345)
    ref = O.ref_masked_scaled(c["a"], b_rows_int8, c["a_scale"].unsqueeze(-1), b_scale_kernel.unsqueeze(-1))
    for g in range(G):
        m = int(c["masked_m"][g])
        assert_bf16_within_ulp(d[g, :m], ref[g, :m], 1, f"{what} group {g} vs reference formula")


def test_config1_masked_int8_bit_exact():
    """G=4, max_m=64, N=512, K=256, masked_m uniform in [1,64]."""
    gen = torch.Generator().manual_seed(0)
    mm = torch.randint(1, 65, (4,), generator=gen)
    c = gen_masked_int8(4, 64, 512, 256, mm, seed=0)
    bp = P.marlin_i8_masked_weight(c["b"].clone())
    _check_int_case(c, _cabi.KIND_I8, c["b"], bp, c["b_scale"], what="config 1")


def test_config1_through_public_api_and_both_tile_widths():
    gen = torch.Generator().manual_seed(1)
    mm = torch.randint(1, 65, (4,), generator=gen)
    c = gen_masked_int8(4, 64, 512, 256, mm, seed=1)
    bp = P.marlin_i8_masked_weight(c["b"].clone().to(DEV))          # GPU packer
    outs = []
    for fn in (deepgemm.m_grouped_w8a8_gemm_nt_masked, deepgemm.m_grouped_i8_gemm_nt_masked,
               deepgemm.m_grouped_w8a8_gemm_nt_masked_ll):
        d = torch.zeros(4, 64, 512, dtype=torch.bfloat16, device=DEV)
        r = fn([c["a"].to(DEV), c["a_scale"].unsqueeze(-1).to(DEV)],
               [bp, c["b_scale"].unsqueeze(-1).to(DEV)], d, c["masked_m"].to(DEV), int(mm.max()))
        assert r is d
        outs.append(d.cpu())
    assert torch.equal(outs[0].view(torch.int16), outs[1].view(torch.int16))
    assert torch.equal(outs[0].view(torch.int16), outs[2].view(torch.int16))
    for bn in (128, 256):
        _check_int_case(c, _cabi.KIND_I8, c["b"], bp.cpu(), c["b_scale"], block_n=bn, what=f"BN={bn}")


def test_golden_masked_int8():
    g = load_golden("masked_int8")
    E, M, K = g["a"].shape
    bp = P.marlin_i8_masked_weight(g["b"].clone())
    d = torch.zeros(E, M, g["b"].shape[1], dtype=torch.bfloat16, device=DEV)
    deepgemm.m_grouped_w8a8_gemm_nt_masked((g["a"].to(DEV), g["a_scale"].to(DEV)),
                                           (bp.to(DEV), g["b_scale"].to(DEV)), d,
                                           torch.full((E,), M, dtype=torch.int32, device=DEV), M)
    assert_bf16_within_ulp(d.cpu(), g["out"], 1, "golden masked int8")


def test_every_masked_m_from_0_to_max():
    """One group per possible row count, crossing the 128-row tile boundary."""
    max_m, N, K = 160, 128, 128
    mm = torch.arange(0, max_m + 1)
    c = gen_masked_int8(max_m + 1, max_m, N, K, mm, seed=2)
    bp = P.marlin_i8_masked_weight(c["b"].clone())
    _check_int_case(c, _cabi.KIND_I8, c["b"], bp, c["b_scale"], what="masked_m sweep")


def test_skewed_routing_and_empty_groups():
    """Many empty groups, one very long one (the shape of real decode routing)."""
    mm = torch.tensor([0, 0, 700, 0, 1, 0, 0, 129, 0, 0, 0, 31, 0, 0, 0, 0, 256, 0, 0, 3])
    c = gen_masked_int8(len(mm), 704, 256, 256, mm, seed=3)
    bp = P.marlin_i8_masked_weight(c["b"].clone())
    for bn in (128, 256, 512):
        _check_int_case(c, _cabi.KIND_I8, c["b"], bp, c["b_scale"], block_n=bn, what=f"skew BN={bn}")


def test_all_groups_empty_is_a_no_op():
    c = gen_masked_int8(3, 16, 64, 128, [0, 0, 0], seed=4)
    bp = P.marlin_i8_masked_weight(c["b"].clone())
    _check_int_case(c, _cabi.KIND_I8, c["b"], bp, c["b_scale"], what="all empty")


@pytest.mark.parametrize("N,K", [(48, 128), (192, 384), (272, 7168)])
def test_ragged_n_and_deep_k(N, K):
    """N not a multiple of the tile width; K long enough to wrap the stage ring many times."""
    c = gen_masked_int8(2, 128, N, K, [77, 128], seed=5)
    bp = P.marlin_i8_masked_weight(c["b"].clone())
    for bn in (128, 256, 512):
        _check_int_case(c, _cabi.KIND_I8, c["b"], bp, c["b_scale"], block_n=bn, what=f"N={N} K={K} BN={bn}")


def test_int32_accumulator_beyond_fp32_exact_range():
    """All-extreme operands: |acc| = K*127*127 > 2^24, where an fp32-accumulating path would round."""
    G, M, N, K = 1, 16, 64, 7168
    a = torch.full((G, M, K), 127, dtype=torch.int8)
    b = torch.full((G, N, K), -127, dtype=torch.int8)
    a[0, 1, 5] = 126
    c = dict(a=a, a_scale=torch.ones(G, M), b=b, b_scale=torch.ones(G, N),
             masked_m=torch.tensor([M], dtype=torch.int32))
    _check_int_case(c, _cabi.KIND_I8, b, P.marlin_i8_masked_weight(b.clone()), c["b_scale"], what="big acc")


# ----------------------------------------------------------------------------- FP8
def _run_fp8(c, tensor_wise, fn, block_n=0):
    G, max_m, K = c["a"].shape
    N = c["b"].shape[1]
    bp = P.marlin_fp8_masked_weight(c["b"].clone().to(DEV))
    d = torch.full((G, max_m, N), SENTINEL, dtype=torch.bfloat16, device=DEV)
    if fn is None:
        st = _status()
        _core.grouped_gemm_masked(_cabi.KIND_E4M3,
                                  _cabi.SCALE_TENSOR_WISE if tensor_wise else _cabi.SCALE_PER_CHANNEL,
                                  c["a"].to(DEV), bp, d, c["a_scale"].to(DEV), c["b_scale"].to(DEV),
                                  c["masked_m"].to(DEV), int(c["masked_m"].max()), block_n=block_n, status=st)
        torch.cuda.synchronize()
        assert st.tolist() == [0, 0, 0, 0]
    else:
        fn((c["a"].to(DEV), c["a_scale"].to(DEV)), (bp, c["b_scale"].to(DEV)), d,
           c["masked_m"].to(DEV), int(c["masked_m"].max()))
    return d.cpu()


@pytest.mark.parametrize("tensor_wise", [False, True])
def test_masked_fp8_random(tensor_wise):
    mm = [0, 5, 64, 128, 100, 1]
    c = gen_masked_fp8(6, 128, 512, 1024, mm, seed=6, tensor_wise=tensor_wise)
    fn = deepgemm.m_grouped_fp8_gemm_nt_masked_tensor_wise if tensor_wise else deepgemm.m_grouped_fp8_gemm_nt_masked
    d = _run_fp8(c, tensor_wise, fn)
    ref = (O.ref_masked_tensor_wise if tensor_wise else O.ref_masked_scaled)(
        c["a"], c["b"], c["a_scale"], c["b_scale"])
    for g, m in enumerate(mm):
        if m:
            assert_calc_diff(d[g, :m], ref[g, :m], 1e-3, f"fp8 group {g}")   # tolerance: calc_diff < 1e-3
        assert torch.all(d[g, m:].float() == SENTINEL)


@pytest.mark.parametrize("bn", [128, 256, 512])
def test_masked_fp8_integer_inputs_are_bit_exact(bn):
    """Small-integer e4m3 operands (as the reference's unified tests use): every partial sum is
    exact in fp32, so the result must equal the oracle's bit for bit."""
    mm = [128, 3, 0, 77]
    c = gen_masked_fp8(4, 128, 256, 512, mm, seed=7, integer=True)
    d = _run_fp8(c, False, None, block_n=bn)
    ref = O.ref_masked_scaled(c["a"], c["b"], c["a_scale"], c["b_scale"])
    for g, m in enumerate(mm):
        assert_bf16_within_ulp(d[g, :m], ref[g, :m], 0, f"fp8 integer group {g}")


def test_golden_masked_fp8_and_tensor_wise():
    for name, tw in (("masked_fp8", False), ("masked_fp8_tensor_wise", True)):
        g = load_golden(name)
        E, M, K = g["a"].shape
        c = dict(a=g["a"], a_scale=g["a_scale"], b=g["b"], b_scale=g["b_scale"],
                 masked_m=torch.full((E,), M, dtype=torch.int32))
        fn = deepgemm.m_grouped_fp8_gemm_nt_masked_ll_tensor_wise if tw else deepgemm.m_grouped_fp8_gemm_nt_masked_ll
        d = _run_fp8(c, tw, fn)
        assert_bf16_within_ulp(d, g["out"], 0, f"golden {name}")


def test_fp8_nan_rows_above_masked_m_do_not_leak():
    """Rows >= masked_m may hold anything, even NaN bit patterns: valid rows are unaffected."""
    mm = [40, 128]
    c = gen_masked_fp8(2, 128, 256, 256, mm, seed=8)
    ref = O.ref_masked_scaled(c["a"], c["b"], c["a_scale"], c["b_scale"])
    a_bits = c["a"].view(torch.uint8).clone()
    a_bits[0, 40:] = 0x7F                       # e4m3 NaN
    c["a"] = a_bits.view(torch.float8_e4m3fn)
    d = _run_fp8(c, False, None)
    assert torch.isfinite(d[0, :40].float()).all()
    assert_calc_diff(d[0, :40], ref[0, :40], 1e-3, "rows below a NaN tail")


# ----------------------------------------------------------------------------- W4A8
@pytest.mark.parametrize("order", ["high_first", "low_first"])
def test_masked_w4a8_bit_exact(order):
    mm = [0, 256, 17, 130]
    c = gen_masked_w4a8(4, 256, 384, 512, mm, seed=9, nibble_order=order)
    bp = P.pack_w4a8_moe_hipc_weight(c["b_framework"].clone().to(DEV), nibble_order=order)
    w_x16 = (c["w4"].to(torch.int16) * 16).to(torch.int8)     # what the kernel multiplies by
    assert torch.equal(w_x16, O.unpack_int4_to_int8_x16(c["b_framework"], order))
    _check_int_case(c, _cabi.KIND_W4A8, w_x16, bp, c["b_scale"] / 16.0, what=f"w4a8 {order}")


def test_masked_w4a8_public_api_and_golden():
    g = load_golden("masked_w4a8")
    E, M, K = g["a"].shape
    N = g["framework"].shape[1]
    bp = P.pack_w4a8_moe_hipc_weight(g["framework"].clone().to(DEV))
    mm = torch.full((E,), M, dtype=torch.int32, device=DEV)
    for fn in (deepgemm.m_grouped_w4a8_gemm_nt_masked, deepgemm.m_grouped_w4a8_gemm_nt_masked_hipc):
        d = torch.zeros(E, M, N, dtype=torch.bfloat16, device=DEV)
        fn((g["a"].to(DEV), g["a_scale"].to(DEV)), (bp, g["b_scale"].to(DEV)), d, mm, M)
        assert_bf16_within_ulp(d.cpu(), g["out"], 1, "golden masked w4a8")


# ----------------------------------------------------------------------------- BF16
def test_masked_bf16():
    gen = torch.Generator().manual_seed(10)
    G, M, N, K = 4, 128, 512, 1024
    a = (torch.randn(G, M, K, generator=gen) * 0.1).bfloat16()
    w = (torch.randn(G, N, K, generator=gen) * 0.1).bfloat16()
    mm = [14, 56, 0, 128]
    packed, cfg = deepgemm.pack_bf16_masked_weight(w.clone().to(DEV))
    d = torch.zeros(G, M, N, dtype=torch.bfloat16, device=DEV)
    r = deepgemm.m_grouped_bf16_gemm_nt_masked(a.to(DEV), packed, d,
                                               torch.tensor(mm, dtype=torch.int32, device=DEV), 128, cfg)
    assert r is d
    d2 = torch.zeros(G, M, N, dtype=torch.bfloat16, device=DEV)          # two-CTA tiles
    _core.grouped_gemm_masked(_cabi.KIND_BF16, _cabi.SCALE_NONE, a.to(DEV), packed, d2, None, None,
                              torch.tensor(mm, dtype=torch.int32, device=DEV), 128, block_n=512)
    ref = O.ref_masked_bf16(a, w)
    for out in (d.cpu(), d2.cpu()):
        for g, m in enumerate(mm):
            if m:
                assert_calc_diff(out[g, :m], ref[g, :m], 1e-3, f"bf16 group {g}")      # calc_diff < 1e-3
                assert torch.allclose(out[g, :m].float(), ref[g, :m].float(), rtol=1e-2, atol=1e-2)
            assert torch.all(out[g, m:] == 0), "tail rows of a zero-initialised output must stay zero"


@pytest.mark.parametrize("active,n,k", [(1, 512, 512), (3, 4096, 384), (2, 1040, 896)])
def test_sparse_routing_narrow_tiles_bit_exact(active, n, k):
    """Few experts with rows: the 128-column kernel narrows its tiles to 64 or 32 columns so that
    every SM streams weights, several K blocks then share a pipeline stage (K / 128 here is not
    always a multiple of that number).  Same parity bar as the wide tiles at each forced width
    and at the width the library picks; idle experts stay untouched."""
    G, max_m = 8, 96
    mm = torch.zeros(G, dtype=torch.int64)
    gen = torch.Generator().manual_seed(40 + active)
    mm[torch.randperm(G, generator=gen)[:active]] = torch.tensor([5, 40, 96])[:active]
    c = gen_masked_int8(G, max_m, n, k, mm, seed=41)
    bp = P.marlin_i8_masked_weight(c["b"].clone())
    for bn in (32, 64, 0):
        _check_int_case(c, _cabi.KIND_I8, c["b"], bp, c["b_scale"], block_n=bn,
                        what=f"sparse: {active} active, N={n}, K={k}, block_n={bn}")


def test_sparse_routing_fp8_narrow_tiles():
    """FP8 at forced narrow widths: integer-valued inputs make the f32 sums order independent,
    so the result must equal the 128-column result bit for bit."""
    mm = [0, 7, 0, 0, 33, 0]
    c = gen_masked_fp8(6, 64, 768, 640, mm, seed=42, integer=True)
    outs = {bn: _run_fp8(c, False, None, block_n=bn) for bn in (128, 64, 32, 0)}
    for bn in (64, 32, 0):
        assert torch.equal(outs[bn].view(torch.int16), outs[128].view(torch.int16)), f"block_n={bn}"
    assert torch.all(outs[32][0].float() == SENTINEL) and torch.all(outs[32][1, 7:].float() == SENTINEL)


def test_tail_round_split_into_half_tiles_bit_exact():
    """256-column tiles, 40 groups x 4 column tiles = 160 items on (at most) 148 SMs: the 12
    items of the second round are computed as 24 half tiles.  Same parity bar; the split must
    not show in the result.  (On a GPU with more SMs than items nothing is split and the test
    still checks the 256-column path.)"""
    G, max_m, n, k = 40, 32, 1024, 384
    gen = torch.Generator().manual_seed(77)
    mm = torch.randint(1, max_m + 1, (G,), generator=gen)
    c = gen_masked_int8(G, max_m, n, k, mm, seed=78)
    bp = P.marlin_i8_masked_weight(c["b"].clone())
    _check_int_case(c, _cabi.KIND_I8, c["b"], bp, c["b_scale"], block_n=256, what="tail split, 256-column tiles")


def test_tail_round_split_with_128_column_tiles():
    """The same split for the 128-column instantiation: 40 groups x 4 tiles of 128 columns."""
    G, max_m, n, k = 40, 32, 512, 256
    gen = torch.Generator().manual_seed(79)
    mm = torch.randint(1, max_m + 1, (G,), generator=gen)
    c = gen_masked_int8(G, max_m, n, k, mm, seed=80)
    bp = P.marlin_i8_masked_weight(c["b"].clone())
    _check_int_case(c, _cabi.KIND_I8, c["b"], bp, c["b_scale"], block_n=128, what="tail split, 128-column tiles")


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_decode_like_sparse_histogram(seed):
    """Row counts drawn the way real decode steps look in the reference's log statistics
    (op_test/generate_masked_m.py:10-41: about 92 % of the (expert, step) pairs have no row, 6 %
    one, 1 % two, a thin tail up to max_m = 32): most experts are idle, so the library's own
    choice (narrow tiles, 32-row activation slices) is what runs.  INT8 bit-exact and FP8
    against the oracle; idle experts untouched."""
    gen = torch.Generator().manual_seed(100 + seed)
    G, max_m, n, k = 64, 32, 1024, 512
    u = torch.rand(G, generator=gen)
    tail = torch.randint(3, max_m + 1, (G,), generator=gen)
    mm = torch.where(u < 0.92, 0, torch.where(u < 0.98, 1, torch.where(u < 0.99, 2, tail)))
    if int(mm.sum()) == 0:
        mm[int(torch.randint(0, G, (1,), generator=gen))] = 1
    c = gen_masked_int8(G, max_m, n, k, mm, seed=200 + seed)
    bp = P.marlin_i8_masked_weight(c["b"].clone())
    _check_int_case(c, _cabi.KIND_I8, c["b"], bp, c["b_scale"], block_n=0, what=f"sparse histogram {mm.tolist()}")
    cf = gen_masked_fp8(G, max_m, n, k, mm, seed=300 + seed)
    d = _run_fp8(cf, False, None, block_n=0)
    ref = O.ref_masked_scaled(cf["a"], cf["b"], cf["a_scale"], cf["b_scale"])
    for g in range(G):
        m = int(mm[g])
        if m:
            assert_calc_diff(d[g, :m], ref[g, :m], 1e-3, f"fp8 sparse group {g}")   # calc_diff < 1e-3
        assert torch.all(d[g, m:].float() == SENTINEL)


@pytest.mark.parametrize("seed", range(24))
def test_random_shapes_and_tile_choices_bit_exact(seed):
    """Seeded random problems over every tile option (library's choice, forced narrow widths,
    one-CTA 128 / 256 columns, two-CTA): group count, rows, N (any multiple of 16) and K vary, a
    third of the groups are empty.  INT8: accumulators bit-exact, output 0 ulp from the exact
    epilogue."""
    gen = torch.Generator().manual_seed(1000 + seed)
    r = lambda lo, hi: int(torch.randint(lo, hi + 1, (1,), generator=gen))
    G, max_m = r(1, 12), r(1, 200)
    n, k = 16 * r(1, 40), 128 * r(1, 6)
    mm = torch.randint(0, max_m + 1, (G,), generator=gen)
    mm[torch.rand(G, generator=gen) < 0.33] = 0
    bn = (0, 32, 64, 128, 256, 512)[seed % 6]
    c = gen_masked_int8(G, max_m, n, k, mm, seed=2000 + seed)
    bp = P.marlin_i8_masked_weight(c["b"].clone())
    _check_int_case(c, _cabi.KIND_I8, c["b"], bp, c["b_scale"], block_n=bn,
                    what=f"random G={G} max_m={max_m} N={n} K={k} block_n={bn} masked_m={mm.tolist()}")


@pytest.mark.parametrize("seed", range(12))
def test_w4a8_random_shapes_bit_exact(seed):
    """Seeded random W4A8 cases: group counts, ragged masked_m with empty experts and experts of
    more than 128 rows (two token tiles), N not a multiple of the 128-channel tile, K of one to
    five 256-value rounds (odd round counts change which unpack group starts an item)."""
    gen = torch.Generator().manual_seed(5000 + seed)
    r = lambda lo, hi: int(torch.randint(lo, hi + 1, (1,), generator=gen))
    G, max_m = r(1, 10), r(1, 300)
    n, k = 16 * r(1, 40), 256 * r(1, 5)
    mm = torch.randint(0, max_m + 1, (G,), generator=gen)
    mm[torch.rand(G, generator=gen) < 0.25] = 0
    order = ("high_first", "low_first")[seed % 2]
    c = gen_masked_w4a8(G, max_m, n, k, mm, seed=6000 + seed, nibble_order=order)
    bp = P.pack_w4a8_moe_hipc_weight(c["b_framework"].clone().to(DEV), nibble_order=order)
    w_x16 = (c["w4"].to(torch.int16) * 16).to(torch.int8)
    _check_int_case(c, _cabi.KIND_W4A8, w_x16, bp, c["b_scale"] / 16.0,
                    what=f"seed {seed}: G={G} max_m={max_m} N={n} K={k} masked_m={mm.tolist()} {order}")


@pytest.mark.parametrize("tensor_wise", [False, True])
def test_overlap_mode_completion_counters(tensor_wise):
    """enable_overlap with a signal tensor: every 128-row block of every expert that has rows ends
    with N credited (a finished tile adds the columns it covers), blocks without rows stay 0, and
    the result is the one the plain call gives.  (The reference declares this mode and refuses it at
    run time: m_grouped_fp8_gemm_nt_maksed_low_latency.cu:1022-1029,1148.)"""
    G, max_m, N, K = 6, 300, 640, 256
    mm = [0, 1, 128, 129, 300, 64]
    c = gen_masked_fp8(G, max_m, N, K, mm, seed=77, tensor_wise=tensor_wise)
    bp = P.marlin_fp8_masked_weight(c["b"].clone().to(DEV))
    fn = deepgemm.m_grouped_fp8_gemm_nt_masked_ll_tensor_wise if tensor_wise else deepgemm.m_grouped_fp8_gemm_nt_masked_ll
    plain = torch.zeros(G, max_m, N, dtype=torch.bfloat16, device=DEV)
    fn((c["a"].to(DEV), c["a_scale"].to(DEV)), (bp, c["b_scale"].to(DEV)), plain, c["masked_m"].to(DEV), 300)
    blocks = (max_m + 127) // 128
    signal = torch.zeros(G, blocks, dtype=torch.int32, device=DEV)
    d = torch.zeros(G, max_m, N, dtype=torch.bfloat16, device=DEV)
    fn((c["a"].to(DEV), c["a_scale"].to(DEV)), (bp, c["b_scale"].to(DEV)), d, c["masked_m"].to(DEV), 300,
       enable_overlap=True, signal=signal)
    torch.cuda.synchronize()
    want = torch.tensor([[N if 128 * b < m else 0 for b in range(blocks)] for m in mm], dtype=torch.int32)
    assert torch.equal(signal.cpu(), want)
    assert torch.equal(d.view(torch.int16), plain.view(torch.int16))
    with pytest.raises(RuntimeError, match="signal"):
        fn((c["a"].to(DEV), c["a_scale"].to(DEV)), (bp, c["b_scale"].to(DEV)), d, c["masked_m"].to(DEV), 300,
           enable_overlap=True)
    with pytest.raises(RuntimeError, match="signal"):
        fn((c["a"].to(DEV), c["a_scale"].to(DEV)), (bp, c["b_scale"].to(DEV)), d, c["masked_m"].to(DEV), 300,
           signal=signal)


@pytest.mark.parametrize("order", ["high_first", "low_first"])
def test_masked_w4a8_shared_memory_unpack_kernel_bit_exact(order):
    """The second W4A8 kernel (tokens on UMMA M, int4 -> int8 unpack in shared memory; block_n =
    512) against the same bar as the default one: ragged masked_m with empty experts and experts of
    more than 128 rows, N that is not a multiple of its 256-channel tile, K of several rounds."""
    mm = [0, 256, 17, 130, 64, 1]
    c = gen_masked_w4a8(6, 256, 640, 1024, mm, seed=19, nibble_order=order)
    bp = P.pack_w4a8_moe_hipc_weight(c["b_framework"].clone().to(DEV), nibble_order=order)
    w_x16 = (c["w4"].to(torch.int16) * 16).to(torch.int8)
    _check_int_case(c, _cabi.KIND_W4A8, w_x16, bp, c["b_scale"] / 16.0, block_n=512,
                    what=f"w4a8 shared-memory unpack {order}")


@pytest.mark.parametrize("K", [64, 192, 448, 7232])
def test_k_an_odd_multiple_of_64(K):
    """The reference's packers and kernels take K % 64 (deepgemm/m_group_gemm.py:815-818).  Here the
    packed weight gets a zero-filled last half block and TMA reads zeros past the end of an
    activation row: int32 accumulators bit-exact through every tile width, also with garbage
    where a kernel reading past the row's end would find it (the next row)."""
    c = gen_masked_int8(3, 128, 272, K, [128, 0, 61], seed=K)
    bp = P.marlin_i8_masked_weight(c["b"].clone())
    assert tuple(bp.shape) == (3, (K + 64) // 128, 272, 128)
    assert bool((bp[:, -1, :, 64:] == 0).all())
    for bn in (0, 128, 256, 512):
        _check_int_case(c, _cabi.KIND_I8, c["b"], bp, c["b_scale"], block_n=bn, what=f"K={K} BN={bn}")
    # FP8, small integers (exact in fp32), public API
    mm = [128, 3, 77]
    f = gen_masked_fp8(3, 128, 256, K, mm, seed=K + 1, integer=True)
    d = _run_fp8(f, False, None)
    ref = O.ref_masked_scaled(f["a"], f["b"], f["a_scale"], f["b_scale"])
    for g, m in enumerate(mm):
        assert_bf16_within_ulp(d[g, :m], ref[g, :m], 0, f"fp8 K={K} group {g}")
