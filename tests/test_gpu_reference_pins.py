"""GPU parity on the fixtures made from the reference's remaining pins (tests/golden/make_golden.py
items 10-13): the signed-nibble W4A8 convention of the HIPC ops with bf16 and fp16 outputs, masked
BF16, and the six routing vectors logged from a serving run (36 experts, one with 16 384 rows).
Also the BF16 configuration the reference benchmarks (16 experts, M = 2048, (N, K) = (2048, 6144)),
checked on sampled rows and timed."""
import pytest
import torch

import deepgemm
from deepgemm import _cabi, _core
from deepgemm import group_gemm_weight_pack as P

import dg_oracle as O
from helpers import assert_bf16_within_ulp, assert_calc_diff, load_golden

pytestmark = pytest.mark.gpu
DEV = "cuda"
SENTINEL = 17.0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_masked_w4a8_hipc_golden(dtype):
    """The op is given w_scale / 16 and multiplies by 16 x the nibble: bit for bit the number the
    reference's expectation holds (both scalings are by powers of two)."""
    g = load_golden("masked_w4a8_hipc")
    E, M, K = g["a"].shape
    N = g["framework"].shape[1]
    bp = P.pack_w4a8_moe_hipc_weight(g["framework"].clone().to(DEV))
    mm = torch.tensor([M, 17], dtype=torch.int32, device=DEV)
    want = g["out"] if dtype == torch.bfloat16 else g["out_f16"]
    for fn in (deepgemm.m_grouped_w4a8_gemm_nt_masked_hipc, deepgemm.m_grouped_w4a8_gemm_nt_masked):
        d = torch.full((E, M, N), SENTINEL, dtype=dtype, device=DEV)
        r = fn((g["a"].to(DEV), g["a_scale"].to(DEV)), (bp, g["kernel_w_scale"].to(DEV)), d, mm, M)
        assert r is d
        d = d.cpu()
        for e, m in enumerate(mm.tolist()):
            assert torch.equal(d[e, :m].view(torch.int16), want[e, :m].view(torch.int16)), f"expert {e}"
            assert torch.all(d[e, m:].float() == SENTINEL)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_contiguous_w4a8_hipc_golden(dtype):
    g = load_golden("contig_w4a8_hipc")
    bp = P.pack_w4a8_moe_hipc_weight(g["framework"].clone().to(DEV))
    mt, n = g["a"].shape[0], g["framework"].shape[1]
    want = g["out"] if dtype == torch.bfloat16 else g["out_f16"]
    d = torch.full((mt, n), SENTINEL, dtype=dtype, device=DEV)
    deepgemm.m_grouped_w4a8_gemm_nt_contiguous_hipc(
        (g["a"].to(DEV), g["a_scale"].to(DEV)), (bp, g["kernel_w_scale"].to(DEV)), d, g["m_indices"].to(DEV))
    d = d.cpu()
    valid = g["m_indices"] >= 0
    assert torch.equal(d[valid].view(torch.int16), want[valid].view(torch.int16))
    assert torch.all(d[~valid].float() == SENTINEL)


def test_w4a8_fp16_output_other_kinds_reject():
    a = torch.zeros(2, 8, 128, dtype=torch.int8, device=DEV)
    b = P.marlin_i8_masked_weight(torch.zeros(2, 16, 128, dtype=torch.int8, device=DEV))
    d = torch.zeros(2, 8, 16, dtype=torch.float16, device=DEV)
    with pytest.raises(RuntimeError, match="bfloat16"):
        deepgemm.m_grouped_w8a8_gemm_nt_masked((a, torch.ones(2, 8, device=DEV)), (b, torch.ones(2, 16, device=DEV)),
                                               d, torch.zeros(2, dtype=torch.int32, device=DEV), 8)


def test_masked_bf16_golden():
    g = load_golden("masked_bf16")
    packed, cfg = deepgemm.pack_bf16_masked_weight(g["b"].clone().to(DEV))
    d = torch.zeros(g["out"].shape, dtype=torch.bfloat16, device=DEV)
    m = int(g["masked_m"][0])
    deepgemm.m_grouped_bf16_gemm_nt_masked(g["a"].to(DEV), packed, d, g["masked_m"].to(DEV), m, cfg)
    d = d.cpu()
    assert_calc_diff(d[:, :m], g["out"][:, :m], 1e-3, "masked bf16 golden")                 # calc_diff < 1e-3
    assert torch.allclose(d[:, :m].float(), g["out"][:, :m].float(), rtol=1e-2, atol=1e-2)   # the reference's own bar
    assert torch.all(d[:, m:] == 0), "tail rows of a zero-initialised output stay zero"


@pytest.mark.parametrize("active_m", [14, 112])
def test_masked_bf16_reference_benchmark_shape(active_m):
    """16 experts, M = 2048, N = 2048, K = 6144 (op_test/test_deepgemm_masked_w16a16_bf16.py:11-20)."""
    E, M, N, K = 16, 2048, 2048, 6144
    gen = torch.Generator(device=DEV).manual_seed(5)
    a = (torch.randn(E, M, K, device=DEV, generator=gen) * 0.1).bfloat16()
    w = (torch.randn(E, N, K, device=DEV, generator=gen) * 0.1).bfloat16()
    w_rows = w[::5].cpu()
    packed, cfg = deepgemm.pack_bf16_masked_weight(w)
    mm = torch.full((E,), active_m, dtype=torch.int32, device=DEV)
    d = torch.zeros(E, M, N, dtype=torch.bfloat16, device=DEV)
    deepgemm.m_grouped_bf16_gemm_nt_masked(a, packed, d, mm, active_m, cfg)
    for i, e in enumerate(range(0, E, 5)):
        ref = O.ref_masked_bf16(a[e:e + 1, :active_m].cpu(), w_rows[i:i + 1])[0]
        assert_calc_diff(d[e, :active_m].cpu(), ref, 1e-3, f"bf16 expert {e}")
    assert bool((d[:, active_m:] == 0).all())
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(5):
        deepgemm.m_grouped_bf16_gemm_nt_masked(a, packed, d, mm, active_m, cfg)
    e0.record()
    for _ in range(20):
        deepgemm.m_grouped_bf16_gemm_nt_masked(a, packed, d, mm, active_m, cfg)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) / 20 * 1e3
    gbs = E * (active_m * K + N * K + active_m * N) * 2 / (us * 1e-6) / 1e9      # the reference's own byte count
    print(f"masked bf16 E=16 N=2048 K=6144 masked_m={active_m}: {us:.1f} us, {gbs:.0f} GB/s")
    assert gbs > 1000


@pytest.mark.parametrize("case", range(6))
def test_logged_routing_vectors_int8(case):
    """Rows per expert as logged from a serving run (36 experts; thousands of rows in a few, none in
    most), max_m = 16 384, at small N and K: int32 accumulators bit-exact on every row of the
    smaller experts and on sampled rows of the big ones, no row beyond masked_m written."""
    g = load_golden("skew_masked_m")
    mm = g["masked_m"][case].to(torch.int32)
    G, max_m, N, K = mm.numel(), 16384, 256, 256
    gen = torch.Generator(device=DEV).manual_seed(90 + case)
    a = torch.randint(-127, 128, (G, max_m, K), dtype=torch.int8, device=DEV, generator=gen)
    a_s = torch.rand(G, max_m, device=DEV, generator=gen) + 0.5
    b = torch.randint(-127, 128, (G, N, K), dtype=torch.int8, device=DEV, generator=gen)
    b_s = torch.rand(G, N, device=DEV, generator=gen) + 0.5
    b_rows = b.cpu()
    bp = P.marlin_i8_masked_weight(b)
    d = torch.full((G, max_m, N), SENTINEL, dtype=torch.bfloat16, device=DEV)
    acc = torch.full((G, max_m, N), -12345, dtype=torch.int32, device=DEV)
    deepgemm.check_device_status()
    _core.grouped_gemm_masked(_cabi.KIND_I8, 0, a, bp, d, a_s, b_s, mm.to(DEV), int(mm.max()), debug_acc=acc)
    deepgemm.check_device_status()
    for e in range(G):
        m = int(mm[e])
        rows = torch.arange(m) if m <= 600 else torch.cat([torch.arange(300), torch.arange(m - 300, m),
                                                           torch.randint(0, m, (200,))])
        if m:
            want = O.exact_int_acc(a[e, rows.to(DEV)].cpu(), b_rows[e])
            assert torch.equal(acc[e, rows.to(DEV)].cpu(), want), f"expert {e} ({m} rows)"
            out = O.epilogue_from_acc(want, a_s[e, rows.to(DEV)].cpu(), b_s[e].cpu())
            assert_bf16_within_ulp(d[e, rows.to(DEV)].cpu(), out, 0, f"expert {e}")
        assert bool((d[e, m:].float() == SENTINEL).all()) and bool((acc[e, m:] == -12345).all())


def test_device_status_is_reported_to_public_api_callers():
    """No public call fails silently: a row block whose m_indices entry names no expert is skipped
    and check_device_status() says so once."""
    from helpers import gen_contig
    c = gen_contig("int8", [128, 128], 128, 128, seed=27, align=128)
    bad = c["m_indices"].clone()
    bad[128:] = 9
    bp = P.marlin_i8_contiguous_weight(c["b"].clone().to(DEV))
    d = torch.full((256, 128), SENTINEL, dtype=torch.bfloat16, device=DEV)
    deepgemm.check_device_status()
    deepgemm.m_grouped_i8_gemm_nt_contiguous((c["a"].to(DEV), c["a_scale"].to(DEV)),
                                             (bp, c["b_scale"].to(DEV)), d, bad.to(DEV))
    with pytest.raises(RuntimeError, match="outside"):
        deepgemm.check_device_status()
    deepgemm.check_device_status()                      # cleared by the call that reported it
    assert torch.all(d[128:].float() == SENTINEL)
