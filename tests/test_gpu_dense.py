"""Dense (batched) GEMM front-ends fp8_gemm / fp8_gemm_hipc against the CPU oracle.

Shapes follow the reference's op_test/test_fp8_gemm.py:66-72 (including N = 342, which is not
a multiple of 8, and M = 1) and its output types.  Tolerance: calc_diff < 1e-3 (the reference
itself only asks for atol = 1); small-integer inputs with unit scales must be exact."""
import pytest
import torch

import deepgemm

import dg_oracle as O
from helpers import assert_calc_diff, load_golden

pytestmark = pytest.mark.gpu
DEV = "cuda"
FP8 = torch.float8_e4m3fn


def _operands(m, n, k, seed, dtype=FP8):
    g = torch.Generator().manual_seed(seed)
    if dtype == torch.int8:
        a = torch.randint(-128, 128, (m, k), generator=g).to(torch.int8)
        b = torch.randint(-128, 128, (n, k), generator=g).to(torch.int8)
    else:
        a = (torch.randn(m, k, generator=g) * 0.5).to(FP8)
        b = (torch.randn(n, k, generator=g) * 0.5).to(FP8)
    sa = torch.randn(m, generator=g).abs() * 0.01 + 0.01
    sb = torch.randn(n, generator=g).abs() * 0.01 + 0.01
    return a, b, sa, sb


@pytest.mark.parametrize("m,n,k", [(168, 342, 512), (1, 16, 1024), (128, 128, 1024), (512, 512, 1024),
                                   (1024, 1024, 4096)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float16])
def test_fp8_gemm_accuracy(m, n, k, out_dtype):
    a, b, sa, sb = _operands(m, n, k, m + n)
    d = torch.full((m, n), 7.0, dtype=out_dtype, device=DEV)
    assert deepgemm.fp8_gemm((a.to(DEV), sa.to(DEV)), (b.to(DEV), sb.to(DEV)), d) is None
    ref = O.ref_dense_scaled(a, b, sa, sb, torch.float32)
    assert_calc_diff(d.cpu().float(), ref, 1e-3, f"fp8_gemm {m}x{n}x{k} {out_dtype}")   # calc_diff < 1e-3


def test_golden_dense_fp8():
    g = load_golden("dense_fp8")
    m, n = g["out"].shape
    for dt, key in ((torch.bfloat16, "out"), (torch.float16, "out_f16")):
        d = torch.zeros(m, n, dtype=dt, device=DEV)
        deepgemm.fp8_gemm((g["a"].to(DEV), g["a_scale"].to(DEV)), (g["b"].to(DEV), g["b_scale"].to(DEV)), d)
        assert_calc_diff(d.cpu().float(), g[key].float(), 1e-3, f"golden dense {dt}")


def test_int8_fp32_out_batched_is_exact():
    """int8 operands, unit scales, fp32 output: every element is the exact integer dot product
    (|acc| < 2^24 here), for each batch entry, through both tile kernels."""
    batch, m, n, k = 3, 300, 264, 256
    g = torch.Generator().manual_seed(4)
    a = torch.randint(-8, 9, (batch, m, k), generator=g).to(torch.int8)
    b = torch.randint(-8, 9, (batch, n, k), generator=g).to(torch.int8)
    ones_m, ones_n = torch.ones(batch, m), torch.ones(batch, n)
    want = torch.stack([O.exact_int_acc(a[i], b[i]).float() for i in range(batch)])
    d = torch.zeros(batch, m, n, dtype=torch.float32, device=DEV)
    deepgemm.fp8_gemm((a.to(DEV), ones_m.to(DEV)), (b.to(DEV), ones_n.to(DEV)), d)
    assert torch.equal(d.cpu(), want)
    d16 = torch.zeros(batch, m, n, dtype=torch.bfloat16, device=DEV)        # vector-store path (N % 8 == 0)
    deepgemm.fp8_gemm((a.to(DEV), ones_m.to(DEV)), (b.to(DEV), ones_n.to(DEV)), d16)
    assert torch.equal(d16.cpu(), want.bfloat16())


def test_identity_scales_and_large_shape_use_the_two_cta_tiles():
    """Empty scale tensors mean no scaling (reference gemm.py:66-68); 16 x 10 tiles of 256 x 256
    are enough for the two-CTA kernel to be chosen, which must read row-major weights as well."""
    m, n, k = 4096, 2560, 256
    g = torch.Generator().manual_seed(8)
    a = torch.randint(-4, 5, (m, k), generator=g).float().to(FP8)
    b = torch.randint(-4, 5, (n, k), generator=g).float().to(FP8)
    empty = torch.empty(0, device=DEV)
    d = torch.zeros(m, n, dtype=torch.bfloat16, device=DEV)
    deepgemm.fp8_gemm_hipc((a.to(DEV), empty), (b.to(DEV), empty), d)
    want = (a.float() @ b.float().t()).bfloat16()          # small integers: exact in fp32
    assert torch.equal(d.cpu(), want)


def test_argument_errors():
    a = torch.zeros(16, 128, dtype=torch.bfloat16, device=DEV)
    d = torch.zeros(16, 16, dtype=torch.bfloat16, device=DEV)
    e = torch.empty(0, device=DEV)
    with pytest.raises(ValueError):
        deepgemm.fp8_gemm((a, e), (a, e), d)                              # bf16 operands
    q = a.to(FP8)
    with pytest.raises(ValueError):
        deepgemm.fp8_gemm_hipc((q.view(torch.int8), e), (q.view(torch.int8), e), d)   # int8 on the fp8-only entry
    with pytest.raises(ValueError):
        deepgemm.fp8_gemm((q, e), (q[:, :64].contiguous(), e), d)         # K mismatch
    with pytest.raises(RuntimeError):
        deepgemm.fp8_gemm((q[:, :32].contiguous(), e), (q[:, :32].contiguous(), e), d)   # K % 64 != 0
    with pytest.raises(RuntimeError):
        deepgemm.fp8_gemm((q.cpu(), e.cpu()), (q.cpu(), e.cpu()), d.cpu())


@pytest.mark.parametrize("k", [64, 192, 1088])
def test_dense_k_an_odd_multiple_of_64(k):
    m, n = 130, 264
    g = torch.Generator().manual_seed(k)
    a = torch.randint(-8, 9, (m, k), generator=g).to(torch.int8)
    b = torch.randint(-8, 9, (n, k), generator=g).to(torch.int8)
    d = torch.zeros(m, n, dtype=torch.float32, device=DEV)
    deepgemm.fp8_gemm((a.to(DEV), torch.ones(m, device=DEV)), (b.to(DEV), torch.ones(n, device=DEV)), d)
    assert torch.equal(d.cpu(), O.exact_int_acc(a, b).float())
