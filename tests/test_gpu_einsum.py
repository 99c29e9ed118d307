"""einsum / fp8_einsum against torch.einsum on the dequantised operands (the reference's own
check, op_test/test_einsum.py:41-62,134-170).  Tolerance: calc_diff < 1e-3 (fp32 accumulation
order differs from torch's); integer-valued inputs with unit scales must be exact."""
import pytest
import torch

import deepgemm

import dg_oracle as O
from helpers import assert_calc_diff

pytestmark = pytest.mark.gpu
DEV = "cuda"
FP8 = torch.float8_e4m3fn


def _cast_rows(x):                                   # per-row (last dim) e4m3 quantisation
    q, s = O.per_token_quant_fp8(x)
    return q, s.reshape(x.shape[:-1])


@pytest.mark.parametrize("b,h,r,d", [(48, 4, 512, 128), (7, 16, 256, 128)])
def test_fp8_bhr_hdr_bhd_and_bhd_hdr_bhr(b, h, r, d):
    g = torch.Generator().manual_seed(b + h)
    x, y = torch.randn(b, h, r, generator=g), torch.randn(h, d, r, generator=g)
    qx, sx = _cast_rows(x)
    qy, sy = _cast_rows(y)
    out = torch.zeros(b, h, d, dtype=torch.bfloat16, device=DEV)
    deepgemm.fp8_einsum("bhr,hdr->bhd", (qx.to(DEV), sx.to(DEV)), (qy.to(DEV), sy.to(DEV)), out)
    ref = torch.einsum("bhr,hdr->bhd", qx.float() * sx[..., None], qy.float() * sy[..., None])
    assert_calc_diff(out.cpu().float(), ref, 1e-3, "fp8 bhr,hdr->bhd")
    # bhd,hdr->bhr: B scaled per (h, r), i.e. per column of the [d, r] matrix
    x2 = torch.randn(b, h, d, generator=g)
    qx2, sx2 = _cast_rows(x2)
    sy2 = y.abs().amax(dim=1).clamp_min(1e-4) / 448.0
    qy2 = (y / sy2.unsqueeze(1)).clamp(-448, 448).to(FP8)
    out2 = torch.zeros(b, h, r, dtype=torch.bfloat16, device=DEV)
    deepgemm.fp8_einsum("bhd,hdr->bhr", (qx2.to(DEV), sx2.to(DEV)), (qy2.to(DEV), sy2.to(DEV)), out2)
    ref2 = torch.einsum("bhd,hdr->bhr", qx2.float() * sx2[..., None], qy2.float() * sy2.unsqueeze(1))
    assert_calc_diff(out2.cpu().float(), ref2, 1e-3, "fp8 bhd,hdr->bhr")


def test_fp8_bhd_bhr_hdr_with_accumulator_and_ragged_batch():
    """K is the batch dimension here (100: padded to 128 inside); fp32 d with c accumulates."""
    g = torch.Generator().manual_seed(3)
    b, h, d, r = 100, 3, 128, 256
    x = torch.randint(-3, 4, (b, h, d), generator=g).float()
    y = torch.randint(-3, 4, (b, h, r), generator=g).float()
    ones_hd, ones_hr = torch.ones(h, d), torch.ones(h, r)
    c = torch.randn(h, d, r, generator=g)
    out = torch.zeros(h, d, r, dtype=torch.float32, device=DEV)
    deepgemm.fp8_einsum("bhd,bhr->hdr", (x.to(FP8).to(DEV), ones_hd.to(DEV)), (y.to(FP8).to(DEV), ones_hr.to(DEV)),
                        out, c.to(DEV))
    ref = c + torch.einsum("bhd,bhr->hdr", x, y)
    assert torch.equal(out.cpu(), ref)                           # small integers: exact


def test_bf16_einsum_expressions():
    g = torch.Generator().manual_seed(5)
    s, m, n, k = 6, 96, 80, 192
    a, b = torch.randn(s, m, k, generator=g).bfloat16(), torch.randn(s, n, k, generator=g).bfloat16()
    d = torch.zeros(m, n, dtype=torch.bfloat16, device=DEV)
    deepgemm.einsum("bmk,bnk->mn", a.to(DEV), b.to(DEV), d)
    ref = torch.einsum("bmk,bnk->mn", a.float(), b.float())
    assert_calc_diff(d.cpu().float(), ref, 1e-3, "bf16 bmk,bnk->mn")
    c = torch.randn(m, n, generator=g)
    d32 = c.clone().to(DEV)
    deepgemm.einsum("bmk,bnk->mn", a.to(DEV), b.to(DEV), d32, d32)
    assert_calc_diff(d32.cpu(), c + ref, 1e-3, "bf16 bmk,bnk->mn with accumulator")
    bb, h, r, dd = 20, 4, 128, 64
    x, y = torch.randn(bb, h, r, generator=g).bfloat16(), torch.randn(h, dd, r, generator=g).bfloat16()
    o = torch.zeros(bb, h, dd, dtype=torch.bfloat16, device=DEV)
    deepgemm.einsum("bhr,hdr->bhd", x.to(DEV), y.to(DEV), o)
    assert_calc_diff(o.cpu().float(), torch.einsum("bhr,hdr->bhd", x.float(), y.float()), 1e-3, "bf16 bhr,hdr->bhd")
    x2 = torch.randn(bb, h, dd, generator=g).bfloat16()
    o2 = torch.zeros(bb, h, r, dtype=torch.bfloat16, device=DEV)
    deepgemm.einsum("bhd,hdr->bhr", x2.to(DEV), y.to(DEV), o2)
    assert_calc_diff(o2.cpu().float(), torch.einsum("bhd,hdr->bhr", x2.float(), y.float()), 1e-3, "bf16 bhd,hdr->bhr")


def test_unsupported_expression_and_types():
    x = torch.zeros(2, 2, 128, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(RuntimeError):
        deepgemm.einsum("abc,abd->cd", x, x, x)
    with pytest.raises(ValueError):
        deepgemm.einsum("bhr,hdr->bhd", x.float(), x, x)
    with pytest.raises(ValueError):
        deepgemm.fp8_einsum("bhr,hdr->bhd", (x, x), (x, x), x)
