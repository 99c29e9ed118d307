"""The CPU oracle against the golden vectors produced by the reference's own helpers
(tests/golden/make_golden.py).  Bit-exact comparisons: both sides are torch CPU fp32."""
import torch

import dg_oracle as O
from helpers import load_golden


def _same_bits(x, y):
    assert x.dtype == y.dtype and x.shape == y.shape
    xb = x.contiguous().view(torch.int16) if x.dtype == torch.bfloat16 else x
    yb = y.contiguous().view(torch.int16) if y.dtype == torch.bfloat16 else y
    assert torch.equal(xb, yb)


def test_per_token_quant_int8_matches_reference():
    g = load_golden("quant_int8")
    q, s = O.per_token_quant_int8(g["x"])
    assert torch.equal(q, g["q"]) and torch.equal(s, g["scale"])


def test_masked_int8_matches_reference():
    g = load_golden("masked_int8")
    _same_bits(O.ref_masked_scaled(g["a"], g["b"], g["a_scale"], g["b_scale"]), g["out"])


def test_masked_fp8_matches_reference():
    g = load_golden("masked_fp8")
    _same_bits(O.ref_masked_scaled(g["a"], g["b"], g["a_scale"], g["b_scale"]), g["out"])


def test_masked_fp8_tensor_wise_matches_reference():
    g = load_golden("masked_fp8_tensor_wise")
    _same_bits(O.ref_masked_tensor_wise(g["a"], g["b"], g["a_scale"], g["b_scale"]), g["out"])


def test_int4_unpack_and_w4a8_match_reference():
    g = load_golden("masked_w4a8")
    unpacked = O.unpack_int4_to_int8_x16(g["framework"])
    assert torch.equal(unpacked, g["unpacked"])
    # nibble in the high bits == 16 x the signed nibble
    assert torch.equal(unpacked.to(torch.int16), O.signed_int4(g["u4"]).to(torch.int16) * 16)
    _same_bits(O.ref_masked_w4a8(g["a"], g["framework"], g["a_scale"], g["b_scale"]), g["out"])


def test_contiguous_int8_matches_reference():
    g = load_golden("contig_int8")
    _same_bits(O.ref_contiguous(g["a"], g["b"], g["a_scale"], g["b_scale"], g["m_indices"]), g["out"])


def test_contiguous_fp8_matches_reference():
    g = load_golden("contig_fp8")
    _same_bits(O.ref_contiguous(g["a"], g["b"], g["a_scale"], g["b_scale"], g["m_indices"]), g["out"])


def test_contiguous_fp8_tensor_wise_matches_reference():
    # The reference helper for this case accumulates with torch.dot per element, so summation
    # order differs from a matmul: compare within 1 bf16 ulp rather than bit for bit.
    g = load_golden("contig_fp8_tensor_wise")
    got = O.ref_contiguous(g["a"], g["b"], g["a_scale"], g["b_scale"], g["m_indices"],
                           tensor_wise=True)
    assert int(O.bf16_ulp_distance(got, g["out"]).max()) <= 1
    pad = g["m_indices"] < 0
    assert torch.equal(got[pad].float(), torch.zeros_like(got[pad].float()))


def test_exact_accumulator_and_epilogue_agree_with_fp32_reference_on_small_sums():
    # With |acc| < 2^24 the reference's fp32 matmul is exact, so the exact-accumulator route
    # (the one the GPU parity tests use) must reproduce it bit for bit.
    g = load_golden("masked_int8")
    for e in range(g["a"].shape[0]):
        acc = O.exact_int_acc(g["a"][e], g["b"][e])
        assert int(acc.abs().max()) < 2 ** 24
        out = O.epilogue_from_acc(acc, g["a_scale"][e], g["b_scale"][e])
        _same_bits(out, g["out"][e])


def test_calc_diff_and_ulp_helpers():
    x = torch.randn(64, 64)
    assert O.calc_diff(x, x) < 1e-12
    assert abs(O.calc_diff(x, -x) - 2.0) < 1e-9
    a = torch.tensor([1.0, -1.0, 0.0], dtype=torch.bfloat16)
    b = torch.tensor([1.0078125, -1.0078125, 0.0], dtype=torch.bfloat16)
    assert O.bf16_ulp_distance(a, b).tolist() == [1, 1, 0]
    assert O.bf16_ulp_distance(torch.tensor([0.0], dtype=torch.bfloat16),
                               torch.tensor([-0.0], dtype=torch.bfloat16)).tolist() == [0]


def test_contiguous_layout_builder():
    idx, m = O.build_contiguous_layout([3, 0, 256, 257], align=256)
    assert m == 256 + 0 + 256 + 512
    assert idx[:3].tolist() == [0, 0, 0] and int(idx[3]) == -1
    assert int((idx == 3).sum()) == 257 and int((idx == -1).sum()) == m - 3 - 256 - 257


def test_chain_oracle_matches_the_unfused_torch_ops():
    """ref_silu_mul is torch's own bf16 `silu(gate) * up` (two roundings); ref_combine is a plain
    weighted gather-sum; ref_moe_layer with one expert and top-1 reduces to two dequant matmuls."""
    gen = torch.Generator().manual_seed(5)
    x = (torch.randn(64, 256, generator=gen) * 3).bfloat16()
    assert torch.equal(O.ref_silu_mul(x), torch.nn.functional.silu(x[:, :128]) * x[:, 128:])
    y = torch.randn(10, 16, generator=gen).bfloat16()
    src = torch.tensor([[0, 9], [3, -1], [12, 2]], dtype=torch.int32)
    w = torch.tensor([[0.5, 2.0], [1.0, 7.0], [3.0, 0.25]])
    want = torch.stack([0.5 * y[0].double() + 2.0 * y[9].double(), y[3].double(), 0.25 * y[2].double()])
    assert torch.allclose(O.ref_combine(y, src, w), want, rtol=0, atol=1e-12)
    hidden = torch.randn(7, 64, generator=gen).bfloat16()
    w13, s13 = O.per_token_quant_int8(torch.randn(1, 32, 64, generator=gen))
    w2, s2 = O.per_token_quant_int8(torch.randn(1, 64, 16, generator=gen))
    ids = torch.zeros(7, 1, dtype=torch.int64)
    out = O.ref_moe_layer(hidden, ids, torch.full((7, 1), 2.0), w13, s13.reshape(1, -1), w2,
                          s2.reshape(1, -1), kind="int8")
    qa, sa = O.per_token_quant_int8(hidden)
    h = O.ref_masked_scaled(qa[None], w13, sa.reshape(1, -1, 1), s13.reshape(1, -1, 1))[0]
    q, s = O.per_token_quant_int8(O.ref_silu_mul(h))
    y2 = O.ref_masked_scaled(q[None], w2, s.reshape(1, -1, 1), s2.reshape(1, -1, 1))[0]
    assert torch.equal(out.float().bfloat16(), (2.0 * y2.double()).float().bfloat16())


def test_dense_fp8_matches_reference():
    g = load_golden("dense_fp8")
    out = O.ref_dense_scaled(g["a"], g["b"], g["a_scale"], g["b_scale"], torch.bfloat16)
    assert torch.equal(out.view(torch.int16), g["out"].view(torch.int16))
    out16 = O.ref_dense_scaled(g["a"], g["b"], g["a_scale"], g["b_scale"], torch.float16)
    assert torch.equal(out16.view(torch.int16), g["out_f16"].view(torch.int16))


def test_sorted_routing_oracle_equals_the_per_pair_formula():
    """build_sorted_routing + ref_prefill_down (block walk of the reference kernel) give every
    (token, slot) row the plain formula; rows of experts marked remote are zero."""
    g = torch.Generator().manual_seed(0)
    t, k, e, hid, n = 50, 3, 5, 64, 32
    topk = torch.rand(t, e, generator=g).topk(k, dim=1).indices
    ids, ex, used = O.build_sorted_routing(topk, e, 16, local_experts={0, 1, 2, 4}, extra_blocks=1)
    assert ids.numel() % 16 == 0 and ex.numel() == ids.numel() // 16 and int(used) == ids.numel() - 16
    inp = torch.randint(-128, 128, (t * k, hid), generator=g).to(torch.int8)
    w = torch.randint(-128, 128, (e, n, hid), generator=g).to(torch.int8)
    a_s, b_s, tw = torch.rand(t * k, generator=g), torch.rand(e, n, generator=g), torch.rand(t, k, generator=g)
    out = O.ref_prefill_down(inp, w, a_s, b_s, tw, ids, ex, used, k,
                             torch.full((t * k, n), 9.0, dtype=torch.bfloat16))
    for tok in range(t):
        for s in range(k):
            r, ee = tok * k + s, int(topk[tok, s])
            want = ((inp[r].double() @ w[ee].double().t()).float() * (tw[tok, s] * a_s[r])) * b_s[ee]
            want = torch.zeros(n) if ee == 3 else want
            assert torch.equal(out[r], want.bfloat16()), (tok, s)


def test_w4a8_signed_nibble_convention_matches_reference():
    """The expectation the reference's HIPC W4A8 tests compute inline (signed nibbles, the op
    gets w_scale / 16), masked and contiguous, bf16 and fp16 outputs."""
    g = load_golden("masked_w4a8_hipc")
    assert torch.equal(O.signed_int4(g["u4"]).to(torch.int16) * 16,
                       O.unpack_int4_to_int8_x16(g["framework"]).to(torch.int16))
    _same_bits(O.ref_masked_w4a8_hipc(g["a"], g["framework"], g["a_scale"], g["w_scale"]), g["out"])
    got16 = O.ref_masked_w4a8_hipc(g["a"], g["framework"], g["a_scale"], g["w_scale"], torch.float16)
    assert torch.equal(got16.view(torch.int16), g["out_f16"].view(torch.int16))
    # what the kernel computes, 16 x nibble with w_scale / 16, is the same number bit for bit
    _same_bits(O.ref_masked_w4a8(g["a"], g["framework"], g["a_scale"], g["kernel_w_scale"]), g["out"])
    c = load_golden("contig_w4a8_hipc")
    _same_bits(O.ref_contiguous_w4a8_hipc(c["a"], c["framework"], c["a_scale"], c["w_scale"], c["m_indices"]),
               c["out"])
    got16 = O.ref_contiguous_w4a8_hipc(c["a"], c["framework"], c["a_scale"], c["w_scale"], c["m_indices"],
                                       torch.float16)
    assert torch.equal(got16.view(torch.int16), c["out_f16"].view(torch.int16))


def test_masked_bf16_matches_reference():
    g = load_golden("masked_bf16")
    m = int(g["masked_m"][0])
    got = O.ref_masked_bf16(g["a"], g["b"])
    _same_bits(got[:, :m].contiguous(), g["out"][:, :m].contiguous())
    assert bool((g["out"][:, m:] == 0).all())


def test_logged_routing_vectors_fixture():
    g = load_golden("skew_masked_m")
    mm = g["masked_m"]
    assert tuple(mm.shape) == (6, 36) and int(mm.max()) == 16384
    assert int((mm == 0).sum()) > 20          # many experts without a row, a few with thousands
