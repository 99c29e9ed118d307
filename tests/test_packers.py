"""Weight packers on CPU tensors: layout definition, in-place contract, exact inverse,
argument errors (reference contract: deepgemm/group_gemm_weight_pack.py:483-602,691-769)."""
import pytest
import torch

import deepgemm
from deepgemm import _cabi
from deepgemm import group_gemm_weight_pack as P

import dg_oracle as O


def test_int8_layout_is_kblock_major_and_in_place():
    w = torch.randint(-128, 128, (3, 48, 384), dtype=torch.int8)
    w0 = w.clone()
    p = P.marlin_i8_masked_weight(w)
    assert p.shape == (3, 3, 48, 128) and p.data_ptr() == w.data_ptr()
    for e, kb, n in [(0, 0, 0), (1, 2, 47), (2, 1, 13)]:
        assert torch.equal(p[e, kb, n], w0[e, n, kb * 128:(kb + 1) * 128])
    assert torch.equal(P.unpack_weight(p, _cabi.KIND_I8), w0)
    # every alias produces the same bytes
    for fn in (P.marlin_i8_contiguous_weight, P.pack_i8_masked_weight, P.pack_i8_contiguous_weight,
               P.pack_int8_weight_enk_to_w6_low_latency, deepgemm.pack_int8_weight_enk_to_w6_low_latency_inplace):
        assert torch.equal(fn(w0.clone()), p)


def test_fp8_pack_keeps_dtype_and_bytes():
    w = torch.randn(2, 32, 256).to(torch.float8_e4m3fn)
    w0 = w.clone()
    p = P.marlin_fp8_masked_weight(w)
    assert p.dtype == torch.float8_e4m3fn and p.shape == (2, 2, 32, 128)
    assert torch.equal(P.unpack_weight(p, _cabi.KIND_E4M3).view(torch.uint8), w0.view(torch.uint8))
    assert torch.equal(P.marlin_fp8_contiguous_weight(w0.clone()).view(torch.uint8), p.view(torch.uint8))


def test_bf16_pack_returns_config_and_inverts():
    w = torch.randn(2, 32, 192).bfloat16()
    w0 = w.clone()
    p, cfg = P.pack_bf16_masked_weight(w)
    assert p.shape == (2, 3, 32, 64) and cfg["PACKED_WEIGHT"] is True and cfg["MODE"] == 2000
    assert torch.equal(p[1, 2, 5], w0[1, 5, 128:192])
    assert torch.equal(P.unpack_weight(p, _cabi.KIND_BF16), w0)
    with pytest.raises(ValueError):
        P.pack_bf16_masked_weight(w0.clone(), mode=7)
    with pytest.raises(TypeError):
        P.pack_bf16_masked_weight(w0.float())


@pytest.mark.parametrize("order", ["high_first", "low_first"])
def test_int4_layout_pairs_nibbles_for_the_unpack_rule(order):
    g = torch.Generator().manual_seed(3)
    u4 = torch.randint(0, 16, (2, 32, 512), generator=g).to(torch.int8)
    fw = P.pack_w4a8_weight_k_contiguous(u4)          # high nibble = even k
    if order == "low_first":
        b = fw.view(torch.uint8)
        fw = (((b & 0xF) << 4) | (b >> 4)).view(torch.int8)
    fw0 = fw.clone()
    pk = P.pack_w4a8_moe_hipc_weight(fw, nibble_order=order)
    assert pk.shape == fw0.shape and pk.data_ptr() == fw.data_ptr()
    v = P.view_w4a8_moe_hipc_weight_n32_layout(pk).view(torch.uint8)
    assert v.shape == (2, 2, 32, 128)
    # applying the kernel's two-instruction unpack to the packed bytes must give 16 x w in K order
    hi = (v & 0xF0).view(2, 2, 32, 8, 16)
    lo = ((v << 4) & 0xF0).view(2, 2, 32, 8, 16)
    int8_tile = torch.stack((hi, lo), dim=-2).reshape(2, 2, 32, 256)      # [e][kb][n][k in block]
    k_major = int8_tile.permute(0, 2, 1, 3).reshape(2, 32, 512).view(torch.int8)
    assert torch.equal(k_major.to(torch.int16), O.signed_int4(u4).to(torch.int16) * 16)
    assert torch.equal(k_major, O.unpack_int4_to_int8_x16(fw0, order))
    assert torch.equal(P.unpack_weight(pk, _cabi.KIND_W4A8, nibble_order=order), fw0)


def test_reference_framework_packer_matches_golden():
    from helpers import load_golden
    g = load_golden("masked_w4a8")
    assert torch.equal(P.pack_w4a8_weight_k_contiguous(g["u4"]), g["framework"])


def test_k_an_odd_multiple_of_64_gets_a_zero_filled_last_block():
    """K % 128 == 64 (accepted by the reference's packers, deepgemm/m_group_gemm.py:815-818): the
    packed tensor is a new one with ceil(K / 128) blocks, the tail of the last block is zero and
    the first K columns unpack to the source."""
    g = torch.Generator().manual_seed(3)
    w = torch.randint(-128, 128, (2, 32, 192), generator=g).to(torch.int8)
    src = w.clone()
    packed = P.marlin_i8_contiguous_weight(w)
    assert tuple(packed.shape) == (2, 2, 32, 128)
    assert torch.equal(w, src), "the source is left alone when the packed tensor cannot share its storage"
    back = P.unpack_weight(packed, P.KIND_I8)
    assert torch.equal(back[:, :, :192], src) and bool((back[:, :, 192:] == 0).all())
    f = (torch.randn(1, 16, 64, generator=g)).to(torch.float8_e4m3fn)
    pf = P.marlin_fp8_masked_weight(f.clone())
    assert tuple(pf.shape) == (1, 1, 16, 128) and pf.dtype == torch.float8_e4m3fn
    assert torch.equal(pf.view(torch.uint8)[0, 0, :, :64], f.view(torch.uint8)[0])
    assert bool((pf.view(torch.uint8)[0, 0, :, 64:] == 0).all())


def test_packer_argument_errors():
    with pytest.raises(ValueError):
        P.marlin_i8_masked_weight(torch.zeros(2, 32, 100, dtype=torch.int8))       # K % 64
    with pytest.raises(ValueError):
        P.marlin_i8_masked_weight(torch.zeros(2, 30, 128, dtype=torch.int8))       # N % 16
    with pytest.raises(ValueError):
        P.marlin_i8_masked_weight(torch.zeros(2, 32, 128, dtype=torch.int16))      # not 8-bit
    with pytest.raises(ValueError):
        P.marlin_i8_masked_weight(torch.zeros(2, 32, 256, dtype=torch.int8)[:, :, ::2])  # strided
    with pytest.raises(ValueError):
        P.marlin_i8_masked_weight(torch.zeros(2, 32, 128, dtype=torch.int8), shuffle_unique=2)
    with pytest.raises(ValueError):
        P.marlin_i8_contiguous_weight(torch.zeros(2, 32, 128, dtype=torch.int8), mode=5)
    with pytest.raises(ValueError):
        P.marlin_i8_contiguous_weight(torch.zeros(2, 32, 128, dtype=torch.int8), mode=2, shuffle_unique=0)
    with pytest.raises(ValueError):
        P.pack_w4a8_weight_k_contiguous(torch.zeros(2, 32, 7, dtype=torch.int8))
    with pytest.raises(ValueError):
        P.pack_w4a8_moe_hipc_weight(torch.zeros(2, 32, 64, dtype=torch.int8))      # K/2 % 128
    with pytest.raises(ValueError):
        P.pack_w4a8_moe_hipc_weight(torch.zeros(2, 32, 128, dtype=torch.int16))
    with pytest.raises(ValueError):
        P.pack_w4a8_moe_hipc_weight(torch.zeros(2, 32, 128, dtype=torch.int8), nibble_order="middle")
    with pytest.raises(ValueError):
        P.view_w4a8_moe_hipc_weight_n32_layout(torch.zeros(32, 64, dtype=torch.int8))
