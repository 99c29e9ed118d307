"""Host-side behaviour of the Python entry points that needs no GPU: argument handling and
the exception types the reference raises for the same mistakes
(deepgemm/m_group_gemm_nt_masked.py:158-161,226-227; deepgemm/m_group_gemm.py:132-162,215-216,319-329;
deepgemm/m_group_gemm_nt_contiguous.py:72-84,398-402)."""
import pytest
import torch

import deepgemm
from deepgemm import group_gemm_weight_pack as P

FP8 = torch.float8_e4m3fn


def _masked_int8_args(G=2, M=8, N=32, K=128):
    a = (torch.zeros(G, M, K, dtype=torch.int8), torch.ones(G, M))
    b = (P.marlin_i8_masked_weight(torch.zeros(G, N, K, dtype=torch.int8)), torch.ones(G, N))
    d = torch.zeros(G, M, N, dtype=torch.bfloat16)
    return a, b, d, torch.full((G,), M, dtype=torch.int32)


def test_public_names_exist():
    for name in ["m_grouped_w8a8_gemm_nt_masked", "m_grouped_fp8_gemm_nt_masked",
                 "m_grouped_fp8_gemm_nt_masked_ll", "m_grouped_fp8_gemm_nt_masked_tensor_wise",
                 "m_grouped_fp8_gemm_nt_masked_ll_tensor_wise", "m_grouped_w4a8_gemm_nt_masked",
                 "m_grouped_w4a8_gemm_nt_masked_hipc", "m_grouped_bf16_gemm_nt_masked",
                 "m_grouped_i8_gemm_nt_masked", "m_grouped_w8a8_gemm_nt_masked_impl",
                 "m_grouped_i8_gemm_nt_contiguous", "m_grouped_fp8_gemm_nt_contiguous",
                 "m_grouped_fp8_gemm_nt_contiguous_tensor_wise",
                 "m_grouped_w4a8_gemm_nt_contiguous_hipc", "marlin_i8_masked_weight",
                 "marlin_i8_contiguous_weight", "marlin_fp8_masked_weight",
                 "marlin_fp8_contiguous_weight", "pack_bf16_masked_weight",
                 "pack_w4a8_moe_hipc_weight", "pack_w4a8_weight_k_contiguous",
                 "pack_int8_weight_enk_to_w6_low_latency", "view_w4a8_moe_hipc_weight_n32_layout"]:
        assert callable(getattr(deepgemm, name)), name
    for name in ["low_latency_grouped_gemm", "low_latency_grouped_gemm_tensor_wise",
                 "m_grouped_marlin_w8a8_gemm_nt_masked", "m_grouped_marlin_w4a8_gemm_nt_masked",
                 "m_grouped_marlin_w4a8_gemm_nt_masked_hipc", "m_grouped_bf16_gemm_nt_masked",
                 "m_grouped_marlin_w4a8_gemm_nt_contiguous_hipc", "m_grouped_w8a8_gemm_nt_contiguous"]:
        assert callable(getattr(deepgemm.op, name)), name
    for name in ["low_latency_grouped_gemm", "low_latency_grouped_gemm_tensor_wise",
                 "m_grouped_w8a8_gemm_nt_masked_gfx936", "m_grouped_i8_gemm_nt_contiguous",
                 "m_grouped_fp8_gemm_nt_contiguous",
                 "m_grouped_fp8_gemm_nt_contiguous_marlin_tensor_wise"]:
        assert hasattr(torch.ops.deep_gemm, name), name


def test_overlap_and_signal_are_rejected():
    a, b, d, mm = _masked_int8_args()
    with pytest.raises(RuntimeError, match="overlap"):
        deepgemm.m_grouped_w8a8_gemm_nt_masked(a, b, d, mm, 8, enable_overlap=True)
    with pytest.raises(RuntimeError, match="signal"):
        deepgemm.m_grouped_w8a8_gemm_nt_masked(a, b, d, mm, 8, signal=torch.zeros(1))


def test_masked_m_must_be_int32():
    a, b, d, mm = _masked_int8_args()
    with pytest.raises(ValueError, match="int32"):
        deepgemm.m_grouped_i8_gemm_nt_masked(a, b, d, mm.long(), 8)
    with pytest.raises(ValueError, match="int32"):
        deepgemm.m_grouped_w8a8_gemm_nt_masked_ll(a, b, d, mm.long(), 8)


def test_block_wise_is_rejected():
    a, b, d, mm = _masked_int8_args()
    a8 = (a[0].view(torch.uint8).view(FP8), a[1])
    with pytest.raises(RuntimeError, match="block-wise"):
        deepgemm.m_grouped_fp8_gemm_nt_masked(a8, b, d, mm, 8, block_wise=True)


def test_expert_count_mismatch_and_scale_shapes():
    a, b, d, mm = _masked_int8_args()
    with pytest.raises(ValueError, match="masked_m length"):
        deepgemm.m_grouped_w8a8_gemm_nt_masked_ll(a, b, d, mm[:1], 8)
    with pytest.raises(ValueError, match="a_scale"):
        deepgemm.m_grouped_w8a8_gemm_nt_masked_ll((a[0], torch.ones(2, 8, 2)), b, d, mm, 8)
    with pytest.raises(ValueError, match=r"\[E\] or \[E, 1\]"):
        deepgemm.m_grouped_fp8_gemm_nt_masked_tensor_wise(a, b, d, mm, 8)      # b_scale is [E,N]
    with pytest.raises(ValueError, match=r"\[E\] or \[E, 1\]"):
        deepgemm.m_grouped_fp8_gemm_nt_contiguous_tensor_wise(
            (a[0][0], torch.ones(8)), b, d[0], torch.zeros(8, dtype=torch.int32))


def test_unpacked_weights_are_rejected():
    a, b, d, mm = _masked_int8_args()
    raw = torch.zeros(2, 32, 128, dtype=torch.int8)
    with pytest.raises(ValueError, match="packed weight"):
        deepgemm.m_grouped_i8_gemm_nt_contiguous((a[0][0], torch.ones(8)), (raw, b[1]), d[0],
                                                 torch.zeros(8, dtype=torch.int32))
    with pytest.raises(ValueError, match="pre-packed"):
        deepgemm.m_grouped_bf16_gemm_nt_masked(torch.zeros(2, 8, 128, dtype=torch.bfloat16),
                                               torch.zeros(2, 32, 128, dtype=torch.bfloat16), d, mm, 8)
    with pytest.raises(KeyError):
        deepgemm.m_grouped_w4a8_gemm_nt_masked(a, b, d, mm, 8, config={})      # like the reference


def test_contiguous_w4a8_shape_errors():
    a2 = (torch.zeros(8, 256, dtype=torch.int8), torch.ones(8))
    bw = (torch.zeros(2, 32, 128, dtype=torch.int8), torch.ones(2, 32))
    out = torch.zeros(8, 32, dtype=torch.bfloat16)
    mi = torch.zeros(8, dtype=torch.int32)
    with pytest.raises(ValueError, match=r"\[M,K\]"):
        deepgemm.m_grouped_w4a8_gemm_nt_contiguous_hipc((a2[0][None], a2[1]), bw, out, mi)
    with pytest.raises(ValueError, match="m_indices length"):
        deepgemm.m_grouped_w4a8_gemm_nt_contiguous_hipc(a2, bw, out, mi[:4])
    with pytest.raises(ValueError, match="a_scale"):
        deepgemm.m_grouped_w4a8_gemm_nt_contiguous_hipc((a2[0], torch.ones(8, 2)), bw, out, mi)


def test_cpu_tensors_never_compute():
    # There is no CPU implementation: the dispatcher has no kernel for CPU tensors.
    a, b, d, mm = _masked_int8_args()
    before = d.clone()
    with pytest.raises((NotImplementedError, RuntimeError)):
        deepgemm.m_grouped_w8a8_gemm_nt_masked(a, b, d, mm, 8)
    with pytest.raises((NotImplementedError, RuntimeError)):
        deepgemm.m_grouped_fp8_gemm_nt_masked((a[0].view(torch.uint8).view(FP8), a[1]), b, d, mm, 8)
    assert torch.equal(before, d)


def test_op_size_printer_reports_operands_without_touching_the_call(capsys, monkeypatch):
    """DEEPGEMM_PRINT_OP_SIZE: one '[DeepGEMM][size] <op> ...' line per call, filter honoured,
    the wrapped function still gets its arguments (reference deepgemm/print_size.py:97-118)."""
    import types
    from deepgemm import print_size

    seen = []
    mod = types.ModuleType("fake_op")

    def m_grouped_fake_masked(input, b_qweight, output, a_scale, b_scale, masked_m, expected_m, mode):
        seen.append((tuple(input.shape), mode))
        return output
    m_grouped_fake_masked.__module__ = "fake_op"
    mod.m_grouped_fake_masked = m_grouped_fake_masked
    print_size.install_op_size_printer(mod, force=True)
    print_size.install_op_size_printer(mod, force=True)        # wrapping twice is a no-op

    a = torch.zeros(4, 64, 256, dtype=torch.int8)
    w = torch.zeros(4, 2, 512, 128, dtype=torch.int8)
    d = torch.zeros(4, 64, 512, dtype=torch.bfloat16)
    mm = torch.tensor([1, 2, 3, 4], dtype=torch.int32)
    monkeypatch.setenv("DEEPGEMM_PRINT_OP_SIZE_STATS", "1")
    assert mod.m_grouped_fake_masked(a, w, d, None, None, mm, 64, mode=1002) is d
    line = capsys.readouterr().out.strip()
    assert line.startswith("[DeepGEMM][size] m_grouped_fake_masked input=(4,64,256):int8:cpu")
    for field in ("output=(4,64,512):bfloat16:cpu", "a_scale=None", "E=4", "M=64", "N=512", "K=256",
                  "mode=1002", "masked_m_sum=10", "masked_m_max=4"):
        assert field in line, field
    monkeypatch.setenv("DEEPGEMM_PRINT_OP_SIZE_FILTER", "contiguous")
    mod.m_grouped_fake_masked(a, w, d, None, None, mm, 64, mode=1)
    assert capsys.readouterr().out == ""
    assert seen == [((4, 64, 256), 1002), ((4, 64, 256), 1)]


def test_w4a8_weight_that_was_never_packed_is_rejected():
    """The packed int4 tensor keeps the framework shape [E, N, K/2]: a tensor that did not go
    through the packer must not be read as if it had."""
    from deepgemm import _core, _cabi
    from deepgemm import group_gemm_weight_pack as P
    fw = torch.zeros(2, 16, 128, dtype=torch.int8)
    with pytest.raises(ValueError, match="has not been through"):
        _core.packed_weight_dims(fw, _cabi.KIND_W4A8)
    packed = P.pack_w4a8_moe_hipc_weight(fw)
    assert _core.packed_weight_dims(packed, _cabi.KIND_W4A8) == (2, 16, 256)
    other = P.register_packed_w4a8_weight(torch.zeros(2, 16, 128, dtype=torch.int8))
    assert _core.packed_weight_dims(other, _cabi.KIND_W4A8) == (2, 16, 256)
