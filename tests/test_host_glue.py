"""The native host path (deepgemm/_glue.so, csrc/dg_torch_glue.cpp): it only ever accepts a call
whose arguments pass every check; anything else comes back to the Python marshalling, which owns
the error messages."""
import pytest
import torch

import deepgemm
from deepgemm import _cabi, _core

glue = _core._glue


def test_glue_is_built_and_matches_the_library():
    assert glue is not None, "deepgemm/_glue.so missing or built against another header (python deepgemm-das_b200/build.py)"
    assert glue.abi_version() == _cabi.query(_cabi.QUERY_ABI_VERSION)


def test_glue_declines_cpu_tensors_and_python_raises_the_message():
    if glue is None:
        pytest.skip("glue not built")
    a = torch.zeros(2, 128, 128, dtype=torch.int8)
    b = torch.zeros(2, 1, 64, 128, dtype=torch.int8)
    d = torch.zeros(2, 128, 64, dtype=torch.bfloat16)
    s = torch.ones(2, 128)
    sb = torch.ones(2, 64)
    m = torch.zeros(2, dtype=torch.int32)
    before = glue.stats()
    assert glue.masked(_cabi.KIND_I8, _cabi.SCALE_PER_CHANNEL, a, b, d, s, sb, m, 1, 0, None, None) is False
    assert glue.contiguous(_cabi.KIND_I8, _cabi.SCALE_PER_CHANNEL, a[0], b, d[0], s[0], sb, m, 0, None) is False
    after = glue.stats()
    assert after[0] == before[0] and after[1] == before[1] + 2
    with pytest.raises(RuntimeError, match="CUDA tensors"):
        _core.grouped_gemm_masked(_cabi.KIND_I8, _cabi.SCALE_PER_CHANNEL, a, b, d, s, sb, m, 1)


@pytest.mark.gpu
def test_glue_takes_the_plain_call_and_hands_back_the_unusual_one():
    assert glue is not None
    dev = "cuda"
    g, max_m, n, k = 3, 128, 256, 256
    gen = torch.Generator().manual_seed(5)
    a = torch.randint(-8, 8, (g, max_m, k), generator=gen, dtype=torch.int8).to(dev)
    w = torch.randint(-8, 8, (g, n, k), generator=gen, dtype=torch.int8)
    bp = deepgemm.marlin_i8_masked_weight(w.clone()).to(dev)
    sa = torch.rand(g, max_m, generator=gen).to(dev)
    sb = torch.rand(g, n, generator=gen).to(dev)
    mm = torch.tensor([128, 0, 77], dtype=torch.int32, device=dev)
    d1 = torch.zeros(g, max_m, n, dtype=torch.bfloat16, device=dev)
    d2 = torch.zeros_like(d1)
    _core.device_status_words(torch.device(dev, 0))          # registered with the glue
    before = glue.stats()
    _core.grouped_gemm_masked(_cabi.KIND_I8, _cabi.SCALE_PER_CHANNEL, a, bp, d1, sa, sb, mm, 64)
    mid = glue.stats()
    assert mid[0] == before[0] + 1, "the plain call did not take the native path"
    # a scale with a trailing 1 is still the native path; a strided scale is not, and raises in Python
    _core.grouped_gemm_masked(_cabi.KIND_I8, _cabi.SCALE_PER_CHANNEL, a, bp, d2, sa.unsqueeze(-1), sb, mm, 64)
    assert glue.stats()[0] == mid[0] + 1
    torch.cuda.synchronize()
    assert torch.equal(d1.view(torch.int16), d2.view(torch.int16))
    ref = (a.float() @ w.to(dev).float().transpose(1, 2)) * sa[..., None] * sb[:, None, :]
    for i, rows in enumerate(mm.tolist()):
        assert torch.allclose(d1[i, :rows].float(), ref[i, :rows], rtol=1e-2, atol=1e-2)
        assert bool((d1[i, rows:] == 0).all())
    wide = torch.rand(g, 2 * max_m, generator=gen).to(dev)[:, ::2]
    declined = glue.stats()[1]
    with pytest.raises(RuntimeError, match="contiguous"):
        _core.grouped_gemm_masked(_cabi.KIND_I8, _cabi.SCALE_PER_CHANNEL, a, bp, d2, wide, sb, mm, 64)
    assert glue.stats()[1] == declined + 1
    # the same call with the glue switched off gives the same bytes
    saved, _core._glue = _core._glue, None
    try:
        d3 = torch.zeros_like(d1)
        _core.grouped_gemm_masked(_cabi.KIND_I8, _cabi.SCALE_PER_CHANNEL, a, bp, d3, sa, sb, mm, 64)
    finally:
        _core._glue = saved
    torch.cuda.synchronize()
    assert torch.equal(d1.view(torch.int16), d3.view(torch.int16))
    deepgemm.check_device_status()
