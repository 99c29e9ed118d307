"""dg_quant_group_rows_noalloc: the quantise + group + pad producer for callers that are not
allowed to allocate device memory (an engine whose memory pool is frozen, a plugin that only
gets fixed buffers).  Those callers cannot pass a scratch buffer, so the library keeps one
inside itself; inputs and outputs remain the caller's.

The test drives both entry points through the C ABI with the same inputs and demands
identical bytes, twice in a row with different problems, because the second call runs on
scratch words the first one left behind.  This file sorts last so that a failure here cannot
hide the result of any other test."""
import ctypes as C

import pytest
import torch

from deepgemm import _cabi

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _run(entry, rows, expert, groups, align, m_cap, with_scratch):
    r, h = rows.shape
    out = dict(a=torch.zeros((m_cap, h), dtype=torch.uint8, device=DEV),
               a_scale=torch.zeros((m_cap,), dtype=torch.float32, device=DEV),
               m_indices=torch.zeros((m_cap,), dtype=torch.int32, device=DEV),
               dest=torch.zeros((r,), dtype=torch.int32, device=DEV),
               m_total=torch.zeros((1,), dtype=torch.int32, device=DEV))
    scratch = None
    if with_scratch:
        scratch = torch.empty((int(_cabi.lib.dg_quant_group_scratch_bytes(r, groups)),),
                              dtype=torch.uint8, device=DEV)
    args = _cabi.QuantGroupArgs(
        kind=_cabi.KIND_E4M3, num_rows=r, hidden=h, num_groups=groups, align=align, m_cap=m_cap,
        rows=rows.data_ptr(), expert=expert.data_ptr(), a_out=out["a"].data_ptr(),
        a_scale_out=out["a_scale"].data_ptr(), m_indices_out=out["m_indices"].data_ptr(),
        dest_out=out["dest"].data_ptr(), m_total_out=out["m_total"].data_ptr(),
        scratch=None if scratch is None else scratch.data_ptr(),
        scratch_bytes=0 if scratch is None else scratch.numel())
    stream = torch.cuda.current_stream().cuda_stream
    rc = entry(C.byref(args), C.c_void_p(stream))
    assert rc == 0, _cabi.lib.dg_strerror(rc)
    torch.cuda.synchronize()
    return {k: v.cpu() for k, v in out.items()}


def test_noalloc_entry_matches_regular_entry_on_two_calls_in_a_row():
    gen = torch.Generator().manual_seed(77)
    problems = [(3000, 1024, 48, 256), (517, 256, 5, 128)]     # the second reuses dirtied scratch
    for r, h, groups, align in problems:
        rows = (torch.randn(r, h, generator=gen) * 2).bfloat16().to(DEV)
        expert = torch.randint(-1, groups, (r,), generator=gen).to(torch.int32).to(DEV)
        m_cap = (r + groups * (align - 1) + align - 1) // align * align
        want = _run(_cabi.lib.dg_quant_group_rows, rows, expert, groups, align, m_cap, True)
        got = _run(_cabi.lib.dg_quant_group_rows_noalloc, rows, expert, groups, align, m_cap, False)
        assert int(want["m_total"]) > 0
        for key in want:                                        # byte and integer work: exact
            assert torch.equal(got[key], want[key]), f"{key} differs for problem {(r, h, groups, align)}"


def test_noalloc_entry_rejects_problems_beyond_its_scratch():
    # 65536 rows x 256 groups needs 2048 * 256 + 256 scratch words: more than the built-in array
    args = _cabi.QuantGroupArgs(kind=_cabi.KIND_E4M3, num_rows=65536, hidden=64, num_groups=256,
                                align=256, m_cap=1)
    assert 2048 * 256 + 256 > _cabi.NOALLOC_MAX_SCRATCH_INTS
    assert _cabi.lib.dg_quant_group_rows_noalloc(C.byref(args), None) == -8
    assert b"exceeds" in _cabi.lib.dg_strerror(-8)
