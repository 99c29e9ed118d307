"""Parity at the full benchmark sizes.  Inputs are generated on the GPU (too large to
quantise on the host in reasonable time); the oracle is evaluated on a sample of rows per
expert against all N output channels, and size-independent properties are checked on the
whole output: rows that must not be written keep their sentinel, and the result is
invariant to the tile width the library picks."""
import pytest
import torch

import deepgemm
from deepgemm import _cabi, _core
from deepgemm.quant_utils import (contiguous_layout, pack_int4_pairs, per_channel_quant_int4,
                                  per_token_quant_fp8, per_token_quant_int8)

import dg_oracle as O
from helpers import assert_bf16_within_ulp, assert_calc_diff

pytestmark = pytest.mark.gpu
DEV = "cuda"
SENTINEL = 17.0


def _weights(G, N, K, quant, gen, dtype):
    b = torch.empty(G, N, K, dtype=dtype, device=DEV)
    s = torch.empty(G, N, dtype=torch.float32, device=DEV)
    for g in range(G):
        q, sc = quant(torch.randn(N, K, device=DEV, generator=gen))
        b[g], s[g] = q, sc.reshape(N)
    return b, s


def test_config2_masked_fp8_decode_full_size():
    G, K, N, max_m = 32, 7168, 4096, 128
    cpu_gen = torch.Generator().manual_seed(0)
    picks = torch.rand(256, G, generator=cpu_gen).topk(8, dim=1).indices
    mm = torch.bincount(picks.flatten(), minlength=G).clamp(max=max_m).to(torch.int32)
    gen = torch.Generator(device=DEV).manual_seed(0)
    a, a_s = per_token_quant_fp8(torch.randn(G, max_m, K, device=DEV, generator=gen))
    a_s = a_s.reshape(G, max_m).contiguous()
    b, b_s = _weights(G, N, K, per_token_quant_fp8, gen, torch.float8_e4m3fn)
    b_rows = b.cpu()
    bp = deepgemm.marlin_fp8_masked_weight(b)
    outs = []
    for bn in (128, 256):
        d = torch.full((G, max_m, N), SENTINEL, dtype=torch.bfloat16, device=DEV)
        _core.grouped_gemm_masked(_cabi.KIND_E4M3, 0, a, bp, d, a_s, b_s, mm.to(DEV), max_m, block_n=bn)
        outs.append(d.cpu())
    assert_calc_diff(outs[0], outs[1], 1e-6, "tile-width invariance")
    d = outs[0]
    a_c, as_c, bs_c = a.cpu(), a_s.cpu(), b_s.cpu()
    for g in range(0, G, 5):
        m = int(mm[g])
        ref = O.ref_masked_scaled(a_c[g:g + 1, :m], b_rows[g:g + 1], as_c[g:g + 1, :m], bs_c[g:g + 1])[0]
        assert_calc_diff(d[g, :m], ref, 1e-3, f"config 2 group {g}")              # calc_diff < 1e-3
    for g in range(G):
        assert torch.all(d[g, int(mm[g]):].float() == SENTINEL)
    # per-expert weight scale variant on the same operands
    bt = b_s.mean(dim=1).contiguous()
    d = torch.full((G, max_m, N), SENTINEL, dtype=torch.bfloat16, device=DEV)
    deepgemm.m_grouped_fp8_gemm_nt_masked_tensor_wise((a, a_s), (bp, bt), d, mm.to(DEV), max_m)
    d = d.cpu()
    for g in (1, 17):
        m = int(mm[g])
        ref = O.ref_masked_tensor_wise(a_c[g:g + 1, :m], b_rows[g:g + 1], as_c[g:g + 1, :m], bt.cpu()[g:g + 1])[0]
        assert_calc_diff(d[g, :m], ref, 1e-3, f"config 2 tensor-wise group {g}")


def test_config3_contiguous_int8_prefill_full_size():
    G, K, N = 32, 7168, 4096
    cpu_gen = torch.Generator().manual_seed(3)
    rows = torch.bincount(torch.rand(4096, G, generator=cpu_gen).topk(8, dim=1).indices.flatten(), minlength=G)
    m_indices, starts, m_total = contiguous_layout(rows.tolist(), 256, DEV)
    gen = torch.Generator(device=DEV).manual_seed(3)
    a, a_s = per_token_quant_int8(torch.randn(m_total, K, device=DEV, generator=gen))
    a_s = a_s.reshape(-1).contiguous()
    b, b_s = _weights(G, N, K, per_token_quant_int8, gen, torch.int8)
    b_rows = b.cpu()
    bp = deepgemm.marlin_i8_contiguous_weight(b)
    d = torch.full((m_total, N), SENTINEL, dtype=torch.bfloat16, device=DEV)
    acc = torch.zeros((m_total, N), dtype=torch.int32, device=DEV)
    st = torch.zeros(4, dtype=torch.int32, device=DEV)
    _core.grouped_gemm_contiguous(_cabi.KIND_I8, 0, a, bp, d, a_s, b_s, m_indices, debug_acc=acc, status=st)
    torch.cuda.synchronize()
    assert st.tolist() == [0, 0, 0, 0]
    idx = m_indices.cpu()
    pad = (idx < 0).to(DEV)
    assert torch.all(d[pad].float() == SENTINEL), "padding rows were written"
    gsel = torch.Generator().manual_seed(9)
    for g in range(G):
        r = int(rows[g])
        pick = (int(starts[g]) + torch.randperm(r, generator=gsel)[:6]).tolist() + [int(starts[g]) + r - 1]
        pick_t = torch.tensor(pick, device=DEV)
        want_acc = O.exact_int_acc(a[pick_t].cpu(), b_rows[g])
        assert torch.equal(acc[pick_t].cpu(), want_acc), f"config 3 accumulators, group {g}"
        want = O.epilogue_from_acc(want_acc, a_s[pick_t].cpu(), b_s[g].cpu())
        assert_bf16_within_ulp(d[pick_t].cpu(), want, 0, f"config 3 group {g}")
    # public API, default tile width, same bits
    d2 = torch.zeros((m_total, N), dtype=torch.bfloat16, device=DEV)
    deepgemm.m_grouped_i8_gemm_nt_contiguous((a, a_s), (bp, b_s), d2, m_indices)
    assert torch.equal(d2[~pad].view(torch.int16), d[~pad].view(torch.int16))


def test_config4_masked_w4a8_full_size():
    G, N, K, max_m = 32, 7168, 2048, 256
    cpu_gen = torch.Generator().manual_seed(4)
    mm = torch.randint(0, max_m + 1, (G,), generator=cpu_gen).to(torch.int32)
    mm[3] = 0
    gen = torch.Generator(device=DEV).manual_seed(4)
    a, a_s = per_token_quant_int8(torch.randn(G, max_m, K, device=DEV, generator=gen))
    a_s = a_s.reshape(G, max_m).contiguous()
    fw = torch.empty(G, N, K // 2, dtype=torch.int8, device=DEV)
    w4 = torch.empty(G, N, K, dtype=torch.int8)
    b_s = torch.empty(G, N, dtype=torch.float32, device=DEV)
    for g in range(G):
        q, s = per_channel_quant_int4(torch.randn(N, K, device=DEV, generator=gen))
        fw[g], b_s[g], w4[g] = pack_int4_pairs(q, "low_first"), s.reshape(N) / 16.0, q.cpu()
    bp = deepgemm.pack_w4a8_moe_hipc_weight(fw, nibble_order="low_first")
    d = torch.full((G, max_m, N), SENTINEL, dtype=torch.bfloat16, device=DEV)
    acc = torch.zeros((G, max_m, N), dtype=torch.int32, device=DEV)
    _core.grouped_gemm_masked(_cabi.KIND_W4A8, 0, a, bp, d, a_s, b_s, mm.to(DEV), max_m, debug_acc=acc)
    d, acc = d.cpu(), acc.cpu()
    a_c, as_c, bs_c = a.cpu(), a_s.cpu(), b_s.cpu()
    for g in range(G):
        m = int(mm[g])
        assert torch.all(d[g, m:].float() == SENTINEL)
        if m and g % 4 == 0:
            rows_ = sorted({0, m - 1, m // 2, min(m - 1, 127), min(m - 1, 128)})
            w16 = (w4[g].to(torch.int16) * 16).to(torch.int8)
            want_acc = O.exact_int_acc(a_c[g, rows_], w16)
            assert torch.equal(acc[g, rows_], want_acc), f"config 4 accumulators, group {g}"
            want = O.epilogue_from_acc(want_acc, as_c[g, rows_], bs_c[g])
            assert_bf16_within_ulp(d[g, rows_], want, 0, f"config 4 group {g}")
