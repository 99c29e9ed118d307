"""Shared helpers for the tests: golden-fixture loading, seeded input generators for the
benchmark configurations, and parity assertions (bit-exact accumulators, <= 1 bf16 ulp,
calc_diff)."""
from __future__ import annotations

import os

import numpy as np
import torch

import dg_oracle as O

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
FP8 = torch.float8_e4m3fn
_FP8_CASES = {"masked_fp8", "masked_fp8_tensor_wise", "contig_fp8", "contig_fp8_tensor_wise",
              "dense_fp8"}


def load_golden(name: str) -> dict:
    raw = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    out = {}
    for k in raw.files:
        arr = raw[k]
        if arr.dtype.kind in "US":  # names
            out[k] = [str(v) for v in arr.tolist()]
        elif arr.dtype == np.uint16:  # bf16 bit patterns
            out[k] = torch.from_numpy(arr.view(np.int16).copy()).view(torch.bfloat16)
        elif arr.dtype == np.uint8 and name in _FP8_CASES and k in ("a", "b"):
            out[k] = torch.from_numpy(arr.copy()).view(FP8)
        else:
            out[k] = torch.from_numpy(arr.copy())
    return out


# ----------------------------------------------------------------------------- generators
def gen_masked_int8(G, max_m, N, K, masked_m, seed=0):
    """Per-token int8 activations and per-channel int8 weights quantised from N(0,1)."""
    g = torch.Generator().manual_seed(seed)
    a, a_s = O.per_token_quant_int8(torch.randn(G, max_m, K, generator=g))
    b, b_s = O.per_token_quant_int8(torch.randn(G, N, K, generator=g))
    return dict(a=a, a_scale=a_s.reshape(G, max_m), b=b, b_scale=b_s.reshape(G, N),
                masked_m=torch.as_tensor(masked_m, dtype=torch.int32))


def gen_masked_fp8(G, max_m, N, K, masked_m, seed=0, tensor_wise=False, integer=False):
    g = torch.Generator().manual_seed(seed)
    if integer:  # exactly representable values: fp32 sums are order independent
        a = torch.randint(-4, 5, (G, max_m, K), generator=g).float().to(FP8)
        b = torch.randint(-4, 5, (G, N, K), generator=g).float().to(FP8)
        a_s = torch.rand(G, max_m, generator=g) + 0.5
        b_s = torch.rand(G, N, generator=g) + 0.5
    else:
        a, a_s = O.per_token_quant_fp8(torch.randn(G, max_m, K, generator=g))
        b, b_s = O.per_token_quant_fp8(torch.randn(G, N, K, generator=g))
        a_s, b_s = a_s.reshape(G, max_m), b_s.reshape(G, N)
    if tensor_wise:
        b_s = torch.rand(G, generator=g) * 0.01 + 0.001
    return dict(a=a, a_scale=a_s, b=b, b_scale=b_s,
                masked_m=torch.as_tensor(masked_m, dtype=torch.int32))


def gen_masked_w4a8(G, max_m, N, K, masked_m, seed=0, nibble_order="high_first"):
    """int8 activations; int4 weights in [-7,7] per-channel quantised from N(0,1), packed two
    per byte in the given nibble order.  b_scale is the true scale; the kernel gets b_scale/16."""
    g = torch.Generator().manual_seed(seed)
    a, a_s = O.per_token_quant_int8(torch.randn(G, max_m, K, generator=g))
    w = torch.randn(G, N, K, generator=g)
    amax = w.abs().amax(dim=-1, keepdim=True).clamp_min(1e-10)
    w4 = torch.round(w * (7.0 / amax)).clamp(-7, 7).to(torch.int8)
    b_s = (amax / 7.0).reshape(G, N)
    nib = (w4.to(torch.int16) & 0xF).view(G, N, K // 2, 2)
    if nibble_order == "high_first":
        packed = ((nib[..., 0] << 4) | nib[..., 1])
    else:
        packed = ((nib[..., 1] << 4) | nib[..., 0])
    packed = torch.where(packed > 127, packed - 256, packed).to(torch.int8)
    return dict(a=a, a_scale=a_s.reshape(G, max_m), w4=w4, b_framework=packed, b_scale=b_s,
                masked_m=torch.as_tensor(masked_m, dtype=torch.int32))


def gen_contig(kind, rows_per_group, N, K, seed=0, align=256, tensor_wise=False):
    g = torch.Generator().manual_seed(seed)
    G = len(rows_per_group)
    m_indices, M = O.build_contiguous_layout(rows_per_group, align)
    quant = O.per_token_quant_int8 if kind == "int8" else O.per_token_quant_fp8
    a, a_s = quant(torch.randn(M, K, generator=g))
    b, b_s = quant(torch.randn(G, N, K, generator=g))
    b_s = b_s.reshape(G, N)
    if tensor_wise:
        b_s = torch.rand(G, generator=g) * 0.01 + 0.001
    return dict(a=a, a_scale=a_s.reshape(M), b=b, b_scale=b_s, m_indices=m_indices)


# ----------------------------------------------------------------------------- assertions
def assert_bf16_within_ulp(got: torch.Tensor, want: torch.Tensor, max_ulp: int, what: str):
    d = O.bf16_ulp_distance(got, want)
    worst = int(d.max()) if d.numel() else 0
    assert worst <= max_ulp, f"{what}: {int((d > max_ulp).sum())} elements differ by more than " \
                             f"{max_ulp} bf16 ulp (worst {worst})"


def assert_calc_diff(got: torch.Tensor, want: torch.Tensor, tol: float, what: str):
    diff = O.calc_diff(got.float(), want.float())
    assert diff < tol, f"{what}: calc_diff {diff:.3e} >= {tol:.1e}"
