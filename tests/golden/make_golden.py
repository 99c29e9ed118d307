"""Generates tests/golden/*.npz from the REFERENCE's own helper functions.

Run where a checkout of the reference is available, passing its path (or setting
DEEPGEMM_REFERENCE_DIR):   python tests/golden/make_golden.py <reference_dir>

It imports the pure-torch oracles that the reference's op_test/ scripts compare their GPU
kernels with, feeds them small seeded inputs and stores inputs and outputs.  The reference
package itself cannot be imported without ROCm, so `deepgemm` is replaced by a stub module
while its test scripts are imported (only their CPU helper functions are called), and
torch.cuda's device-property query, which some scripts run at import time, is patched to
return a dummy.  Nothing here is imported by the tests; they only read the .npz files.
"""
from __future__ import annotations

import importlib
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("DEEPGEMM_REFERENCE_DIR", "")
if not os.path.isdir(os.path.join(REF, "op_test")):
    sys.exit("usage: make_golden.py <directory of the HYGON-AI/deepgemm-das checkout>")


class _Stub(types.ModuleType):
    __path__ = []  # lets `import deepgemm.xyz` resolve through the finder below

    def __getattr__(self, name):
        if name.startswith("__"):
            raise AttributeError(name)
        return lambda *a, **k: None


class _StubFinder:
    def find_spec(self, name, path=None, target=None):
        if name == "deepgemm" or name.startswith("deepgemm."):
            from importlib.machinery import ModuleSpec
            return ModuleSpec(name, self)
        return None

    def create_module(self, spec):
        return _Stub(spec.name)

    def exec_module(self, module):
        pass


def _import_reference_helpers():
    sys.meta_path.insert(0, _StubFinder())
    sys.path.insert(0, os.path.join(REF, "op_test"))
    torch.cuda.get_device_properties = lambda *a, **k: types.SimpleNamespace(
        multi_processor_count=1, name="none", gcnArchName="none")
    torch.cuda.current_device = lambda: 0
    mods = {}
    for name in ("quant_utils", "masked_w8a8_int8_common", "contiguous_w8a8_int8_common",
                 "test_deepgemm_masked_w8a8_fp8", "test_deepgemm_masked_w8a8_fp8_tensor_wise",
                 "test_deepgemm_masked_w4a8", "test_deepgemm_contiguous_w8a8_fp8",
                 "test_deepgemm_contiguous_w8a8_fp8_tensor_wise", "test_fp8_gemm"):
        mods[name] = importlib.import_module(name)
    # The reference's int4 framework packer lives in its package; load that one file with
    # its sibling import stubbed.
    pkg = types.ModuleType("refdg")
    pkg.__path__ = [os.path.join(REF, "deepgemm")]
    sys.modules["refdg"] = pkg
    sys.modules["refdg.m_group_gemm"] = _Stub("refdg.m_group_gemm")
    mods["weight_pack"] = importlib.import_module("refdg.group_gemm_weight_pack")
    return mods


def _np(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16)
    if t.dtype == torch.float8_e4m3fn:
        return t.view(torch.uint8).numpy()
    return t.numpy()


def _save(name: str, **arrays):
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **{k: _np(v) if torch.is_tensor(v) else np.asarray(v)
                                 for k, v in arrays.items()})
    print(f"{name}.npz  {os.path.getsize(path) / 1024:.1f} KB")


def main():
    m = _import_reference_helpers()
    g = torch.Generator().manual_seed(20251125)
    E, M, N, K = 2, 32, 128, 256

    # 1. per-token int8 quantiser
    x = (torch.randn(E, M, K, generator=g) * 5).to(torch.bfloat16)
    q, s = m["quant_utils"].per_token_quant_int8(x)
    _save("quant_int8", x=x, q=q, scale=s)

    # 2. masked INT8, per-token x per-channel
    w = m["masked_w8a8_int8_common"].to_int8(torch.randn(E, N, K, generator=g) * 40)
    w_scale = torch.randn(E, N, 1, generator=g)
    ref = m["masked_w8a8_int8_common"].torch_gemm(q, w, s, w_scale, torch.bfloat16)
    _save("masked_int8", a=q, a_scale=s, b=w, b_scale=w_scale, out=ref)

    # 3. masked FP8 per-channel (small integers are exact in e4m3, as the reference tests use)
    a8 = torch.randint(-16, 17, (E, M, K), generator=g).float().to(torch.float8_e4m3fn)
    w8 = torch.randint(-16, 17, (E, N, K), generator=g).float().to(torch.float8_e4m3fn)
    a_s = torch.randn(E, M, 1, generator=g)
    w_s = torch.randn(E, N, 1, generator=g)
    ref = m["test_deepgemm_masked_w8a8_fp8"].native_fp8_perChannel_batch_matmul_cpu(
        a8, w8, a_s, w_s, torch.bfloat16)
    _save("masked_fp8", a=a8, a_scale=a_s, b=w8, b_scale=w_s, out=ref)

    # 4. masked FP8, one weight scale per expert
    w_t = torch.randn(E, generator=g)
    ref = m["test_deepgemm_masked_w8a8_fp8_tensor_wise"].native_fp8_perChannel_batch_matmul(
        a8, w8, a_s, w_t, torch.bfloat16)
    _save("masked_fp8_tensor_wise", a=a8, a_scale=a_s, b=w8, b_scale=w_t, out=ref)

    # 5. masked W4A8: int4 unpack (nibble in the high bits = 16 x value) + reference matmul
    u4 = torch.randint(0, 16, (E, N, K), generator=g).to(torch.int8)
    framework = m["weight_pack"].pack_w4a8_weight_k_contiguous(u4)
    unpacked = m["test_deepgemm_masked_w4a8"].unpack_int8_to_int4(framework)
    qa4 = torch.randint(-128, 128, (E, M, K), generator=g).to(torch.int8)
    ref = m["test_deepgemm_masked_w4a8"].native_w8a8_perChannel_batch_matmul(
        qa4, unpacked, a_s, w_s, torch.bfloat16)
    _save("masked_w4a8", u4=u4, framework=framework, unpacked=unpacked, a=qa4, a_scale=a_s,
          b_scale=w_s, out=ref)

    # 6. contiguous INT8 (groups padded to 256 rows, -1 on padding, one empty group)
    rows = [100, 0, 256]
    idx = []
    for e, r in enumerate(rows):
        pad = (r + 255) // 256 * 256
        idx += [e] * r + [-1] * (pad - r)
    m_indices = torch.tensor(idx, dtype=torch.int32)
    Mt, Kc, Nc = len(idx), 128, 128
    ac = m["contiguous_w8a8_int8_common"].to_int8(torch.randn(Mt, Kc, generator=g) * 40)
    bc = m["contiguous_w8a8_int8_common"].to_int8(torch.randn(len(rows), Nc, Kc, generator=g) * 40)
    sa = torch.randn(Mt, generator=g)
    sb = torch.randn(len(rows), Nc, 1, generator=g)
    ref = m["contiguous_w8a8_int8_common"].torch_gemm(
        ac, bc, torch.zeros(Mt, Nc, dtype=torch.bfloat16), sa, sb, 1.0, 0.0, m_indices)
    _save("contig_int8", a=ac, a_scale=sa, b=bc, b_scale=sb, m_indices=m_indices, out=ref)

    # 7. contiguous FP8 per-channel
    to_fp8 = m["test_deepgemm_contiguous_w8a8_fp8"].to_fp8
    af = to_fp8(torch.randn(Mt, Kc, generator=g) * 6)
    bf = to_fp8(torch.randn(len(rows), Nc, Kc, generator=g) * 6)
    sa = torch.rand(Mt, generator=g) * 1.5 + 0.5
    sb2 = torch.rand(len(rows), Nc, generator=g) * 1.5 + 0.5
    ref = m["test_deepgemm_contiguous_w8a8_fp8"].torch_gemm(
        af, bf, torch.zeros(Mt, Nc, dtype=torch.bfloat16), sa, sb2, 1.0, 0.0, m_indices)
    _save("contig_fp8", a=af, a_scale=sa, b=bf, b_scale=sb2, m_indices=m_indices, out=ref)

    # 8. contiguous FP8, one weight scale per expert (the reference helper loops in Python:
    #    keep it tiny)
    rows_t = [5, 3]
    idx_t = []
    for e, r in enumerate(rows_t):
        idx_t += [e] * r + [-1] * (8 - r)
    mi_t = torch.tensor(idx_t, dtype=torch.int32)
    at = to_fp8(torch.randn(len(idx_t), 128, generator=g) * 6)
    bt = to_fp8(torch.randn(2, 16, 128, generator=g) * 6)
    sat = torch.rand(len(idx_t), generator=g) * 1.5 + 0.5
    sbt = torch.rand(2, 1, generator=g) * 1.5 + 0.5
    ref = m["test_deepgemm_contiguous_w8a8_fp8_tensor_wise"].torch_gemm(
        at, bt, torch.zeros(len(idx_t), 16, dtype=torch.bfloat16), sat, sbt, 1.0, 0.0, mi_t)
    _save("contig_fp8_tensor_wise", a=at, a_scale=sat, b=bt, b_scale=sbt, m_indices=mi_t, out=ref)

    # 9. dense FP8 GEMM with per-row scales on both operands (N not a multiple of 8, as the
    #    reference's own first accuracy case)
    md, nd, kd = 24, 22, 256
    ad = to_fp8(torch.randn(md, kd, generator=g) * 0.5)
    bd = to_fp8(torch.randn(nd, kd, generator=g) * 0.5)
    sad = torch.randn(md, generator=g).abs() * 0.01 + 0.01
    sbd = torch.randn(nd, generator=g).abs() * 0.01 + 0.01
    ref = m["test_fp8_gemm"].torch_fp8_gemm(ad, bd.t(), sad, sbd, out_dtype=torch.bfloat16)
    ref16 = m["test_fp8_gemm"].torch_fp8_gemm(ad, bd.t(), sad, sbd, out_dtype=torch.float16)
    _save("dense_fp8", a=ad, a_scale=sad, b=bd, b_scale=sbd, out=ref, out_f16=ref16)


if __name__ == "__main__":
    main()
