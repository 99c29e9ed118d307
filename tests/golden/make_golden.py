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
                 "test_deepgemm_contiguous_w8a8_fp8_tensor_wise", "test_fp8_gemm",
                 "test_masked_w8a8_big_tile_real6"):
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

    # The cases below draw from a generator of their own, so that the files above stay byte for
    # byte what they were before these were added.
    g2 = torch.Generator().manual_seed(20251126)

    # 10. masked W4A8, signed-nibble convention of the HIPC path.  The reference computes the
    #     expectation inline (op_test/test_deepgemm_masked_w4a8_hipc.py:63-82): int8 activations in
    #     [-8, 8), unsigned nibbles 0..14 read as two's complement, ref = bmm * a_scale * w_scale,
    #     while the op is given w_scale / 16.  Same statements here; the framework layout comes
    #     from the reference's own packer.
    e4, m4, n4, k4 = 2, 48, 128, 256
    q_a = torch.randint(-8, 8, (e4, m4, k4), generator=g2, dtype=torch.int8)
    a_scale4 = torch.rand((e4, m4, 1), generator=g2) * 0.02 + 0.001
    w_scale4 = torch.rand((e4, n4, 1), generator=g2) * 0.02 + 0.001
    weight_u4 = torch.randint(0, 15, (e4, n4, k4), generator=g2, dtype=torch.int8)
    framework4 = m["weight_pack"].pack_w4a8_weight_k_contiguous(weight_u4)
    w_ref = torch.where(weight_u4 > 7, weight_u4 - 16, weight_u4)
    ref = torch.bmm(q_a.float(), w_ref.float().transpose(1, 2))
    ref = ref * a_scale4 * w_scale4.transpose(1, 2)
    _save("masked_w4a8_hipc", a=q_a, a_scale=a_scale4, u4=weight_u4, framework=framework4, w_scale=w_scale4,
          kernel_w_scale=w_scale4 / 16.0, out=ref.to(torch.bfloat16), out_f16=ref.to(torch.float16))

    # 11. contiguous W4A8 (op_test/test_deepgemm_contiguous_w4a8_hipc.py:36-90): groups aligned to
    #     128 rows, -1 on padding rows, same conventions
    actual_ms, n5, k5 = [70, 128, 5], 128, 256
    aligned = [(v + 127) // 128 * 128 for v in actual_ms]
    size_m = sum(aligned)
    q_a5 = torch.randint(-8, 8, (size_m, k5), generator=g2, dtype=torch.int8)
    a_scale5 = torch.rand((size_m, 1), generator=g2) * 0.02 + 0.001
    w_scale5 = torch.rand((len(actual_ms), n5, 1), generator=g2) * 0.02 + 0.001
    weight_u45 = torch.randint(0, 15, (len(actual_ms), n5, k5), generator=g2, dtype=torch.int8)
    framework5 = m["weight_pack"].pack_w4a8_weight_k_contiguous(weight_u45)
    w_ref5 = torch.where(weight_u45 > 7, weight_u45 - 16, weight_u45)
    m_indices5 = torch.empty((size_m,), dtype=torch.int32)
    start = 0
    for expert, (actual_m, aligned_m) in enumerate(zip(actual_ms, aligned)):
        m_indices5[start:start + actual_m] = expert
        m_indices5[start + actual_m:start + aligned_m] = -1
        start += aligned_m
    ref5 = torch.zeros((size_m, n5))
    for expert in range(len(actual_ms)):
        rows5 = m_indices5 == expert
        acc = q_a5[rows5].float() @ w_ref5[expert].float().t()
        ref5[rows5] = acc * a_scale5[rows5].float() * w_scale5[expert].float().t()
    _save("contig_w4a8_hipc", a=q_a5, a_scale=a_scale5, u4=weight_u45, framework=framework5,
          w_scale=w_scale5, kernel_w_scale=w_scale5 / 16.0, m_indices=m_indices5,
          out=ref5.to(torch.bfloat16), out_f16=ref5.to(torch.float16))

    # 12. masked BF16 (op_test/test_deepgemm_masked_w16a16_bf16.py:55-80): N(0, 0.1) operands,
    #     ref = (a.float() @ w.float().t()).to(bf16) on the active rows, zero tail rows
    eb, mb, nb, kb, active = 2, 64, 256, 128, 40
    ab = (torch.randn(eb, mb, kb, generator=g2) * 0.1).to(torch.bfloat16)
    wb = (torch.randn(eb, nb, kb, generator=g2) * 0.1).to(torch.bfloat16)
    refb = torch.zeros(eb, mb, nb, dtype=torch.bfloat16)
    for expert in range(eb):
        refb[expert, :active] = (ab[expert, :active].float() @ wb[expert].float().t()).to(torch.bfloat16)
    _save("masked_bf16", a=ab, b=wb, masked_m=torch.full((eb,), active, dtype=torch.int32), out=refb)

    # 13. the six routing vectors logged from a serving run that the reference replays
    #     (op_test/test_masked_w8a8_big_tile_real6.py:46-53): rows per expert, 36 experts, one with
    #     16 384 rows; N and K of each case
    real6 = m["test_masked_w8a8_big_tile_real6"]
    names = list(real6.DEFAULT_CASES)
    _save("skew_masked_m", names=np.array(names),
          masked_m=np.array([real6.CASES[n].masked_m for n in names], dtype=np.int32),
          n=np.array([getattr(real6.CASES[n], "n", 0) for n in names], dtype=np.int32),
          k=np.array([getattr(real6.CASES[n], "k", 0) for n in names], dtype=np.int32))


if __name__ == "__main__":
    main()
