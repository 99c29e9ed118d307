"""The C-ABI library loads on a CPU-only box and exports exactly what include/*.h declares.
No compute call is made here."""
import ctypes
import os
import re

import pytest

import deepgemm
from deepgemm import _cabi

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(REPO, "include", "deepgemm_b200.h")


def _declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\bDG_API\s+[\w\s\*]+?\b(dg_\w+)\s*\(", text)))


def test_header_functions_are_exported():
    names = _declared_functions()
    assert set(names) == set(_cabi.EXPORTED_SYMBOLS), names
    lib = ctypes.CDLL(_cabi.LIB_PATH)
    for n in names:
        assert getattr(lib, n) is not None


def test_struct_layouts_match_header_field_order():
    text = open(HEADER).read()
    for struct, cls in (("dg_masked_args", _cabi.MaskedArgs), ("dg_contig_args", _cabi.ContigArgs),
                        ("dg_ep_plan_args", _cabi.EpPlanArgs), ("dg_ep_push_args", _cabi.EpPushArgs),
                        ("dg_ep_barrier_args", _cabi.EpBarrierArgs)):
        body = re.search(r"typedef struct %s \{(.*?)\} %s;" % (struct, struct), text, flags=re.S).group(1)
        body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
        fields = re.findall(r"(\w+)\s*;", body)
        assert fields == [f[0] for f in cls._fields_], (struct, fields)
    assert ctypes.sizeof(_cabi.MaskedArgs) == 112 and ctypes.sizeof(_cabi.ContigArgs) == 120


def test_query_and_strerror_without_a_device():
    assert _cabi.query(_cabi.QUERY_ABI_VERSION) == 2
    assert _cabi.lib.dg_strerror(0) == b"ok"
    assert b"16-byte" in _cabi.lib.dg_strerror(-4)
    assert _cabi.lib.dg_strerror(12345) == b"unknown status code"
    assert _cabi.query(_cabi.QUERY_LAUNCH_COUNT) >= 0


def test_calls_validate_before_touching_the_device():
    # argument errors are reported by code, never by a crash, also without any GPU
    assert _cabi.lib.dg_masked_gemm(None, None) == -1
    a = _cabi.MaskedArgs(kind=9)
    assert _cabi.lib.dg_masked_gemm(ctypes.byref(a), None) == -2
    a = _cabi.MaskedArgs(kind=_cabi.KIND_I8, scale_mode=_cabi.SCALE_NONE, num_groups=1, max_m=4, n=64, k=128)
    assert _cabi.lib.dg_masked_gemm(ctypes.byref(a), None) == -5      # int8 needs scales
    a = _cabi.MaskedArgs(kind=_cabi.KIND_I8, scale_mode=0, num_groups=1, max_m=4, n=60, k=128)
    assert _cabi.lib.dg_masked_gemm(ctypes.byref(a), None) == -3      # N % 16
    a = _cabi.MaskedArgs(kind=_cabi.KIND_I8, scale_mode=0, num_groups=1, max_m=4, n=64, k=100)
    assert _cabi.lib.dg_masked_gemm(ctypes.byref(a), None) == -3      # K % 64
    a = _cabi.MaskedArgs(kind=_cabi.KIND_I8, scale_mode=0, num_groups=5000, max_m=4, n=64, k=128)
    assert _cabi.lib.dg_masked_gemm(ctypes.byref(a), None) == -8
    a = _cabi.MaskedArgs(kind=_cabi.KIND_I8, scale_mode=0, num_groups=1, max_m=4, n=64, k=128)
    assert _cabi.lib.dg_masked_gemm(ctypes.byref(a), None) == -1      # null pointers
    assert _cabi.lib.dg_sorted_gemm(None, None) == -1
    g = _cabi.SortedGemmArgs(kind=_cabi.KIND_BF16)
    assert _cabi.lib.dg_sorted_gemm(ctypes.byref(g), None) == -2      # INT8 / FP8 only
    g = _cabi.SortedGemmArgs(kind=_cabi.KIND_I8, num_groups=2, num_sorted=64, num_blocks=1, block_m=32,
                             size_m=8, real_topk=2, n=64, k=128)
    assert _cabi.lib.dg_sorted_gemm(ctypes.byref(g), None) == -9      # blocks do not cover the list
    g = _cabi.SortedGemmArgs(kind=_cabi.KIND_I8, num_groups=2, num_sorted=64, num_blocks=2, block_m=32,
                             size_m=8, real_topk=2, n=64, k=128)
    assert _cabi.lib.dg_sorted_gemm(ctypes.byref(g), None) == -1      # null pointers
    c = _cabi.ContigArgs(kind=_cabi.KIND_E4M3, scale_mode=0, num_groups=1, m_total=1 << 22, n=64, k=128)
    assert _cabi.lib.dg_contig_gemm(ctypes.byref(c), None) == -8
    c = _cabi.ContigArgs(kind=_cabi.KIND_E4M3, scale_mode=0, num_groups=1, m_total=128, n=64, k=128,
                         scatter_tag=16, scatter_world=2)
    assert _cabi.lib.dg_contig_gemm(ctypes.byref(c), None) == -1      # scatter buffers missing
    assert _cabi.lib.dg_ep_plan(None, None) == -1
    e = _cabi.EpPlanArgs(world=4, rank=4, num_experts=16, align=256, m_cap=1024)
    assert _cabi.lib.dg_ep_plan(ctypes.byref(e), None) == -9          # rank outside the world
    e = _cabi.EpPlanArgs(world=4, rank=0, num_experts=18, align=256, m_cap=1024)
    assert _cabi.lib.dg_ep_plan(ctypes.byref(e), None) == -3          # experts not a multiple of ranks
    u = _cabi.EpPushArgs(world=2, rank=0, num_experts=16, num_tokens=8, top_k=2, row_bytes=100, m_cap=256)
    assert _cabi.lib.dg_ep_push(ctypes.byref(u), None) == -3          # rows must be whole 16-byte chunks
    u = _cabi.EpPushArgs(world=2, rank=0, num_experts=16, num_tokens=8, top_k=2, row_bytes=128, m_cap=256)
    assert _cabi.lib.dg_ep_push(ctypes.byref(u), None) == -1          # null pointers
    assert _cabi.lib.dg_pack_weight(0, None, None, 1, 16, 128, 0, None) == -1
    assert _cabi.lib.dg_pack_weight(7, 16, 32, 1, 16, 128, 0, None) == -2
    assert _cabi.lib.dg_pack_weight(0, 16, 32, 1, 16, 100, 0, None) == -3
    assert _cabi.lib.dg_pack_weight(0, 17, 32, 1, 16, 128, 0, None) == -4
    assert _cabi.lib.dg_pack_weight(2, 16, 32, 1, 16, 128, 0, None) == -3   # int4 needs K % 256
    assert _cabi.lib.dg_pack_weight(2, 16, 32, 1, 16, 256, 5, None) == -9


def test_missing_library_is_a_loud_import_error(tmp_path, monkeypatch):
    import importlib
    monkeypatch.setenv("DEEP_GEMM_LIB_PATH", str(tmp_path / "nope.so"))
    spec = importlib.util.spec_from_file_location("cabi_probe", _cabi.__file__)
    mod = importlib.util.module_from_spec(spec)
    with pytest.raises(ImportError, match="no fallback"):
        spec.loader.exec_module(mod)


def test_header_is_valid_c99_and_cxx(tmp_path):
    """The boundary is a C ABI: the header must compile as plain C (what a cgo / JNI / FFI binding
    generator reads) and as C++, with no CUDA or torch headers."""
    import shutil
    import subprocess
    inc = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include")
    body = (
        '#include "deepgemm_b200.h"\n'
        "int use(void) {\n"
        "  dg_masked_args m; dg_contig_args c; dg_compact_args p; dg_dense_args d; dg_quant_group_args q;\n"
        "  dg_group_sorted_args s; dg_act_quant_args a; dg_combine_args b;\n"
        "  dg_ep_plan_args e1; dg_ep_push_args e2; dg_ep_barrier_args e3; (void)e1; (void)e2; (void)e3;\n"
        "  (void)m; (void)c; (void)p; (void)d; (void)q; (void)s; (void)a; (void)b;\n"
        "  return (int)sizeof(dg_masked_args) + DG_STATUS_WORDS + DG_ABI_VERSION;\n"
        "}\n")
    for compiler, name, std in (("gcc", "t.c", "-std=c99"), ("g++", "t.cpp", "-std=c++11")):
        if shutil.which(compiler) is None:
            pytest.skip(f"{compiler} not available")
        src = tmp_path / name
        src.write_text(body)
        r = subprocess.run([compiler, std, "-Wall", "-Werror", "-pedantic", "-fsyntax-only", "-I", inc, str(src)],
                           capture_output=True, text=True)
        assert r.returncode == 0, r.stderr
