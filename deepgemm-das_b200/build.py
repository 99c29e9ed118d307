"""Builds libdeepgemm_b200.so (sm_100a only) with nvcc, in-tree, and the host glue beside it.

Usage:  python deepgemm-das_b200/build.py [--force] [--verbose]

The library has no torch dependency: it links the static CUDA runtime only and obtains
cuTensorMapEncodeTiled through cudaGetDriverEntryPoint, so libcuda is not linked either.
deepgemm/_glue.so is a Python extension (g++, torch headers) that checks torch tensors and calls
the library natively; the package works without it through the ctypes marshalling, only slower
per call, so a failure to build it is reported and not fatal.
"""
from __future__ import annotations

import argparse
import hashlib
import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
REPO_DIR = os.path.dirname(PKG_DIR)
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_DIR = os.path.join(PKG_DIR, "deepgemm", "lib")
LIB_PATH = os.path.join(LIB_DIR, "libdeepgemm_b200.so")
STAMP_PATH = LIB_PATH + ".stamp"
GLUE_SRC = os.path.join(CSRC, "dg_torch_glue.cpp")
GLUE_PATH = os.path.join(PKG_DIR, "deepgemm", "_glue.so")
GLUE_STAMP = GLUE_PATH + ".stamp"

SOURCES = ["dg_api.cu"]
HEADERS = ["dg_ptx.cuh", "dg_grouped_gemm.cuh", "dg_grouped_gemm_pair.cuh", "dg_grouped_gemm_w4.cuh", "dg_grouped_gemm_w4s.cuh",
           "dg_pack.cuh", "dg_quant_group.cuh", "dg_moe_chain.cuh", "dg_ep.cuh"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found (set NVCC or put it on PATH)")


def _digest() -> str:
    h = hashlib.sha256()
    files = [os.path.join(CSRC, f) for f in SOURCES + HEADERS]
    files.append(os.path.join(REPO_DIR, "include", "deepgemm_b200.h"))
    files.append(os.path.abspath(__file__))
    for f in files:
        with open(f, "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()


def nvcc_command(verbose: bool = False) -> list[str]:
    cmd = [
        _nvcc(),
        "-gencode", "arch=compute_100a,code=sm_100a",
        "-O3", "-std=c++17", "-lineinfo",
        "-shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
        "-cudart", "static",
        "-I", os.path.join(REPO_DIR, "include"), "-I", CSRC,
    ]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += [os.path.join(CSRC, s) for s in SOURCES]
    cmd += ["-o", LIB_PATH]
    return cmd


def glue_command() -> list[str]:
    """g++ line for deepgemm/_glue.so: torch's headers and libraries, the C ABI header, and the
    library itself found at run time beside the module ($ORIGIN/lib)."""
    import sysconfig
    import torch
    tdir = os.path.dirname(torch.__file__)
    cxx = os.environ.get("CXX") or shutil.which("g++") or "g++"
    abi = int(getattr(torch._C, "_GLIBCXX_USE_CXX11_ABI", True))
    cuda_inc = os.path.join(os.path.dirname(os.path.dirname(_nvcc())), "include")
    return [cxx, "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden",
            f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-DTORCH_EXTENSION_NAME=_glue", "-DTORCH_API_INCLUDE_EXTENSION_H",
            "-I", os.path.join(REPO_DIR, "include"), "-I", os.path.join(tdir, "include"),
            "-I", os.path.join(tdir, "include", "torch", "csrc", "api", "include"),
            "-I", sysconfig.get_paths()["include"], "-I", cuda_inc,
            GLUE_SRC, "-o", GLUE_PATH,
            "-L", LIB_DIR, "-ldeepgemm_b200", "-L", os.path.join(tdir, "lib"),
            "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch", "-ltorch_python",
            "-Wl,-rpath,$ORIGIN/lib", "-Wl,-rpath," + os.path.join(tdir, "lib")]


def build_glue(force: bool = False, verbose: bool = False):
    """Compiles deepgemm/_glue.so if its inputs changed.  Returns its path, or None (with the
    compiler's output on stderr) when it cannot be built here."""
    h = hashlib.sha256()
    for f in (GLUE_SRC, os.path.join(REPO_DIR, "include", "deepgemm_b200.h"), os.path.abspath(__file__)):
        with open(f, "rb") as fh:
            h.update(fh.read())
    try:
        import torch
        h.update(torch.__version__.encode())
    except ImportError:
        sys.stderr.write("deepgemm build: torch is not importable, the host glue is not built\n")
        return None
    digest = h.hexdigest()
    if not force and os.path.exists(GLUE_PATH) and os.path.exists(GLUE_STAMP):
        with open(GLUE_STAMP) as fh:
            if fh.read().strip() == digest:
                return GLUE_PATH
    cmd = glue_command()
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or proc.returncode != 0:
        sys.stderr.write(proc.stdout)
        sys.stderr.write(proc.stderr)
    if proc.returncode != 0:
        sys.stderr.write("deepgemm build: the host glue did not compile (calls use the ctypes path):\n"
                         + " ".join(cmd) + "\n")
        return None
    with open(GLUE_STAMP, "w") as fh:
        fh.write(digest)
    return GLUE_PATH


def build(force: bool = False, verbose: bool = False) -> str:
    """Compiles the library (and the host glue) if their sources changed; returns the path of
    libdeepgemm_b200.so."""
    os.makedirs(LIB_DIR, exist_ok=True)
    digest = _digest()
    fresh = False
    if not force and os.path.exists(LIB_PATH) and os.path.exists(STAMP_PATH):
        with open(STAMP_PATH) as fh:
            fresh = fh.read().strip() == digest
    if not fresh:
        cmd = nvcc_command(verbose)
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or proc.returncode != 0:
            sys.stderr.write(proc.stdout)
            sys.stderr.write(proc.stderr)
        if proc.returncode != 0:
            raise RuntimeError("nvcc failed building libdeepgemm_b200.so:\n" + " ".join(cmd))
        with open(STAMP_PATH, "w") as fh:
            fh.write(digest)
    build_glue(force=force, verbose=verbose)
    return LIB_PATH


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true", help="pass -Xptxas -v (registers, spills)")
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose))
