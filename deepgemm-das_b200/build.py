"""Builds libdeepgemm_b200.so (sm_100a only) with nvcc, in-tree.

Usage:  python deepgemm-das_b200/build.py [--force] [--verbose]

The library has no torch dependency: it links the static CUDA runtime only and obtains
cuTensorMapEncodeTiled through cudaGetDriverEntryPoint, so libcuda is not linked either.
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


def build(force: bool = False, verbose: bool = False) -> str:
    """Compiles the library if its sources changed; returns the path of the .so."""
    os.makedirs(LIB_DIR, exist_ok=True)
    digest = _digest()
    if not force and os.path.exists(LIB_PATH) and os.path.exists(STAMP_PATH):
        with open(STAMP_PATH) as fh:
            if fh.read().strip() == digest:
                return LIB_PATH
    cmd = nvcc_command(verbose)
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or proc.returncode != 0:
        sys.stderr.write(proc.stdout)
        sys.stderr.write(proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed building libdeepgemm_b200.so:\n" + " ".join(cmd))
    with open(STAMP_PATH, "w") as fh:
        fh.write(digest)
    return LIB_PATH


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true", help="pass -Xptxas -v (registers, spills)")
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose))
