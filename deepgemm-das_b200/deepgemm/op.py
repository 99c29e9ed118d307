"""Op layer: ``torch.ops.deep_gemm.*`` custom ops plus the reference's pybind names.

The reference exposes its C++ launchers twice: as the pybind module ``deepgemm.op``
(csrc/common/deepgemm_ops.cpp:127-144, argument names in csrc/include/deepgemm_ops.hpp) and
as dispatcher ops in namespace ``deep_gemm`` (csrc/common/000_deep_gemm_torch_library_root.cu:6,
schemas e.g. csrc/arch/gfx936_gfx938_shared/low_latency_grouped_gemm.cu:56-103).  Both are
kept and reach the same implementation: a function of this module calls it directly, as a
pybind function would (the dispatcher hop costs about 5 us of host time per call, as much as
everything else on the host path); ``torch.ops.deep_gemm.<name>`` goes through the dispatcher
for callers that need an op (graph capture by a compiler).  Each op has a CUDA implementation
only, which marshals to the C ABI of libdeepgemm_b200.so.  The
``mode`` / ``cu_s`` / ``block_m`` / ``block_n`` / ``n_loop_num`` integers selected Hygon tile
variants; here they are accepted and ignored (the library picks its own tile).
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _core
from ._core import (KIND_BF16, KIND_E4M3, KIND_I8, KIND_W4A8, SCALE_NONE, SCALE_PER_CHANNEL,
                    SCALE_TENSOR_WISE)

_NS = "deep_gemm"
_lib = torch.library.Library(_NS, "FRAGMENT")


class _Impls:
    """Implementation of every op by name (attribute access, as on ``torch.ops.deep_gemm``)."""


_impl = _Impls()


def _define(name: str, schema: str, fn) -> None:
    _lib.define(f"{name}{schema}")
    _lib.impl(name, fn, "CUDA")
    setattr(_impl, name, fn)


# --------------------------------------------------------------------------- masked
def _check_overlap(b_overlap, signal) -> None:
    """The reference declares the overlap mode (per row-block completion counters in `signal`,
    m_grouped_fp8_gemm_nt_maksed_low_latency.cu:1022-1029) and then refuses it at run time
    (:1148).  Here it works: with b_overlap the counters are maintained (see
    _core.grouped_gemm_masked); a signal tensor without b_overlap is still an error."""
    if b_overlap and signal is None:
        raise RuntimeError("tensor signal empty")                  # the reference's message (:1137)
    if signal is not None and not b_overlap:
        raise RuntimeError("signal is only valid together with enable_overlap / b_overlap")


def _ll_impl(matrix_a, matrix_b, matrix_a_scale, matrix_b_scale, actual_tokens, matrix_c,
             max_tokens, experts, cu_s, block_wise, b_overlap, signal):
    if block_wise:
        raise RuntimeError("block-wise scales are not supported")
    _check_overlap(b_overlap, signal)
    if int(experts) != int(matrix_a.shape[0]):
        raise RuntimeError(f"experts={experts} does not match matrix_a.shape[0]={matrix_a.shape[0]}")
    kind = _core.kind_of_activation(matrix_a)
    return _core.grouped_gemm_masked(kind, SCALE_PER_CHANNEL, matrix_a, matrix_b, matrix_c,
                                     matrix_a_scale, matrix_b_scale, actual_tokens, max_tokens,
                                     signal=signal if b_overlap else None)


def _ll_tw_impl(matrix_a, matrix_b, matrix_a_scale, matrix_b_scale, actual_tokens, matrix_c,
                max_tokens, experts, cu_s, b_overlap, signal):
    _check_overlap(b_overlap, signal)
    if int(experts) != int(matrix_a.shape[0]):
        raise RuntimeError(f"experts={experts} does not match matrix_a.shape[0]={matrix_a.shape[0]}")
    kind = _core.kind_of_activation(matrix_a)
    return _core.grouped_gemm_masked(kind, SCALE_TENSOR_WISE, matrix_a, matrix_b, matrix_c,
                                     matrix_a_scale, matrix_b_scale, actual_tokens, max_tokens,
                                     signal=signal if b_overlap else None)


_LL_SCHEMA = ("(Tensor matrix_a, Tensor matrix_b, Tensor matrix_a_scale, Tensor matrix_b_scale, "
              "Tensor actual_tokens, Tensor(a!) matrix_c, int max_tokens, int experts, int cu_s, "
              "bool block_wise, bool b_overlap, Tensor? signal) -> Tensor(a!)")
_define("low_latency_grouped_gemm", _LL_SCHEMA, _ll_impl)
_define("m_grouped_w8a8_gemm_nt_masked_gfx936", _LL_SCHEMA, _ll_impl)
_define("low_latency_grouped_gemm_tensor_wise",
        "(Tensor matrix_a, Tensor matrix_b, Tensor matrix_a_scale, Tensor matrix_b_scale, "
        "Tensor actual_tokens, Tensor(a!) matrix_c, int max_tokens, int experts, int cu_s, "
        "bool b_overlap, Tensor? signal) -> Tensor(a!)", _ll_tw_impl)

_MASKED_SCHEMA = ("(Tensor input, Tensor b_qweight, Tensor(a!) output, Tensor a_scale, "
                  "Tensor b_scale, Tensor masked_m, int expected_m_per_group, int mode) -> Tensor(a!)")


def _masked_i8_impl(input, b_qweight, output, a_scale, b_scale, masked_m, expected_m_per_group,
                    mode):
    return _core.grouped_gemm_masked(KIND_I8, SCALE_PER_CHANNEL, input, b_qweight, output,
                                     a_scale, b_scale, masked_m, expected_m_per_group)


def _masked_w4a8_impl(input, b_qweight, output, a_scale, b_scale, masked_m,
                      expected_m_per_group, mode):
    return _core.grouped_gemm_masked(KIND_W4A8, SCALE_PER_CHANNEL, input, b_qweight, output,
                                     a_scale, b_scale, masked_m, expected_m_per_group)


def _masked_bf16_impl(input, b_qweight, output, masked_m, expected_m_per_group, mode):
    return _core.grouped_gemm_masked(KIND_BF16, SCALE_NONE, input, b_qweight, output, None, None,
                                     masked_m, expected_m_per_group)


_define("m_grouped_marlin_w8a8_gemm_nt_masked", _MASKED_SCHEMA, _masked_i8_impl)
_define("m_grouped_marlin_w4a8_gemm_nt_masked", _MASKED_SCHEMA, _masked_w4a8_impl)
_define("m_grouped_marlin_w4a8_gemm_nt_masked_hipc", _MASKED_SCHEMA, _masked_w4a8_impl)
_BF16_SCHEMA = ("(Tensor input, Tensor b_qweight, Tensor(a!) output, Tensor masked_m, "
                "int expected_m_per_group, int mode) -> Tensor(a!)")
_define("m_grouped_bf16_gemm_nt_masked", _BF16_SCHEMA, _masked_bf16_impl)
_define("m_grouped_bf16_gemm_nt_masked_hipc", _BF16_SCHEMA, _masked_bf16_impl)


# --------------------------------------------------------------------------- contiguous
def _contig_block_impl(kind, scale_mode):
    def impl(input, b_qweight, output, a_scale, b_scale, m_indices, block_m, block_n, n_loop_num):
        return _core.grouped_gemm_contiguous(kind, scale_mode, input, b_qweight, output, a_scale,
                                             b_scale, m_indices)
    return impl


def _contig_mode_impl(kind, scale_mode):
    def impl(input, b_qweight, output, a_scale, b_scale, m_indices, mode):
        return _core.grouped_gemm_contiguous(kind, scale_mode, input, b_qweight, output, a_scale,
                                             b_scale, m_indices)
    return impl


def _contig_fp8_marlin_impl(scale_mode):
    def impl(input, b_qweight, output, a_scale, b_scale, m_indices, mode, n_loop_num):
        return _core.grouped_gemm_contiguous(KIND_E4M3, scale_mode, input, b_qweight, output,
                                             a_scale, b_scale, m_indices)
    return impl


_CONTIG_BLOCK_SCHEMA = ("(Tensor input, Tensor b_qweight, Tensor(a!) output, Tensor a_scale, "
                        "Tensor b_scale, Tensor m_indices, int block_m, int block_n, "
                        "int n_loop_num) -> Tensor(a!)")
_CONTIG_MODE_SCHEMA = ("(Tensor input, Tensor b_qweight, Tensor(a!) output, Tensor a_scale, "
                       "Tensor b_scale, Tensor m_indices, int mode) -> Tensor(a!)")
_CONTIG_MARLIN_SCHEMA = ("(Tensor input, Tensor b_qweight, Tensor(a!) output, Tensor a_scale, "
                         "Tensor b_scale, Tensor m_indices, int mode, int n_loop_num) -> Tensor(a!)")
_define("m_grouped_i8_gemm_nt_contiguous", _CONTIG_BLOCK_SCHEMA,
        _contig_block_impl(KIND_I8, SCALE_PER_CHANNEL))
_define("m_grouped_w8a8_gemm_nt_contiguous_gfx936", _CONTIG_BLOCK_SCHEMA,
        _contig_block_impl(KIND_I8, SCALE_PER_CHANNEL))
_define("m_grouped_fp8_gemm_nt_contiguous", _CONTIG_BLOCK_SCHEMA,
        _contig_block_impl(KIND_E4M3, SCALE_PER_CHANNEL))
_define("m_grouped_fp8_gemm_nt_contiguous_marlin", _CONTIG_MARLIN_SCHEMA,
        _contig_fp8_marlin_impl(SCALE_PER_CHANNEL))
_define("m_grouped_fp8_gemm_nt_contiguous_marlin_tensor_wise", _CONTIG_MARLIN_SCHEMA,
        _contig_fp8_marlin_impl(SCALE_TENSOR_WISE))
_define("m_grouped_w8a8_gemm_nt_contiguous", _CONTIG_MODE_SCHEMA,
        _contig_mode_impl(KIND_I8, SCALE_PER_CHANNEL))
_define("m_grouped_marlin_w4a8_gemm_nt_contiguous_hipc", _CONTIG_MODE_SCHEMA,
        _contig_mode_impl(KIND_W4A8, SCALE_PER_CHANNEL))

def _compact_impl(input, b_qweight, output, a_scale, b_scale, masked_m, expert_offsets,
                  expected_m_per_group):
    return _core.grouped_gemm_compact(KIND_I8, SCALE_PER_CHANNEL, input, b_qweight, output, a_scale,
                                      b_scale, masked_m, expert_offsets, expected_m_per_group)


def _nopad_impl(input, b_qweight, output, a_scale, b_scale, m_indices, token_per_expert):
    # rows of each expert follow one another without padding: offsets = running sum of counts
    counts = token_per_expert.to(torch.int32).contiguous()
    offsets = (torch.cumsum(counts, 0, dtype=torch.int32) - counts).contiguous()
    return _core.grouped_gemm_compact(KIND_I8, SCALE_PER_CHANNEL, input, b_qweight, output, a_scale,
                                      b_scale, counts, offsets, 0)


def _contig_bf16_impl(input, b_qweight, output, a_scale, b_scale, m_indices, mode):
    return _core.grouped_gemm_contiguous(KIND_BF16, SCALE_NONE, input, b_qweight, output, None, None,
                                         m_indices)


_define("m_grouped_marlin_w8a8_gemm_nt_compact_masked",
        "(Tensor input, Tensor b_qweight, Tensor(a!) output, Tensor a_scale, Tensor b_scale, "
        "Tensor masked_m, Tensor expert_offsets, int expected_m_per_group) -> Tensor(a!)", _compact_impl)
_define("m_grouped_w8a8_gemm_nt_nopad_contiguous",
        "(Tensor input, Tensor b_qweight, Tensor(a!) output, Tensor a_scale, Tensor b_scale, "
        "Tensor m_indices, Tensor token_per_expert) -> Tensor(a!)", _nopad_impl)
_define("m_grouped_w16a16_gemm_nt_contiguous", _CONTIG_MODE_SCHEMA, _contig_bf16_impl)

_ops = getattr(torch.ops, _NS)


# --------------------------------------------------------------------------- pybind names
def low_latency_grouped_gemm(matrix_a, matrix_b, matrix_a_scale, matrix_b_scale, actual_tokens,
                             matrix_c, max_tokens, experts, cu_s, block_wise, b_overlap,
                             signal: Optional[torch.Tensor] = None):
    return _impl.low_latency_grouped_gemm(matrix_a, matrix_b, matrix_a_scale, matrix_b_scale,
                                         actual_tokens, matrix_c, int(max_tokens), int(experts),
                                         int(cu_s), bool(block_wise), bool(b_overlap), signal)


def m_grouped_w8a8_gemm_nt_masked_gfx936(matrix_a, matrix_b, matrix_a_scale, matrix_b_scale,
                                         actual_tokens, matrix_c, max_tokens, experts, cu_s,
                                         block_wise, b_overlap,
                                         signal: Optional[torch.Tensor] = None):
    return _impl.m_grouped_w8a8_gemm_nt_masked_gfx936(
        matrix_a, matrix_b, matrix_a_scale, matrix_b_scale, actual_tokens, matrix_c,
        int(max_tokens), int(experts), int(cu_s), bool(block_wise), bool(b_overlap), signal)


def low_latency_grouped_gemm_tensor_wise(matrix_a, matrix_b, matrix_a_scale, matrix_b_scale,
                                         actual_tokens, matrix_c, max_tokens, experts, cu_s,
                                         b_overlap, signal: Optional[torch.Tensor] = None):
    return _impl.low_latency_grouped_gemm_tensor_wise(
        matrix_a, matrix_b, matrix_a_scale, matrix_b_scale, actual_tokens, matrix_c,
        int(max_tokens), int(experts), int(cu_s), bool(b_overlap), signal)


def m_grouped_marlin_w8a8_gemm_nt_masked(input, b_qweight, output, a_scale, b_scale, masked_m,
                                         expected_m_per_group, mode):
    return _impl.m_grouped_marlin_w8a8_gemm_nt_masked(input, b_qweight, output, a_scale, b_scale,
                                                     masked_m, int(expected_m_per_group), int(mode))


def m_grouped_marlin_w4a8_gemm_nt_masked(input, b_qweight, output, a_scale, b_scale, masked_m,
                                         expected_m_per_group, mode):
    return _impl.m_grouped_marlin_w4a8_gemm_nt_masked(input, b_qweight, output, a_scale, b_scale,
                                                     masked_m, int(expected_m_per_group), int(mode))


def m_grouped_marlin_w4a8_gemm_nt_masked_hipc(input, b_qweight, output, a_scale, b_scale,
                                              masked_m, expected_m_per_group, mode):
    return _impl.m_grouped_marlin_w4a8_gemm_nt_masked_hipc(
        input, b_qweight, output, a_scale, b_scale, masked_m, int(expected_m_per_group), int(mode))


def m_grouped_bf16_gemm_nt_masked(input, b_qweight, output, masked_m, expected_m_per_group, mode):
    return _impl.m_grouped_bf16_gemm_nt_masked(input, b_qweight, output, masked_m,
                                              int(expected_m_per_group), int(mode))


def m_grouped_bf16_gemm_nt_masked_hipc(input, b_qweight, output, masked_m, expected_m_per_group,
                                       mode):
    return _impl.m_grouped_bf16_gemm_nt_masked_hipc(input, b_qweight, output, masked_m,
                                                   int(expected_m_per_group), int(mode))


def m_grouped_w8a8_gemm_nt_contiguous(input, b_qweight, output, a_scale, b_scale, m_indices, mode):
    return _impl.m_grouped_w8a8_gemm_nt_contiguous(input, b_qweight, output, a_scale, b_scale,
                                                  m_indices, int(mode))


def m_grouped_marlin_w4a8_gemm_nt_contiguous_hipc(input, b_qweight, output, a_scale, b_scale,
                                                  m_indices, mode):
    return _impl.m_grouped_marlin_w4a8_gemm_nt_contiguous_hipc(input, b_qweight, output, a_scale,
                                                              b_scale, m_indices, int(mode))


def m_grouped_marlin_w8a8_gemm_nt_compact_masked(input, b_qweight, output, a_scale, b_scale,
                                                 masked_m, expert_offsets, expected_m_per_group):
    return _impl.m_grouped_marlin_w8a8_gemm_nt_compact_masked(
        input, b_qweight, output, a_scale, b_scale, masked_m, expert_offsets,
        int(expected_m_per_group))


def m_grouped_w8a8_gemm_nt_nopad_contiguous(input, b_qweight, output, a_scale, b_scale, m_indices,
                                            token_per_expert):
    return _impl.m_grouped_w8a8_gemm_nt_nopad_contiguous(input, b_qweight, output, a_scale, b_scale,
                                                        m_indices, token_per_expert)


def m_grouped_w16a16_gemm_nt_contiguous(input, b_qweight, output, a_scale, b_scale, m_indices, mode):
    return _impl.m_grouped_w16a16_gemm_nt_contiguous(input, b_qweight, output, a_scale, b_scale,
                                                    m_indices, int(mode))


def m_grouped_fp8_gemm_nt_contiguous(input, b_qweight, output, a_scale, b_scale, m_indices, mode):
    return _impl.m_grouped_fp8_gemm_nt_contiguous(input, b_qweight, output, a_scale, b_scale,
                                                 m_indices, int(mode), 256, 4)


# --------------------------------------------------------------------------- dense GEMM, einsum
def _check_identity_epilogue(alpha, beta, bias, where: str) -> None:
    if bias is not None:
        raise RuntimeError(f"{where}: bias is not supported")
    if float(alpha) != 1.0 or float(beta) != 0.0:
        raise RuntimeError(f"{where}: only alpha = 1, beta = 0 are supported")


def fp8_gemm(mat_a, mat_b, scale_a, scale_b, output, m, n, k, batch, transpose_flag, alpha, beta,
             bias=None):
    """Pybind name and argument order of the reference (csrc/include/deepgemm_ops.hpp; called
    from deepgemm/gemm.py:42 as ``op.fp8_gemm(B, A, scale_B, scale_A, d, n, m, k, batch, "TN",
    alpha, beta, None)``): the first operand is the [N, K] matrix, the second the [M, K] one."""
    from .gemm import _dense
    _check_identity_epilogue(alpha, beta, bias, "fp8_gemm")
    if transpose_flag != "TN":
        raise RuntimeError(f"fp8_gemm: only the TN layout is supported, got {transpose_flag!r}")
    _dense((mat_b, scale_b), (mat_a, scale_a), output, "fp8_gemm", (torch.float8_e4m3fn, torch.int8))
    return output


def fp8_gemm_hipc(mat_a, mat_b, scale_a, scale_b, output, m, n, k, batch, transpose_flag, alpha,
                  beta, bias=None):
    """As ``fp8_gemm``, e4m3 only (reference deepgemm/gemm.py:83)."""
    from .gemm import _dense
    _check_identity_epilogue(alpha, beta, bias, "fp8_gemm_hipc")
    if transpose_flag != "TN":
        raise RuntimeError(f"fp8_gemm_hipc: only the TN layout is supported, got {transpose_flag!r}")
    _dense((mat_b, scale_b), (mat_a, scale_a), output, "fp8_gemm_hipc", (torch.float8_e4m3fn,))
    return output


def einsum(expr, a, b, d, c=None):
    """Reference csrc/arch/gfx938/einsum.cu:157-183."""
    from .einsum import einsum as _einsum
    return _einsum(expr, a, b, d, c)


def fp8_einsum(expr, a, b, d, c=None, recipe=(1, 128, 128)):
    """Reference csrc/arch/gfx938/einsum.cu:185-222."""
    from .einsum import fp8_einsum as _fp8_einsum
    return _fp8_einsum(expr, a, b, d, c, recipe)
