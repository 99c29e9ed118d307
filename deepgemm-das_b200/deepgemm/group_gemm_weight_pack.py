"""Weight packers: row-major ``[E, N, K]`` -> the Blackwell tile layout of the kernels.

Same entry points as the reference's ``deepgemm/group_gemm_weight_pack.py`` (and the W6
packer of ``deepgemm/m_group_gemm.py:822-863``), same in-place contract -- the caller's
storage is rewritten expert by expert through one expert-sized temporary and a re-shaped view
of it is returned -- but a single target layout per element width instead of the W6 /
marlin / marlin2 / HIPC-N32 family:

    packed[e][kb][n][0:128 bytes] = bytes of row n of expert e covering K block kb

i.e. ``[E, K/128, N, 128]`` for int8 / fp8, ``[E, K/64, N, 64]`` for bf16 and, for int4,
``[E, K/256, N, 128]`` bytes where byte ``i`` of 16-byte chunk ``j`` holds ``w[32j+i]`` in the
high and ``w[32j+16+i]`` in the low nibble.  A (K-block, n-range) tile is one contiguous
span, fetched by a single TMA box.  The ``arch`` / ``mode`` / ``shuffle_unique`` /
``low_memory`` arguments selected among Hygon layouts; they are validated like the reference
does and otherwise ignored.

Packing runs on the tensor's device: a CUDA tensor goes through ``dg_pack_weight`` of the
C ABI, a CPU tensor through the equivalent torch index shuffles (used by the CPU tests and
by callers that pack before moving weights to the GPU).
"""
from __future__ import annotations

import ctypes as C
from typing import Any, Optional

import torch

from . import _cabi, _core
from ._cabi import KIND_BF16, KIND_E4M3, KIND_I8, KIND_W4A8, NIBBLE_HIGH_FIRST, NIBBLE_LOW_FIRST

# Layout-mode constants kept for API compatibility (reference :12-33).
I8_LAYOUT_MODE_W6_HIPC = 1
I8_LAYOUT_MODE_MASKED_LAYOUT_ASM = 2
I8_LAYOUT_MODE_W6 = I8_LAYOUT_MODE_W6_HIPC
I8_LAYOUT_MODE_MASKED_LAYOUT = I8_LAYOUT_MODE_MASKED_LAYOUT_ASM
I8_LAYOUT_MODE_DEFAULT = I8_LAYOUT_MODE_W6_HIPC
_I8_LAYOUT_MODES = (I8_LAYOUT_MODE_W6_HIPC, I8_LAYOUT_MODE_MASKED_LAYOUT_ASM)

BF16_MASKED_BM64_BN256_BK128_AUTO_MODE = 2000
BF16_MASKED_BM64_BN256_BK128_SMALL_M_MODE = 2001
BF16_MASKED_BM64_BN256_BK128_PREFETCH_MODE = 2002
BF16_MASKED_BM64_BN256_BK128_MODES = (
    BF16_MASKED_BM64_BN256_BK128_AUTO_MODE,
    BF16_MASKED_BM64_BN256_BK128_SMALL_M_MODE,
    BF16_MASKED_BM64_BN256_BK128_PREFETCH_MODE,
)
BF16_MASKED_BM64_BN256_BK128_LAYOUT = "bm64_bn256_bk128"
BF16_MASKED_ASM_MODES = (1000, 1001)
BF16_MASKED_ASM_LAYOUT = "native_nt"
# The one bf16 layout of this library; pack_bf16_masked_weight reports it in its config.
BF16_MASKED_TILE_LAYOUT = "kblock_n_64"

_ROW_BYTES = 128


def _get_current_gfx_arch() -> str:
    """The reference returns a Hygon gfx name; this library has one target."""
    return "sm_100a"


def _resolve_arch(arch: Optional[str]) -> str:
    return _get_current_gfx_arch() if arch is None else str(arch).split(":")[0]


def _resolve_shuffle_unique(shuffle_unique: int) -> int:
    value = int(shuffle_unique)
    if value not in (0, 1):
        raise ValueError(f"shuffle_unique must be 0 or 1, got {shuffle_unique}")
    return value


def _resolve_i8_layout_mode(mode: Any) -> int:
    value = int(mode)
    if value not in _I8_LAYOUT_MODES:
        raise ValueError(f"INT8 layout mode must be one of {_I8_LAYOUT_MODES}, got {mode}")
    return value


# ----------------------------------------------------------------------------- core re-layout
def _nibble_order(order) -> int:
    if order in (NIBBLE_HIGH_FIRST, "high_first", "high"):
        return NIBBLE_HIGH_FIRST
    if order in (NIBBLE_LOW_FIRST, "low_first", "low"):
        return NIBBLE_LOW_FIRST
    raise ValueError(f"nibble_order must be 'high_first' or 'low_first', got {order!r}")


def _torch_pack_rows(rows_u8: torch.Tensor, w4: bool, nibble_order: int) -> torch.Tensor:
    """CPU/any-device twin of dg_pack_weight for one expert: uint8 [N, row_bytes] -> packed."""
    n, row_bytes = rows_u8.shape
    blk = _ROW_BYTES
    x = rows_u8.view(n, row_bytes // blk, blk)
    if w4:
        x = x.reshape(n, row_bytes // blk, 8, 16)
        hi, lo = x >> 4, x & 0xF
        first, second = (hi, lo) if nibble_order == NIBBLE_HIGH_FIRST else (lo, hi)
        w = torch.stack((first, second), dim=-1).reshape(n, row_bytes // blk, 8, 2, 16)
        x = ((w[..., 0, :] << 4) | w[..., 1, :]).reshape(n, row_bytes // blk, blk)
    return x.permute(1, 0, 2).contiguous()


def _torch_unpack_rows(packed_u8: torch.Tensor, w4: bool, nibble_order: int) -> torch.Tensor:
    """Inverse of _torch_pack_rows: packed uint8 [KB, N, blk] -> [N, row_bytes]."""
    kb, n, blk = packed_u8.shape
    x = packed_u8.permute(1, 0, 2)
    if w4:
        x = x.reshape(n, kb, 8, 16)
        w = torch.stack((x >> 4, x & 0xF), dim=-2).reshape(n, kb, 8, 16, 2)  # value index 2t+h
        first, second = w[..., 0], w[..., 1]
        x = ((first << 4) | second) if nibble_order == NIBBLE_HIGH_FIRST else ((second << 4) | first)
    return x.reshape(n, kb * blk).contiguous()


def _pack_inplace(weight: torch.Tensor, kind: int, nibble_order: int = NIBBLE_HIGH_FIRST
                  ) -> torch.Tensor:
    """Rewrites ``weight`` ([E, N, row] row-major) to the tile layout in place; returns the
    4-D view ``[E, KB, N, row_per_block]`` of the same storage."""
    e, n, last = (int(v) for v in weight.shape)
    w4 = kind == KIND_W4A8
    row_bytes = last * weight.element_size()
    blk = _ROW_BYTES
    kb = row_bytes // blk
    k = last * 2 if w4 else last
    for ei in range(e):
        dst = weight[ei]
        if weight.is_cuda:
            tmp = dst.clone()
            with torch.cuda.device(weight.device):
                stream = torch.cuda.current_stream(weight.device).cuda_stream
                _cabi.check(_cabi.lib.dg_pack_weight(kind, tmp.data_ptr(), dst.data_ptr(), 1, n, k,
                                                     nibble_order, C.c_void_p(stream)),
                            "dg_pack_weight")
            # tmp is freed stream-ordered by the caching allocator after the kernel is queued
        else:
            rows = dst.reshape(n, last).view(torch.uint8)
            packed = _torch_pack_rows(rows, w4, nibble_order)
            dst.view(-1).view(torch.uint8).copy_(packed.view(-1))
    return weight.view(e, kb, n, blk // weight.element_size())


def unpack_weight(packed: torch.Tensor, kind: int, *, nibble_order="high_first") -> torch.Tensor:
    """Inverse of the packers (out of place): tile layout -> row-major ``[E, N, K]``
    (``[E, N, K/2]`` bytes for int4).  The reference has no inverse; tests use this one to
    prove that packing is a lossless permutation."""
    order = _nibble_order(nibble_order)
    w4 = kind == KIND_W4A8
    if w4 and packed.dim() == 3:
        e, n, kh = (int(v) for v in packed.shape)
        packed = packed.view(e, kh // 128, n, 128)
    if packed.dim() != 4:
        raise ValueError(f"packed weight must be 4-D [E, KB, N, row], got {tuple(packed.shape)}")
    e, kb, n, row = (int(v) for v in packed.shape)
    k = kb * {KIND_BF16: 64, KIND_W4A8: 256}.get(kind, 128)
    out = torch.empty((e, n, kb * row), dtype=packed.dtype, device=packed.device)
    if packed.is_cuda:
        src = packed.contiguous()
        with torch.cuda.device(packed.device):
            stream = torch.cuda.current_stream(packed.device).cuda_stream
            _cabi.check(_cabi.lib.dg_unpack_weight(kind, src.data_ptr(), out.data_ptr(), e, n, k,
                                                   order, C.c_void_p(stream)), "dg_unpack_weight")
    else:
        for ei in range(e):
            pk = packed[ei].contiguous().view(torch.uint8).reshape(kb, n, -1)
            rows = _torch_unpack_rows(pk, w4, order)
            out[ei].view(-1).view(torch.uint8).copy_(rows.view(-1))
    return out


def _validate_8bit_enk(weight: torch.Tensor, what: str) -> torch.Tensor:
    if weight.dim() == 2:
        weight = weight.unsqueeze(0)
    if weight.dim() != 3:
        raise ValueError(f"{what}: weight must be [E,N,K], got dim {weight.dim()} shape {tuple(weight.shape)}")
    if weight.element_size() != 1:
        raise ValueError(f"{what}: weight must be an 8-bit tensor")
    if not weight.is_contiguous():
        raise ValueError(f"{what}: in-place pack requires contiguous [E,N,K] weight input")
    n, k = int(weight.size(1)), int(weight.size(2))
    if n % 16 != 0 or k % 64 != 0:
        raise ValueError(f"{what}: N={n}, K={k} must satisfy N%16==0 and K%64==0")
    if k % 128 != 0:
        # The reference's W6 block is 64 values (m_group_gemm.py:815-818); the kernels here step K
        # in 128-byte blocks, so the last block is completed with zeros.  That tensor is larger
        # than its source: it is a new allocation, the one case where the pack is not in place.
        weight = torch.nn.functional.pad(weight.view(torch.uint8), (0, 64)).view(weight.dtype)
    return weight


# ----------------------------------------------------------------------------- int8 / fp8
def pack_int8_weight_enk_to_w6_low_latency_inplace(weight_enk: torch.Tensor) -> torch.Tensor:
    """8-bit ``[E,N,K]`` -> ``[E, K/128, N, 128]`` in place (reference: m_group_gemm.py:826-863,
    which produced the 6-D W6 view ``[E,K/64,N/16,4,16,16]``)."""
    weight_enk = _validate_8bit_enk(weight_enk, "pack_int8_weight_enk_to_w6_low_latency")
    kind = KIND_E4M3 if weight_enk.dtype == torch.float8_e4m3fn else KIND_I8
    return _pack_inplace(weight_enk, kind)


def pack_int8_weight_enk_to_w6_low_latency(weight_enk: torch.Tensor) -> torch.Tensor:
    return pack_int8_weight_enk_to_w6_low_latency_inplace(weight_enk)


def _marlin_i8(weight, shuffle_unique, mode, arch, what):
    _resolve_arch(arch)
    shuffle_unique = _resolve_shuffle_unique(shuffle_unique)
    mode = _resolve_i8_layout_mode(mode)
    if mode == I8_LAYOUT_MODE_MASKED_LAYOUT_ASM and shuffle_unique != 1:
        raise ValueError("INT8 layout mode=2 is only valid with shuffle_unique=1")
    return pack_int8_weight_enk_to_w6_low_latency_inplace(_validate_8bit_enk(weight, what))


def marlin_i8_contiguous_weight(weight: torch.Tensor, *, shuffle_unique: int = 1,
                                mode: int = I8_LAYOUT_MODE_DEFAULT, arch: Optional[str] = None,
                                low_memory: bool = True) -> torch.Tensor:
    """Reference: group_gemm_weight_pack.py:483-511."""
    return _marlin_i8(weight, shuffle_unique, mode, arch, "marlin_i8_contiguous_weight")


def marlin_i8_masked_weight(weight: torch.Tensor, *, shuffle_unique: int = 1,
                            mode: int = I8_LAYOUT_MODE_DEFAULT, arch: Optional[str] = None,
                            low_memory: bool = True) -> torch.Tensor:
    """Reference: group_gemm_weight_pack.py:514-542."""
    return _marlin_i8(weight, shuffle_unique, mode, arch, "marlin_i8_masked_weight")


def marlin_fp8_masked_weight(weight: torch.Tensor, *, arch: Optional[str] = None) -> torch.Tensor:
    """Reference: group_gemm_weight_pack.py:558-568."""
    _resolve_arch(arch)
    return pack_int8_weight_enk_to_w6_low_latency_inplace(
        _validate_8bit_enk(weight, "marlin_fp8_masked_weight"))


def marlin_fp8_contiguous_weight(weight: torch.Tensor, *, arch: Optional[str] = None
                                 ) -> torch.Tensor:
    """Reference: group_gemm_weight_pack.py:571-581."""
    _resolve_arch(arch)
    return pack_int8_weight_enk_to_w6_low_latency_inplace(
        _validate_8bit_enk(weight, "marlin_fp8_contiguous_weight"))


pack_i8_contiguous_weight = marlin_i8_contiguous_weight
pack_i8_masked_weight = marlin_i8_masked_weight
pack_fp8_contiguous_weight = marlin_fp8_contiguous_weight
pack_fp8_masked_weight = marlin_fp8_masked_weight
# Names of Hygon-specific variants: all produce the one tile layout here.
pack_i8_contiguous_weight_gfx936_asm_inplace = pack_int8_weight_enk_to_w6_low_latency_inplace
pack_i8_masked_weight_gfx936_asm_inplace = pack_int8_weight_enk_to_w6_low_latency_inplace
pack_w8a8_gfx936_weight_to_w6 = pack_int8_weight_enk_to_w6_low_latency_inplace
pack_int8_weight_enk_to_w6_gfx936_pack_permute = pack_int8_weight_enk_to_w6_low_latency_inplace


# ----------------------------------------------------------------------------- bf16
def pack_bf16_masked_weight(weight: torch.Tensor,
                            mode: int = BF16_MASKED_BM64_BN256_BK128_AUTO_MODE
                            ) -> tuple[torch.Tensor, dict[str, Any]]:
    """bf16 ``[E,N,K]`` -> (``[E, K/64, N, 64]`` in place, config for the front-end).
    Reference: group_gemm_weight_pack.py:463-480 (every accepted mode packs here)."""
    mode = int(mode)
    if mode not in BF16_MASKED_BM64_BN256_BK128_MODES and mode not in BF16_MASKED_ASM_MODES:
        raise ValueError(
            "BF16 masked mode must be 1000/1001 for asm layout or "
            f"2000/2001/2002 for BM64/BN256/BK128 layout, got {mode}")
    if weight.dim() != 3:
        raise ValueError(f"weight must be [E, N, K], got dim={weight.dim()}")
    if weight.dtype != torch.bfloat16:
        raise TypeError(f"weight must be torch.bfloat16, got {weight.dtype}")
    if not weight.is_contiguous():
        weight = weight.contiguous()
    n, k = int(weight.size(1)), int(weight.size(2))
    if n % 16 != 0:
        raise ValueError(f"N must be divisible by 16, got {n}")
    if k % 64 != 0:
        raise ValueError(f"K must be divisible by 64, got {k}")
    packed = _pack_inplace(weight, KIND_BF16)
    return packed, {"MODE": mode, "WEIGHT_LAYOUT": BF16_MASKED_TILE_LAYOUT, "PACKED_WEIGHT": True}


def marlin_bf16_masked_weight(weight: torch.Tensor, *, arch: Optional[str] = None) -> torch.Tensor:
    """Reference: group_gemm_weight_pack.py:545-555 (returned a new tensor; so does this)."""
    return pack_bf16_masked_weight(weight.clone())[0]


# ----------------------------------------------------------------------------- int4
def pack_w4a8_weight_k_contiguous(weight_u4: torch.Tensor) -> torch.Tensor:
    """int4 values ``[E,N,K]`` (one per element, low 4 bits used) -> framework bytes
    ``[E,N,K/2]`` with the even-k value in the high nibble (reference :594-602)."""
    if weight_u4.dim() != 3:
        raise ValueError(f"weight_u4 must be [E,N,K], got shape {tuple(weight_u4.shape)}")
    experts, n, k = weight_u4.shape
    if k % 2 != 0:
        raise ValueError(f"K must be divisible by 2 for W4 packing, got {k}")
    nib = (weight_u4.to(torch.uint8) & 0x0F).view(experts, n, k // 2, 2)
    return ((nib[..., 0] << 4) | nib[..., 1]).to(torch.int8)


def register_packed_w4a8_weight(weight: torch.Tensor) -> torch.Tensor:
    """Marks an ``[E,N,K/2]`` int4 tensor as being in the kernel layout.  The packed tensor keeps the
    framework shape (as the reference's does), so the shape cannot tell the two apart; the W4A8 ops
    accept a 3-D weight only if its storage was marked here -- the packers do it themselves.  Call
    it for weights that were packed elsewhere (for example loaded from a file that already holds
    the kernel layout)."""
    _core.PACKED_W4A8_STORAGES.add((weight.device.type, weight.device.index, weight.data_ptr()))
    return weight


def pack_w4a8_moe_hipc_weight_inplace(packed_k_contiguous: torch.Tensor, *,
                                      nibble_order="high_first") -> torch.Tensor:
    """Framework int4 bytes ``[E,N,K/2]`` -> kernel layout, in place; the returned tensor keeps
    the ``[E,N,K/2]`` shape like the reference's (:691-714).  ``nibble_order='low_first'``
    accepts sources whose even-k value sits in the low nibble."""
    if packed_k_contiguous.element_size() != 1:
        raise ValueError("packed_k_contiguous must be an 8-bit tensor")
    if packed_k_contiguous.dim() != 3:
        raise ValueError(
            f"packed_k_contiguous must be [E,N,K/2], got shape {tuple(packed_k_contiguous.shape)}")
    if not packed_k_contiguous.is_contiguous():
        packed_k_contiguous = packed_k_contiguous.contiguous()
    original_shape = packed_k_contiguous.shape
    _, n, k_half = (int(v) for v in original_shape)
    if k_half % 128 != 0:
        raise ValueError(f"K/2 must be divisible by 128 for the W4A8 tile layout, got {k_half}")
    if n % 16 != 0:
        raise ValueError(f"N must be divisible by 16 for the W4A8 tile layout, got {n}")
    _pack_inplace(packed_k_contiguous, KIND_W4A8, _nibble_order(nibble_order))
    register_packed_w4a8_weight(packed_k_contiguous)
    return packed_k_contiguous.view(original_shape)


def pack_w4a8_moe_hipc_weight(packed_k_contiguous: torch.Tensor, *,
                              nibble_order="high_first") -> torch.Tensor:
    """In-place; callers that still need the framework bytes pass a clone (reference :756-769)."""
    return pack_w4a8_moe_hipc_weight_inplace(packed_k_contiguous, nibble_order=nibble_order)


def view_w4a8_moe_hipc_weight_n32_layout(packed_hipc_weight: torch.Tensor) -> torch.Tensor:
    """The packed int4 tensor seen in kernel order ``[E, K/256, N, 128]`` (reference :717-727
    returned its N32 6-D order)."""
    if packed_hipc_weight.dim() != 3:
        raise ValueError(
            f"packed_hipc_weight must be [E,N,K/2], got shape {tuple(packed_hipc_weight.shape)}")
    experts, n, k_half = (int(v) for v in packed_hipc_weight.shape)
    if k_half % 128 != 0 or n % 16 != 0:
        raise ValueError(
            f"packed_hipc_weight shape [E,N,K/2]={tuple(packed_hipc_weight.shape)} must satisfy "
            "N%16==0 and K/2%128==0")
    return packed_hipc_weight.view(experts, k_half // 128, n, 128)


def weight4bit_nt_kpack2_marlin2_qqq_from_packed(packed_w: torch.Tensor) -> torch.Tensor:
    """Test-side packer name of the reference's ASM W4A8 path
    (op_test/deepgemm_marlin_quant.py:104-117): framework bytes -> kernel layout, out of place."""
    return pack_w4a8_moe_hipc_weight_inplace(packed_w.clone())
