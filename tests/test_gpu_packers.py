"""dg_pack_weight / dg_unpack_weight on the GPU against the torch (CPU) definition of the
layout, and the C ABI's device queries."""
import pytest
import torch

from deepgemm import _cabi
from deepgemm import group_gemm_weight_pack as P

pytestmark = pytest.mark.gpu
DEV = "cuda"


def test_device_queries():
    assert _cabi.query(_cabi.QUERY_CC) // 10 == 10
    assert _cabi.query(_cabi.QUERY_SM_COUNT) == torch.cuda.get_device_properties(0).multi_processor_count
    assert _cabi.query(_cabi.QUERY_MAX_SMEM) >= 227 * 1024


@pytest.mark.parametrize("dtype", [torch.int8, torch.float8_e4m3fn])
def test_gpu_pack_matches_cpu_pack_8bit(dtype):
    w = torch.randint(-128, 128, (5, 272, 896), dtype=torch.int8).view(dtype)
    cpu = P.pack_int8_weight_enk_to_w6_low_latency(w.clone())
    wg = w.clone().to(DEV)
    gpu = P.pack_int8_weight_enk_to_w6_low_latency(wg)
    assert gpu.data_ptr() == wg.data_ptr() and gpu.shape == cpu.shape
    assert torch.equal(gpu.cpu().view(torch.uint8), cpu.view(torch.uint8))
    kind = _cabi.KIND_E4M3 if dtype == torch.float8_e4m3fn else _cabi.KIND_I8
    assert torch.equal(P.unpack_weight(gpu, kind).cpu().view(torch.uint8), w.view(torch.uint8))


def test_gpu_pack_matches_cpu_pack_bf16_and_int4():
    w = torch.randn(3, 48, 320).bfloat16()
    cpu, _ = P.pack_bf16_masked_weight(w.clone())
    gpu, _ = P.pack_bf16_masked_weight(w.clone().to(DEV))
    assert torch.equal(gpu.cpu().view(torch.int16), cpu.view(torch.int16))
    assert torch.equal(P.unpack_weight(gpu, _cabi.KIND_BF16).cpu().view(torch.int16), w.view(torch.int16))
    for order in ("high_first", "low_first"):
        fw = torch.randint(-128, 128, (3, 48, 384), dtype=torch.int8)
        cpu = P.pack_w4a8_moe_hipc_weight(fw.clone(), nibble_order=order)
        gpu = P.pack_w4a8_moe_hipc_weight(fw.clone().to(DEV), nibble_order=order)
        assert torch.equal(gpu.cpu(), cpu)
        assert torch.equal(P.unpack_weight(gpu, _cabi.KIND_W4A8, nibble_order=order).cpu(), fw)
