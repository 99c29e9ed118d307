"""moe_w8a8_marlin_prefill_down_fp8 (second-stage MoE GEMM on a sorted routing list) against a
block-by-block CPU restatement of the reference kernel.  INT8: within 1 bf16 ulp (the int32
accumulators are exact, only the fp32 scale products can round differently from the float64
oracle); FP8 with small-integer values: the same bar."""
import pytest
import torch

import deepgemm

import dg_oracle as O
from helpers import assert_bf16_within_ulp

pytestmark = pytest.mark.gpu
DEV = "cuda"
FP8 = torch.float8_e4m3fn


@pytest.fixture(params=["gather", "regroup"], autouse=True)
def _path(request):
    """Every test runs through both implementations: the one-launch GEMM that gathers the rows
    itself, and the regroup step + scattering contiguous GEMM used for large problems."""
    from deepgemm import moe_marlin_prefill as M
    M.FORCE_PATH = request.param
    yield request.param
    M.FORCE_PATH = None


def _case(kind, t, k, e, hid, n, block_m, seed, local=None, extra_blocks=0):
    g = torch.Generator().manual_seed(seed)
    topk_ids = torch.rand(t, e, generator=g).topk(k, dim=1).indices
    if kind == "int8":
        inp = torch.randint(-128, 128, (t * k, hid), generator=g).to(torch.int8)
        w = torch.randint(-128, 128, (e, n, hid), generator=g).to(torch.int8)
    else:
        inp = torch.randint(-6, 7, (t * k, hid), generator=g).float().to(FP8)
        w = torch.randint(-6, 7, (e, n, hid), generator=g).float().to(FP8)
    a_scale = torch.rand(t * k, generator=g) * 0.02 + 0.01
    b_scale = torch.rand(e, n, generator=g) * 0.02 + 0.01
    topk_w = torch.softmax(torch.randn(t, k, generator=g), dim=1)
    ids, experts, used = O.build_sorted_routing(topk_ids, e, block_m, local, extra_blocks)
    return dict(inp=inp, w=w, a_scale=a_scale, b_scale=b_scale, topk_w=topk_w, ids=ids, experts=experts,
                used=used, k=k)


def _call(c, kind, sentinel=3.0):
    pack = deepgemm.marlin_fp8_contiguous_weight if kind == "fp8" else deepgemm.marlin_i8_contiguous_weight
    size_m, n = c["inp"].shape[0], c["w"].shape[1]
    out = torch.full((size_m, n), sentinel, dtype=torch.bfloat16, device=DEV)
    r = deepgemm.moe_w8a8_marlin_prefill_down_fp8(
        c["inp"].to(DEV), pack(c["w"].clone().to(DEV)), out, c["a_scale"].to(DEV), c["b_scale"].to(DEV),
        c["topk_w"].to(DEV), c["ids"].to(DEV), c["experts"].to(DEV), c["used"].to(DEV), c["k"], c["k"])
    assert r is out
    return out


def _run(c, kind, sentinel=3.0):
    out = _call(c, kind, sentinel)
    size_m, n = c["inp"].shape[0], c["w"].shape[1]
    want = O.ref_prefill_down(c["inp"], c["w"], c["a_scale"], c["b_scale"], c["topk_w"], c["ids"],
                              c["experts"], c["used"], c["k"],
                              torch.full((size_m, n), sentinel, dtype=torch.bfloat16))
    return out.cpu(), want


@pytest.mark.parametrize("kind", ["int8", "fp8"])
@pytest.mark.parametrize("t,k,e,hid,n,block_m", [(200, 4, 6, 256, 512, 32), (64, 2, 3, 128, 1024, 16),
                                                 (1500, 8, 32, 512, 512, 32),
                                                 (100, 2, 4, 192, 512, 32)])   # K % 128 == 64, as the reference takes
def test_matches_the_block_by_block_oracle(kind, t, k, e, hid, n, block_m):
    c = _case(kind, t, k, e, hid, n, block_m, seed=t + e, extra_blocks=2)
    out, want = _run(c, kind)
    assert_bf16_within_ulp(out, want, 1, f"prefill-down {kind} T={t} top{k} E={e}")


def test_rows_the_list_never_names_stay_untouched():
    """Only the rows named by sorted_token_ids are written (the reference's kernel touches nothing
    else), so several calls can fill disjoint rows of one output tensor."""
    c = _case("int8", 96, 4, 6, 256, 512, 32, seed=9)
    keep = c["ids"].clone()
    blocks = keep.numel() // 32
    dropped = keep.view(blocks, 32)[::2].clone()
    keep.view(blocks, 32)[::2] = (4 << 24)                    # every other block becomes padding (slot >= top-k)
    c2 = dict(c, ids=keep)
    out, want = _run(c2, "int8", sentinel=5.0)
    assert_bf16_within_ulp(out, want, 1, "prefill-down with half of the blocks masked out")
    rows = ((dropped.long() & 0xFFFFFF) * 4 + (dropped.long() >> 24)).flatten()
    rows = rows[(dropped.flatten().long() >> 24) < 4]
    named = ((keep.long() & 0xFFFFFF) * 4 + (keep.long() >> 24))[(keep.long() >> 24) < 4]
    only_dropped = rows[~torch.isin(rows, named)]
    assert only_dropped.numel() > 0 and bool((out[only_dropped].float() == 5.0).all())


def test_experts_of_other_ranks_give_zero_rows():
    c = _case("int8", 120, 4, 8, 256, 512, 32, seed=5, local={0, 1, 2, 3})
    out, want = _run(c, "int8")
    assert_bf16_within_ulp(out, want, 1, "prefill-down, half of the experts remote")
    assert float(want.abs().sum()) > 0 and torch.any(torch.all(out == 0, dim=1))


def test_gathering_gemm_is_one_launch_and_matches_the_regroup_path_bit_for_bit(_path):
    from deepgemm import _cabi, moe_marlin_prefill as M
    if _path != "gather":
        pytest.skip("compares the two paths once")
    # the last case is large enough for the regroup path's GEMM to take the two-CTA tiles (1024
    # routed rows per expert, 160 units); two of its experts live elsewhere
    for kind, n, shape in (("int8", 512, (300, 4, 7, 448, 16)), ("fp8", 384, (300, 4, 7, 448, 16)),
                           ("int8", 1280, (2048, 4, 8, 192, 32))):
        t_, k_, e_, hid_, bm_ = shape
        c = _case(kind, t_, k_, e_, hid_, n, bm_, seed=77, local=set(range(e_)) - {1, 4}, extra_blocks=3)
        before = _cabi.query(_cabi.QUERY_LAUNCH_COUNT)
        out_g, _ = _run(c, kind)
        # the weight packer launches once per expert; the op itself is one launch
        assert _cabi.query(_cabi.QUERY_LAUNCH_COUNT) - before == c["w"].shape[0] + 1
        M.FORCE_PATH = "regroup"
        out_r, _ = _run(c, kind)
        M.FORCE_PATH = "gather"
        assert torch.equal(out_g.view(torch.int16), out_r.view(torch.int16)), kind
    deepgemm.check_device_status()


@pytest.mark.parametrize("block_m", [16, 64, 128])
def test_other_block_sizes(block_m):
    c = _case("int8", 150, 4, 5, 256, 512, block_m, seed=block_m, extra_blocks=1)
    out, want = _run(c, "int8")
    assert_bf16_within_ulp(out, want, 1, f"prefill-down block_m={block_m}")


def test_a_list_that_is_not_sorted_by_expert(_path):
    """Blocks of one expert need not be neighbours: every run of blocks is tiled on its own.  The
    gathering GEMM holds 2 * experts + 2 runs; beyond that it computes nothing and says so."""
    c = _case("int8", 200, 4, 4, 256, 512, 16, seed=31)
    blocks = c["experts"].numel()
    used_blocks = int(c["used"]) // 16
    g = torch.Generator().manual_seed(3)
    perm = torch.cat([torch.randperm(used_blocks, generator=g), torch.arange(used_blocks, blocks)])
    ids = c["ids"].view(blocks, 16)[perm].reshape(-1).contiguous()
    experts = c["experts"][perm].contiguous()
    runs = 1 + int((experts[1:used_blocks] != experts[:used_blocks - 1]).sum())
    c2 = dict(c, ids=ids, experts=experts)
    if _path == "gather" and runs > 2 * 4 + 2:
        out, _ = _run(c2, "int8", sentinel=5.0)
        assert bool((out.float() == 5.0).all()), "a refused list must leave the output alone"
        with pytest.raises(RuntimeError, match="expert index"):
            deepgemm.check_device_status()
        # a few runs more than experts are fine: swap two neighbouring blocks of different experts
        b = int(torch.nonzero(c["experts"][1:used_blocks] != c["experts"][:used_blocks - 1])[0]) + 1
        perm2 = torch.arange(blocks)
        perm2[b - 1], perm2[b] = b, b - 1
        c3 = dict(c, ids=c["ids"].view(blocks, 16)[perm2].reshape(-1).contiguous(),
                  experts=c["experts"][perm2].contiguous())
        out, want = _run(c3, "int8")
        assert_bf16_within_ulp(out, want, 1, "two blocks swapped")
    else:
        out, want = _run(c2, "int8")
        assert_bf16_within_ulp(out, want, 1, "unsorted list")
    deepgemm.check_device_status()


def test_empty_list_and_unknown_experts(_path):
    c = _case("int8", 40, 2, 3, 128, 256, 32, seed=8)
    out, _ = _run(dict(c, used=torch.zeros(1, dtype=torch.int32)), "int8", sentinel=5.0)
    assert bool((out.float() == 5.0).all()), "a list with no entries in use writes nothing"
    deepgemm.check_device_status()
    bad = c["experts"].clone()
    bad[0] = 7                                                  # only experts 0..2 exist
    out = _call(dict(c, experts=bad), "int8", sentinel=5.0).cpu()
    if _path == "gather":
        with pytest.raises(RuntimeError, match="expert index"):
            deepgemm.check_device_status()
    else:
        try:
            deepgemm.check_device_status()
        except RuntimeError:
            pass
    rows = ((c["ids"][:32].long() & 0xFFFFFF) * 2 + (c["ids"][:32].long() >> 24))[(c["ids"][:32].long() >> 24) < 2]
    assert bool((out[rows].float() == 5.0).all()), "rows of a block with an unknown expert are skipped"
    others = torch.ones(out.shape[0], dtype=torch.bool)
    others[rows] = False
    c_ok = dict(c)
    out_ok, want_ok = _run(c_ok, "int8", sentinel=5.0)
    assert torch.equal(out[others].view(torch.int16), out_ok[others].view(torch.int16))


def test_argument_errors():
    c = _case("int8", 16, 2, 2, 128, 512, 32, seed=1)
    pk = deepgemm.marlin_i8_contiguous_weight(c["w"].clone().to(DEV))
    out = torch.zeros(32, 512, dtype=torch.bfloat16, device=DEV)
    args = [c["inp"].to(DEV), pk, out, c["a_scale"].to(DEV), c["b_scale"].to(DEV), c["topk_w"].to(DEV),
            c["ids"].to(DEV), c["experts"].to(DEV), c["used"].to(DEV), 2, 2]
    bad = list(args)
    bad[6] = bad[6].to(torch.int64)
    with pytest.raises(RuntimeError):
        deepgemm.moe_w8a8_marlin_prefill_down_fp8(*bad)
    bad = list(args)
    bad[1] = c["w"].to(DEV)                                   # not packed
    with pytest.raises(RuntimeError):
        deepgemm.moe_w8a8_marlin_prefill_down_fp8(*bad)
    bad = list(args)
    bad[2] = out.float()
    with pytest.raises(RuntimeError):
        deepgemm.moe_w8a8_marlin_prefill_down_fp8(*bad)
    with pytest.raises(ValueError):
        deepgemm.assert_moe_prefill_down_fp8_shapes(k=100, n=512)
    with pytest.raises(ValueError):
        deepgemm.assert_moe_prefill_down_fp8_shapes(k=128, n=640)
    deepgemm.assert_moe_prefill_down_fp8_shapes(k=128, n=1024)
