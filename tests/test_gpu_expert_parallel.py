"""Expert-parallel harness on GPUs: dispatch -> fused quantise/group -> contiguous FP8 GEMM.

One GPU: the world-size-1 path against the CPU oracle.  Two or more GPUs (skipped otherwise):
two NCCL ranks, experts split between them; every routed (token, expert) pair must produce
the same output row as the single-rank run of the same global routing, bit for bit (rows are
quantised per token and each row's result depends on that row and its expert only)."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

import deepgemm
from deepgemm import expert_parallel as ep
from deepgemm.quant_utils import per_token_quant_fp8

import dg_oracle as O
from helpers import assert_calc_diff

pytestmark = pytest.mark.gpu
E, T, H, N, TOPK = 8, 192, 512, 256, 2


def _weights():
    g = torch.Generator().manual_seed(5)
    return O.per_token_quant_fp8(torch.randn(E, N, H, generator=g))


def _tokens(rank):
    g = torch.Generator().manual_seed(60 + rank)
    hidden = torch.randn(T, H, generator=g).bfloat16()
    topk = ep.route_topk(torch.randn(T, E, generator=g), TOPK)
    return hidden, topk


def _run_rank(rank, world, dev):
    b, b_s = _weights()
    e_local = E // world
    bl = b[rank * e_local:(rank + 1) * e_local].clone().to(dev)
    bp = deepgemm.marlin_fp8_contiguous_weight(bl)
    bs = b_s[rank * e_local:(rank + 1) * e_local].reshape(e_local, N).to(dev)
    hidden, topk = _tokens(rank)
    out, m_idx, recv_expert, dest = ep.ep_gate_up_forward(hidden.to(dev), topk.to(dev), bp, bs, E, rank, world)
    torch.cuda.synchronize()
    return out.cpu(), recv_expert.cpu(), dest.cpu().long()


def test_single_rank_forward_matches_oracle():
    out, recv_expert, dest = _run_rank(0, 1, torch.device("cuda", 0))
    b, b_s = _weights()
    hidden, topk = _tokens(0)
    plan = ep.build_dispatch_plan(topk, E, 1)
    rows = hidden.index_select(0, plan.send_token)
    qa, sa = O.per_token_quant_fp8(rows)
    assert torch.equal(recv_expert, plan.send_expert)
    for e in range(E):
        r = torch.nonzero(recv_expert == e).flatten()
        if r.numel():
            ref = O.ref_masked_scaled(qa[r][None], b[e][None], sa[r][None], b_s[e][None])[0]
            assert_calc_diff(out[dest[r]], ref, 1e-3, f"expert {e}")           # calc_diff < 1e-3


def _worker(rank, world, port, q):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        out, recv_expert, dest = _run_rank(rank, world, dev)
        q.put((rank, out[dest].clone(), recv_expert))
    finally:
        dist.barrier()
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_two_ranks_match_single_rank_rows():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = {}
    for _ in range(world):
        r, rows_out, recv_expert = q.get(timeout=240)
        got[r] = (rows_out, recv_expert)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    # single-device recomputation of every (source rank, token, expert) row with all experts
    b, b_s = _weights()
    bp = deepgemm.marlin_fp8_contiguous_weight(b.clone().cuda())
    e_local = E // world
    for r in range(world):
        want_rows = []
        for src in range(world):
            hidden, topk = _tokens(src)
            plan = ep.build_dispatch_plan(topk, E, world)
            sel = (plan.send_expert >= r * e_local) & (plan.send_expert < (r + 1) * e_local)
            rows = hidden.index_select(0, plan.send_token[sel]).cuda()
            a, a_s, m_idx, dest, _ = deepgemm.quantize_group_rows(rows, plan.send_expert[sel].cuda(), E)
            out = torch.zeros(a.shape[0], N, dtype=torch.bfloat16, device="cuda")
            deepgemm.m_grouped_fp8_gemm_nt_contiguous((a, a_s), (bp, b_s.reshape(E, N).cuda()), out, m_idx)
            want_rows.append(out[dest.long()].cpu())
        want = torch.cat(want_rows)
        assert torch.equal(got[r][0].view(torch.int16), want.view(torch.int16)), f"rank {r} rows differ"


# ---------------------------------------------------------------- whole layer (gate/up -> down)
INTER = 128


def _layer_weights():
    g = torch.Generator().manual_seed(6)
    w13, s13 = O.per_token_quant_fp8(torch.randn(E, 2 * INTER, H, generator=g) * 0.05)
    w2, s2 = O.per_token_quant_fp8(torch.randn(E, H, INTER, generator=g) * 0.05)
    return w13, s13.reshape(E, -1), w2, s2.reshape(E, -1)


def _layer_tokens(rank):
    hidden, topk = _tokens(rank)
    w = torch.softmax(torch.randn(T, TOPK, generator=torch.Generator().manual_seed(80 + rank)), dim=1)
    return hidden, topk, w


def _run_layer(rank, world, dev, quantise_before_dispatch=True):
    w13, s13, w2, s2 = _layer_weights()
    e_local = E // world
    sl = slice(rank * e_local, (rank + 1) * e_local)
    pk = deepgemm.marlin_fp8_contiguous_weight
    hidden, topk, w = _layer_tokens(rank)
    out = ep.ep_moe_forward(hidden.to(dev), topk.to(dev), w.to(dev),
                            (pk(w13[sl].clone().to(dev)), s13[sl].to(dev)),
                            (pk(w2[sl].clone().to(dev)), s2[sl].to(dev)), E, rank, world,
                            quantise_before_dispatch=quantise_before_dispatch)
    torch.cuda.synchronize()
    return out.cpu()


def test_single_rank_layer_matches_oracle():
    out = _run_layer(0, 1, torch.device("cuda", 0))
    hidden, topk, w = _layer_tokens(0)
    ref = O.ref_moe_layer(hidden, topk, w, *_layer_weights())
    assert_calc_diff(out, ref.float(), 1e-3, "expert-parallel layer, one rank")    # calc_diff < 1e-3
    late = _run_layer(0, 1, torch.device("cuda", 0), quantise_before_dispatch=False)
    assert torch.equal(out.view(torch.int16), late.view(torch.int16)), \
        "quantising before or after the dispatch must not change a single bit"


def _layer_worker(rank, world, port, q):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        early = _run_layer(rank, world, dev, quantise_before_dispatch=True)
        late = _run_layer(rank, world, dev, quantise_before_dispatch=False)
        assert torch.equal(early.view(torch.int16), late.view(torch.int16))
        q.put((rank, early))
    finally:
        dist.barrier()
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_two_rank_layer_matches_one_gpu_layer():
    """Every token's output from the two-rank layer equals, bit for bit, what one GPU holding all
    experts computes for the same token (each pair's row depends only on its token and expert,
    and the top-k sum runs in the same order)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_layer_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=240) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    w13, s13, w2, s2 = _layer_weights()
    pk = deepgemm.marlin_fp8_contiguous_weight
    dev = torch.device("cuda", 0)
    for r in range(world):
        hidden, topk, w = _layer_tokens(r)
        want = deepgemm.moe_forward(hidden.to(dev), topk.to(dev), w.to(dev),
                                    (pk(w13.clone().to(dev)), s13.to(dev)),
                                    (pk(w2.clone().to(dev)), s2.to(dev))).cpu()
        assert torch.equal(got[r].view(torch.int16), want.view(torch.int16)), f"rank {r} tokens differ"
