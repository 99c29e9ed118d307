"""Host-side logic of the expert-parallel harness on CPU: routing plan, all-to-all dispatch
between two gloo ranks, grouping/padding into the contiguous layout.  The GEMM itself is
covered by the GPU tests; here a rank-by-rank result is compared with a single-process
computation of the same global routing."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from deepgemm import expert_parallel as ep

E, T, H, TOPK = 8, 24, 16, 3


def _inputs(rank):
    g = torch.Generator().manual_seed(50 + rank)
    hidden = torch.randn(T, H, generator=g).to(torch.bfloat16)
    topk = ep.route_topk(torch.randn(T, E, generator=g), TOPK)
    return hidden, topk


def test_plan_orders_rows_by_expert():
    hidden, topk = _inputs(0)
    plan = ep.build_dispatch_plan(topk, E, 2)
    assert plan.send_expert.tolist() == sorted(topk.flatten().tolist())
    assert sum(plan.send_splits) == T * TOPK
    assert plan.send_splits[0] == int((topk < E // 2).sum())
    for tok, e in zip(plan.send_token.tolist(), plan.send_expert.tolist()):
        assert e in topk[tok].tolist()


def test_group_and_pad_layout():
    g = torch.Generator().manual_seed(1)
    rows = torch.randn(37, H, generator=g)
    expert = torch.randint(0, 4, (37,), generator=g)
    expert[expert == 2] = 3                                   # leave expert 2 empty
    padded, m_indices, dest = ep.group_and_pad(rows, expert, 4, align=8)
    assert padded.shape[0] % 8 == 0 and m_indices.shape[0] == padded.shape[0]
    assert torch.equal(padded[dest], rows)                    # every row landed where dest says
    assert torch.equal(m_indices[dest], expert.to(torch.int32))
    assert int((m_indices >= 0).sum()) == 37
    valid = m_indices[m_indices >= 0]
    assert torch.equal(valid, torch.sort(valid).values)       # grouped by expert
    for e in range(4):                                        # each group starts on a multiple of align
        pos = torch.nonzero(m_indices == e).flatten()
        if pos.numel():
            assert int(pos[0]) % 8 == 0 and int(pos[-1] - pos[0]) == pos.numel() - 1
    assert torch.all(padded[m_indices < 0] == 0)
    # stable: rows of one expert keep their arrival order
    e3 = torch.nonzero(expert == 3).flatten()
    assert torch.equal(dest[e3], torch.sort(dest[e3]).values)


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        hidden, topk = _inputs(rank)
        plan = ep.build_dispatch_plan(topk, E, world)
        rows, expert_local = ep.dispatch_tokens(hidden, plan, E, rank, world)
        # quantised rows travel as bytes with their scales: here the "scale" names (rank, token)
        tag = torch.arange(T, dtype=torch.float32) + 1000.0 * rank
        rows8, _, scale = ep.dispatch_tokens(hidden.view(torch.uint8), plan, E, rank, world, row_scale=tag)
        assert torch.equal(rows8.view(torch.bfloat16), rows)
        # each token once per destination rank: the pairs must read the same rows as before
        urows, src_index, uexpert, usplits, uscale = ep.dispatch_unique(hidden, plan, E, rank, world,
                                                                         row_scale=tag)
        assert torch.equal(urows.index_select(0, src_index.long()), rows)
        assert torch.equal(uexpert.long(), expert_local) and torch.equal(uscale[src_index.long()], scale)
        assert urows.shape[0] <= rows.shape[0] and len(torch.unique(uscale)) == urows.shape[0]
        q.put((rank, rows.float(), expert_local, scale))
    finally:
        dist.barrier()
        dist.destroy_process_group()


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.timeout(120)
def test_two_rank_dispatch_matches_single_process_routing():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = {}
    for _ in range(world):
        r, rows, expert_local, scale = q.get(timeout=90)
        got[r] = (rows, expert_local, scale)
    for p in procs:
        p.join(timeout=30)
        assert p.exitcode == 0
    e_local = E // world
    for r in range(world):
        # expectation: for each source rank in order, its rows for r's experts, ordered by expert
        want_rows, want_exp, want_tag = [], [], []
        for src in range(world):
            hidden, topk = _inputs(src)
            plan = ep.build_dispatch_plan(topk, E, world)
            sel = (plan.send_expert >= r * e_local) & (plan.send_expert < (r + 1) * e_local)
            want_rows.append(hidden.index_select(0, plan.send_token[sel]).float())
            want_exp.append(plan.send_expert[sel] - r * e_local)
            want_tag.append(plan.send_token[sel].float() + 1000.0 * src)
        rows, expert_local, scale = got[r]
        assert torch.equal(scale, torch.cat(want_tag))
        assert torch.equal(rows, torch.cat(want_rows))
        assert torch.equal(expert_local, torch.cat(want_exp))


def _toy_mlp(rows, local_expert, first_expert):
    """Stand-in for the experts' two GEMMs: depends on the row and on the global expert id."""
    return rows.float() * (1.0 + (local_expert + first_expert).float()[:, None])


def _toy_combine(y, src_row, weights):
    return (y[src_row.long()] * weights[:, :, None]).sum(dim=1)


def _layer_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        hidden, topk = _inputs(rank)
        w = torch.softmax(torch.randn(T, TOPK, generator=torch.Generator().manual_seed(70 + rank)), dim=1)
        first = rank * (E // world)
        out = ep.ep_moe_forward(hidden, topk, w, None, None, E, rank, world,
                                expert_mlp=lambda r, e: _toy_mlp(r, e, first), combine=_toy_combine)
        q.put((rank, out))
    finally:
        dist.barrier()
        dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_two_rank_layer_returns_every_pair_to_its_token():
    """dispatch -> per-expert function -> reverse all-to-all -> weighted sum over two gloo ranks
    equals the direct per-token computation (the GEMMs are replaced by an expert-dependent toy
    function, so a row sent to the wrong expert or returned to the wrong token shows)."""
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_layer_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=90) for _ in range(world))
    for p in procs:
        p.join(timeout=30)
        assert p.exitcode == 0
    for r in range(world):
        hidden, topk = _inputs(r)
        w = torch.softmax(torch.randn(T, TOPK, generator=torch.Generator().manual_seed(70 + r)), dim=1)
        want = (hidden.float()[:, None, :] * (1.0 + topk.float())[:, :, None] * w[:, :, None]).sum(dim=1)
        assert torch.allclose(got[r], want, rtol=1e-6, atol=1e-6), f"rank {r}"
    # world size 1 takes the same code path without communication
    hidden, topk = _inputs(0)
    w = torch.ones(T, TOPK)
    out = ep.ep_moe_forward(hidden, topk, w, None, None, E, 0, 1,
                            expert_mlp=lambda r, e: _toy_mlp(r, e, 0), combine=_toy_combine)
    assert torch.allclose(out, (hidden.float()[:, None, :] * (1.0 + topk.float())[:, :, None]).sum(dim=1))
