"""Expert-parallel layer with the device-side exchange (dg_ep_plan / dg_ep_push / dg_ep_barrier and
the scattering epilogue of dg_contig_gemm).

One GPU: four ranks played on the same device, each with its own buffers and every rank's
pointers; the phases of all ranks are enqueued one after the other, so no kernel ever waits for a
kernel that has not been launched.  Every token's output must equal, bit for bit, what the
one-GPU layer that holds all experts computes for it (a row's result depends only on the row and
its expert; the top-k sum runs in the same order).  Two GPUs (skipped otherwise): the same check
with real ranks over symmetric memory."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

import deepgemm
from deepgemm import _cabi, ep_exchange as epx
from deepgemm.moe_chain import moe_forward

import dg_oracle as O

pytestmark = pytest.mark.gpu
E, T, H, INTER, TOPK = 16, 160, 512, 128, 4


def _layer_weights():
    g = torch.Generator().manual_seed(16)
    w13, s13 = O.per_token_quant_fp8(torch.randn(E, 2 * INTER, H, generator=g) * 0.05)
    w2, s2 = O.per_token_quant_fp8(torch.randn(E, H, INTER, generator=g) * 0.05)
    return w13, s13.reshape(E, -1), w2, s2.reshape(E, -1)


def _tokens(rank, t=T):
    g = torch.Generator().manual_seed(160 + rank)
    hidden = torch.randn(t, H, generator=g).bfloat16()
    # skewed routing: a few experts take most of the rows, some take none
    logits = torch.randn(t, E, generator=g) + torch.linspace(2.0, -2.0, E)
    topk = logits.topk(TOPK, dim=1).indices.to(torch.int32)
    w = torch.softmax(torch.randn(t, TOPK, generator=g), dim=1)
    return hidden, topk, w


def _one_gpu_layer(dev, rank, t=T):
    w13, s13, w2, s2 = _layer_weights()
    pk = deepgemm.marlin_fp8_contiguous_weight
    hidden, topk, w = _tokens(rank, t)
    return moe_forward(hidden.to(dev), topk.to(dev), w.to(dev), (pk(w13.clone().to(dev)), s13.to(dev)),
                       (pk(w2.clone().to(dev)), s2.to(dev))).cpu()


def _rank_weights(rank, world, dev):
    w13, s13, w2, s2 = _layer_weights()
    e_local = E // world
    sl = slice(rank * e_local, (rank + 1) * e_local)
    pk = deepgemm.marlin_fp8_contiguous_weight
    return (pk(w13[sl].clone().to(dev)), s13[sl].contiguous().to(dev)), \
           (pk(w2[sl].clone().to(dev)), s2[sl].contiguous().to(dev))


@pytest.mark.parametrize("world,slices", [(1, 1), (4, 1), (2, 3), (4, 2), (8, 1), (8, 2)])
def test_emulated_ranks_match_one_gpu_layer(world, slices):
    dev = torch.device("cuda", 0)
    m_cap = 4 * T * TOPK + (E // world) * 256
    ranks = epx.make_emulated_ranks(world, E, H, 2 * INTER, H, T, TOPK, m_cap, dev)
    toks = [_tokens(r) for r in range(world)]
    ws = [_rank_weights(r, world, dev) for r in range(world)]
    for rep in range(2):     # twice: epochs advance, buffers are re-used
        outs = epx.emulated_forward(ranks, [t[0].to(dev) for t in toks], [t[1].to(dev) for t in toks],
                                    [t[2].to(dev) for t in toks], [w[0] for w in ws], [w[1] for w in ws],
                                    slices=slices)
        torch.cuda.synchronize()
        for r in range(world):
            ranks[r].check_status()
            want = _one_gpu_layer(dev, r)
            assert torch.equal(outs[r].cpu().view(torch.int16), want.view(torch.int16)), \
                f"rank {r} of {world}, pass {rep}: layer output differs from the one-GPU layer"
    # the plan every rank derived is the one the counts table implies
    counts = torch.stack([torch.bincount(t[1].flatten().long(), minlength=E) for t in toks])
    for r in range(world):
        assert torch.equal(ranks[r].counts.cpu().long(), counts)
        my_base, m_indices, m_total = epx.layout_from_counts(counts, r, 256)
        assert torch.equal(ranks[r].my_base.cpu(), my_base)
        assert int(ranks[r].m_total) == m_total
        got = ranks[r].m_indices.cpu()
        assert torch.equal(got[:m_total], m_indices) and bool((got[m_total:] == -1).all())
        # every pair landed inside its expert's block of the owner's buffer, no row twice
        dest = ranks[r].pair_dest[:T * TOPK].cpu().long()
        assert int(dest.min()) >= 0
        for owner in range(world):
            sel = torch.div(toks[r][1].flatten().long(), E // world, rounding_mode="floor") == owner
            d = dest[sel]
            assert d.unique().numel() == d.numel()
            assert torch.equal(ranks[owner].m_indices.cpu()[d].long() + owner * (E // world),
                               toks[r][1].flatten().long()[sel])


def test_sliced_push_on_a_second_stream_one_rank():
    """``forward(slices=4)`` with one rank: the pushes run on a second stream, each gate/up GEMM waits
    for its slice only; same bits as the unsliced layer."""
    dev = torch.device("cuda", 0)
    x = epx.EPExchange(0, 1, E, H, 2 * INTER, H, T, TOPK, T * TOPK + E * 256, dev)
    w13, w2 = _rank_weights(0, 1, dev)
    hidden, topk, w = (t.to(dev) for t in _tokens(0))
    want = _one_gpu_layer(dev, 0)
    for slices in (4, 1, 16, 5):
        got = x.forward(hidden, topk, w, w13, w2, slices=slices).clone()
        torch.cuda.synchronize()
        x.check_status()
        assert torch.equal(got.cpu().view(torch.int16), want.view(torch.int16)), f"slices={slices}"


def test_rows_that_do_not_fit_are_dropped_and_reported():
    dev = torch.device("cuda", 0)
    ranks = epx.make_emulated_ranks(2, E, H, 2 * INTER, H, T, TOPK, 256, dev)   # far too small
    toks = [_tokens(r) for r in range(2)]
    ws = [_rank_weights(r, 2, dev) for r in range(2)]
    epx.emulated_forward(ranks, [t[0].to(dev) for t in toks], [t[1].to(dev) for t in toks],
                         [t[2].to(dev) for t in toks], [w[0] for w in ws], [w[1] for w in ws])
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="did not fit"):
        for r in ranks:
            r.check_status()


def test_a_peer_that_never_arrives_is_reported_not_waited_for_ever():
    """The waiting half of a barrier whose signal nobody posts gives up after its limit (2 s),
    records which peer was missing and returns; the device stays usable."""
    dev = torch.device("cuda", 0)
    ranks = epx.make_emulated_ranks(2, E, H, 2 * INTER, H, T, TOPK, 1024, dev)
    ranks[0].barrier(_cabi.EP_PHASE_POST)               # rank 0 posts its own arrival ...
    ranks[0].barrier(_cabi.EP_PHASE_WAIT)               # ... rank 1 never posts this epoch
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="gave up waiting for peer 1"):
        ranks[0].check_status()
    assert int(torch.ones(4, device=dev).sum()) == 4     # the context still works


def test_argument_errors():
    dev = torch.device("cuda", 0)
    x = epx.EPExchange(0, 1, E, H, 2 * INTER, H, T, TOPK, 4096, dev)
    hidden, topk, w = _tokens(0)
    with pytest.raises(ValueError):
        x.forward(hidden.to(dev), topk.to(dev).long(), w.to(dev), None, None)       # ids must be int32
    with pytest.raises(ValueError):
        epx.EPExchange(0, 3, E, H, 2 * INTER, H, T, TOPK, 4096, dev)                 # 16 experts over 3 ranks
    bad = _cabi.EpBarrierArgs(world=2, rank=5, epoch=1, phases=0, peer_flags=None, status=None)
    assert _cabi.lib.dg_ep_barrier(bad, None) != 0


def _worker(rank, world, port, q):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                      TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        x = epx.EPExchange(rank, world, E, H, 2 * INTER, H, T, TOPK, 4 * T * TOPK + 2048, dev)
        w13, w2 = _rank_weights(rank, world, dev)
        hidden, topk, w = _tokens(rank)
        outs = []
        for slices in (1, 2, 4):
            outs.append(x.forward(hidden.to(dev), topk.to(dev), w.to(dev), w13, w2, slices=slices).clone())
        torch.cuda.synchronize()
        x.check_status()
        assert all(torch.equal(o.view(torch.int16), outs[0].view(torch.int16)) for o in outs)
        q.put((rank, outs[0].cpu()))
    finally:
        dist.barrier()
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_two_gpus_match_one_gpu_layer():
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
    got = dict(q.get(timeout=240) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    dev = torch.device("cuda", 0)
    for r in range(world):
        want = _one_gpu_layer(dev, r)
        assert torch.equal(got[r].view(torch.int16), want.view(torch.int16)), f"rank {r} differs"
