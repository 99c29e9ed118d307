"""Expert-parallel MoE layer whose token exchange runs over peer memory (NVLink / NVSwitch).

The reference library is single-GPU; a serving framework that shards its experts over the GPUs
of a box moves the routed rows itself.  ``expert_parallel.py`` does that with NCCL all-to-alls
(host-known split sizes, hence a host synchronisation, plus a regroup pass on the receiver).
This module is the device-side form: every rank maps one buffer of every other rank
(``torch.distributed``'s symmetric memory) and the kernels behind ``dg_ep_plan`` /
``dg_ep_push`` / ``dg_ep_barrier`` write each routed row straight into the owning rank's
grouped, padded activation buffer; the second GEMM's epilogue writes every result row straight
back into the buffer of the rank the token came from (``scatter_tag`` of ``dg_contig_gemm``), so
the return transfer overlaps the GEMM tile by tile and the final weighted sum is a local read.
A layer is eight launches on one stream (the two barriers included) and never synchronises with
the host:

    plan (counts exchange) -> push (quantising each token on the way out) -> barrier ->
    gate/up GEMM -> SiLU*up + requantise -> down GEMM (scattering) -> barrier -> weighted top-k sum

With one rank the same code runs on plain tensors.  ``make_emulated_ranks`` plays several ranks
on one GPU for tests (every phase of all ranks is enqueued before the next phase).
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence, Tuple

import torch

from . import _cabi, _core
from ._core import _launch

__all__ = ["EPExchange", "make_emulated_ranks", "layout_from_counts"]


def _round_up(x: int, a: int) -> int:
    return (x + a - 1) // a * a


def layout_from_counts(counts: torch.Tensor, rank: int, align: int):
    """What ``dg_ep_plan`` derives from the full counts table, restated with torch ops (used by
    the tests as the expected value).  ``counts`` int [world, E].  Returns ``(my_base [E],
    m_indices of rank's receive buffer (unpadded tail not included), m_total)``."""
    world, e = counts.shape
    e_local = e // world
    c = counts.to(torch.int64)
    tot = c.sum(dim=0)
    padded = (tot + align - 1) // align * align
    before = c[:rank].sum(dim=0)
    start = torch.zeros(e, dtype=torch.int64)
    for r in range(world):
        seg = padded[r * e_local:(r + 1) * e_local]
        start[r * e_local:(r + 1) * e_local] = torch.cumsum(seg, 0) - seg
    my_base = (start + before).to(torch.int32)
    rows = []
    for el in range(e_local):
        g = rank * e_local + el
        rows.append(torch.full((int(tot[g]),), el, dtype=torch.int32))
        rows.append(torch.full((int(padded[g] - tot[g]),), -1, dtype=torch.int32))
    m_indices = torch.cat(rows) if rows else torch.zeros(0, dtype=torch.int32)
    return my_base, m_indices, int(padded[rank * e_local:(rank + 1) * e_local].sum())


class EPExchange:
    """Buffers, peer pointers and the layer driver of one rank.

    ``hidden`` / ``out_hidden``: row lengths going into the gate/up GEMM and coming out of the
    down GEMM; ``inter2`` = columns of the gate/up GEMM (gate | up).  ``m_cap``: rows of every
    rank's receive buffer (the same on all ranks); pairs that do not fit are dropped and
    reported through ``check_status``.  The exchange buffers and the GEMM intermediates are
    allocated here, once; ``forward`` allocates nothing (rows longer than 8192 elements take a
    separate quantisation step that allocates its outputs).
    """

    _ALIGN = 256

    @staticmethod
    def _sizes(world, num_experts, hidden, out_hidden, max_tokens, top_k, m_cap):
        return {"recv_a": m_cap * hidden, "recv_scale": m_cap * 4, "recv_tag": m_cap * 4,
                "counts": world * num_experts * 4, "flags": _cabi.EP_MAX_WORLD * 4,
                "y_back": max_tokens * top_k * out_hidden * 2}

    @classmethod
    def shared_size(cls, world, num_experts, hidden, out_hidden, max_tokens, top_k, m_cap) -> int:
        """Bytes of the buffer every rank maps."""
        sizes = cls._sizes(world, num_experts, hidden, out_hidden, max_tokens, top_k,
                           _round_up(m_cap, cls._ALIGN))
        return sum(_round_up(v, 256) for v in sizes.values())

    def __init__(self, rank: int, world: int, num_experts: int, hidden: int, inter2: int, out_hidden: int,
                 max_tokens: int, top_k: int, m_cap: int, device: torch.device, *, kind: str = "fp8",
                 group=None, _shared: Optional[Tuple[torch.Tensor, List[int]]] = None):
        if num_experts % world:
            raise ValueError("num_experts must be a multiple of the number of ranks")
        if world > _cabi.EP_MAX_WORLD:
            raise ValueError(f"at most {_cabi.EP_MAX_WORLD} ranks")
        if kind not in ("fp8", "int8"):
            raise ValueError("kind must be 'fp8' or 'int8'")
        self.rank, self.world, self.num_experts = rank, world, num_experts
        self.e_local = num_experts // world
        self.hidden, self.inter2, self.out_hidden = hidden, inter2, out_hidden
        self.max_tokens, self.top_k, self.kind = max_tokens, top_k, kind
        self.m_cap = _round_up(m_cap, self._ALIGN)
        self.device = device
        self.epoch = 0
        self._comm = None                              # second stream of a sliced push
        self.default_slices = 4 if world >= 8 else 1
        self.overlap_push_blocks = torch.cuda.get_device_properties(device).multi_processor_count
        # ^ grid of a push that runs beside a GEMM: one block per SM fits next to a GEMM CTA
        # ---- the one buffer every rank maps: receive side of the dispatch and of the return
        sizes = self._sizes(world, num_experts, hidden, out_hidden, max_tokens, top_k, self.m_cap)
        self._off, total = {}, 0
        for name, nbytes in sizes.items():
            self._off[name] = total
            total += _round_up(nbytes, 256)
        self.shared_bytes = total
        if _shared is not None:                       # emulated ranks / one rank: plain tensors
            self._buf, bases = _shared
        elif world == 1:
            self._buf = torch.zeros(total, dtype=torch.uint8, device=device)
            bases = [self._buf.data_ptr()]
        else:
            import os
            # peer loads and stores only: do not bind the buffer to an NVLink multicast object
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
            import torch.distributed as dist
            import torch.distributed._symmetric_memory as symm
            grp = group if group is not None else dist.group.WORLD
            self._buf = symm.empty(total, dtype=torch.uint8, device=device)
            self._buf.zero_()
            self._hdl = symm.rendezvous(self._buf, grp.group_name)
            bases = [int(p) for p in self._hdl.buffer_ptrs]
            torch.cuda.synchronize(device)
            dist.barrier(group=grp)                    # every rank's flags are zero before first use
        self._bases = bases
        self._peer = {name: _cabi.pointer_array([b + off for b in bases]) for name, off in self._off.items()}

        def view(name, dtype, shape):
            n = sizes[name]
            return self._buf[self._off[name]:self._off[name] + n].view(dtype).view(shape)
        qdtype = torch.float8_e4m3fn if kind == "fp8" else torch.int8
        self.recv_a = view("recv_a", qdtype, (self.m_cap, hidden))
        self.recv_scale = view("recv_scale", torch.float32, (self.m_cap,))
        self.recv_tag = view("recv_tag", torch.int32, (self.m_cap,))
        self.counts = view("counts", torch.int32, (world, num_experts))
        self.y_back = view("y_back", torch.bfloat16, (max_tokens * top_k, out_hidden))
        # ---- this rank's own working set
        i32 = dict(dtype=torch.int32, device=device)
        self.my_base = torch.zeros(num_experts, **i32)
        self.cursor = torch.zeros(num_experts, **i32)
        self.m_indices = torch.full((self.m_cap,), -1, **i32)
        self.m_total = torch.zeros(1, **i32)
        self.status = torch.zeros(_cabi.STATUS_WORDS, **i32)
        self.pair_dest = torch.zeros(max_tokens * top_k, **i32)
        self.pair_index = torch.arange(max_tokens * top_k, **i32)
        self.h13 = torch.empty((self.m_cap, inter2), dtype=torch.bfloat16, device=device)
        self.act_q = torch.empty((self.m_cap, inter2 // 2), dtype=qdtype, device=device)
        self.act_scale = torch.empty((self.m_cap,), dtype=torch.float32, device=device)

    # ------------------------------------------------------------------ the steps
    def plan(self, topk_ids: torch.Tensor, phases: int = 0) -> None:
        """Counts exchange + layout (``dg_ep_plan``).  ``topk_ids`` int32 [T, top_k]."""
        if phases in (0, _cabi.EP_PHASE_POST):
            self.epoch += 1
        args = _cabi.EpPlanArgs(
            world=self.world, rank=self.rank, num_experts=self.num_experts, num_pairs=topk_ids.numel(),
            align=self._ALIGN, m_cap=self.m_cap, epoch=self.epoch, phases=phases,
            topk_ids=topk_ids.data_ptr(), peer_counts=self._peer["counts"], peer_flags=self._peer["flags"],
            my_base=self.my_base.data_ptr(), cursor=self.cursor.data_ptr(),
            m_indices=self.m_indices.data_ptr(), m_total=self.m_total.data_ptr(),
            status=self.status.data_ptr())
        _launch(_cabi.lib.dg_ep_plan, args, self.device, "dg_ep_plan")

    def push(self, q: torch.Tensor, q_scale: Optional[torch.Tensor], topk_ids: torch.Tensor,
             experts: Optional[Tuple[int, int]] = None, max_blocks: int = 0) -> None:
        """Writes every routed row into its owner's receive buffer (``dg_ep_push``).  ``q`` holds the
        quantised rows and ``q_scale`` their scales, or ``q`` holds the bf16 rows and ``q_scale`` is
        None: the kernel then quantises each token on the way out.  ``experts`` = (lo, hi): only
        the pairs whose expert is number lo .. hi - 1 among its owner's experts.  ``max_blocks``
        bounds the grid (0 = eight blocks per SM) for a push that shares the GPU with a GEMM."""
        t, k = topk_ids.shape
        lo, hi = experts if experts is not None else (0, 0)
        if q_scale is None:
            if q.dtype != torch.bfloat16 or not q.is_contiguous() or q.shape[1] != self.hidden:
                raise ValueError("rows to quantise must be a contiguous bf16 [T, hidden] tensor")
            quantise = _cabi.EP_QUANT_E4M3 if self.kind == "fp8" else _cabi.EP_QUANT_I8
        else:
            quantise = _cabi.EP_QUANT_NONE
        args = _cabi.EpPushArgs(
            world=self.world, rank=self.rank, num_experts=self.num_experts, num_tokens=t, top_k=k,
            row_bytes=self.hidden, m_cap=self.m_cap, quantise=quantise, rows=q.data_ptr(),
            row_scale=q_scale.data_ptr() if q_scale is not None else None,
            topk_ids=topk_ids.data_ptr(), my_base=self.my_base.data_ptr(),
            cursor=self.cursor.data_ptr(), peer_a=self._peer["recv_a"], peer_scale=self._peer["recv_scale"],
            peer_tag=self._peer["recv_tag"], pair_dest=self.pair_dest.data_ptr(),
            status=self.status.data_ptr(), local_lo=lo, local_hi=hi, max_blocks=max_blocks)
        _launch(_cabi.lib.dg_ep_push, args, self.device, "dg_ep_push")

    def barrier(self, phases: int = 0) -> None:
        if phases in (0, _cabi.EP_PHASE_POST):
            self.epoch += 1
        args = _cabi.EpBarrierArgs(world=self.world, rank=self.rank, epoch=self.epoch, phases=phases,
                                   peer_flags=self._peer["flags"], status=self.status.data_ptr())
        _launch(_cabi.lib.dg_ep_barrier, args, self.device, "dg_ep_barrier")

    def gate_up(self, w13, experts: Optional[Tuple[int, int]] = None) -> None:
        """The gate/up GEMM over the received rows; ``experts`` = (lo, hi) restricts it to the rows
        of this rank's experts lo .. hi - 1 (the other rows of ``h13`` are left alone)."""
        kind = _cabi.KIND_E4M3 if self.kind == "fp8" else _cabi.KIND_I8
        if experts is None:
            _core.grouped_gemm_contiguous(kind, _cabi.SCALE_PER_CHANNEL, self.recv_a, w13[0], self.h13,
                                          self.recv_scale, w13[1], self.m_indices)
        else:
            lo, hi = experts
            _core.grouped_gemm_contiguous(kind, _cabi.SCALE_PER_CHANNEL, self.recv_a, w13[0][lo:hi], self.h13,
                                          self.recv_scale, w13[1][lo:hi], self.m_indices, group_window=lo)

    def experts(self, w13, w2, gate_up_done: bool = False) -> None:
        """gate/up GEMM -> SiLU*up + requantise -> down GEMM whose result rows go home."""
        from .moe_chain import silu_mul_quant
        kind = _cabi.KIND_E4M3 if self.kind == "fp8" else _cabi.KIND_I8
        if not gate_up_done:
            self.gate_up(w13)
        silu_mul_quant(self.h13, kind=self.kind, m_indices=self.m_indices, out=(self.act_q, self.act_scale))
        # the scattering GEMM never writes `d`; it only has to be a valid bf16 tensor
        _core.grouped_gemm_contiguous(kind, _cabi.SCALE_PER_CHANNEL, self.act_q, w2[0], self.y_back,
                                      self.act_scale, w2[1], self.m_indices,
                                      scatter=(self.recv_tag, self._peer["y_back"], self.world))

    def combine(self, topk_weights: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        from .moe_chain import combine_rows
        t, k = topk_weights.shape
        return combine_rows(self.y_back[:t * k], self.pair_index[:t * k].view(t, k), topk_weights, out=out)

    def quantise(self, hidden: torch.Tensor):
        from .quant_group import quantize_rows
        return quantize_rows(hidden, kind=self.kind)

    def slices(self, n: int) -> List[Tuple[int, int]]:
        """This rank's experts cut into ``n`` runs of (almost) equal length."""
        n = max(1, min(int(n), self.e_local))
        cuts = [self.e_local * i // n for i in range(n + 1)]
        return [(cuts[i], cuts[i + 1]) for i in range(n)]

    def forward(self, hidden: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor, w13, w2,
                out: Optional[torch.Tensor] = None, *, slices: Optional[int] = None) -> torch.Tensor:
        """One layer for this rank's tokens: hidden bf16 [T, hidden], topk_ids int32 [T, top_k],
        topk_weights fp32 [T, top_k]; ``w13`` / ``w2`` = (packed weight, scale) of this rank's
        experts.  Returns bf16 [T, out_hidden].  Enqueues only; call ``check_status`` after a
        synchronisation to learn of dropped pairs or a peer that never arrived.

        ``slices`` > 1 (the same on every rank): the rows are pushed in that many slices of every
        owner's experts on a second stream, and the gate/up GEMM of a slice starts as soon as that
        slice has arrived everywhere, while the next slice is still crossing NVLink.  The result
        is the same bit for bit.  None picks ``default_slices``: 4 from eight ranks upwards (where
        seven eighths of the rows cross NVLink and slicing measured 4 % faster, twice), else 1
        (at two and four ranks it measured within noise of the unsliced layer)."""
        if slices is None:
            slices = self.default_slices
        if topk_ids.dtype != torch.int32 or not topk_ids.is_contiguous():
            raise ValueError("topk_ids must be contiguous int32 [T, top_k]")
        if topk_ids.shape[0] > self.max_tokens or topk_ids.shape[1] != self.top_k:
            raise ValueError("more tokens than the exchange was sized for, or another top_k")
        if self.hidden > 8192:
            rows, row_scale = self.quantise(hidden)
        else:
            rows, row_scale = hidden, None              # quantised on the way out
        self.plan(topk_ids)
        parts = self.slices(slices)
        if len(parts) == 1:
            self.push(rows, row_scale, topk_ids)
            self.barrier()
            self.experts(w13, w2)
        else:
            main = torch.cuda.current_stream(self.device)
            if self._comm is None:
                self._comm = torch.cuda.Stream(self.device)
                self._arrived = [torch.cuda.Event() for _ in range(self.e_local)]
            self._comm.wait_stream(main)
            with torch.cuda.stream(self._comm):
                for i, part in enumerate(parts):
                    # slices after the first run beside a GEMM: one block per SM fits next to its CTA
                    self.push(rows, row_scale, topk_ids, experts=part, max_blocks=self.overlap_push_blocks if i else 0)
                    self.barrier()
                    self._arrived[i].record(self._comm)
            for i, part in enumerate(parts):
                main.wait_event(self._arrived[i])
                self.gate_up(w13, part)
            self.experts(w13, w2, gate_up_done=True)
        self.barrier()
        return self.combine(topk_weights.to(torch.float32), out=out)

    def check_status(self) -> None:
        """Reads the device status words (synchronises the device) and raises on a problem."""
        st = self.status.tolist()
        if st[0] == 1:
            raise RuntimeError(f"expert-parallel exchange: rank {st[1]} gave up waiting for peer "
                               f"{st[2] - 100} at epoch {st[3]}")
        if st[0] != 0:
            raise RuntimeError("expert-parallel exchange: routed rows did not fit the receive buffer "
                               f"(m_cap = {self.m_cap}) and were dropped")


def make_emulated_ranks(world: int, num_experts: int, hidden: int, inter2: int, out_hidden: int,
                        max_tokens: int, top_k: int, m_cap: int, device: torch.device, *,
                        kind: str = "fp8") -> List[EPExchange]:
    """``world`` ranks on one GPU, each with its own buffers and everyone's pointers (tests)."""
    nbytes = EPExchange.shared_size(world, num_experts, hidden, out_hidden, max_tokens, top_k, m_cap)
    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device=device) for _ in range(world)]
    bases = [b.data_ptr() for b in bufs]
    return [EPExchange(r, world, num_experts, hidden, inter2, out_hidden, max_tokens, top_k, m_cap, device,
                       kind=kind, _shared=(bufs[r], bases)) for r in range(world)]


def emulated_forward(ranks: Sequence[EPExchange], hidden: Sequence[torch.Tensor],
                     topk_ids: Sequence[torch.Tensor], topk_weights: Sequence[torch.Tensor],
                     w13: Sequence, w2: Sequence, slices: int = 1) -> List[torch.Tensor]:
    """One layer of every emulated rank, phase by phase (the posting half of each barrier for all
    ranks before any waiting half); with ``slices`` > 1 the push and the gate/up GEMM run slice
    by slice as in ``EPExchange.forward`` (on one stream)."""
    for r, ids in zip(ranks, topk_ids):
        r.plan(ids, _cabi.EP_PHASE_POST)
    for r, ids in zip(ranks, topk_ids):
        r.plan(ids, _cabi.EP_PHASE_WAIT)
    parts = ranks[0].slices(slices)
    for part in parts:
        only = part if len(parts) > 1 else None
        for i, (r, h, ids) in enumerate(zip(ranks, hidden, topk_ids)):
            if i % 2 == 0 and r.hidden <= 8192:
                r.push(h, None, ids, experts=only)            # quantised on the way out
            else:
                r.push(*r.quantise(h), ids, experts=only)     # quantised first: the same bytes
        for ph in (_cabi.EP_PHASE_POST, _cabi.EP_PHASE_WAIT):
            for r in ranks:
                r.barrier(ph)
        if only is not None:
            for r, a in zip(ranks, w13):
                r.gate_up(a, only)
    for r, a, b in zip(ranks, w13, w2):
        r.experts(a, b, gate_up_done=len(parts) > 1)
    for ph in (_cabi.EP_PHASE_POST, _cabi.EP_PHASE_WAIT):
        for r in ranks:
            r.barrier(ph)
    return [r.combine(w.to(torch.float32)) for r, w in zip(ranks, topk_weights)]
