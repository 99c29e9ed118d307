#!/usr/bin/env python
"""Benchmark of the grouped MoE GEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-extras]

A step is one pass of the hot path over one batch of synthetic input: one launch of the
masked FP8 low-latency decode GEMM of the headline configuration (32 local experts,
K=7168, N=4096, max_m=128, 256 tokens routed top-8; per-token x per-channel e4m3 scales).
The metric is achieved HBM bandwidth: algorithmic bytes (activations and outputs of valid
rows, weights of experts that have rows, scales, masked_m) per second.  With N > 1 every
rank holds its own 32 local experts and its own routed tokens (expert parallel, weak
scaling, no data-path collective inside the GEMM step); the expert-parallel prefill
configuration, whose dispatch is a real NCCL all-to-all, is measured after the timed region
and reported under "ep_prefill" with the all-to-all time kept separate from the GEMM time.

One JSON line is printed by rank 0.  `--impl reference` times the reference's CPU
implementation of the same path (its torch dequant-matmul, restated in oracle/dg_oracle.py)
on the host cores, on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(REPO, "deepgemm-das_b200"))

import torch  # noqa: E402

# dram__bytes_read.sum + dram__bytes_write.sum of one full-size decode launch (32 experts), from an
# ncu capture of this kernel; DRAM traffic grows in proportion to the number of experts.
NCU_DECODE_DRAM_BYTES_PER_EXPERT = 966.73e6 / 32
PREHEAT_S = 0.1
PREHEAT_MAX_S = 0.3   # long preheats push a power-capped GPU deeper into its cap
METRIC = "masked_fp8_decode_hbm_bandwidth"
UNIT = "GB/s"
C2 = dict(G=32, K=7168, N=4096, max_m=128, tokens=256, top_k=8)


def algorithmic_bytes(valid_rows, groups_with_rows, groups, n, k, a_bytes, b_bytes, tensor_wise=False,
                      index_entries=0):
    """Bytes a grouped GEMM must move at minimum: activations and outputs of valid rows, weights
    of groups that have rows, scales, and the masked_m / m_indices array."""
    v, gp = valid_rows, groups_with_rows
    return (v * k * a_bytes + gp * n * k * b_bytes + v * n * 2 + 4 * v +
            (4 * gp if tensor_wise else 4 * gp * n) + 4 * (index_entries or groups))


def _peaks():
    path = os.path.join(REPO, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            p = json.load(fh)
        return dict(hbm_gbs=float(p["hbm_gbs"]), bf16_tflops=float(p["bf16_tflops"]),
                    bf16_tflops_sustained=float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


# ----------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while a region runs."""
    _REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown",
                0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown",
                0x2: "applications_clocks_setting", 0x10: "sync_boost"}

    def __init__(self, index: int, period_s: float = 0.005):
        self.samples, self.period, self._stop, self._thread, self.h = [], period_s, False, None, None
        self.max_mhz = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.h = None
        self.power_limit_w = None
        try:
            self.power_limit_w = self.nv.nvmlDeviceGetEnforcedPowerLimit(self.h) / 1000.0
        except Exception:
            pass

    def _loop(self):
        nv = self.nv
        while not self._stop:
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                try:
                    rs = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    rs = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                try:
                    watts = nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0
                except Exception:
                    watts = None
                self.samples.append((time.perf_counter(), mhz, int(rs), watts))
            except Exception:
                pass
            time.sleep(self.period)

    def read_mhz(self):
        try:
            return self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM) if self.h is not None else None
        except Exception:
            return None

    def read_throttled(self) -> bool:
        """True when a power or thermal limit (not idleness) is holding the clock right now."""
        try:
            try:
                rs = self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
            except Exception:
                rs = self.nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
            return bool(int(rs) & (0x4 | 0x8 | 0x20 | 0x40 | 0x80))
        except Exception:
            return False

    def start(self):
        if self.h is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop = True
        if self._thread is not None:
            self._thread.join(timeout=1.0)

    def summary(self, t0: float, t1: float) -> dict:
        inside = [s for s in self.samples if t0 <= s[0] <= t1] or self.samples
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        mhz = sorted(s[1] for s in inside)
        bits = 0
        for s in inside:
            bits |= s[2]
        watts = sorted(s[3] for s in inside if s[3] is not None)
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": self.max_mhz,
                "reasons": sorted(n for b, n in self._REASONS.items() if bits & b),
                "samples": len(inside),
                "power_w": watts[len(watts) // 2] if watts else None,
                "power_limit_w": self.power_limit_w}


# ----------------------------------------------------------------------------- workloads
def make_decode_workload(device, seed: int, cfg=C2, tensor_wise: bool = False):
    """Headline decode workload, built on the device (torch ops are plumbing here)."""
    import deepgemm
    from deepgemm.quant_utils import per_token_quant_fp8
    G, K, N, max_m = cfg["G"], cfg["K"], cfg["N"], cfg["max_m"]
    cpu_gen = torch.Generator().manual_seed(seed)
    picks = torch.rand(cfg["tokens"], G, generator=cpu_gen).topk(cfg["top_k"], dim=1).indices
    masked_m = torch.bincount(picks.flatten(), minlength=G).clamp(max=max_m).to(torch.int32)
    gen = torch.Generator(device=device).manual_seed(seed)
    a, a_scale = per_token_quant_fp8(torch.randn(G, max_m, K, device=device, generator=gen))
    b = torch.empty(G, N, K, dtype=torch.float8_e4m3fn, device=device)
    b_scale = torch.empty(G, N, dtype=torch.float32, device=device)
    for g in range(G):
        q, s = per_token_quant_fp8(torch.randn(N, K, device=device, generator=gen))
        b[g], b_scale[g] = q, s.reshape(N)
    if tensor_wise:  # one scale per expert for the weights (per-token scales stay)
        b_scale = b_scale.mean(dim=1).contiguous()
    b_packed = deepgemm.marlin_fp8_masked_weight(b)
    d = torch.zeros(G, max_m, N, dtype=torch.bfloat16, device=device)
    return dict(a=a, a_scale=a_scale.reshape(G, max_m).contiguous(), b=b_packed, b_scale=b_scale,
                masked_m=masked_m.to(device), masked_m_cpu=masked_m, d=d, cfg=cfg,
                tensor_wise=tensor_wise)


def decode_bytes(w) -> float:
    cfg, mm = w["cfg"], w["masked_m_cpu"]
    return algorithmic_bytes(int(mm.sum()), int((mm > 0).sum()), cfg["G"], cfg["N"], cfg["K"], 1, 1,
                             tensor_wise=w["tensor_wise"])


def run_decode(w):
    import deepgemm
    fn = deepgemm.m_grouped_fp8_gemm_nt_masked_tensor_wise if w["tensor_wise"] \
        else deepgemm.m_grouped_fp8_gemm_nt_masked
    fn((w["a"], w["a_scale"]), (w["b"], w["b_scale"]), w["d"], w["masked_m"], int(w["cfg"]["max_m"]))


def time_launches(fn, steps: int, warmup: int, barrier=None):
    """CUDA-event time in ms of `steps` back-to-back calls on the current stream."""
    for _ in range(warmup):
        fn()
    if barrier:
        barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    if barrier:
        barrier()
    return e0.elapsed_time(e1), t0, t1


# ----------------------------------------------------------------------------- extra configurations
def make_contig_prefill(device, small=False, kind="int8"):
    """Contiguous INT8 / FP8 prefill: 32 experts, K=7168, N=4096, 4096 tokens top-8, groups padded
    to 256 (small: 8 experts, 1024 tokens).  Returns (launch function, info)."""
    import deepgemm
    from deepgemm.quant_utils import contiguous_layout, per_token_quant_fp8, per_token_quant_int8
    quant = per_token_quant_int8 if kind == "int8" else per_token_quant_fp8
    wdtype = torch.int8 if kind == "int8" else torch.float8_e4m3fn
    G, K, N, tokens = (8, 7168, 4096, 1024) if small else (32, 7168, 4096, 4096)
    cpu_gen = torch.Generator().manual_seed(3)
    picks = torch.rand(tokens, G, generator=cpu_gen).topk(8, dim=1).indices
    rows = torch.bincount(picks.flatten(), minlength=G)
    m_indices, _, m_total = contiguous_layout(rows.tolist(), 256, device)
    gen = torch.Generator(device=device).manual_seed(3)
    a, a_s = quant(torch.randn(m_total, K, device=device, generator=gen))
    b = torch.empty(G, N, K, dtype=wdtype, device=device)
    b_s = torch.empty(G, N, dtype=torch.float32, device=device)
    for g in range(G):
        q, s = quant(torch.randn(N, K, device=device, generator=gen))
        b[g], b_s[g] = q, s.reshape(N)
    out = torch.zeros(m_total, N, dtype=torch.bfloat16, device=device)
    a_s = a_s.reshape(m_total).contiguous()
    if kind == "int8":
        bp = deepgemm.marlin_i8_contiguous_weight(b)
        fn = lambda: deepgemm.m_grouped_i8_gemm_nt_contiguous((a, a_s), (bp, b_s), out, m_indices)
    else:
        bp = deepgemm.marlin_fp8_contiguous_weight(b)
        fn = lambda: deepgemm.m_grouped_fp8_gemm_nt_contiguous((a, a_s), (bp, b_s), out, m_indices)
    v = int(rows.sum())
    info = {"workload": "contiguous_%s_prefill G=%d K=%d N=%d V=%d M_total=%d" % (kind, G, K, N, v, m_total),
            "ops": 2.0 * v * N * K,
            "bytes": algorithmic_bytes(v, int((rows > 0).sum()), G, N, K, 1, 1, index_entries=m_total)}
    return fn, info


def measure_dense_8bit_peak(device, kind="int8", size=8192, reps=10):
    """Dense 8-bit tensor throughput of this GPU, measured with this library's own dense GEMM
    (dg_dense_gemm, two-CTA 256x256 tiles) at size^3, best of `reps` single launches: the
    denominator for the prefill fractions beside 2 x the measured bf16 cuBLAS figure (no 8-bit
    figure is measured by anyone else)."""
    from deepgemm.gemm import fp8_gemm
    dt = torch.int8 if kind == "int8" else torch.float8_e4m3fn
    if kind == "int8":
        a = torch.randint(-127, 128, (size, size), dtype=torch.int8, device=device)
        b = torch.randint(-127, 128, (size, size), dtype=torch.int8, device=device)
    else:
        a = torch.randn(size, size, device=device).to(dt)
        b = torch.randn(size, size, device=device).to(dt)
    ones = torch.ones(size, dtype=torch.float32, device=device)
    d = torch.empty(size, size, dtype=torch.bfloat16, device=device)
    for _ in range(3):
        fp8_gemm((a, ones), (b, ones), d)
    torch.cuda.synchronize()
    best = float("inf")
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fp8_gemm((a, ones), (b, ones), d)
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1))
    return 2.0 * size ** 3 / (best * 1e-3) / 1e12


def bench_contig_prefill(device, steps, warmup, peaks, kind="int8"):
    fn, info = make_contig_prefill(device, kind=kind)
    sampler = ClockSampler(device.index or 0, period_s=0.002)
    sampler.start()
    ms, t0, t1 = time_launches(fn, steps, warmup)
    sampler.stop()
    tops = info["ops"] * steps / (ms * 1e-3) / 1e12
    peak = 2.0 * peaks["bf16_tflops"]
    own = measure_dense_8bit_peak(device, kind)
    return {"workload": info["workload"], "ms": ms / steps, "tops": tops, "peak_tops": peak,
            "peak_note": "2 x %s dense bf16 cuBLAS burst TFLOP/s (8-bit tcgen05 rate is twice bf16; "
                         "no 8-bit peak is measured by the driver)" % peaks["source"],
            "frac_of_tensor_peak": tops / peak,
            "own_dense_8bit_tops": own, "own_dense_note": "this library's dense GEMM, 8192^3, best of 10 launches",
            "frac_of_own_dense_8bit": tops / own, "clocks": sampler.summary(t0, t1)}


def make_masked_w4a8(device, small=False, smem_unpack=False):
    """Masked W4A8 down projection: 32 experts, N=7168, K=2048, max_m=256, masked_m uniform in
    [0,256]; int4 source bytes low-nibble-first.  Returns (launch function, info).  With
    `smem_unpack` the launch goes to the kernel that unpacks into shared memory (block_n = 512)
    instead of the default one (unpacked weights through tensor memory)."""
    import deepgemm
    from deepgemm.quant_utils import pack_int4_pairs, per_channel_quant_int4, per_token_quant_int8
    G, N, K, max_m = 32, 7168, 2048, 256
    cpu_gen = torch.Generator().manual_seed(4)
    mm = torch.randint(0, max_m + 1, (G,), generator=cpu_gen).to(torch.int32)
    gen = torch.Generator(device=device).manual_seed(4)
    a, a_s = per_token_quant_int8(torch.randn(G, max_m, K, device=device, generator=gen))
    fw = torch.empty(G, N, K // 2, dtype=torch.int8, device=device)
    b_s = torch.empty(G, N, dtype=torch.float32, device=device)
    for g in range(G):
        q, s = per_channel_quant_int4(torch.randn(N, K, device=device, generator=gen))
        fw[g], b_s[g] = pack_int4_pairs(q, "low_first"), s.reshape(N) / 16.0
    bp = deepgemm.pack_w4a8_moe_hipc_weight(fw, nibble_order="low_first")
    d = torch.zeros(G, max_m, N, dtype=torch.bfloat16, device=device)
    a_s = a_s.reshape(G, max_m).contiguous()
    mmd = mm.to(device)
    if smem_unpack:
        from deepgemm import _cabi, _core
        fn = lambda: _core.grouped_gemm_masked(_cabi.KIND_W4A8, 0, a, bp, d, a_s, b_s, mmd, max_m, block_n=512)
    else:
        fn = lambda: deepgemm.m_grouped_w4a8_gemm_nt_masked((a, a_s), (bp, b_s), d, mmd, max_m)
    v = int(mm.sum())
    info = {"workload": "masked_w4a8 G=32 N=7168 K=2048 max_m=256 V=%d" % v,
            "ops": 2.0 * v * N * K, "bytes": algorithmic_bytes(v, int((mm > 0).sum()), G, N, K, 1, 0.5)}
    return fn, info


def bench_masked_w4a8(device, steps, warmup, peaks):
    fn, info = make_masked_w4a8(device)
    sampler = ClockSampler(device.index or 0, period_s=0.002)
    sampler.start()
    ms, t0, t1 = time_launches(fn, steps, warmup)
    sampler.stop()
    sec = ms * 1e-3 / steps
    res = {"workload": info["workload"], "ms": ms / steps, "gbs": info["bytes"] / sec / 1e9,
           "frac_of_hbm_peak": info["bytes"] / sec / 1e9 / peaks["hbm_gbs"],
           "tops": info["ops"] / sec / 1e12, "kernel": "grouped_gemm_w4_kernel (unpacked weights through TMEM)",
           "clocks": sampler.summary(t0, t1)}
    fn2, _ = make_masked_w4a8(device, smem_unpack=True)
    ms2, _, _ = time_launches(fn2, steps, warmup)
    res["smem_unpack_kernel_ms"] = ms2 / steps     # the other W4A8 kernel on the same inputs, same box
    return res


def profile_chain(device, steps, warmup):
    """Profiler driver for the memory-bound kernels around the GEMMs, on a small case (8192 rows of
    7168; a few hundred MB): quantise + group, SiLU*up + requantise, weighted top-k sum, and the
    expert-parallel push with one rank."""
    import deepgemm
    from deepgemm import ep_exchange as epx
    from deepgemm.moe_chain import combine_rows, silu_mul_quant
    rows, hidden, experts, top_k = 8192, 7168, 32, 8
    gen = torch.Generator(device=device).manual_seed(9)
    x = torch.randn(rows, hidden, device=device, generator=gen).bfloat16()
    expert = torch.randint(0, experts, (rows,), device=device, generator=gen, dtype=torch.int32)
    h13 = torch.randn(rows, 4096, device=device, generator=gen).bfloat16()
    m_idx = torch.zeros(rows, dtype=torch.int32, device=device)
    tokens = rows // top_k
    y = torch.randn(rows, hidden, device=device, generator=gen).bfloat16()
    src = torch.arange(rows, dtype=torch.int32, device=device).view(tokens, top_k)
    w = torch.softmax(torch.randn(tokens, top_k, device=device, generator=gen), dim=1)
    ex = epx.EPExchange(0, 1, experts, hidden, 4096, hidden, tokens, top_k, 2 * rows, device)
    ids = torch.rand(tokens, experts, device=device, generator=gen).topk(top_k, dim=1).indices.to(torch.int32)
    q, qs = ex.quantise(x[:tokens].contiguous())
    ex.plan(ids)

    def step():
        deepgemm.quantize_group_rows(x, expert, experts)
        silu_mul_quant(h13, kind="fp8", m_indices=m_idx)
        combine_rows(y, src, w)
        ex.plan(ids)
        ex.push(q, qs, ids)
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    for _ in range(steps):
        step()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    print(json.dumps({"profile_run": True, "workload": "chain kernels rows=%d hidden=%d" % (rows, hidden),
                      "steps": steps}))


EP = dict(experts=256, K=7168, N=4096, tokens=4096, top_k=8)


def _ep_expert_weights(e, device, cfg=EP):
    """Weights of global expert e, a function of e alone, so that any rank can rebuild any expert
    for the parity check: (gate|up e4m3 [N, K], scale [N], down e4m3 [K, N/2], scale [K])."""
    from deepgemm.quant_utils import per_token_quant_fp8
    g = torch.Generator(device=device).manual_seed(1000 + e)
    w13, s13 = per_token_quant_fp8(torch.randn(cfg["N"], cfg["K"], device=device, generator=g) * 0.02)
    w2, s2 = per_token_quant_fp8(torch.randn(cfg["K"], cfg["N"] // 2, device=device, generator=g) * 0.02)
    return w13, s13.reshape(-1), w2, s2.reshape(-1)


def _ep_tokens(rank, device, cfg=EP):
    gen = torch.Generator(device=device).manual_seed(100 + rank)
    shared = torch.Generator().manual_seed(7)                     # same expert bias on every rank
    bias = (torch.randn(cfg["experts"], generator=shared) * 0.5).to(device)
    hidden = torch.randn(cfg["tokens"], cfg["K"], device=device, generator=gen).to(torch.bfloat16)
    logits = torch.randn(cfg["tokens"], cfg["experts"], device=device, generator=gen) + bias
    topk = logits.topk(cfg["top_k"], dim=1).indices.to(torch.int32).contiguous()
    weights = torch.softmax(torch.randn(cfg["tokens"], cfg["top_k"], device=device, generator=gen), dim=1)
    return hidden, topk, weights


def _ep_parity(out, hidden, topk, weights, device, cfg=EP, sample=6):
    """On-box check of the layer's result for a sample of this rank's tokens: (a) against the
    oracle's formulas (torch fp32 dequant-matmul, calc_diff < 1e-3), (b) bit for bit against the
    one-GPU layer of this library run on the same tokens with the experts they use."""
    sys.path.insert(0, os.path.join(REPO, "oracle"))
    import dg_oracle as O
    import deepgemm
    from deepgemm.moe_chain import moe_forward
    idx = torch.linspace(0, cfg["tokens"] - 1, sample).long().to(device)
    ids = topk[idx].long()
    used = ids.flatten().unique()
    remap = torch.full((cfg["experts"],), -1, dtype=torch.long, device=device)
    remap[used] = torch.arange(used.numel(), device=device)
    ws = [_ep_expert_weights(int(e), device, cfg) for e in used.tolist()]
    w13 = torch.stack([w[0] for w in ws]); s13 = torch.stack([w[1] for w in ws])
    w2 = torch.stack([w[2] for w in ws]); s2 = torch.stack([w[3] for w in ws])
    local_ids = remap[ids].to(torch.int32).contiguous()
    pk = deepgemm.marlin_fp8_contiguous_weight
    one_gpu = moe_forward(hidden[idx].contiguous(), local_ids, weights[idx].contiguous(),
                          (pk(w13.clone()), s13), (pk(w2.clone()), s2))
    got = out[idx]
    bit_equal = bool(torch.equal(got.view(torch.int16), one_gpu.view(torch.int16)))
    ref = O.ref_moe_layer(hidden[idx].cpu(), local_ids.cpu().long(), weights[idx].cpu(), w13.cpu(), s13.cpu(),
                          w2.cpu(), s2.cpu())
    diff = float(O.calc_diff(got.cpu().double(), ref.double()))
    return {"sample_tokens": sample, "calc_diff_vs_oracle": diff, "bit_equal_one_gpu_layer": bit_equal,
            "ok": bool(bit_equal and diff < 1e-3)}


def bench_ep_prefill(device, rank, world, steps, warmup, peaks, cfg=EP):
    """Expert-parallel FP8 MoE layer: 256 experts sharded over the ranks, 4096 tokens per rank routed
    top-8 (mildly skewed).  Reports the contiguous FP8 gate/up GEMM and the NCCL all-to-all dispatch
    separately (max over ranks), then the whole layer through the peer-memory exchange
    (deepgemm.ep_exchange) as one timed step with its phases, and a parity flag computed here."""
    import deepgemm
    from deepgemm import _cabi, ep_exchange as epx, expert_parallel as ep
    dist = None
    if world > 1:
        import torch.distributed as dist
    E, K, N, T, top_k = cfg["experts"], cfg["K"], cfg["N"], cfg["tokens"], cfg["top_k"]
    e_local, inter = E // world, N // 2
    hidden, topk, weights = _ep_tokens(rank, device, cfg)
    w13 = torch.empty(e_local, N, K, dtype=torch.float8_e4m3fn, device=device)
    s13 = torch.empty(e_local, N, dtype=torch.float32, device=device)
    w2 = torch.empty(e_local, K, inter, dtype=torch.float8_e4m3fn, device=device)
    s2 = torch.empty(e_local, K, dtype=torch.float32, device=device)
    for el in range(e_local):
        w13[el], s13[el], w2[el], s2[el] = _ep_expert_weights(rank * e_local + el, device, cfg)
    w13p = (deepgemm.marlin_fp8_contiguous_weight(w13), s13)
    w2p = (deepgemm.marlin_fp8_contiguous_weight(w2), s2)
    m_cap = 2 * T * top_k + e_local * 256
    x = epx.EPExchange(rank, world, E, K, N, K, T, top_k, m_cap, device)

    def ev():
        return torch.cuda.Event(enable_timing=True)

    def sync():
        if dist:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n=steps, w=warmup):
        for _ in range(w):
            fn()
        sync()
        e0, e1 = ev(), ev()
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        sync()
        return e0.elapsed_time(e1) / n

    # ---- the whole layer, one timed step (every launch of forward() between the two events)
    # with the push in 1, 2 and 4 slices (the later slices cross NVLink under the gate/up GEMM of the
    # earlier ones); every variant is checked; the layer figure is the one forward() takes by
    # default (EPExchange.default_slices: 4 from eight ranks upwards, else 1)
    out = torch.empty(T, K, dtype=torch.bfloat16, device=device)
    by_slices, parity = {}, None
    for n_slices in ((1, 2, 4) if world > 1 else (1,)):
        out.zero_()
        by_slices[n_slices] = timed(lambda: x.forward(hidden, topk, weights, w13p, w2p, out=out, slices=n_slices))
        x.check_status()
        p_n = _ep_parity(out, hidden, topk, weights, device, cfg)
        if parity is None or not p_n["ok"]:
            parity = p_n
    sl = torch.tensor([by_slices.get(n, 0.0) for n in (1, 2, 4)], device=device, dtype=torch.float64)
    if dist:
        dist.all_reduce(sl, op=dist.ReduceOp.MAX)
    by_slices = {n: float(v) for n, v in zip((1, 2, 4), sl.tolist()) if v > 0.0}
    layer_ms = by_slices[x.default_slices]

    # ---- its phases, each timed on its own (a barrier closes every phase that writes to peers)
    quant_ms = 0.0            # fused into the push
    plan_ms = timed(lambda: x.plan(topk))

    def push():
        x.plan(topk)          # hands out the rows again
        x.push(hidden, None, topk)
        x.barrier()
    push_ms = timed(push) - plan_ms
    kind = _cabi.KIND_E4M3
    from deepgemm import _core
    from deepgemm.moe_chain import silu_mul_quant
    g13 = lambda: _core.grouped_gemm_contiguous(kind, 0, x.recv_a, w13p[0], x.h13, x.recv_scale, w13p[1], x.m_indices)
    gemm_ms = timed(g13)
    act_ms = timed(lambda: silu_mul_quant(x.h13, kind="fp8", m_indices=x.m_indices, out=(x.act_q, x.act_scale)))

    def down_scatter():
        _core.grouped_gemm_contiguous(kind, 0, x.act_q, w2p[0], x.y_back, x.act_scale, w2p[1], x.m_indices,
                                      scatter=(x.recv_tag, x._peer["y_back"], world))
        x.barrier()
    down_ms = timed(down_scatter)
    y_local = torch.empty((x.m_cap, K), dtype=torch.bfloat16, device=device)
    down_local_ms = timed(lambda: _core.grouped_gemm_contiguous(kind, 0, x.act_q, w2p[0], y_local, x.act_scale,
                                                                w2p[1], x.m_indices))
    del y_local
    combine_ms = timed(lambda: x.combine(weights, out=out))
    x.check_status()

    # ---- the NCCL all-to-all dispatch of the bf16 rows, as the configuration words it
    plan = ep.build_dispatch_plan(topk.long(), E, world)
    a2a_ms = timed(lambda: ep.dispatch_tokens(hidden, plan, E, rank, world)) if world > 1 else 0.0

    valid = int((x.m_indices >= 0).sum())
    m_total = int(x.m_total)
    remote_pairs = int((torch.div(topk.long(), e_local, rounding_mode="floor") != rank).sum())
    vals = torch.tensor([layer_ms, quant_ms, plan_ms, push_ms, gemm_ms, act_ms, down_ms, down_local_ms,
                         combine_ms, a2a_ms], device=device, dtype=torch.float64)
    sums = torch.tensor([2.0 * valid * N * K, 2.0 * valid * K * inter, 1.0 if parity["ok"] else 0.0],
                        device=device, dtype=torch.float64)
    mx = torch.tensor([float(remote_pairs)], device=device, dtype=torch.float64)
    if dist:
        dist.all_reduce(vals, op=dist.ReduceOp.MAX)
        dist.all_reduce(sums, op=dist.ReduceOp.SUM)
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
    (layer_ms, quant_ms, plan_ms, push_ms, gemm_ms, act_ms, down_ms, down_local_ms, combine_ms,
     a2a_ms) = (float(v) for v in vals.tolist())
    flops13, flops2, ok_ranks = (float(v) for v in sums.tolist())
    tflops = flops13 / (gemm_ms * 1e-3) / 1e12
    res = {"workload": "ep_fp8_moe_layer experts=%d K=%d N=%d tokens/rank=%d top%d" % (E, K, N, T, top_k),
           "world": world, "all figures": "max over ranks, CUDA events",
           "gemm_ms_max_over_ranks": gemm_ms, "gemm_tflops_aggregate": tflops,
           "gemm_tflops_per_gpu": tflops / world,
           "all_to_all_ms_max_over_ranks": a2a_ms,
           "all_to_all_note": "NCCL all_to_all_single of the routed bf16 rows (counts first), as the "
                              "configuration states; the layer below does not use it",
           "valid_rows_this_rank": valid, "m_total_this_rank": m_total,
           "parity": "ok" if ok_ranks == world else "FAILED", "parity_rank0": parity,
           "layer_ms": layer_ms, "layer_push_slices": x.default_slices,
           "layer_ms_by_push_slices": {str(n): v for n, v in by_slices.items()},
           "layer": {"exchange": "peer-memory stores (dg_ep_plan / dg_ep_push with the per-token quantisation "
                                 "fused in / dg_ep_barrier), result rows scattered home by the down GEMM's "
                                 "epilogue; no host synchronisation",
                     "plan_counts_exchange_ms": plan_ms,
                     "quantise_push_rows_and_barrier_ms": push_ms,
                     "push_remote_gbs_max_rank": float(mx) * (K + 8) / (push_ms * 1e-3) / 1e9 if world > 1 else None,
                     "gate_up_gemm_ms": gemm_ms, "silu_mul_quant_ms": act_ms,
                     "down_gemm_scatter_and_barrier_ms": down_ms, "down_gemm_local_store_ms": down_local_ms,
                     "down_gemm_tflops_aggregate": flops2 / (down_ms * 1e-3) / 1e12,
                     "return_remote_gbs_max_rank": float(mx) * K * 2 / (down_ms * 1e-3) / 1e9 if world > 1 else None,
                     "combine_ms": combine_ms,
                     "exposed_exchange_ms": plan_ms + push_ms + max(0.0, down_ms - down_local_ms),
                     "gemm_ms_sum": gemm_ms + down_local_ms,
                     "layer_over_gemms": layer_ms / (gemm_ms + down_local_ms)}}
    if peaks:
        weight_bytes = e_local * N * K
        t_hbm = (weight_bytes + valid * K + valid * N * 2) / (peaks["hbm_gbs"] * 1e9)
        t_tc = 2.0 * valid * N * K / (2.0 * peaks["bf16_tflops"] * 1e12)
        res["gemm_roofline_ms"] = max(t_hbm, t_tc) * 1e3
        res["gemm_bound"] = "hbm" if t_hbm > t_tc else "tensor"
        res["gemm_frac_of_roofline"] = max(t_hbm, t_tc) * 1e3 / gemm_ms
    return res


def _sorted_routing(topk_ids, experts, block_m):
    """A routing list as vLLM's moe_align_block_size produces it (torch ops, plumbing): pairs
    sorted by expert, every expert's run padded to a multiple of block_m with an id no row has;
    entry = slot << 24 | token.  Returns (sorted_token_ids, expert_ids, num_tokens_post_pad)."""
    t, k = topk_ids.shape
    dev = topk_ids.device
    flat = topk_ids.flatten().long()
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=experts)
    padded = (counts + block_m - 1) // block_m * block_m
    starts = torch.cumsum(padded, 0) - padded
    total = int(padded.sum())
    ids = torch.full((total,), (k << 24), dtype=torch.int64, device=dev)       # slot = top_k: padding
    rank_in_expert = torch.arange(flat.numel(), device=dev) - (torch.cumsum(counts, 0) - counts)[flat[order]]
    ids[starts[flat[order]] + rank_in_expert] = ((order % k) << 24) | (order // k)
    expert_ids = torch.repeat_interleave(torch.arange(experts, device=dev), padded // block_m)
    return ids.to(torch.int32), expert_ids.to(torch.int32), torch.tensor([total], dtype=torch.int32, device=dev)


def make_prefill_down(device, small=False, path=None):
    """Second-stage op on a routing list (moe_w8a8_marlin_prefill_down_fp8): FP8, N=7168, K=2048,
    4096 tokens top-8 over 256 experts (small: 512 tokens, 32 experts), blocks of 32 entries.
    `path` pins the implementation ("gather": the one-launch GEMM that fetches the rows by index;
    "regroup": regroup step + contiguous GEMM); None lets the op choose."""
    import deepgemm
    from deepgemm import moe_marlin_prefill as M
    t, e = (512, 32) if small else (4096, 256)
    k, n, hid, block_m = 8, 7168, 2048, 32
    gen = torch.Generator(device=device).manual_seed(12)
    topk_ids = torch.rand(t, e, device=device, generator=gen).topk(k, dim=1).indices
    inp = (torch.randn(t * k, hid, device=device, generator=gen) * 0.5).to(torch.float8_e4m3fn)
    w = deepgemm.marlin_fp8_contiguous_weight(
        (torch.randn(e, n, hid, device=device, generator=gen) * 0.05).to(torch.float8_e4m3fn))
    a_s = torch.rand(t * k, device=device, generator=gen) * 0.02 + 0.01
    b_s = torch.rand(e, n, device=device, generator=gen) * 0.02 + 0.01
    tw = torch.softmax(torch.randn(t, k, device=device, generator=gen), dim=1)
    ids, experts, used = _sorted_routing(topk_ids, e, block_m)
    out = torch.zeros(t * k, n, dtype=torch.bfloat16, device=device)

    def fn():
        M.FORCE_PATH = path
        try:
            deepgemm.moe_w8a8_marlin_prefill_down_fp8(inp, w, out, a_s, b_s, tw, ids, experts, used, k, k)
        finally:
            M.FORCE_PATH = None
    info = {"workload": "prefill_down_fp8 tokens=%d top%d experts=%d N=%d K=%d" % (t, k, e, n, hid),
            "ops": 2.0 * t * k * n * hid, "bytes": algorithmic_bytes(t * k, e, e, n, hid, 1, 1)}
    return fn, info


def bench_prefill_down(device, steps, warmup):
    res = None
    for path in ("gather", "regroup"):
        fn, info = make_prefill_down(device, path=path)
        ms, _, _ = time_launches(fn, steps, warmup)
        if res is None:
            res = {"workload": info["workload"]}
        res["ms_" + ("one_launch_gathering_gemm" if path == "gather" else "regroup_then_gemm")] = ms / steps
        del fn
        torch.cuda.empty_cache()
    res["tflops_one_launch"] = info["ops"] / (res["ms_one_launch_gathering_gemm"] * 1e-3) / 1e12
    return res


def bench_masked_bf16(device, steps, warmup, peaks, active_m=112):
    """Masked BF16 at the shape the reference benchmarks (16 experts, M = 2048, N = 2048, K = 6144,
    op_test/test_deepgemm_masked_w16a16_bf16.py:11-20) with `active_m` rows in every expert: weight
    streaming, so the figure is GB/s of the reference's own byte count against the copy rate."""
    import deepgemm
    E, M, N, K = 16, 2048, 2048, 6144
    gen = torch.Generator(device=device).manual_seed(5)
    a = (torch.randn(E, M, K, device=device, generator=gen) * 0.1).bfloat16()
    packed, cfg = deepgemm.pack_bf16_masked_weight((torch.randn(E, N, K, device=device, generator=gen) * 0.1).bfloat16())
    mm = torch.full((E,), active_m, dtype=torch.int32, device=device)
    d = torch.zeros(E, M, N, dtype=torch.bfloat16, device=device)
    ms, _, _ = time_launches(lambda: deepgemm.m_grouped_bf16_gemm_nt_masked(a, packed, d, mm, active_m, cfg),
                             steps, warmup)
    nbytes = E * (active_m * K + N * K + active_m * N) * 2
    gbs = nbytes / (ms * 1e-3 / steps) / 1e9
    return {"workload": "masked_bf16 E=16 max_m=2048 N=2048 K=6144 masked_m=%d" % active_m, "ms": ms / steps,
            "gbs": gbs, "frac_of_hbm_peak": gbs / peaks["hbm_gbs"],
            "tflops": 2.0 * E * active_m * N * K / (ms * 1e-3 / steps) / 1e12,
            "l2": "0.4 GB of weights, larger than the 126 MB L2"}


def bench_host_path(device, cfg, calls=4000):
    """Host time per call of the public Python entry point (decode shape, no routed rows, so the
    kernel is an empty launch and the host is what is timed), with no CUDA graph: wall clock over
    back-to-back asynchronous calls."""
    import deepgemm
    from deepgemm import _core
    G, max_m, N, K = cfg["G"], cfg["max_m"], cfg["N"], cfg["K"]
    a = torch.zeros(G, max_m, K, device=device, dtype=torch.float8_e4m3fn)
    bp = deepgemm.marlin_fp8_masked_weight(torch.zeros(G, N, K, device=device, dtype=torch.float8_e4m3fn))
    a_s, b_s = torch.ones(G, max_m, device=device), torch.ones(G, N, device=device)
    d = torch.zeros(G, max_m, N, dtype=torch.bfloat16, device=device)
    mm = torch.zeros(G, dtype=torch.int32, device=device)

    def run(n):
        for _ in range(n):
            deepgemm.m_grouped_fp8_gemm_nt_masked((a, a_s), (bp, b_s), d, mm, 4)
    run(200)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    run(calls)
    t1 = time.perf_counter()
    torch.cuda.synchronize()
    return {"entry": "deepgemm.m_grouped_fp8_gemm_nt_masked", "calls": calls,
            "host_us_per_call": (t1 - t0) / calls * 1e6,
            "native_argument_checks": _core._glue is not None}


# ----------------------------------------------------------------------------- CPU arm
def cpu_reference_arm(steps: int, warmup: int, budget_s: float = 120.0):
    """The reference's CPU path (torch fp32 dequant-matmul, via the oracle) on a bounded sample
    of the headline workload: `ge` experts x `nc` output channels, same K, same routing."""
    sys.path.insert(0, os.path.join(REPO, "oracle"))
    import dg_oracle as O
    cfg = C2
    K, max_m = cfg["K"], cfg["max_m"]
    cpu_gen = torch.Generator().manual_seed(0)
    picks = torch.rand(cfg["tokens"], cfg["G"], generator=cpu_gen).topk(cfg["top_k"], dim=1).indices
    masked_m = torch.bincount(picks.flatten(), minlength=cfg["G"]).clamp(max=max_m)

    def build(ge, nc):
        g = torch.Generator().manual_seed(1)
        a, a_s = O.per_token_quant_fp8(torch.randn(ge, max_m, K, generator=g))
        b, b_s = O.per_token_quant_fp8(torch.randn(ge, nc, K, generator=g))
        return a, a_s, b, b_s

    def run(t, ge):
        a, a_s, b, b_s = t
        for e in range(ge):  # one expert at a time, valid rows only, like the reference tests compare
            m = int(masked_m[e])
            if m:
                O.ref_masked_scaled(a[e:e + 1, :m], b[e:e + 1], a_s[e:e + 1, :m], b_s[e:e + 1])

    # calibrate on one expert x 512 channels, then size the sample to fit the time budget
    probe = build(1, 512)
    run(probe, 1)
    t0 = time.perf_counter()
    run(probe, 1)
    per_unit = max(time.perf_counter() - t0, 1e-4)          # seconds per (expert x 512 channels)
    units = max(1.0, budget_s / max(steps + warmup, 1) / per_unit)
    ge = int(min(cfg["G"], max(1, units // 8)))              # 8 units = one full expert (N=4096)
    nc = cfg["N"] if units >= 8 else int(max(1, min(8, units))) * 512
    t = build(ge, nc)
    for _ in range(warmup):
        run(t, ge)
    t0 = time.perf_counter()
    for _ in range(steps):
        run(t, ge)
    sec = (time.perf_counter() - t0) / max(steps, 1)
    mm = masked_m[:ge]
    by = algorithmic_bytes(int(mm.sum()), int((mm > 0).sum()), ge, nc, K, 1, 1)
    return {"value": by / sec / 1e9, "unit": UNIT, "cores": torch.get_num_threads(),
            "host_cpus": os.cpu_count(), "kind": "port",
            "sample": "%d of %d experts x %d of %d output channels, K=%d, valid rows only; "
                      "torch fp32 dequant-matmul" % (ge, cfg["G"], nc, cfg["N"], K),
            "seconds_per_step": sec}


# ----------------------------------------------------------------------------- main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=500)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extras", action="store_true", help="skip the other configurations")
    ap.add_argument("--small", action="store_true", help="reduced problem (8 experts) for profiler captures")
    ap.add_argument("--profile", action="store_true",
                    help="profiler run: one workload's timed region only, bracketed by cudaProfilerStart/Stop")
    ap.add_argument("--workload", default="decode",
                    choices=["decode", "prefill_int8", "prefill_fp8", "w4a8", "w4a8_smem", "chain", "prefill_down"],
                    help="with --profile: which configuration to run (the JSON line is always decode)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    warmup = max(args.warmup, 3)
    cfg = dict(C2, G=8) if args.small else C2
    config = {"workload": "masked_fp8_decode G=%d K=%d N=%d max_m=%d tokens=%d top%d per GPU" % (
        cfg["G"], cfg["K"], cfg["N"], cfg["max_m"], cfg["tokens"], cfg["top_k"]),
        "sharding": "expert parallel, %d local experts per GPU" % cfg["G"],
        "l2": "inputs (%.0f MB per GPU) exceed the 126 MB L2; no flush" % (
            cfg["G"] * cfg["N"] * cfg["K"] / 1e6)}
    measurement = {}   # how this run measured (not part of the workload's description)

    if args.impl == "reference":
        if rank != 0:
            return
        torch.set_num_threads(os.cpu_count() or 1)
        cb = cpu_reference_arm(args.steps, args.warmup)
        line = {"impl": "reference", "metric": METRIC, "value": cb["value"], "unit": UNIT,
                "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": cb["seconds_per_step"] * 1e3, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": config, "cpu_baseline": cb,
                "e2e": {"value": cb["value"], "unit": UNIT, "h2d_bytes_per_step": 0,
                        "d2h_bytes_per_step": 0}, "gpu_launches": 0}
        print(json.dumps(line))
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (B200); there is no CPU path. "
                         "Use --impl reference for the CPU baseline.")
    import deepgemm
    from deepgemm import _cabi
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
    barrier = (lambda: dist.barrier()) if dist else None
    peaks = _peaks()

    if args.profile and args.workload == "chain":
        profile_chain(device, args.steps, warmup)
        return
    if args.profile and args.workload != "decode":
        if args.workload in ("w4a8", "w4a8_smem"):
            fn, info = make_masked_w4a8(device, args.small, smem_unpack=args.workload == "w4a8_smem")
        elif args.workload == "prefill_down":
            fn, info = make_prefill_down(device, args.small, path="gather")
        else:
            fn, info = make_contig_prefill(device, args.small, "int8" if args.workload == "prefill_int8" else "fp8")
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        ms, _, _ = time_launches(fn, args.steps, 0)
        torch.cuda.profiler.stop()
        sec = ms * 1e-3 / args.steps
        print(json.dumps({"profile_run": True, "workload": info["workload"], "ms_per_step": ms / args.steps,
                          "steps": args.steps, "tops": info["ops"] / sec / 1e12,
                          "gbs": info["bytes"] / sec / 1e9, "bytes_per_launch": info["bytes"],
                          "ops_per_launch": info["ops"]}))
        return

    w = make_decode_workload(device, seed=rank, cfg=cfg)
    bytes_per_step = decode_bytes(w)
    step = lambda: run_decode(w)

    # Bring the SM clock up from idle before the W warm-up steps (a freshly acquired GPU sits
    # at its idle clock and a few milliseconds of warm-up do not ramp it): untimed launches
    # of the same step for PREHEAT_S seconds.
    # If NVML still reports an SM clock below 90 % of the maximum after that and no power or
    # thermal limit explains it, keep going for up to PREHEAT_MAX_S (the clock is only read,
    # never set).
    sampler = ClockSampler(local_rank)
    t_pre = time.perf_counter()
    while True:
        for _ in range(50):
            step()
        torch.cuda.synchronize()
        spent = time.perf_counter() - t_pre
        if spent < PREHEAT_S:
            continue
        mhz = sampler.read_mhz()
        if mhz is None or sampler.max_mhz is None or mhz >= 0.9 * sampler.max_mhz or spent >= PREHEAT_MAX_S:
            break
        if sampler.read_throttled():   # a power or thermal limit, not the ramp from idle: more launches only deepen it
            break
    measurement["preheat_s"] = round(time.perf_counter() - t_pre, 3)

    sampler.start()
    launches0 = _cabi.query(_cabi.QUERY_LAUNCH_COUNT)
    if args.profile:
        for _ in range(warmup):
            step()
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        ms, t0, t1 = time_launches(step, args.steps, 0, barrier)
        torch.cuda.profiler.stop()
    else:
        # A timed region whose SM clock sat well below the maximum with no throttle reason
        # reported (the GPU had not ramped up, or dropped its clock for a moment) says nothing
        # about the kernel: such a region is measured again, at most twice, after more untimed
        # launches.  A genuinely capped clock (a reason is reported) is kept as it is.  All
        # ranks take the decision together.
        attempts = 0
        measurement["attempts"] = []   # every timed region, kept or not: ms per step, clock, reasons
        while True:
            attempts += 1
            launches0 = _cabi.query(_cabi.QUERY_LAUNCH_COUNT)
            ms, t0, t1 = time_launches(step, args.steps, warmup, barrier)
            c = sampler.summary(t0, t1)
            measurement["attempts"].append({
                "ms_per_step": ms / args.steps, "sm_mhz": c["sm_mhz"], "reasons": c["reasons"],
                "ms_x_mhz": (ms / args.steps * c["sm_mhz"]) if c["sm_mhz"] else None})
            low = (c["sm_mhz"] is not None and c["sm_max_mhz"] and c["sm_mhz"] < 0.9 * c["sm_max_mhz"]
                   and not c["reasons"])
            flag = torch.tensor([1 if low else 0], device=device)
            if dist:
                dist.all_reduce(flag, op=dist.ReduceOp.MAX)
            if int(flag) == 0 or attempts >= 3:
                break
            t_pre = time.perf_counter()
            while time.perf_counter() - t_pre < PREHEAT_MAX_S:
                for _ in range(50):
                    step()
                torch.cuda.synchronize()
        measurement["reported_attempt"] = attempts
    launches = _cabi.query(_cabi.QUERY_LAUNCH_COUNT) - launches0
    sampler.stop()
    clocks = sampler.summary(t0, t1)
    if args.profile:
        print(json.dumps({"profile_run": True, "ms_per_step": ms / args.steps, "steps": args.steps,
                          "gbs": bytes_per_step / (ms * 1e-3 / args.steps) / 1e9,
                          "bytes_per_launch": bytes_per_step, "clocks": clocks}))
        return

    # ---- end to end: host buffers in, host buffer out, through the public API
    host_in = [t.cpu().pin_memory() for t in (w["a"], w["a_scale"], w["masked_m"])]
    dev_in = [w["a"], w["a_scale"], w["masked_m"]]
    h2d = sum(t.numel() * t.element_size() for t in host_in)
    d2h = w["d"].numel() * w["d"].element_size()

    # Double-buffered pipeline over three streams: the host-to-device copy of step i+1 and the
    # device-to-host copy of step i-1 overlap the kernel of step i (PCIe is full duplex).  Every
    # step still moves all of its inputs in and all of its output out inside the timed region.
    import deepgemm
    fn_gemm = deepgemm.m_grouped_fp8_gemm_nt_masked
    cur = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    bufs = []
    for _ in range(2):
        bufs.append({"in": [torch.empty_like(t) for t in dev_in], "d": torch.zeros_like(w["d"]),
                     "host": torch.empty(w["d"].shape, dtype=w["d"].dtype).pin_memory(),
                     "ev_in": torch.cuda.Event(), "ev_kernel": torch.cuda.Event(),
                     "ev_out": torch.cuda.Event()})
    max_m = int(w["cfg"]["max_m"])

    def e2e_run(n):
        for i in range(n):
            b = bufs[i & 1]
            s_in.wait_event(b["ev_kernel"])          # the kernel two steps back has read this buffer
            with torch.cuda.stream(s_in):
                for h, dv in zip(host_in, b["in"]):
                    dv.copy_(h, non_blocking=True)
                b["ev_in"].record(s_in)
            cur.wait_event(b["ev_in"])
            cur.wait_event(b["ev_out"])              # its previous output has left the device
            fn_gemm((b["in"][0], b["in"][1]), (w["b"], w["b_scale"]), b["d"], b["in"][2], max_m)
            b["ev_kernel"].record(cur)
            s_out.wait_event(b["ev_kernel"])
            with torch.cuda.stream(s_out):
                b["host"].copy_(b["d"], non_blocking=True)
                b["ev_out"].record(s_out)
        for b in bufs:                               # the timed region ends when everything has landed
            cur.wait_event(b["ev_out"])

    e2e_steps = max(3, min(args.steps, 100))
    e2e_run(3)
    if barrier:
        barrier()
    torch.cuda.synchronize()
    ee0, ee1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ee0.record(cur)
    s_in.wait_event(ee0)
    s_out.wait_event(ee0)
    e2e_run(e2e_steps)
    ee1.record(cur)
    torch.cuda.synchronize()
    if barrier:
        barrier()
    ms_e2e = ee0.elapsed_time(ee1)
    resident = w["d"].cpu().view(torch.int16)   # result of the device-resident runs above
    e2e_check = all(bool(torch.equal(b["host"].view(torch.int16), resident)) for b in bufs)
    del bufs

    t_ms, t_e2e = torch.tensor([ms], device=device), torch.tensor([ms_e2e], device=device)
    tot = torch.tensor([bytes_per_step], device=device, dtype=torch.float64)
    if dist:
        dist.all_reduce(t_ms, op=dist.ReduceOp.MAX)
        dist.all_reduce(t_e2e, op=dist.ReduceOp.MAX)
        dist.all_reduce(tot, op=dist.ReduceOp.SUM)
    sec_step = float(t_ms) * 1e-3 / args.steps
    value = float(tot) / sec_step / 1e9
    e2e_value = float(tot) / (float(t_e2e) * 1e-3 / e2e_steps) / 1e9
    own_gbs = bytes_per_step / (ms * 1e-3 / args.steps) / 1e9

    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": float(t_ms) / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3 (f32 accumulate, bf16 out)",
            "data": "synthetic", "config": config,
            "roofline": {"bound": "hbm", "achieved": own_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": own_gbs / peaks["hbm_gbs"], "peak_source": peaks["source"],
                         "traffic": NCU_DECODE_DRAM_BYTES_PER_EXPERT * cfg["G"],
                         "traffic_note": "ncu dram__bytes_read + write of one full-size launch (32 experts), per expert x local experts",
                         "kernel": "grouped_gemm_kernel<E4M3,BN=256,4 stages> (rank 0)",
                         "algorithmic_bytes_per_launch": bytes_per_step},
            "clocks": clocks, "measurement": measurement,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                    "pipeline": "double-buffered: H2D, kernel and D2H of neighbouring steps overlap",
                    "outputs_equal_resident_run": e2e_check},
            "gpu_launches": int(launches),
            "tflops": 2.0 * int(w["masked_m_cpu"].sum()) * cfg["N"] * cfg["K"] / sec_step / 1e12 * world}

    if not args.no_extras and not args.small:
        extras = {}
        del host_in
        try:
            if world == 1:
                wt = make_decode_workload(device, seed=rank, cfg=cfg, tensor_wise=True)
                ms_t, _, _ = time_launches(lambda: run_decode(wt), 200, 10)
                gb = decode_bytes(wt) / (ms_t * 1e-3 / 200) / 1e9
                extras["masked_fp8_decode_tensor_wise"] = {"ms": ms_t / 200, "gbs": gb,
                                                           "frac_of_hbm_peak": gb / peaks["hbm_gbs"]}
                del wt
                extras["contiguous_int8_prefill"] = bench_contig_prefill(device, 20, 3, peaks, "int8")
                extras["contiguous_fp8_prefill"] = bench_contig_prefill(device, 20, 3, peaks, "fp8")
                extras["masked_w4a8"] = bench_masked_w4a8(device, 200, 10, peaks)
                extras["masked_bf16"] = bench_masked_bf16(device, 100, 10, peaks)
                extras["host_path"] = bench_host_path(device, cfg)
                extras["prefill_down_routing_list"] = bench_prefill_down(device, 20, 3)
            del w
            torch.cuda.empty_cache()
            extras["ep_prefill"] = bench_ep_prefill(device, rank, world, 10, 3, peaks)
        except Exception as exc:  # an extra must never cost the headline line
            extras["error"] = "%s: %s" % (type(exc).__name__, exc)
        line["other_configs"] = extras

    if rank == 0 and world == 1 and not args.small:
        torch.set_num_threads(os.cpu_count() or 1)
        line["cpu_baseline"] = cpu_reference_arm(3, 1, budget_s=20.0)
    elif rank == 0:
        line["cpu_baseline"] = None
    if dist:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line))


if __name__ == "__main__":
    main()
