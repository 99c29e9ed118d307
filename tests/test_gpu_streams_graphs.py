"""Properties of the entry points that a serving engine relies on (reference behaviour: launch on
the current stream of the input's device, asynchronous, no allocation, re-entrant --
csrc/arch/gfx936_gfx938_shared/m_grouped_fp8_gemm_nt_maksed_low_latency.cu:1149): capture into
a CUDA graph, launches from several host threads on their own streams, a non-default stream."""
import threading

import pytest
import torch

import deepgemm
from deepgemm import group_gemm_weight_pack as P

import dg_oracle as O
from helpers import assert_bf16_within_ulp, gen_masked_int8

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _problem(seed, g=6, max_m=96, n=512, k=512):
    mm = torch.randint(0, max_m + 1, (g,), generator=torch.Generator().manual_seed(seed))
    c = gen_masked_int8(g, max_m, n, k, mm, seed=seed)
    dev = {k_: v.to(DEV) for k_, v in c.items() if torch.is_tensor(v)}
    dev["bp"] = P.marlin_i8_masked_weight(c["b"].clone().to(DEV))
    ref = O.ref_masked_scaled(c["a"], c["b"], c["a_scale"].unsqueeze(-1), c["b_scale"].unsqueeze(-1))
    return c, dev, ref, int(mm.max())


def _launch(dev, d, expected_m):
    deepgemm.m_grouped_w8a8_gemm_nt_masked((dev["a"], dev["a_scale"]), (dev["bp"], dev["b_scale"]), d,
                                           dev["masked_m"], expected_m)


def _check(c, d, ref, what):
    d = d.cpu()
    for g in range(d.shape[0]):
        m = int(c["masked_m"][g])
        assert_bf16_within_ulp(d[g, :m], ref[g, :m], 1, f"{what} group {g}")


def test_cuda_graph_capture_and_replay():
    """The whole op (Python front-end -> custom op -> C ABI) is captured: nothing in it
    allocates, synchronises or queries the device.  Replays must recompute from the current
    contents of the input buffers."""
    c, dev, ref, em = _problem(1)
    d = torch.zeros_like(ref, device=DEV)
    _launch(dev, d, em)                                   # first call outside capture (lazy set-up)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        d.zero_()
        side.synchronize()
        with torch.cuda.graph(graph, stream=side):
            _launch(dev, d, em)
        graph.replay()
    torch.cuda.synchronize()
    _check(c, d, ref, "graph replay")
    c2, dev2, ref2, _ = _problem(2)                        # new data, same shapes, same buffers
    for key in ("a", "a_scale", "masked_m", "b_scale"):
        dev[key].copy_(dev2[key])
    dev["bp"].copy_(dev2["bp"])
    d.zero_()
    graph.replay()
    torch.cuda.synchronize()
    _check(c2, d, ref2, "graph replay on new inputs")


def test_concurrent_host_threads_on_their_own_streams():
    problems = [_problem(10 + i) for i in range(4)]
    outs = [torch.zeros_like(p[2], device=DEV) for p in problems]
    errors = []

    def worker(i):
        try:
            s = torch.cuda.Stream()
            with torch.cuda.stream(s):
                for _ in range(20):
                    _launch(problems[i][1], outs[i], problems[i][3])
            s.synchronize()
        except Exception as exc:                              # surfaced by the assert below
            errors.append(repr(exc))

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(4)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    torch.cuda.synchronize()
    for (c, _, ref, _), d in zip(problems, outs):
        _check(c, d, ref, "threaded launch")


def test_launch_goes_to_the_current_stream():
    """The kernel must be ordered after work already queued on the current (side) stream: the
    inputs are produced there by a long copy chain right before the call."""
    c, dev, ref, em = _problem(3)
    d = torch.zeros_like(ref, device=DEV)
    a_src = dev["a"].clone()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        dev["a"].zero_()
        junk = torch.empty(64 << 20, dtype=torch.uint8, device=DEV)
        for _ in range(8):
            junk.fill_(1)                                   # keeps the stream busy before the real input lands
        dev["a"].copy_(a_src)
        _launch(dev, d, em)
    side.synchronize()
    _check(c, d, ref, "side stream")


def test_tensors_on_a_device_other_than_the_current_one():
    """Like the reference (device guard on the input's device), the op runs where its tensors
    live, whatever the caller's current device is; per-device set-up must not leak across."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    c, dev0, ref, em = _problem(7)
    dev1 = {k: v.to("cuda:1") for k, v in dev0.items()}
    d1 = torch.zeros_like(ref, device="cuda:1")
    d0 = torch.zeros_like(ref, device="cuda:0")
    assert torch.cuda.current_device() == 0
    _launch(dev1, d1, em)                       # first use of device 1 in this process
    _launch(dev0, d0, em)
    _launch(dev1, d1, em)
    torch.cuda.synchronize(0)
    torch.cuda.synchronize(1)
    _check(c, d1, ref, "device 1 while device 0 is current")
    _check(c, d0, ref, "device 0")
