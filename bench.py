#!/usr/bin/env python
"""Benchmark of the chunked GLA hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]
                    [--scaling strong|weak] [--grads primal|fp32]
                    [--workload gla_train|decode|simple_gla_long|kda|kda_long|neighbours]

One "step" is one forward + backward pass of `chunk_gla` over one synthetic
batch of the headline configuration (bf16, B=8, T=4096, H=16, K=V=128,
chunk 64, initial state and final-state gradient included), made through the
public differentiable op (`tops_b200.ops.gla.chunk_gla` followed by
`torch.autograd.grad`).  Prints ONE JSON line (rank 0).

Under torchrun the ONE global batch of 8 sequences is split over the ranks
(batch x heads shard with no communication; 8/N sequences per rank:
`"scaling": "strong"`).  `--scaling weak` gives every rank its own batch of 8.

  value      tokens/s with inputs resident in HBM (CUDA events, max over ranks)
  e2e        the same metric with host buffers: one pinned host -> device copy
             of the packed inputs and one device -> host copy of the packed
             results per step inside the timed region
  roofline   the dominant kernel: algorithmic bytes per launch (its API inputs
             read once, its API outputs written once; scratch tensors are not
             counted) / its average launch duration (CUDA events recorded by
             the library around each launch during the timed steps) against
             the measured HBM peak
  cpu_baseline  the CPU oracle (a torch-CPU port of the reference's tops.cpu
             implementation) timed on this box's cores

`--impl reference` times that CPU port alone on the same configuration (the
reference itself is pure JAX; JAX is installed neither where this repository
is built nor on the GPU boxes).  It never loads the CUDA library.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "pallas-kernel_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

METRIC = "chunk_gla fwd+bwd tokens/sec (bf16, T=4096,H=16,D=128)"
# BASELINE.json configs[1]
GLA_TRAIN = dict(B=8, T=4096, H=16, K=128, V=128, C=64, dtype="bfloat16", seed=2)


def gla_train_bytes_per_token_head(grad_bytes):
    """Bytes every API tensor contributes once per (token, head) for fwd+bwd of gla_train:
    fwd reads q,k,v,g (4 x 256) writes o (256); bwd reads q,k,v,g,do (5 x 256), writes dq,dk,dg
    (3 x 128 x grad_bytes) and dv bf16 (256), plus the four fp32 states (h0, ht, dht, dh0:
    4 x 64 KiB per (b, h)) spread over T=4096 tokens: 64 B."""
    return 4 * 256 + 256 + 5 * 256 + 3 * 128 * grad_bytes + 256 + 64


GLA_TRAIN_FLOP_PER_TOKEN_HEAD = 98304 + 245760


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "measured"
    return 6650.0, 1400.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU while the timed region runs (read-only NVML)."""

    def __init__(self, index):
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for n, bit in names.items():
                    if mask & bit:
                        self.reasons.add(n)
            except Exception:
                pass
            self._stop.wait(0.02)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": (s[len(s) // 2] if s else None), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


def kernel_bytes(label, w, grad_bytes=2):
    """Algorithmic bytes of one launch of a kernel of the gla_train step: the API tensors it must
    read once and the API tensors it must write once.  Scratch (chunk-start states h', dh', the
    cumulative gates, A) is NOT counted; `scratch_bytes` below gives it separately."""
    tok = w["B"] * w["T"] * w["H"]
    K, V = w["K"], w["V"]
    in2 = 2  # bf16
    bhkv = w["B"] * w["H"] * K * V
    t = {
        # tcgen05 path
        "sm100_fwd_fused": tok * (3 * K + 2 * V) * in2 + 2 * bhkv * 4,                  # q,k,g,v in; o out; h0, ht
        "sm100_fwd_h": tok * (2 * K + V) * in2 + 2 * bhkv * 4,                           # k,g,v in; h0, ht
        "sm100_fwd_h_summary": tok * (2 * K + V) * in2,
        "sm100_fwd_o": tok * (3 * K + 2 * V) * in2,                                      # q,k,g,v in; o out
        "sm100_bwd_dh": tok * (2 * K + V) * in2 + 2 * bhkv * 4,                          # q,g,do in; dht, dh0
        "sm100_bwd_dh_summary": tok * (2 * K + V) * in2,
        "sm100_bwd_main": tok * (3 * K + 2 * V) * in2 + 3 * tok * K * grad_bytes + tok * V * in2,
    }
    return t.get(label)


def scratch_bytes(label, w):
    """Scratch one launch reads or writes besides its API tensors (bf16 [B,NT,H,K,V] state tensors)."""
    state = (w["B"] * w["T"] * w["H"] // w["C"]) * w["K"] * w["V"] * 2
    return {"sm100_fwd_fused": state, "sm100_fwd_h": state, "sm100_fwd_o": state, "sm100_bwd_dh": state,
            "sm100_bwd_main": 2 * state}.get(label, 0)


class Packed:
    """Named tensors laid out back to back (256-byte aligned) in one byte buffer, so that a whole set
    moves between host and device with a single copy."""

    def __init__(self, specs, device, pin=False):
        self.offsets, off = {}, 0
        for name, shape, dtype in specs:
            n = int(torch.tensor([], dtype=dtype).element_size())
            for d in shape:
                n *= d
            self.offsets[name] = (off, n, tuple(shape), dtype)
            off += (n + 255) // 256 * 256
        self.nbytes = off
        self.buf = torch.empty(off, dtype=torch.uint8, device=device)
        if pin:
            self.buf = self.buf.pin_memory()

    def view(self, name):
        off, n, shape, dtype = self.offsets[name]
        return self.buf[off:off + n].view(dtype).view(shape)

    def payload_bytes(self):
        return sum(n for _, n, _, _ in self.offsets.values())


def run_b200(args):
    rank, local_rank, world = dist_env()
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU fallback)"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    from tops_b200 import _lib as L
    from tops_b200.ops._chunk import chunk_bwd_call, chunk_fwd_call
    from tops_b200.ops.gla import chunk_gla
    from tops_b200.synth import make_inputs

    w = dict(GLA_TRAIN)
    strong = world > 1 and args.scaling == "strong"
    if strong:
        assert w["B"] % world == 0, f"the global batch of {w['B']} sequences does not split over {world} ranks"
    if args.batch:
        w["B"] = args.batch      # smaller batches are for profiler captures only
    dtype = getattr(torch, w["dtype"])
    scale = w["K"] ** -0.5
    names = ("q", "k", "v", "g", "do", "h0", "dht")
    if strong:
        # one global batch (the single-GPU workload), contiguous rows of it per rank
        full = make_inputs(w["seed"], w["B"], w["T"], w["H"], w["K"], w["V"], dtype=dtype, with_h0=True, with_grads=True)
        per = w["B"] // world
        host = {n: full[n][rank * per:(rank + 1) * per].contiguous() for n in names}
        del full
        w["B"] = per
    else:
        host = make_inputs(w["seed"] + 1000 * rank, w["B"], w["T"], w["H"], w["K"], w["V"], dtype=dtype,
                           with_h0=True, with_grads=True)
    specs = [(n, tuple(host[n].shape), host[n].dtype) for n in names]
    pinned_in = Packed(specs, "cpu", pin=True)
    for n in names:
        pinned_in.view(n).copy_(host[n])
    del host

    # "primal": dq, dk, dg come back in the dtypes of q, k, g (bf16), as the differentiable op returns
    # them and as the reference's accelerator kernel writes them; "fp32": as the reference's CPU
    # orchestrator returns them (explicit chunk_gla_fwd/_bwd-style calls, not the autograd op)
    primal = args.grads == "primal"
    grad_bytes = 2 if primal else 4

    def device_set():
        p = Packed(specs, dev)
        t = {n: p.view(n) for n in names}
        for n in ("q", "k", "v", "g", "h0"):
            t[n] = t[n].detach().requires_grad_(True)
        return p, t

    def step_public(t):
        """What a user runs: the differentiable op, then autograd."""
        o, ht = chunk_gla(t["q"], t["k"], t["v"], t["g"], scale=scale, initial_state=t["h0"], output_final_state=True,
                          chunk_size=w["C"])
        dq, dk, dv, dg, dh0 = torch.autograd.grad((o, ht), (t["q"], t["k"], t["v"], t["g"], t["h0"]), (t["do"], t["dht"]))
        return o, ht, dq, dk, dv, dg, dh0

    def step_calls(t, primal_dtypes):
        """The two C-ABI calls of a step without autograd around them."""
        with torch.no_grad():
            o, ht, _, _, hs = chunk_fwd_call(t["q"], t["k"], t["v"], t["g"], L.GATE_PER_CHANNEL, scale, t["h0"], True, w["C"],
                                             want_saved=True)
            dq, dk, dv, dg, dh0 = chunk_bwd_call(t["q"], t["k"], t["v"], t["g"], L.GATE_PER_CHANNEL, scale, t["h0"],
                                                 t["do"], t["dht"], w["C"], torch.float32, True, True, h_saved=hs,
                                                 primal_dtypes=primal_dtypes)
        return o, ht, dq, dk, dv, dg, dh0

    step = step_public if primal else (lambda t: step_calls(t, False))

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world > 1:
            tms = torch.tensor([ms], device=dev)
            torch.distributed.all_reduce(tms, op=torch.distributed.ReduceOp.MAX)
            ms = float(tms.item())
        return ms

    # A rank's step inputs must not sit in L2 (126 MB) from the previous step.  With two or more
    # sequences per rank the inputs alone (84 MB per sequence) exceed it; with one sequence per rank
    # (8 GPUs) every timed step is bracketed by its own event pair and a 256 MB write in between
    # evicts the cache outside the timed intervals.
    in_bytes = sum(n for _, n, _, _ in pinned_in.offsets.values())
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if in_bytes < 1.2 * (126 << 20) else None

    def timed(fn, steps, drain=None):
        barrier()
        if flush is not None and drain is None:
            pairs = []
            for _ in range(steps):
                flush.zero_()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn()
                e1.record()
                pairs.append((e0, e1))
            barrier()
            return max_over_ranks(sum(a.elapsed_time(b) for a, b in pairs) / steps)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        if drain is not None:
            drain()      # side streams join the timed stream before the closing event
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1) / steps)

    def read_profile():
        buf = ctypes.create_string_buffer(1 << 16)
        L.lib.tops_b200_profile_read(buf, len(buf))
        out = {}
        for line in buf.value.decode().splitlines():
            label, count, total = line.split()
            out[label] = (int(count), float(total))
        return out

    dev_sets = [device_set() for _ in range(2)]
    x_buf, x = dev_sets[0]
    x_buf.buf.copy_(pinned_in.buf, non_blocking=True)
    torch.cuda.synchronize()

    # ---- device-resident throughput (the public op) -------------------------------------
    for _ in range(args.warmup):
        step(x)
    L.lib.tops_b200_profile_enable(1)
    launches0 = L.launch_count()
    with ClockSampler(local_rank) as clocks:
        ms = timed(lambda: step(x), args.steps)
    launches = L.launch_count() - launches0
    L.lib.tops_b200_profile_enable(0)
    kernels = read_profile()

    if args.kernel_only:
        if rank == 0:
            print(json.dumps({"kernel_only": True, "batch": w["B"], "ms_per_step": ms,
                              "kernels_ms_per_launch": {k: v[1] / v[0] for k, v in sorted(kernels.items())}}), flush=True)
        return

    # the same two library calls without autograd, allocation of outputs included
    ms_calls = timed(lambda: step_calls(x, primal), args.steps)

    # ---- sustained: the same loop for at least two seconds ---------------------------------
    sustained = None
    if not args.batch:
        chunk_steps = max(50, int(0.25 / (ms * 1e-3)))
        with ClockSampler(local_rank) as sclocks:
            barrier()
            t0 = time.perf_counter()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            n_sus = 0
            while True:
                for _ in range(chunk_steps):
                    step(x)
                n_sus += chunk_steps
                torch.cuda.synchronize()
                if time.perf_counter() - t0 >= 2.0:
                    break
            e1.record()
            barrier()
        sustained = {"ms_per_step": max_over_ranks(e0.elapsed_time(e1) / n_sus), "steps": n_sus,
                     "clocks": sclocks.summary()}

    # ---- CUDA-graph replay of the public step (launch-bound cases: few sequences per GPU) ---
    graph = None
    try:
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                step(x)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        l0 = L.launch_count()
        with torch.cuda.graph(g):
            graph_outs = step(x)
        per_replay = L.launch_count() - l0
        for _ in range(3):
            g.replay()
        ms_graph = timed(g.replay, args.steps)
        graph = {"ms_per_step": ms_graph, "kernels_per_replay": int(per_replay)}
        del graph_outs
    except Exception as exc:   # capture is an optimisation of the launch path, not a requirement
        graph = {"error": f"{type(exc).__name__}: {exc}"[:200]}
        torch.cuda.synchronize()

    # ---- end to end: host buffers in, host buffers out --------------------------------------
    # Per step: ONE copy of the packed inputs from pinned host memory, the step through the public op,
    # the seven results gathered into one device buffer, ONE copy of it to pinned host memory.  Two
    # buffer sets and three streams let the upload of step i+1, the kernels of step i and the download
    # of step i-1 overlap (PCIe is full duplex); every copy runs inside the timed region.
    outs = step(x)
    out_names = ("o", "ht", "dq", "dk", "dv", "dg", "dh0")
    out_specs = [(n, tuple(o.shape), o.dtype) for n, o in zip(out_names, outs)]
    del outs
    out_dev = [Packed(out_specs, dev) for _ in range(2)]
    out_host = [Packed(out_specs, "cpu", pin=True) for _ in range(2)]
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    uploaded = [torch.cuda.Event() for _ in range(2)]
    computed = [torch.cuda.Event() for _ in range(2)]
    downloaded = [torch.cuda.Event() for _ in range(2)]
    counter = [0]

    def e2e_step():
        slot = counter[0] & 1
        counter[0] += 1
        cur = torch.cuda.current_stream()
        buf, t = dev_sets[slot]
        s_in.wait_event(computed[slot])          # the kernels of two steps ago have read this input set
        with torch.cuda.stream(s_in):
            buf.buf.copy_(pinned_in.buf, non_blocking=True)
            uploaded[slot].record(s_in)
        cur.wait_event(uploaded[slot])
        cur.wait_event(downloaded[slot])         # the result buffer of this slot has left the device
        res = step(t)
        for n, r in zip(out_names, res):
            out_dev[slot].view(n).copy_(r)
        computed[slot].record(cur)
        s_out.wait_event(computed[slot])
        with torch.cuda.stream(s_out):
            out_host[slot].buf.copy_(out_dev[slot].buf, non_blocking=True)
            downloaded[slot].record(s_out)

    def e2e_drain():
        torch.cuda.current_stream().wait_stream(s_out)

    e2e_steps = max(3, min(args.steps, 10))
    for _ in range(2):
        e2e_step()
    ms_e2e = timed(e2e_step, e2e_steps, e2e_drain)

    # the copies alone: the same bytes each way, both directions at once, nothing else running
    def copy_only():
        cur = torch.cuda.current_stream()
        s_in.wait_stream(cur)
        s_out.wait_stream(cur)
        with torch.cuda.stream(s_in):
            dev_sets[0][0].buf.copy_(pinned_in.buf, non_blocking=True)
        with torch.cuda.stream(s_out):
            out_host[0].buf.copy_(out_dev[0].buf, non_blocking=True)
        cur.wait_stream(s_in)
        cur.wait_stream(s_out)
    copy_only()
    ms_copy = timed(copy_only, e2e_steps)
    h2d, d2h = pinned_in.payload_bytes(), out_host[0].payload_bytes()

    device_err = L.device_error()
    assert device_err == 0, f"a kernel gave up on a bounded wait (code {device_err}): results are invalid"

    tokens = w["B"] * w["T"] * world
    hbm_peak, tf_peak, peak_kind = measured_peaks()
    use_graph = graph is not None and "ms_per_step" in graph and graph["ms_per_step"] < ms
    ms_value = graph["ms_per_step"] if use_graph else ms
    result = {
        "metric": METRIC,
        "value": tokens / (ms_value * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_value, "higher_is_better": True,
        "scaling": "strong" if strong else "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"chunk_gla fwd+bwd, B={w['B'] * world if strong else w['B']}"
                               f"{'' if strong or world == 1 else ' per GPU'}, T=4096, H=16, K=V=128, chunk 64, "
                               "h0+dht (BASELINE configs[1])",
                   "grads": "dq, dk, dg in bf16 (the primal dtypes)" if primal else "dq, dk, dg in fp32",
                   "global_batch": w["B"] * world, "seq_len": w["T"],
                   "parallelism": (f"one batch of {w['B'] * world} sequences split {w['B']} per GPU over {world} GPUs, "
                                   "no communication") if strong else f"batch x heads shard x{world}, no communication",
                   "api": "tops_b200.ops.gla.chunk_gla + torch.autograd.grad" if primal
                          else "chunk_fwd_call / chunk_bwd_call (explicit forward and backward entry points)",
                   "launch": "CUDA graph replay of the step" if use_graph else "eager",
                   "l2": ("256 MB written between timed steps (one event pair per step): a rank's inputs are smaller than L2"
                          if flush is not None else "a rank's step inputs are larger than L2 (126 MB); no flush")},
        "eager": {"ms_per_step": ms, "value": tokens / (ms * 1e-3)},
        "graph_replay": graph,
        "kernels_only": {"ms_per_step": ms_calls, "what": "the two C-ABI calls of a step without autograd"},
        "sustained": sustained,
        "e2e": {"value": tokens / (ms_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": ms_e2e, "steps": e2e_steps,
                "copy_roofline_ms": ms_copy,
                "frac_of_copy_roofline": ms_copy / ms_e2e,
                "pipeline": "one packed H2D and one packed D2H copy per step; upload of step i+1, kernels of "
                            "step i and download of step i-1 overlap (3 streams)"},
        "gpu_launches": int(launches),
        "clocks": clocks.summary(),
        "device_error": device_err,
    }
    # whole-step view against both roofs
    th = w["B"] * w["T"] * w["H"]
    per_th = gla_train_bytes_per_token_head(grad_bytes)
    result["step_roofline"] = {
        "hbm_frac": th * per_th / (ms_value * 1e-3) / (hbm_peak * 1e9),
        "tensor_frac": th * GLA_TRAIN_FLOP_PER_TOKEN_HEAD / (ms_value * 1e-3) / (tf_peak * 1e12),
        "bytes_per_token_head": per_th, "flop_per_token_head": GLA_TRAIN_FLOP_PER_TOKEN_HEAD,
        "peaks": peak_kind}
    if kernels:
        top = max(kernels, key=lambda k: kernels[k][1])
        count, total = kernels[top]
        per_launch_ms = total / count
        nbytes = kernel_bytes(top, w, grad_bytes)
        achieved = None if nbytes is None else nbytes / (per_launch_ms * 1e-3) / 1e9
        traffic = None
        tpath = os.path.join(ROOT, "profiles", "traffic.json")
        if os.path.exists(tpath) and w["B"] == 8:
            tj = json.load(open(tpath))
            traffic = tj.get(top if primal else top + "_fp32")
        result["roofline"] = {"bound": "hbm", "kernel": top, "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                              "frac": None if achieved is None else achieved / hbm_peak, "traffic": traffic,
                              "traffic_source": "profiles/traffic.json (ncu dram bytes of one full-size launch; not "
                                                "measured in this run)" if traffic else None,
                              "algorithmic_bytes": nbytes, "scratch_bytes": scratch_bytes(top, w),
                              "frac_with_scratch": None if nbytes is None else
                              (nbytes + scratch_bytes(top, w)) / (per_launch_ms * 1e-3) / 1e9 / hbm_peak,
                              "ms_per_launch": per_launch_ms, "peak_source": peak_kind,
                              "kernels_ms_per_step": {k: v[1] / args.steps for k, v in sorted(kernels.items())}}
    if rank == 0 and world == 1 and not args.batch:
        # the other gradient dtype and the secondary workloads, each a few timed steps
        extra = {}
        other = (lambda t: step_calls(t, False)) if primal else step_public
        for _ in range(3):
            other(x)
        ms_o = timed(lambda: other(x), args.steps)
        ob = gla_train_bytes_per_token_head(4 if primal else 2)
        extra["gla_train_fp32_grads" if primal else "gla_train_primal_grads"] = {
            "ms": ms_o, "tokens_per_s": tokens / (ms_o * 1e-3), "algorithmic_bytes": th * ob,
            "frac": th * ob / (ms_o * 1e-3) / (hbm_peak * 1e9)}
        del dev_sets, out_dev, x, x_buf
        torch.cuda.empty_cache()
        for name in ("decode", "simple_gla_long", "kda"):
            try:
                r = secondary(name, steps=args.steps, seq=0)
                extra[name] = {"ms": r["ms_per_step"], "value": r["value"], "unit": r["unit"],
                               "algorithmic_bytes": r["algorithmic_bytes"], "frac": r["frac"],
                               "kernels_ms_per_launch": r["kernels_ms_per_launch"],
                               "workload": r["config"]["workload"]}
            except Exception as exc:
                extra[name] = {"error": f"{type(exc).__name__}: {exc}"[:200]}
            torch.cuda.empty_cache()
        result["other_workloads"] = extra
        result["device_error"] = L.device_error()
        result["cpu_baseline"] = cpu_baseline(sample_B=8, passes=2)
    if rank == 0:
        print(json.dumps(result), flush=True)
    if world > 1:
        torch.distributed.destroy_process_group()


def _load_synth():
    """tops_b200.synth without importing the package (which would load the CUDA library)."""
    import importlib.util
    path = os.path.join(ROOT, "pallas-kernel_b200", "tops_b200", "synth.py")
    spec = importlib.util.spec_from_file_location("tops_b200_synth_standalone", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def cpu_baseline(sample_B, passes, warm=1, budget_s=None):
    """The oracle (torch-CPU port of tops.cpu chunk_gla / chunk_gla_bwd) on a
    batch slice of the workload, all host threads."""
    from oracle import gla as G
    make_inputs = _load_synth().make_inputs
    # torchrun exports OMP_NUM_THREADS=1; the CPU arm uses every host core
    try:
        torch.set_num_threads(len(os.sched_getaffinity(0)))
    except Exception:
        torch.set_num_threads(os.cpu_count() or 1)
    w = GLA_TRAIN
    x = make_inputs(w["seed"], sample_B, w["T"], w["H"], w["K"], w["V"], dtype=getattr(torch, w["dtype"]),
                    with_h0=True, with_grads=True)
    scale = w["K"] ** -0.5

    def one():
        G.chunk_gla(x["q"], x["k"], x["v"], x["g"], scale, x["h0"], True, chunk_size=w["C"])
        G.chunk_gla_bwd(x["q"], x["k"], x["v"], x["g"], None, scale, x["h0"], None, None, x["do"], x["dht"],
                        chunk_size=w["C"])
    for _ in range(warm):
        one()
    t0 = time.perf_counter()
    done = 0
    for _ in range(passes):
        one()
        done += 1
        if budget_s is not None and time.perf_counter() - t0 > budget_s:
            break
    dt = (time.perf_counter() - t0) / done
    return {"value": sample_B * w["T"] / dt, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"fwd+bwd of the whole workload (B={sample_B}, T=4096, H=16, K=V=128), {done} timed passes",
            "seconds_per_pass": dt, "passes": done}


def run_reference(args):
    rank, _, world = dist_env()
    if rank != 0:
        return
    w = GLA_TRAIN
    # the GPU arm's configuration: the whole B=8 batch per step; at most two minutes of timed passes
    cb = cpu_baseline(w["B"], passes=max(1, args.steps), warm=max(1, min(args.warmup, 1)), budget_s=120.0)
    ms = cb["seconds_per_pass"] * 1e3
    loaded = [ln.split()[-1] for ln in open("/proc/self/maps") if "libtops_b200" in ln]
    line = {
        "impl": "reference", "metric": METRIC,
        "value": cb["value"], "unit": "tokens/s", "n_gpus": world, "steps": cb["passes"], "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "strong" if world > 1 else "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "chunk_gla fwd+bwd, B=8, T=4096, H=16, K=V=128, chunk 64, h0+dht (BASELINE configs[1])",
                   "grads": "dq, dk, dg in fp32 (what the reference's CPU orchestrator returns)",
                   "global_batch": w["B"], "seq_len": w["T"], "parallelism": "host cores of rank 0",
                   "steps_note": f"{cb['passes']} timed passes of the whole batch (capped at 120 s of CPU time)"},
        "cpu_baseline": {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": cb["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "cuda_library_loaded": bool(loaded),
        "note": "torch-CPU port of the reference's tops.cpu (the reference is pure JAX; `import jax` fails on the GPU "
                "box with ModuleNotFoundError and there is no wheel to install it from)",
    }
    print(json.dumps(line), flush=True)


def simple_gla_bytes(B, T, H, K, V):
    """Every API tensor of a simple_gla forward + backward once (bf16 activations, bf16 scalar gate, fp32 gate
    gradient, fp32 states): q, k, v, g in, o out; q, k, v, g, do in, dq, dk, dv, dg out; h0, ht, dht, dh0.
    Scratch (chunk-start states, segment summaries) is not counted."""
    per_token_head = (2 * 2 * K + 2 * V + 2 + 2 * V) + (2 * 2 * K + 2 * 2 * V + 2 + 2 * 2 * K + 2 * V + 4)
    return B * T * H * per_token_head + 4 * B * H * K * V * 4


def kda_bytes(B, T, H, K, V):
    """Every API tensor of a KDA forward + backward once, at the dtypes of the differentiable op (all bf16 but
    the fp32 states): q, k, v, g, beta in, o out; q, k, v, g, beta, do in, dq, dk, dv, dg, dbeta out; h0, ht,
    dht, dh0.  The residuals the forward keeps for the backward are not counted."""
    per_token_head = (3 * 2 * K + 2 * V + 2 + 2 * V) + (3 * 2 * K + 2 * 2 * V + 2 + 3 * 2 * K + 2 * V + 2)
    return B * T * H * per_token_head + 4 * B * H * K * V * 4


def secondary(name, steps, seq):
    """One secondary workload (BASELINE configs[2..4]) on the current GPU, device-resident, through
    the public ops.  Returns a dict with ms_per_step, value, unit, algorithmic_bytes, frac, config."""
    from tops_b200 import _lib as L
    from tops_b200.synth import make_inputs

    def timed(fn, n, warmup):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    hbm_peak, _, peak_kind = measured_peaks()
    n0 = L.launch_count()
    L.lib.tops_b200_profile_enable(1)
    if name == "decode":
        from tops_b200.ops.gla import fused_recurrent_gla_decode_
        B, H, K, V = 128, 32, 128, 128
        x = {k: v.cuda() for k, v in make_inputs(3, B, 1, H, K, V, dtype=torch.bfloat16, with_h0=True).items()}
        state = x["h0"].clone()
        ms = timed(lambda: fused_recurrent_gla_decode_(x["q"], x["k"], x["v"], x["g"], state), max(steps, 200), 20)
        nbytes = 2 * B * H * K * V * 4
        out = {"metric": "fused_recurrent_gla decode GB/s (state read+write)", "value": nbytes / (ms * 1e-3) / 1e9,
               "unit": "GB/s",
               "config": {"workload": "decode B=128 H=32 K=V=128, 1 token per call, fp32 state in place (BASELINE configs[2])"}}
    elif name == "simple_gla_long":
        from tops_b200.ops.simple_gla import chunk_simple_gla
        B, T, H, K, V = 1, seq or 65536, 32, 128, 128
        x = {k: v.cuda() for k, v in make_inputs(4, B, T, H, K, V, dtype=torch.bfloat16, gate="scalar", with_h0=True,
                                                   with_grads=True).items()}
        leaves = [x[n].requires_grad_(True) for n in ("q", "k", "v", "g", "h0")]

        def step():
            o, ht = chunk_simple_gla(x["q"], x["k"], x["v"], g=x["g"], initial_state=x["h0"], output_final_state=True,
                                     chunk_size=64)
            return torch.autograd.grad((o, ht), leaves, (x["do"], x["dht"]))
        ms = timed(step, max(3, min(steps, 10)), 3)
        nbytes = simple_gla_bytes(B, T, H, K, V)
        out = {"metric": "simple_gla chunk fwd+bwd tokens/s", "value": B * T / (ms * 1e-3), "unit": "tokens/s",
               "config": {"workload": f"simple_gla fwd+bwd B=1 T={T} H=32 K=V=128 chunk 64 bf16, scalar bf16 gate, one GPU "
                                      "(BASELINE configs[3] without the time sharding)"}}
    elif name in ("kda", "kda_long"):
        from tops_b200.ops.kda import chunk_kda
        B, T, H, K, V = (4, seq or 8192, 32, 128, 128) if name == "kda" else (1, seq or 32768, 32, 128, 128)
        x = {k: v.cuda() for k, v in make_inputs(5, B, T, H, K, V, dtype=torch.bfloat16, with_h0=True, with_grads=True,
                                                   with_beta=True, l2norm_qk=True).items()}
        leaves = [x[n].requires_grad_(True) for n in ("q", "k", "v", "g", "beta", "h0")]

        def step():
            o, ht = chunk_kda(x["q"], x["k"], x["v"], x["g"], x["beta"], initial_state=x["h0"], output_final_state=True,
                              chunk_size=64)
            return torch.autograd.grad((o, ht), leaves, (x["do"], x["dht"]))
        ms = timed(step, max(2, min(steps, 5)), 2)
        nbytes = kda_bytes(B, T, H, K, V)
        out = {"metric": "KDA chunk fwd+bwd tokens/s", "value": B * T / (ms * 1e-3), "unit": "tokens/s",
               "config": {"workload": f"KDA fwd+bwd B={B} T={T} H=32 K=V=128 chunk 64 bf16, one GPU"
                                      + (" (BASELINE configs[4])" if name == "kda" else "")}}
    elif name == "neighbours":
        # the elementwise steps either side of the path, each forward + backward through its public op, at the
        # tensor sizes of BASELINE configs[1]: one [8, 4096, 16, 128] bf16 tensor is 134 MB
        from tops_b200.ops.gate import gla_gate, kda_gate_fwd
        from tops_b200.ops.norm import l2norm, rmsnorm_gated
        B, T, H, D = 8, seq or 4096, 16, 128
        gen = torch.Generator(device="cuda").manual_seed(6)
        mk = lambda *shape, dt=torch.bfloat16: torch.randn(*shape, device="cuda", generator=gen).to(dt).requires_grad_(True)
        x, g, dy = mk(B, T, H, D), mk(B, T, H, D), mk(B, T, H, D)
        w, A_log, bias = mk(D, dt=torch.float32), mk(H, dt=torch.float32), mk(H * D, dt=torch.float32)
        dy32 = dy.detach().float()

        def step():
            torch.autograd.grad(gla_gate(g), g, dy.detach())
            torch.autograd.grad(kda_gate_fwd(g, A_log, bias), (g, A_log, bias), dy32)
            torch.autograd.grad(l2norm(x), x, dy.detach())
            torch.autograd.grad(rmsnorm_gated(x, g, w), (x, g, w), dy.detach())
        ms = timed(step, max(3, min(steps, 10)), 3)
        n = B * T * H * D
        # gla gate 2+2 / 2+2+2; kda gate (fp32 out) 2+4 / 2+4+2; l2norm 2+2 / 2+2+2; norm+gate 2+2+2 / 2+2+2+2+2
        per_label = {"gate_act_fwd": (4 + 6) * n / 2, "gate_act_bwd": (6 + 8) * n / 2, "l2norm_fwd": 4 * n,
                     "l2norm_bwd": 6 * n, "rmsnorm_gated_fwd": 6 * n, "rmsnorm_gated_bwd": 10 * n}
        nbytes = int(sum(2 * v if k.startswith("gate_act") else v for k, v in per_label.items()))
        out = {"metric": "gate / l2norm / norm+gate forward + backward, GB/s per kernel", "value": nbytes / (ms * 1e-3) / 1e9,
               "unit": "GB/s", "bytes_per_launch": per_label,
               "config": {"workload": f"gla_gate, kda_gate, l2norm, rmsnorm_gated fwd+bwd on [8,{T},16,128] bf16, one GPU"}}
    else:
        raise ValueError(name)
    L.lib.tops_b200_profile_enable(0)
    buf = ctypes.create_string_buffer(1 << 16)
    L.lib.tops_b200_profile_read(buf, len(buf))
    out["kernels_ms_per_launch"] = {ln.split()[0]: float(ln.split()[2]) / int(ln.split()[1])
                                    for ln in buf.value.decode().splitlines()}
    if "bytes_per_launch" in out:
        out["kernels_gbs"] = {k: out["bytes_per_launch"][k] / (v * 1e-3) / 1e9
                              for k, v in out["kernels_ms_per_launch"].items() if k in out["bytes_per_launch"]}
    out["ms_per_step"] = ms
    out["algorithmic_bytes"] = nbytes
    out["frac"] = nbytes / (ms * 1e-3) / 1e9 / hbm_peak
    out["roofline"] = {"bound": "hbm", "achieved": nbytes / (ms * 1e-3) / 1e9, "peak": hbm_peak, "unit": "GB/s",
                       "frac": out["frac"], "peak_source": peak_kind}
    out["gpu_launches"] = L.launch_count() - n0
    err = L.device_error()
    assert err == 0, f"a kernel gave up on a bounded wait (code {err})"
    return out


def run_time_shard(args):
    """`--workload simple_gla_long --gpus N`: BASELINE configs[3], ONE sequence of 65536 tokens sharded
    over time across N ranks.  A step is forward + backward of every shard, with one all-gather of the shard
    summaries (fp32 [B,H,K,V] + the summed gates) per direction; strong scaling (the sequence is fixed).
    `--workload kda_long --gpus N`: the same for ONE KDA sequence (B=1, T=32768, H=32), whose shards exchange
    their dense transitions [B,H,K,K] as well (no BASELINE configuration: KDA there shards over batch x head)."""
    rank, local_rank, world = dist_env()
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    import torch.distributed as dist
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dist.init_process_group("nccl", device_id=dev)
    from tops_b200 import _lib as L
    from tops_b200 import time_shard as TS
    from tops_b200.synth import make_inputs
    kda = args.workload == "kda_long"
    B, T, H, K, V, C = 1, args.seq or (32768 if kda else 65536), 32, 128, 128, 64
    assert T % (world * C) == 0
    if kda:
        full = make_inputs(5, B, T, H, K, V, dtype=torch.bfloat16, with_h0=True, with_grads=True, with_beta=True,
                           l2norm_qk=True)
    else:
        full = make_inputs(4, B, T, H, K, V, dtype=torch.bfloat16, gate="scalar", with_h0=True, with_grads=True)
    sl = slice(rank * T // world, (rank + 1) * T // world)
    x = {n: (t[:, sl] if t.ndim >= 3 and t.shape[1] == T else t).contiguous().to(dev) for n, t in full.items()}
    del full
    scale = K ** -0.5
    ops = TS.kda_cuda_ops() if kda else TS.cuda_ops("simple_gla", C)
    # the exchange alone, timed with its own events inside the step
    ev = []

    gather = TS._gather

    def timed_gather(t, group):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out = gather(t, group)
        e1.record()
        ev.append((e0, e1))
        return out
    TS._gather = timed_gather

    def step():
        if kda:
            o, final, ctx = TS.kda_forward(ops, x["q"], x["k"], x["v"], x["g"], x["beta"], scale, x["h0"])
            return TS.kda_backward(ops, x["q"], x["k"], x["v"], x["g"], x["beta"], scale, ctx, x["do"], x["dht"])
        o, final, h_in = TS.forward(ops, x["q"], x["k"], x["v"], x["g"], scale, x["h0"])
        return TS.backward(ops, x["q"], x["k"], x["v"], x["g"], scale, h_in, x["do"], x["dht"])

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()
    for _ in range(max(args.warmup, 3)):
        step()
    ev.clear()
    n0 = L.launch_count()
    steps = max(3, min(args.steps, 10))
    with ClockSampler(local_rank) as clocks:
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        barrier()
    ms = e0.elapsed_time(e1) / steps
    ms_x = sum(a.elapsed_time(b) for a, b in ev) / steps
    t = torch.tensor([ms, ms_x], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_x = float(t[0]), float(t[1])
    err = L.device_error()
    assert err == 0, f"a kernel gave up on a bounded wait (code {err})"
    hbm_peak, _, peak_kind = measured_peaks()
    nbytes = kda_bytes(B, T, H, K, V) if kda else simple_gla_bytes(B, T, H, K, V)
    if rank == 0 and kda:
        print(json.dumps({
            "metric": "KDA chunk fwd+bwd tokens/s, one sequence sharded over time", "value": B * T / (ms * 1e-3),
            "unit": "tokens/s", "n_gpus": world, "steps": steps, "warmup": max(args.warmup, 3), "ms_per_step": ms,
            "higher_is_better": True, "scaling": "strong", "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"KDA fwd+bwd B=1 T={T} H=32 K=V=128 chunk 64 bf16, {T // world} tokens per GPU",
                       "exchange": "NCCL all-gathers of fp32 [B,H,K,K] transitions and [B,H,K,V] summaries forward, "
                                   "[B,H,K,V] summaries backward, NVLS off",
                       "extra_passes": "per shard: two forward passes for the transition and the summary, one reverse "
                                       "scan for the backward summary"},
            "exchange_ms_per_step": ms_x, "exchange_share": ms_x / ms,
            "roofline": {"bound": "hbm", "achieved": nbytes / (ms * 1e-3) / 1e9 / world, "peak": hbm_peak, "unit": "GB/s per GPU",
                         "frac": nbytes / (ms * 1e-3) / 1e9 / world / hbm_peak, "peak_source": peak_kind},
            "gpu_launches": int(L.launch_count() - n0), "clocks": clocks.summary(), "device_error": err}), flush=True)
    elif rank == 0:
        print(json.dumps({
            "metric": "simple_gla chunk fwd+bwd tokens/s, one sequence sharded over time", "value": B * T / (ms * 1e-3),
            "unit": "tokens/s", "n_gpus": world, "steps": steps, "warmup": max(args.warmup, 3), "ms_per_step": ms,
            "higher_is_better": True, "scaling": "strong", "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"simple_gla fwd+bwd B=1 T={T} H=32 K=V=128 chunk 64 bf16, scalar bf16 gate, "
                                   f"{T // world} tokens per GPU (BASELINE configs[3])",
                       "exchange": "2 NCCL all-gathers per direction (summed gates, fp32 [B,H,K,V] shard summary), NVLS off"},
            "exchange_ms_per_step": ms_x, "exchange_share": ms_x / ms,
            "roofline": {"bound": "hbm", "achieved": nbytes / (ms * 1e-3) / 1e9 / world, "peak": hbm_peak, "unit": "GB/s per GPU",
                         "frac": nbytes / (ms * 1e-3) / 1e9 / world / hbm_peak, "peak_source": peak_kind},
            "gpu_launches": int(L.launch_count() - n0), "clocks": clocks.summary(), "device_error": err}), flush=True)
    dist.destroy_process_group()


def run_extra(args):
    """`--workload decode|simple_gla_long|kda`: one JSON line for that workload on one GPU."""
    assert torch.cuda.is_available()
    torch.cuda.set_device(0)
    out = secondary(args.workload, args.steps, args.seq)
    out["n_gpus"] = 1
    print(json.dumps(out), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--scaling", default="strong", choices=["strong", "weak"],
                    help="N > 1: split the one batch of 8 sequences over the ranks (strong) or give every rank its own (weak)")
    ap.add_argument("--grads", default="primal", choices=["primal", "fp32"],
                    help="dtype of dq, dk, dg in the timed step: the primal dtypes (bf16) or fp32")
    ap.add_argument("--batch", type=int, default=0, help="override B (profiler captures on a smaller case)")
    ap.add_argument("--kernel-only", action="store_true", help="device-resident timed steps only, short JSON")
    ap.add_argument("--workload", default="gla_train", choices=["gla_train", "decode", "simple_gla_long", "kda", "kda_long", "neighbours"],
                    help="gla_train is the headline metric; the others are secondary one-GPU measurements")
    ap.add_argument("--seq", type=int, default=0, help="override T of a secondary workload")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    if args.gpus > 1 and "WORLD_SIZE" not in os.environ:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", os.environ.get("MASTER_PORT", "29517"),
               os.path.abspath(__file__), *sys.argv[1:]]
        sys.exit(subprocess.call(cmd))
    if args.impl == "reference":
        run_reference(args)
    elif args.workload in ("simple_gla_long", "kda_long") and int(os.environ.get("WORLD_SIZE", 1)) > 1:
        run_time_shard(args)
    elif args.workload != "gla_train":
        run_extra(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
