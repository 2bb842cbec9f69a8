#!/usr/bin/env python
"""Benchmark of the chunked GLA hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]
                    [--workload gla_train|decode|simple_gla_long|kda]

One "step" is one forward + backward pass of `chunk_gla` over one synthetic
batch of the headline configuration (bf16, B=8, T=4096, H=16, K=V=128,
chunk 64, initial state and final-state gradient included).  Prints ONE JSON
line (rank 0).  Under torchrun every rank processes its own batch of the same
size (batch x heads shard with no communication: weak scaling).

  value      tokens/s with inputs resident in HBM (CUDA events, max over ranks)
  e2e        the same metric with host buffers: pinned host -> device copies of
             every input and device -> host copies of every output inside the
             timed region
  roofline   the dominant kernel: algorithmic bytes per launch / its average
             launch duration (CUDA events recorded by the library around each
             launch during the timed steps) against the measured HBM peak
  cpu_baseline  the CPU oracle (a torch-CPU port of the reference's tops.cpu
             implementation) on a bounded sample, timed on this box's cores

`--impl reference` times that CPU port alone (the reference itself is pure
JAX and cannot be installed without network access).
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

WORKLOADS = {
    # BASELINE.json configs[1]
    "gla_train": dict(B=8, T=4096, H=16, K=128, V=128, C=64, dtype="bfloat16", seed=2),
    # BASELINE.json configs[2]: one decode token per call, state updated in place
    "decode": dict(B=128, T=1, H=32, K=128, V=128, dtype="bfloat16", seed=3),
}

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
            self._stop.wait(0.05)

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
                "reasons": sorted(self.reasons)}


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


def kernel_bytes(label, w, grad_bytes=4):
    """Algorithmic bytes one launch of a kernel must move for the gla_train
    workload: every operand it needs read once, every result written once."""
    tok = w["B"] * w["T"] * w["H"]
    K, V, C = w["K"], w["V"], w["C"]
    nchunk = tok // C
    in2 = 2  # bf16
    state = nchunk * K * V            # elements of one [B,NT,H,K,V] tensor
    bhkv = w["B"] * w["H"] * K * V
    t = {
        "generic_cumsum": tok * K * (in2 + 4),
        "generic_scan_h": tok * (K + V) * in2 + tok * K * 4 + state * 4 + bhkv * 4,
        "generic_scan_dh": tok * (K + V) * in2 + tok * K * 4 + state * 4 + 2 * bhkv * 4,
        "generic_fwd_o": tok * (2 * K + 2 * V) * in2 + tok * K * 4 + state * in2,
        "generic_bwd_A": tok * (2 * K + 2 * V) * in2 + tok * K * 4 + 2 * tok * C * 4,
        "generic_bwd_dv": tok * (K + 2 * V) * in2 + tok * K * 4 + tok * C * 4 + state * 4,
        "generic_bwd_dqkg": tok * (2 * K + 2 * V) * in2 + tok * K * 4 + tok * C * 4 + 2 * state * 4 + 3 * tok * K * 4,
        # tcgen05 path
        "sm100_fwd_h": tok * (K + V + K) * in2 + state * in2 + 2 * bhkv * 4,
        "sm100_fwd_o": tok * (3 * K + 2 * V) * in2 + state * in2,
        "sm100_fwd_fused": tok * (3 * K + 2 * V) * in2 + state * in2 + 2 * bhkv * 4,
        "sm100_bwd_dh": tok * (K + V + K) * in2 + state * in2 + 2 * bhkv * 4,
        "sm100_bwd_main": tok * (3 * K + 2 * V) * in2 + 2 * state * in2 + 3 * tok * K * grad_bytes + tok * V * in2,
    }
    return t.get(label)


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
    from tops_b200.synth import make_inputs

    w = dict(WORKLOADS["gla_train"])
    if args.batch:
        w["B"] = args.batch      # smaller batches are for profiler captures only
    dtype = getattr(torch, w["dtype"])
    scale = w["K"] ** -0.5
    host = make_inputs(w["seed"] + 1000 * rank, w["B"], w["T"], w["H"], w["K"], w["V"], dtype=dtype,
                       with_h0=True, with_grads=True)
    names = ("q", "k", "v", "g", "do", "h0", "dht")
    pinned = {n: host[n].pin_memory() for n in names}
    x = {n: pinned[n].to(dev) for n in names}

    # "primal": dq, dk, dg come back in the dtypes of q, k, g (bf16), as the differentiable op returns
    # them and as the reference's accelerator kernel writes them; "fp32": as the reference's CPU
    # orchestrator returns them
    primal = args.grads == "primal"
    grad_bytes = 2 if primal else 4

    def step(t):
        # the forward keeps its chunk-start states for the backward (what the differentiable op does)
        o, ht, _, _, hs = chunk_fwd_call(t["q"], t["k"], t["v"], t["g"], L.GATE_PER_CHANNEL, scale, t["h0"], True, w["C"],
                                         want_saved=True)
        dq, dk, dv, dg, dh0 = chunk_bwd_call(t["q"], t["k"], t["v"], t["g"], L.GATE_PER_CHANNEL, scale, t["h0"],
                                             t["do"], t["dht"], w["C"], torch.float32, True, True, h_saved=hs,
                                             primal_dtypes=primal)
        return o, ht, dq, dk, dv, dg, dh0

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, drain=None):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        if drain is not None:
            drain()      # side streams join the timed stream before the closing event
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1) / steps
        if world > 1:
            tms = torch.tensor([ms], device=dev)
            torch.distributed.all_reduce(tms, op=torch.distributed.ReduceOp.MAX)
            ms = float(tms.item())
        return ms

    # ---- device-resident throughput ------------------------------------------------
    for _ in range(args.warmup):
        step(x)
    L.lib.tops_b200_profile_enable(1)
    launches0 = L.launch_count()
    with ClockSampler(local_rank) as clocks:
        ms = timed(lambda: step(x), args.steps)
    launches = L.launch_count() - launches0
    L.lib.tops_b200_profile_enable(0)
    buf = ctypes.create_string_buffer(1 << 16)
    L.lib.tops_b200_profile_read(buf, len(buf))
    kernels = {}
    for line in buf.value.decode().splitlines():
        label, count, total = line.split()
        kernels[label] = (int(count), float(total))

    if args.kernel_only:
        if rank == 0:
            print(json.dumps({"kernel_only": True, "batch": w["B"], "ms_per_step": ms,
                              "kernels_ms_per_launch": {k: v[1] / v[0] for k, v in sorted(kernels.items())}}), flush=True)
        return

    # ---- end to end: host buffers in, host buffers out --------------------------------
    # Every step copies its inputs from pinned host memory and its results back to pinned host
    # memory.  Three streams and two buffer sets let the upload of step i+1, the kernels of step i
    # and the download of step i-1 overlap (PCIe is full duplex); each step's copies and kernels
    # still all run inside the timed region.
    outs = step(x)
    out_host = [[torch.empty(o.shape, dtype=o.dtype).pin_memory() for o in outs] for _ in range(2)]
    dev_in = [{n: torch.empty_like(x[n]) for n in names} for _ in range(2)]
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    uploaded = [torch.cuda.Event() for _ in range(2)]
    computed = [torch.cuda.Event() for _ in range(2)]
    counter = [0]

    def e2e_step():
        slot = counter[0] & 1
        counter[0] += 1
        cur = torch.cuda.current_stream()
        s_in.wait_event(computed[slot])          # the kernels of two steps ago have read this input set
        with torch.cuda.stream(s_in):
            for n in names:
                dev_in[slot][n].copy_(pinned[n], non_blocking=True)
            uploaded[slot].record(s_in)
        cur.wait_event(uploaded[slot])
        res = step(dev_in[slot])
        computed[slot].record(cur)
        s_out.wait_event(computed[slot])
        with torch.cuda.stream(s_out):
            for dst, src in zip(out_host[slot], res):
                dst.copy_(src, non_blocking=True)
                src.record_stream(s_out)

    def e2e_drain():
        torch.cuda.current_stream().wait_stream(s_out)

    e2e_steps = max(3, min(args.steps, 10))
    for _ in range(2):
        e2e_step()
    ms_e2e = timed(e2e_step, e2e_steps, e2e_drain)
    h2d = sum(pinned[n].numel() * pinned[n].element_size() for n in names)
    d2h = sum(o.numel() * o.element_size() for o in out_host[0])

    tokens = w["B"] * w["T"] * world
    hbm_peak, tf_peak, peak_kind = measured_peaks()
    result = {
        "metric": "chunk_gla fwd+bwd tokens/sec (bf16, T=4096,H=16,D=128)",
        "value": tokens / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"chunk_gla fwd+bwd, B={w['B']} per GPU, T=4096, H=16, K=V=128, chunk 64, h0+dht (BASELINE configs[1])",
                   "grads": "dq, dk, dg in bf16 (the primal dtypes)" if primal else "dq, dk, dg in fp32",
                   "global_batch": w["B"] * world, "seq_len": w["T"], "parallelism": f"batch x heads shard x{world}, no communication",
                   "l2": "inputs (671 MB) and outputs are larger than L2; no flush needed"},
        "e2e": {"value": tokens / (ms_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": ms_e2e, "steps": e2e_steps,
                "pipeline": "upload of step i+1, kernels of step i and download of step i-1 overlap (3 streams)"},
        "gpu_launches": int(launches),
        "clocks": clocks.summary(),
    }
    # whole-step view against both roofs
    th = w["B"] * w["T"] * w["H"]
    GLA_TRAIN_BYTES_PER_TOKEN_HEAD = gla_train_bytes_per_token_head(grad_bytes)
    result["step_roofline"] = {
        "hbm_frac": th * GLA_TRAIN_BYTES_PER_TOKEN_HEAD / (ms * 1e-3) / (hbm_peak * 1e9),
        "tensor_frac": th * GLA_TRAIN_FLOP_PER_TOKEN_HEAD / (ms * 1e-3) / (tf_peak * 1e12),
        "bytes_per_token_head": GLA_TRAIN_BYTES_PER_TOKEN_HEAD, "flop_per_token_head": GLA_TRAIN_FLOP_PER_TOKEN_HEAD,
        "peaks": peak_kind}
    if kernels:
        top = max(kernels, key=lambda k: kernels[k][1])
        count, total = kernels[top]
        per_launch_ms = total / count
        nbytes = kernel_bytes(top, w, grad_bytes)
        achieved = None if nbytes is None else nbytes / (per_launch_ms * 1e-3) / 1e9
        traffic = None
        tpath = os.path.join(ROOT, "profiles", "traffic.json")
        if os.path.exists(tpath):
            tj = json.load(open(tpath))
            traffic = tj.get(top if primal else top + "_fp32", tj.get(top)) if w["B"] == 8 else None
        result["roofline"] = {"bound": "hbm", "kernel": top, "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                              "frac": None if achieved is None else achieved / hbm_peak, "traffic": traffic,
                              "ms_per_launch": per_launch_ms, "peak_source": peak_kind,
                              "kernels_ms_per_step": {k: v[1] / args.steps for k, v in sorted(kernels.items())}}
    if rank == 0 and world == 1:
        result["cpu_baseline"] = cpu_baseline(sample_B=8, passes=4)
    if rank == 0:
        print(json.dumps(result), flush=True)
    if world > 1:
        torch.distributed.destroy_process_group()


def cpu_baseline(sample_B, passes, warm=1):
    """The oracle (torch-CPU port of tops.cpu chunk_gla / chunk_gla_bwd) on a
    batch slice of the workload, all host threads."""
    from oracle import gla as G
    from tops_b200.synth import make_inputs
    # torchrun exports OMP_NUM_THREADS=1; the CPU arm uses every host core
    try:
        torch.set_num_threads(len(os.sched_getaffinity(0)))
    except Exception:
        torch.set_num_threads(os.cpu_count() or 1)
    w = WORKLOADS["gla_train"]
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
    for _ in range(passes):
        one()
    dt = (time.perf_counter() - t0) / passes
    return {"value": sample_B * w["T"] / dt, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"fwd+bwd of a B={sample_B} slice of the workload (T=4096, H=16, K=V=128), {passes} timed passes",
            "seconds_per_pass": dt}


def run_reference(args):
    rank, _, world = dist_env()
    if rank != 0:
        return
    w = WORKLOADS["gla_train"]
    sample_B = 1
    cb = cpu_baseline(sample_B, passes=max(1, args.steps), warm=max(1, min(args.warmup, 2)))
    ms = cb["seconds_per_pass"] * 1e3
    line = {
        "impl": "reference", "metric": "chunk_gla fwd+bwd tokens/sec (bf16, T=4096,H=16,D=128)",
        "value": cb["value"], "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": "chunk_gla fwd+bwd, T=4096, H=16, K=V=128, chunk 64, h0+dht (BASELINE configs[1]); "
                               f"each step is a B={sample_B} slice on the host cores",
                   "global_batch": sample_B, "seq_len": w["T"], "parallelism": "cpu"},
        "cpu_baseline": {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": cb["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "CPU port of the reference's tops.cpu (the reference is pure JAX; JAX is not installable offline)",
    }
    print(json.dumps(line), flush=True)


def run_extra(args):
    """Secondary workloads (BASELINE configs[2..4]) on one GPU: device-resident timing, one JSON line."""
    assert torch.cuda.is_available()
    torch.cuda.set_device(0)
    from tops_b200 import _lib as L
    from tops_b200.synth import make_inputs

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    hbm_peak, _, peak_kind = measured_peaks()
    n0 = L.launch_count()
    if args.workload == "decode":
        from tops_b200.ops.gla import fused_recurrent_gla_decode_
        B, H, K, V = 128, 32, 128, 128
        x = {k: v.cuda() for k, v in make_inputs(3, B, 1, H, K, V, dtype=torch.bfloat16, with_h0=True).items()}
        state = x["h0"].clone()
        ms = timed(lambda: fused_recurrent_gla_decode_(x["q"], x["k"], x["v"], x["g"], state), max(args.steps, 200), 20)
        nbytes = 2 * B * H * K * V * 4
        out = {"metric": "fused_recurrent_gla decode GB/s (state read+write)", "value": nbytes / (ms * 1e-3) / 1e9,
               "unit": "GB/s", "ms_per_step": ms, "config": {"workload": "decode B=128 H=32 K=V=128, 1 token per call, fp32 state in place"},
               "roofline": {"bound": "hbm", "achieved": nbytes / (ms * 1e-3) / 1e9, "peak": hbm_peak, "unit": "GB/s",
                            "frac": nbytes / (ms * 1e-3) / 1e9 / hbm_peak, "peak_source": peak_kind}}
    elif args.workload == "simple_gla_long":
        from tops_b200.ops.simple_gla import _fwd as simple_gla_fwd_keep, chunk_simple_gla_bwd
        B, T, H, K, V = 1, args.seq or 65536, 32, 128, 128
        x = {k: v.cuda() for k, v in make_inputs(4, B, T, H, K, V, dtype=torch.bfloat16, gate="scalar", with_h0=True,
                                                   with_grads=True).items()}
        sc = K ** -0.5

        def step():
            # what the differentiable op does: the forward keeps its chunk-start states for the backward
            _, _, hs = simple_gla_fwd_keep(x["q"], x["k"], x["v"], x["g"], None, sc, x["h0"], True, 64, None, True)
            chunk_simple_gla_bwd(x["q"], x["k"], x["v"], x["g"], None, x["h0"], x["do"], x["dht"], sc, 64, h_saved=hs)
        ms = timed(step, args.steps, 2)
        out = {"metric": "simple_gla chunk fwd+bwd tokens/s", "value": B * T / (ms * 1e-3), "unit": "tokens/s", "ms_per_step": ms,
               "config": {"workload": f"simple_gla B=1 T={T} H=32 K=V=128 chunk 64 bf16 (bf16 gate), one GPU"}}
    else:
        from tops_b200.ops.kda import kda_bwd, kda_fwd
        B, T, H, K, V = 4, args.seq or 8192, 32, 128, 128
        x = {k: v.cuda() for k, v in make_inputs(5, B, T, H, K, V, dtype=torch.bfloat16, with_h0=True, with_grads=True,
                                                   with_beta=True, l2norm_qk=True).items()}
        sc = K ** -0.5

        def step():
            kda_fwd(x["q"], x["k"], x["v"], x["g"], x["beta"], sc, x["h0"], True)
            kda_bwd(x["q"], x["k"], x["v"], x["g"], x["beta"], x["do"], sc, x["h0"], x["dht"])
        ms = timed(step, min(args.steps, 3), 1)
        out = {"metric": "KDA fwd+bwd tokens/s", "value": B * T / (ms * 1e-3), "unit": "tokens/s", "ms_per_step": ms,
               "config": {"workload": f"KDA B=4 T={T} H=32 K=V=128 bf16, one GPU (token-serial kernels)"}}
    out["gpu_launches"] = L.launch_count() - n0
    out["n_gpus"] = 1
    print(json.dumps(out), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--grads", default="primal", choices=["primal", "fp32"],
                    help="dtype of dq, dk, dg in the timed step: the primal dtypes (bf16) or fp32")
    ap.add_argument("--batch", type=int, default=0, help="override B (profiler captures on a smaller case)")
    ap.add_argument("--kernel-only", action="store_true", help="device-resident timed steps only, short JSON")
    ap.add_argument("--workload", default="gla_train", choices=["gla_train", "decode", "simple_gla_long", "kda"],
                    help="gla_train is the headline metric; the others are secondary one-GPU measurements")
    ap.add_argument("--seq", type=int, default=0, help="override T of a secondary workload")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    if args.gpus > 1 and "WORLD_SIZE" not in os.environ:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", os.environ.get("MASTER_PORT", "29517"),
               os.path.abspath(__file__), *sys.argv[1:]]
        sys.exit(subprocess.call(cmd))
    if args.workload != "gla_train":
        run_extra(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
