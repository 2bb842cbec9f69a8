"""Seeded synthetic inputs with the shapes and value distributions of the
benchmark configurations (the reference measures on synthetic data only:
`benchmarks/ops/benchmark_gla.py`, `tests/ref/gla/test_chunk_gla.py:312-317`).

Draws are made on the host with `numpy.random.Generator(PCG64(seed))` in fp32
and then cast, so a CPU computation and the GPU kernels see identical values.
Sub-streams are drawn in the fixed order q, k, v, g, beta, h0, do, dht.
"""
from __future__ import annotations

import numpy as np
import torch


def _log_sigmoid(x):
    return -np.logaddexp(0.0, -x)


def make_inputs(seed, B, T, H, K, V, dtype=torch.float32, gate="per_channel", gate_norm=16.0,
                with_h0=False, with_grads=False, with_beta=False, l2norm_qk=False, gate_dtype=None):
    """Return a dict of CPU tensors: q, k, v `[B,T,H,K|V]` ~ N(0,1) in `dtype`;
    g = log_sigmoid(N(0,1)) / gate_norm, `[B,T,H,K]` (per_channel) or `[B,T,H]`
    (scalar), in `gate_dtype` (default `dtype`); optional beta = sigmoid(N(0,1))
    `[B,T,H]`; h0 ~ 0.1 N(0,1) fp32 `[B,H,K,V]`; do ~ N(0,1); dht ~ 0.1 N(0,1)."""
    rng = np.random.Generator(np.random.PCG64(seed))

    def normal(*shape):
        return rng.standard_normal(shape, dtype=np.float32)

    q, k, v = normal(B, T, H, K), normal(B, T, H, K), normal(B, T, H, V)
    gshape = (B, T, H, K) if gate == "per_channel" else (B, T, H)
    g = (_log_sigmoid(normal(*gshape).astype(np.float64)) / gate_norm).astype(np.float32)
    beta = 1.0 / (1.0 + np.exp(-normal(B, T, H))) if with_beta else None
    h0 = 0.1 * normal(B, H, K, V) if with_h0 else None
    do = normal(B, T, H, V) if with_grads else None
    dht = 0.1 * normal(B, H, K, V) if with_grads else None
    if l2norm_qk:
        q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6)
        k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    gd = dtype if gate_dtype is None else gate_dtype
    out = {
        "q": torch.from_numpy(q).to(dtype), "k": torch.from_numpy(k).to(dtype),
        "v": torch.from_numpy(v).to(dtype), "g": torch.from_numpy(g).to(gd),
    }
    if beta is not None:
        out["beta"] = torch.from_numpy(beta.astype(np.float32)).to(dtype)
    if h0 is not None:
        out["h0"] = torch.from_numpy(h0.astype(np.float32))
    if do is not None:
        out["do"] = torch.from_numpy(do).to(dtype)
        out["dht"] = torch.from_numpy(dht.astype(np.float32))
    return out
