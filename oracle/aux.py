"""Oracle for the steps either side of the attention path (test infrastructure only): the gate
activations of `tops/cpu/ops/kda/gate.py:60-126` and `tops/layers/gla.py:277-279`, the q/k L2
normalisation of `tops/cpu/ops/kda/fused_recurrent.py:14-18` and the gated RMS norm of
`tops/modules/fused_norm_gate.py:28-37`, in torch on the CPU (fp32 arithmetic, fp64 for fp64 inputs).
Gradients come from torch autograd, which is what the reference's `kda_gate_bwd` does with `jax.vjp`
(`tops/cpu/ops/kda/gate.py:129-178`)."""
from __future__ import annotations

import torch

from .common import acc_dtype


def _params(A_log, dt_bias, H, K, acc):
    base = A_log.shape[0]
    A = A_log.to(acc).repeat_interleave(H // base)
    b = None
    if dt_bias is not None:
        b = dt_bias.to(acc)
        b = b.reshape(H, K) if b.shape[0] == H * K else b.reshape(base, K).repeat_interleave(H // base, dim=0)
    return A, b


def kda_gate_fwd(g, A_log, dt_bias=None, lower_bound=None, output_dtype=torch.float32):
    H, K = g.shape[-2:]
    acc = acc_dtype(g.dtype)
    A, b = _params(A_log, dt_bias, H, K, acc)
    x = g.to(acc)
    if b is not None:
        x = x + b
    if lower_bound is None:
        y = -torch.exp(A).reshape(H, 1) * torch.nn.functional.softplus(x)
    else:
        y = lower_bound * torch.sigmoid(torch.exp(A).reshape(H, 1) * x)
    return y.to(output_dtype)


def gla_gate(g, normalizer=16.0, clamp_min=None):
    acc = acc_dtype(g.dtype)
    y = torch.nn.functional.logsigmoid(g.to(acc)) / normalizer
    if clamp_min is not None:
        y = torch.clamp(y, min=clamp_min)
    return y.to(g.dtype)


def l2norm(x, eps=1e-6):
    acc = acc_dtype(x.dtype)
    xf = x.to(acc)
    return (xf / torch.sqrt((xf * xf).sum(-1, keepdim=True) + eps)).to(x.dtype)


def rmsnorm_gated(x, g, weight=None, eps=1e-5):
    acc = acc_dtype(x.dtype)
    xf, gf = x.to(acc), g.to(acc)
    y = xf * torch.rsqrt((xf * xf).mean(-1, keepdim=True) + eps)
    if weight is not None:
        y = y * weight.to(acc)
    return (y * torch.nn.functional.silu(gf)).to(x.dtype)
