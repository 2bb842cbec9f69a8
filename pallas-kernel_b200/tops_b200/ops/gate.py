"""Gate activations next to the attention kernels, with the reference's names:

* `fused_kda_gate` / `kda_gate_fwd` / `kda_gate_bwd` / `kda_gate_chunk_cumsum`
  (`tops/cpu/ops/kda/gate.py:60-204`, accelerator `tops/ops/kda/gate.py:19-125`):
  `-exp(A_log) softplus(g + dt_bias)`, or with `lower_bound` the bounded form
  `lower_bound sigmoid(exp(A_log) (g + dt_bias))`;
* `gla_gate`: `log_sigmoid(g) / normalizer` with an optional lower clip, the gate of the GLA
  layer (`tops/layers/gla.py:277-279`).

All are differentiable (torch.autograd.Function over one forward and one backward kernel); `g` is
`[..., H, K]`, `A_log` `[H]`, `dt_bias` `[H*K]`.
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _lib as L


def _fill(p, g, H, K, kind, A_log, dt_bias, lower_bound, normalizer, clamp_min, out_dtype):
    p.rows, p.H, p.K, p.kind = g.numel() // (H * K), H, K, kind
    p.dtype, p.out_dtype = L.dtype_code(g.dtype), L.dtype_code(out_dtype)
    p.g, p.A_log, p.dt_bias = L.ptr(g), L.ptr(A_log), L.ptr(dt_bias)
    p.lower_bound = 0.0 if lower_bound is None else float(lower_bound)
    p.normalizer = float(normalizer)
    p.clamp_min = 0.0 if clamp_min is None else float(clamp_min)
    p.has_clamp_min = int(clamp_min is not None)


def _expand(A_log, dt_bias, H, K):
    """Head-wise parameters of fewer heads are repeated (`tops/cpu/ops/kda/gate.py:20-57`)."""
    assert A_log.ndim == 1, f"A_log must be 1D, got shape {tuple(A_log.shape)}"
    base = A_log.shape[0]
    assert H % base == 0, f"Effective heads {H} must be divisible by A_log heads {base}"
    A = A_log.float().repeat_interleave(H // base).contiguous()
    b = None
    if dt_bias is not None:
        assert dt_bias.ndim == 1 and dt_bias.shape[0] in (base * K, H * K), \
            f"dt_bias shape {tuple(dt_bias.shape)} incompatible with (base={base * K}, expanded={H * K})"
        b = dt_bias.float()
        if b.shape[0] != H * K:
            b = b.reshape(base, K).repeat_interleave(H // base, dim=0).reshape(-1)
        b = b.contiguous()
    return A, b


@L.on_tensor_device
def _gate_fwd_call(g, kind, A, b, lower_bound, normalizer, clamp_min, out_dtype):
    assert g.ndim >= 2, f"g must have at least 2 dims, got shape {tuple(g.shape)}"
    H, K = g.shape[-2:]
    assert K % 4 == 0, "K must be a multiple of 4"
    g = g.contiguous()
    out = torch.empty(g.shape, dtype=out_dtype, device=g.device)
    p = L.GateActParams()
    _fill(p, g, H, K, kind, A, b, lower_bound, normalizer, clamp_min, out_dtype)
    p.out = L.ptr(out)
    L.check(L.lib.tops_b200_gate_act_fwd(C.byref(p), L.stream_ptr(g.device)), "gate_act_fwd")
    return out


@L.on_tensor_device
def _gate_bwd_call(g, dy, kind, A, b, lower_bound, normalizer, clamp_min, want_params):
    H, K = g.shape[-2:]
    g, dy = g.contiguous(), dy.contiguous()
    dg = torch.empty_like(g)
    dA = torch.empty(H, dtype=torch.float32, device=g.device) if want_params else None
    db = torch.empty(H * K, dtype=torch.float32, device=g.device) if (want_params and b is not None) else None
    p = L.GateActBwdParams()
    _fill(p.fwd, g, H, K, kind, A, b, lower_bound, normalizer, clamp_min, g.dtype)
    p.dy, p.dy_dtype, p.dg, p.dA_log, p.dbias = L.ptr(dy), L.dtype_code(dy.dtype), L.ptr(dg), L.ptr(dA), L.ptr(db)
    ws = L.workspace(L.lib.tops_b200_gate_act_bwd_workspace_bytes(C.byref(p)), g.device)
    L.check(L.lib.tops_b200_gate_act_bwd(C.byref(p), ws.data_ptr(), ws.numel(), L.stream_ptr(g.device)), "gate_act_bwd")
    return dg, dA, db


def _kind(lower_bound):
    return L.GATE_ACT_KDA if lower_bound is None else L.GATE_ACT_KDA_LOWER_BOUND


def kda_gate_bwd(g, A_log, dt_bias=None, dyg=None, lower_bound=None):
    """Explicit backward (`tops/ops/kda/gate.py:54-125`): returns (dg in g.dtype, dA_log `[H]`,
    d dt_bias `[H*K]` or None) in the dtypes of the parameters."""
    assert dyg is not None, "dyg must be provided"
    H, K = g.shape[-2:]
    A, b = _expand(A_log, dt_bias, H, K)
    dg, dA, db = _gate_bwd_call(g, dyg, _kind(lower_bound), A, b, lower_bound, 1.0, None, True)
    base = A_log.shape[0]
    dA = dA.reshape(base, H // base).sum(1).to(A_log.dtype)
    if dt_bias is not None:
        if dt_bias.shape[0] != H * K:
            db = db.reshape(base, H // base, K).sum(1).reshape(-1)
        db = db.to(dt_bias.dtype)
    return dg, dA, db


class _KdaGate(torch.autograd.Function):
    @staticmethod
    def forward(ctx, g, A_log, dt_bias, lower_bound, out_dtype):
        H, K = g.shape[-2:]
        A, b = _expand(A_log, dt_bias, H, K)
        ctx.save_for_backward(g, A_log, dt_bias)
        ctx.lower_bound = lower_bound
        return _gate_fwd_call(g, _kind(lower_bound), A, b, lower_bound, 1.0, None, out_dtype)

    @staticmethod
    def backward(ctx, dy):
        g, A_log, dt_bias = ctx.saved_tensors
        dg, dA, db = kda_gate_bwd(g, A_log, dt_bias, dy, ctx.lower_bound)
        return dg, dA, db, None, None


def kda_gate_fwd(g, A_log, dt_bias=None, lower_bound=None, output_dtype=torch.float32):
    """KDA gate activation (`tops/cpu/ops/kda/gate.py:60-126`); differentiable in g, A_log, dt_bias."""
    return _KdaGate.apply(g, A_log, dt_bias, lower_bound, output_dtype)


fused_kda_gate = kda_gate_fwd


def kda_gate_chunk_cumsum(g, A_log, chunk_size, scale=None, dt_bias=None, cu_seqlens=None,
                          output_dtype=torch.float32, lower_bound=None):
    """Gate activation followed by the chunk-local cumulative sum (`tops/cpu/ops/kda/gate.py:182-203`);
    `scale` (1 / ln 2 for the log2-space kernels) multiplies the result."""
    from .common import chunk_local_cumsum
    assert cu_seqlens is None, "packed batches are not supported here"
    out = chunk_local_cumsum(kda_gate_fwd(g, A_log, dt_bias, lower_bound, torch.float32), chunk_size)
    if scale is not None:
        out = out * scale
    return out.to(output_dtype)


class _GlaGate(torch.autograd.Function):
    @staticmethod
    def forward(ctx, g, normalizer, clamp_min):
        ctx.save_for_backward(g)
        ctx.normalizer, ctx.clamp_min = normalizer, clamp_min
        return _gate_fwd_call(g, L.GATE_ACT_LOG_SIGMOID, None, None, None, normalizer, clamp_min, g.dtype)

    @staticmethod
    def backward(ctx, dy):
        (g,) = ctx.saved_tensors
        dg, _, _ = _gate_bwd_call(g, dy, L.GATE_ACT_LOG_SIGMOID, None, None, None, ctx.normalizer, ctx.clamp_min, False)
        return dg, None, None


def gla_gate(g, gate_logit_normalizer=16.0, clamp_min=None):
    """`log_sigmoid(g) / gate_logit_normalizer`, clipped from below by `clamp_min` when given: the gate
    of the GLA layer (`tops/layers/gla.py:277-279`), in g's dtype.  Differentiable."""
    return _GlaGate.apply(g, float(gate_logit_normalizer), clamp_min)
