"""simple_gla ops (one scalar log-gate per head and token `g:[B,T,H]`, or a
constant per-head decay `g_gamma:[H]`) with the reference's signatures
(`tops/ops/simple_gla/__init__.py:15-158`, oracle `tops/cpu/ops/simple_gla/chunk.py`).

Unlike the reference's accelerator path, which only takes `g_gamma` in the
chunked modes (`tops/ops/simple_gla/__init__.py:93-97`), the chunked kernels
here also take the per-token gate `g` and return its gradient.
"""
from __future__ import annotations

import torch

from .. import _lib as L
from ._chunk import chunk_bwd_call, chunk_fwd_call
from .gla import fused_recurrent_gla


def _check(q, k, v, g, g_gamma, initial_state, cu_seqlens):
    assert q.ndim == 4, f"q must be 4D [B,T,H,K], got {q.ndim}D"
    B, T, H, K = q.shape
    assert k.shape == q.shape, f"k shape {tuple(k.shape)} != q shape {tuple(q.shape)}"
    assert v.ndim == 4 and v.shape[:3] == q.shape[:3], f"v shape {tuple(v.shape)} incompatible with q"
    assert k.dtype == q.dtype and v.dtype == q.dtype, "q, k, v must share a dtype"
    if g is not None:
        assert g.ndim == 3 and g.shape == q.shape[:3], f"g shape {tuple(g.shape)} != {tuple(q.shape[:3])}"
    if g_gamma is not None:
        assert g_gamma.ndim == 1 and g_gamma.shape[0] == H, f"g_gamma shape {tuple(g_gamma.shape)} != (H={H},)"
    assert not (g is not None and g_gamma is not None), \
        "use only one of g or g_gamma (the reference's backward rejects both together)"
    N = B
    if cu_seqlens is not None:
        assert B == 1, f"B must be 1 for varlen, got {B}"
        cu = [int(x) for x in cu_seqlens]
        N = len(cu) - 1
        assert all(b > a for a, b in zip(cu[:-1], cu[1:])), "Empty segments not supported"
    if initial_state is not None:
        assert initial_state.shape == (N, H, K, v.shape[-1]), \
            f"initial_state shape {tuple(initial_state.shape)} != ({N}, {H}, {K}, {v.shape[-1]})"
    return K


def _gate(g, g_gamma):
    if g is not None:
        return g, L.GATE_SCALAR
    if g_gamma is not None:
        return g_gamma, L.GATE_GAMMA
    return None, L.GATE_NONE


def _cu(cu_seqlens):
    return None if cu_seqlens is None else [int(x) for x in cu_seqlens]


def _kernel_chunk(chunk_size):
    """The chunk length the kernels run with.  Neither (o, ht) nor the gradients depend on it beyond where
    roundings fall, and the orchestrators of this family hand no chunk-shaped tensor to the caller: the kernels
    hold chunks of 16, 32 or 64 time steps, other powers of two (the reference's tests use 128) run with the
    nearest."""
    assert chunk_size >= 1 and (chunk_size & (chunk_size - 1)) == 0, \
        f"chunk_size must be a power of 2, got {chunk_size}"   # tops/ops/common/cumsum.py:506-508
    return min(max(int(chunk_size), 16), 64)


def _fwd(q, k, v, g, g_gamma, scale, initial_state, output_final_state, chunk_size, cu_seqlens, want_saved):
    _check(q, k, v, g, g_gamma, initial_state, cu_seqlens)
    gate, kind = _gate(g, g_gamma)
    chunk_size = _kernel_chunk(chunk_size)
    o, ht, _, _, saved = chunk_fwd_call(q, k, v, gate, kind, scale, initial_state, output_final_state, chunk_size,
                                        _cu(cu_seqlens), want_saved=want_saved)
    return o, ht, saved


def chunk_simple_gla_fwd(q, k, v, g, g_gamma, scale, initial_state, output_final_state, chunk_size=64,
                         cu_seqlens=None):
    """Forward orchestrator (reference `tops/cpu/ops/simple_gla/chunk.py:53-129`).
    Returns (o in v.dtype, ht fp32 or None)."""
    o, ht, _ = _fwd(q, k, v, g, g_gamma, scale, initial_state, output_final_state, chunk_size, cu_seqlens, False)
    return o, ht


def chunk_simple_gla_bwd(q, k, v, g, g_gamma, initial_state, do, dht, scale, chunk_size=64, cu_seqlens=None,
                         h_saved=None):
    """Backward orchestrator (reference `tops/cpu/ops/simple_gla/chunk.py:668-788`).
    Returns (dq, dk in the input dtype, dv in do.dtype, dg fp32 `[B,T,H]` or
    None, dh0 fp32 or None).  `h_saved`: the chunk-start states the tcgen05
    forward kept (None recomputes them, as the reference does)."""
    _check(q, k, v, g, g_gamma, initial_state, cu_seqlens)
    gate, kind = _gate(g, g_gamma)
    return chunk_bwd_call(q, k, v, gate, kind, scale, initial_state, do, dht, _kernel_chunk(chunk_size), q.dtype,
                          g is not None, initial_state is not None, _cu(cu_seqlens), h_saved=h_saved)


class _ChunkSimpleGLA(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, g, g_gamma, initial_state, scale, output_final_state, cu, chunk_size):
        keep = any(t is not None and t.requires_grad for t in (q, k, v, g, initial_state))
        o, ht, hs = _fwd(q, k, v, g, g_gamma, scale, initial_state, output_final_state, chunk_size, cu, keep)
        ctx.save_for_backward(q, k, v, g, g_gamma, initial_state, hs)
        ctx.scale, ctx.cu, ctx.chunk = scale, cu, chunk_size
        return o, ht

    @staticmethod
    def backward(ctx, do, dht):
        q, k, v, g, g_gamma, h0, hs = ctx.saved_tensors
        dq, dk, dv, dg, dh0 = chunk_simple_gla_bwd(q, k, v, g, g_gamma, h0, do.to(q.dtype), dht, ctx.scale, ctx.chunk,
                                                   ctx.cu, h_saved=hs)
        # a constant decay gets a zero cotangent, as in the reference (tops/ops/simple_gla/chunk.py:764)
        if L.CHECK_DEVICE:
            L.raise_on_device_error("chunk_simple_gla backward")
        dgamma = None if g_gamma is None else torch.zeros_like(g_gamma)
        return (dq, dk, dv, None if g is None else dg.to(g.dtype), dgamma,
                None if h0 is None else dh0.to(h0.dtype), None, None, None, None)


def chunk_simple_gla(q, k, v, g=None, g_gamma=None, scale=None, initial_state=None, output_final_state=False,
                     cu_seqlens=None, chunk_size=64):
    """Chunked simple_gla (reference `tops/cpu/ops/simple_gla/chunk.py:796-889`;
    custom_vjp form `tops/ops/simple_gla/chunk.py:778-827`).  Differentiable in
    q, k, v, g, initial_state.  Returns (o in v.dtype, final state fp32 or None)."""
    K = _check(q, k, v, g, g_gamma, initial_state, cu_seqlens)
    if scale is None:
        scale = K ** -0.5
    if initial_state is not None:
        initial_state = initial_state.to(torch.float32)
    chunk_size = _kernel_chunk(chunk_size)
    o, ht = _ChunkSimpleGLA.apply(q, k, v, g, g_gamma, initial_state, float(scale), bool(output_final_state),
                                  _cu(cu_seqlens), int(chunk_size))
    return o, (ht if output_final_state else None)


def fused_chunk_simple_gla(q, k, v, g_gamma=None, initial_state=None, scale=None, output_final_state=False,
                           chunk_size=64, g=None):
    """Same computation as `chunk_simple_gla` (reference
    `tops/ops/simple_gla/fused_chunk.py:503-555` keeps the state on chip; the
    kernels here make that choice internally)."""
    return chunk_simple_gla(q, k, v, g, g_gamma, scale, initial_state, output_final_state, None, chunk_size)


def fused_recurrent_simple_gla(q, k, v, g=None, g_gamma=None, scale=None, initial_state=None,
                               output_final_state=False, reverse=False, cu_seqlens=None):
    """Token-serial simple_gla (reference `tops/ops/simple_gla/fused_recurrent.py:146-240`,
    oracle `tops/cpu/ops/simple_gla/fused_recurrent.py:35-162`): decay
    exp(g_t + g_gamma) on the whole state.  Runs the recurrent GLA kernel with
    the scalar log-gate replicated over K."""
    B, T, H, K = q.shape
    gk = None
    if g is not None or g_gamma is not None:
        tot = torch.zeros(B, T, H, dtype=torch.float32, device=q.device)
        if g is not None:
            tot = tot + g.float()
        if g_gamma is not None:
            tot = tot + g_gamma.float().view(1, 1, H)
        gk = tot.unsqueeze(-1).expand(B, T, H, K).contiguous()
    return fused_recurrent_gla(q, k, v, gk=gk, scale=scale, initial_state=initial_state,
                               output_final_state=output_final_state, reverse=reverse, cu_seqlens=cu_seqlens)


def simple_gla(q, k, v, *args, g=None, g_gamma=None, scale=None, initial_state=None, output_final_state=False,
               chunk_size=64, reverse=False, cu_seqlens_cpu=None, mode="chunk", **kwargs):
    """Unified front door (reference `tops/ops/simple_gla/__init__.py:15-158`).
    `chunk` / `fused_chunk` reject `reverse`; all modes but `naive` exist."""
    assert not args and not kwargs, "unexpected arguments"
    if mode in ("chunk", "fused_chunk"):
        if reverse:
            raise ValueError(f"mode={mode!r} does not support `reverse`")
        return chunk_simple_gla(q, k, v, g, g_gamma, scale, initial_state, output_final_state, cu_seqlens_cpu,
                                chunk_size)
    if mode == "fused_recurrent":
        return fused_recurrent_simple_gla(q, k, v, g=g, g_gamma=g_gamma, scale=scale, initial_state=initial_state,
                                          output_final_state=output_final_state, reverse=reverse,
                                          cu_seqlens=cu_seqlens_cpu)
    raise ValueError(f"Unknown mode {mode!r}; expected one of 'chunk', 'fused_chunk', 'fused_recurrent'")
