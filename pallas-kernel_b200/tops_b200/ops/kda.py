"""KDA (Kimi delta attention: per-channel decay plus a beta-weighted delta-rule
update) with the reference's signatures (`tops/ops/kda/chunk.py:193-216`,
`tops/ops/kda/fused_recurrent.py:19-105`; oracle `tops/cpu/ops/kda/naive.py`).

    S' = S exp(g_t);  e = v_t - k_t^T S';  S = S' + beta_t k_t (x) e;  o_t = scale q_t^T S

`g` is the natural-log decay `[B,T,H,K]`, `beta` `[B,T,H]`.  `chunk_kda` and
`fused_recurrent_kda` compute the same function; both are differentiable in
q, k, v, g, beta, initial_state.  The kernels behind them walk the tokens one
by one (the chunked WY form on the tensor cores is not built), so
`chunk_size` only has to be valid, it does not change the result.
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _lib as L


def _check(q, k, v, g, beta, initial_state):
    assert q.ndim == 4, f"q must be 4D [B,T,H,K], got {q.ndim}D"
    B, T, H, K = q.shape
    assert k.shape == q.shape, f"k shape {tuple(k.shape)} != q shape {tuple(q.shape)}"
    assert v.ndim == 4 and v.shape[:3] == q.shape[:3], f"v shape {tuple(v.shape)} incompatible with q"
    assert g.ndim == 4 and g.shape == q.shape, f"g shape {tuple(g.shape)} != q shape {tuple(q.shape)}"
    assert beta.ndim == 3 and beta.shape == q.shape[:3], f"beta shape {tuple(beta.shape)} != {tuple(q.shape[:3])}"
    assert k.dtype == q.dtype and v.dtype == q.dtype, "q, k, v must share a dtype"
    V = v.shape[-1]
    assert K <= 256, "K <= 256 (reference: tops/ops/common/chunk_delta_h.py:952)"
    if initial_state is not None:
        assert initial_state.shape == (B, H, K, V), \
            f"initial_state shape {tuple(initial_state.shape)} != ({B}, {H}, {K}, {V})"
    return B, T, H, K, V


def kda_fwd(q, k, v, g, beta, scale, initial_state, output_final_state):
    """One call of tops_b200_kda_fwd.  Returns (o in q.dtype, final state fp32 or None)."""
    B, T, H, K, V = _check(q, k, v, g, beta, initial_state)
    dev = q.device
    q, k, v, g = q.contiguous(), k.contiguous(), v.contiguous(), g.contiguous()
    beta = beta.to(q.dtype).contiguous()
    h0 = None if initial_state is None else initial_state.float().contiguous()
    o = torch.empty(B, T, H, V, dtype=q.dtype, device=dev)
    ht = torch.empty(B, H, K, V, dtype=torch.float32, device=dev) if output_final_state else None
    p = L.KdaFwdParams()
    p.B, p.T, p.H, p.K, p.V = B, T, H, K, V
    p.dtype, p.gate_dtype, p.scale = L.dtype_code(q.dtype), L.dtype_code(g.dtype), float(scale)
    p.q, p.k, p.v, p.g, p.beta = L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(g), L.ptr(beta)
    p.h0, p.o, p.ht = L.ptr(h0), L.ptr(o), L.ptr(ht)
    L.check(L.lib.tops_b200_kda_fwd(C.byref(p), L.stream_ptr(dev)), "kda_fwd")
    return o, ht


def kda_bwd(q, k, v, g, beta, do, scale, initial_state=None, dht=None):
    """Explicit backward (reference `tops/cpu/ops/kda/fused_recurrent.py:212-418`,
    `tops/cpu/ops/kda/chunk_bwd.py:525-668`).  Returns (dq, dk, dv, dg, dbeta in
    the input dtypes, dh0 fp32 or None — only when initial_state is given)."""
    B, T, H, K, V = _check(q, k, v, g, beta, initial_state)
    assert K <= 128 and V <= 128, "the KDA backward kernel takes K, V <= 128"
    dev = q.device
    q, k, v, g = q.contiguous(), k.contiguous(), v.contiguous(), g.contiguous()
    do = do.to(q.dtype).contiguous()
    beta_c = beta.to(q.dtype).contiguous()
    h0 = None if initial_state is None else initial_state.float().contiguous()
    dhtc = None if dht is None else dht.float().contiguous()
    dq, dk, dv, dg = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v), torch.empty_like(g)
    dbeta = torch.empty_like(beta_c)
    dh0 = torch.empty(B, H, K, V, dtype=torch.float32, device=dev) if h0 is not None else None
    p = L.KdaBwdParams()
    p.B, p.T, p.H, p.K, p.V = B, T, H, K, V
    p.dtype, p.gate_dtype, p.scale = L.dtype_code(q.dtype), L.dtype_code(g.dtype), float(scale)
    p.q, p.k, p.v, p.g, p.beta, p.h0 = L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(g), L.ptr(beta_c), L.ptr(h0)
    p.do_, p.dht = L.ptr(do), L.ptr(dhtc)
    p.dq, p.dk, p.dv, p.dg, p.dbeta, p.dh0 = L.ptr(dq), L.ptr(dk), L.ptr(dv), L.ptr(dg), L.ptr(dbeta), L.ptr(dh0)
    ws = L.workspace(L.lib.tops_b200_kda_bwd_workspace_bytes(C.byref(p)), dev)
    L.check(L.lib.tops_b200_kda_bwd(C.byref(p), ws.data_ptr(), ws.numel(), L.stream_ptr(dev)), "kda_bwd")
    return dq, dk, dv, dg, dbeta.to(beta.dtype), dh0


class _KDA(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, g, beta, initial_state, scale, output_final_state):
        o, ht = kda_fwd(q, k, v, g, beta, scale, initial_state, output_final_state)
        ctx.save_for_backward(q, k, v, g, beta, initial_state)
        ctx.scale = scale
        return o, ht

    @staticmethod
    def backward(ctx, do, dht):
        q, k, v, g, beta, h0 = ctx.saved_tensors
        dq, dk, dv, dg, dbeta, dh0 = kda_bwd(q, k, v, g, beta, do, ctx.scale, h0, dht)
        return dq, dk, dv, dg, dbeta, None if h0 is None else dh0.to(h0.dtype), None, None


def fused_recurrent_kda(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False):
    """Token-serial KDA (reference `tops/ops/kda/fused_recurrent.py:19-105`)."""
    B, T, H, K, V = _check(q, k, v, g, beta, initial_state)
    if scale is None:
        scale = K ** -0.5
    o, ht = _KDA.apply(q, k, v, g, beta, initial_state, float(scale), bool(output_final_state))
    return o, (ht if output_final_state else None)


def chunk_kda(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False, cu_seqlens=None,
              chunk_size=64):
    """Chunked KDA (reference `tops/ops/kda/chunk.py:193-216`): same function as
    `fused_recurrent_kda`.  T must be divisible by chunk_size, as upstream."""
    assert cu_seqlens is None, "packed KDA batches are not supported"
    assert chunk_size >= 1 and (chunk_size & (chunk_size - 1)) == 0, "chunk_size must be a power of 2"
    assert q.shape[1] % chunk_size == 0, f"T ({q.shape[1]}) must be divisible by chunk_size ({chunk_size})"
    return fused_recurrent_kda(q, k, v, g, beta, scale, initial_state, output_final_state)
