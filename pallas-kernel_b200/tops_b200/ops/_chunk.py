"""Calls of the fused chunked forward / backward entry points shared by the
GLA (per-channel gate) and simple_gla (scalar / constant gate) front-ends."""
from __future__ import annotations

import ctypes as C

import torch

from .. import _lib as L
from .common import make_problem, total_chunks


@L.on_tensor_device
def chunk_fwd_call(q, k, v, gate, gate_kind, scale, h0, want_ht, chunk, cu_seqlens=None,
                   want_gcum=False, want_A=False, want_h=False, impl=L.IMPL_AUTO, want_saved=False, segments=None):
    """Run tops_b200_chunk_gla_fwd.  Returns (o, ht, g_cumsum, A, h); the last
    three are None unless asked for.  With `want_saved` the fifth value is
    instead the opaque scratch the tcgen05 forward keeps for its backward
    (None when another kernel family runs): pass it to chunk_bwd_call as `h_saved`.  `segments`: the
    workspace of a state-exchange pack call on the same problem (time sharding), see the C header."""
    B, T, H, K = q.shape
    V = v.shape[-1]
    dev = q.device
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    gate = None if gate is None else gate.contiguous()
    if gate_kind == L.GATE_GAMMA:
        gate = gate.float().contiguous()
    h0 = None if h0 is None else h0.float().contiguous()
    N = B if cu_seqlens is None else len(cu_seqlens) - 1
    o = torch.empty(B, T, H, V, dtype=v.dtype, device=dev)
    ht = torch.empty(N, H, K, V, dtype=torch.float32, device=dev) if want_ht else None
    gcum = torch.empty(gate.shape, dtype=torch.float32, device=dev) \
        if (want_gcum and gate_kind in (L.GATE_PER_CHANNEL, L.GATE_SCALAR)) else None
    A = torch.zeros(B, T, H, chunk, dtype=torch.float32, device=dev) if want_A else None
    nch = total_chunks(B, T, chunk, cu_seqlens)
    hs = torch.empty(1 if cu_seqlens is not None else B, nch // (1 if cu_seqlens is not None else B), H, K, V,
                     dtype=k.dtype, device=dev) if want_h else None
    keep = []
    p = L.ChunkFwdParams()
    p.pb = make_problem(B, T, H, K, V, chunk, L.dtype_code(q.dtype),
                        L.F32 if gate is None else L.dtype_code(gate.dtype), gate_kind, scale, impl,
                        cu_seqlens, keep)
    p.q, p.k, p.v, p.g, p.h0, p.o, p.ht = L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(gate), L.ptr(h0), L.ptr(o), L.ptr(ht)
    p.g_cumsum_out, p.A_out, p.h_out = L.ptr(gcum), L.ptr(A), L.ptr(hs)
    if want_saved and not (want_gcum or want_A or want_h) \
            and L.lib.tops_b200_chunk_selected_impl(C.byref(p.pb)) == L.IMPL_SM100:
        hs = torch.empty(B, nch // B, H, K, V, dtype=k.dtype, device=dev)
        p.saved_out = L.ptr(hs)
    if segments is not None and L.lib.tops_b200_chunk_selected_impl(C.byref(p.pb)) == L.IMPL_SM100:
        p.segments = L.ptr(segments)
    ws = L.workspace(L.lib.tops_b200_chunk_fwd_workspace_bytes(C.byref(p)), dev)
    L.check(L.lib.tops_b200_chunk_gla_fwd(C.byref(p), ws.data_ptr(), ws.numel(), L.stream_ptr(dev)),
            "chunk_gla_fwd")
    return o, ht, gcum, A, hs


@L.on_tensor_device
def chunk_bwd_call(q, k, v, gate, gate_kind, scale, h0, do, dht, chunk, grad_dtype, want_dg, want_dh0,
                   cu_seqlens=None, impl=L.IMPL_AUTO, h_saved=None, primal_dtypes=False, rev_segments=None):
    """Run tops_b200_chunk_gla_bwd.  Returns (dq, dk, dv, dg, dh0).  `h_saved`
    is the scratch returned by chunk_fwd_call(want_saved=True) on the same inputs.
    With `primal_dtypes` the gradients come back in the dtypes of their primals
    (dq, dk as q, k; dg as the gate), as the reference's accelerator kernel
    writes them (`tops/ops/gla/chunk.py:1551-1554`): the tcgen05 kernel then
    writes bf16 directly, any other kernel family writes fp32 and is cast.
    A scalar gate's dg is fp32 `[B,T,H]` on every kernel family."""
    B, T, H, K = q.shape
    V = v.shape[-1]
    dev = q.device
    q, k, v, do = q.contiguous(), k.contiguous(), v.contiguous(), do.contiguous()
    assert do.dtype == q.dtype, "do must have the dtype of q/k/v"
    gate = None if gate is None else gate.contiguous()
    if gate_kind == L.GATE_GAMMA:
        gate = gate.float().contiguous()
    h0 = None if h0 is None else h0.float().contiguous()
    dht = None if dht is None else dht.float().contiguous()
    N = B if cu_seqlens is None else len(cu_seqlens) - 1
    keep = []
    p = L.ChunkBwdParams()
    p.pb = make_problem(B, T, H, K, V, chunk, L.dtype_code(q.dtype),
                        L.F32 if gate is None else L.dtype_code(gate.dtype), gate_kind, scale, impl,
                        cu_seqlens, keep)
    dg_dtype = torch.float32
    direct = primal_dtypes and L.lib.tops_b200_chunk_selected_impl(C.byref(p.pb)) == L.IMPL_SM100
    if direct:
        grad_dtype = q.dtype
        dg_dtype = torch.float32 if gate_kind == L.GATE_SCALAR else gate.dtype   # a scalar gate's dg is always fp32
    dq = torch.empty(B, T, H, K, dtype=grad_dtype, device=dev)
    dk = torch.empty(B, T, H, K, dtype=grad_dtype, device=dev)
    dv = torch.empty(B, T, H, V, dtype=do.dtype, device=dev)
    dg = None
    if want_dg and gate_kind == L.GATE_PER_CHANNEL:
        dg = torch.empty(B, T, H, K, dtype=dg_dtype, device=dev)
    elif want_dg and gate_kind == L.GATE_SCALAR:
        dg = torch.empty(B, T, H, dtype=torch.float32, device=dev)
    dh0 = torch.empty(N, H, K, V, dtype=torch.float32, device=dev) if want_dh0 else None
    p.q, p.k, p.v, p.g, p.h0, p.do_, p.dht = (L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(gate), L.ptr(h0), L.ptr(do),
                                              L.ptr(dht))
    p.dq, p.dk, p.dv, p.dg, p.dh0 = L.ptr(dq), L.ptr(dk), L.ptr(dv), L.ptr(dg), L.ptr(dh0)
    p.grad_dtype = L.dtype_code(grad_dtype)
    p.dg_dtype = L.dtype_code(dg_dtype)
    if h_saved is not None:
        assert h_saved.dtype == q.dtype and h_saved.shape[-3:] == (H, K, V)
        p.h_saved = L.ptr(h_saved)
    if rev_segments is not None and L.lib.tops_b200_chunk_selected_impl(C.byref(p.pb)) == L.IMPL_SM100:
        p.rev_segments = L.ptr(rev_segments)
    ws = L.workspace(L.lib.tops_b200_chunk_bwd_workspace_bytes(C.byref(p)), dev)
    L.check(L.lib.tops_b200_chunk_gla_bwd(C.byref(p), ws.data_ptr(), ws.numel(), L.stream_ptr(dev)),
            "chunk_gla_bwd")
    if primal_dtypes and not direct:
        dq, dk = dq.to(q.dtype), dk.to(k.dtype)
        dg = dg if dg is None or gate is None else dg.to(gate.dtype)
    return dq, dk, dv, dg, dh0
