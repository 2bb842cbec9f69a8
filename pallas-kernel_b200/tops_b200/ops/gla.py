"""GLA (per-channel gate) ops with the reference's Python signatures
(`tops/ops/gla/__init__.py`, oracle in `tops/cpu/ops/gla/`): `chunk_gla`,
`fused_chunk_gla`, `chunk_gla_fwd`, `chunk_gla_bwd`, `fused_recurrent_gla`,
`fused_recurrent_fwd`, `fused_recurrent_bwd`.

Tensors are CUDA tensors `[B, T, H, D]`; states `[N, H, K, V]` fp32.  The
public `chunk_gla` / `fused_chunk_gla` / `fused_recurrent_gla` are
differentiable (torch.autograd.Function standing where the reference's JAX ops
use / would use `custom_vjp`); the explicit `*_bwd` functions return the
oracle's dtypes (dq, dk, dg fp32; dv in do.dtype).
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _lib as L
from ._chunk import chunk_bwd_call, chunk_fwd_call


def _check_qkvg(q, k, v, g, initial_state, cu_seqlens):
    assert q.ndim == 4, f"q must be [B,T,H,K], got {tuple(q.shape)}"
    B, T, H, K = q.shape
    assert k.shape == q.shape, f"k shape {tuple(k.shape)} != q shape {tuple(q.shape)}"
    assert v.ndim == 4 and v.shape[:3] == q.shape[:3], f"v shape {tuple(v.shape)} incompatible with q"
    assert k.dtype == q.dtype and v.dtype == q.dtype, "q, k, v must share a dtype"
    V = v.shape[-1]
    assert g is None or g.shape == q.shape, f"g shape {tuple(g.shape)} != q shape {tuple(q.shape)}"
    N = B
    if cu_seqlens is not None:
        assert B == 1, f"B must be 1 for varlen, got {B}"
        cu = [int(x) for x in cu_seqlens]
        N = len(cu) - 1
        assert all(b > a for a, b in zip(cu[:-1], cu[1:])), "Empty segments not supported"
        assert cu[0] == 0 and cu[-1] == T, "cu_seqlens must span [0, T]"
    if initial_state is not None:
        assert initial_state.shape == (N, H, K, V), \
            f"initial_state shape {tuple(initial_state.shape)} != expected {(N, H, K, V)}"
    return B, T, H, K, V, N


def _cu_list(cu_seqlens):
    return None if cu_seqlens is None else [int(x) for x in cu_seqlens]


def chunk_gla_fwd(q, k, v, g, g_cumsum, scale, initial_state, output_final_state, chunk_size=64,
                  cu_seqlens=None):
    """Forward orchestrator (reference `tops/cpu/ops/gla/chunk.py:159-269`).
    Returns (g_cumsum fp32, A fp32 `[B,T,H,C]`, h `[B,NT,H,K,V]` k.dtype, ht, o).
    `g_cumsum` is accepted for signature parity and recomputed."""
    _check_qkvg(q, k, v, g, initial_state, cu_seqlens)
    assert chunk_size in (16, 32, 64), \
        f"chunk_gla_fwd returns per-chunk tensors; the kernels hold chunks of 16, 32 or 64, got {chunk_size}"
    cu = _cu_list(cu_seqlens)
    o, ht, gcum, A, h = chunk_fwd_call(q, k, v, g, L.GATE_PER_CHANNEL, scale, initial_state,
                                       output_final_state, chunk_size, cu, want_gcum=True, want_A=True,
                                       want_h=True, impl=L.IMPL_GENERIC)
    return gcum, A, h, ht, o


def chunk_gla_bwd(q, k, v, g, g_cumsum, scale, initial_state, h, A, do, dht, chunk_size=64,
                  cu_seqlens=None):
    """Backward orchestrator (reference `tops/cpu/ops/gla/chunk.py:469-640`).
    `g_cumsum`, `h`, `A` are accepted for signature parity and recomputed, so the gradients do not depend
    on `chunk_size` beyond rounding: a power of two the kernels do not hold (128) runs with the nearest.
    Returns (dq fp32, dk fp32, dv do.dtype, dg fp32, dh0 fp32 or None)."""
    _check_qkvg(q, k, v, g, initial_state, cu_seqlens)
    assert chunk_size >= 1 and (chunk_size & (chunk_size - 1)) == 0, \
        f"chunk_size must be a power of 2, got {chunk_size}"   # tops/ops/common/cumsum.py:506-508
    chunk_size = min(max(int(chunk_size), 16), 64)
    return chunk_bwd_call(q, k, v, g, L.GATE_PER_CHANNEL, scale, initial_state, do, dht, chunk_size,
                          torch.float32, True, initial_state is not None, _cu_list(cu_seqlens))


def _kernel_chunk(q, v, g, cu_seqlens, chunk_size):
    """Chunk length the kernels use for the differentiable op.  The op's results (o, final state,
    gradients) do not depend on the chunk length beyond where bf16 roundings fall, so a problem the
    tcgen05 kernels can take (bf16, K = V = 128, dense, T a multiple of 64) runs with their chunk of
    64 whatever `chunk_size` asks for (the reference's default is 16); everything else keeps the
    requested length.  The orchestrators that return per-chunk intermediates never change it."""
    assert chunk_size >= 1 and (chunk_size & (chunk_size - 1)) == 0, \
        f"chunk_size must be a power of 2, got {chunk_size}"   # tops/ops/common/cumsum.py:506-508
    if (g is not None and cu_seqlens is None and q.dtype == torch.bfloat16 and g.dtype == torch.bfloat16
            and q.shape[-1] == 128 and v.shape[-1] == 128 and q.shape[1] % 64 == 0):
        return 64
    # the kernels hold chunks of 16, 32 or 64 time steps; longer (or shorter) powers of two give the
    # same results computed with the nearest length they hold
    return min(max(chunk_size, 16), 64)


class _ChunkGLA(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, g, initial_state, scale, output_final_state, cu, chunk_size):
        # the tcgen05 forward keeps its chunk-start states for the backward (one bf16 [B,NT,H,K,V] tensor)
        keep = any(t is not None and t.requires_grad for t in (q, k, v, g, initial_state))
        o, ht, _, _, hs = chunk_fwd_call(q, k, v, g, L.GATE_PER_CHANNEL if g is not None else L.GATE_NONE,
                                         scale, initial_state, output_final_state, chunk_size, cu, want_saved=keep)
        ctx.save_for_backward(q, k, v, g, initial_state, hs)
        ctx.scale, ctx.cu, ctx.chunk = scale, cu, chunk_size
        return o, ht

    @staticmethod
    def backward(ctx, do, dht):
        q, k, v, g, h0, hs = ctx.saved_tensors
        kind = L.GATE_PER_CHANNEL if g is not None else L.GATE_NONE
        # cotangents take the primal's dtype at this boundary
        dq, dk, dv, dg, dh0 = chunk_bwd_call(q, k, v, g, kind, ctx.scale, h0, do.to(q.dtype), dht, ctx.chunk,
                                             torch.float32, g is not None, h0 is not None, ctx.cu, h_saved=hs,
                                             primal_dtypes=True)
        if L.CHECK_DEVICE:
            L.raise_on_device_error("chunk_gla backward")
        return (dq, dk, dv, dg, None if h0 is None else dh0.to(h0.dtype), None, None, None, None)


def chunk_gla(q, k, v, g=None, g_gamma=None, scale=None, initial_state=None, output_final_state=False,
              cu_seqlens=None, chunk_size=16):
    """Chunked GLA (reference `tops/cpu/ops/gla/chunk.py:648-709`; the
    accelerator signature `tops/ops/gla/chunk.py:1207-1218` adds `g_gamma`).
    g defaults to zeros, scale to K^-0.5, chunk_size to 16.  Returns
    (o in v.dtype, final state fp32 or None).  Differentiable in q, k, v, g,
    initial_state."""
    B, T, H, K, V, N = _check_qkvg(q, k, v, g, initial_state, cu_seqlens)
    if scale is None:
        scale = K ** -0.5
    # `g_gamma` is "used only when g is None" upstream (tops/ops/gla/chunk.py:1224-1228)
    if g is None and g_gamma is not None:
        # constant decay: `[H]` (one log-gate per head) or anything that broadcasts to [B,T,H,K]
        gg = g_gamma.to(torch.float32)
        gg = gg.view(1, 1, H, 1) if gg.ndim == 1 and gg.shape[0] == H else gg
        g = torch.broadcast_to(gg, (B, T, H, K)).contiguous()
    if initial_state is not None:
        initial_state = initial_state.to(torch.float32)
    o, ht = _ChunkGLA.apply(q, k, v, g, initial_state, float(scale), bool(output_final_state),
                            _cu_list(cu_seqlens), int(_kernel_chunk(q, v, g, cu_seqlens, chunk_size)))
    return o, (ht if output_final_state else None)


def fused_chunk_gla(q, k, v, g=None, scale=None, initial_state=None, output_final_state=False,
                    cu_seqlens=None, chunk_size=16):
    """Alias of `chunk_gla` (reference `tops/cpu/ops/gla/fused_chunk.py:4-44`)."""
    return chunk_gla(q, k, v, g, None, scale, initial_state, output_final_state, cu_seqlens, chunk_size)


# ---------------------------------------------------------------------------
# token-serial recurrence
# ---------------------------------------------------------------------------
@L.on_tensor_device
def _rec_fwd_call(q, k, v, gk, gv, scale, initial_state, want_state, reverse, cu, o_dtype, state_out=None):
    B, T, H, K = q.shape
    V = v.shape[-1]
    dev = q.device
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    gk = None if gk is None else gk.contiguous()
    gv = None if gv is None else gv.contiguous()
    if gk is not None and gv is not None:
        assert gk.dtype == gv.dtype
    gate_dt = gk.dtype if gk is not None else (gv.dtype if gv is not None else torch.float32)
    N = B if cu is None else len(cu) - 1
    h0 = None if initial_state is None else initial_state.float().contiguous()
    o = torch.empty(B, T, H, V, dtype=o_dtype, device=dev)
    if state_out is None and want_state:
        state_out = torch.empty(N, H, K, V, dtype=torch.float32, device=dev)
    cu_dev = None if cu is None else torch.tensor(cu, dtype=torch.int32, device=dev)
    p = L.RecurrentFwdParams()
    p.B, p.T, p.H, p.K, p.V = B, T, H, K, V
    p.dtype, p.gate_dtype, p.o_dtype = L.dtype_code(q.dtype), L.dtype_code(gate_dt), L.dtype_code(o_dtype)
    p.reverse, p.scale = int(reverse), float(scale)
    p.q, p.k, p.v, p.gk, p.gv = L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(gk), L.ptr(gv)
    p.state_in, p.state_out, p.o = L.ptr(h0), L.ptr(state_out), L.ptr(o)
    p.cu_seqlens, p.N = L.ptr(cu_dev), N
    L.check(L.lib.tops_b200_fused_recurrent_gla_fwd(C.byref(p), L.stream_ptr(dev)), "fused_recurrent_gla_fwd")
    return o, state_out


def _check_rec(q, k, v, gk, gv, initial_state, cu_seqlens):
    B, T, H, K = q.shape
    V = v.shape[-1]
    N = len(cu_seqlens) - 1 if cu_seqlens is not None else B
    assert k.shape == (B, T, H, K), f"k shape {tuple(k.shape)} != expected {(B, T, H, K)}"
    assert v.shape[:3] == (B, T, H), f"v shape {tuple(v.shape)} incompatible with q"
    assert gk is None or gk.shape == (B, T, H, K), f"gk shape {tuple(gk.shape)} != expected {(B, T, H, K)}"
    assert gv is None or gv.shape == (B, T, H, V), f"gv shape {tuple(gv.shape)} != expected {(B, T, H, V)}"
    assert initial_state is None or initial_state.shape == (N, H, K, V), \
        f"initial_state shape {tuple(initial_state.shape)} != expected {(N, H, K, V)}"
    assert cu_seqlens is None or B == 1, f"cu_seqlens requires B=1, got B={B}"
    return K


def fused_recurrent_fwd(q, k, v, gk=None, gv=None, scale=None, initial_state=None,
                        output_final_state=False, reverse=False, cu_seqlens=None):
    """Recurrent forward with fp32 output (reference
    `tops/cpu/ops/gla/fused_recurrent.py:51-162`)."""
    K = _check_rec(q, k, v, gk, gv, initial_state, cu_seqlens)
    if scale is None:
        scale = K ** -0.5
    return _rec_fwd_call(q, k, v, gk, gv, scale, initial_state, output_final_state, reverse,
                         _cu_list(cu_seqlens), torch.float32)


@L.on_tensor_device
def fused_recurrent_bwd(q, k, v, gk=None, gv=None, o=None, do=None, dht=None, scale=None,
                        initial_state=None, reverse=False, cu_seqlens=None):
    """Two-pass recurrent backward (reference
    `tops/cpu/ops/gla/fused_recurrent.py:171-353`).  Returns
    (dq, dk, dv in input dtypes, dgk, dgv in gate dtypes or None, dh0 or None)."""
    K = _check_rec(q, k, v, gk, gv, initial_state, cu_seqlens)
    assert do is not None
    if gv is not None:
        assert o is not None, "o (forward output) required when gv is used"
    if scale is None:
        scale = K ** -0.5
    B, T, H, _ = q.shape
    V = v.shape[-1]
    dev = q.device
    cu = _cu_list(cu_seqlens)
    N = B if cu is None else len(cu) - 1
    q, k, v, do = q.contiguous(), k.contiguous(), v.contiguous(), do.to(q.dtype).contiguous()
    gk = None if gk is None else gk.contiguous()
    gv = None if gv is None else gv.contiguous()
    gate_dt = gk.dtype if gk is not None else (gv.dtype if gv is not None else torch.float32)
    o32 = None if o is None else o.float().contiguous()
    h0 = None if initial_state is None else initial_state.float().contiguous()
    dhtc = None if dht is None else dht.float().contiguous()
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    dgk = None if gk is None else torch.empty_like(gk)
    dgv = None if gv is None else torch.empty_like(gv)
    dh0 = None if h0 is None else torch.empty(N, H, K, V, dtype=torch.float32, device=dev)
    cu_dev = None if cu is None else torch.tensor(cu, dtype=torch.int32, device=dev)
    p = L.RecurrentBwdParams()
    p.B, p.T, p.H, p.K, p.V = B, T, H, K, V
    p.dtype, p.gate_dtype, p.reverse, p.scale = L.dtype_code(q.dtype), L.dtype_code(gate_dt), int(reverse), float(scale)
    p.q, p.k, p.v, p.gk, p.gv, p.o, p.do_ = L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(gk), L.ptr(gv), L.ptr(o32), L.ptr(do)
    p.h0, p.dht, p.dq, p.dk, p.dv = L.ptr(h0), L.ptr(dhtc), L.ptr(dq), L.ptr(dk), L.ptr(dv)
    p.dgk, p.dgv, p.dh0, p.cu_seqlens, p.N = L.ptr(dgk), L.ptr(dgv), L.ptr(dh0), L.ptr(cu_dev), N
    ws = L.workspace(L.lib.tops_b200_fused_recurrent_gla_bwd_workspace_bytes(C.byref(p)), dev)
    L.check(L.lib.tops_b200_fused_recurrent_gla_bwd(C.byref(p), ws.data_ptr(), ws.numel(), L.stream_ptr(dev)),
            "fused_recurrent_gla_bwd")
    if dh0 is not None:
        dh0 = dh0.to(initial_state.dtype)
    return dq, dk, dv, dgk, dgv, dh0


class _FusedRecurrentGLA(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, gk, gv, initial_state, scale, output_final_state, reverse, cu):
        o32, ht = _rec_fwd_call(q, k, v, gk, gv, scale, initial_state, output_final_state, reverse, cu,
                                torch.float32)
        ctx.save_for_backward(q, k, v, gk, gv, initial_state, o32 if gv is not None else None)
        ctx.scale, ctx.reverse, ctx.cu = scale, reverse, cu
        return o32.to(q.dtype), ht

    @staticmethod
    def backward(ctx, do, dht):
        q, k, v, gk, gv, h0, o32 = ctx.saved_tensors
        dq, dk, dv, dgk, dgv, dh0 = fused_recurrent_bwd(q, k, v, gk, gv, o32, do, dht, ctx.scale, h0,
                                                        ctx.reverse, ctx.cu)
        return dq, dk, dv, dgk, dgv, dh0, None, None, None, None


def fused_recurrent_gla(q, k, v, gk=None, gv=None, scale=None, initial_state=None,
                        output_final_state=False, reverse=False, cu_seqlens=None):
    """Recurrent GLA (reference `tops/cpu/ops/gla/fused_recurrent.py:362-422`):
    o in q.dtype, final state fp32.  Differentiable."""
    K = _check_rec(q, k, v, gk, gv, initial_state, cu_seqlens)
    if scale is None:
        scale = K ** -0.5
    o, ht = _FusedRecurrentGLA.apply(q, k, v, gk, gv, initial_state, float(scale), bool(output_final_state),
                                     bool(reverse), _cu_list(cu_seqlens))
    return o, (ht if output_final_state else None)


def fused_recurrent_gla_decode_(q, k, v, gk, state, scale=None, gv=None):
    """One decode step per call: `state` `[B,H,K,V]` fp32 is updated in place
    and o `[B,1,H,V]` is returned in q.dtype.  (The reference returns a fresh
    state, `tops/ops/gla/fused_recurrent.py:262`; in-place is the B200 path.)"""
    K = _check_rec(q, k, v, gk, gv, state, None)
    assert state.dtype == torch.float32 and state.is_contiguous()
    if scale is None:
        scale = K ** -0.5
    o, _ = _rec_fwd_call(q, k, v, gk, gv, scale, state, True, False, None, q.dtype, state_out=state)
    return o
