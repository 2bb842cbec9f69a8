"""KDA (Kimi delta attention: per-channel decay plus a beta-weighted delta-rule
update) with the reference's signatures (`tops/ops/kda/chunk.py:193-216`,
`tops/ops/kda/fused_recurrent.py:19-105`; oracle `tops/cpu/ops/kda/naive.py`).

    S' = S exp(g_t);  e = v_t - k_t^T S';  S = S' + beta_t k_t (x) e;  o_t = scale q_t^T S

`g` is the natural-log decay `[B,T,H,K]`, `beta` `[B,T,H]`.  `chunk_kda` and
`fused_recurrent_kda` compute the same function; both are differentiable in
q, k, v, g, beta, initial_state.  bf16 problems with K = V = 128, chunk 64 and
T a multiple of 64 run the chunked WY / UT-transform kernels on the tensor
cores (`chunk_kda_fwd`); everything else walks the tokens one by one.
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


@L.on_tensor_device
def kda_fwd(q, k, v, g, beta, scale, initial_state, output_final_state, state_out=None):
    """One call of tops_b200_kda_fwd.  Returns (o in q.dtype, final state fp32 or None).  `state_out`
    may be the initial state itself: every thread reads its part of the state before it writes it."""
    B, T, H, K, V = _check(q, k, v, g, beta, initial_state)
    dev = q.device
    q, k, v, g = q.contiguous(), k.contiguous(), v.contiguous(), g.contiguous()
    beta = beta.to(q.dtype).contiguous()
    h0 = None if initial_state is None else initial_state.float().contiguous()
    o = torch.empty(B, T, H, V, dtype=q.dtype, device=dev)
    ht = state_out
    if ht is None and output_final_state:
        ht = torch.empty(B, H, K, V, dtype=torch.float32, device=dev)
    p = L.KdaFwdParams()
    p.B, p.T, p.H, p.K, p.V = B, T, H, K, V
    p.dtype, p.gate_dtype, p.scale = L.dtype_code(q.dtype), L.dtype_code(g.dtype), float(scale)
    p.q, p.k, p.v, p.g, p.beta = L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(g), L.ptr(beta)
    p.h0, p.o, p.ht = L.ptr(h0), L.ptr(o), L.ptr(ht)
    L.check(L.lib.tops_b200_kda_fwd(C.byref(p), L.stream_ptr(dev)), "kda_fwd")
    return o, ht


@L.on_tensor_device
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


def _chunk_params(q, k, v, g, beta, scale, chunk_size):
    B, T, H, K = q.shape
    p = L.ChunkKdaFwdParams()
    p.B, p.T, p.H, p.K, p.V, p.chunk = B, T, H, K, v.shape[-1], int(chunk_size)
    p.dtype, p.gate_dtype, p.scale = L.dtype_code(q.dtype), L.dtype_code(g.dtype), float(scale)
    return p


def chunk_kernels_take(q, k, v, g, beta, chunk_size=64):
    """True when the chunked tensor-core kernels serve this problem."""
    if not (q.is_cuda and q.dtype == torch.bfloat16 and g.dtype == torch.bfloat16):
        return False
    with torch.cuda.device(q.device):
        return bool(L.lib.tops_b200_chunk_kda_supported(C.byref(_chunk_params(q, k, v, g, beta, 1.0, chunk_size))))


@L.on_tensor_device
def _chunk_fwd_call(q, k, v, g, beta, scale, initial_state, output_final_state, chunk_size, want_A, want_saved):
    """One call of tops_b200_chunk_kda_fwd.  Returns (o, ht, Aqk, Akk, saved) with Aqk / Akk fp32
    `[B,T,H,C]` when `want_A`, and saved = (h', v', T, R) residuals for the backward when `want_saved`."""
    B, T, H, K, V = _check(q, k, v, g, beta, initial_state)
    dev = q.device
    q, k, v, g = q.contiguous(), k.contiguous(), v.contiguous(), g.contiguous()
    beta_c = beta.to(q.dtype).contiguous()
    h0 = None if initial_state is None else initial_state.float().contiguous()
    o = torch.empty(B, T, H, V, dtype=q.dtype, device=dev)
    ht = torch.empty(B, H, K, V, dtype=torch.float32, device=dev) if output_final_state else None
    Aqk = torch.empty(B, T, H, chunk_size, dtype=torch.float32, device=dev) if want_A else None
    Akk = torch.empty(B, T, H, chunk_size, dtype=torch.float32, device=dev) if want_A else None
    saved = None
    if want_saved:
        saved = (torch.empty(B, T // chunk_size, H, K, V, dtype=q.dtype, device=dev),
                 torch.empty(B, T, H, V, dtype=q.dtype, device=dev),
                 torch.empty(B, T, H, chunk_size, dtype=q.dtype, device=dev),
                 torch.empty(B, T, H, V, dtype=q.dtype, device=dev))
    p = _chunk_params(q, k, v, g, beta_c, scale, chunk_size)
    p.q, p.k, p.v, p.g, p.beta, p.h0 = L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(g), L.ptr(beta_c), L.ptr(h0)
    p.o, p.ht, p.Aqk_out, p.Akk_out = L.ptr(o), L.ptr(ht), L.ptr(Aqk), L.ptr(Akk)
    if saved is not None:
        p.saved_h, p.saved_vnew, p.saved_T, p.saved_R = (L.ptr(t) for t in saved)
    L.check(L.lib.tops_b200_chunk_kda_fwd(C.byref(p), L.stream_ptr(dev)), "chunk_kda_fwd")
    return o, ht, Aqk, Akk, saved


def chunk_kda_fwd(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False, cu_seqlens=None,
                  chunk_size=64):
    """Chunked forward orchestrator (reference `tops/ops/kda/chunk.py:25-190`).  Returns
    (o, final state or None, g_cumsum, Aqk, Akk): g_cumsum the chunk-local cumulative gate in log2
    space (fp32 `[B,T,H,K]`, `tops/ops/kda/gate.py:19-51`), Aqk / Akk fp32 `[B,T,H,chunk]` — row i of
    its chunk at token i of tril(scale q k^T 2^(G_i-G_j)) and of (I + stril(beta k k^T 2^(G_i-G_j)))^-1."""
    from .common import chunk_local_cumsum
    assert cu_seqlens is None, "packed KDA batches are not supported"
    assert q.shape[1] % chunk_size == 0, \
        f"Sequence length T={q.shape[1]} must be divisible by chunk_size={chunk_size}"
    assert chunk_kernels_take(q, k, v, g, beta, chunk_size), \
        "chunk_kda_fwd takes bf16 q/k/v/g with K = V = 128 and chunk_size 64 (use chunk_kda for other problems)"
    if scale is None:
        scale = q.shape[-1] ** -0.5
    o, ht, Aqk, Akk, _ = _chunk_fwd_call(q, k, v, g, beta, scale, initial_state, output_final_state, chunk_size,
                                         True, False)
    g_cumsum = chunk_local_cumsum(g, chunk_size) * 1.4426950408889634
    return o, ht, g_cumsum, Aqk, Akk


@L.on_tensor_device
def _chunk_bwd_call(q, k, v, g, beta, do, scale, dht, saved, want_dh0, grad_dtype):
    """One call of tops_b200_chunk_kda_bwd with the residuals of _chunk_fwd_call(want_saved=True).
    Returns (dq, dk, dv, dg, dbeta, dh0): dq, dk, dg, dbeta in `grad_dtype`, dv in q.dtype."""
    B, T, H, K = q.shape
    V = v.shape[-1]
    dev = q.device
    q, k, v, g = q.contiguous(), k.contiguous(), v.contiguous(), g.contiguous()
    beta_c = beta.to(q.dtype).contiguous()
    do = do.to(q.dtype).contiguous()
    dhtc = None if dht is None else dht.float().contiguous()
    dq = torch.empty(B, T, H, K, dtype=grad_dtype, device=dev)
    dk, dg = torch.empty_like(dq), torch.empty_like(dq)
    dbeta = torch.empty(B, T, H, dtype=grad_dtype, device=dev)
    dv = torch.empty(B, T, H, V, dtype=q.dtype, device=dev)
    dh0 = torch.empty(B, H, K, V, dtype=torch.float32, device=dev) if want_dh0 else None
    p = L.ChunkKdaBwdParams()
    p.B, p.T, p.H, p.K, p.V, p.chunk = B, T, H, K, V, 64
    p.dtype, p.gate_dtype, p.scale = L.dtype_code(q.dtype), L.dtype_code(g.dtype), float(scale)
    p.q, p.k, p.v, p.g, p.beta, p.do_, p.dht = (L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(g), L.ptr(beta_c), L.ptr(do),
                                                L.ptr(dhtc))
    p.saved_h, p.saved_vnew, p.saved_T, p.saved_R = (L.ptr(t) for t in saved)
    p.dq, p.dk, p.dg, p.dbeta, p.dv, p.dh0 = L.ptr(dq), L.ptr(dk), L.ptr(dg), L.ptr(dbeta), L.ptr(dv), L.ptr(dh0)
    p.grad_dtype = L.dtype_code(grad_dtype)
    ws = L.workspace(L.lib.tops_b200_chunk_kda_bwd_workspace_bytes(C.byref(p)), dev)
    L.check(L.lib.tops_b200_chunk_kda_bwd(C.byref(p), ws.data_ptr(), ws.numel(), L.stream_ptr(dev)), "chunk_kda_bwd")
    return dq, dk, dv, dg, dbeta, dh0


@L.on_tensor_device
def _chunk_bwd_state_gradient(q, k, v, g, beta, do, scale, dht, saved):
    """The state-gradient-only form of tops_b200_chunk_kda_bwd: the reverse scan alone.  Returns dh0 fp32
    `[B,H,K,V]` (for `dht = None`: the shard summary D of a time-sharded sequence)."""
    B, T, H, K = q.shape
    V = v.shape[-1]
    dev = q.device
    q, k, v, g = q.contiguous(), k.contiguous(), v.contiguous(), g.contiguous()
    beta_c = beta.to(q.dtype).contiguous()
    do = do.to(q.dtype).contiguous()
    dhtc = None if dht is None else dht.float().contiguous()
    dv = torch.empty(B, T, H, V, dtype=q.dtype, device=dev)
    dh0 = torch.empty(B, H, K, V, dtype=torch.float32, device=dev)
    p = L.ChunkKdaBwdParams()
    p.B, p.T, p.H, p.K, p.V, p.chunk = B, T, H, K, V, 64
    p.dtype, p.gate_dtype, p.scale = L.dtype_code(q.dtype), L.dtype_code(g.dtype), float(scale)
    p.q, p.k, p.v, p.g, p.beta, p.do_, p.dht = (L.ptr(q), L.ptr(k), L.ptr(v), L.ptr(g), L.ptr(beta_c), L.ptr(do),
                                                L.ptr(dhtc))
    p.saved_h, p.saved_vnew, p.saved_T, p.saved_R = (L.ptr(t) for t in saved)
    p.dv, p.dh0 = L.ptr(dv), L.ptr(dh0)
    p.grad_dtype = L.F32
    ws = L.workspace(L.lib.tops_b200_chunk_kda_bwd_workspace_bytes(C.byref(p)), dev)
    L.check(L.lib.tops_b200_chunk_kda_bwd(C.byref(p), ws.data_ptr(), ws.numel(), L.stream_ptr(dev)), "chunk_kda_bwd")
    return dh0


def chunk_kda_bwd(q, k, v, g, beta, do, scale=None, initial_state=None, dht=None, chunk_size=64):
    """Explicit chunked backward (reference `tops/cpu/ops/kda/chunk_bwd.py:525-668`) for problems the
    tensor-core kernels take: recomputes the forward's residuals, then the three backward kernels.
    Returns (dq, dk fp32, dv in v.dtype, dbeta fp32, dg fp32 with respect to the natural-log gate,
    dh0 fp32 or None — only when initial_state is given)."""
    assert chunk_size == 64 and chunk_kernels_take(q, k, v, g, beta, 64), \
        "chunk_kda_bwd takes bf16 q/k/v/g with K = V = 128 and chunk_size 64 (use kda_bwd for other problems)"
    if scale is None:
        scale = q.shape[-1] ** -0.5
    _, _, _, _, saved = _chunk_fwd_call(q, k, v, g, beta, scale, initial_state, False, 64, False, True)
    dq, dk, dv, dg, dbeta, dh0 = _chunk_bwd_call(q, k, v, g, beta, do, scale, dht, saved, initial_state is not None,
                                                 torch.float32)
    return dq, dk, dv, dbeta, dg, dh0


class _KDA(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, g, beta, initial_state, scale, output_final_state, chunked):
        saved = None
        if chunked:
            keep = any(t is not None and t.requires_grad for t in (q, k, v, g, beta, initial_state))
            o, ht, _, _, saved = _chunk_fwd_call(q, k, v, g, beta, scale, initial_state, output_final_state, 64, False,
                                                 keep)
        else:
            o, ht = kda_fwd(q, k, v, g, beta, scale, initial_state, output_final_state)
        ctx.save_for_backward(q, k, v, g, beta, initial_state, *(saved or ()))
        ctx.scale, ctx.chunked = scale, saved is not None
        return o, ht

    @staticmethod
    def backward(ctx, do, dht):
        q, k, v, g, beta, h0 = ctx.saved_tensors[:6]
        if ctx.chunked:
            # cotangents take the primal's dtype at this boundary
            dq, dk, dv, dg, dbeta, dh0 = _chunk_bwd_call(q, k, v, g, beta, do, ctx.scale, dht, ctx.saved_tensors[6:],
                                                         h0 is not None, q.dtype)
            if L.CHECK_DEVICE:
                L.raise_on_device_error("chunk_kda backward")
            return (dq, dk, dv, dg.to(g.dtype), dbeta.to(beta.dtype), None if h0 is None else dh0.to(h0.dtype),
                    None, None, None)
        dq, dk, dv, dg, dbeta, dh0 = kda_bwd(q, k, v, g, beta, do, ctx.scale, h0, dht)
        return dq, dk, dv, dg, dbeta, None if h0 is None else dh0.to(h0.dtype), None, None, None


def fused_recurrent_kda(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False):
    """Token-serial KDA (reference `tops/ops/kda/fused_recurrent.py:19-105`)."""
    B, T, H, K, V = _check(q, k, v, g, beta, initial_state)
    if scale is None:
        scale = K ** -0.5
    o, ht = _KDA.apply(q, k, v, g, beta, initial_state, float(scale), bool(output_final_state), False)
    return o, (ht if output_final_state else None)


def fused_recurrent_kda_decode_(q, k, v, g, beta, state, scale=None):
    """Decode: the tokens of this call (usually one) update `state` `[B,H,K,V]` fp32 IN PLACE and the outputs
    `[B,T,H,V]` come back in q.dtype (reference, functional form: `tops/cpu/ops/kda/fused_recurrent.py:71-209`)."""
    B, T, H, K, V = _check(q, k, v, g, beta, state)
    assert state.dtype == torch.float32 and state.is_contiguous()
    if scale is None:
        scale = K ** -0.5
    with torch.no_grad():
        o, _ = kda_fwd(q, k, v, g, beta, float(scale), state, True, state_out=state)
    return o


def chunk_kda(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False, cu_seqlens=None,
              chunk_size=64):
    """Chunked KDA (reference `tops/ops/kda/chunk.py:193-216`): same function as
    `fused_recurrent_kda`.  T must be divisible by chunk_size, as upstream."""
    assert cu_seqlens is None, "packed KDA batches are not supported"
    assert chunk_size >= 1 and (chunk_size & (chunk_size - 1)) == 0, "chunk_size must be a power of 2"
    assert q.shape[1] % chunk_size == 0, f"T ({q.shape[1]}) must be divisible by chunk_size ({chunk_size})"
    B, T, H, K, V = _check(q, k, v, g, beta, initial_state)
    if scale is None:
        scale = K ** -0.5
    # the result does not depend on the chunk length beyond where roundings fall: a problem the
    # tensor-core kernels take runs with their chunk of 64
    chunked = T % 64 == 0 and chunk_kernels_take(q, k, v, g, beta, 64)
    o, ht = _KDA.apply(q, k, v, g, beta, initial_state, float(scale), bool(output_final_state), chunked)
    return o, (ht if output_final_state else None)
