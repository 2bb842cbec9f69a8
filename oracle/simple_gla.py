"""Oracle for simple_gla (one scalar log-gate per head and token, or a constant
per-head decay) — test infrastructure only.

Restates `tops/cpu/ops/simple_gla/{chunk,naive,fused_recurrent}.py` of the
reference in torch-on-CPU.  Packed (`cu_seqlens`) inputs are handled by running
the dense code per sequence.
"""
from __future__ import annotations

import torch

from .common import (acc_dtype, cdiv, chunk_bwd_dh, chunk_fwd_h, chunk_fwd_o, chunk_local_cumsum, dot,
                     pad_time, _segments)


def chunk_simple_gla_fwd(q, k, v, g, g_gamma, scale, initial_state, output_final_state,
                         chunk_size=64, cu_seqlens=None):
    """Forward orchestrator (`tops/cpu/ops/simple_gla/chunk.py:53-129`): pad,
    cumsum, state scan (states in k.dtype), output.  Returns (o, ht)."""
    T0 = q.shape[1]
    C = chunk_size
    if cu_seqlens is None:
        q, k, v = (pad_time(x, C) for x in (q, k, v))
        if g is not None:
            g = pad_time(g, C)
    if g is not None:
        g = chunk_local_cumsum(g, C, cu_seqlens=cu_seqlens)
    h, ht = chunk_fwd_h(k, v, g=g, g_gamma=g_gamma, h0=initial_state,
                        output_final_state=output_final_state, chunk_size=C, states_in_fp32=False,
                        original_T=None if cu_seqlens is not None else T0, cu_seqlens=cu_seqlens)
    o = chunk_fwd_o(q, k, v, h, g=g, g_gamma=g_gamma, scale=scale, chunk_size=C, cu_seqlens=cu_seqlens)
    return o[:, :T0], ht


def _per_sequence(fn, tensors, gates, states, cu_seqlens, C):
    """Run `fn(tensors, gates, states, original_T)` on every sequence of a
    packed batch; inputs padded to whole chunks, cumulative gates by repeating
    their last value."""
    outs = []
    c0 = 0
    for n, (bos, eos) in enumerate(_segments(cu_seqlens)):
        sl = slice(bos, eos)
        nch = cdiv(eos - bos, C)

        def pad_gate(x):
            if x is None:
                return None
            seg = x[:, sl]
            extra = (-seg.shape[1]) % C
            if extra:
                seg = torch.cat([seg, seg[:, -1:].expand(-1, extra, *seg.shape[2:])], 1)
            return seg
        outs.append(fn([pad_time(x[:, sl], C) for x in tensors], [pad_gate(x) for x in gates],
                       [None if s is None else s[:, c0:c0 + nch] for s in states], eos - bos))
        c0 += nch
    return outs


def chunk_bwd_dqkwg(q, k, v, h, dh, do, *, g=None, g_gamma=None, scale=1.0, chunk_size=64,
                    original_T=None, cu_seqlens=None):
    """dq, dk (input dtype) and the pre-cumsum gate gradient
    (`tops/cpu/ops/simple_gla/chunk.py:137-468`).  Per chunk:
      ds = do v^T; dq = do cast(h)^T; dk = v cast(dh)^T
      gate g: dq *= exp(G) scale; dk *= exp(G_n - G);
              ds = tril(ds * exp(G_i - G_j)) scale
              dg = sum_k q dq - sum_k k dk + rowsum(ds*(q k^T)) - colsum(ds*(q k^T))
              dg[last] += exp(G_n) sum(h dh) + sum(dk k)
              dq += cast(ds) k; dk += cast(ds^T) q
      g_gamma: same with G_i = gamma (i+1), no dg;  no gate: ds cast, scale applied last.
    """
    B, T, H, K = q.shape
    C = chunk_size
    acc = acc_dtype(q.dtype)
    if cu_seqlens is not None:
        assert B == 1
        T0 = T
        res = _per_sequence(
            lambda t, gt, st, oT: chunk_bwd_dqkwg(t[0], t[1], t[2], st[0], st[1], t[3], g=gt[0],
                                                  g_gamma=g_gamma, scale=scale, chunk_size=C, original_T=oT),
            [q, k, v, do], [g], [h, dh], cu_seqlens, C)
        dq = q.new_zeros(1, T0, H, K)
        dk = k.new_zeros(1, T0, H, K)
        dg = torch.zeros(1, T0, H, dtype=acc) if g is not None else None
        for (bos, eos), (a, b, c) in zip(_segments(cu_seqlens), res):
            dq[:, bos:eos], dk[:, bos:eos] = a[:, : eos - bos], b[:, : eos - bos]
            if dg is not None:
                # the chunk-end term sits on the padded last row: fold it onto the last valid row
                n = eos - bos
                c = c.clone()
                if n % C:
                    c[:, n - 1] += c[:, n:].sum(1)
                dg[:, bos:eos] = c[:, :n]
        return dq, dk, dg
    NT = T // C
    tril = torch.tril(torch.ones(C, C, dtype=torch.bool))
    zero = torch.zeros((), dtype=acc)
    dqs, dks, dgs = [], [], []
    for c in range(NT):
        sl = slice(c * C, (c + 1) * C)
        bq, bk, bv, bdo = q[:, sl], k[:, sl], v[:, sl], do[:, sl]
        bh, bdh = h[:, c], dh[:, c]
        ds = dot("bihv,bjhv->bihj", bdo, bv, acc)
        dq = dot("bchv,bhkv->bchk", bdo, bh.to(do.dtype), acc)
        dk = dot("bchv,bhkv->bchk", bv, bdh.to(v.dtype), acc)
        if g is not None or g_gamma is not None:
            if g is not None:
                gc = g[:, sl]                                           # [B,C,H]
                glast = gc[:, -1]                                       # [B,H]
            else:
                ramp = g_gamma.to(acc)[None, :] * torch.arange(1, C + 1, dtype=acc)[:, None]
                gc = ramp[None].expand(B, C, H)
                oT = T if original_T is None else original_T
                glast = (g_gamma.to(acc) * min(C, oT - c * C))[None].expand(B, H)
            dq = dq * torch.exp(gc)[..., None] * scale
            dk = dk * torch.exp(glast[:, None, :, None] - gc[..., None])
            ds = torch.where(tril[None, :, None, :],
                             ds * torch.exp(gc[:, :, :, None] - gc.permute(0, 2, 1)[:, None]), zero) * scale
            if g is not None:
                dg_last = (bh.to(acc) * bdh).sum((-2, -1)) * torch.exp(glast)
                dg = (dq * bq.to(acc)).sum(-1) - (bk.to(acc) * dk).sum(-1)
                dg_last = dg_last + (dk * bk.to(acc)).sum((1, 3))
                ds2 = ds * dot("bihk,bjhk->bihj", bq.to(acc), bk.to(acc), acc)
                dg = dg + ds2.sum(-1) - ds2.sum(1).permute(0, 2, 1)
                dg[:, -1] = dg[:, -1] + dg_last
                dgs.append(dg)
            dq = dq + dot("bihj,bjhk->bihk", ds.to(k.dtype), bk, acc)
            dk = dk + dot("bjhi,bihk->bjhk", ds.permute(0, 3, 2, 1).to(q.dtype), bq, acc)
        else:
            ds = torch.where(tril[None, :, None, :], ds, zero).to(k.dtype)
            dq = (dq + dot("bihj,bjhk->bihk", ds, bk, acc)) * scale
            dk = dk + dot("bjhi,bihk->bjhk", ds.permute(0, 3, 2, 1), bq, acc) * scale
        dqs.append(dq.to(q.dtype))
        dks.append(dk.to(k.dtype))
    dq = torch.stack(dqs, 1).reshape(B, T, H, K)
    dk = torch.stack(dks, 1).reshape(B, T, H, K)
    dg = torch.stack(dgs, 1).reshape(B, T, H) if g is not None else None
    return dq, dk, dg


def chunk_bwd_dv(q, k, do, dh, *, g=None, g_gamma=None, scale=1.0, chunk_size=64, original_T=None,
                 cu_seqlens=None):
    """dv = cast( (k cast(dh)) exp(G_n - G_j) + cast(triu((k q^T) exp(G_i - G_j)) scale) do )
    (`tops/cpu/ops/simple_gla/chunk.py:476-661`)."""
    B, T, H, K = q.shape
    V = do.shape[-1]
    C = chunk_size
    acc = acc_dtype(q.dtype)
    if cu_seqlens is not None:
        assert B == 1
        res = _per_sequence(
            lambda t, gt, st, oT: chunk_bwd_dv(t[0], t[1], t[2], st[0], g=gt[0], g_gamma=g_gamma,
                                               scale=scale, chunk_size=C, original_T=oT),
            [q, k, do], [g], [dh], cu_seqlens, C)
        dv = do.new_zeros(1, T, H, V)
        for (bos, eos), a in zip(_segments(cu_seqlens), res):
            dv[:, bos:eos] = a[:, : eos - bos]
        return dv
    NT = T // C
    triu = torch.triu(torch.ones(C, C, dtype=torch.bool))   # [j, i] with j <= i
    zero = torch.zeros((), dtype=acc)
    outs = []
    for c in range(NT):
        sl = slice(c * C, (c + 1) * C)
        bq, bk, bdo = q[:, sl], k[:, sl], do[:, sl]
        A = dot("bjhk,bihk->bjhi", bk, bq, acc)
        dv = dot("bchk,bhkv->bchv", bk, dh[:, c].to(k.dtype), acc)
        if g is not None or g_gamma is not None:
            if g is not None:
                gc = g[:, sl]
                glast = gc[:, -1]
            else:
                ramp = g_gamma.to(acc)[None, :] * torch.arange(1, C + 1, dtype=acc)[:, None]
                gc = ramp[None].expand(B, C, H)
                oT = T if original_T is None else original_T
                glast = (g_gamma.to(acc) * min(C, oT - c * C))[None].expand(B, H)
            A = torch.where(triu[None, :, None, :],
                            A * torch.exp(gc.permute(0, 2, 1)[:, None] - gc[:, :, :, None]) * scale,
                            zero).to(do.dtype)
            dv = dv * torch.exp(glast[:, None, :, None] - gc[..., None])
        else:
            A = torch.where(triu[None, :, None, :], A * scale, zero).to(do.dtype)
        dv = dv + dot("bjhi,bihv->bjhv", A, bdo, acc)
        outs.append(dv.to(do.dtype))
    return torch.stack(outs, 1).reshape(B, T, H, V)


def chunk_simple_gla_bwd(q, k, v, g, g_gamma, initial_state, do, dht, scale, chunk_size=64,
                         cu_seqlens=None):
    """Backward orchestrator (`tops/cpu/ops/simple_gla/chunk.py:668-788`).
    Returns (dq, dk input dtype, dv do.dtype, dg fp32 `[B,T,H]` or None, dh0)."""
    assert not (g is not None and g_gamma is not None), "use g or g_gamma, not both"
    T0 = q.shape[1]
    C = chunk_size
    if cu_seqlens is None:
        q, k, v, do = (pad_time(x, C) for x in (q, k, v, do))
        if g is not None:
            g = pad_time(g, C)
    if g is not None:
        g = chunk_local_cumsum(g, C, cu_seqlens=cu_seqlens)
    oT = None if cu_seqlens is not None else T0
    h, _ = chunk_fwd_h(k, v, g=g, g_gamma=g_gamma, h0=initial_state, output_final_state=False,
                       chunk_size=C, states_in_fp32=True, original_T=oT, cu_seqlens=cu_seqlens)
    dh, dh0 = chunk_bwd_dh(q, do, g=g, g_gamma=g_gamma, h0=initial_state, dht=dht, scale=scale,
                           chunk_size=C, original_T=oT, cu_seqlens=cu_seqlens)
    dq, dk, dg = chunk_bwd_dqkwg(q, k, v, h, dh, do, g=g, g_gamma=g_gamma, scale=scale, chunk_size=C,
                                 original_T=oT, cu_seqlens=cu_seqlens)
    dv = chunk_bwd_dv(q, k, do, dh, g=g, g_gamma=g_gamma, scale=scale, chunk_size=C, original_T=oT,
                      cu_seqlens=cu_seqlens)
    if dg is not None:
        dg = chunk_local_cumsum(dg, C, reverse=True, cu_seqlens=cu_seqlens)
    dq, dk, dv = dq[:, :T0], dk[:, :T0], dv[:, :T0]
    if dg is not None:
        dg = dg[:, :T0]
    return dq, dk, dv, dg, dh0


def chunk_simple_gla(q, k, v, g=None, g_gamma=None, scale=None, initial_state=None,
                     output_final_state=False, cu_seqlens=None, chunk_size=64):
    """Public chunked simple_gla (`tops/cpu/ops/simple_gla/chunk.py:796-889`)."""
    B, T, H, K = q.shape
    assert q.ndim == 4
    assert k.shape == q.shape
    assert v.ndim == 4 and v.shape[:3] == q.shape[:3]
    if g is not None:
        assert g.ndim == 3 and g.shape == q.shape[:3]
    if g_gamma is not None:
        assert g_gamma.ndim == 1 and g_gamma.shape[0] == H
    N = B
    if cu_seqlens is not None:
        assert B == 1
        N = len(cu_seqlens) - 1
        assert all(e > b for b, e in _segments(cu_seqlens)), "Empty segments not supported"
    if initial_state is not None:
        assert initial_state.shape == (N, H, K, v.shape[-1])
        initial_state = initial_state.to(acc_dtype(q.dtype))
    if scale is None:
        scale = K ** -0.5
    o, ht = chunk_simple_gla_fwd(q, k, v, g, g_gamma, scale, initial_state, output_final_state,
                                 chunk_size, cu_seqlens=cu_seqlens)
    return o, (ht if output_final_state else None)


def naive_recurrent_simple_gla(q, k, v, g=None, g_gamma=None, scale=None, initial_state=None,
                               output_final_state=False):
    """Token-by-token ground truth (`tops/cpu/ops/simple_gla/naive.py:30-144`):
    h = h * exp(g_t + g_gamma) + k_t (x) v_t; o_t = (q_t scale)^T h."""
    acc = acc_dtype(q.dtype)
    B, T, H, K = q.shape
    V = v.shape[-1]
    if scale is None:
        scale = K ** -0.5
    qf, kf, vf = q.to(acc), k.to(acc), v.to(acc)
    h = torch.zeros(B, H, K, V, dtype=acc)
    if initial_state is not None:
        h = h + initial_state.to(acc)
    o = []
    for t in range(T):
        decay = torch.zeros(B, H, dtype=acc)
        if g is not None:
            decay = decay + g[:, t].to(acc)
        if g_gamma is not None:
            decay = decay + g_gamma.to(acc)[None]
        h = h * torch.exp(decay)[..., None, None] + kf[:, t][..., None] * vf[:, t][..., None, :]
        o.append(((qf[:, t] * scale)[..., None] * h).sum(-2))
    return torch.stack(o, 1).to(q.dtype), (h if output_final_state else None)
