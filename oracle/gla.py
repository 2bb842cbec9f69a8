"""Oracle for GLA (per-channel gates) — test infrastructure only.

Restates `tops/cpu/ops/gla/{chunk,naive,fused_recurrent,fused_chunk}.py` of the
reference in torch-on-CPU, keeping its cast points: the forward stores chunk
states in the input dtype, gated operands are rounded to the input dtype where
the reference rounds them, every contraction accumulates in fp32 (fp64 for
fp64 inputs).
"""
from __future__ import annotations

import torch

from .common import (acc_dtype, cdiv, chunk_bwd_dh, chunk_fwd_h, chunk_local_cumsum, dot,
                     pad_time, _segments)


def _tril(C):
    return torch.tril(torch.ones(C, C, dtype=torch.bool))


def _chunks(x, C):
    B, T = x.shape[:2]
    return x.reshape(B, T // C, C, *x.shape[2:])


def chunk_gla_fwd_intra_gk(q, k, g, scale, chunk_size=64):
    """A[i,j] = scale * sum_k q_i exp(G_i - G_0) * k_j exp(G_0 - G_j), unmasked,
    fp32 (`tops/cpu/ops/gla/chunk.py:52-92`).  g is the chunk-local cumsum."""
    B, T, H, K = q.shape
    C = chunk_size
    acc = acc_dtype(q.dtype)
    qc, kc, gc = _chunks(q, C), _chunks(k, C), _chunks(g, C)
    ref = gc[:, :, :1]
    A = dot("bnihk,bnjhk->bnihj", qc * torch.exp(gc - ref), kc * torch.exp(ref - gc), acc) * scale
    return A.reshape(B, T, H, C)


def chunk_gla_fwd_o_gk(q, v, g, A, h, scale, chunk_size=64):
    """o = cast( scale * cast(q exp(G)) . cast(h_c)  +  cast(A) . v )
    (`tops/cpu/ops/gla/chunk.py:100-151`)."""
    B, T, H, K = q.shape
    V = v.shape[-1]
    C = chunk_size
    acc = acc_dtype(q.dtype)
    qg = (_chunks(q, C) * torch.exp(_chunks(g, C))).to(q.dtype)
    o = scale * dot("bnchk,bnhkv->bnchv", qg, h.to(q.dtype), acc)
    o = o + dot("bnihj,bnjhv->bnihv", _chunks(A, C).to(v.dtype), _chunks(v, C), acc)
    return o.to(v.dtype).reshape(B, T, H, V)


def _pack_varlen(tensors, cu_seqlens, C):
    """Lay every sequence out padded to whole chunks, concatenated along time
    (the reference gathers chunks, `tops/cpu/ops/gla/chunk.py:182-210`)."""
    outs = [[] for _ in tensors]
    flat = [0]
    for bos, eos in _segments(cu_seqlens):
        for i, x in enumerate(tensors):
            outs[i].append(pad_time(x[:, bos:eos], C))
        flat.append(flat[-1] + cdiv(eos - bos, C) * C)
    return [torch.cat(o, 1) for o in outs], flat


def _unpack_varlen(x, cu_seqlens, flat, T):
    out = x.new_zeros(1, T, *x.shape[2:])
    for n, (bos, eos) in enumerate(_segments(cu_seqlens)):
        out[:, bos:eos] = x[:, flat[n]:flat[n] + eos - bos]
    return out


def chunk_gla_fwd(q, k, v, g, g_cumsum, scale, initial_state, output_final_state,
                  chunk_size=64, cu_seqlens=None):
    """Forward orchestrator (`tops/cpu/ops/gla/chunk.py:159-269`): pad T,
    cumsum, state scan (states kept in k.dtype), masked intra matrix, output.
    Returns (g_cumsum, A, h, ht, o)."""
    B, T0, H, K = q.shape
    C = chunk_size
    flat = None
    if cu_seqlens is not None:
        assert B == 1
        (q, k, v, g), flat = _pack_varlen([q, k, v, g], cu_seqlens, C)
        g_cumsum = None
    else:
        q, k, v, g = (pad_time(x, C) for x in (q, k, v, g))
    if g_cumsum is None or g_cumsum.shape[1] != q.shape[1]:
        g_cumsum = chunk_local_cumsum(g, C)
    h, ht = chunk_fwd_h(k, v, gk=g_cumsum, h0=initial_state,
                        output_final_state=output_final_state, chunk_size=C,
                        states_in_fp32=False, cu_seqlens=flat)
    A = chunk_gla_fwd_intra_gk(q, k, g_cumsum, scale, C)
    A = torch.where(_tril(C)[None, None, :, None, :], _chunks(A, C),
                    torch.zeros((), dtype=A.dtype)).reshape(A.shape)
    o = chunk_gla_fwd_o_gk(q, v, g_cumsum, A, h, scale, C)
    if cu_seqlens is not None:
        o = _unpack_varlen(o, cu_seqlens, flat, T0)
        return g_cumsum, A, h, ht, o
    return g_cumsum[:, :T0], A[:, :T0], h, ht, o[:, :T0]


def chunk_gla_bwd_dA(v, do, scale, chunk_size=64):
    """dA = tril(do v^T) * scale, fp32 (`tops/cpu/ops/gla/chunk.py:277-302`)."""
    B, T, H, V = v.shape
    C = chunk_size
    acc = acc_dtype(v.dtype)
    dA = dot("bnihv,bnjhv->bnihj", _chunks(do, C), _chunks(v, C), acc) * scale
    dA = torch.where(_tril(C)[None, None, :, None, :], dA, torch.zeros((), dtype=acc))
    return dA.reshape(B, T, H, C)


def chunk_gla_bwd_dv(k, g_cumsum, A, do, dh, chunk_size=64):
    """dv = cast( A^T fp32(do) + cast(k exp(G_n - G)) . cast(dh_c) )
    (`tops/cpu/ops/gla/chunk.py:310-349`)."""
    B, T, H, K = k.shape
    V = do.shape[-1]
    C = chunk_size
    acc = acc_dtype(k.dtype)
    kc, gc = _chunks(k, C), _chunks(g_cumsum, C)
    dv = dot("bnihj,bnihv->bnjhv", _chunks(A, C), _chunks(do, C).to(acc), acc)
    kd = (kc * torch.exp(gc[:, :, -1:] - gc)).to(k.dtype)
    dv = dv + dot("bnchk,bnhkv->bnchv", kd, dh.to(k.dtype), acc)
    return dv.to(do.dtype).reshape(B, T, H, V)


def chunk_gla_bwd_dqk_intra(q, k, g_cumsum, dA, chunk_size=64):
    """dq = exp(G) * (dA . (k exp(-G))),  dk = exp(-G) * (dA^T . (q exp(G))), fp32
    (`tops/cpu/ops/gla/chunk.py:357-388`)."""
    B, T, H, K = q.shape
    C = chunk_size
    acc = acc_dtype(q.dtype)
    qc, kc, gc, dAc = (_chunks(x, C) for x in (q, k, g_cumsum, dA))
    dq = torch.exp(gc) * dot("bnihj,bnjhk->bnihk", dAc, kc.to(acc) * torch.exp(-gc), acc)
    dk = torch.exp(-gc) * dot("bnihj,bnihk->bnjhk", dAc, qc.to(acc) * torch.exp(gc), acc)
    return dq.reshape(B, T, H, K), dk.reshape(B, T, H, K)


def chunk_gla_bwd_dqkg(q, k, v, h, g_cumsum, do, dh, dq, dk, scale, chunk_size=64):
    """Inter-chunk parts of dq/dk and the gate gradient, fp32
    (`tops/cpu/ops/gla/chunk.py:396-461`):
      dq += scale exp(G) * (do . cast(h_c)^T);  dk += exp(G_n - G) * (v . cast(dh_c)^T)
      dg  = suffix_sum_chunk(q dq - k dk) + [exp(G_n) sum_v h_c dh_c + sum_i dk_inter k]
    """
    B, T, H, K = q.shape
    C = chunk_size
    acc = acc_dtype(q.dtype)
    qc, kc, vc, gc, doc, dqc, dkc = (_chunks(x, C) for x in (q, k, v, g_cumsum, do, dq, dk))
    gn = gc[:, :, -1]
    dq_inter = scale * torch.exp(gc) * dot("bnchv,bnhkv->bnchk", doc, h.to(do.dtype), acc)
    dk_inter = torch.exp(gn[:, :, None] - gc) * dot("bnchv,bnhkv->bnchk", vc, dh.to(v.dtype), acc)
    dq_t, dk_t = dqc + dq_inter, dkc + dk_inter
    dg_chunk = torch.exp(gn) * dot("bnhkv,bnhkv->bnhk", h.to(acc), dh, acc) \
        + (dk_inter * kc.to(acc)).sum(2)
    raw = qc.to(acc) * dq_t - kc.to(acc) * dk_t
    dg = raw.flip(2).cumsum(2).flip(2) + dg_chunk[:, :, None]
    return dq_t.reshape(B, T, H, K), dk_t.reshape(B, T, H, K), dg.reshape(B, T, H, K)


def chunk_gla_bwd(q, k, v, g, g_cumsum, scale, initial_state, h, A, do, dht,
                  chunk_size=64, cu_seqlens=None):
    """Backward orchestrator (`tops/cpu/ops/gla/chunk.py:469-640`): recompute
    the cumsum, fp32 chunk states and the intra matrix, reverse-scan dh, then
    dv, dA, dq/dk (intra + inter) and dg.
    Returns (dq fp32, dk fp32, dv do.dtype, dg fp32, dh0 fp32 or None)."""
    B, T0, H, K = q.shape
    C = chunk_size
    flat = None
    if cu_seqlens is not None:
        assert B == 1
        (q, k, v, g, do), flat = _pack_varlen([q, k, v, g, do], cu_seqlens, C)
        g_cumsum = h = A = None
    else:
        q, k, v, g, do = (pad_time(x, C) for x in (q, k, v, g, do))
    Tp = q.shape[1]
    if g_cumsum is None or g_cumsum.shape[1] != Tp:
        g_cumsum = chunk_local_cumsum(g, C)
    if h is None:
        h, _ = chunk_fwd_h(k, v, gk=g_cumsum, h0=initial_state, output_final_state=False,
                           chunk_size=C, states_in_fp32=True, cu_seqlens=flat)
    dh, dh0 = chunk_bwd_dh(q, do, gk=g_cumsum, h0=initial_state, dht=dht, scale=scale,
                           chunk_size=C, cu_seqlens=flat)
    if A is None or A.shape[1] != Tp:
        A = chunk_gla_fwd_intra_gk(q, k, g_cumsum, scale, C)
        A = torch.where(_tril(C)[None, None, :, None, :], _chunks(A, C),
                        torch.zeros((), dtype=A.dtype)).reshape(A.shape)
    dv = chunk_gla_bwd_dv(k, g_cumsum, A, do, dh, C)
    dA = chunk_gla_bwd_dA(v, do, scale, C)
    dq, dk = chunk_gla_bwd_dqk_intra(q, k, g_cumsum, dA, C)
    dq, dk, dg = chunk_gla_bwd_dqkg(q, k, v, h, g_cumsum, do, dh, dq, dk, scale, C)
    if cu_seqlens is not None:
        dq, dk, dv, dg = (_unpack_varlen(x, cu_seqlens, flat, T0) for x in (dq, dk, dv, dg))
    else:
        dq, dk, dv, dg = (x[:, :T0] for x in (dq, dk, dv, dg))
    return dq, dk, dv, dg, dh0


def chunk_gla(q, k, v, g=None, scale=None, initial_state=None, output_final_state=False,
              cu_seqlens=None, chunk_size=16):
    """Public chunked GLA (`tops/cpu/ops/gla/chunk.py:648-709`): g defaults to
    zeros, scale to K^-0.5, chunk_size to 16; o in v.dtype, final state fp32."""
    B, T, H, K = q.shape
    V = v.shape[-1]
    if cu_seqlens is not None:
        assert B == 1, f"B must be 1 for varlen, got {B}"
        N = len(cu_seqlens) - 1
        assert all(e > b for b, e in _segments(cu_seqlens)), "Empty segments not supported"
        if initial_state is not None:
            assert initial_state.shape == (N, H, K, V)
    if g is None:
        g = torch.zeros_like(q)
    if scale is None:
        scale = K ** -0.5
    if initial_state is not None:
        initial_state = initial_state.to(acc_dtype(q.dtype))
    _, _, _, ht, o = chunk_gla_fwd(q, k, v, g, None, scale, initial_state, output_final_state,
                                   chunk_size=chunk_size, cu_seqlens=cu_seqlens)
    return o, (ht if output_final_state else None)


def fused_chunk_gla(q, k, v, g=None, scale=None, initial_state=None,
                    output_final_state=False, cu_seqlens=None, chunk_size=16):
    """Alias of `chunk_gla` (`tops/cpu/ops/gla/fused_chunk.py:4-44`)."""
    return chunk_gla(q, k, v, g, scale, initial_state, output_final_state, cu_seqlens, chunk_size)


def naive_recurrent_gla(q, k, v, gk, initial_state=None, output_final_state=False):
    """Token-by-token ground truth (`tops/cpu/ops/gla/naive.py:30-105`):
    h = h*exp(gk_t) + k_t (x) v_t; o_t = (q_t K^-0.5)^T h.  scale is fixed."""
    acc = acc_dtype(q.dtype)
    B, T, H, K = q.shape
    V = v.shape[-1]
    qf, kf, vf, gf = (x.to(acc) for x in (q, k, v, gk))
    h = torch.zeros(B, H, K, V, dtype=acc)
    if initial_state is not None:
        h = h + initial_state.to(acc)
    o = torch.zeros(B, T, H, V, dtype=acc)
    for t in range(T):
        h = h * torch.exp(gf[:, t])[..., None] + kf[:, t][..., None] * vf[:, t][..., None, :]
        o[:, t] = ((qf[:, t] * K ** -0.5)[..., None] * h).sum(-2)
    return o.to(q.dtype), (h if output_final_state else None)


def _recurrent_ranges(B, T, cu_seqlens):
    if cu_seqlens is None:
        return [(b, 0, T) for b in range(B)]
    return [(0, bos, eos) for bos, eos in _segments(cu_seqlens)]


def fused_recurrent_fwd(q, k, v, gk=None, gv=None, scale=None, initial_state=None,
                        output_final_state=False, reverse=False, cu_seqlens=None):
    """Recurrent forward, all math in the accumulator dtype, o returned fp32
    (`tops/cpu/ops/gla/fused_recurrent.py:51-162`)."""
    acc = acc_dtype(q.dtype)
    B, T, H, K = q.shape
    V = v.shape[-1]
    if scale is None:
        scale = K ** -0.5
    qf, kf, vf = q.to(acc), k.to(acc), v.to(acc)
    gkf = None if gk is None else gk.to(acc)
    gvf = None if gv is None else gv.to(acc)
    o = torch.zeros(B, T, H, V, dtype=acc)
    hts = []
    for n, (b, bos, eos) in enumerate(_recurrent_ranges(B, T, cu_seqlens)):
        h = torch.zeros(H, K, V, dtype=acc)
        if initial_state is not None:
            h = h + initial_state[n].to(acc)
        steps = range(eos - 1, bos - 1, -1) if reverse else range(bos, eos)
        for t in steps:
            if gkf is not None:
                h = h * torch.exp(gkf[b, t])[:, :, None]
            if gvf is not None:
                h = h * torch.exp(gvf[b, t])[:, None, :]
            h = h + kf[b, t][:, :, None] * vf[b, t][:, None, :]
            o[b, t] = (h * (qf[b, t] * scale)[:, :, None]).sum(1)
        hts.append(h)
    return o, (torch.stack(hts) if output_final_state else None)


def fused_recurrent_bwd(q, k, v, gk=None, gv=None, o=None, do=None, dht=None, scale=None,
                        initial_state=None, reverse=False, cu_seqlens=None):
    """Two-pass recurrent backward (`tops/cpu/ops/gla/fused_recurrent.py:171-353`):
    replay -> dq and the final state; reverse -> dk, dv, running gate gradients
    (seeded with sum(h_final * dht)), dh0.  Outputs cast to input dtypes."""
    acc = acc_dtype(q.dtype)
    B, T, H, K = q.shape
    V = v.shape[-1]
    if scale is None:
        scale = K ** -0.5
    assert do is not None
    if gv is not None:
        assert o is not None, "o (forward output) required when gv is used"
    qf, kf, vf, dof = q.to(acc), k.to(acc), v.to(acc), do.to(acc)
    gkf = None if gk is None else gk.to(acc)
    gvf = None if gv is None else gv.to(acc)
    of = None if gv is None else o.to(acc)
    dq = torch.zeros(B, T, H, K, dtype=acc)
    dk = torch.zeros(B, T, H, K, dtype=acc)
    dv = torch.zeros(B, T, H, V, dtype=acc)
    dgk = None if gk is None else torch.zeros(B, T, H, K, dtype=acc)
    dgv = None if gv is None else torch.zeros(B, T, H, V, dtype=acc)
    dh0s = []
    for n, (b, bos, eos) in enumerate(_recurrent_ranges(B, T, cu_seqlens)):
        h = torch.zeros(H, K, V, dtype=acc)
        if initial_state is not None:
            h = h + initial_state[n].to(acc)
        fwd = range(eos - 1, bos - 1, -1) if reverse else range(bos, eos)
        for t in fwd:
            if gkf is not None:
                h = h * torch.exp(gkf[b, t])[:, :, None]
            if gvf is not None:
                h = h * torch.exp(gvf[b, t])[:, None, :]
            h = h + kf[b, t][:, :, None] * vf[b, t][:, None, :]
            dq[b, t] = scale * (h * dof[b, t][:, None, :]).sum(2)
        dh = torch.zeros(H, K, V, dtype=acc)
        if dht is not None:
            dh = dh + dht[n].to(acc)
        run_k = (h * dh).sum(2)
        run_v = (h * dh).sum(1)
        for t in reversed(list(fwd)):
            dh = dh + (qf[b, t] * scale)[:, :, None] * dof[b, t][:, None, :]
            dk_t = (dh * vf[b, t][:, None, :]).sum(2)
            dv_t = (dh * kf[b, t][:, :, None]).sum(1)
            dk[b, t], dv[b, t] = dk_t, dv_t
            if gkf is not None:
                run_k = run_k + qf[b, t] * dq[b, t] - kf[b, t] * dk_t
                dgk[b, t] = run_k
                dh = dh * torch.exp(gkf[b, t])[:, :, None]
            if gvf is not None:
                run_v = run_v + of[b, t] * dof[b, t] - vf[b, t] * dv_t
                dgv[b, t] = run_v
                dh = dh * torch.exp(gvf[b, t])[:, None, :]
        dh0s.append(dh)
    dh0 = torch.stack(dh0s).to(initial_state.dtype) if initial_state is not None else None
    return (dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype),
            None if gk is None else dgk.to(gk.dtype),
            None if gv is None else dgv.to(gv.dtype), dh0)


def fused_recurrent_gla(q, k, v, gk=None, gv=None, scale=None, initial_state=None,
                        output_final_state=False, reverse=False, cu_seqlens=None):
    """Public recurrent GLA (`tops/cpu/ops/gla/fused_recurrent.py:362-422`):
    shape asserts, then the fp32 forward with o cast to q.dtype."""
    B, T, H, K = q.shape
    V = v.shape[-1]
    N = len(cu_seqlens) - 1 if cu_seqlens is not None else B
    assert k.shape == (B, T, H, K)
    assert v.shape[:3] == (B, T, H)
    assert gk is None or gk.shape == (B, T, H, K)
    assert gv is None or gv.shape == (B, T, H, V)
    assert initial_state is None or initial_state.shape == (N, H, K, V)
    assert cu_seqlens is None or B == 1
    o, ht = fused_recurrent_fwd(q, k, v, gk, gv, scale, initial_state, output_final_state,
                                reverse, cu_seqlens)
    return o.to(q.dtype), ht
