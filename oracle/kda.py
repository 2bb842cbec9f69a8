"""Oracle for KDA (Kimi delta attention: per-channel decay plus a beta-weighted
delta-rule update) — test infrastructure only.

Restates, in torch-on-CPU, `tops/cpu/ops/kda/naive.py` (token recurrence and
chunked WY form) and the explicit token-level backward of
`tops/cpu/ops/kda/fused_recurrent.py:212-418`.  The gate `g` is a natural-log
decay per key channel; q and k are used as given (no normalisation inside).
"""
from __future__ import annotations

import torch

from .common import acc_dtype, cdiv, pad_time


def _check(q, k, v, g, beta, initial_state):
    assert q.ndim == 4, f"q must be 4D [B,T,H,K], got {q.ndim}D"
    assert k.shape == q.shape
    assert v.ndim == 4 and v.shape[:3] == q.shape[:3]
    assert g.ndim == 4 and g.shape == q.shape
    assert beta.ndim == 3 and beta.shape == q.shape[:3]
    B, T, H, K = q.shape
    V = v.shape[-1]
    if initial_state is not None:
        assert initial_state.shape == (B, H, K, V)
    return B, T, H, K, V


def naive_recurrent_kda(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False):
    """Ground truth (`tops/cpu/ops/kda/naive.py:10-118`), all in the accumulator dtype:
        S' = S exp(g_t)[:,None];  r = v_t - k_t^T S';  S = S' + (beta_t k_t) (x) r;  o_t = (q_t scale)^T S
    o is cast to v.dtype, the final state stays fp32."""
    B, T, H, K, V = _check(q, k, v, g, beta, initial_state)
    acc = acc_dtype(q.dtype)
    if scale is None:
        scale = K ** -0.5
    qf, kf, vf, gf, bf = (x.to(acc) for x in (q, k, v, g, beta))
    S = torch.zeros(B, H, K, V, dtype=acc)
    if initial_state is not None:
        S = S + initial_state.to(acc)
    outs = []
    for t in range(T):
        S = S * torch.exp(gf[:, t])[..., None]
        r = vf[:, t] - (kf[:, t][..., None] * S).sum(-2)
        S = S + (bf[:, t][..., None] * kf[:, t])[..., None] * r[..., None, :]
        outs.append(((qf[:, t] * scale)[..., None] * S).sum(-2))
    return torch.stack(outs, 1).to(v.dtype), (S if output_final_state else None)


def naive_chunk_kda(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False, chunk_size=64):
    """Chunked WY form (`tops/cpu/ops/kda/naive.py:121-313`).  Per chunk, with G the
    chunk-local cumulative gate:
        A0[c,i] = beta_c sum_k k_c k_i exp(G_c - G_i)   (i < c)
        Tm = (I + A0)^-1 diag(beta)          (forward substitution)
        w = Tm (exp(G) k),  u = Tm v
        v' = u - w S;  o = (q scale exp(G)) S + tril(Aqk) v';  S = S exp(G_n) + (k exp(G_n - G))^T v'
        Aqk[c,j] = sum_k q_c scale exp(G_c - G_j) k_j
    """
    B, T0, H, K, V = _check(q, k, v, g, beta, initial_state)
    acc = acc_dtype(q.dtype)
    C = chunk_size
    if scale is None:
        scale = K ** -0.5
    q, k, v, g = (pad_time(x, C) for x in (q, k, v, g))
    beta = pad_time(beta, C)
    T = q.shape[1]
    NT = T // C
    # [B,H,NT,C,D]
    q, k, v, g = (x.to(acc).permute(0, 2, 1, 3).reshape(B, H, NT, C, -1) for x in (q, k, v, g))
    beta = beta.to(acc).permute(0, 2, 1).reshape(B, H, NT, C)
    q = q * scale
    G = g.cumsum(3)
    # A0[c,i] = beta_c sum_k k_c k_i exp(G_c - G_i), strictly below the diagonal
    A0 = (k[..., :, None, :] * k[..., None, :, :] * torch.exp(G[..., :, None, :] - G[..., None, :, :])).sum(-1)
    A0 = torch.tril(A0 * beta[..., None], -1)
    # (I + A0)^-1 diag(beta): what the reference's row-by-row forward substitution produces (:237-243)
    eye = torch.eye(C, dtype=acc).expand(A0.shape)
    A = torch.linalg.solve_triangular(eye + A0, eye, upper=False) * beta[..., None, :]
    w = A @ (torch.exp(G) * k)
    u = A @ v
    S = torch.zeros(B, H, K, V, dtype=acc)
    if initial_state is not None:
        S = S + initial_state.to(acc)
    strict_upper = torch.triu(torch.ones(C, C, dtype=torch.bool), 1)
    outs = []
    for n in range(NT):
        qn, kn, un, Gn, wn = q[:, :, n], k[:, :, n], u[:, :, n], G[:, :, n], w[:, :, n]
        Aqk = torch.einsum("bhck,bhjk->bhcj", qn * torch.exp(Gn), kn * torch.exp(-Gn))
        Aqk = torch.where(strict_upper, torch.zeros((), dtype=acc), Aqk)
        vc = un - wn @ S
        outs.append(torch.einsum("bhck,bhkv->bhcv", qn * torch.exp(Gn), S) + Aqk @ vc)
        last = Gn[:, :, -1]
        S = S * torch.exp(last)[..., None] + torch.einsum("bhck,bhcv->bhkv", torch.exp(last[:, :, None] - Gn) * kn, vc)
    o = torch.stack(outs, 2).reshape(B, H, T, V).permute(0, 2, 1, 3)[:, :T0]
    return o.to(v.dtype), (S if output_final_state else None)


def fused_recurrent_kda(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False):
    """Public recurrent KDA (`tops/ops/kda/fused_recurrent.py:19-105`,
    `tops/cpu/ops/kda/fused_recurrent.py:524-565` with its default flags): the
    same recurrence, o in q.dtype."""
    o, S = naive_recurrent_kda(q, k, v, g, beta, scale, initial_state, output_final_state)
    return o.to(q.dtype), S


def fused_recurrent_kda_bwd(q, k, v, g, beta, do, scale=None, initial_state=None, dht=None):
    """Explicit token-level backward (`tops/cpu/ops/kda/fused_recurrent.py:212-418`).
    Replay stores h'_t (decayed state before the delta update); reverse pass:
        dh += (q scale) (x) do;  e = v - k^T h';  de = beta (k^T dh)
        dk = beta sum_v dh e - sum_v de h';  dv = de;  dbeta = sum_v (k^T dh) e
        dh' = dh - k (x) de;  dg = sum_v dh' h';  dh = dh' exp(g)
    Returns (dq, dk, dv, dg, dbeta in input dtypes, dh0 fp32 or None)."""
    B, T, H, K, V = _check(q, k, v, g, beta, initial_state)
    acc = acc_dtype(q.dtype)
    if scale is None:
        scale = K ** -0.5
    qf, kf, vf, gf, bf, dof = (x.to(acc) for x in (q, k, v, g, beta, do))
    h = torch.zeros(B, H, K, V, dtype=acc)
    if initial_state is not None:
        h = h + initial_state.to(acc)
    hp_all = []
    dq = torch.zeros(B, T, H, K, dtype=acc)
    for t in range(T):
        hp = h * torch.exp(gf[:, t])[..., None]
        hp_all.append(hp)
        e = vf[:, t] - (kf[:, t][..., None] * hp).sum(-2)
        h = hp + (bf[:, t][..., None] * kf[:, t])[..., None] * e[..., None, :]
        dq[:, t] = (h * dof[:, t][..., None, :]).sum(-1) * scale
    dh = torch.zeros(B, H, K, V, dtype=acc)
    if dht is not None:
        dh = dh + dht.to(acc)
    dk = torch.zeros(B, T, H, K, dtype=acc)
    dv = torch.zeros(B, T, H, V, dtype=acc)
    dg = torch.zeros(B, T, H, K, dtype=acc)
    db = torch.zeros(B, T, H, dtype=acc)
    for t in range(T - 1, -1, -1):
        hp = hp_all[t]
        kt, bt = kf[:, t], bf[:, t]
        dh = dh + (qf[:, t] * scale)[..., None] * dof[:, t][..., None, :]
        e = vf[:, t] - (kt[..., None] * hp).sum(-2)
        ktdh = (dh * kt[..., None]).sum(-2)
        de = bt[..., None] * ktdh
        dk[:, t] = bt[..., None] * (dh * e[..., None, :]).sum(-1) - (de[..., None, :] * hp).sum(-1)
        dv[:, t] = de
        db[:, t] = (ktdh * e).sum(-1)
        dhp = dh - kt[..., None] * de[..., None, :]
        dg[:, t] = (dhp * hp).sum(-1)
        dh = dhp * torch.exp(gf[:, t])[..., None]
    dh0 = dh if initial_state is not None else None
    return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype), dg.to(g.dtype), db.to(beta.dtype), dh0


def chunk_kda(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False, cu_seqlens=None,
              chunk_size=64):
    """Public chunked KDA (`tops/ops/kda/chunk.py:193-216`): output and final state of
    the recurrence; here through the chunked WY form."""
    assert cu_seqlens is None
    return naive_chunk_kda(q, k, v, g, beta, scale, initial_state, output_final_state, chunk_size)
