"""Oracle for KDA (Kimi delta attention: per-channel decay plus a beta-weighted
delta-rule update) — test infrastructure only.

Restates, in torch-on-CPU, `tops/cpu/ops/kda/naive.py` (token recurrence and
chunked WY form) and the explicit token-level backward of
`tops/cpu/ops/kda/fused_recurrent.py:212-418`.  The gate `g` is a natural-log
decay per key channel; q and k are used as given (no normalisation inside).
"""
from __future__ import annotations

import torch

from .common import acc_dtype, cdiv, dot, pad_time


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
    out_dtype = v.dtype
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
    return o.to(out_dtype), (S if output_final_state else None)


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


# ---------------------------------------------------------------------------
# Chunked WY / UT-transform form, stage by stage (log2-space cumulative gates,
# as the reference's chunk kernels and their CPU restatements use)
# ---------------------------------------------------------------------------
RCP_LN2 = 1.4426950408889634
LN2 = 0.6931471805599453


def kda_gate_chunk_cumsum(g, chunk_size=64):
    """Chunk-local cumulative sum of the natural-log gate, converted to log2 space
    (`tops/ops/kda/gate.py:19-51`; `tops/cpu/ops/kda/gate.py:182-203` with scale = 1/ln2).
    fp32 (fp64 for fp64 inputs) `[B,T,H,K]`."""
    from .common import chunk_local_cumsum
    return chunk_local_cumsum(g, chunk_size) * RCP_LN2


def _chunked(x, C):
    """[B,T,H,D] -> [B,NT,C,H,D]"""
    B, T = x.shape[:2]
    return x.reshape(B, T // C, C, *x.shape[2:])


def kda_intra_chunk_fwd(q, k, g_cumsum, beta, scale, chunk_size=64):
    """Per-chunk matrices of the forward (`tops/ops/kda/chunk_intra.py:91-165`; built in plain
    JAX by the reference's own test `tests/ops/kda/test_chunk_kda_bwd_tpu.py:56-97`):
        Aqk[i,j] = scale sum_k q_i k_j 2^(G_i - G_j)      (j <= i, else 0)
        Akk      = (I + stril(beta_i sum_k k_i k_j 2^(G_i - G_j)))^-1      (unit lower triangular)
    Both `[B,T,H,C]` in the accumulator dtype (row i of its chunk at token i)."""
    acc = acc_dtype(q.dtype)
    C = chunk_size
    B, T, H, K = q.shape
    qc, kc, gc = (_chunked(x.to(acc), C) for x in (q, k, g_cumsum))
    bc = _chunked(beta.to(acc), C)                                   # [B,NT,C,H]
    # decay[i,j,k] = 2^(G_i - G_j), only ever used for j <= i (where it is <= 1)
    diff = gc[:, :, :, None] - gc[:, :, None, :]                     # [B,NT,C(i),C(j),H,K]
    lower = torch.tril(torch.ones(C, C, dtype=torch.bool))
    dec = torch.where(lower[None, None, :, :, None, None], torch.exp2(diff), torch.zeros((), dtype=acc))
    Aqk = torch.einsum("bnihk,bnijhk,bnjhk->bnihj", qc, dec, kc) * scale
    Lkk = torch.einsum("bnihk,bnijhk,bnjhk->bnihj", kc, dec, kc) * bc[..., None]
    strict = torch.tril(torch.ones(C, C, dtype=torch.bool), -1)
    Lm = torch.where(strict[None, None, :, None, :], Lkk, torch.zeros((), dtype=acc)).permute(0, 1, 3, 2, 4)
    eye = torch.eye(C, dtype=acc).expand(Lm.shape)
    Akk = torch.linalg.solve_triangular(eye + Lm, eye.clone(), upper=False).permute(0, 1, 3, 2, 4)
    return Aqk.reshape(B, T, H, C), Akk.reshape(B, T, H, C)


def recompute_w_u_fwd(k, v, beta, A, q=None, gk=None):
    """u = A (beta v);  w = A (beta k 2^G);  qg = q 2^G;  kg = k 2^(G_n - G)
    (`tops/cpu/ops/kda/wy_fast.py:15-93`).  w, u, qg, kg are cast to the input dtypes."""
    acc = acc_dtype(k.dtype)
    B, T, H, K = k.shape
    C = A.shape[-1]
    kc, vc, Ac = _chunked(k.to(acc), C), _chunked(v.to(acc), C), _chunked(A.to(acc), C)
    bc = _chunked(beta.to(acc), C)
    u = torch.einsum("bnihj,bnjhv->bnihv", Ac, vc * bc[..., None])
    kb = kc * bc[..., None]
    gc = None
    if gk is not None:
        gc = _chunked(gk.to(acc), C)
        kb = kb * torch.exp2(gc)
    w = torch.einsum("bnihj,bnjhk->bnihk", Ac, kb)
    qg = None
    if q is not None:
        qg = (q * torch.exp2(gk)).to(q.dtype) if gk is not None else q
    kg = None
    if gk is not None:
        kg = (kc * torch.exp2(gc[:, :, -1:] - gc)).reshape(B, T, H, K).to(k.dtype)
    return w.reshape(B, T, H, K).to(k.dtype), u.reshape(v.shape).to(v.dtype), qg, kg


def chunk_gated_delta_rule_fwd_h(k, w, u, *, gk=None, initial_state=None, output_final_state=False,
                                 chunk_size=64):
    """Delta-rule state scan (`tops/cpu/ops/common/chunk_delta_h.py:22-113`, exp2 form).  `k` is the
    gated key kg.  Per chunk: store h;  v' = u - w h;  h <- h 2^(G_n) + kg^T v'.
    Returns (h `[B,NT,H,K,V]`, v' `[B,T,H,V]`, final state or None), all in the accumulator dtype."""
    acc = acc_dtype(k.dtype)
    B, T, H, K = k.shape
    V = u.shape[-1]
    C = chunk_size
    kc, wc, uc = _chunked(k, C), _chunked(w, C), _chunked(u, C)
    gc = None if gk is None else _chunked(gk, C)
    h = torch.zeros(B, H, K, V, dtype=acc)
    if initial_state is not None:
        h = h + initial_state.to(acc)
    hs, vn = [], []
    for n in range(T // C):
        hs.append(h)
        vc = uc[:, n].to(acc) - torch.einsum("bchk,bhkv->bchv", wc[:, n].to(acc), h)
        vn.append(vc)
        if gc is not None:
            h = h * torch.exp2(gc[:, n, -1].to(acc))[..., None]
        h = h + dot("bchk,bchv->bhkv", kc[:, n], vc, acc)
    return torch.stack(hs, 1), torch.cat(vn, 1).reshape(B, T, H, V), (h if output_final_state else None)


def chunk_gla_fwd_o_gk_exp2(q, v, g_cumsum, A, h, scale, chunk_size=64):
    """Output of a chunk from the state and the intra-chunk matrix (`tops/ops/gla/chunk.py:1279-1440`
    with use_exp2, as `tops/ops/kda/chunk.py:171-180` calls it; A already carries the scale and the mask):
        o = scale (q 2^G) h + A v."""
    acc = acc_dtype(q.dtype)
    C = chunk_size
    qc, vc, gc, Ac = (_chunked(x.to(acc), C) for x in (q, v, g_cumsum, A))
    o = scale * torch.einsum("bnchk,bnhkv->bnchv", qc * torch.exp2(gc), h.to(acc))
    o = o + torch.einsum("bnihj,bnjhv->bnihv", Ac, vc)
    return o.reshape(v.shape)


def chunk_kda_fwd(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False, chunk_size=64):
    """Chunked forward orchestrator (`tops/ops/kda/chunk.py:25-190`):
    returns (o in v.dtype, final state or None, g_cumsum (log2), Aqk, Akk)."""
    B, T, H, K, V = _check(q, k, v, g, beta, initial_state)
    assert T % chunk_size == 0, f"Sequence length T={T} must be divisible by chunk_size={chunk_size}"
    if scale is None:
        scale = K ** -0.5
    gcs = kda_gate_chunk_cumsum(g, chunk_size)
    Aqk, Akk = kda_intra_chunk_fwd(q, k, gcs, beta, scale, chunk_size)
    w, u, _, kg = recompute_w_u_fwd(k, v, beta, Akk, q=q, gk=gcs)
    h, v_new, ht = chunk_gated_delta_rule_fwd_h(kg, w, u, gk=gcs, initial_state=initial_state,
                                                output_final_state=output_final_state, chunk_size=chunk_size)
    o = chunk_gla_fwd_o_gk_exp2(q, v_new, gcs, Aqk, h, scale, chunk_size)
    return o.to(v.dtype), ht, gcs, Aqk, Akk


def chunk_kda_bwd_dAv(q, k, v_new, do, A, scale, chunk_size=64):
    """Stage 1 (`tops/cpu/ops/kda/chunk_bwd.py:391-517`): dAqk = tril(do v'^T) scale (fp32);
    dv = tril(Aqk)^T do (do.dtype)."""
    acc = acc_dtype(q.dtype)
    C = chunk_size
    vc, doc, Ac = (_chunked(x.to(acc), C) for x in (v_new, do, A))
    lower = torch.tril(torch.ones(C, C, dtype=torch.bool))[None, None, :, None, :]
    Am = torch.where(lower, Ac, torch.zeros((), dtype=acc)).to(do.dtype).to(acc)
    dA = torch.einsum("bnihv,bnjhv->bnihj", doc, vc)
    dA = torch.where(lower, dA * scale, torch.zeros((), dtype=acc))
    dv = torch.einsum("bnihj,bnihv->bnjhv", Am, doc)
    return dA.reshape(A.shape), dv.reshape(do.shape).to(do.dtype)


def chunk_gated_delta_rule_bwd_dhu(q, k, w, do, dv, *, gk, h0=None, dht=None, scale=1.0, chunk_size=64):
    """Stage 2, the reverse scan (`tops/cpu/ops/common/chunk_delta_h.py:116-301`, exp2 form).  `q`, `k`
    are the gated qg = q 2^G and kg = k 2^(G_n - G).  Right to left per chunk:
        store dh;  dv2 = kg dh + dv;  dh <- dh 2^(G_n) + scale qg^T do - w^T dv2.
    Returns (dh `[B,NT,H,K,V]`, dh0 or None, dv2 `[B,T,H,V]`), accumulator dtype."""
    acc = acc_dtype(q.dtype)
    B, T, H, K = q.shape
    V = do.shape[-1]
    C = chunk_size
    qc, kc, wc, gc, doc, dvc = (_chunked(x.to(acc), C) for x in (q, k, w, gk, do, dv))
    dh = torch.zeros(B, H, K, V, dtype=acc)
    if dht is not None:
        dh = dh + dht.to(acc)
    NT = T // C
    dhs, dv2s = [None] * NT, [None] * NT
    for n in range(NT - 1, -1, -1):
        dhs[n] = dh
        dv2 = torch.einsum("bchk,bhkv->bchv", kc[:, n], dh) + dvc[:, n]
        dv2s[n] = dv2
        dh = dh * torch.exp2(gc[:, n, -1])[..., None]
        dh = dh + scale * torch.einsum("bchk,bchv->bhkv", qc[:, n], doc[:, n]) \
            - torch.einsum("bchk,bchv->bhkv", wc[:, n], dv2)
    return torch.stack(dhs, 1), (dh if h0 is not None else None), torch.cat(dv2s, 1).reshape(B, T, H, V)


def chunk_kda_bwd_wy_dqkg_fused(q, k, v, v_new, g, beta, A, h, do, dh, dv, scale, chunk_size=64):
    """Stage 3 (`tops/cpu/ops/kda/chunk_bwd.py:27-383`): the inter-chunk parts of dq, dk, the value
    and beta gradients through u = A (beta v), w = A (beta k 2^G), and the gradient of the solve.
    Returns (dq, dk, dv, db, dg, dAkk); dv in v.dtype, the rest in the accumulator dtype."""
    acc = acc_dtype(q.dtype)
    C = chunk_size
    B, T, H, K = q.shape
    qc, kc, vc, vnc, gc, Ac, doc, dvc = (_chunked(x.to(acc), C) for x in (q, k, v, v_new, g, A, do, dv))
    bc = _chunked(beta.to(acc), C)
    hh, dhh = h.to(acc), dh.to(acc)
    gn = gc[:, :, -1:]                                                # [B,NT,1,H,K]
    eg = torch.exp2(gc)
    dgk = (hh * dhh).sum(-1) * torch.exp2(gn[:, :, 0])                # [B,NT,H,K]
    dq = torch.einsum("bnchv,bnhkv->bnchk", doc, hh) * eg * scale
    dk = torch.einsum("bnchv,bnhkv->bnchk", vnc, dhh) * torch.exp2(gn - gc)
    dw = torch.einsum("bnchv,bnhkv->bnchk", dvc, hh)
    kg = kc * eg
    # u branch
    dA = torch.einsum("bnihv,bnjhv->bnihj", dvc, vc)
    dvb = torch.einsum("bnihj,bnihv->bnjhv", Ac, dvc)
    dv2 = (dvb * bc[..., None]).to(v.dtype)
    db = (dvb * vc).sum(-1)
    # w branch (dw enters with a minus sign: v' = u - w h)
    dA = dA + torch.einsum("bnihk,bnjhk->bnihj", -dw, kg)
    dkgb = torch.einsum("bnihj,bnihk->bnjhk", Ac, -dw)
    db = db + (dkgb * kg).sum(-1)
    kdk = kc * dk
    dgk_sum = dgk + kdk.sum(2)                                        # [B,NT,H,K]
    last = torch.zeros(C, dtype=acc)
    last[-1] = 1
    dg = qc * dq - kdk + last[None, None, :, None, None] * dgk_sum[:, :, None] + kg * dkgb * bc[..., None]
    dk = dk + dkgb * eg * bc[..., None]
    # gradient of the inverse: columns scaled by beta, strict lower part, - A^T (.) A^T
    strict = torch.tril(torch.ones(C, C, dtype=torch.bool), -1)[None, None, :, None, :]
    dA = torch.where(strict, dA * bc.permute(0, 1, 3, 2)[:, :, None], torch.zeros((), dtype=acc))
    Am, dAm = Ac.permute(0, 1, 3, 2, 4), dA.permute(0, 1, 3, 2, 4)    # [B,NT,H,C,C]
    dAm = -(Am.transpose(-1, -2) @ dAm @ Am.transpose(-1, -2))
    dA = torch.where(strict, dAm.permute(0, 1, 3, 2, 4), torch.zeros((), dtype=acc))
    sh = lambda x: x.reshape(B, T, H, -1)
    return sh(dq), sh(dk), dv2.reshape(v.shape), db.reshape(B, T, H), sh(dg), sh(dA)


def chunk_kda_bwd_intra(q, k, g, beta, dAqk, dAkk, dq, dk, db, dg, chunk_size=64):
    """Stage 4 (`tops/cpu/ops/kda/chunk_intra.py:16-228`): gradients through
    Aqk[i,j] = sum_k q_i k_j 2^(G_i-G_j) (j <= i; dAqk carries the scale) and
    Lkk[i,j] = beta_i sum_k k_i k_j 2^(G_i-G_j) (j < i).  The reference walks 16 x 16 sub-blocks;
    the sums are the same taken over the whole chunk at once.
        dg = q dq + k (2 dk_row - dk_total)   with dk_row the Lkk row-side part."""
    acc = acc_dtype(q.dtype)
    C = chunk_size
    B, T, H, K = q.shape
    qc, kc, gc, dAq, dAk = (_chunked(x.to(acc), C) for x in (q, k, g, dAqk, dAkk))
    bc = _chunked(beta.to(acc), C)
    diff = gc[:, :, :, None] - gc[:, :, None, :]
    lower = torch.tril(torch.ones(C, C, dtype=torch.bool))[None, None, :, :, None, None]
    dec = torch.where(lower, torch.exp2(diff), torch.zeros((), dtype=acc))   # [B,NT,i,j,H,K]
    strict = torch.tril(torch.ones(C, C, dtype=torch.bool), -1)[None, None, :, None, :]
    lower2 = torch.tril(torch.ones(C, C, dtype=torch.bool))[None, None, :, None, :]
    dAq = torch.where(lower2, dAq, torch.zeros((), dtype=acc))
    dAk = torch.where(strict, dAk, torch.zeros((), dtype=acc))
    dq_i = torch.einsum("bnihj,bnijhk,bnjhk->bnihk", dAq, dec, kc)
    dk_q = torch.einsum("bnihj,bnijhk,bnihk->bnjhk", dAq, dec, qc)
    dk_row = torch.einsum("bnihj,bnijhk,bnjhk->bnihk", dAk, dec, kc)      # before beta
    db_i = (dk_row * kc).sum(-1)
    dk_row = dk_row * bc[..., None]
    dk_col = torch.einsum("bnihj,bnijhk,bnihk->bnjhk", dAk, dec, kc * bc[..., None])
    dk_i = dk_q + dk_row + dk_col
    dg_i = qc * dq_i + kc * (2 * dk_row - dk_i)
    sh = lambda x: x.reshape(B, T, H, -1)
    return (dq.to(acc) + sh(dq_i), dk.to(acc) + sh(dk_i), db.to(acc) + db_i.reshape(B, T, H),
            dg.to(acc) + sh(dg_i))


def chunk_kda_bwd(q, k, v, beta, Aqk, Akk, scale, initial_state, do, dht, *, g, chunk_size=64):
    """Backward orchestrator (`tops/cpu/ops/kda/chunk_bwd.py:525-668`); `g` is the log2-space chunk
    cumsum the forward returned.  Returns (dq, dk, dv, db, dg, dh0).  The stage formulas differentiate
    2^(G2) = exp(G) through the natural exponent (dG = q dq - k dk ..., no ln 2 factor), so after the
    reverse chunk cumsum dg IS the gradient with respect to the natural-log gate the public op takes:
    it equals autodiff of the token recurrence (pinned in tests/test_oracle_kda.py).  The reference's
    custom_vjp wrapper divides this once more by ln 2 (`tops/ops/kda/chunk.py:246-248`), which no longer
    agrees with autodiff of its own `naive_recurrent_kda`; that rescale is not reproduced."""
    from .common import chunk_local_cumsum
    w, u, qg, kg = recompute_w_u_fwd(k, v, beta, Akk, q=q, gk=g)
    h, v_new, _ = chunk_gated_delta_rule_fwd_h(kg, w, u, gk=g, initial_state=initial_state, chunk_size=chunk_size)
    dAqk, dv0 = chunk_kda_bwd_dAv(q, k, v_new, do, Aqk, scale, chunk_size)
    dh, dh0, dv2 = chunk_gated_delta_rule_bwd_dhu(qg, kg, w, do, dv0, gk=g, h0=initial_state, dht=dht, scale=scale,
                                                  chunk_size=chunk_size)
    dq, dk, dv, db, dg, dAkk = chunk_kda_bwd_wy_dqkg_fused(q, k, v, v_new, g, beta, Akk, h, do, dh, dv2, scale,
                                                           chunk_size)
    dq, dk, db, dg = chunk_kda_bwd_intra(q, k, g, beta, dAqk, dAkk, dq, dk, db, dg, chunk_size)
    dg = chunk_local_cumsum(dg, chunk_size, reverse=True)
    return dq, dk, dv, db, dg, dh0


def chunk_kda_with_grads(q, k, v, g, beta, do, scale=None, initial_state=None, dht=None, chunk_size=64):
    """chunk_kda_fwd followed by chunk_kda_bwd, the residuals handed over as the custom_vjp does
    (`tops/ops/kda/chunk.py:219-252`, without its final dg / ln 2: see chunk_kda_bwd):
    (o, ht, dq, dk, dv, dg (natural-log gate), dbeta, dh0)."""
    if scale is None:
        scale = q.shape[-1] ** -0.5
    o, ht, gcs, Aqk, Akk = chunk_kda_fwd(q, k, v, g, beta, scale, initial_state, True, chunk_size)
    dq, dk, dv, db, dg, dh0 = chunk_kda_bwd(q, k, v, beta, Aqk, Akk, scale, initial_state, do, dht, g=gcs,
                                            chunk_size=chunk_size)
    return o, ht, dq, dk, dv, dg, db, dh0
