"""Oracle pieces shared by GLA and simple_gla (test infrastructure only).

Restates `tops/cpu/ops/common/utils.py`, `tops/cpu/ops/common/chunk_h.py` and
`tops/cpu/ops/common/chunk_o.py` of the reference in torch-on-CPU.  All
tensors use the reference layout `[B, T, H, D]`, states `[B, H, K, V]`.

Variable-length (packed) inputs are handled by running the dense code on each
sequence slice, which is what the reference's per-sequence loops amount to
(`chunk_h.py:100-168`, `:292-372`).
"""
from __future__ import annotations

import torch

_HALF = (torch.bfloat16, torch.float16)


def acc_dtype(dtype: torch.dtype) -> torch.dtype:
    """fp64 inputs accumulate in fp64, everything else in fp32
    (`tops/cpu/ops/common/utils.py:189-191`)."""
    return torch.float64 if dtype == torch.float64 else torch.float32


def weak_scalar(x: float, dtype: torch.dtype) -> float:
    """The value a python scalar takes when the reference multiplies an array of `dtype` by it.
    jax.numpy gives the scalar the array's dtype before the operation (weak typing), so `q_bf16 * scale`
    is bf16(q * bf16(scale)); torch keeps the scalar in fp32 and would give bf16(q * scale).  Only half
    types are affected, and only for scalars that are not exactly representable in them."""
    if dtype in (torch.bfloat16, torch.float16):
        return float(torch.tensor(x, dtype=dtype))
    return x


def dot(spec: str, a: torch.Tensor, b: torch.Tensor, acc: torch.dtype) -> torch.Tensor:
    """einsum with accumulator-dtype operands (`utils.py:194-208`): half inputs
    are widened first, which is exact, so the product matches a tensor-core
    dot with fp32 accumulation."""
    return torch.einsum(spec, a.to(acc), b.to(acc))


def cdiv(a: int, b: int) -> int:
    return -(-a // b)


def pad_time(x: torch.Tensor, C: int) -> torch.Tensor:
    """Zero-pad axis 1 to a multiple of C (`utils.py:15-33`)."""
    T = x.shape[1]
    extra = (-T) % C
    if extra == 0:
        return x
    shape = list(x.shape)
    shape[1] = extra
    return torch.cat([x, x.new_zeros(shape)], dim=1)


def prepare_chunk_indices(cu_seqlens, C: int) -> torch.Tensor:
    """(sequence id, chunk-in-sequence) for every chunk of a packed batch
    (`tops/utils.py:71-90`)."""
    cu = [int(x) for x in cu_seqlens]
    rows = []
    for n in range(len(cu) - 1):
        for c in range(cdiv(cu[n + 1] - cu[n], C)):
            rows.append((n, c))
    return torch.tensor(rows, dtype=torch.int32).reshape(-1, 2)


def _segments(cu_seqlens):
    cu = [int(x) for x in cu_seqlens]
    return list(zip(cu[:-1], cu[1:]))


def chunk_local_cumsum(g: torch.Tensor, chunk_size: int, reverse: bool = False,
                       cu_seqlens=None) -> torch.Tensor:
    """Inclusive cumulative sum of the log-gates inside each chunk, along time,
    in the accumulator dtype; `reverse` gives suffix sums.  Works on `[B,T,H]`
    and `[B,T,H,K]` (`tops/cpu/ops/common/chunk_o.py:18-112`).  With
    `cu_seqlens` (packed, B == 1) chunks restart at every sequence start."""
    acc = acc_dtype(g.dtype)
    C = chunk_size
    if cu_seqlens is not None:
        assert g.shape[0] == 1
        out = torch.zeros_like(g, dtype=acc)
        for bos, eos in _segments(cu_seqlens):
            if eos > bos:
                seg = pad_time(g[:, bos:eos], C)
                out[:, bos:eos] = chunk_local_cumsum(seg, C, reverse)[:, : eos - bos]
        return out
    T = g.shape[1]
    assert T % C == 0, f"T ({T}) must be a multiple of chunk_size ({C})"
    x = g.to(acc).reshape(g.shape[0], T // C, C, *g.shape[2:])
    if reverse:
        x = x.flip(2).cumsum(2).flip(2)
    else:
        x = x.cumsum(2)
    return x.reshape(g.shape)


def chunk_fwd_h(k, v, *, g=None, g_gamma=None, gk=None, h0=None,
                output_final_state=False, states_in_fp32=False, chunk_size=64,
                original_T=None, cu_seqlens=None):
    """Chunk-start states of the gated recurrence
    (`tops/cpu/ops/common/chunk_h.py:31-226`).

    For every chunk c: record h_c (in k.dtype unless `states_in_fp32`), then
      scalar gate g      : h *= exp(g_last);  v~ = cast(v * exp(g_last - g))
      constant g_gamma   : h *= exp(gamma*len); v~ = cast(v * exp(gamma*len - gamma*(i+1)))
      per-channel gate gk: h *= exp(gk_last)[:,None]; k~ = cast(k * exp(gk_last - gk))
      h += k~^T v~   (accumulator dtype)
    `g`/`gk` are chunk-local cumulative sums.  Passing g and g_gamma together
    is rejected here (the reference reproduces an upstream variable-reuse
    quirk for that case and its backward refuses it, `chunk_h.py:1-21`).

    Returns (h `[B, NT, H, K, V]`, ht fp32 or None).
    """
    assert not (g is not None and g_gamma is not None), "use g or g_gamma, not both"
    B, T, H, K = k.shape
    V = v.shape[-1]
    C = chunk_size
    acc = acc_dtype(k.dtype)
    if cu_seqlens is not None:
        assert B == 1, f"cu_seqlens requires B=1, got B={B}"
        hs, hts = [], []
        for n, (bos, eos) in enumerate(_segments(cu_seqlens)):
            sl = slice(bos, eos)
            pad = lambda x: None if x is None else pad_time(x[:, sl], C)
            # padded rows of a cumulative gate must repeat the last valid value
            def pad_gate(x):
                if x is None:
                    return None
                seg = x[:, sl]
                extra = (-seg.shape[1]) % C
                if extra:
                    seg = torch.cat([seg, seg[:, -1:].expand(-1, extra, *seg.shape[2:])], 1)
                return seg
            h_n, ht_n = chunk_fwd_h(
                pad(k), pad(v), g=pad_gate(g), g_gamma=g_gamma, gk=pad_gate(gk),
                h0=None if h0 is None else h0[n:n + 1], output_final_state=output_final_state,
                states_in_fp32=states_in_fp32, chunk_size=C, original_T=eos - bos)
            hs.append(h_n)
            hts.append(ht_n)
        return torch.cat(hs, 1), (torch.cat(hts, 0) if output_final_state else None)

    if original_T is None:
        original_T = T
    NT = T // C
    store = acc if k.dtype == torch.float64 else (torch.float32 if states_in_fp32 else k.dtype)
    h = torch.zeros(B, H, K, V, dtype=acc)
    if h0 is not None:
        h = h + h0.to(acc)
    out = []
    for c in range(NT):
        out.append(h.to(store))
        sl = slice(c * C, (c + 1) * C)
        bk, bv = k[:, sl], v[:, sl]
        if g is not None:
            bg = g[:, sl]                                   # [B,C,H]
            last = bg[:, -1]                                # [B,H]
            h = h * torch.exp(last)[:, :, None, None]
            bv = (bv * torch.exp(last[:, None, :, None] - bg[..., None])).to(v.dtype)
        if g_gamma is not None:
            gam = g_gamma.to(acc)
            n_valid = min(C, original_T - c * C)
            last = gam * n_valid                            # [H]
            ramp = gam[None, :] * torch.arange(1, C + 1, dtype=acc)[:, None]   # [C,H]
            ramp = torch.where(torch.arange(C)[:, None] < n_valid, ramp, last[None, :])
            h = h * torch.exp(last)[None, :, None, None]
            bv = (bv * torch.exp(last[None, None, :, None] - ramp[None, :, :, None])).to(v.dtype)
        if gk is not None:
            bgk = gk[:, sl]                                 # [B,C,H,K]
            last = bgk[:, -1]                               # [B,H,K]
            h = h * torch.exp(last)[..., None]
            bk = (bk * torch.exp(last[:, None] - bgk)).to(k.dtype)
        h = h + dot("bchk,bchv->bhkv", bk, bv, acc)
    return torch.stack(out, 1), (h if output_final_state else None)


def chunk_bwd_dh(q, do, *, g=None, g_gamma=None, gk=None, h0=None, dht=None,
                 scale=1.0, chunk_size=64, original_T=None, cu_seqlens=None):
    """Reverse scan of the state gradient (`tops/cpu/ops/common/chunk_h.py:229-427`).

    For c = NT-1 .. 0: record dh_c, then
      q^ = cast(q*scale*exp(gk))  |  cast(cast(q*scale)*exp(g))  |  cast(cast(q*scale)*exp(gamma*(i+1)))
      dh  = dh * exp(gate_last) + q^^T cast(do)
    Starts from `dht` (or zero); `dh0` is returned only when `h0` was given.

    Returns (dh `[B, NT, H, K, V]` accumulator dtype, dh0 or None).
    """
    assert not (g is not None and g_gamma is not None), "use g or g_gamma, not both"
    B, T, H, K = q.shape
    V = do.shape[-1]
    C = chunk_size
    acc = acc_dtype(q.dtype)
    if cu_seqlens is not None:
        assert B == 1, f"cu_seqlens requires B=1, got B={B}"
        dhs, dh0s = [], []
        for n, (bos, eos) in enumerate(_segments(cu_seqlens)):
            sl = slice(bos, eos)

            def pad_gate(x):
                if x is None:
                    return None
                seg = x[:, sl]
                extra = (-seg.shape[1]) % C
                if extra:
                    seg = torch.cat([seg, seg[:, -1:].expand(-1, extra, *seg.shape[2:])], 1)
                return seg
            dh_n, dh0_n = chunk_bwd_dh(
                pad_time(q[:, sl], C), pad_time(do[:, sl], C), g=pad_gate(g), g_gamma=g_gamma,
                gk=pad_gate(gk), h0=None if h0 is None else h0[n:n + 1],
                dht=None if dht is None else dht[n:n + 1], scale=scale, chunk_size=C,
                original_T=eos - bos)
            dhs.append(dh_n)
            dh0s.append(dh0_n)
        return torch.cat(dhs, 1), (torch.cat(dh0s, 0) if h0 is not None else None)

    if original_T is None:
        original_T = T
    NT = T // C
    dh = torch.zeros(B, H, K, V, dtype=acc)
    if dht is not None:
        dh = dh + dht.to(acc)
    out = [None] * NT
    for c in range(NT - 1, -1, -1):
        out[c] = dh
        sl = slice(c * C, (c + 1) * C)
        bq, bdo = q[:, sl], do[:, sl]
        s_in = weak_scalar(scale, q.dtype)      # `b_q * scale` with b_q in q.dtype (chunk_h.py:401-404)
        if gk is not None:
            bgk = gk[:, sl]
            bq = (bq * s_in * torch.exp(bgk)).to(q.dtype)
            dh = dh * torch.exp(bgk[:, -1])[..., None]
        else:
            bq = (bq * s_in).to(q.dtype)
        if g is not None:
            bg = g[:, sl]
            bq = (bq * torch.exp(bg[..., None])).to(q.dtype)
            dh = dh * torch.exp(bg[:, -1])[:, :, None, None]
        if g_gamma is not None:
            gam = g_gamma.to(acc)
            n_valid = min(C, original_T - c * C)
            ramp = gam[None, :] * torch.arange(1, C + 1, dtype=acc)[:, None]
            bq = (bq * torch.exp(ramp)[None, :, :, None]).to(q.dtype)
            dh = dh * torch.exp(gam * n_valid)[None, :, None, None]
        dh = dh + dot("bchk,bchv->bhkv", bq, bdo.to(q.dtype), acc)
    return torch.stack(out, 1), (dh if h0 is not None else None)


def chunk_fwd_o(q, k, v, h, *, g=None, g_gamma=None, scale=1.0, chunk_size=64,
                cu_seqlens=None):
    """simple_gla output: inter-chunk read of the state plus the masked
    intra-chunk product (`tops/cpu/ops/common/chunk_o.py:115-259`):

      o = cast( scale*(q h_c) * exp(G_i) + scale * tril((q k^T) * exp(G_i - G_j)) fp32(v) )

    The intra matrix stays fp32 and v is widened (`:252-254`).  `h` holds one
    state per chunk in packed-chunk order when `cu_seqlens` is given.
    """
    B, T, H, K = q.shape
    V = v.shape[-1]
    C = chunk_size
    acc = acc_dtype(q.dtype)
    if cu_seqlens is not None:
        assert B == 1
        o = torch.zeros(1, T, H, V, dtype=v.dtype)
        c0 = 0
        for bos, eos in _segments(cu_seqlens):
            sl = slice(bos, eos)
            n = cdiv(eos - bos, C)

            def pad_gate(x):
                if x is None:
                    return None
                seg = x[:, sl]
                extra = (-seg.shape[1]) % C
                if extra:
                    seg = torch.cat([seg, seg[:, -1:].expand(-1, extra, *seg.shape[2:])], 1)
                return seg
            o_n = chunk_fwd_o(pad_time(q[:, sl], C), pad_time(k[:, sl], C), pad_time(v[:, sl], C),
                              h[:, c0:c0 + n], g=pad_gate(g), g_gamma=g_gamma, scale=scale,
                              chunk_size=C)
            o[:, sl] = o_n[:, : eos - bos]
            c0 += n
        return o

    NT = T // C
    tril = torch.tril(torch.ones(C, C, dtype=torch.bool))
    outs = []
    for c in range(NT):
        sl = slice(c * C, (c + 1) * C)
        bq, bk, bv = q[:, sl], k[:, sl], v[:, sl]
        bo = dot("bchk,bhkv->bchv", bq, h[:, c].to(q.dtype), acc)
        bA = dot("bchk,bjhk->bchj", bq, bk, acc)
        if g is not None:
            bg = g[:, sl]                                   # [B,C,H]
            bo = bo * torch.exp(bg)[..., None]
            bA = bA * torch.exp(bg[:, :, :, None] - bg.permute(0, 2, 1)[:, None])
        if g_gamma is not None:
            ramp = g_gamma.to(acc)[None, :] * torch.arange(1, C + 1, dtype=acc)[:, None]   # [C,H]
            bo = bo * torch.exp(ramp)[None, :, :, None]
            bA = bA * torch.exp(ramp[None, :, :, None] - ramp.t()[None, None])
        bA = torch.where(tril[None, :, None, :], bA, torch.zeros((), dtype=acc))
        bo = bo * scale + dot("bihj,bjhv->bihv", bA, bv.to(acc), acc) * scale
        outs.append(bo.to(v.dtype))
    return torch.stack(outs, 1).reshape(B, T, H, V)
