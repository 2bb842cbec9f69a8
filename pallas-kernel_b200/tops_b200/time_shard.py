"""Sharding ONE long sequence over time across ranks (one process per GPU).

The reference has no multi-device path; its primitive for carrying a
recurrence across calls is `initial_state` / `output_final_state`
(`tops/cpu/ops/gla/chunk.py:655-656,694-709`) and its kernel tests check that
two halves chained through the state equal one pass
(`tests/ops/gla/test_pallas_chunk_gla.py:223-247`).  This module generalises
that to R ranks with one small exchange per direction:

forward   rank r owns tokens [r T/R, (r+1) T/R).  Its shard acts on an incoming
          state as  h_out = h_in * exp(P_r) + S_r  with P_r the summed log-gates
          of the shard (per head, or per head and channel) and S_r the shard's
          end state from a zero start.  Every rank computes (P_r, S_r) with the
          state-scan kernel, all ranks all-gather them (fp32 [B,H,K,V] + decay:
          ~2 MiB per rank at H=32, K=V=128), fold the ranks before them locally,
          and then run the ordinary forward with that `initial_state`.
backward  the state gradient flows right to left the same way:
          dh_in(r) = dh_out(r) * exp(P_r) + D_r with D_r the shard's `dh0` for a
          zero `dht`; all-gather D_r, fold the ranks after r, then run the
          ordinary backward with `initial_state = h_in(r)` and `dht = dh_in(r)`.

Remote summaries always land in local memory through the collective before any
kernel reads them.  The local kernels are injected (`LocalOps`) so that the
exchange logic also runs on CPU ranks under gloo with the oracle as local op.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.distributed as dist


@dataclass
class LocalOps:
    """The single-device ops a rank applies to its shard.
    end_state(k, v, g) -> S [B,H,K,V] fp32: state after the shard from a zero start
    grad_start(q, do, g, scale) -> D [B,H,K,V] fp32: dh0 of the shard for dht = 0
    fwd(q, k, v, g, scale, h_in) -> (o, h_out)
    bwd(q, k, v, g, scale, h_in, do, dh_out) -> (dq, dk, dv, dg, dh_in)
    fold(first, decays [R,...], states [R,B,H,K,V], rank, reverse) -> (value entering shard `rank`,
         value pushed through all shards); None: the torch loops of fold_left / fold_right
    """
    end_state: Callable
    grad_start: Callable
    fwd: Callable
    bwd: Callable
    fold: Optional[Callable] = None


def _acc(t: torch.Tensor) -> torch.Tensor:
    return t if t.dtype == torch.float64 else t.float()


def shard_decay(g: torch.Tensor) -> torch.Tensor:
    """Summed log-gates of the shard as a [B,H,K or 1,1] fp32 factor exponent."""
    p = _acc(g).sum(1)                         # [B,H] or [B,H,K]
    return p[..., None, None] if p.ndim == 2 else p[..., None]


def _gather(x: torch.Tensor, group) -> torch.Tensor:
    """All-gather into one [R, ...] tensor (one collective; every shard summary lands in local memory)."""
    world = dist.get_world_size(group)
    x = x.contiguous()
    out = torch.empty((world,) + tuple(x.shape), dtype=x.dtype, device=x.device)
    dist.all_gather(list(out.unbind(0)), x, group=group)   # the views receive in place
    return out


def fold_left(decays, states, h0, rank):
    """State entering rank `rank`: h0 pushed through ranks 0 .. rank-1."""
    h = torch.zeros_like(states[0]) if h0 is None else _acc(h0).clone()
    for s in range(rank):
        h = h * torch.exp(decays[s]) + states[s]
    return h


def fold_right(decays, grads, dht, rank):
    """State gradient leaving rank `rank` on its right: dht pushed through ranks R-1 .. rank+1."""
    d = torch.zeros_like(grads[0]) if dht is None else _acc(dht).clone()
    for s in range(len(grads) - 1, rank, -1):
        d = d * torch.exp(decays[s]) + grads[s]
    return d


def forward(ops: LocalOps, q, k, v, g, scale, initial_state=None, group=None):
    """Forward of this rank's time shard.  `initial_state` is the state before
    token 0 of the whole sequence (same tensor on every rank, or None).
    Returns (o_shard, final_state_of_the_whole_sequence, h_in) — h_in is kept for the backward."""
    rank = dist.get_rank(group)
    P = shard_decay(g)
    S = _acc(ops.end_state(k, v, g))
    decays, states = _gather(P, group), _gather(S, group)
    if ops.fold is not None:
        h_in, final = ops.fold(initial_state, decays, states, rank, False)
    else:
        h_in = fold_left(decays, states, initial_state, rank)
        final = fold_left(decays, states, initial_state, len(states))
    o, _ = ops.fwd(q, k, v, g, scale, h_in)
    return o, final, h_in


def backward(ops: LocalOps, q, k, v, g, scale, h_in, do, dht=None, group=None):
    """Backward of this rank's time shard.  `dht` is the gradient of the final
    state of the whole sequence (same on every rank, or None).  Returns
    (dq, dk, dv, dg of the shard, dh0 of the whole sequence)."""
    rank = dist.get_rank(group)
    P = shard_decay(g)
    D = _acc(ops.grad_start(q, do, g, scale))
    decays, grads = _gather(P, group), _gather(D, group)
    if ops.fold is not None:
        dh_out, dh0 = ops.fold(dht, decays, grads, rank, True)
    else:
        dh_out = fold_right(decays, grads, dht, rank)
        dh0 = fold_right(decays, grads, dht, -1)
    dq, dk, dv, dg, _ = ops.bwd(q, k, v, g, scale, h_in, do, dh_out)
    return dq, dk, dv, dg, dh0


def cuda_ops(kind: str = "simple_gla", chunk_size: int = 64) -> LocalOps:
    """LocalOps on the CUDA kernels of this package; `kind` is "simple_gla"
    (g: [B,T,H]) or "gla" (g: [B,T,H,K]).  Shards the tcgen05 kernels take (bf16 q/k/v and gate,
    K = V = 128, chunk 64, whole chunks) get their summaries from the library's state-exchange entry
    points (`tops_b200_chunk_state_exchange_pack` / `_apply`); other problems from the generic scans."""
    import ctypes as C_

    from . import _lib as L
    from .ops import _chunk, common, gla, simple_gla
    C = chunk_size

    def gates(g):
        gc = common.chunk_local_cumsum(g, C)
        return dict(g=gc) if g.ndim == 3 else dict(gk=gc)

    def pack_problem(x, y, g):
        B, T, H, K = x.shape
        pb = common.make_problem(B, T, H, K, y.shape[-1], C, L.dtype_code(x.dtype), L.dtype_code(g.dtype),
                                 L.GATE_PER_CHANNEL if g.ndim == 4 else L.GATE_SCALAR, 1.0)
        ok = (x.dtype == torch.bfloat16 and g.dtype == torch.bfloat16
              and L.lib.tops_b200_chunk_selected_impl(C_.byref(pb)) == L.IMPL_SM100)
        return pb if ok else None

    # What one shard's calls share: the chunk-start states its forward kept and the workspaces the two
    # pack calls leave behind (the time segments' summaries), which the forward / backward of the same
    # shard take back so that they do not scan the shard a third time.
    kept = {}

    def kind_of(g):
        return L.GATE_PER_CHANNEL if g.ndim == 4 else L.GATE_SCALAR

    def pack(x, y, g, reverse, scale):
        """Shard summary through the tcgen05 summary scan; None when the problem is not one it takes."""
        with torch.cuda.device(x.device):
            pb = pack_problem(x, y, g)
            if pb is None:
                return None
            pb.scale = float(scale)
            B, T, H, K = x.shape
            x, y = x.contiguous(), y.contiguous()
            gk = g.contiguous()
            out = torch.empty(B, H, K, y.shape[-1], dtype=torch.float32, device=x.device)
            p = L.StatePackParams()
            p.pb, p.reverse, p.x, p.g, p.y, p.state_out = pb, int(reverse), L.ptr(x), L.ptr(gk), L.ptr(y), L.ptr(out)
            ws = L.workspace(L.lib.tops_b200_chunk_state_exchange_pack_workspace_bytes(C_.byref(p)), x.device)
            L.check(L.lib.tops_b200_chunk_state_exchange_pack(C_.byref(p), ws.data_ptr(), ws.numel(),
                                                              L.stream_ptr(x.device)), "chunk_state_exchange_pack")
            kept["rev" if reverse else "fwd"] = (x.data_ptr(), ws)
            return out

    def segments(which, x):
        ent = kept.get(which)
        return ent[1] if ent is not None and ent[0] == x.data_ptr() else None

    def end_state(k, v, g):
        s = pack(k, v, g, False, 1.0)
        if s is not None:
            return s
        _, ht = common.chunk_fwd_h(k, v, **gates(g), output_final_state=True, states_in_fp32=True, chunk_size=C)
        return ht

    def grad_start(q, do, g, scale):
        d = pack(q, do, g, True, scale)
        if d is not None:
            return d
        zero = torch.zeros(q.shape[0], q.shape[2], q.shape[3], do.shape[3], dtype=torch.float32, device=q.device)
        _, dh0 = common.chunk_bwd_dh(q, do, **gates(g), h0=zero, dht=None, scale=scale, chunk_size=C)
        return dh0

    def fold(first, decays, states, rank, reverse):
        R, B, H, K, V = states.shape
        with torch.cuda.device(states.device):
            P = decays.float().expand(R, B, H, K, 1).contiguous()
            S = states.float().contiguous()
            f = None if first is None else first.float().contiguous()
            out_in, out_all = torch.empty_like(S[0]), torch.empty_like(S[0])
            p = L.StateApplyParams()
            p.R, p.rank, p.reverse, p.BH, p.K, p.V = R, rank, int(reverse), B * H, K, V
            p.first, p.P, p.S, p.out_in, p.out_all = L.ptr(f), L.ptr(P), L.ptr(S), L.ptr(out_in), L.ptr(out_all)
            L.check(L.lib.tops_b200_chunk_state_exchange_apply(C_.byref(p), L.stream_ptr(S.device)),
                    "chunk_state_exchange_apply")
        return out_in, out_all

    def fast(q, v, g):
        return pack_problem(q, v, g) is not None

    if kind == "simple_gla":
        def fwd(q, k, v, g, scale, h_in):
            if fast(q, v, g):   # the tcgen05 kernels in their scalar-gate form, segment summaries reused
                o, ht, _, _, hs = _chunk.chunk_fwd_call(q, k, v, g, kind_of(g), scale, h_in,
                                                        True, C, want_saved=True, segments=segments("fwd", k))
                kept["hs"] = (q.data_ptr(), hs)
                return o, ht
            return simple_gla.chunk_simple_gla_fwd(q, k, v, g, None, scale, h_in, True, C)

        def bwd(q, k, v, g, scale, h_in, do, dh_out):
            if fast(q, v, g):
                hs = kept.get("hs")
                hs = hs[1] if hs is not None and hs[0] == q.data_ptr() else None
                return _chunk.chunk_bwd_call(q, k, v, g, kind_of(g), scale, h_in, do, dh_out,
                                             C, q.dtype, True, True, h_saved=hs, rev_segments=segments("rev", q))
            return simple_gla.chunk_simple_gla_bwd(q, k, v, g, None, h_in, do, dh_out, scale, C)
    else:
        def fwd(q, k, v, g, scale, h_in):
            if fast(q, v, g):
                o, ht, _, _, hs = _chunk.chunk_fwd_call(q, k, v, g, L.GATE_PER_CHANNEL, scale, h_in, True, C,
                                                        want_saved=True, segments=segments("fwd", k))
                kept["hs"] = (q.data_ptr(), hs)
                return o, ht
            o, ht = gla.chunk_gla(q, k, v, g, scale=scale, initial_state=h_in, output_final_state=True, chunk_size=C)
            return o, ht

        def bwd(q, k, v, g, scale, h_in, do, dh_out):
            if fast(q, v, g):
                hs = kept.get("hs")
                hs = hs[1] if hs is not None and hs[0] == q.data_ptr() else None
                return _chunk.chunk_bwd_call(q, k, v, g, L.GATE_PER_CHANNEL, scale, h_in, do, dh_out, C, torch.float32,
                                             True, True, h_saved=hs, rev_segments=segments("rev", q))
            return gla.chunk_gla_bwd(q, k, v, g, None, scale, h_in, None, None, do, dh_out, C)
    return LocalOps(end_state, grad_start, fwd, bwd, fold)


# ---------------------------------------------------------------------------------------------------
# KDA: the delta rule's transition is not diagonal.  A shard acts on an incoming state as
#     h_out = M_r h_in + S_r,     M_r [B,H,K,K] dense,
# and on the state gradient leaving it as  dh_in = M_r^T dh_out + D_r  (the reverse scan is linear in dh and
# its coefficients depend on q, k, g, beta only).  M_r is what the ordinary forward returns as final state
# for v = 0 and initial_state = I (V = K), so no extra kernel is needed; the exchange is one all-gather of
# (M_r, S_r) forward and one of D_r backward, 2 MiB per tensor and rank at H = 32, K = V = 128.
# ---------------------------------------------------------------------------------------------------
@dataclass
class KdaLocalOps:
    """The single-device KDA ops a rank applies to its shard.
    transition(k, g, beta) -> M [B,H,K,K] fp32
    end_state(k, v, g, beta) -> S [B,H,K,V] fp32: state after the shard from a zero start
    fwd(q, k, v, g, beta, scale, h_in) -> (o, kept): kept is whatever `grad_start` / `bwd` want back
    grad_start(q, k, v, g, beta, scale, h_in, do, kept) -> D [B,H,K,V] fp32: dh0 of the shard for dht = 0
    bwd(q, k, v, g, beta, scale, h_in, do, dh_out, kept) -> (dq, dk, dv, dg, dbeta)
    """
    transition: Callable
    end_state: Callable
    fwd: Callable
    grad_start: Callable
    bwd: Callable


def kda_fold_left(Ms, Ss, h0, rank):
    """State entering rank `rank`: h0 pushed through the affine maps of ranks 0 .. rank-1."""
    h = torch.zeros_like(Ss[0]) if h0 is None else _acc(h0).clone()
    for s in range(rank):
        h = Ms[s] @ h + Ss[s]
    return h


def kda_fold_right(Ms, Ds, dht, rank):
    """State gradient leaving rank `rank` on its right: dht pulled back through ranks R-1 .. rank+1."""
    d = torch.zeros_like(Ds[0]) if dht is None else _acc(dht).clone()
    for s in range(len(Ds) - 1, rank, -1):
        d = Ms[s].transpose(-1, -2) @ d + Ds[s]
    return d


def kda_forward(ops: KdaLocalOps, q, k, v, g, beta, scale, initial_state=None, group=None):
    """Forward of this rank's time shard of ONE KDA sequence (K = V).  Returns
    (o_shard, final_state_of_the_whole_sequence, ctx); ctx goes to kda_backward."""
    assert q.shape[-1] == v.shape[-1], "the transition is obtained from a forward with V = K"
    rank = dist.get_rank(group)
    M = _acc(ops.transition(k, g, beta))
    S = _acc(ops.end_state(k, v, g, beta))
    Ms, Ss = _gather(M, group), _gather(S, group)
    h_in = kda_fold_left(Ms, Ss, initial_state, rank)
    final = kda_fold_left(Ms, Ss, initial_state, len(Ss))
    o, kept = ops.fwd(q, k, v, g, beta, scale, h_in)
    return o, final, dict(Ms=Ms, h_in=h_in, kept=kept)


def kda_backward(ops: KdaLocalOps, q, k, v, g, beta, scale, ctx, do, dht=None, group=None):
    """Backward of this rank's time shard.  Returns (dq, dk, dv, dg, dbeta of the shard, dh0 of the whole
    sequence)."""
    rank = dist.get_rank(group)
    Ms, h_in, kept = ctx["Ms"], ctx["h_in"], ctx["kept"]
    D = _acc(ops.grad_start(q, k, v, g, beta, scale, h_in, do, kept))
    Ds = _gather(D, group)
    dh_out = kda_fold_right(Ms, Ds, dht, rank)
    dh0 = kda_fold_right(Ms, Ds, dht, -1)
    dq, dk, dv, dg, dbeta = ops.bwd(q, k, v, g, beta, scale, h_in, do, dh_out, kept)
    return dq, dk, dv, dg, dbeta, dh0


def kda_cuda_ops() -> KdaLocalOps:
    """KdaLocalOps on the chunked tcgen05 KDA kernels (bf16 q/k/v/g, K = V = 128, whole chunks of 64)."""
    from .ops import kda as K_

    def eye_like(k):
        B, _, H, K = k.shape
        return torch.eye(K, dtype=torch.float32, device=k.device).expand(B, H, K, K).contiguous()

    def transition(k, g, beta):
        assert K_.chunk_kernels_take(k, k, k, g, beta, 64), "time-sharded KDA takes bf16, K = V = 128, T % 64 == 0"
        _, M, _, _, _ = K_._chunk_fwd_call(k, k, torch.zeros_like(k), g, beta, 1.0, eye_like(k), True, 64, False, False)
        return M

    def end_state(k, v, g, beta):
        _, S, _, _, _ = K_._chunk_fwd_call(k, k, v, g, beta, 1.0, None, True, 64, False, False)
        return S

    def fwd(q, k, v, g, beta, scale, h_in):
        o, _, _, _, saved = K_._chunk_fwd_call(q, k, v, g, beta, scale, h_in, False, 64, False, True)
        return o, saved

    def grad_start(q, k, v, g, beta, scale, h_in, do, saved):
        return K_._chunk_bwd_state_gradient(q, k, v, g, beta, do, scale, None, saved)

    def bwd(q, k, v, g, beta, scale, h_in, do, dh_out, saved):
        dq, dk, dv, dg, dbeta, _ = K_._chunk_bwd_call(q, k, v, g, beta, do, scale, dh_out, saved, False, q.dtype)
        return dq, dk, dv, dg, dbeta
    return KdaLocalOps(transition, end_state, fwd, grad_start, bwd)
