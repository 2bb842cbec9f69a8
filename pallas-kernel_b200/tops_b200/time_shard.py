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
    """
    end_state: Callable
    grad_start: Callable
    fwd: Callable
    bwd: Callable


def _acc(t: torch.Tensor) -> torch.Tensor:
    return t if t.dtype == torch.float64 else t.float()


def shard_decay(g: torch.Tensor) -> torch.Tensor:
    """Summed log-gates of the shard as a [B,H,K or 1,1] fp32 factor exponent."""
    p = _acc(g).sum(1)                         # [B,H] or [B,H,K]
    return p[..., None, None] if p.ndim == 2 else p[..., None]


def _gather(x: torch.Tensor, group) -> list:
    world = dist.get_world_size(group)
    out = [torch.empty_like(x) for _ in range(world)]
    dist.all_gather(out, x.contiguous(), group=group)
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
    h_in = fold_left(decays, states, initial_state, rank)
    o, _ = ops.fwd(q, k, v, g, scale, h_in)
    final = fold_left(decays, states, initial_state, len(states))
    return o, final, h_in


def backward(ops: LocalOps, q, k, v, g, scale, h_in, do, dht=None, group=None):
    """Backward of this rank's time shard.  `dht` is the gradient of the final
    state of the whole sequence (same on every rank, or None).  Returns
    (dq, dk, dv, dg of the shard, dh0 of the whole sequence)."""
    rank = dist.get_rank(group)
    P = shard_decay(g)
    D = _acc(ops.grad_start(q, do, g, scale))
    decays, grads = _gather(P, group), _gather(D, group)
    dh_out = fold_right(decays, grads, dht, rank)
    dq, dk, dv, dg, _ = ops.bwd(q, k, v, g, scale, h_in, do, dh_out)
    dh0 = fold_right(decays, grads, dht, -1)
    return dq, dk, dv, dg, dh0


def cuda_ops(kind: str = "simple_gla", chunk_size: int = 64) -> LocalOps:
    """LocalOps on the CUDA kernels of this package; `kind` is "simple_gla"
    (g: [B,T,H]) or "gla" (g: [B,T,H,K])."""
    from .ops import common, gla, simple_gla
    C = chunk_size

    def gates(g):
        gc = common.chunk_local_cumsum(g, C)
        return dict(g=gc) if g.ndim == 3 else dict(gk=gc)

    def end_state(k, v, g):
        _, ht = common.chunk_fwd_h(k, v, **gates(g), output_final_state=True, states_in_fp32=True, chunk_size=C)
        return ht

    def grad_start(q, do, g, scale):
        zero = torch.zeros(q.shape[0], q.shape[2], q.shape[3], do.shape[3], dtype=torch.float32, device=q.device)
        _, dh0 = common.chunk_bwd_dh(q, do, **gates(g), h0=zero, dht=None, scale=scale, chunk_size=C)
        return dh0

    if kind == "simple_gla":
        def fwd(q, k, v, g, scale, h_in):
            return simple_gla.chunk_simple_gla_fwd(q, k, v, g, None, scale, h_in, True, C)

        def bwd(q, k, v, g, scale, h_in, do, dh_out):
            return simple_gla.chunk_simple_gla_bwd(q, k, v, g, None, h_in, do, dh_out, scale, C)
    else:
        def fwd(q, k, v, g, scale, h_in):
            o, ht = gla.chunk_gla(q, k, v, g, scale=scale, initial_state=h_in, output_final_state=True, chunk_size=C)
            return o, ht

        def bwd(q, k, v, g, scale, h_in, do, dh_out):
            return gla.chunk_gla_bwd(q, k, v, g, None, scale, h_in, None, None, do, dh_out, C)
    return LocalOps(end_state, grad_start, fwd, bwd)
