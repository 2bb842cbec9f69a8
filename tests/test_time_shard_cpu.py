"""World-size-2 (and 3) gloo ranks on CPU exercise the time-sharding exchange
(tops_b200.time_shard) with the CPU oracle as the local op: the shards'
outputs and gradients must equal one pass over the whole sequence — the
reference's state-split check (tests/ops/gla/test_pallas_chunk_gla.py:223-247)
generalised to R ranks and to the backward direction."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _oracle_ops(kind, C):
    from oracle import common as OC
    from oracle import gla as OG
    from oracle import simple_gla as OS
    from tops_b200.time_shard import LocalOps

    def gates(g):
        gc = OC.chunk_local_cumsum(g, C)
        return dict(g=gc) if g.ndim == 3 else dict(gk=gc)

    def end_state(k, v, g):
        return OC.chunk_fwd_h(k, v, **gates(g), output_final_state=True, states_in_fp32=True, chunk_size=C)[1]

    def grad_start(q, do, g, scale):
        zero = torch.zeros(q.shape[0], q.shape[2], q.shape[3], do.shape[3], dtype=q.dtype)
        return OC.chunk_bwd_dh(q, do, **gates(g), h0=zero, dht=None, scale=scale, chunk_size=C)[1]

    if kind == "simple_gla":
        fwd = lambda q, k, v, g, scale, h: OS.chunk_simple_gla_fwd(q, k, v, g, None, scale, h, True, C)
        bwd = lambda q, k, v, g, scale, h, do, dh: OS.chunk_simple_gla_bwd(q, k, v, g, None, h, do, dh, scale, C)
    else:
        fwd = lambda q, k, v, g, scale, h: OG.chunk_gla(q, k, v, g, scale, h, True, chunk_size=C)
        bwd = lambda q, k, v, g, scale, h, do, dh: OG.chunk_gla_bwd(q, k, v, g, None, scale, h, None, None, do, dh, C)
    return LocalOps(end_state, grad_start, fwd, bwd)


def _worker(rank, world, port, kind, out):
    for p in (ROOT, os.path.join(ROOT, "pallas-kernel_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from tops_b200 import time_shard as TS
        torch.manual_seed(0)
        B, T, H, K, V, C = 1, 48 * world, 2, 8, 12, 16
        dt = torch.float64
        q, k = torch.randn(B, T, H, K, dtype=dt), torch.randn(B, T, H, K, dtype=dt)
        v, do = torch.randn(B, T, H, V, dtype=dt), torch.randn(B, T, H, V, dtype=dt)
        gshape = (B, T, H) if kind == "simple_gla" else (B, T, H, K)
        g = torch.nn.functional.logsigmoid(torch.randn(*gshape, dtype=dt))
        h0, dht = torch.randn(B, H, K, V, dtype=dt), torch.randn(B, H, K, V, dtype=dt)
        ops = _oracle_ops(kind, C)
        scale = K ** -0.5
        sl = slice(rank * T // world, (rank + 1) * T // world)
        o, final, h_in = TS.forward(ops, q[:, sl], k[:, sl], v[:, sl], g[:, sl], scale, h0)
        dq, dk, dv, dg, dh0 = TS.backward(ops, q[:, sl], k[:, sl], v[:, sl], g[:, sl], scale, h_in, do[:, sl], dht)
        # single pass over the whole sequence
        o_ref, ht_ref = ops.fwd(q, k, v, g, scale, h0)
        r = ops.bwd(q, k, v, g, scale, h0, do, dht)
        errs = [(o - o_ref[:, sl]).abs().max().item(), (final - ht_ref).abs().max().item(), (dh0 - r[4]).abs().max().item()]
        errs += [(a - b[:, sl]).abs().max().item() for a, b in zip((dq, dk, dv, dg), r[:4])]
        out[rank] = max(errs)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,kind", [(2, "simple_gla"), (3, "simple_gla"), (2, "gla")])
def test_time_sharded_equals_single_pass(world, kind):
    mgr = mp.get_context("spawn").Manager()
    out = mgr.dict()
    port = 29600 + os.getpid() % 200 + world
    mp.spawn(_worker, args=(world, port, kind, out), nprocs=world, join=True)
    assert len(out) == world
    for r in range(world):
        assert out[r] < 1e-9, (r, out[r])


def test_fold_helpers():
    from tops_b200.time_shard import fold_left, fold_right
    dec = [torch.full((1, 1, 1, 1), -0.5), torch.full((1, 1, 1, 1), -0.25)]
    st = [torch.ones(1, 1, 2, 2), 2 * torch.ones(1, 1, 2, 2)]
    h0 = 4 * torch.ones(1, 1, 2, 2)
    import math
    assert torch.allclose(fold_left(dec, st, h0, 0), h0)
    assert torch.allclose(fold_left(dec, st, h0, 1), h0 * math.exp(-0.5) + 1)
    assert torch.allclose(fold_left(dec, st, h0, 2), (h0 * math.exp(-0.5) + 1) * math.exp(-0.25) + 2)
    assert torch.allclose(fold_right(dec, st, h0, 1), h0)
    assert torch.allclose(fold_right(dec, st, h0, 0), h0 * math.exp(-0.25) + 2)
    assert torch.allclose(fold_right(dec, st, None, -1), torch.full((1, 1, 2, 2), 2 * math.exp(-0.5) + 1))


def _oracle_kda_ops():
    from oracle import kda as OK
    from tops_b200.time_shard import KdaLocalOps

    def transition(k, g, beta):
        B, T, H, K = k.shape
        eye = torch.eye(K, dtype=k.dtype).expand(B, H, K, K).contiguous()
        return OK.naive_recurrent_kda(k, k, torch.zeros_like(k), g, beta, 1.0, eye, True)[1]

    def end_state(k, v, g, beta):
        return OK.naive_recurrent_kda(k, k, v, g, beta, 1.0, None, True)[1]

    def fwd(q, k, v, g, beta, scale, h_in):
        return OK.naive_recurrent_kda(q, k, v, g, beta, scale, h_in, False)[0], None

    def grad_start(q, k, v, g, beta, scale, h_in, do, kept):
        return OK.fused_recurrent_kda_bwd(q, k, v, g, beta, do, scale, h_in, None)[5]

    def bwd(q, k, v, g, beta, scale, h_in, do, dh_out, kept):
        return OK.fused_recurrent_kda_bwd(q, k, v, g, beta, do, scale, h_in, dh_out)[:5]
    return KdaLocalOps(transition, end_state, fwd, grad_start, bwd)


def _kda_worker(rank, world, port, out):
    for p in (ROOT, os.path.join(ROOT, "pallas-kernel_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import kda as OK
        from tops_b200 import time_shard as TS
        torch.manual_seed(1)
        B, T, H, K = 1, 24 * world, 2, 8
        dt = torch.float64
        q, k = torch.randn(B, T, H, K, dtype=dt), torch.randn(B, T, H, K, dtype=dt)
        q, k = q / q.norm(dim=-1, keepdim=True), k / k.norm(dim=-1, keepdim=True)
        v, do = torch.randn(B, T, H, K, dtype=dt), torch.randn(B, T, H, K, dtype=dt)
        g = torch.nn.functional.logsigmoid(torch.randn(B, T, H, K, dtype=dt)) / 4
        beta = torch.sigmoid(torch.randn(B, T, H, dtype=dt))
        h0, dht = 0.1 * torch.randn(B, H, K, K, dtype=dt), 0.1 * torch.randn(B, H, K, K, dtype=dt)
        scale = K ** -0.5
        ops = _oracle_kda_ops()
        sl = slice(rank * T // world, (rank + 1) * T // world)
        o, final, ctx = TS.kda_forward(ops, q[:, sl], k[:, sl], v[:, sl], g[:, sl], beta[:, sl], scale, h0)
        got = TS.kda_backward(ops, q[:, sl], k[:, sl], v[:, sl], g[:, sl], beta[:, sl], scale, ctx, do[:, sl], dht)
        o_ref, ht_ref = OK.naive_recurrent_kda(q, k, v, g, beta, scale, h0, True)
        ref = OK.fused_recurrent_kda_bwd(q, k, v, g, beta, do, scale, h0, dht)
        errs = [(o - o_ref[:, sl]).abs().max().item(), (final - ht_ref).abs().max().item(),
                (got[5] - ref[5]).abs().max().item()]
        errs += [(a - b[:, sl]).abs().max().item() for a, b in zip(got[:5], ref[:5])]
        out[rank] = max(errs)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_time_sharded_kda_equals_single_pass(world):
    """KDA's transition is dense: shards exchange (M, S) with h_out = M h_in + S forward and D with
    dh_in = M^T dh_out + D backward; M comes from a forward with v = 0 and initial_state = I."""
    mgr = mp.get_context("spawn").Manager()
    out = mgr.dict()
    port = 29800 + os.getpid() % 150 + world
    mp.spawn(_kda_worker, args=(world, port, out), nprocs=world, join=True)
    assert len(out) == world
    for r in range(world):
        assert out[r] < 1e-9, (r, out[r])
