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
