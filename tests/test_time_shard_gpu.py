"""Time sharding on real GPUs (needs >= 2): simple_gla (BASELINE config 4 at a
reduced length) split over ranks with NCCL all-gathers of the shard summaries,
against one pass of the CPU oracle over the whole sequence."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out):
    for p in (ROOT, os.path.join(ROOT, "pallas-kernel_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from oracle import simple_gla as OS
        from tests.util import rel_l2
        from tops_b200 import time_shard as TS
        from tops_b200.synth import make_inputs
        B, T, H, K, V, C = 1, 1024 * world, 4, 128, 128, 64
        # bf16 gate: every local op (summaries through the state-exchange entry points, forward,
        # backward) runs on the tcgen05 kernels
        x = make_inputs(61, B, T, H, K, V, dtype=torch.bfloat16, gate="scalar", with_h0=True, with_grads=True)
        scale = K ** -0.5
        sl = slice(rank * T // world, (rank + 1) * T // world)
        c = {n: (t[:, sl] if t.ndim >= 3 and t.shape[1] == T else t).cuda().contiguous() for n, t in x.items()}
        ops = TS.cuda_ops("simple_gla", C)
        o, final, h_in = TS.forward(ops, c["q"], c["k"], c["v"], c["g"], scale, c["h0"])
        dq, dk, dv, dg, dh0 = TS.backward(ops, c["q"], c["k"], c["v"], c["g"], scale, h_in, c["do"], c["dht"])
        torch.cuda.synchronize()
        from tops_b200 import _lib as L
        assert L.device_error() == 0
        o_ref, ht_ref = OS.chunk_simple_gla(x["q"], x["k"], x["v"], x["g"], None, scale, x["h0"], True, chunk_size=C)
        r = OS.chunk_simple_gla_bwd(x["q"], x["k"], x["v"], x["g"], None, x["h0"], x["do"], x["dht"], scale, chunk_size=C)
        errs = {"o": rel_l2(o, o_ref[:, sl]), "ht": rel_l2(final, ht_ref), "dh0": rel_l2(dh0, r[4])}
        for n, a, b in zip(("dq", "dk", "dv", "dg"), (dq, dk, dv, dg), r[:4]):
            errs[n] = rel_l2(a, b[:, sl])
        out[rank] = errs
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2])
def test_time_sharded_simple_gla_on_gpus(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    mgr = mp.get_context("spawn").Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, 29731, out), nprocs=world, join=True)
    assert len(out) == world
    for r in range(world):
        for name, e in out[r].items():
            assert e <= 2e-2, (r, name, e)      # bf16 bar: relative L2


def _kda_worker(rank, world, port, out):
    for p in (ROOT, os.path.join(ROOT, "pallas-kernel_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from oracle import kda as OK
        from tests.util import rel_l2
        from tops_b200 import _lib as L
        from tops_b200 import time_shard as TS
        from tops_b200.synth import make_inputs
        B, T, H, K, V = 1, 256 * world, 2, 128, 128
        x = make_inputs(71, B, T, H, K, V, dtype=torch.bfloat16, with_h0=True, with_grads=True, with_beta=True,
                        l2norm_qk=True)
        scale = K ** -0.5
        sl = slice(rank * T // world, (rank + 1) * T // world)
        c = {n: (t[:, sl] if t.ndim >= 3 and t.shape[1] == T else t).cuda().contiguous() for n, t in x.items()}
        ops = TS.kda_cuda_ops()
        o, final, ctx = TS.kda_forward(ops, c["q"], c["k"], c["v"], c["g"], c["beta"], scale, c["h0"])
        dq, dk, dv, dg, dbeta, dh0 = TS.kda_backward(ops, c["q"], c["k"], c["v"], c["g"], c["beta"], scale, ctx,
                                                     c["do"], c["dht"])
        torch.cuda.synchronize()
        assert L.device_error() == 0
        o_ref, ht_ref = OK.naive_recurrent_kda(x["q"], x["k"], x["v"], x["g"], x["beta"], scale, x["h0"], True)
        r = OK.fused_recurrent_kda_bwd(x["q"], x["k"], x["v"], x["g"], x["beta"], x["do"], scale, x["h0"], x["dht"])
        errs = {"o": rel_l2(o, o_ref[:, sl]), "ht": rel_l2(final, ht_ref), "dh0": rel_l2(dh0, r[5])}
        for n, a, b in zip(("dq", "dk", "dv", "dg", "dbeta"), (dq, dk, dv, dg, dbeta), r[:5]):
            errs[n] = rel_l2(a, b[:, sl])
        out[rank] = errs
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2])
def test_time_sharded_kda_on_gpus(world):
    """One KDA sequence split over ranks: the shards exchange their dense transitions and summaries
    (NCCL all-gathers) and must reproduce one pass of the CPU oracle over the whole sequence."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    mgr = mp.get_context("spawn").Manager()
    out = mgr.dict()
    mp.spawn(_kda_worker, args=(world, 29741, out), nprocs=world, join=True)
    assert len(out) == world
    for r in range(world):
        for name, e in out[r].items():
            assert e <= 2e-2, (r, name, e)      # bf16 bar: relative L2
