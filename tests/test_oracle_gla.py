"""Pins of the CPU oracle (no GPU): the relations the reference's own tests use
to pin `tops/cpu` — chunked == token recurrence in fp64 at 1e-10
(tests/ref/gla/test_chunk_gla.py:372-402), explicit backward == autodiff of the
naive recurrence at 1e-8 (tests/ref/simple_gla/test_chunk_simple_gla.py:304-360),
recurrent == naive == chunk (tests/ref/gla/test_fused_recurrent_gla.py:171-232),
the dtype contract (tests/ref/gla/test_chunk_gla.py:245-293) — plus the frozen
vectors in tests/golden/."""
import os

import pytest
import torch

from oracle import gla as G
from oracle import simple_gla as S
from oracle.common import chunk_local_cumsum

DT = torch.float64


def _rand(seed, B, T, H, K, V, scalar_gate=False):
    g = torch.Generator().manual_seed(seed)
    q, k = torch.randn(B, T, H, K, dtype=DT, generator=g), torch.randn(B, T, H, K, dtype=DT, generator=g)
    v = torch.randn(B, T, H, V, dtype=DT, generator=g)
    gs = (B, T, H) if scalar_gate else (B, T, H, K)
    gate = torch.nn.functional.logsigmoid(torch.randn(*gs, dtype=DT, generator=g))
    h0 = torch.randn(B, H, K, V, dtype=DT, generator=g)
    return q, k, v, gate, h0


@pytest.mark.parametrize("B,T,H,K,V,C", [(2, 64, 3, 16, 24, 16), (1, 100, 2, 32, 16, 32), (2, 37, 1, 8, 8, 16),
                                         (1, 1, 2, 16, 16, 16), (1, 3, 1, 8, 16, 64)])
@pytest.mark.parametrize("use_h0", [False, True])
def test_gla_chunk_equals_naive_fp64(B, T, H, K, V, C, use_h0):
    q, k, v, g, h0 = _rand(0, B, T, H, K, V)
    h0 = h0 if use_h0 else None
    o1, s1 = G.chunk_gla(q, k, v, g, None, h0, True, chunk_size=C)
    o2, s2 = G.naive_recurrent_gla(q, k, v, g, h0, True)
    o3, s3 = G.fused_recurrent_gla(q, k, v, g, None, None, h0, True)
    assert (o1 - o2).abs().max() < 1e-10 and (s1 - s2).abs().max() < 1e-10
    assert (o3 - o2).abs().max() < 1e-10 and (s3 - s2).abs().max() < 1e-10


def test_gla_chunk_fp32_close_to_naive():
    q, k, v, g, h0 = (x.float() for x in _rand(1, 2, 128, 2, 32, 32))
    o1, s1 = G.chunk_gla(q, k, v, g, None, h0, True, chunk_size=64)
    o2, s2 = G.naive_recurrent_gla(q, k, v, g, h0, True)
    assert (o1 - o2).abs().max() < 5e-3 and (s1 - s2).abs().max() < 5e-3


def test_gla_explicit_backward_equals_autodiff_fp64():
    B, T, H, K, V = 2, 70, 2, 16, 24
    q, k, v, g, h0 = _rand(2, B, T, H, K, V)
    leaves = [x.clone().requires_grad_() for x in (q, k, v, g, h0)]
    o, ht = G.naive_recurrent_gla(*leaves[:4], leaves[4], True)
    gen = torch.Generator().manual_seed(3)
    do, dht = torch.randn(o.shape, dtype=DT, generator=gen), torch.randn(ht.shape, dtype=DT, generator=gen)
    ((o * do).sum() + (ht * dht).sum()).backward()
    got = G.chunk_gla_bwd(q, k, v, g, None, K ** -0.5, h0, None, None, do, dht, chunk_size=32)
    for a, b in zip(got, leaves):
        assert (a - b.grad).abs().max() < 1e-8
    rec = G.fused_recurrent_bwd(q, k, v, g, None, None, do, dht, None, h0)
    for a, b in zip((rec[0], rec[1], rec[2], rec[3], rec[5]), leaves):
        assert (a - b.grad).abs().max() < 1e-8


def test_gla_recurrent_gv_reverse_backward_equals_autodiff():
    B, T, H, K, V = 1, 20, 2, 8, 12
    q, k, v, gk, h0 = _rand(4, B, T, H, K, V)
    gv = torch.nn.functional.logsigmoid(torch.randn(B, T, H, V, dtype=DT, generator=torch.Generator().manual_seed(5)))
    leaves = [x.clone().requires_grad_() for x in (q, k, v, gk, gv, h0)]
    o, ht = G.fused_recurrent_fwd(*leaves[:5], None, leaves[5], True, True)
    do, dht = torch.randn_like(o), torch.randn_like(ht)
    ((o * do).sum() + (ht * dht).sum()).backward()
    got = G.fused_recurrent_bwd(q, k, v, gk, gv, o.detach(), do, dht, None, h0, True)
    for a, b in zip(got, leaves):
        assert (a - b.grad).abs().max() < 1e-8


def test_gla_dtype_contract():
    q, k, v, g, h0 = _rand(6, 1, 64, 2, 16, 16)
    qb, kb, vb, gb = (x.to(torch.bfloat16) for x in (q, k, v, g))
    gc, A, h, ht, o = G.chunk_gla_fwd(qb, kb, vb, gb, None, 0.25, h0.float(), True, chunk_size=16)
    assert gc.dtype == torch.float32 and A.dtype == torch.float32 and ht.dtype == torch.float32
    assert h.dtype == torch.bfloat16 and o.dtype == torch.bfloat16
    do = torch.randn(1, 64, 2, 16).to(torch.bfloat16)
    dq, dk, dv, dg, dh0 = G.chunk_gla_bwd(qb, kb, vb, gb, None, 0.25, h0.float(), None, None, do, None, chunk_size=16)
    assert dq.dtype == dk.dtype == dg.dtype == dh0.dtype == torch.float32 and dv.dtype == torch.bfloat16


def test_gla_varlen_equals_per_sequence():
    q, k, v, g, _ = _rand(7, 1, 100, 2, 16, 24)
    cu = [0, 37, 38, 100]
    h0 = torch.randn(3, 2, 16, 24, dtype=DT)
    o, ht = G.chunk_gla(q, k, v, g, None, h0, True, cu_seqlens=cu, chunk_size=16)
    for n in range(3):
        s = slice(cu[n], cu[n + 1])
        on, hn = G.naive_recurrent_gla(q[:, s], k[:, s], v[:, s], g[:, s], h0[n:n + 1], True)
        assert (o[:, s] - on).abs().max() < 1e-10 and (ht[n] - hn[0]).abs().max() < 1e-10


def test_state_split_equals_single_pass():
    q, k, v, g, h0 = _rand(8, 2, 128, 2, 16, 16)
    o, ht = G.chunk_gla(q, k, v, g, None, h0, True, chunk_size=32)
    o1, s1 = G.chunk_gla(q[:, :64], k[:, :64], v[:, :64], g[:, :64], None, h0, True, chunk_size=32)
    o2, s2 = G.chunk_gla(q[:, 64:], k[:, 64:], v[:, 64:], g[:, 64:], None, s1, True, chunk_size=32)
    assert (torch.cat([o1, o2], 1) - o).abs().max() < 1e-10 and (s2 - ht).abs().max() < 1e-10


@pytest.mark.parametrize("gate", ["g", "gamma", "none"])
@pytest.mark.parametrize("T,C", [(64, 16), (37, 16), (1, 16)])
def test_simple_gla_chunk_equals_naive_and_autodiff(gate, T, C):
    B, H, K, V = 2, 3, 16, 24
    q, k, v, g, h0 = _rand(9, B, T, H, K, V, scalar_gate=True)
    gam = -torch.rand(H, dtype=DT) * 0.3 if gate == "gamma" else None
    g = g if gate == "g" else None
    o1, s1 = S.chunk_simple_gla(q, k, v, g, gam, None, h0, True, chunk_size=C)
    o2, s2 = S.naive_recurrent_simple_gla(q, k, v, g, gam, None, h0, True)
    assert (o1 - o2).abs().max() < 1e-10 and (s1 - s2).abs().max() < 1e-10
    leaves = [x.clone().requires_grad_() for x in (q, k, v, h0)]
    gl = g.clone().requires_grad_() if g is not None else None
    o, ht = S.naive_recurrent_simple_gla(leaves[0], leaves[1], leaves[2], gl, gam, None, leaves[3], True)
    do, dht = torch.randn_like(o), torch.randn_like(ht)
    ((o * do).sum() + (ht * dht).sum()).backward()
    dq, dk, dv, dg, dh0 = S.chunk_simple_gla_bwd(q, k, v, g, gam, h0, do, dht, K ** -0.5, chunk_size=C)
    for a, b in zip((dq, dk, dv, dh0), leaves):
        assert (a - b.grad).abs().max() < 1e-8
    if g is not None:
        assert (dg - gl.grad).abs().max() < 1e-8


def test_cumsum_reverse_and_packed():
    g = torch.randn(1, 50, 2, 4, dtype=DT)
    cu = [0, 7, 30, 50]
    out = chunk_local_cumsum(g, 16, cu_seqlens=cu)
    rev = chunk_local_cumsum(g, 16, reverse=True, cu_seqlens=cu)
    for a, b in zip(cu[:-1], cu[1:]):
        for c0 in range(a, b, 16):
            c1 = min(c0 + 16, b)
            assert torch.allclose(out[0, c0:c1], g[0, c0:c1].cumsum(0))
            assert torch.allclose(rev[0, c0:c1], g[0, c0:c1].flip(0).cumsum(0).flip(0))


GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


@pytest.mark.parametrize("name", sorted(f for f in os.listdir(GOLDEN) if f.endswith(".pt") and not f.startswith("ref_"))
                         if os.path.isdir(GOLDEN) else [])
def test_golden_vectors_reproduce(name):
    """The fixtures produced by tests/golden/make_golden.py (outputs of the oracle itself; the `ref_*` files,
    outputs of the reference's code, have tests/test_reference_golden.py): the oracle must keep reproducing them."""
    from tests.golden.make_golden import CASES, run_case
    blob = torch.load(os.path.join(GOLDEN, name))
    out = run_case(CASES[blob["case"]])
    for key, ref in blob["outputs"].items():
        assert torch.allclose(out[key].float(), ref.float(), rtol=1e-5, atol=1e-6), key


@pytest.mark.parametrize("C,g_scale", [(64, 0.8), (128, 0.8), (128, 1.0)])
def test_large_gates_stay_finite_and_exact(C, g_scale):
    """Per-step gates uniform in (-g_scale, 0): their chunk-local sums reach -C g_scale, where exp() of the raw
    cumulative gate over- or underflows fp32; the mid-point anchored factorisation must stay finite and equal to the
    token recurrence (the reference's tests/ops/gla/test_exp_overflow_stabilization.py:62-221, same gate law)."""
    g = torch.Generator().manual_seed(42)
    B, T, H, Kd = 1, 2 * C, 2, 32
    q, k, v, do = (torch.randn(B, T, H, Kd, generator=g) for _ in range(4))
    gate = -g_scale * torch.rand(B, T, H, Kd, generator=g)
    scale = Kd ** -0.5
    o, ht = G.chunk_gla(q, k, v, gate, scale, None, True, chunk_size=C)
    grads = G.chunk_gla_bwd(q, k, v, gate, None, scale, None, None, None, do, None, chunk_size=C)
    for t in (o, ht, *grads[:4]):
        assert torch.isfinite(t).all()
    o_ref, ht_ref = G.naive_recurrent_gla(q.double(), k.double(), v.double(), gate.double(), output_final_state=True)
    assert (o.double() - o_ref).abs().max() < 1e-3
    assert (ht.double() - ht_ref).abs().max() < 1e-3
