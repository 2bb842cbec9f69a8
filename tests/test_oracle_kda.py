"""Pins of the KDA oracle (no GPU): chunked WY form == token recurrence in fp64
at 1e-10 and explicit backward == autodiff at 1e-7, the relations of the
reference's tests/ref/kda/test_naive_kda.py:198-293."""
import pytest
import torch

from oracle import kda as K

DT = torch.float64


def _rand(seed, B, T, H, Kd, V):
    g = torch.Generator().manual_seed(seed)
    q = torch.nn.functional.normalize(torch.randn(B, T, H, Kd, dtype=DT, generator=g), dim=-1)
    k = torch.nn.functional.normalize(torch.randn(B, T, H, Kd, dtype=DT, generator=g), dim=-1)
    v = torch.randn(B, T, H, V, dtype=DT, generator=g)
    gate = torch.nn.functional.logsigmoid(torch.randn(B, T, H, Kd, dtype=DT, generator=g))
    beta = torch.sigmoid(torch.randn(B, T, H, dtype=DT, generator=g))
    h0 = torch.randn(B, H, Kd, V, dtype=DT, generator=g)
    return q, k, v, gate, beta, h0


@pytest.mark.parametrize("B,T,H,Kd,V,C", [(2, 64, 2, 16, 24, 16), (1, 70, 2, 32, 16, 32), (1, 1, 1, 8, 8, 16)])
@pytest.mark.parametrize("use_h0", [False, True])
def test_chunk_equals_recurrent(B, T, H, Kd, V, C, use_h0):
    q, k, v, g, beta, h0 = _rand(0, B, T, H, Kd, V)
    h0 = h0 if use_h0 else None
    o1, s1 = K.naive_recurrent_kda(q, k, v, g, beta, None, h0, True)
    o2, s2 = K.naive_chunk_kda(q, k, v, g, beta, None, h0, True, chunk_size=C)
    assert (o1 - o2).abs().max() < 1e-10 and (s1 - s2).abs().max() < 1e-10


def test_explicit_backward_equals_autodiff():
    q, k, v, g, beta, h0 = _rand(1, 2, 40, 2, 16, 24)
    leaves = [x.clone().requires_grad_() for x in (q, k, v, g, beta, h0)]
    o, s = K.naive_recurrent_kda(*leaves[:5], None, leaves[5], True)
    do, dht = torch.randn_like(o), torch.randn_like(s)
    ((o * do).sum() + (s * dht).sum()).backward()
    got = K.fused_recurrent_kda_bwd(q, k, v, g, beta, do, None, h0, dht)
    for a, b in zip(got, leaves):
        assert (a - b.grad).abs().max() < 1e-7
    # gradients of the chunked form agree too
    leaves2 = [x.clone().requires_grad_() for x in (q, k, v, g, beta, h0)]
    o2, s2 = K.naive_chunk_kda(*leaves2[:5], None, leaves2[5], True, chunk_size=16)
    ((o2 * do).sum() + (s2 * dht).sum()).backward()
    for a, b in zip(leaves2, leaves):
        assert (a.grad - b.grad).abs().max() < 1e-7
