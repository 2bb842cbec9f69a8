"""`scale` other than K^-0.5 through every kernel family (the reference's `scale=0.1` / `0.01` cases,
tests/ops/gla/test_pallas_chunk_gla.py:52,60-61,75-76): forward and autograd backward of the public ops
against the oracle called with the same scale."""
import pytest
import torch

from oracle import gla as OG
from oracle import kda as OK
from oracle import simple_gla as OS
from tests.util import assert_close, to_cuda

pytestmark = pytest.mark.gpu

CASES = [
    # B, T, H, K, V, dtype, scale
    (2, 32, 4, 32, 64, torch.float32, 0.1),        # generic kernels
    (1, 100, 2, 32, 64, torch.float32, 0.01),
    (1, 256, 2, 128, 128, torch.bfloat16, 0.1),    # tensor-core kernels: state scan + chunk outputs
    (4, 128, 12, 128, 128, torch.bfloat16, 0.25),  # tensor-core kernels: fused forward
]


def _leaves(c, names):
    return [c[n].clone().requires_grad_(True) for n in names]


@pytest.mark.parametrize("B,T,H,K,V,dtype,scale", CASES)
def test_chunk_gla_custom_scale(B, T, H, K, V, dtype, scale):
    from tops_b200.ops.gla import chunk_gla
    from tops_b200.synth import make_inputs
    x = make_inputs(200, B, T, H, K, V, dtype=dtype, with_h0=True, with_grads=True)
    o_ref, ht_ref = OG.chunk_gla(x["q"], x["k"], x["v"], x["g"], scale, x["h0"], True, chunk_size=64)
    ref = OG.chunk_gla_bwd(x["q"], x["k"], x["v"], x["g"], None, scale, x["h0"], None, None, x["do"], x["dht"],
                           chunk_size=64)
    c = to_cuda(x)
    leaves = _leaves(c, ("q", "k", "v", "g", "h0"))
    o, ht = chunk_gla(*leaves[:4], scale=scale, initial_state=leaves[4], output_final_state=True, chunk_size=64)
    got = torch.autograd.grad((o, ht), leaves, (c["do"], c["dht"]))
    assert_close("o", o.detach(), o_ref, dtype)
    assert_close("ht", ht.detach(), ht_ref, dtype)
    for name, a, b in zip(("dq", "dk", "dv", "dg", "dh0"), got, ref):
        assert_close(name, a, b, dtype)


@pytest.mark.parametrize("B,T,H,K,V,dtype,scale", CASES)
def test_chunk_simple_gla_custom_scale(B, T, H, K, V, dtype, scale):
    from tops_b200.ops.simple_gla import chunk_simple_gla
    from tops_b200.synth import make_inputs
    x = make_inputs(201, B, T, H, K, V, dtype=dtype, gate="scalar", with_h0=True, with_grads=True)
    o_ref, ht_ref = OS.chunk_simple_gla(x["q"], x["k"], x["v"], x["g"], None, scale, x["h0"], True, chunk_size=64)
    ref = OS.chunk_simple_gla_bwd(x["q"], x["k"], x["v"], x["g"], None, x["h0"], x["do"], x["dht"], scale,
                                  chunk_size=64)
    c = to_cuda(x)
    leaves = _leaves(c, ("q", "k", "v", "g", "h0"))
    o, ht = chunk_simple_gla(*leaves[:3], g=leaves[3], scale=scale, initial_state=leaves[4], output_final_state=True,
                             chunk_size=64)
    got = torch.autograd.grad((o, ht), leaves, (c["do"], c["dht"]))
    assert_close("o", o.detach(), o_ref, dtype)
    assert_close("ht", ht.detach(), ht_ref, dtype)
    for name, a, b in zip(("dq", "dk", "dv", "dg", "dh0"), got, ref):
        assert_close(name, a, b, dtype)


@pytest.mark.parametrize("T,K,V,dtype,scale", [(128, 128, 128, torch.bfloat16, 0.1),    # chunked WY kernels
                                               (64, 32, 64, torch.float32, 0.1)])       # token-serial kernels
def test_chunk_kda_custom_scale(T, K, V, dtype, scale):
    from tops_b200.ops.kda import chunk_kda
    from tops_b200.synth import make_inputs
    B, H = 2, 2
    x = make_inputs(202, B, T, H, K, V, dtype=dtype, with_h0=True, with_grads=True, with_beta=True, l2norm_qk=True)
    f = {n: x[n].float() for n in ("q", "k", "v", "g", "beta", "do")}
    o_ref, ht_ref = OK.naive_recurrent_kda(f["q"], f["k"], f["v"], f["g"], f["beta"], scale, x["h0"], True)
    ref = OK.fused_recurrent_kda_bwd(f["q"], f["k"], f["v"], f["g"], f["beta"], f["do"], scale, x["h0"], x["dht"])
    c = to_cuda(x)
    leaves = _leaves(c, ("q", "k", "v", "g", "beta", "h0"))
    o, ht = chunk_kda(*leaves[:5], scale=scale, initial_state=leaves[5], output_final_state=True)
    got = torch.autograd.grad((o, ht), leaves, (c["do"], c["dht"]))
    assert_close("o", o.detach().float(), o_ref, dtype)
    assert_close("ht", ht.detach(), ht_ref, dtype)
    return_order = ("dq", "dk", "dv", "dg", "dbeta", "dh0")
    for name, a, b in zip(return_order, got, ref):
        assert_close(name, a.float(), b.float(), dtype)
