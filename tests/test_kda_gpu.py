"""GPU parity of the KDA kernels (forward and backward, through the C ABI)
against the CPU oracle.  Inputs follow BASELINE config 5: q, k L2-normalised,
beta = sigmoid(N(0,1)), g = log_sigmoid(N(0,1))/16, h0 ~ 0.1 N(0,1)."""
import pytest
import torch

from oracle import kda as O
from tests.util import assert_close, to_cuda

pytestmark = pytest.mark.gpu

SHAPES = [
    # B, T, H, K, V, dtype, h0
    (2, 64, 2, 32, 32, torch.float32, True),
    (1, 37, 3, 16, 24, torch.float32, True),
    (2, 1, 2, 16, 16, torch.float32, False),
    (1, 130, 2, 64, 128, torch.float32, False),
    (1, 100, 2, 100, 72, torch.float32, True),
    (2, 192, 2, 128, 128, torch.bfloat16, True),
    (1, 128, 4, 64, 64, torch.bfloat16, False),
]


def _inputs(seed, B, T, H, K, V, dtype, h0):
    from tops_b200.synth import make_inputs
    return make_inputs(seed, B, T, H, K, V, dtype=dtype, with_h0=h0, with_grads=True, with_beta=True, l2norm_qk=True)


@pytest.mark.parametrize("B,T,H,K,V,dtype,h0", SHAPES)
def test_kda_forward_backward(B, T, H, K, V, dtype, h0):
    from tops_b200.ops.kda import chunk_kda, fused_recurrent_kda, kda_bwd
    x = _inputs(51, B, T, H, K, V, dtype, h0)
    o_ref, ht_ref = O.naive_recurrent_kda(x["q"], x["k"], x["v"], x["g"], x["beta"], None, x.get("h0"), True)
    ref = O.fused_recurrent_kda_bwd(x["q"], x["k"], x["v"], x["g"], x["beta"], x["do"], None, x.get("h0"), x["dht"])
    c = to_cuda(x)
    o, ht = fused_recurrent_kda(c["q"], c["k"], c["v"], c["g"], c["beta"], None, c.get("h0"), True)
    assert o.dtype == dtype and ht.dtype == torch.float32
    assert_close("o", o, o_ref, dtype)
    assert_close("ht", ht, ht_ref, dtype)
    if T % 16 == 0:
        o2, _ = chunk_kda(c["q"], c["k"], c["v"], c["g"], c["beta"], None, c.get("h0"), False, chunk_size=16)
        assert_close("o(chunk)", o2, o_ref, dtype)
    got = kda_bwd(c["q"], c["k"], c["v"], c["g"], c["beta"], c["do"], K ** -0.5, c.get("h0"), c["dht"])
    for name, a, b in zip(("dq", "dk", "dv", "dg", "dbeta", "dh0"), got, ref):
        if b is None:
            assert a is None, name
            continue
        assert a.dtype == b.dtype, name
        assert_close(name, a, b, dtype)


def test_kda_autograd():
    from tops_b200.ops.kda import chunk_kda
    B, T, H, K, V = 1, 64, 2, 32, 32
    x = _inputs(52, B, T, H, K, V, torch.float32, True)
    c = to_cuda(x)
    leaves = {n: c[n].clone().requires_grad_() for n in ("q", "k", "v", "g", "beta", "h0")}
    o, ht = chunk_kda(leaves["q"], leaves["k"], leaves["v"], leaves["g"], leaves["beta"], initial_state=leaves["h0"],
                      output_final_state=True, chunk_size=64)
    ((o * c["do"]).sum() + (ht * c["dht"]).sum()).backward()
    ref = O.fused_recurrent_kda_bwd(x["q"], x["k"], x["v"], x["g"], x["beta"], x["do"], None, x["h0"], x["dht"])
    for n, r in zip(("q", "k", "v", "g", "beta", "h0"), ref):
        assert_close("d" + n, leaves[n].grad, r, torch.float32)


def test_kda_state_split():
    from tops_b200.ops.kda import fused_recurrent_kda
    B, T, H, K, V = 2, 128, 2, 64, 64
    c = to_cuda(_inputs(53, B, T, H, K, V, torch.float32, True))
    o, ht = fused_recurrent_kda(c["q"], c["k"], c["v"], c["g"], c["beta"], None, c["h0"], True)
    h = T // 2
    a = [c[n][:, :h] for n in ("q", "k", "v", "g", "beta")]
    bb = [c[n][:, h:] for n in ("q", "k", "v", "g", "beta")]
    o1, s1 = fused_recurrent_kda(*a, None, c["h0"], True)
    o2, s2 = fused_recurrent_kda(*bb, None, s1, True)
    assert_close("o", torch.cat([o1, o2], 1), o, torch.float32)
    assert_close("ht", s2, ht, torch.float32)


def test_kda_decode_in_place():
    """One token per call on a state updated in place == one pass of the oracle over the tokens."""
    from oracle import kda as OK
    from tops_b200.ops.kda import fused_recurrent_kda_decode_
    from tops_b200.synth import make_inputs
    B, T, H, K, V = 3, 24, 2, 128, 128
    host = make_inputs(91, B, T, H, K, V, dtype=torch.bfloat16, with_h0=True, with_beta=True, l2norm_qk=True)
    x = {n: t.cuda() for n, t in host.items()}
    state = x["h0"].clone()
    ptr = state.data_ptr()
    outs = [fused_recurrent_kda_decode_(*(x[n][:, t:t + 1].contiguous() for n in ("q", "k", "v", "g", "beta")), state)
            for t in range(T)]
    assert state.data_ptr() == ptr
    o_ref, ht_ref = OK.naive_recurrent_kda(host["q"], host["k"], host["v"], host["g"], host["beta"], None, host["h0"], True)
    got = torch.cat(outs, 1)
    assert ((got.float().cpu() - o_ref.float()).norm() / o_ref.float().norm()).item() <= 2e-2
    assert ((state.cpu() - ht_ref).norm() / ht_ref.norm()).item() <= 2e-2
