"""The headline configuration at full size (bf16, B=8, T=4096, H=16, K=V=128,
chunk 64: 128 (batch, head) pairs, the fused forward + reverse scan + chunk
backward) checked through properties that do not need a full-size oracle:

* scaling v (and h0) or do (and dht) by 2 scales the results by exactly 2 — every
  product is linear in them and a power of two is exact in bf16 and fp32;
* one (batch) slice computed alone — which takes the time-segmented path (16 pairs
  x 4 segments) — agrees with the same slice of the full batch;
* two halves of the sequence chained through the state agree with one pass
  (tests/ops/gla/test_pallas_chunk_gla.py:223-247 at full length);
* one (batch, head) pair agrees with the CPU oracle over all 4096 tokens.
"""
import pytest
import torch

from oracle import gla as O
from tests.util import assert_close, rel_l2, to_cuda

pytestmark = pytest.mark.gpu

B, T, H, K, V, C = 8, 4096, 16, 128, 128, 64
SCALE = K ** -0.5


@pytest.fixture(scope="module")
def data():
    from tops_b200.synth import make_inputs
    host = make_inputs(77, B, T, H, K, V, dtype=torch.bfloat16, with_h0=True, with_grads=True)
    return host, to_cuda(host)


def _fwd(x, **over):
    from tops_b200 import _lib as L
    from tops_b200.ops._chunk import chunk_fwd_call
    a = {**x, **over}
    o, ht, _, _, hs = chunk_fwd_call(a["q"], a["k"], a["v"], a["g"], L.GATE_PER_CHANNEL, SCALE, a["h0"], True, C,
                                     want_saved=True)
    return o, ht, hs


def _bwd(x, hs, **over):
    from tops_b200 import _lib as L
    from tops_b200.ops._chunk import chunk_bwd_call
    a = {**x, **over}
    return chunk_bwd_call(a["q"], a["k"], a["v"], a["g"], L.GATE_PER_CHANNEL, SCALE, a["h0"], a["do"], a["dht"], C,
                          torch.float32, True, True, h_saved=hs, primal_dtypes=True)


def test_exact_linearity_in_v_and_do(data):
    from tops_b200 import _lib as L
    _, x = data
    o, ht, hs = _fwd(x)
    o2, ht2, _ = _fwd(x, v=x["v"] * 2, h0=x["h0"] * 2)
    assert torch.equal(o2.float(), o.float() * 2) and torch.equal(ht2, ht * 2)
    g1 = _bwd(x, hs)
    g2 = _bwd(x, hs, do=x["do"] * 2, dht=x["dht"] * 2)
    for name, a, b in zip(("dq", "dk", "dv", "dg", "dh0"), g1, g2):
        assert torch.equal(b.float(), a.float() * 2), name
    torch.cuda.synchronize()
    assert L.device_error() == 0


def test_one_batch_alone_equals_its_slice_of_the_full_batch(data):
    _, x = data
    o, ht, hs = _fwd(x)
    full = _bwd(x, hs)
    b = 5
    one = {k: v[b:b + 1].contiguous() for k, v in x.items()}
    o1, ht1, hs1 = _fwd(one)
    part = _bwd(one, hs1)
    # (the two paths round the gated keys of the state product to bf16 at different points)
    assert rel_l2(o1, o[b:b + 1]) <= 4e-3 and rel_l2(ht1, ht[b:b + 1]) <= 5e-3
    for name, a, f in zip(("dq", "dk", "dv", "dg", "dh0"), part, full):
        assert rel_l2(a, f[b:b + 1]) <= 6e-3, (name, rel_l2(a, f[b:b + 1]))


def test_two_halves_chained_through_the_state_equal_one_pass(data):
    _, x = data
    o, ht, _ = _fwd(x)
    h = T // 2
    first = {k: (v[:, :h].contiguous() if v.ndim == 4 and v.shape[1] == T else v) for k, v in x.items()}
    o1, s1, _ = _fwd(first)
    second = {k: (v[:, h:].contiguous() if v.ndim == 4 and v.shape[1] == T else v) for k, v in x.items()}
    o2, s2, _ = _fwd(second, h0=s1)
    assert rel_l2(torch.cat([o1, o2], 1), o) <= 4e-3
    assert rel_l2(s2, ht) <= 5e-3


def test_one_pair_against_the_oracle_over_the_whole_sequence(data):
    host, x = data
    o, ht, hs = _fwd(x)
    dq, dk, dv, dg, dh0 = _bwd(x, hs)
    b, h = 6, 11
    one = {k: v[b:b + 1, :, h:h + 1].contiguous() for k, v in host.items() if v.ndim == 4 and v.shape[1] == T}
    h0 = host["h0"][b:b + 1, h:h + 1].contiguous()
    dht = host["dht"][b:b + 1, h:h + 1].contiguous()
    o_ref, ht_ref = O.chunk_gla(one["q"], one["k"], one["v"], one["g"], SCALE, h0, True, chunk_size=C)
    ref = O.chunk_gla_bwd(one["q"], one["k"], one["v"], one["g"], None, SCALE, h0, None, None, one["do"], dht,
                          chunk_size=C)
    assert_close("o", o[b:b + 1, :, h:h + 1].cpu(), o_ref, torch.bfloat16)
    assert_close("ht", ht[b:b + 1, h:h + 1].cpu(), ht_ref, torch.bfloat16)
    got = (dq, dk, dv, dg)
    for name, a, r in zip(("dq", "dk", "dv", "dg"), got, ref[:4]):
        assert_close(name, a[b:b + 1, :, h:h + 1].float().cpu(), r.float(), torch.bfloat16)
    assert_close("dh0", dh0[b:b + 1, h:h + 1].cpu(), ref[4], torch.bfloat16)
