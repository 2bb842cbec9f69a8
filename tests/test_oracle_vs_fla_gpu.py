"""The oracle against flash-linear-attention (FLA), the third-party Triton
implementation the reference's own tests cross-check `tops.cpu` against
(`tests/ref/gla/test_chunk_gla.py:24-30,136-193`,
`tests/ref/simple_gla/test_chunk_simple_gla.py`, `tests/ref/kda/special/test_chunk_bwd.py:250-271`).

The reference stores no arrays, so nothing it produced can be compared with
directly; what its test-suite pins `tops.cpu` to is agreement with FLA on seeded
random inputs.  This file re-enacts that pin with `oracle/` in the place of
`tops.cpu`: the oracle runs on the CPU in fp32, FLA on the GPU through its
public differentiable ops, on the reference's test shapes.  FLA is used as a
black box and only here; no product code imports it.

Only the GLA family (chunk_gla forward + backward, fused_recurrent_gla) is
compared: on a B200 FLA 0.5.1's simple_gla backward raised a CUDA "misaligned
address" error inside its own Triton kernels, so that family (and KDA after it)
is not run.  FLA autotunes every kernel per shape (about ten minutes for this
file), so the module only runs when TOPS_B200_FLA_CHECK=1 is set; it is skipped
otherwise, and when FLA or a working Triton back end is not there.

Bars: fp32 inputs relative L2 <= 2e-3 (Triton's fp32 dot products may run in
TF32); bf16 inputs relative L2 <= 2e-2.  A convention error (gate sign, inclusive
vs exclusive cumsum, which state an output sees, the scale of dg) shows up at
order one, far above either bar.
"""
import pytest
import torch

from tests.util import rel_l2

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def fla_ops():
    import os
    if os.environ.get("TOPS_B200_FLA_CHECK", "0") in ("", "0"):
        pytest.skip("set TOPS_B200_FLA_CHECK=1 to run the cross-check against flash-linear-attention")
    try:
        from fla.ops.gla import chunk_gla, fused_recurrent_gla
    except Exception as exc:     # ImportError, or a Triton back end that does not load
        pytest.skip(f"flash-linear-attention is not importable: {exc!r}")
    try:                         # one tiny call: does its Triton code compile for this GPU?
        x = torch.randn(1, 64, 1, 32, device="cuda")
        g = torch.nn.functional.logsigmoid(torch.randn(1, 64, 1, 32, device="cuda"))
        chunk_gla(x, x, x, g)
        torch.cuda.synchronize()
    except Exception as exc:
        pytest.skip(f"flash-linear-attention does not run on this box: {exc!r}")
    return dict(chunk_gla=chunk_gla, fused_recurrent_gla=fused_recurrent_gla)


def _bar(dtype):
    return 2e-3 if dtype == torch.float32 else 2e-2


def _inputs(seed, B, T, H, K, V, dtype):
    from tops_b200.synth import make_inputs
    # un-normalised log-sigmoid gates like the reference's tests (tests/ref/gla/test_chunk_gla.py:312-317)
    return make_inputs(seed, B, T, H, K, V, dtype=dtype, gate_norm=1.0, with_h0=True, with_grads=True)


def _fla_grads(fn, host, names, **kw):
    x = {n: host[n].cuda().requires_grad_(True) for n in names}
    h0 = host["h0"].cuda().requires_grad_(True)
    o, ht = fn(**x, initial_state=h0, output_final_state=True, **kw)
    grads = torch.autograd.grad((o, ht), [*x.values(), h0], (host["do"].cuda().to(o.dtype), host["dht"].cuda()))
    return o.detach().cpu(), ht.detach().cpu(), [t.cpu() for t in grads]


GLA_SHAPES = [(2, 64, 4, 32, 64), (1, 128, 2, 64, 128), (2, 64, 4, 16, 128), (2, 64, 4, 128, 16), (1, 256, 2, 32, 64)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,T,H,K,V", GLA_SHAPES)
def test_gla_oracle_matches_fla(fla_ops, B, T, H, K, V, dtype):
    from oracle import gla as O
    host = _inputs(11, B, T, H, K, V, dtype)
    scale = K ** -0.5
    o, ht, grads = _fla_grads(fla_ops["chunk_gla"], host, ("q", "k", "v", "g"), scale=scale)
    o_ref, ht_ref = O.chunk_gla(host["q"], host["k"], host["v"], host["g"], scale, host["h0"], True, chunk_size=64)
    ref = O.chunk_gla_bwd(host["q"], host["k"], host["v"], host["g"], None, scale, host["h0"], None, None, host["do"],
                          host["dht"], chunk_size=64)
    bar = _bar(dtype)
    assert rel_l2(o_ref, o) <= bar and rel_l2(ht_ref, ht) <= bar
    for name, a, r in zip(("dq", "dk", "dv", "dg", "dh0"), grads, ref):
        assert rel_l2(r, a) <= bar, (name, rel_l2(r, a))
    # the token recurrence too
    orr, htr = fla_ops["fused_recurrent_gla"](host["q"].cuda(), host["k"].cuda(), host["v"].cuda(), gk=host["g"].cuda(),
                                              scale=scale, initial_state=host["h0"].cuda(), output_final_state=True)
    o_rec, ht_rec = O.fused_recurrent_gla(host["q"], host["k"], host["v"], gk=host["g"], scale=scale,
                                          initial_state=host["h0"], output_final_state=True)
    assert rel_l2(o_rec, orr.cpu()) <= bar and rel_l2(ht_rec, htr.cpu()) <= bar
