"""GPU parity: chunked simple_gla (scalar gate g, constant decay g_gamma, no
gate) against the CPU oracle.  Shapes follow
tests/ref/simple_gla/test_chunk_simple_gla.py:94-121 of the reference."""
import pytest
import torch

from oracle import simple_gla as O
from tests.util import assert_close, to_cuda

pytestmark = pytest.mark.gpu

SHAPES = [
    # B, T, H, K, V, chunk, dtype, gate, h0
    (2, 128, 2, 64, 64, 64, torch.float32, "g", True),
    (1, 37, 3, 16, 24, 16, torch.float32, "g", True),
    (2, 1, 2, 32, 32, 16, torch.float32, "g", False),
    (2, 100, 2, 32, 64, 32, torch.float32, "gamma", True),
    (1, 64, 2, 64, 64, 64, torch.float32, "none", True),
    (1, 130, 2, 128, 128, 64, torch.float32, "gamma", False),
    (2, 256, 4, 128, 128, 64, torch.bfloat16, "g", True),
    (1, 256, 2, 128, 128, 64, torch.bfloat16, "gamma", True),
    (1, 192, 2, 64, 64, 64, torch.bfloat16, "none", False),
]


def _make(seed, B, T, H, K, V, dtype, gate, h0):
    from tops_b200.synth import make_inputs
    x = make_inputs(seed, B, T, H, K, V, dtype=dtype, gate="scalar", with_h0=h0, with_grads=True,
                    gate_dtype=torch.float32)
    g = x["g"] if gate == "g" else None
    gamma = -(0.02 + 0.1 * torch.rand(H, generator=torch.Generator().manual_seed(seed))) if gate == "gamma" else None
    return x, g, gamma


@pytest.mark.parametrize("B,T,H,K,V,C,dtype,gate,h0", SHAPES)
def test_chunk_simple_gla_forward_backward(B, T, H, K, V, C, dtype, gate, h0):
    from tops_b200.ops.simple_gla import chunk_simple_gla, chunk_simple_gla_bwd
    x, g, gamma = _make(21, B, T, H, K, V, dtype, gate, h0)
    scale = K ** -0.5
    o_ref, ht_ref = O.chunk_simple_gla(x["q"], x["k"], x["v"], g, gamma, None, x.get("h0"), True, chunk_size=C)
    ref = O.chunk_simple_gla_bwd(x["q"], x["k"], x["v"], g, gamma, x.get("h0"), x["do"], x["dht"], scale, chunk_size=C)
    c = to_cuda(x)
    gc = None if g is None else g.cuda()
    gamc = None if gamma is None else gamma.cuda()
    o, ht = chunk_simple_gla(c["q"], c["k"], c["v"], gc, gamc, None, c.get("h0"), True, chunk_size=C)
    assert o.dtype == dtype and ht.dtype == torch.float32
    assert_close("o", o, o_ref, dtype)
    assert_close("ht", ht, ht_ref, dtype)
    got = chunk_simple_gla_bwd(c["q"], c["k"], c["v"], gc, gamc, c.get("h0"), c["do"], c["dht"], scale, chunk_size=C)
    assert got[0].dtype == dtype and got[1].dtype == dtype and got[2].dtype == dtype
    for name, a, b in zip(("dq", "dk", "dv", "dg", "dh0"), got, ref):
        if b is None:
            assert a is None, name
            continue
        assert_close(name, a, b, dtype)


def test_simple_gla_modes_and_autograd():
    from tops_b200.ops.simple_gla import simple_gla
    B, T, H, K, V, C = 1, 96, 2, 32, 32, 32
    x, g, _ = _make(22, B, T, H, K, V, torch.float32, "g", True)
    c = to_cuda(x)
    leaves = {n: c[n].clone().requires_grad_() for n in ("q", "k", "v", "h0")}
    gl = g.cuda().requires_grad_()
    o, ht = simple_gla(leaves["q"], leaves["k"], leaves["v"], g=gl, initial_state=leaves["h0"],
                       output_final_state=True, chunk_size=C, mode="chunk")
    ((o * c["do"]).sum() + (ht * c["dht"]).sum()).backward()
    ref = O.chunk_simple_gla_bwd(x["q"], x["k"], x["v"], g, None, x["h0"], x["do"], x["dht"], K ** -0.5, chunk_size=C)
    for n, r in zip(("q", "k", "v"), ref):
        assert_close("d" + n, leaves[n].grad, r, torch.float32)
    assert_close("dg", gl.grad, ref[3], torch.float32)
    assert_close("dh0", leaves["h0"].grad, ref[4], torch.float32)
    # the recurrent mode gives the same output, also reversed / packed
    o_rec, ht_rec = simple_gla(c["q"], c["k"], c["v"], g=g.cuda(), initial_state=c["h0"], output_final_state=True,
                               mode="fused_recurrent")
    assert_close("o(rec)", o_rec, o.detach(), torch.float32)
    assert_close("ht(rec)", ht_rec, ht.detach(), torch.float32)
    with pytest.raises(ValueError):
        simple_gla(c["q"], c["k"], c["v"], g=g.cuda(), reverse=True, mode="chunk")
    with pytest.raises(ValueError):
        simple_gla(c["q"], c["k"], c["v"], g=g.cuda(), mode="bogus")


def test_chunk_simple_gla_varlen():
    from tops_b200.ops.simple_gla import chunk_simple_gla, chunk_simple_gla_bwd
    cu = [0, 5, 21, 70]
    T, H, K, V, C = cu[-1], 2, 32, 32, 16
    x, g, _ = _make(23, 1, T, H, K, V, torch.float32, "g", False)
    gen = torch.Generator().manual_seed(3)
    h0, dht = 0.1 * torch.randn(3, H, K, V, generator=gen), 0.1 * torch.randn(3, H, K, V, generator=gen)
    o_ref, ht_ref = O.chunk_simple_gla(x["q"], x["k"], x["v"], g, None, None, h0, True, cu_seqlens=cu, chunk_size=C)
    ref = O.chunk_simple_gla_bwd(x["q"], x["k"], x["v"], g, None, h0, x["do"], dht, K ** -0.5, chunk_size=C,
                                 cu_seqlens=cu)
    c = to_cuda(x)
    o, ht = chunk_simple_gla(c["q"], c["k"], c["v"], g.cuda(), None, None, h0.cuda(), True, cu_seqlens=cu, chunk_size=C)
    assert_close("o", o, o_ref, torch.float32)
    assert_close("ht", ht, ht_ref, torch.float32)
    got = chunk_simple_gla_bwd(c["q"], c["k"], c["v"], g.cuda(), None, h0.cuda(), c["do"], dht.cuda(), K ** -0.5,
                               chunk_size=C, cu_seqlens=cu)
    for name, a, b in zip(("dq", "dk", "dv", "dg", "dh0"), got, ref):
        assert_close(name, a, b, torch.float32)


@pytest.mark.parametrize("B,T,H", [
    (1, 64, 1),        # a single chunk
    (1, 512, 2),
    (3, 192, 16),      # 48 (batch, head) pairs: the fused forward
    (1, 2048, 3),      # few pairs, 32 chunks: time segments with summary scans and the join kernel
    (2, 1536, 37),     # fused forward over two segments
])
def test_scalar_gate_on_tensor_core_kernels(B, T, H):
    """bf16 scalar gates with K = V = 128, chunk 64 run on the tcgen05 GLA kernels in their scalar-gate
    form (the gate is read as [B,T,H]; the gate gradient comes back summed over the channels)."""
    from tops_b200 import _lib as L
    from tops_b200.ops.simple_gla import chunk_simple_gla, chunk_simple_gla_bwd
    from tops_b200.synth import make_inputs
    K, V, C = 128, 128, 64
    x = make_inputs(24, B, T, H, K, V, dtype=torch.bfloat16, gate="scalar", with_h0=True, with_grads=True)
    assert x["g"].dtype == torch.bfloat16
    scale = K ** -0.5
    o_ref, ht_ref = O.chunk_simple_gla(x["q"], x["k"], x["v"], x["g"], None, scale, x["h0"], True, chunk_size=C)
    ref = O.chunk_simple_gla_bwd(x["q"], x["k"], x["v"], x["g"], None, x["h0"], x["do"], x["dht"], scale, chunk_size=C)
    c = to_cuda(x)
    L.lib.tops_b200_profile_enable(1)
    o, ht = chunk_simple_gla(c["q"], c["k"], c["v"], c["g"], None, scale, c["h0"], True, chunk_size=C)
    got = chunk_simple_gla_bwd(c["q"], c["k"], c["v"], c["g"], None, c["h0"], c["do"], c["dht"], scale, chunk_size=C)
    L.lib.tops_b200_profile_enable(0)
    import ctypes
    buf = ctypes.create_string_buffer(4096)
    L.lib.tops_b200_profile_read(buf, len(buf))
    assert all(ln.startswith("sm100_") for ln in buf.value.decode().splitlines()), buf.value
    assert L.device_error() == 0
    assert_close("o", o, o_ref, torch.bfloat16)
    assert_close("ht", ht, ht_ref, torch.bfloat16)
    assert got[0].dtype == torch.bfloat16 and got[3].shape == (B, T, H)
    for name, a, b in zip(("dq", "dk", "dv", "dg", "dh0"), got, ref):
        assert_close(name, a, b, torch.bfloat16)


@pytest.mark.parametrize("C", [64, 128])
@pytest.mark.parametrize("gamma_val", [-0.5, -0.8, -1.0])
def test_large_constant_decay_stays_finite(gamma_val, C):
    """|g_gamma|·(C−1) beyond the range of fp32 exp() (the no-NaN cases of the reference's
    tests/ops/simple_gla/test_chunk_simple_gla_tpu.py:309-383): every exponent the kernels form is anchored,
    so outputs and gradients stay finite and keep the bf16 bar."""
    from tops_b200.ops.simple_gla import chunk_simple_gla, chunk_simple_gla_bwd
    B, T, H, K, V = 1, 256, 2, 128, 128
    gen = torch.Generator().manual_seed(42)
    x = {n: torch.randn(B, T, H, 128, generator=gen).to(torch.bfloat16) for n in ("q", "k", "v", "do")}
    gamma = torch.full((H,), gamma_val)
    scale = K ** -0.5
    o_ref, ht_ref = O.chunk_simple_gla(x["q"], x["k"], x["v"], None, gamma, None, None, True, chunk_size=C)
    ref = O.chunk_simple_gla_bwd(x["q"], x["k"], x["v"], None, gamma, None, x["do"], None, scale, chunk_size=C)
    c = to_cuda(x)
    o, ht = chunk_simple_gla(c["q"], c["k"], c["v"], None, gamma.cuda(), None, None, True, chunk_size=C)
    got = chunk_simple_gla_bwd(c["q"], c["k"], c["v"], None, gamma.cuda(), None, c["do"], None, scale, chunk_size=C)
    for name, a, b in (("o", o, o_ref), ("ht", ht, ht_ref), ("dq", got[0], ref[0]), ("dk", got[1], ref[1]),
                       ("dv", got[2], ref[2])):
        assert torch.isfinite(a.float()).all(), name
        assert_close(name, a, b, torch.bfloat16)
