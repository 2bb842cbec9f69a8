"""GPU parity: chunked / recurrent GLA kernels (through the C ABI) against the
CPU oracle on identical seeded inputs.  Shape lists follow the reference's
kernel tests (tests/ops/gla/test_pallas_chunk_gla.py:24-100,
tests/ref/gla/test_chunk_gla.py:62-109, test_fused_recurrent_gla.py:153-160)."""
import pytest
import torch

from oracle import gla as O
from tests.util import assert_close, to_cuda

pytestmark = pytest.mark.gpu


def _inputs(seed, B, T, H, K, V, dtype, **kw):
    from tops_b200.synth import make_inputs
    return make_inputs(seed, B, T, H, K, V, dtype=dtype, **kw)


FWD_SHAPES = [
    # B, T, H, K, V, chunk, dtype, h0
    (2, 512, 4, 64, 64, 64, torch.float32, False),     # BASELINE config 1
    (1, 64, 1, 32, 32, 16, torch.float32, True),
    (2, 1, 2, 16, 16, 16, torch.float32, False),        # T = 1
    (1, 3, 1, 8, 16, 16, torch.float32, True),          # T = 3, K != V, tiny dims
    (2, 37, 3, 16, 24, 16, torch.float32, True),        # ragged T
    (1, 100, 2, 64, 128, 32, torch.float32, True),
    (2, 130, 2, 128, 64, 64, torch.float32, False),
    (1, 256, 2, 96, 80, 64, torch.float32, True),       # K, V not multiples of 64
    (2, 256, 4, 128, 128, 64, torch.bfloat16, True),
    (1, 200, 2, 64, 64, 64, torch.bfloat16, False),
    (1, 128, 2, 64, 64, 32, torch.float16, True),
]


@pytest.mark.parametrize("B,T,H,K,V,C,dtype,h0", FWD_SHAPES)
def test_chunk_gla_forward(B, T, H, K, V, C, dtype, h0):
    from tops_b200.ops.gla import chunk_gla
    x = _inputs(1, B, T, H, K, V, dtype, with_h0=h0)
    o_ref, ht_ref = O.chunk_gla(x["q"], x["k"], x["v"], x["g"], None, x.get("h0"), True, chunk_size=C)
    c = to_cuda(x)
    o, ht = chunk_gla(c["q"], c["k"], c["v"], c["g"], scale=None, initial_state=c.get("h0"),
                      output_final_state=True, chunk_size=C)
    assert o.dtype == dtype and ht.dtype == torch.float32
    assert_close("o", o, o_ref, dtype)
    assert_close("ht", ht, ht_ref, dtype)


def test_chunk_gla_fwd_intermediates_and_dtypes():
    """dtype contract of the reference (tests/ref/gla/test_chunk_gla.py:245-293)."""
    from tops_b200.ops.gla import chunk_gla_fwd
    B, T, H, K, V, C = 2, 128, 2, 64, 64, 32
    x = _inputs(3, B, T, H, K, V, torch.bfloat16, with_h0=True)
    gc_ref, A_ref, h_ref, ht_ref, o_ref = O.chunk_gla_fwd(x["q"], x["k"], x["v"], x["g"], None, K ** -0.5,
                                                         x["h0"], True, chunk_size=C)
    c = to_cuda(x)
    gc, A, h, ht, o = chunk_gla_fwd(c["q"], c["k"], c["v"], c["g"], None, K ** -0.5, c["h0"], True, chunk_size=C)
    assert gc.dtype == torch.float32 and A.dtype == torch.float32 and ht.dtype == torch.float32
    assert h.dtype == torch.bfloat16 and o.dtype == torch.bfloat16
    assert_close("g_cumsum", gc, gc_ref, torch.float32)
    assert_close("A", A, A_ref, torch.bfloat16)
    assert_close("h", h, h_ref, torch.bfloat16)
    assert_close("o", o, o_ref, torch.bfloat16)


BWD_SHAPES = [
    (2, 128, 2, 64, 64, 64, torch.float32, True),
    (1, 37, 2, 16, 24, 16, torch.float32, True),
    (2, 100, 1, 32, 64, 32, torch.float32, False),
    (1, 192, 2, 128, 128, 64, torch.float32, True),
    (2, 256, 2, 128, 128, 64, torch.bfloat16, True),
    (1, 130, 2, 64, 96, 64, torch.bfloat16, False),
    (2, 128, 2, 64, 64, 32, torch.float16, True),
    (1, 192, 3, 128, 128, 64, torch.float16, False),
]


@pytest.mark.parametrize("B,T,H,K,V,C,dtype,h0", BWD_SHAPES)
def test_chunk_gla_backward(B, T, H, K, V, C, dtype, h0):
    from tops_b200.ops.gla import chunk_gla_bwd
    x = _inputs(2, B, T, H, K, V, dtype, with_h0=h0, with_grads=True)
    scale = K ** -0.5
    ref = O.chunk_gla_bwd(x["q"], x["k"], x["v"], x["g"], None, scale, x.get("h0"), None, None, x["do"],
                          x["dht"], chunk_size=C)
    c = to_cuda(x)
    got = chunk_gla_bwd(c["q"], c["k"], c["v"], c["g"], None, scale, c.get("h0"), None, None, c["do"], c["dht"],
                        chunk_size=C)
    assert got[0].dtype == torch.float32 and got[1].dtype == torch.float32 and got[3].dtype == torch.float32
    assert got[2].dtype == dtype
    for name, a, b in zip(("dq", "dk", "dv", "dg"), got, ref):
        assert_close(name, a, b, dtype)
    if h0:
        assert_close("dh0", got[4], ref[4], dtype)
    else:
        assert got[4] is None and ref[4] is None


def test_chunk_gla_autograd_matches_explicit_backward():
    from tops_b200.ops.gla import chunk_gla
    B, T, H, K, V, C = 1, 96, 2, 32, 32, 32
    x = to_cuda(_inputs(4, B, T, H, K, V, torch.float32, with_h0=True, with_grads=True))
    leaves = {n: x[n].clone().requires_grad_() for n in ("q", "k", "v", "g", "h0")}
    o, ht = chunk_gla(leaves["q"], leaves["k"], leaves["v"], leaves["g"], initial_state=leaves["h0"],
                      output_final_state=True, chunk_size=C)
    ((o * x["do"]).sum() + (ht * x["dht"]).sum()).backward()
    cpu = {n: t.detach().cpu() for n, t in x.items()}
    ref = O.chunk_gla_bwd(cpu["q"], cpu["k"], cpu["v"], cpu["g"], None, K ** -0.5, cpu["h0"], None, None,
                          cpu["do"], cpu["dht"], chunk_size=C)
    for n, r in zip(("q", "k", "v", "g", "h0"), ref):
        assert_close("d" + n, leaves[n].grad, r, torch.float32)


def test_state_split_equals_single_pass():
    """Two halves chained through the state equal one pass
    (tests/ops/gla/test_pallas_chunk_gla.py:223-247)."""
    from tops_b200.ops.gla import chunk_gla
    B, T, H, K, V, C = 2, 256, 2, 64, 64, 64
    x = to_cuda(_inputs(5, B, T, H, K, V, torch.float32, with_h0=True))
    o, ht = chunk_gla(x["q"], x["k"], x["v"], x["g"], initial_state=x["h0"], output_final_state=True, chunk_size=C)
    h = T // 2
    o1, s1 = chunk_gla(x["q"][:, :h], x["k"][:, :h], x["v"][:, :h], x["g"][:, :h], initial_state=x["h0"],
                       output_final_state=True, chunk_size=C)
    o2, s2 = chunk_gla(x["q"][:, h:], x["k"][:, h:], x["v"][:, h:], x["g"][:, h:], initial_state=s1,
                       output_final_state=True, chunk_size=C)
    assert_close("o", torch.cat([o1, o2], 1), o, torch.float32)
    assert_close("ht", s2, ht, torch.float32)


def test_large_gates_stay_finite():
    """Raw log-sigmoid gates (not divided by 16) and stronger decays must not
    overflow (tests/ops/gla/test_exp_overflow_stabilization.py:62-221)."""
    from tops_b200.ops.gla import chunk_gla, chunk_gla_bwd
    B, T, H, K, V, C = 1, 128, 2, 64, 64, 64
    x = _inputs(6, B, T, H, K, V, torch.float32, gate_norm=1.0, with_grads=True)
    x["g"] = x["g"] * 1.2
    ref_o, _ = O.naive_recurrent_gla(x["q"].double(), x["k"].double(), x["v"].double(), x["g"].double())
    c = to_cuda(x)
    o, _ = chunk_gla(c["q"], c["k"], c["v"], c["g"], chunk_size=C)
    assert torch.isfinite(o).all()
    assert (o.cpu().double() - ref_o).abs().max().item() < 1e-3
    grads = chunk_gla_bwd(c["q"], c["k"], c["v"], c["g"], None, K ** -0.5, None, None, None, c["do"], None,
                          chunk_size=C)
    for t in grads[:4]:
        assert torch.isfinite(t).all()


@pytest.mark.parametrize("cu", [[0, 37, 38, 100], [0, 64, 128], [0, 5, 21, 150]])
def test_chunk_gla_varlen(cu):
    from tops_b200.ops.gla import chunk_gla, chunk_gla_bwd
    T, H, K, V, C = cu[-1], 2, 32, 48, 16
    N = len(cu) - 1
    x = _inputs(7, 1, T, H, K, V, torch.float32, with_grads=True)
    torch.manual_seed(0)
    h0 = 0.1 * torch.randn(N, H, K, V)
    dht = 0.1 * torch.randn(N, H, K, V)
    o_ref, ht_ref = O.chunk_gla(x["q"], x["k"], x["v"], x["g"], None, h0, True, cu_seqlens=cu, chunk_size=C)
    ref = O.chunk_gla_bwd(x["q"], x["k"], x["v"], x["g"], None, K ** -0.5, h0, None, None, x["do"], dht,
                          chunk_size=C, cu_seqlens=cu)
    c = to_cuda(x)
    o, ht = chunk_gla(c["q"], c["k"], c["v"], c["g"], initial_state=h0.cuda(), output_final_state=True,
                      cu_seqlens=cu, chunk_size=C)
    assert_close("o", o, o_ref, torch.float32)
    assert_close("ht", ht, ht_ref, torch.float32)
    got = chunk_gla_bwd(c["q"], c["k"], c["v"], c["g"], None, K ** -0.5, h0.cuda(), None, None, c["do"],
                        dht.cuda(), chunk_size=C, cu_seqlens=cu)
    for name, a, b in zip(("dq", "dk", "dv", "dg", "dh0"), got, ref):
        assert_close(name, a, b, torch.float32)


def test_chunk_primitives():
    """chunk_local_cumsum / chunk_fwd_h / chunk_bwd_dh as separate calls."""
    from tops_b200.ops.common import chunk_bwd_dh, chunk_fwd_h, chunk_local_cumsum
    from oracle import common as OC
    B, T, H, K, V, C = 2, 128, 2, 64, 32, 32
    x = _inputs(8, B, T, H, K, V, torch.float32, with_h0=True, with_grads=True)
    c = to_cuda(x)
    for rev in (False, True):
        assert_close("cumsum", chunk_local_cumsum(c["g"], C, reverse=rev), OC.chunk_local_cumsum(x["g"], C, rev),
                     torch.float32)
    gs = x["g"][..., 0].contiguous()
    assert_close("cumsum3d", chunk_local_cumsum(gs.cuda(), C), OC.chunk_local_cumsum(gs, C), torch.float32)
    gc = OC.chunk_local_cumsum(x["g"], C)
    h_ref, ht_ref = OC.chunk_fwd_h(x["k"], x["v"], gk=gc, h0=x["h0"], output_final_state=True,
                                   states_in_fp32=True, chunk_size=C)
    h, ht = chunk_fwd_h(c["k"], c["v"], gk=gc.cuda(), h0=c["h0"], output_final_state=True, states_in_fp32=True,
                        chunk_size=C)
    assert_close("h", h, h_ref, torch.float32)
    assert_close("ht", ht, ht_ref, torch.float32)
    dh_ref, dh0_ref = OC.chunk_bwd_dh(x["q"], x["do"], gk=gc, h0=x["h0"], dht=x["dht"], scale=K ** -0.5, chunk_size=C)
    dh, dh0 = chunk_bwd_dh(c["q"], c["do"], gk=gc.cuda(), h0=c["h0"], dht=c["dht"], scale=K ** -0.5, chunk_size=C)
    assert_close("dh", dh, dh_ref, torch.float32)
    assert_close("dh0", dh0, dh0_ref, torch.float32)
    # scalar gate and constant decay variants of the state scan
    gsc = OC.chunk_local_cumsum(gs, C)
    h_ref, _ = OC.chunk_fwd_h(x["k"], x["v"], g=gsc, h0=x["h0"], states_in_fp32=True, chunk_size=C)
    h, _ = chunk_fwd_h(c["k"], c["v"], g=gsc.cuda(), h0=c["h0"], states_in_fp32=True, chunk_size=C)
    assert_close("h(g)", h, h_ref, torch.float32)
    gam = -torch.rand(H) * 0.1
    h_ref, _ = OC.chunk_fwd_h(x["k"], x["v"], g_gamma=gam, h0=x["h0"], states_in_fp32=True, chunk_size=C)
    h, _ = chunk_fwd_h(c["k"], c["v"], g_gamma=gam.cuda(), h0=c["h0"], states_in_fp32=True, chunk_size=C)
    assert_close("h(gamma)", h, h_ref, torch.float32)


REC_SHAPES = [
    # B, T, H, K, V, dtype, gk, gv, h0, reverse
    (2, 64, 2, 32, 32, torch.float32, True, False, True, False),
    (1, 37, 3, 16, 24, torch.float32, True, True, True, False),
    (2, 50, 1, 64, 128, torch.float32, False, False, False, False),
    (1, 40, 2, 128, 128, torch.float32, True, False, True, True),
    (2, 1, 2, 128, 128, torch.bfloat16, True, False, True, False),
    (1, 96, 2, 64, 64, torch.bfloat16, True, True, False, False),
    (1, 20, 2, 100, 72, torch.float32, False, True, True, False),
]


@pytest.mark.parametrize("B,T,H,K,V,dtype,use_gk,use_gv,h0,reverse", REC_SHAPES)
def test_fused_recurrent_forward_backward(B, T, H, K, V, dtype, use_gk, use_gv, h0, reverse):
    from tops_b200.ops.gla import fused_recurrent_bwd, fused_recurrent_fwd, fused_recurrent_gla
    x = _inputs(9, B, T, H, K, V, dtype, with_h0=h0, with_grads=True)
    rng = torch.Generator().manual_seed(1)
    gv = (torch.nn.functional.logsigmoid(torch.randn(B, T, H, V, generator=rng)) / 16).to(dtype) if use_gv else None
    gk = x["g"] if use_gk else None
    o32_ref, ht_ref = O.fused_recurrent_fwd(x["q"], x["k"], x["v"], gk, gv, None, x.get("h0"), True, reverse)
    c = to_cuda(x)
    gvc = None if gv is None else gv.cuda()
    gkc = c["g"] if use_gk else None
    o32, ht = fused_recurrent_fwd(c["q"], c["k"], c["v"], gkc, gvc, None, c.get("h0"), True, reverse)
    assert o32.dtype == torch.float32
    assert_close("o", o32, o32_ref, dtype)
    assert_close("ht", ht, ht_ref, dtype)
    o, _ = fused_recurrent_gla(c["q"], c["k"], c["v"], gkc, gvc, None, c.get("h0"), False, reverse)
    assert o.dtype == dtype
    if max(K, V) > 128:
        return
    ref = O.fused_recurrent_bwd(x["q"], x["k"], x["v"], gk, gv, o32_ref, x["do"], x["dht"], None, x.get("h0"), reverse)
    got = fused_recurrent_bwd(c["q"], c["k"], c["v"], gkc, gvc, o32, c["do"], c["dht"], None, c.get("h0"), reverse)
    for name, a, b in zip(("dq", "dk", "dv", "dgk", "dgv", "dh0"), got, ref):
        if b is None:
            assert a is None, name
            continue
        assert a.dtype == b.dtype, name
        assert_close(name, a, b, dtype)


def test_fused_recurrent_varlen_and_decode():
    from tops_b200.ops.gla import fused_recurrent_gla, fused_recurrent_gla_decode_
    H, K, V = 2, 64, 64
    cu = [0, 1, 20, 33]
    x = _inputs(10, 1, cu[-1], H, K, V, torch.float32)
    h0 = 0.1 * torch.randn(3, H, K, V, generator=torch.Generator().manual_seed(2))
    o_ref, ht_ref = O.fused_recurrent_gla(x["q"], x["k"], x["v"], x["g"], None, None, h0, True, False, cu)
    c = to_cuda(x)
    o, ht = fused_recurrent_gla(c["q"], c["k"], c["v"], c["g"], None, None, h0.cuda(), True, False, cu)
    assert_close("o", o, o_ref, torch.float32)
    assert_close("ht", ht, ht_ref, torch.float32)
    # decode: token-by-token in-place state updates equal one multi-token call
    B, T = 3, 8
    y = _inputs(11, B, T, H, K, V, torch.bfloat16, with_h0=True)
    o_ref, ht_ref = O.fused_recurrent_gla(y["q"], y["k"], y["v"], y["g"], None, None, y["h0"], True)
    d = to_cuda(y)
    state = d["h0"].clone()
    outs = [fused_recurrent_gla_decode_(d["q"][:, t:t + 1], d["k"][:, t:t + 1], d["v"][:, t:t + 1],
                                        d["g"][:, t:t + 1], state) for t in range(T)]
    assert_close("o", torch.cat(outs, 1), o_ref, torch.bfloat16)
    assert_close("state", state, ht_ref, torch.bfloat16)


def test_bad_arguments_raise_before_launch():
    from tops_b200.ops.gla import chunk_gla
    x = to_cuda(_inputs(12, 1, 32, 2, 16, 16, torch.float32))
    with pytest.raises(AssertionError):
        chunk_gla(x["q"], x["k"][:, :16], x["v"], x["g"])
    with pytest.raises(AssertionError):
        chunk_gla(x["q"], x["k"], x["v"], x["g"], initial_state=torch.zeros(2, 2, 16, 16, device="cuda"))
    with pytest.raises(AssertionError):
        chunk_gla(x["q"], x["k"], x["v"], x["g"], cu_seqlens=[0, 16, 16, 32])


@pytest.mark.parametrize("chunk_size", [8, 128, 256])
def test_chunk_sizes_beyond_the_kernel_tiles(chunk_size):
    """Any power of two is a valid chunk_size (tops/ops/common/cumsum.py:506-508; the reference's tests use
    128): the differentiable ops give the chunk-size independent result, computed with a length the kernels hold."""
    from tops_b200.ops.gla import chunk_gla
    from tops_b200.ops.simple_gla import chunk_simple_gla
    B, T, H, K, V = 1, 256, 2, 64, 64
    x = _inputs(9, B, T, H, K, V, torch.float32, with_h0=True)
    c = to_cuda(x)
    o, ht = chunk_gla(c["q"], c["k"], c["v"], c["g"], initial_state=c["h0"], output_final_state=True, chunk_size=chunk_size)
    o_ref, ht_ref = O.chunk_gla(x["q"], x["k"], x["v"], x["g"], K ** -0.5, x["h0"], True, chunk_size=64)
    assert_close("o", o, o_ref, torch.float32)
    assert_close("ht", ht, ht_ref, torch.float32)
    gs = c["g"].mean(-1)
    o2, _ = chunk_simple_gla(c["q"], c["k"], c["v"], g=gs, initial_state=c["h0"], chunk_size=chunk_size)
    o3, _ = chunk_simple_gla(c["q"], c["k"], c["v"], g=gs, initial_state=c["h0"], chunk_size=64)
    assert_close("simple_gla o", o2, o3.cpu(), torch.float32)
    with pytest.raises(AssertionError):
        chunk_gla(c["q"], c["k"], c["v"], c["g"], chunk_size=48)
    # the explicit backward hands no per-chunk tensor back either; the forward orchestrator does and says so
    from tops_b200.ops.gla import chunk_gla_bwd, chunk_gla_fwd
    do = torch.randn_like(c["v"])
    got = chunk_gla_bwd(c["q"], c["k"], c["v"], c["g"], None, K ** -0.5, c["h0"], None, None, do, None,
                        chunk_size=chunk_size)
    want = chunk_gla_bwd(c["q"], c["k"], c["v"], c["g"], None, K ** -0.5, c["h0"], None, None, do, None, chunk_size=64)
    for name, a, b in zip(("dq", "dk", "dv", "dg", "dh0"), got, want):
        assert_close(name, a, b.cpu(), torch.float32)
    with pytest.raises(AssertionError):
        chunk_gla_fwd(c["q"], c["k"], c["v"], c["g"], None, K ** -0.5, None, False, chunk_size=chunk_size)
