"""The CUDA kernels against outputs of the REFERENCE's own CPU implementation (`tests/golden/ref_*.pt`,
produced by `tests/golden/make_reference_golden.py` from the reference's unmodified source files): the direct
link kernel <-> reference, without the oracle in between.  float64 cases run in float32 on the GPU (the
kernels' widest type) and meet the float32 bar; half-precision cases meet the relative-L2 bar."""
import os

import pytest
import torch

from tests.golden.make_reference_golden import CASES as ALL_CASES, case_inputs, gate_inputs
from tests.util import assert_close, to_cuda

pytestmark = pytest.mark.gpu
CASES = {n: c for n, c in ALL_CASES.items() if not c.get("cpu_only")}
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _inputs(c):
    x = case_inputs(c)
    if c["dtype"] == "float64":
        x = {k: (v.float() if v.is_floating_point() else v) for k, v in x.items()}
    return x, (torch.float32 if c["dtype"] == "float64" else getattr(torch, c["dtype"]))


def _check(ref, got, dtype):
    """Every tensor inside the bar; the errors are printed (`pytest -s`) as max-abs for fp32, relative L2 for half."""
    errs = {}
    for key, a in got.items():
        if key not in ref:        # a forward-only fixture
            continue
        r = ref[key]
        if r is None:
            assert a is None, key
            continue
        errs[key] = assert_close(key, a.float() if a.dtype != torch.float32 else a, r.float(), dtype)
    print({k: float(f"{v:.2e}") for k, v in errs.items()})


@pytest.mark.parametrize("name", [n for n, c in CASES.items() if c["op"] == "gla"])
def test_gla_kernels_match_the_reference(name):
    from tops_b200.ops import gla
    c = CASES[name]
    ref = torch.load(os.path.join(GOLDEN, name + ".pt"))
    host, dtype = _inputs(c)
    x = to_cuda(host)
    scale = c["K"] ** -0.5
    cu = c.get("cu_seqlens")
    fin = c.get("state") is not False
    o, ht = gla.chunk_gla(x["q"], x["k"], x["v"], x["g"], scale=scale, initial_state=x["h0"], output_final_state=fin,
                          cu_seqlens=cu, chunk_size=c["C"])
    dq, dk, dv, dg, dh0 = gla.chunk_gla_bwd(x["q"], x["k"], x["v"], x["g"], None, scale, x["h0"], None, None, x["do"],
                                            x["dht"], chunk_size=c["C"], cu_seqlens=cu)
    got = dict(o=o, dq=dq, dk=dk, dv=dv, dg=dg)
    if fin:
        got.update(ht=ht, dh0=dh0)
    else:
        assert ht is None and dh0 is None
    _check(ref, got, dtype)
    if "A" in ref:        # the per-chunk tensors of the forward orchestrator
        gcum, A, h, _, _ = gla.chunk_gla_fwd(x["q"], x["k"], x["v"], x["g"], None, scale, x["h0"], fin, chunk_size=c["C"])
        _check(ref, dict(g_cumsum=gcum, A=A, h=h), dtype)


@pytest.mark.parametrize("name", [n for n, c in CASES.items() if c["op"] == "recurrent"])
def test_recurrent_kernels_match_the_reference(name):
    from tops_b200.ops import gla
    c = CASES[name]
    ref = torch.load(os.path.join(GOLDEN, name + ".pt"))
    host, dtype = _inputs(c)
    x = to_cuda(host)
    scale = c["K"] ** -0.5
    cu = c.get("cu_seqlens")
    o, ht = gla.fused_recurrent_fwd(x["q"], x["k"], x["v"], x["g"], x["gv"], scale, x["h0"], True, c["reverse"], cu)
    dq, dk, dv, dgk, dgv, dh0 = gla.fused_recurrent_bwd(x["q"], x["k"], x["v"], x["g"], x["gv"], o, x["do"], x["dht"],
                                                        scale, x["h0"], c["reverse"], cu)
    _check(ref, dict(o=o, ht=ht, dq=dq, dk=dk, dv=dv, dgk=dgk, dgv=dgv, dh0=dh0), dtype)


@pytest.mark.parametrize("name", [n for n, c in CASES.items() if c["op"] == "simple_gla"])
def test_simple_gla_kernels_match_the_reference(name):
    from tops_b200.ops import simple_gla
    c = CASES[name]
    ref = torch.load(os.path.join(GOLDEN, name + ".pt"))
    host, dtype = _inputs(c)
    x = to_cuda(host)
    scale = c["K"] ** -0.5
    g = x["g"] if c["gate"] == "g" else None
    gam = x["gamma"] if c["gate"] == "gamma" else None
    cu = c.get("cu_seqlens")
    fin = c.get("state") is not False
    o, ht = simple_gla.chunk_simple_gla(x["q"], x["k"], x["v"], g, gam, scale, x["h0"], fin, cu_seqlens=cu,
                                        chunk_size=c["C"])
    dq, dk, dv, dg, dh0 = simple_gla.chunk_simple_gla_bwd(x["q"], x["k"], x["v"], g, gam, x["h0"], x["do"], x["dht"],
                                                          scale, chunk_size=c["C"], cu_seqlens=cu)
    got = dict(o=o, dq=dq, dk=dk, dv=dv, dg=dg)
    if fin:
        got.update(ht=ht, dh0=dh0)
    else:
        assert ht is None and dh0 is None
    if "o_recurrent" in ref:
        orc, htr = simple_gla.fused_recurrent_simple_gla(x["q"], x["k"], x["v"], g=g, g_gamma=gam, scale=scale,
                                                         initial_state=x["h0"], output_final_state=fin)
        got.update(o_recurrent=orc, **({"ht_recurrent": htr} if fin else {}))
    _check(ref, got, dtype)


@pytest.mark.parametrize("name", [n for n, c in CASES.items() if c["op"] == "cumsum"])
def test_cumsum_kernel_matches_the_reference(name):
    from tops_b200.ops.common import chunk_local_cumsum as cs
    c = CASES[name]
    ref = torch.load(os.path.join(GOLDEN, name + ".pt"))
    host, dtype = _inputs(c)
    g = host["g"].cuda()
    gs = g[..., 0].contiguous()
    cu = c["cu_seqlens"]
    got = dict(fwd4=cs(g, c["C"]), rev4=cs(g, c["C"], reverse=True), fwd3=cs(gs, c["C"]),
               rev3=cs(gs, c["C"], reverse=True), packed4=cs(g, c["C"], cu_seqlens=cu),
               packed_rev3=cs(gs, c["C"], reverse=True, cu_seqlens=cu))
    _check(ref, got, dtype)


@pytest.mark.parametrize("name", [n for n, c in CASES.items() if c["op"] == "kda"])
def test_kda_kernels_match_the_reference(name):
    """The token-serial kernels on the small shapes, the chunked tensor-core kernels at K = V = 128, against the
    reference's token recurrence and its explicit token-level backward."""
    from tops_b200.ops import kda
    c = CASES[name]
    ref = torch.load(os.path.join(GOLDEN, name + ".pt"))
    host, dtype = _inputs(c)
    x = to_cuda(host)
    scale = c["K"] ** -0.5
    fin = c.get("state") is not False
    if c["K"] == 128:
        assert kda.chunk_kernels_take(x["q"], x["k"], x["v"], x["g"], x["beta"], 64)
        o, ht, _, _, _ = kda.chunk_kda_fwd(x["q"], x["k"], x["v"], x["g"], x["beta"], scale, x["h0"], True)
        dq, dk, dv, db, dg, dh0 = kda.chunk_kda_bwd(x["q"], x["k"], x["v"], x["g"], x["beta"], x["do"], scale, x["h0"],
                                                    x["dht"])
    else:
        o, ht = kda.kda_fwd(x["q"], x["k"], x["v"], x["g"], x["beta"], scale, x["h0"], fin)
        dq, dk, dv, dg, db, dh0 = kda.kda_bwd(x["q"], x["k"], x["v"], x["g"], x["beta"], x["do"], scale, x["h0"], x["dht"])
    got = dict(o=o, dq=dq, dk=dk, dv=dv, dg=dg, dbeta=db)
    if fin:
        got.update(ht=ht, dh0=dh0)
    else:
        assert ht is None and dh0 is None
    _check(ref, got, dtype)


@pytest.mark.parametrize("name", [n for n, c in CASES.items() if c["op"] == "kda_gate"])
def test_kda_gate_kernels_match_the_reference(name):
    from tops_b200.ops import gate
    c = CASES[name]
    ref = torch.load(os.path.join(GOLDEN, name + ".pt"))
    x = to_cuda(gate_inputs(c))
    got = dict(plain=gate.kda_gate_fwd(x["g"], x["A_log"]),
               biased=gate.kda_gate_fwd(x["g"], x["A_log"], x["dt_bias"]),
               bounded=gate.kda_gate_fwd(x["g"], x["A_log"], x["dt_bias"], lower_bound=-5.0),
               cumsum_log2=gate.kda_gate_chunk_cumsum(x["g"], x["A_log"], c["C"], scale=1.4426950408889634,
                                                      dt_bias=x["dt_bias"]))
    _check(ref, got, torch.float32)


@pytest.mark.parametrize("name", [n for n, c in CASES.items() if c["op"] == "layer"])
def test_layer_on_the_kernels_matches_the_reference_layer(name):
    """`tops_b200.layers.GatedLinearAttention` on the GPU with the parameters the reference's layer was run with."""
    from tests.golden.make_reference_golden import layer_inputs
    from tests.test_reference_golden import build_layer
    c = CASES[name]
    ref = torch.load(os.path.join(GOLDEN, name + ".pt"))
    layer = build_layer(c, ref).cuda()
    with torch.no_grad():
        y, _, _ = layer(layer_inputs(c).cuda())
    bar = 2e-4 * max(1.0, ref["y"].abs().max().item())
    assert (y.cpu() - ref["y"]).abs().max().item() <= bar


@pytest.mark.parametrize("name", [n for n, c in CASES.items() if c["op"] == "public"])
def test_public_recurrent_ops_match_the_reference(name):
    """`fused_recurrent_kda`, recurrent GLA with an explicit scale, recurrent simple_gla with g + g_gamma and
    reversed, against the pure-jax entry points of the reference's accelerator-side package."""
    from tests.golden.make_reference_golden import public_inputs
    from tests.test_reference_golden import compare_public
    from tops_b200.ops import gla, kda, simple_gla
    c = CASES[name]
    ref = torch.load(os.path.join(GOLDEN, name + ".pt"))
    x = to_cuda(public_inputs(c))
    got = {}
    got["kda_o"], got["kda_ht"] = kda.fused_recurrent_kda(x["q"], x["kn"], x["v"], x["g"], x["beta"], 0.3, x["h0"], True)
    got["gla_o"], got["gla_ht"] = gla.fused_recurrent_gla(x["q"], x["k"], x["v"], gk=x["g"], scale=0.3,
                                                          initial_state=x["h0"], output_final_state=True)
    got["sg_o"], got["sg_ht"] = simple_gla.fused_recurrent_simple_gla(x["q"], x["k"], x["v"], g=x["gs"],
                                                                      g_gamma=x["gamma"], scale=0.3,
                                                                      initial_state=x["h0"], output_final_state=True)
    got["sg_rev_o"], got["sg_rev_ht"] = simple_gla.fused_recurrent_simple_gla(x["q"], x["k"], x["v"], g=x["gs"],
                                                                              scale=0.3, initial_state=x["h0"],
                                                                              output_final_state=True, reverse=True)
    compare_public(name, got, ref, "float32" if c["dtype"] == "float32" else "bfloat16")
