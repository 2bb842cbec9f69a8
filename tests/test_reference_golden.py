"""The oracle against outputs of the REFERENCE's own CPU implementation (no GPU).

`tests/golden/ref_*.pt` hold what the reference's unmodified `tops/cpu/ops/**` source files returned on the
seeded inputs of `tests/golden/make_reference_golden.py` (run on a numpy-backed stand-in for the jax API;
the generator's docstring says what that preserves).  This is the pin of `oracle/` to the reference itself:
float64 cases must agree to summation-order rounding, float32 cases to float32 rounding, and bf16 cases,
where every cast point matters, to a fraction of a bf16 step."""
import os

import pytest
import torch

from oracle import gla as G
from oracle import kda as K
from oracle import simple_gla as S
from oracle import aux as A
from oracle.common import chunk_local_cumsum
from tests.golden.make_reference_golden import CASES, case_inputs, gate_inputs, layer_inputs, public_inputs

HERE = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# |got - ref| <= tol * max|ref| per tensor
TOL = {"float64": 1e-12, "float32": 2e-5, "bfloat16": 2e-5, "float16": 2e-5}
HALF_STEP = {"bfloat16": 2.0 ** -8, "float16": 2.0 ** -11}   # one rounding step, relative to the tensor's largest value


def _load(name):
    return torch.load(os.path.join(HERE, name + ".pt"))


def _compare(name, got, ref, dtype, tol=None):
    for key, r in ref.items():
        if key not in got:
            continue
        g = got[key]
        if r is None:
            assert g is None, (name, key)
            continue
        assert g is not None, (name, key)
        assert g.dtype == r.dtype, (name, key, g.dtype, r.dtype)
        assert g.shape == r.shape, (name, key, g.shape, r.shape)
        diff = (g.double() - r.double()).abs()
        top = max(r.double().abs().max().item(), 1e-30)
        if dtype in ("bfloat16", "float16"):
            # numpy's and torch's float32 sums differ in their last bits; where such a sum is then rounded to bf16
            # (chunk states, gated operands) a value next to a rounding boundary can land on the other side and
            # move the few outputs that use it by one bf16 step.  So: no element further than one step, and all
            # but a few percent of the elements equal to float32 rounding.
            assert diff.max().item() <= HALF_STEP[dtype] * top, (name, key, diff.max().item(), top)
            assert (diff > TOL[dtype] * top).double().mean().item() <= 0.05, (name, key)
        else:
            assert diff.max().item() <= (tol or TOL[dtype]) * top, (name, key, diff.max().item(), top)


def _run(c, x):
    scale = c["K"] ** -0.5
    fin = c.get("state") is not False
    if c["op"] == "gla":
        cu = c.get("cu_seqlens")
        o, ht = G.chunk_gla(x["q"], x["k"], x["v"], x["g"], scale, x["h0"], fin, cu_seqlens=cu, chunk_size=c["C"])
        dq, dk, dv, dg, dh0 = G.chunk_gla_bwd(x["q"], x["k"], x["v"], x["g"], None, scale, x["h0"], None, None, x["do"],
                                              x["dht"], chunk_size=c["C"], cu_seqlens=cu)
        out = dict(o=o, ht=ht, dq=dq, dk=dk, dv=dv, dg=dg, dh0=dh0)
        if cu is None and not c.get("slim"):
            gc, A, h, _, _ = G.chunk_gla_fwd(x["q"], x["k"], x["v"], x["g"], None, scale, x["h0"], fin, chunk_size=c["C"])
            out.update(g_cumsum=gc, A=A, h=h)
            if c["dtype"] not in ("bfloat16", "float16"):
                on, htn = G.naive_recurrent_gla(x["q"], x["k"], x["v"], x["g"], x["h0"], fin)
                out.update(o_naive=on, ht_naive=htn)
        return out
    if c["op"] == "recurrent":
        cu = c.get("cu_seqlens")
        o, ht = G.fused_recurrent_fwd(x["q"], x["k"], x["v"], x["g"], x["gv"], scale, x["h0"], True, c["reverse"], cu)
        dq, dk, dv, dgk, dgv, dh0 = G.fused_recurrent_bwd(x["q"], x["k"], x["v"], x["g"], x["gv"], o, x["do"], x["dht"],
                                                          scale, x["h0"], c["reverse"], cu)
        return dict(o=o, ht=ht, dq=dq, dk=dk, dv=dv, dgk=dgk, dgv=dgv, dh0=dh0)
    if c["op"] == "simple_gla":
        g = x["g"] if c["gate"] == "g" else None
        gam = x["gamma"] if c["gate"] == "gamma" else None
        cu = c.get("cu_seqlens")
        o, ht = S.chunk_simple_gla(x["q"], x["k"], x["v"], g, gam, scale, x["h0"], fin, cu_seqlens=cu, chunk_size=c["C"])
        dq, dk, dv, dg, dh0 = S.chunk_simple_gla_bwd(x["q"], x["k"], x["v"], g, gam, x["h0"], x["do"], x["dht"], scale,
                                                     chunk_size=c["C"], cu_seqlens=cu)
        out = dict(o=o, ht=ht, dq=dq, dk=dk, dv=dv, dg=dg, dh0=dh0)
        if cu is None:
            # the recurrent form of the reference (fp32 state, output in q.dtype) against the oracle's token loop
            orc, htr = S.naive_recurrent_simple_gla(x["q"], x["k"], x["v"], g, gam, scale, x["h0"], fin)
            out.update(o_recurrent=orc.to(x["q"].dtype), ht_recurrent=htr)
        if cu is None and c["dtype"] not in ("bfloat16", "float16"):
            on, htn = S.naive_recurrent_simple_gla(x["q"], x["k"], x["v"], g, gam, scale, x["h0"], fin)
            out.update(o_naive=on, ht_naive=htn)
        return out
    if c["op"] == "defaults":
        out = {}
        out["o_nogate"], none1 = G.chunk_gla(x["q"], x["k"], x["v"])
        out["o_chunk"], none2 = G.chunk_gla(x["q"], x["k"], x["v"], x["g"])
        out["o_fused"], out["ht_fused"] = G.fused_chunk_gla(x["q"], x["k"], x["v"], x["g"], output_final_state=True)
        out["o_rec"], out["ht_rec"] = G.fused_recurrent_gla(x["q"], x["k"], x["v"], x["g"], initial_state=x["h0"],
                                                            output_final_state=True)
        out["o_rec_nogate"], none3 = G.fused_recurrent_gla(x["q"], x["k"], x["v"])
        assert none1 is None and none2 is None and none3 is None
        return out
    if c["op"] == "cumsum":
        from oracle.common import chunk_local_cumsum as cs
        cu = c["cu_seqlens"]
        gs = x["g"][..., 0]
        out = dict(fwd4=cs(x["g"], c["C"]), rev4=cs(x["g"], c["C"], reverse=True), fwd3=cs(gs, c["C"]),
                   rev3=cs(gs, c["C"], reverse=True), packed4=cs(x["g"], c["C"], cu_seqlens=cu),
                   packed_rev3=cs(gs, c["C"], reverse=True, cu_seqlens=cu))
        # the packed-batch helpers (tops/utils.py:71-90, tops/cpu/ops/common/utils.py:36-139): chunk table, chunks
        # cut out of the packed tensor with zero tails, their valid lengths, and the way back
        from oracle.common import prepare_chunk_indices
        ci = prepare_chunk_indices(cu, c["C"])
        rows, lens = [], []
        for n, k in ci.tolist():
            a = cu[n] + k * c["C"]
            b = min(a + c["C"], cu[n + 1])
            rows.append(torch.nn.functional.pad(x["g"][0, a:b], (0, 0, 0, 0, 0, c["C"] - (b - a))))
            lens.append(b - a)
        out.update(chunk_indices=ci, gathered=torch.stack(rows), valid_lens=torch.tensor(lens, dtype=torch.int32),
                   scattered=x["g"].clone())
        return out
    raise AssertionError(c["op"])


@pytest.mark.parametrize("name", [n for n, c in CASES.items() if c["op"] not in ("kda", "kda_gate", "layer", "public")])
def test_oracle_equals_the_reference_cpu_code(name):
    c = CASES[name]
    ref = _load(name)
    got = _run(c, case_inputs(c))
    if c.get("fwd_only"):
        got = {k: v for k, v in got.items() if k in ("o", "ht")}
    assert set(got) == set(ref), (sorted(got), sorted(ref))
    _compare(name, got, ref, c["dtype"])


@pytest.mark.parametrize("name", [n for n, c in CASES.items() if c["op"] == "kda"])
def test_kda_oracle_equals_the_reference_cpu_code(name):
    """Token recurrence, chunked form, the explicit token-level backward, and the six-stage chunk backward
    (which the reference computes in float32 whatever the inputs are: its exp2 helper casts)."""
    c = CASES[name]
    ref = _load(name)
    x = case_inputs(c)
    scale = c["K"] ** -0.5
    fin = c.get("state") is not False
    o, ht = K.naive_recurrent_kda(x["q"], x["k"], x["v"], x["g"], x["beta"], scale, x["h0"], fin)
    oc, htc = K.naive_chunk_kda(x["q"], x["k"], x["v"], x["g"], x["beta"], scale, x["h0"], fin, chunk_size=c["C"])
    of, htf = K.fused_recurrent_kda(x["q"], x["k"], x["v"], x["g"], x["beta"], scale, x["h0"], fin)
    dq, dk, dv, dg, db, dh0 = K.fused_recurrent_kda_bwd(x["q"], x["k"], x["v"], x["g"], x["beta"], x["do"], scale,
                                                        x["h0"], x["dht"])
    got = dict(o=o, ht=ht, o_chunk=oc, ht_chunk=htc, o_fused=of, ht_fused=htf, dq=dq, dk=dk, dv=dv, dg=dg, dbeta=db,
               dh0=dh0)
    _compare(name, got, ref, c["dtype"])
    # the staged chunk backward on the chunk matrices of the oracle's chunk forward
    g2 = K.kda_gate_chunk_cumsum(x["g"], c["C"])
    Aqk, Akk = K.kda_intra_chunk_fwd(x["q"], x["k"], g2, x["beta"], scale, c["C"])
    st = K.chunk_kda_bwd(x["q"], x["k"], x["v"], x["beta"], Aqk, Akk, scale, x["h0"], x["do"], x["dht"], g=g2,
                         chunk_size=c["C"])
    names = ("st_dq", "st_dk", "st_dv", "st_dbeta", "st_dg", "st_dh0")
    for n, a in zip(names, st):
        if n not in ref:
            continue
        r = ref[n]
        if r is None:
            assert a is None, (name, n)
            continue
        err = (a.double() - r.double()).abs().max().item()
        top = r.double().abs().max().item()
        assert err <= 2e-5 * top, (name, n, err, top)
    # the forward stages behind it (WY vectors, delta-rule state scan)
    if "fw_w" in ref:
        w, u, qg, kg = K.recompute_w_u_fwd(x["k"], x["v"], x["beta"], Akk, q=x["q"], gk=g2)
        h, v_new, ht_scan = K.chunk_gated_delta_rule_fwd_h(kg, w, u, gk=g2, initial_state=x["h0"],
                                                          output_final_state=fin, chunk_size=c["C"])
        _compare(name, dict(fw_w=w, fw_u=u, fw_qg=qg, fw_kg=kg, fw_h=h, fw_v_new=v_new, fw_ht=ht_scan),
                 {k: v for k, v in ref.items() if k.startswith("fw_")}, c["dtype"] if c["dtype"] != "float64" else "float32")
    # and the stored matrices (what the generator fed the reference's staged backward) are these
    if "Aqk" in ref:
        assert torch.equal(Aqk, ref["Aqk"]) and torch.equal(Akk, ref["Akk"]) and torch.equal(g2, ref["g2"])


@pytest.mark.parametrize("name", [n for n, c in CASES.items() if c["op"] == "kda_gate"])
def test_kda_gate_oracle_equals_the_reference_cpu_code(name):
    """-exp(A_log) softplus(g + dt_bias), its lower-bounded form, and gate -> chunk cumsum -> log2 scaling."""
    c = CASES[name]
    ref = _load(name)
    x = gate_inputs(c)
    biased = A.kda_gate_fwd(x["g"], x["A_log"], x["dt_bias"])
    got = dict(plain=A.kda_gate_fwd(x["g"], x["A_log"]), biased=biased,
               bounded=A.kda_gate_fwd(x["g"], x["A_log"], x["dt_bias"], lower_bound=-5.0),
               cumsum_log2=chunk_local_cumsum(biased, c["C"]) * 1.4426950408889634)
    assert set(got) == set(ref)
    _compare(name, got, ref, "float32")      # the gate is computed and returned in float32 for every input dtype


def build_layer(c, ref):
    """This package's layer with the parameters the reference's layer was run with."""
    from tops_b200.layers import GatedLinearAttention
    layer = GatedLinearAttention(hidden_size=c["hidden"], num_heads=c["heads"], **c["kw"])
    missing = layer.load_state_dict(ref["weights"], strict=True)
    assert not missing.missing_keys and not missing.unexpected_keys
    return layer


@pytest.mark.parametrize("name", [n for n, c in CASES.items() if c["op"] == "layer"])
def test_layer_arithmetic_equals_the_reference_layer(name):
    """The reference's `GatedLinearAttention` source (projections, short convolutions, grouped heads, gate law,
    feature map, norm + output gate in both forms) against the same parameters pushed through this package's layer
    wiring with the oracle's pieces: pins the oracle's gate / norm and the layer's wiring.  No kernel runs."""
    c = CASES[name]
    ref = _load(name)
    layer = build_layer(c, ref)
    x = layer_inputs(c)
    mode = "fused_recurrent" if c["T"] <= 64 else c["kw"]["mode"]
    with torch.no_grad():
        from tests.layer_oracle import layer_on_cpu
        y = layer_on_cpu(layer, x, mode)
    _compare(name, dict(y=y), dict(y=ref["y"]), "float32")


def public_on_oracle(x):
    """The oracle's counterparts of the pure-jax entry points of the accelerator-side package."""
    Kd = x["q"].shape[-1]
    out = {}
    out["kda_o"], out["kda_ht"] = K.fused_recurrent_kda(x["q"], x["kn"], x["v"], x["g"], x["beta"], 0.3, x["h0"], True)
    out["gla_o"], out["gla_ht"] = G.fused_recurrent_gla(x["q"], x["k"], x["v"], gk=x["g"], scale=0.3,
                                                        initial_state=x["h0"], output_final_state=True)
    out["sg_o"], out["sg_ht"] = S.naive_recurrent_simple_gla(x["q"], x["k"], x["v"], x["gs"], x["gamma"], 0.3, x["h0"],
                                                             True)
    gk = x["gs"][..., None].expand(*x["gs"].shape, Kd).contiguous()
    out["sg_rev_o"], out["sg_rev_ht"] = G.fused_recurrent_gla(x["q"], x["k"], x["v"], gk=gk, scale=0.3,
                                                              initial_state=x["h0"], output_final_state=True,
                                                              reverse=True)
    return out


def compare_public(name, got, ref, dtype):
    """Values only: these reference functions carry no casts of their own, so their output dtypes follow
    jax's promotion of whatever was passed in.  fp32: float32 rounding; bf16: the half-precision bar (the
    reference multiplies k and v in bf16 there, the oracle and the kernels in fp32)."""
    for key, r in ref.items():
        a, b = got[key].double().cpu(), r.double()
        if dtype == "float32":
            assert (a - b).abs().max().item() <= 2e-5 * b.abs().max().item(), (name, key)
        else:
            assert ((a - b).norm() / b.norm()).item() <= 2e-2, (name, key, ((a - b).norm() / b.norm()).item())


@pytest.mark.parametrize("name", [n for n, c in CASES.items() if c["op"] == "public"])
def test_oracle_equals_the_public_pure_jax_entry_points(name):
    c = CASES[name]
    compare_public(name, public_on_oracle(public_inputs(c)), _load(name), c["dtype"])
