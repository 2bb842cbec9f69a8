"""Generate the frozen fixtures in this directory.

    python -m tests.golden.make_golden

These fixtures are outputs of the CPU oracle (`oracle/`, a restatement of
`tops/cpu/ops/**`) on seeded inputs from `tops_b200.synth`.  They freeze the
oracle: a later edit that changes its results fails
tests/test_oracle_gla.py::test_golden_vectors_reproduce, and the GPU parity
tests compare the kernels with the same files.  Outputs of the reference's
own code are the `ref_*.pt` files beside them (make_reference_golden.py).
"""
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
for p in (ROOT, os.path.join(ROOT, "pallas-kernel_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

CASES = {
    "gla_fp32": dict(op="gla", seed=101, B=2, T=80, H=2, K=32, V=48, C=32, dtype="float32", h0=True),
    "gla_bf16": dict(op="gla", seed=102, B=1, T=128, H=2, K=64, V=64, C=64, dtype="bfloat16", h0=True),
    "simple_gla_fp32": dict(op="simple_gla", seed=103, B=2, T=50, H=2, K=32, V=32, C=16, dtype="float32", h0=True),
    "recurrent_fp32": dict(op="recurrent", seed=104, B=2, T=24, H=2, K=32, V=16, dtype="float32", h0=True),
    "kda_fp32": dict(op="kda", seed=105, B=1, T=40, H=2, K=32, V=32, dtype="float32", h0=True),
}


def case_inputs(c):
    from tops_b200.synth import make_inputs
    dtype = getattr(torch, c["dtype"])
    gate = "scalar" if c["op"] == "simple_gla" else "per_channel"
    return make_inputs(c["seed"], c["B"], c["T"], c["H"], c["K"], c["V"], dtype=dtype, gate=gate,
                       with_h0=c["h0"], with_grads=True, with_beta=c["op"] == "kda", l2norm_qk=c["op"] == "kda",
                       gate_dtype=torch.float32 if gate == "scalar" else None)


def run_case(c):
    from oracle import gla as G
    from oracle import simple_gla as S
    x = case_inputs(c)
    scale = c["K"] ** -0.5
    if c["op"] == "gla":
        o, ht = G.chunk_gla(x["q"], x["k"], x["v"], x["g"], scale, x.get("h0"), True, chunk_size=c["C"])
        dq, dk, dv, dg, dh0 = G.chunk_gla_bwd(x["q"], x["k"], x["v"], x["g"], None, scale, x.get("h0"), None, None,
                                              x["do"], x["dht"], chunk_size=c["C"])
        return dict(o=o, ht=ht, dq=dq, dk=dk, dv=dv, dg=dg, dh0=dh0)
    if c["op"] == "simple_gla":
        o, ht = S.chunk_simple_gla(x["q"], x["k"], x["v"], x["g"], None, scale, x.get("h0"), True, chunk_size=c["C"])
        dq, dk, dv, dg, dh0 = S.chunk_simple_gla_bwd(x["q"], x["k"], x["v"], x["g"], None, x.get("h0"), x["do"],
                                                     x["dht"], scale, chunk_size=c["C"])
        return dict(o=o, ht=ht, dq=dq, dk=dk, dv=dv, dg=dg, dh0=dh0)
    if c["op"] == "recurrent":
        o, ht = G.fused_recurrent_fwd(x["q"], x["k"], x["v"], x["g"], None, scale, x.get("h0"), True)
        dq, dk, dv, dgk, _, dh0 = G.fused_recurrent_bwd(x["q"], x["k"], x["v"], x["g"], None, None, x["do"], x["dht"],
                                                        scale, x.get("h0"))
        return dict(o=o, ht=ht, dq=dq, dk=dk, dv=dv, dgk=dgk, dh0=dh0)
    if c["op"] == "kda":
        from oracle import kda as K
        o, ht = K.naive_recurrent_kda(x["q"], x["k"], x["v"], x["g"], x["beta"], scale, x.get("h0"), True)
        dq, dk, dv, dg, db, dh0 = K.fused_recurrent_kda_bwd(x["q"], x["k"], x["v"], x["g"], x["beta"], x["do"], scale,
                                                            x.get("h0"), x["dht"])
        return dict(o=o, ht=ht, dq=dq, dk=dk, dv=dv, dg=dg, dbeta=db, dh0=dh0)
    raise ValueError(c["op"])


def main():
    for name, c in CASES.items():
        out = {k: v.clone() for k, v in run_case(c).items()}
        torch.save({"case": name, "outputs": out}, os.path.join(HERE, name + ".pt"))
        print(name, {k: tuple(v.shape) for k, v in out.items()})


if __name__ == "__main__":
    main()
