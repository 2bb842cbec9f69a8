"""GPU kernels against the committed golden fixtures (tests/golden/*.pt)."""
import os

import pytest
import torch

from tests.golden.make_golden import CASES, case_inputs
from tests.util import assert_close, to_cuda

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


@pytest.mark.parametrize("name", sorted(CASES))
def test_kernels_match_golden(name):
    from tops_b200.ops import gla, simple_gla
    c = CASES[name]
    ref = torch.load(os.path.join(GOLDEN, name + ".pt"))["outputs"]
    x = to_cuda(case_inputs(c))
    dtype = getattr(torch, c["dtype"])
    scale = c["K"] ** -0.5
    if c["op"] == "gla":
        o, ht = gla.chunk_gla(x["q"], x["k"], x["v"], x["g"], scale=scale, initial_state=x["h0"],
                              output_final_state=True, chunk_size=c["C"])
        dq, dk, dv, dg, dh0 = gla.chunk_gla_bwd(x["q"], x["k"], x["v"], x["g"], None, scale, x["h0"], None, None,
                                                x["do"], x["dht"], chunk_size=c["C"])
        got = dict(o=o, ht=ht, dq=dq, dk=dk, dv=dv, dg=dg, dh0=dh0)
    elif c["op"] == "simple_gla":
        o, ht = simple_gla.chunk_simple_gla(x["q"], x["k"], x["v"], x["g"], None, scale, x["h0"], True,
                                            chunk_size=c["C"])
        dq, dk, dv, dg, dh0 = simple_gla.chunk_simple_gla_bwd(x["q"], x["k"], x["v"], x["g"], None, x["h0"], x["do"],
                                                              x["dht"], scale, chunk_size=c["C"])
        got = dict(o=o, ht=ht, dq=dq, dk=dk, dv=dv, dg=dg, dh0=dh0)
    elif c["op"] == "kda":
        from tops_b200.ops import kda
        o, ht = kda.kda_fwd(x["q"], x["k"], x["v"], x["g"], x["beta"], scale, x["h0"], True)
        dq, dk, dv, dg, db, dh0 = kda.kda_bwd(x["q"], x["k"], x["v"], x["g"], x["beta"], x["do"], scale, x["h0"], x["dht"])
        got = dict(o=o, ht=ht, dq=dq, dk=dk, dv=dv, dg=dg, dbeta=db, dh0=dh0)
    else:
        o, ht = gla.fused_recurrent_fwd(x["q"], x["k"], x["v"], x["g"], None, scale, x["h0"], True)
        dq, dk, dv, dgk, _, dh0 = gla.fused_recurrent_bwd(x["q"], x["k"], x["v"], x["g"], None, None, x["do"],
                                                          x["dht"], scale, x["h0"])
        got = dict(o=o, ht=ht, dq=dq, dk=dk, dv=dv, dgk=dgk, dh0=dh0)
    for key, r in ref.items():
        assert_close(key, got[key], r, dtype)
