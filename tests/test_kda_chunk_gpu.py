"""The chunked KDA kernels on the tensor cores (bf16, K = V = 128, chunk 64) through the C ABI against
the oracle: outputs against the token recurrence, the per-chunk matrices Aqk / Akk^-1 and the
cumulative gate against the staged chunk forward."""
import pytest
import torch

from oracle import kda as O
from tests.util import assert_close, rel_l2, to_cuda

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16

SHAPES = [
    # B, T, H, h0
    (1, 64, 1, False),
    (1, 128, 2, True),
    (2, 256, 3, True),
    (1, 1024, 2, False),
    (2, 192, 16, True),
]


def _inputs(seed, B, T, H, h0=True, gate_norm=16.0):
    from tops_b200.synth import make_inputs
    x = make_inputs(seed, B, T, H, 128, 128, dtype=BF16, gate_norm=gate_norm, with_h0=True, with_grads=True,
                    with_beta=True, l2norm_qk=True)
    if not h0:
        x["h0"] = None
    return x


@pytest.mark.parametrize("B,T,H,h0", SHAPES)
def test_chunk_kda_fwd_matches_oracle(B, T, H, h0):
    from tops_b200 import _lib as L
    from tops_b200.ops.kda import chunk_kda_fwd
    host = _inputs(50 + T, B, T, H, h0)
    x = to_cuda(host)
    scale = 128 ** -0.5
    o, ht, gcs, Aqk, Akk = chunk_kda_fwd(x["q"], x["k"], x["v"], x["g"], x["beta"], scale, x["h0"], True, chunk_size=64)
    torch.cuda.synchronize()
    assert L.device_error() == 0
    o_ref, ht_ref = O.naive_recurrent_kda(host["q"], host["k"], host["v"], host["g"], host["beta"], scale, host["h0"], True)
    assert_close("o", o.float().cpu(), o_ref.float(), BF16)
    assert_close("ht", ht.cpu(), ht_ref, BF16)
    # the staged chunk forward: same matrices, same convention for Akk
    _, _, gcs_ref, Aqk_ref, Akk_ref = O.chunk_kda_fwd(host["q"], host["k"], host["v"], host["g"], host["beta"], scale,
                                                      host["h0"], True, chunk_size=64)
    assert (gcs.cpu() - gcs_ref).abs().max().item() <= 1e-4
    assert_close("Aqk", Aqk.cpu(), Aqk_ref, BF16)
    assert_close("Akk", Akk.cpu(), Akk_ref, BF16)
    A = Akk.reshape(B, T // 64, 64, H, 64)
    i = torch.arange(64, device=A.device)
    assert (A[:, :, i, :, i] == 1).all() and torch.triu(A.permute(0, 1, 3, 2, 4), 1).abs().max().item() == 0


def test_chunk_kda_state_split_and_recurrent_kernel_agree():
    """Two halves chained through the state == one pass; chunked kernels == token-serial kernels."""
    from tops_b200.ops.kda import chunk_kda, fused_recurrent_kda
    host = _inputs(61, 2, 512, 4)
    x = to_cuda(host)
    o, ht = chunk_kda(x["q"], x["k"], x["v"], x["g"], x["beta"], initial_state=x["h0"], output_final_state=True)
    h = 256
    a = {n: x[n][:, :h].contiguous() for n in ("q", "k", "v", "g", "beta")}
    b = {n: x[n][:, h:].contiguous() for n in ("q", "k", "v", "g", "beta")}
    o1, s1 = chunk_kda(a["q"], a["k"], a["v"], a["g"], a["beta"], initial_state=x["h0"], output_final_state=True)
    o2, s2 = chunk_kda(b["q"], b["k"], b["v"], b["g"], b["beta"], initial_state=s1, output_final_state=True)
    assert rel_l2(torch.cat([o1, o2], 1), o) <= 5e-3 and rel_l2(s2, ht) <= 5e-3
    o3, s3 = fused_recurrent_kda(x["q"], x["k"], x["v"], x["g"], x["beta"], initial_state=x["h0"], output_final_state=True)
    assert rel_l2(o3, o) <= 1e-2 and rel_l2(s3, ht) <= 1e-2


def test_chunk_kda_raw_log_sigmoid_gates():
    """Un-normalised log-sigmoid gates (cumulative decay of e^-50 over a chunk): the mid-point anchor keeps
    every exponent finite."""
    from tops_b200.ops.kda import chunk_kda_fwd
    host = _inputs(62, 1, 256, 2, gate_norm=1.0)
    x = to_cuda(host)
    scale = 128 ** -0.5
    o, ht, _, _, _ = chunk_kda_fwd(x["q"], x["k"], x["v"], x["g"], x["beta"], scale, x["h0"], True)
    o_ref, ht_ref = O.naive_recurrent_kda(host["q"], host["k"], host["v"], host["g"], host["beta"], scale, host["h0"], True)
    assert_close("o", o.float().cpu(), o_ref.float(), BF16)
    assert_close("ht", ht.cpu(), ht_ref, BF16)


@pytest.mark.parametrize("B,T,H,h0", SHAPES)
def test_chunk_kda_bwd_matches_oracle(B, T, H, h0):
    """The three backward kernels (reverse scan, per-chunk matrix gradients, chunk outputs) against the
    explicit token-level backward of the oracle, fp32 gradients."""
    from tops_b200 import _lib as L
    from tops_b200.ops.kda import chunk_kda_bwd
    host = _inputs(70 + T, B, T, H, h0)
    x = to_cuda(host)
    scale = 128 ** -0.5
    dq, dk, dv, db, dg, dh0 = chunk_kda_bwd(x["q"], x["k"], x["v"], x["g"], x["beta"], x["do"], scale, x["h0"], x["dht"])
    torch.cuda.synchronize()
    assert L.device_error() == 0
    assert dq.dtype == torch.float32 and dg.dtype == torch.float32 and db.dtype == torch.float32 and dv.dtype == BF16
    ref = O.fused_recurrent_kda_bwd(host["q"].float(), host["k"].float(), host["v"].float(), host["g"].float(),
                                    host["beta"].float(), host["do"].float(), scale, host["h0"], host["dht"])
    for name, a, r in zip(("dq", "dk", "dv", "dg", "dbeta"), (dq, dk, dv, dg, db), ref[:5]):
        assert_close(name, a.float().cpu(), r.float(), BF16)
    if h0:
        assert_close("dh0", dh0.cpu(), ref[5], BF16)
    else:
        assert dh0 is None


def test_chunk_kda_autograd_equals_explicit_backward_and_stage_oracle():
    """Autograd through chunk_kda == the explicit backward (bf16 cotangents vs fp32), and both agree with
    the staged chunk backward of the oracle (dAv, dhu, fused WY, intra, reverse cumsum)."""
    from tops_b200.ops.kda import chunk_kda, chunk_kda_bwd
    B, T, H = 2, 256, 3
    host = _inputs(81, B, T, H)
    x = to_cuda(host)
    scale = 128 ** -0.5
    leaves = [x[n].clone().requires_grad_(True) for n in ("q", "k", "v", "g", "beta", "h0")]
    o, ht = chunk_kda(*leaves[:5], scale=scale, initial_state=leaves[5], output_final_state=True)
    got = torch.autograd.grad((o, ht), leaves, (x["do"], x["dht"]))
    dq, dk, dv, db, dg, dh0 = chunk_kda_bwd(x["q"], x["k"], x["v"], x["g"], x["beta"], x["do"], scale, x["h0"], x["dht"])
    for name, a, b in zip(("dq", "dk", "dv", "dg", "dbeta", "dh0"), got, (dq, dk, dv, dg, db, dh0)):
        assert a.dtype == (torch.float32 if name == "dh0" else BF16)
        assert rel_l2(a, b) <= 1e-2, (name, rel_l2(a, b))
    f = {n: host[n].float() for n in ("q", "k", "v", "g", "beta", "do")}
    ref = O.chunk_kda_with_grads(f["q"], f["k"], f["v"], f["g"], f["beta"], f["do"], scale, host["h0"], host["dht"])
    o_ref, ht_ref, rq, rk, rv, rg, rb, rh0 = ref
    assert_close("o", o.detach().float().cpu(), o_ref, BF16)
    for name, a, r in zip(("dq", "dk", "dv", "dg", "dbeta", "dh0"), (dq, dk, dv, dg, db, dh0), (rq, rk, rv, rg, rb, rh0)):
        assert_close(name, a.float().cpu(), r.float(), BF16)


def test_kda_time_shards_chain_on_one_gpu():
    """The pieces of time-sharded KDA without the collective: two halves of one sequence, each summarised as
    h_out = M h_in + S (M from a forward with v = 0 and initial_state = I) and dh_in = M^T dh_out + D
    (the state-gradient-only form of the backward call), folded by hand, against one pass of the CPU oracle."""
    from oracle import kda as OK
    from tops_b200 import _lib as L
    from tops_b200 import time_shard as TS
    from tops_b200.synth import make_inputs
    B, T, H, K, V, R = 1, 512, 2, 128, 128, 2
    x = make_inputs(72, B, T, H, K, V, dtype=torch.bfloat16, with_h0=True, with_grads=True, with_beta=True,
                    l2norm_qk=True)
    scale = K ** -0.5
    ops = TS.kda_cuda_ops()
    sls = [slice(r * T // R, (r + 1) * T // R) for r in range(R)]
    sh = [{n: (t[:, s] if t.ndim >= 3 and t.shape[1] == T else t).cuda().contiguous() for n, t in x.items()}
          for s in sls]
    Ms = [ops.transition(c["k"], c["g"], c["beta"]) for c in sh]
    Ss = [ops.end_state(c["k"], c["v"], c["g"], c["beta"]) for c in sh]
    h_in = [TS.kda_fold_left(Ms, Ss, sh[0]["h0"], r) for r in range(R)]
    final = TS.kda_fold_left(Ms, Ss, sh[0]["h0"], R)
    fw = [ops.fwd(c["q"], c["k"], c["v"], c["g"], c["beta"], scale, h_in[r]) for r, c in enumerate(sh)]
    Ds = [ops.grad_start(c["q"], c["k"], c["v"], c["g"], c["beta"], scale, h_in[r], c["do"], fw[r][1])
          for r, c in enumerate(sh)]
    dh_out = [TS.kda_fold_right(Ms, Ds, sh[0]["dht"], r) for r in range(R)]
    dh0 = TS.kda_fold_right(Ms, Ds, sh[0]["dht"], -1)
    bw = [ops.bwd(c["q"], c["k"], c["v"], c["g"], c["beta"], scale, h_in[r], c["do"], dh_out[r], fw[r][1])
          for r, c in enumerate(sh)]
    torch.cuda.synchronize()
    assert L.device_error() == 0
    o_ref, ht_ref = OK.naive_recurrent_kda(x["q"], x["k"], x["v"], x["g"], x["beta"], scale, x["h0"], True)
    ref = OK.fused_recurrent_kda_bwd(x["q"], x["k"], x["v"], x["g"], x["beta"], x["do"], scale, x["h0"], x["dht"])
    assert rel_l2(torch.cat([f[0] for f in fw], 1), o_ref) <= 2e-2
    assert rel_l2(final, ht_ref) <= 2e-2
    assert rel_l2(dh0, ref[5]) <= 2e-2
    for i, name in enumerate(("dq", "dk", "dv", "dg", "dbeta")):
        e = rel_l2(torch.cat([b[i] for b in bw], 1), ref[i])
        assert e <= 2e-2, (name, e)


@pytest.mark.parametrize("h0", [False, True])
def test_chunk_kda_bwd_unnormalised_inputs_and_strong_gates(h0):
    """The input law of the reference's backward tests (tests/ops/kda/test_chunk_kda_bwd_tpu.py:33-58): q, k, v,
    do ~ 0.1 N(0,1) without L2 normalisation, per-step gates -0.3 |N(0,1)| (a chunk decays by about e^-15 per
    channel), h0 and dht ~ 0.01 N(0,1).  Forward and every gradient against the token recurrence."""
    from tops_b200 import _lib as L
    from tops_b200.ops.kda import chunk_kda_bwd, chunk_kda_fwd
    B, T, H = 1, 256, 2
    gen = torch.Generator().manual_seed(99)
    host = {n: (0.1 * torch.randn(B, T, H, 128, generator=gen)).to(BF16) for n in ("q", "k", "v", "do")}
    host["g"] = (-0.3 * torch.randn(B, T, H, 128, generator=gen).abs()).to(BF16)
    host["beta"] = torch.sigmoid(torch.randn(B, T, H, generator=gen)).to(BF16)
    host["h0"] = 0.01 * torch.randn(B, H, 128, 128, generator=gen) if h0 else None
    host["dht"] = 0.01 * torch.randn(B, H, 128, 128, generator=gen)
    x = {n: (None if t is None else t.cuda()) for n, t in host.items()}
    scale = 128 ** -0.5
    o, ht, _, _, _ = chunk_kda_fwd(x["q"], x["k"], x["v"], x["g"], x["beta"], scale, x["h0"], True)
    dq, dk, dv, db, dg, dh0 = chunk_kda_bwd(x["q"], x["k"], x["v"], x["g"], x["beta"], x["do"], scale, x["h0"], x["dht"])
    torch.cuda.synchronize()
    assert L.device_error() == 0
    f = {n: host[n].float() for n in ("q", "k", "v", "g", "beta", "do")}
    o_ref, ht_ref = O.naive_recurrent_kda(f["q"], f["k"], f["v"], f["g"], f["beta"], scale, host["h0"], True)
    ref = O.fused_recurrent_kda_bwd(f["q"], f["k"], f["v"], f["g"], f["beta"], f["do"], scale, host["h0"], host["dht"])
    assert_close("o", o.float().cpu(), o_ref, BF16)
    assert_close("ht", ht.cpu(), ht_ref, BF16)
    for name, a, r in zip(("dq", "dk", "dv", "dg", "dbeta"), (dq, dk, dv, dg, db), ref[:5]):
        assert torch.isfinite(a).all(), name
        assert_close(name, a.float().cpu(), r.float(), BF16)
    if h0:
        assert_close("dh0", dh0.cpu(), ref[5], BF16)
