"""Every benchmark configuration at its own size against the CPU oracle, on the
`tops_b200.synth` inputs the benchmark uses (seed = configuration number):

* configuration 2 (chunk_gla fwd+bwd, bf16, B=8, T=4096, H=16, K=V=128): all 128
  (batch, head) pairs, gradients in both dtypes the backward writes;
* configuration 3 (decode, B=128, H=32, K=V=128): one in-place step of the whole
  batch, and 64 chained steps of an 8-sequence slice;
* configuration 4 (simple_gla, B=1, T=65536, H=32, scalar bf16 gate): the kernels
  run all 32 heads, the oracle two of them over all 65536 tokens;
* configuration 5 (KDA, B=4, T=8192, H=32): the kernels run the whole problem, the
  oracle (token recurrence + its explicit backward) two (batch, head) pairs over
  all 8192 tokens.

Bar: relative L2 <= 2e-2 on o, the final state and every gradient (bf16 inputs).
"""
import pytest
import torch

from tests.util import assert_close, to_cuda

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


def _threads():
    import os
    try:
        torch.set_num_threads(len(os.sched_getaffinity(0)))
    except Exception:
        pass


def test_config2_chunk_gla_all_pairs_both_gradient_dtypes():
    from oracle import gla as O
    from tops_b200 import _lib as L
    from tops_b200.ops.gla import chunk_gla, chunk_gla_bwd
    from tops_b200.synth import make_inputs
    _threads()
    B, T, H, K, V, C = 8, 4096, 16, 128, 128, 64
    scale = K ** -0.5
    host = make_inputs(2, B, T, H, K, V, dtype=BF16, with_h0=True, with_grads=True)
    x = to_cuda(host)
    # the differentiable op: gradients in the dtypes of their primals
    leaves = [x[n].requires_grad_(True) for n in ("q", "k", "v", "g", "h0")]
    o, ht = chunk_gla(x["q"], x["k"], x["v"], x["g"], scale=scale, initial_state=x["h0"], output_final_state=True,
                      chunk_size=C)
    primal = torch.autograd.grad((o, ht), leaves, (x["do"], x["dht"]))
    # the explicit backward: dq, dk, dg in fp32 like the reference's CPU orchestrator
    with torch.no_grad():
        fp32 = chunk_gla_bwd(x["q"], x["k"], x["v"], x["g"], None, scale, x["h0"], None, None, x["do"], x["dht"],
                             chunk_size=C)
    torch.cuda.synchronize()
    assert L.device_error() == 0
    assert primal[0].dtype == BF16 and primal[3].dtype == BF16 and fp32[0].dtype == torch.float32
    o_ref, ht_ref = O.chunk_gla(host["q"], host["k"], host["v"], host["g"], scale, host["h0"], True, chunk_size=C)
    ref = O.chunk_gla_bwd(host["q"], host["k"], host["v"], host["g"], None, scale, host["h0"], None, None, host["do"],
                          host["dht"], chunk_size=C)
    assert_close("o", o.detach().cpu(), o_ref, BF16)
    assert_close("ht", ht.detach().cpu(), ht_ref, BF16)
    for name, a, b, r in zip(("dq", "dk", "dv", "dg", "dh0"), primal, fp32, ref):
        assert_close(name + " (primal dtype)", a.float().cpu(), r.float(), BF16)
        assert_close(name + " (fp32)", b.float().cpu(), r.float(), BF16)
    # every pair on its own as well: no (batch, head) hides behind the others in the norm
    for name, a, r in (("o", o.detach(), o_ref), ("dq", primal[0], ref[0]), ("dk", primal[1], ref[1]),
                       ("dv", primal[2], ref[2]), ("dg", primal[3], ref[3])):
        d = (a.float().cpu() - r.float()).pow(2).sum(dim=(1, 3)).sqrt() / r.float().pow(2).sum(dim=(1, 3)).sqrt()
        assert d.max().item() <= 2e-2, (name, d.max().item())


def test_config3_decode_whole_batch_and_chained_steps():
    from oracle import gla as O
    from tops_b200.ops.gla import fused_recurrent_gla_decode_
    from tops_b200.synth import make_inputs
    _threads()
    B, H, K, V = 128, 32, 128, 128
    host = make_inputs(3, B, 1, H, K, V, dtype=BF16, with_h0=True)
    x = to_cuda(host)
    state = x["h0"].clone()
    o = fused_recurrent_gla_decode_(x["q"], x["k"], x["v"], x["g"], state)
    torch.cuda.synchronize()
    o_ref, ht_ref = O.fused_recurrent_gla(host["q"], host["k"], host["v"], gk=host["g"], initial_state=host["h0"],
                                          output_final_state=True)
    assert_close("o", o.cpu(), o_ref, BF16)
    assert (state.cpu() - ht_ref).abs().max().item() <= 1e-5 * max(1.0, ht_ref.abs().max().item())
    # 64 chained in-place steps of an 8-sequence slice == one 64-token pass of the oracle
    Bs, steps = 8, 64
    seq = make_inputs(33, Bs, steps, H, K, V, dtype=BF16, with_h0=True)
    xs = to_cuda(seq)
    st = xs["h0"].clone()
    outs = []
    for t in range(steps):
        outs.append(fused_recurrent_gla_decode_(xs["q"][:, t:t + 1].contiguous(), xs["k"][:, t:t + 1].contiguous(),
                                                xs["v"][:, t:t + 1].contiguous(), xs["g"][:, t:t + 1].contiguous(), st))
    torch.cuda.synchronize()
    o_ref, ht_ref = O.fused_recurrent_gla(seq["q"], seq["k"], seq["v"], gk=seq["g"], initial_state=seq["h0"],
                                          output_final_state=True)
    assert_close("o (64 steps)", torch.cat(outs, 1).cpu(), o_ref, BF16)
    assert_close("state (64 steps)", st.cpu(), ht_ref, BF16)


def test_config4_simple_gla_long_sequence():
    from oracle import simple_gla as O
    from tops_b200 import _lib as L
    from tops_b200.ops.simple_gla import chunk_simple_gla
    from tops_b200.synth import make_inputs
    _threads()
    B, T, H, K, V, C = 1, 65536, 32, 128, 128, 64
    scale = K ** -0.5
    host = make_inputs(4, B, T, H, K, V, dtype=BF16, gate="scalar", with_h0=True, with_grads=True)
    x = to_cuda(host)
    leaves = [x[n].requires_grad_(True) for n in ("q", "k", "v", "g", "h0")]
    o, ht = chunk_simple_gla(x["q"], x["k"], x["v"], g=x["g"], scale=scale, initial_state=x["h0"],
                             output_final_state=True, chunk_size=C)
    dq, dk, dv, dg, dh0 = torch.autograd.grad((o, ht), leaves, (x["do"], x["dht"]))
    torch.cuda.synchronize()
    assert L.device_error() == 0
    heads = [3, 30]      # the oracle walks 1024 chunks in a Python loop: two heads of the 32
    sl = {n: host[n][:, :, heads].contiguous() for n in ("q", "k", "v", "g", "do")}
    h0, dht = host["h0"][:, heads].contiguous(), host["dht"][:, heads].contiguous()
    o_ref, ht_ref = O.chunk_simple_gla(sl["q"], sl["k"], sl["v"], g=sl["g"], scale=scale, initial_state=h0,
                                       output_final_state=True, chunk_size=C)
    ref = O.chunk_simple_gla_bwd(sl["q"], sl["k"], sl["v"], sl["g"], None, h0, sl["do"], dht, scale, chunk_size=C)
    assert_close("o", o.detach()[:, :, heads].cpu(), o_ref, BF16)
    assert_close("ht", ht.detach()[:, heads].cpu(), ht_ref, BF16)
    for name, a, r in zip(("dq", "dk", "dv"), (dq, dk, dv), ref[:3]):
        assert_close(name, a[:, :, heads].float().cpu(), r.float(), BF16)
    assert_close("dg", dg[:, :, heads].float().cpu(), ref[3].float(), BF16)
    assert_close("dh0", dh0[:, heads].cpu(), ref[4], BF16)


def test_config5_kda_long_sequence():
    from oracle import kda as O
    from tops_b200 import _lib as L
    from tops_b200.ops.kda import chunk_kda
    from tops_b200.synth import make_inputs
    _threads()
    B, T, H, K, V, C = 4, 8192, 32, 128, 128, 64
    scale = K ** -0.5
    host = make_inputs(5, B, T, H, K, V, dtype=BF16, with_h0=True, with_grads=True, with_beta=True, l2norm_qk=True)
    x = to_cuda(host)
    leaves = [x[n].requires_grad_(True) for n in ("q", "k", "v", "g", "beta", "h0")]
    o, ht = chunk_kda(x["q"], x["k"], x["v"], x["g"], x["beta"], scale=scale, initial_state=x["h0"],
                      output_final_state=True, chunk_size=C)
    grads = torch.autograd.grad((o, ht), leaves, (x["do"], x["dht"]))
    torch.cuda.synchronize()
    assert L.device_error() == 0
    for b, h in ((0, 5), (3, 28)):
        sl = {n: host[n][b:b + 1, :, h:h + 1].contiguous() for n in ("q", "k", "v", "g", "beta", "do")}
        h0, dht = host["h0"][b:b + 1, h:h + 1].contiguous(), host["dht"][b:b + 1, h:h + 1].contiguous()
        o_ref, ht_ref = O.naive_recurrent_kda(sl["q"], sl["k"], sl["v"], sl["g"], sl["beta"], scale, h0, True)
        ref = O.fused_recurrent_kda_bwd(sl["q"], sl["k"], sl["v"], sl["g"], sl["beta"], sl["do"], scale, h0, dht)
        assert_close(f"o[{b},{h}]", o.detach()[b:b + 1, :, h:h + 1].float().cpu(), o_ref.float(), BF16)
        assert_close(f"ht[{b},{h}]", ht.detach()[b:b + 1, h:h + 1].cpu(), ht_ref.float(), BF16)
        for name, a, r in zip(("dq", "dk", "dv", "dg"), grads[:4], ref[:4]):
            assert_close(f"{name}[{b},{h}]", a[b:b + 1, :, h:h + 1].float().cpu(), r.float(), BF16)
        assert_close(f"dbeta[{b},{h}]", grads[4][b:b + 1, :, h:h + 1].float().cpu(), ref[4].float(), BF16)
        assert_close(f"dh0[{b},{h}]", grads[5][b:b + 1, h:h + 1].cpu(), ref[5].float(), BF16)
