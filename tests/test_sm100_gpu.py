"""The tcgen05 / TMA kernels (bf16, K = V = 128, chunk 64) forced through the
C ABI with impl = SM100, against the CPU oracle and against the generic
kernels; the device error word must stay clear."""
import pytest
import torch

from oracle import gla as O
from tests.util import assert_close, rel_l2, to_cuda

pytestmark = pytest.mark.gpu

SHAPES = [
    # B, T, H, h0
    (1, 64, 1, False),
    (1, 128, 2, True),
    (2, 512, 3, True),
    (1, 1024, 2, False),
    (3, 192, 16, True),      # 48 (batch, head) pairs: the fused forward
    (4, 128, 13, False),
    (4, 64, 12, True),       # fused forward, a single chunk
    (1, 2048, 3, True),      # 3 pairs x 8 time segments of 4 chunks
    (2, 1536, 37, False),    # 74 pairs: 2 segments, fused forward over segments
]


def _run(x, B, T, H, impl, h0):
    from tops_b200 import _lib as L
    from tops_b200.ops._chunk import chunk_bwd_call, chunk_fwd_call
    scale = 128 ** -0.5
    o, ht, _, _, _ = chunk_fwd_call(x["q"], x["k"], x["v"], x["g"], L.GATE_PER_CHANNEL, scale, x.get("h0"), True, 64,
                                    impl=impl)
    dq, dk, dv, dg, dh0 = chunk_bwd_call(x["q"], x["k"], x["v"], x["g"], L.GATE_PER_CHANNEL, scale, x.get("h0"),
                                         x["do"], x["dht"], 64, torch.float32, True, h0, impl=impl)
    return dict(o=o, ht=ht, dq=dq, dk=dk, dv=dv, dg=dg, dh0=dh0)


@pytest.mark.parametrize("B,T,H,h0", SHAPES)
def test_sm100_matches_oracle_and_generic(B, T, H, h0):
    from tops_b200 import _lib as L
    from tops_b200.synth import make_inputs
    x = make_inputs(31, B, T, H, 128, 128, dtype=torch.bfloat16, with_h0=h0, with_grads=True)
    scale = 128 ** -0.5
    o_ref, ht_ref = O.chunk_gla(x["q"], x["k"], x["v"], x["g"], scale, x.get("h0"), True, chunk_size=64)
    ref = O.chunk_gla_bwd(x["q"], x["k"], x["v"], x["g"], None, scale, x.get("h0"), None, None, x["do"], x["dht"],
                          chunk_size=64)
    want = dict(o=o_ref, ht=ht_ref, dq=ref[0], dk=ref[1], dv=ref[2], dg=ref[3], dh0=ref[4])
    c = to_cuda(x)
    n0 = L.launch_count()
    fast = _run(c, B, T, H, L.IMPL_SM100, h0)
    torch.cuda.synchronize()
    # fwd: scan + output, or one fused pass from 48 blocks on; bwd: two scans + chunk kernel; with few
    # (batch, head) pairs and at least 8 chunks every scan is preceded by a summary scan and a join kernel
    segmented = 2 * B * H <= 148 and T // 64 >= 8
    assert L.launch_count() - n0 == (4 if B * H >= 48 else 5) + (6 if segmented else 0)
    assert L.device_error() == 0
    slow = _run(c, B, T, H, L.IMPL_GENERIC, h0)
    report = {}
    for name, r in want.items():
        if r is None:
            assert fast[name] is None
            continue
        report[name] = (rel_l2(fast[name], r), rel_l2(slow[name], r))
    print(report)
    for name, r in want.items():
        if r is not None:
            assert_close(name, fast[name], r, torch.bfloat16)


def test_sm100_is_the_default_for_its_shape():
    from tops_b200 import _lib as L
    from tops_b200.ops.gla import chunk_gla
    from tops_b200.synth import make_inputs
    host = make_inputs(32, 1, 128, 1, 128, 128, dtype=torch.bfloat16)
    x = to_cuda(host)
    L.lib.tops_b200_profile_enable(1)
    # the reference's default chunk length (16): the op's results do not depend on it beyond rounding,
    # so the tensor-core kernels serve it with their own chunk of 64
    o, _ = chunk_gla(x["q"], x["k"], x["v"], x["g"])
    L.lib.tops_b200_profile_enable(0)
    o_ref, _ = O.chunk_gla(host["q"], host["k"], host["v"], host["g"], chunk_size=16)
    assert_close("o", o.cpu(), o_ref, torch.bfloat16)
    import ctypes
    buf = ctypes.create_string_buffer(4096)
    L.lib.tops_b200_profile_read(buf, len(buf))
    labels = [ln.split()[0] for ln in buf.value.decode().splitlines()]
    assert sorted(labels) == ["sm100_fwd_h", "sm100_fwd_o"], labels


def test_sm100_rejects_what_it_cannot_take():
    from tops_b200 import _lib as L
    from tops_b200.ops._chunk import chunk_fwd_call
    from tops_b200.synth import make_inputs
    x = to_cuda(make_inputs(33, 1, 100, 1, 128, 128, dtype=torch.bfloat16))      # T not a multiple of 64
    with pytest.raises(L.TopsError):
        chunk_fwd_call(x["q"], x["k"], x["v"], x["g"], L.GATE_PER_CHANNEL, 0.1, None, False, 64, impl=L.IMPL_SM100)


def test_sm100_gradients_in_primal_dtypes():
    """dq, dk, dg written in bf16 by the kernel (what the reference's accelerator kernel does,
    tops/ops/gla/chunk.py:1551-1554) are the fp32 results rounded once."""
    from tops_b200 import _lib as L
    from tops_b200.ops._chunk import chunk_bwd_call
    from tops_b200.synth import make_inputs
    x = to_cuda(make_inputs(34, 2, 256, 3, 128, 128, dtype=torch.bfloat16, with_h0=True, with_grads=True))
    args = (x["q"], x["k"], x["v"], x["g"], L.GATE_PER_CHANNEL, 128 ** -0.5, x["h0"], x["do"], x["dht"], 64,
            torch.float32, True, True)
    wide = chunk_bwd_call(*args)
    narrow = chunk_bwd_call(*args, primal_dtypes=True)
    torch.cuda.synchronize()
    assert L.device_error() == 0
    for i in (0, 1, 3):      # dq, dk, dg
        assert narrow[i].dtype == torch.bfloat16 and wide[i].dtype == torch.float32
        assert torch.equal(narrow[i], wide[i].to(torch.bfloat16))
    assert torch.equal(narrow[2], wide[2]) and torch.equal(narrow[4], wide[4])
    # a kernel family without the narrow outputs returns the same dtypes through a cast
    slow = chunk_bwd_call(*args, impl=L.IMPL_GENERIC, primal_dtypes=True)
    assert slow[0].dtype == torch.bfloat16 and slow[3].dtype == torch.bfloat16


def test_device_error_word_raises_and_clears():
    """Host-side injection: a non-zero device error word (what a kernel leaves behind when a bounded
    wait gives up) turns into TopsError at the next check, and the check clears it."""
    from tops_b200 import _lib as L
    assert L.device_error() == 0
    L.check(L.lib.tops_b200_device_error_set(7), "device_error_set")
    assert L.device_error() == 7
    with pytest.raises(L.TopsError):
        L.raise_on_device_error("test")
    assert L.device_error() == 0
    L.raise_on_device_error("test")   # clean word: no exception


def test_bounded_wait_runs_out_and_the_kernel_returns_by_itself():
    """A tile load that is never issued: the state scan's wait for it gives up after its limit, the kernel
    leaves through its error path (every thread of the block takes the same exit at the same barrier, tensor
    memory is freed), the error word and a NaN in the final state report it, and the next call is correct."""
    from tops_b200 import _lib as L
    from tops_b200.ops._chunk import chunk_fwd_call
    from tops_b200.synth import make_inputs
    B, T, H = 1, 256, 1          # one block, four chunks: the scan + chunk-output form of the forward
    x = to_cuda(make_inputs(31, B, T, H, 128, 128, dtype=torch.bfloat16, with_h0=True))
    scale = 128 ** -0.5
    assert L.device_error() == 0
    L.check(L.lib.tops_b200_test_skip_load(3), "test_skip_load")
    o, ht, _, _, _ = chunk_fwd_call(x["q"], x["k"], x["v"], x["g"], L.GATE_PER_CHANNEL, scale, x["h0"], True, 64,
                                    impl=L.IMPL_SM100)
    torch.cuda.synchronize()
    assert L.device_error() == 1
    assert torch.isnan(ht).any()
    with pytest.raises(L.TopsError):
        L.raise_on_device_error("test")
    assert L.device_error() == 0
    o2, ht2, _, _, _ = chunk_fwd_call(x["q"], x["k"], x["v"], x["g"], L.GATE_PER_CHANNEL, scale, x["h0"], True, 64,
                                      impl=L.IMPL_SM100)
    torch.cuda.synchronize()
    cpu = {k: v.cpu() for k, v in x.items()}
    o_ref, ht_ref = O.chunk_gla(cpu["q"], cpu["k"], cpu["v"], cpu["g"], scale, cpu["h0"], True, chunk_size=64)
    assert_close("o", o2.cpu(), o_ref, torch.bfloat16)
    assert_close("ht", ht2.cpu(), ht_ref, torch.bfloat16)
    assert L.device_error() == 0


@pytest.mark.parametrize("g_scale", [0.8, 1.0])
def test_sm100_large_gates_stay_finite(g_scale):
    """Per-step gates uniform in (-g_scale, 0) (the gate law of the reference's
    tests/ops/gla/test_exp_overflow_stabilization.py): chunk sums near -64 g_scale, where the raw cumulative gate
    leaves the range of exp().  The mid-point anchored exponents of the tensor-core kernels must stay finite and
    keep the bf16 bar, forward and backward."""
    from tops_b200 import _lib as L
    g = torch.Generator().manual_seed(42)
    B, T, H = 1, 256, 2
    x = {n: torch.randn(B, T, H, 128, generator=g).to(torch.bfloat16) for n in ("q", "k", "v", "do")}
    x["g"] = (-g_scale * torch.rand(B, T, H, 128, generator=g)).to(torch.bfloat16)
    x["h0"] = 0.1 * torch.randn(B, H, 128, 128, generator=g)
    x["dht"] = 0.1 * torch.randn(B, H, 128, 128, generator=g)
    scale = 128 ** -0.5
    o_ref, ht_ref = O.chunk_gla(x["q"], x["k"], x["v"], x["g"], scale, x["h0"], True, chunk_size=64)
    ref = O.chunk_gla_bwd(x["q"], x["k"], x["v"], x["g"], None, scale, x["h0"], None, None, x["do"], x["dht"],
                          chunk_size=64)
    got = _run(to_cuda(x), B, T, H, L.IMPL_SM100, True)
    torch.cuda.synchronize()
    assert L.device_error() == 0
    want = dict(o=o_ref, ht=ht_ref, dq=ref[0], dk=ref[1], dv=ref[2], dg=ref[3], dh0=ref[4])
    for name, r in want.items():
        assert torch.isfinite(got[name]).all(), name
        assert_close(name, got[name], r, torch.bfloat16)
