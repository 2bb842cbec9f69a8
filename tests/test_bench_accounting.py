"""The byte and FLOP counts `bench.py` divides by: every API tensor once, no scratch
(the per-token-head figures the benchmark's roofline fractions rest on)."""
import importlib.util
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_config2_kernel_bytes_count_api_tensors_only():
    b = _bench()
    w = dict(b.GLA_TRAIN)
    tok = w["B"] * w["T"] * w["H"]
    assert tok == 524288 and w["K"] == w["V"] == 128 and w["C"] == 64
    states = 2 * w["B"] * w["H"] * 128 * 128 * 4
    # chunk backward: q, k, g, v, do in; dq, dk, dg, dv out, all bf16: 9 x 256 B per token-head
    assert b.kernel_bytes("sm100_bwd_main", w, 2) == tok * 2304
    # with fp32 dq, dk, dg: 6 x 256 + 3 x 512
    assert b.kernel_bytes("sm100_bwd_main", w, 4) == tok * 3072
    # fused forward: q, k, g, v in, o out, h0 in, ht out
    assert b.kernel_bytes("sm100_fwd_fused", w) == tok * 1280 + states
    # reverse scan: q, g, do in, dht in, dh0 out
    assert b.kernel_bytes("sm100_bwd_dh", w) == tok * 768 + states
    # scratch is reported apart: h' (and dh') as bf16 [B,NT,H,K,V] = 512 B per token-head each
    assert b.scratch_bytes("sm100_bwd_main", w) == tok * 1024
    assert b.scratch_bytes("sm100_fwd_fused", w) == tok * 512
    # the step: the three launches together are the 3648 B per token-head of the whole op
    step = sum(b.kernel_bytes(k, w, 2) for k in ("sm100_fwd_fused", "sm100_bwd_dh", "sm100_bwd_main"))
    # (q, g, do are read by two of the backward's launches: the op reads them once)
    assert step - tok * 768 == tok * 3584 + 2 * states
    assert tok * 3584 + 2 * states == tok * 3648


def test_secondary_workload_bytes():
    b = _bench()
    # simple_gla: q, k, v (768) + g (2) + o (256); q, k, v, do (1024) + g (2) + dq, dk, dv (768) + dg fp32 (4)
    n = b.simple_gla_bytes(1, 65536, 32, 128, 128)
    assert n == 65536 * 32 * 2824 + 4 * 32 * 128 * 128 * 4
    # KDA at the dtypes of the differentiable op (bf16 gradients)
    n = b.kda_bytes(4, 8192, 32, 128, 128)
    assert n == 4 * 8192 * 32 * 3590 + 4 * 4 * 32 * 128 * 128 * 4
