"""Comparison helpers shared by the parity tests."""
import torch

# Acceptance bars for the GPU kernels against the CPU oracle on identical
# seeded inputs: fp32 inputs max-abs <= 1e-4 (scaled by the magnitude of the
# reference when that exceeds 1); bf16 / fp16 inputs relative L2 <= 2e-2.
FP32_MAX_ABS = 1e-4
HALF_REL_L2 = 2e-2


def rel_l2(a, b):
    a, b = a.double().cpu(), b.double().cpu()
    return ((a - b).norm() / b.norm().clamp_min(1e-12)).item()


def max_abs(a, b):
    return (a.double().cpu() - b.double().cpu()).abs().max().item()


def assert_close(name, got, ref, dtype):
    assert got.shape == ref.shape, f"{name}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got.float()).all(), f"{name}: non-finite values"
    if dtype == torch.float32:
        bar = FP32_MAX_ABS * max(1.0, ref.double().abs().max().item())
        err = max_abs(got, ref)
        assert err <= bar, f"{name}: max-abs {err:.3e} > {bar:.3e}"
    else:
        err = rel_l2(got, ref)
        assert err <= HALF_REL_L2, f"{name}: rel-L2 {err:.3e} > {HALF_REL_L2}"
    return err


def to_cuda(d):
    return {k: (v.cuda() if isinstance(v, torch.Tensor) else v) for k, v in d.items()}
