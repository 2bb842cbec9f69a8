"""Gate activations, q/k L2 normalisation and the gated RMS norm against the oracle (forward) and
against autograd through the oracle (backward)."""
import pytest
import torch

from oracle import aux as O
from tests.util import assert_close

pytestmark = pytest.mark.gpu


def _grads(fn, inputs, dy):
    leaves = [None if t is None else t.clone().requires_grad_(True) for t in inputs]
    y = fn(*leaves)
    used = [t for t in leaves if t is not None]
    g = torch.autograd.grad(y, used, dy.to(y.dtype))
    it = iter(g)
    return y.detach(), [None if t is None else next(it) for t in leaves]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("lower_bound", [None, -5.0])
@pytest.mark.parametrize("bias,base_heads", [(True, 4), (False, 4), (True, 2)])
def test_kda_gate(dtype, lower_bound, bias, base_heads):
    from tops_b200.ops.gate import kda_gate_fwd
    B, T, H, K = 2, 75, 4, 64
    gen = torch.Generator().manual_seed(5)
    g = torch.randn(B, T, H, K, generator=gen).to(dtype)
    A_log = torch.randn(base_heads, generator=gen) * 0.5
    dt_bias = torch.randn(base_heads * K, generator=gen) if bias else None
    dy = torch.randn(B, T, H, K, generator=gen)
    y_ref, ref = _grads(lambda a, b, c: O.kda_gate_fwd(a, b, c, lower_bound), (g, A_log, dt_bias), dy)
    cu = lambda t: None if t is None else t.cuda()
    y, got = _grads(lambda a, b, c: kda_gate_fwd(a, b, c, lower_bound), (cu(g), cu(A_log), cu(dt_bias)), dy.cuda())
    assert y.dtype == torch.float32
    assert_close("y", y.cpu(), y_ref, torch.float32)
    assert_close("dg", got[0].float().cpu(), ref[0].float(), dtype)
    # parameter gradients are sums over thousands of elements: relative bar
    for name, a, r in (("dA_log", got[1], ref[1]), ("dbias", got[2], ref[2])):
        if r is not None:
            assert ((a.cpu() - r).norm() / r.norm()).item() <= (1e-4 if dtype == torch.float32 else 1e-2), name


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("clamp", [None, -0.05])
def test_gla_gate(dtype, clamp):
    from tops_b200.ops.gate import gla_gate
    gen = torch.Generator().manual_seed(6)
    g = (torch.randn(2, 50, 3, 128, generator=gen) * 2).to(dtype)
    dy = torch.randn(2, 50, 3, 128, generator=gen)
    y_ref, ref = _grads(lambda a: O.gla_gate(a, 16.0, clamp), (g,), dy)
    y, got = _grads(lambda a: gla_gate(a, 16.0, clamp), (g.cuda(),), dy.cuda())
    assert y.dtype == dtype
    assert_close("y", y.float().cpu(), y_ref.float(), dtype)
    assert_close("dg", got[0].float().cpu(), ref[0].float(), dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("D", [64, 128, 256])
def test_l2norm(dtype, D):
    from tops_b200.ops.norm import l2norm
    gen = torch.Generator().manual_seed(7)
    x = torch.randn(3, 37, 5, D, generator=gen).to(dtype)
    dy = torch.randn(3, 37, 5, D, generator=gen)
    y_ref, ref = _grads(lambda a: O.l2norm(a), (x,), dy)
    y, got = _grads(lambda a: l2norm(a), (x.cuda(),), dy.cuda())
    assert_close("y", y.float().cpu(), y_ref.float(), dtype)
    assert_close("dx", got[0].float().cpu(), ref[0].float(), dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("D,affine", [(128, True), (512, True), (1024, False)])
def test_rmsnorm_gated(dtype, D, affine):
    from tops_b200.ops.norm import FusedRMSNormGated
    gen = torch.Generator().manual_seed(8)
    x = torch.randn(4, 33, D, generator=gen).to(dtype)
    g = torch.randn(4, 33, D, generator=gen).to(dtype)
    w = (1 + 0.1 * torch.randn(D, generator=gen)) if affine else None
    dy = torch.randn(4, 33, D, generator=gen)
    y_ref, ref = _grads(lambda a, b, c: O.rmsnorm_gated(a, b, c), (x, g, w), dy)
    mod = FusedRMSNormGated(D, elementwise_affine=affine, device="cuda")
    if affine:
        with torch.no_grad():
            mod.weight.copy_(w.cuda())
    xc, gc = x.cuda().requires_grad_(True), g.cuda().requires_grad_(True)
    y = mod(xc, gc)
    leaves = [xc, gc] + ([mod.weight] if affine else [])
    got = torch.autograd.grad(y, leaves, dy.cuda().to(dtype))
    assert_close("y", y.detach().float().cpu(), y_ref.float(), dtype)
    assert_close("dx", got[0].float().cpu(), ref[0].float(), dtype)
    assert_close("dg", got[1].float().cpu(), ref[1].float(), dtype)
    if affine:
        assert ((got[2].cpu() - ref[2]).norm() / ref[2].norm()).item() <= (1e-4 if dtype == torch.float32 else 1e-2)
