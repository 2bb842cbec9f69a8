"""`GatedLinearAttention` (the reference's one in-tree caller of the GLA ops, tops/layers/gla.py) on the
kernels of this package against the same layer computed on the CPU from the oracle pieces."""
import copy

import pytest
import torch

from tests.layer_oracle import layer_on_cpu as _reference

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kw,T", [
    (dict(mode="chunk"), 96),
    (dict(mode="fused_chunk", num_kv_heads=2, use_short_conv=True), 80),
    (dict(mode="chunk", fuse_norm=False, gate_fn="sigmoid", clamp_min=-0.04), 72),
    (dict(mode="chunk", use_output_gate=False), 40),          # <= 64 tokens: the recurrent kernel
])
def test_layer_matches_cpu_reference(kw, T):
    from tops_b200.layers import GatedLinearAttention
    torch.manual_seed(0)
    layer = GatedLinearAttention(hidden_size=256, num_heads=4, **kw)
    x = torch.randn(2, T, 256)
    ref_layer = copy.deepcopy(layer)
    xr = x.clone().requires_grad_(True)
    y_ref = _reference(ref_layer, xr, "fused_recurrent" if T <= 64 else kw["mode"])
    dy = torch.randn_like(y_ref)
    y_ref.backward(dy)
    layer = layer.cuda()
    xc = x.cuda().requires_grad_(True)
    y, _, _ = layer(xc)
    y.backward(dy.cuda())
    bar = 2e-4 * max(1.0, y_ref.abs().max().item())
    assert (y.detach().cpu() - y_ref.detach()).abs().max().item() <= bar
    rel = lambda a, b: ((a.cpu() - b).norm() / b.norm()).item()
    assert rel(xc.grad, xr.grad) <= 1e-3
    for (n, p), (_, pr) in zip(layer.named_parameters(), ref_layer.named_parameters()):
        assert p.grad is not None and rel(p.grad, pr.grad) <= 2e-3, n


def test_layer_cache_prefill_then_decode_equals_one_pass():
    from tops_b200.layers import Cache, GatedLinearAttention
    torch.manual_seed(1)
    layer = GatedLinearAttention(hidden_size=256, num_heads=2, use_short_conv=True, layer_idx=0).cuda().to(torch.bfloat16)
    x = torch.randn(2, 128 + 8, 256, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        full, _, _ = layer(x)
        cache = Cache()
        y0, _, cache = layer(x[:, :128], past_key_values=cache, use_cache=True)
        outs = [y0]
        for t in range(128, 136):
            yt, _, cache = layer(x[:, t:t + 1], past_key_values=cache, use_cache=True)
            outs.append(yt)
    got = torch.cat(outs, 1)
    assert ((got.float() - full.float()).norm() / full.float().norm()).item() <= 2e-2
