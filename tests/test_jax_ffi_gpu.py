"""`chunk_gla` on jax.Arrays through the XLA FFI handlers (tops_b200/jax_ops.py) against the torch path of
the same kernels.  Skipped where JAX (or the shim library, built only where JAX is) is not installed."""
import pytest

pytestmark = pytest.mark.gpu


def test_jax_chunk_gla_matches_torch_path():
    jax = pytest.importorskip("jax")
    try:
        from tops_b200 import jax_ops
    except ImportError as exc:
        pytest.skip(str(exc))
    import jax.numpy as jnp
    import numpy as np
    import torch
    from tops_b200.ops.gla import chunk_gla
    from tops_b200.synth import make_inputs
    B, T, H, K, V = 2, 256, 4, 128, 128
    x = make_inputs(3, B, T, H, K, V, dtype=torch.bfloat16, with_h0=True, with_grads=True)
    j = {n: jnp.asarray(t.float().numpy(), dtype=jnp.float32 if t.dtype == torch.float32 else jnp.bfloat16) for n, t in x.items()}

    def loss(q, k, v, g, h0):
        o, ht = jax_ops.chunk_gla(q, k, v, g, initial_state=h0, output_final_state=True, chunk_size=64)
        return (o.astype(jnp.float32) * j["do"].astype(jnp.float32)).sum() + (ht * j["dht"]).sum()
    grads = jax.grad(loss, argnums=(0, 1, 2, 3, 4))(j["q"], j["k"], j["v"], j["g"], j["h0"])
    c = {n: t.cuda() for n, t in x.items()}
    leaves = [c[n].requires_grad_(True) for n in ("q", "k", "v", "g", "h0")]
    o, ht = chunk_gla(*leaves[:4], initial_state=leaves[4], output_final_state=True, chunk_size=64)
    ref = torch.autograd.grad((o, ht), leaves, (c["do"], c["dht"]))
    for a, b in zip(grads, ref):
        a = torch.from_numpy(np.asarray(a.astype(jnp.float32)))
        assert ((a - b.float().cpu()).norm() / b.float().norm()).item() <= 1e-3
