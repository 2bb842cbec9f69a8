"""The same kernels for JAX arrays: `chunk_gla`, `chunk_simple_gla` (per-token gate) and an in-place
`fused_recurrent_gla_step`, each a `jax.ffi.ffi_call` of a handler in libtops_b200_jax.so
(pallas-kernel_b200/jax_ffi/jax_ffi_shim.cc) that forwards to the C ABI, wrapped in `jax.custom_vjp`
like the reference's own differentiable ops (`tops/ops/simple_gla/chunk.py:778-827`).

Importing this module needs JAX and the shim library (`python pallas-kernel_b200/build.py --jax`); it
raises ImportError otherwise — there is no fallback.
"""
from __future__ import annotations

import ctypes
import functools
import os

import jax
import jax.numpy as jnp
import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_PATH = os.path.join(_HERE, "libtops_b200_jax.so")
if not os.path.exists(_PATH):
    raise ImportError(f"{_PATH} is missing: build it with `python pallas-kernel_b200/build.py --jax`")
ctypes.CDLL(os.path.join(_HERE, "libtops_b200.so"), mode=ctypes.RTLD_GLOBAL)
_shim = ctypes.CDLL(_PATH)
for _name in ("tops_b200_ffi_chunk_fwd", "tops_b200_ffi_chunk_bwd", "tops_b200_ffi_recurrent_step"):
    jax.ffi.register_ffi_target(_name, jax.ffi.pycapsule(getattr(_shim, _name)), platform="CUDA")


def _chunk_fwd(q, k, v, g, h0, scale, chunk):
    B, T, H, K = q.shape
    V = v.shape[-1]
    out = (jax.ShapeDtypeStruct(v.shape, v.dtype), jax.ShapeDtypeStruct((B, H, K, V), jnp.float32),
           jax.ShapeDtypeStruct((B, -(-T // chunk), H, K, V), q.dtype))
    return jax.ffi.ffi_call("tops_b200_ffi_chunk_fwd", out)(q, k, v, g, h0, scale=np.float32(scale), chunk=np.int32(chunk))


@functools.partial(jax.custom_vjp, nondiff_argnums=(5, 6))
def _chunk_op(q, k, v, g, h0, scale, chunk):
    o, ht, _ = _chunk_fwd(q, k, v, g, h0, scale, chunk)
    return o, ht


def _chunk_op_fwd(q, k, v, g, h0, scale, chunk):
    o, ht, saved = _chunk_fwd(q, k, v, g, h0, scale, chunk)
    return (o, ht), (q, k, v, g, h0, saved)


def _chunk_op_bwd(scale, chunk, res, cot):
    q, k, v, g, h0, saved = res
    do, dht = cot
    out = tuple(jax.ShapeDtypeStruct(x.shape, x.dtype) for x in (q, k, v, g)) + (jax.ShapeDtypeStruct(h0.shape, jnp.float32),)
    dq, dk, dv, dg, dh0 = jax.ffi.ffi_call("tops_b200_ffi_chunk_bwd", out)(
        q, k, v, g, h0, do.astype(q.dtype), dht.astype(jnp.float32), saved, scale=np.float32(scale), chunk=np.int32(chunk))
    return dq, dk, dv, dg, dh0.astype(h0.dtype)


_chunk_op.defvjp(_chunk_op_fwd, _chunk_op_bwd)


def chunk_gla(q, k, v, g, scale=None, initial_state=None, output_final_state=False, chunk_size=64):
    """`tops.ops.gla.chunk_gla` for jax.Arrays on the B200 kernels (g: [B,T,H,K]); differentiable."""
    B, T, H, K = q.shape
    h0 = jnp.zeros((B, H, K, v.shape[-1]), jnp.float32) if initial_state is None else initial_state.astype(jnp.float32)
    o, ht = _chunk_op(q, k, v, g, h0, float(K ** -0.5 if scale is None else scale), int(chunk_size))
    return o, (ht if output_final_state else None)


def chunk_simple_gla(q, k, v, g, scale=None, initial_state=None, output_final_state=False, chunk_size=64):
    """`tops.ops.simple_gla.chunk_simple_gla` with the per-token scalar gate g: [B,T,H]; differentiable."""
    return chunk_gla(q, k, v, g, scale, initial_state, output_final_state, chunk_size)


def fused_recurrent_gla_step(q, k, v, gk, state, scale=None):
    """Token-serial GLA over the tokens of this call (usually one); the state operand is donated to the
    result (`input_output_aliases`), so under jit the update is in place.  Returns (o, state')."""
    K = q.shape[-1]
    out = (jax.ShapeDtypeStruct(v.shape, q.dtype), jax.ShapeDtypeStruct(state.shape, jnp.float32))
    return jax.ffi.ffi_call("tops_b200_ffi_recurrent_step", out, input_output_aliases={4: 1})(
        q, k, v, gk, state, scale=np.float32(K ** -0.5 if scale is None else scale))
