"""A numpy-backed stand-in for the small part of the `jax` API that the reference's CPU
implementation (`tops/cpu/ops/**`, pure `jax.numpy`) touches.

Purpose: JAX is not installed where this repository is built, so the reference cannot be imported as it
is.  With this directory in front of `sys.path`, `tests/golden/make_reference_golden.py` imports the
reference's own, unmodified source files and runs them on seeded inputs; what they return is frozen as
fixtures.  Nothing else imports this package: it is not an implementation of anything this library ships.

Semantics kept: arrays are immutable in use (`x.at[i].set(v)` returns a copy), `lax.dynamic_slice`
clamps its start indices, python scalars do not widen an array's dtype, integer arrays combined with
floating arrays take the floating dtype, and with `jax_enable_x64` off (the default, as in JAX) no
float64 / int64 array is ever produced.  Not kept: XLA's operation fusion and its reduction orders
(sums are numpy's), so float32 results agree with real JAX to rounding, not bit for bit; float64 results
are limited only by summation order.  Transformations: `vmap`, `lax.scan`, `lax.fori_loop`, `lax.cond`
are plain python loops; `jit` is the identity; `grad` / `vjp` are not provided.
"""
import contextlib

from . import _array
from ._array import Array
from . import numpy, lax, nn, random  # noqa: E402,F401


class _Config:
    def update(self, name, value):
        if name == "jax_enable_x64":
            _array.X64 = bool(value)

    @property
    def jax_enable_x64(self):
        return _array.X64


config = _Config()


class _Device:
    platform = "cpu"

    def __repr__(self):
        return "CpuDevice(id=0)"


_CPU = _Device()


def devices(kind=None):
    return [_CPU]


def default_backend():
    return "cpu"


@contextlib.contextmanager
def default_device(dev):
    yield


def device_put(x, device=None):
    return x


def jit(fn=None, **kwargs):
    if fn is None:
        return lambda f: f
    return fn


def _leaves(tree, out):
    if isinstance(tree, (tuple, list)):
        for t in tree:
            _leaves(t, out)
    elif isinstance(tree, dict):
        for t in tree.values():
            _leaves(t, out)
    elif tree is not None:
        out.append(tree)
    return out


def _map(fn, tree):
    if isinstance(tree, tuple):
        return tuple(_map(fn, t) for t in tree)
    if isinstance(tree, list):
        return [_map(fn, t) for t in tree]
    if isinstance(tree, dict):
        return {k: _map(fn, t) for k, t in tree.items()}
    if tree is None:
        return None
    return fn(tree)


def _stack(trees, axis=0):
    first = trees[0]
    if isinstance(first, tuple):
        return tuple(_stack([t[i] for t in trees], axis) for i in range(len(first)))
    if isinstance(first, list):
        return [_stack([t[i] for t in trees], axis) for i in range(len(first))]
    if isinstance(first, dict):
        return {k: _stack([t[k] for t in trees], axis) for k in first}
    if first is None:
        return None
    return numpy.stack([numpy.asarray(t) for t in trees], axis=axis)


def vmap(fn, in_axes=0, out_axes=0):
    """Map over one axis of every argument with a python loop."""
    assert out_axes == 0, "only out_axes=0 is provided"

    def mapped(*args):
        axes = tuple(in_axes) if isinstance(in_axes, (tuple, list)) else (in_axes,) * len(args)
        n = None
        for a, ax in zip(args, axes):
            if ax is not None:
                n = _leaves(a, [])[0].shape[ax]
                break
        outs = []
        for i in range(n):
            sl = [a if ax is None else _map(lambda x, ax=ax: numpy.take(x, i, axis=ax), a) for a, ax in zip(args, axes)]
            outs.append(fn(*sl))
        return _stack(outs)

    return mapped


def grad(*a, **k):
    raise NotImplementedError("the stand-in has no automatic differentiation")


vjp = value_and_grad = grad
