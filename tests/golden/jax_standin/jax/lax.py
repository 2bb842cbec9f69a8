"""`jax.lax` of the stand-in: slicing with JAX's index clamping, loops as python loops."""
import enum

import numpy as _np

from ._array import wrap


class Precision(enum.Enum):
    DEFAULT = 0
    HIGH = 1
    HIGHEST = 2


def _starts(shape, start_indices, sizes):
    out = []
    for dim, s, n in zip(shape, start_indices, sizes):
        if n > dim:
            raise TypeError(f"slice size {n} exceeds the operand's dimension {dim}")      # as JAX does
        s = int(_np.asarray(s))
        if s < 0:
            s += dim
        out.append(min(max(s, 0), dim - n))       # JAX clamps so that the slice stays inside
    return out


def dynamic_slice(operand, start_indices, slice_sizes):
    a = _np.asarray(operand)
    st = _starts(a.shape, start_indices, slice_sizes)
    return wrap(a[tuple(slice(s, s + n) for s, n in zip(st, slice_sizes))].copy())


def dynamic_update_slice(operand, update, start_indices):
    a = _np.array(_np.asarray(operand), copy=True)
    u = _np.asarray(update)
    st = _starts(a.shape, start_indices, u.shape)
    a[tuple(slice(s, s + n) for s, n in zip(st, u.shape))] = u.astype(a.dtype)
    return wrap(a)


def dynamic_slice_in_dim(operand, start_index, slice_size, axis=0):
    a = _np.asarray(operand)
    st = [0] * a.ndim
    sz = list(a.shape)
    st[axis], sz[axis] = start_index, slice_size
    return dynamic_slice(a, st, sz)


def fori_loop(lower, upper, body_fun, init_val):
    val = init_val
    for i in range(int(_np.asarray(lower)), int(_np.asarray(upper))):
        val = body_fun(wrap(_np.asarray(i, dtype=_np.int32)), val)
    return val


def cond(pred, true_fun, false_fun, *operands):
    return true_fun(*operands) if bool(_np.asarray(pred)) else false_fun(*operands)


def scan(f, init, xs=None, length=None, reverse=False, unroll=1):
    from . import _leaves, _map, _stack
    n = length if xs is None else _leaves(xs, [])[0].shape[0]
    order = range(n - 1, -1, -1) if reverse else range(n)
    carry, ys = init, [None] * n
    for i in order:
        x = None if xs is None else _map(lambda a: wrap(_np.asarray(a)[i]), xs)
        carry, y = f(carry, x)
        ys[i] = y
    return carry, (_stack(ys) if n and ys[0] is not None else None)


def stop_gradient(x):
    return x


def rsqrt(x):
    x = _np.asarray(x)
    return wrap((1.0 / _np.sqrt(x)).astype(x.dtype))
