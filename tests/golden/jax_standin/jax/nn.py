"""`jax.nn` of the stand-in."""
import numpy as _np

from ._array import wrap


def sigmoid(x):
    x = _np.asarray(x)
    return wrap((1.0 / (1.0 + _np.exp(-x.astype(_np.float64)))).astype(x.dtype))


def softplus(x):
    x = _np.asarray(x)
    return wrap(_np.logaddexp(x.astype(_np.float64), 0.0).astype(x.dtype))


def log_sigmoid(x):
    x = _np.asarray(x)
    return wrap((-_np.logaddexp(-x.astype(_np.float64), 0.0)).astype(x.dtype))


def silu(x):
    x = _np.asarray(x)
    return wrap((x.astype(_np.float64) / (1.0 + _np.exp(-x.astype(_np.float64)))).astype(x.dtype))


swish = silu


def relu(x):
    return wrap(_np.maximum(_np.asarray(x), 0))


def tanh(x):
    return wrap(_np.tanh(_np.asarray(x)))


def gelu(x, approximate=True):
    x = _np.asarray(x)
    xf = x.astype(_np.float64)
    if approximate:
        y = 0.5 * xf * (1.0 + _np.tanh(_np.sqrt(2.0 / _np.pi) * (xf + 0.044715 * xf ** 3)))
    else:
        from math import erf
        y = 0.5 * xf * (1.0 + _np.vectorize(erf)(xf / _np.sqrt(2.0)))
    return wrap(y.astype(x.dtype))
