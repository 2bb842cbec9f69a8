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
