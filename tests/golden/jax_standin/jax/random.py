"""`jax.random` of the stand-in: keys are seeds of numpy's PCG64.  The streams are NOT JAX's (threefry);
they serve tests that draw their own inputs and compare two implementations on them."""
import numpy as _np

from ._array import demote_dtype, wrap


def PRNGKey(seed):
    return wrap(_np.asarray([0, int(seed) & 0xFFFFFFFF], dtype=_np.uint32))


key = PRNGKey


def _seed(k):
    a = _np.asarray(k).astype(_np.uint64).ravel()
    return int(a[0]) * 4294967296 + int(a[1])


def split(k, num=2):
    rng = _np.random.Generator(_np.random.PCG64(_seed(k)))
    return wrap(rng.integers(0, 2 ** 32, size=(num, 2), dtype=_np.uint64).astype(_np.uint32))


def fold_in(k, data):
    return split(PRNGKey(_seed(k) ^ (int(data) * 0x9E3779B9)), 1)[0]


def _draw(k, fn, shape, dtype):
    rng = _np.random.Generator(_np.random.PCG64(_seed(k)))
    dt = demote_dtype(_np.float64 if dtype is None else dtype)
    return wrap(fn(rng, tuple(shape)).astype(dt))


def normal(k, shape=(), dtype=None):
    return _draw(k, lambda r, s: r.standard_normal(s), shape, dtype)


def uniform(k, shape=(), dtype=None, minval=0.0, maxval=1.0):
    return _draw(k, lambda r, s: minval + (maxval - minval) * r.random(s), shape, dtype)


def randint(k, shape, minval, maxval, dtype=None):
    rng = _np.random.Generator(_np.random.PCG64(_seed(k)))
    return wrap(rng.integers(minval, maxval, size=tuple(shape)).astype(demote_dtype(_np.int64 if dtype is None else dtype)))


def bernoulli(k, p=0.5, shape=()):
    rng = _np.random.Generator(_np.random.PCG64(_seed(k)))
    return wrap(rng.random(tuple(shape)) < p)
