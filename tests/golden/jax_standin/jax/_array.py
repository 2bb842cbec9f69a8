"""The array type of the stand-in: a numpy.ndarray subclass with `.at[...]`, JAX's scalar promotion and
the float64 / int64 demotion of a JAX process that has not enabled x64."""
import numpy as np

X64 = False     # jax_enable_x64


def demote_dtype(dt):
    dt = np.dtype(dt)
    if not X64:
        if dt == np.float64:
            return np.dtype(np.float32)
        if dt == np.int64:
            return np.dtype(np.int32)
        if dt == np.complex128:
            return np.dtype(np.complex64)
    return dt


def wrap(x):
    """numpy result -> Array (demoted when x64 is off); tuples element-wise; python scalars untouched."""
    if isinstance(x, tuple):
        return tuple(wrap(v) for v in x)
    if isinstance(x, list):
        return [wrap(v) for v in x]
    if isinstance(x, (np.ndarray, np.generic)):
        a = np.asarray(x)
        dt = demote_dtype(a.dtype)
        if dt != a.dtype:
            a = a.astype(dt)
        return a.view(Array)
    return x


def _is_float(dt):
    return np.issubdtype(dt, np.floating) or dt.name in ("bfloat16",)


class _At:
    def __init__(self, arr):
        self.arr = arr

    def __getitem__(self, idx):
        return _AtIdx(self.arr, idx)


class _AtIdx:
    def __init__(self, arr, idx):
        self.arr, self.idx = arr, idx

    def _val(self, v):
        return np.asarray(v).astype(self.arr.dtype) if not np.isscalar(v) else v

    def set(self, v):
        out = np.array(self.arr, copy=True)
        out[self.idx] = self._val(v)
        return out.view(Array)

    def add(self, v):
        out = np.array(self.arr, copy=True)
        out[self.idx] = out[self.idx] + self._val(v)
        return out.view(Array)

    def multiply(self, v):
        out = np.array(self.arr, copy=True)
        out[self.idx] = out[self.idx] * self._val(v)
        return out.view(Array)

    def get(self):
        return wrap(np.asarray(self.arr)[self.idx])


class Array(np.ndarray):
    __array_priority__ = 100

    def __new__(cls, a):
        return wrap(np.asarray(a))

    @property
    def at(self):
        return _At(self)

    def astype(self, dtype, *args, **kwargs):
        return np.ndarray.astype(np.asarray(self), demote_dtype(dtype)).view(Array)

    def block_until_ready(self):
        return self

    def __array_ufunc__(self, ufunc, method, *inputs, out=None, **kwargs):
        # JAX's promotion where it differs from numpy's: python scalars are weak also for the
        # ml_dtypes half types, and an integer / bool array meeting a floating array takes its dtype
        arrs = [np.asarray(i) for i in inputs if isinstance(i, np.ndarray)]
        fdts = [a.dtype for a in arrs if _is_float(a.dtype)]
        target = None
        if fdts:
            target = fdts[0]
            for d in fdts[1:]:
                target = np.promote_types(target, d) if d != target else target
        conv = []
        for i in inputs:
            if isinstance(i, np.ndarray):
                a = np.asarray(i)
                if target is not None and not _is_float(a.dtype) and a.dtype != np.bool_ \
                        and ufunc.nin > 1 and ufunc not in (np.left_shift, np.right_shift):
                    a = a.astype(target)
                conv.append(a)
            elif isinstance(i, (bool, int, float)) and target is not None and not isinstance(i, bool):
                conv.append(np.asarray(i, dtype=target))
            else:
                conv.append(i)
        if out is not None:
            kwargs["out"] = tuple(np.asarray(o) for o in out)
        res = getattr(ufunc, method)(*conv, **kwargs)
        return wrap(res)

    def __getitem__(self, idx):
        return wrap(np.ndarray.__getitem__(np.asarray(self), _plain_index(idx)))

    def sum(self, *a, **k):
        return wrap(np.asarray(self).sum(*a, **k))

    def mean(self, *a, **k):
        return wrap(np.asarray(self).mean(*a, **k))

    def max(self, *a, **k):
        return wrap(np.asarray(self).max(*a, **k))

    def min(self, *a, **k):
        return wrap(np.asarray(self).min(*a, **k))

    def cumsum(self, *a, **k):
        return wrap(np.asarray(self).cumsum(*a, **k))

    def __matmul__(self, other):
        return wrap(np.matmul(np.asarray(self), np.asarray(other)))

    def __rmatmul__(self, other):
        return wrap(np.matmul(np.asarray(other), np.asarray(self)))


def _plain_index(idx):
    if isinstance(idx, tuple):
        return tuple(_plain_index(i) for i in idx)
    if isinstance(idx, np.ndarray):
        a = np.asarray(idx)
        return int(a) if a.ndim == 0 and np.issubdtype(a.dtype, np.integer) else a
    return idx
