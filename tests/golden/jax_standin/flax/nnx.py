"""`flax.nnx` of the stand-in: parameters as plain holders, Linear / Conv / Sequential with flax's
conventions (kernels `[in, out]` and `[width, in / groups, out]`, cross-correlation, computation in the
promoted dtype of input and parameters).  Initial values are draws of the stand-in's generator, not flax's
initialisers: callers that compare with another implementation read the parameters back."""
import numpy as _np

import jax.numpy as jnp
from jax._array import wrap


class Param:
    def __init__(self, value):
        self.value = value

    def __getitem__(self, idx):
        return self.value[idx]


class Module:
    pass


class Rngs:
    def __init__(self, seed=0, **kwargs):
        self._rng = _np.random.Generator(_np.random.PCG64(int(seed)))

    def normal(self, shape, scale):
        return wrap((self._rng.standard_normal(shape) * scale).astype(_np.float32))


def _compute(x, *params):
    """flax computes in the promoted dtype of the input and the parameters (fp32 parameters: fp32)."""
    dt = _np.result_type(*[_np.asarray(a).dtype if _np.asarray(a).dtype.name != "bfloat16" else _np.float32
                           for a in (x, *params) if a is not None])
    return [None if a is None else _np.asarray(a).astype(dt) for a in (x, *params)]


class Linear(Module):
    def __init__(self, in_features, out_features, use_bias=True, *, rngs, **kwargs):
        self.in_features, self.out_features, self.use_bias = in_features, out_features, use_bias
        self.kernel = Param(rngs.normal((in_features, out_features), in_features ** -0.5))
        self.bias = Param(rngs.normal((out_features,), 0.1)) if use_bias else None

    def __call__(self, x):
        x, w, b = _compute(x, self.kernel.value, None if self.bias is None else self.bias.value)
        y = x @ w
        return wrap(y if b is None else y + b)


class Conv(Module):
    """1-D convolution, channels last; only what the depthwise causal convolution of the reference needs."""

    def __init__(self, in_features, out_features, kernel_size, feature_group_count=1, use_bias=True,
                 padding="SAME", *, rngs, **kwargs):
        assert padding == "VALID" and feature_group_count == in_features == out_features, "depthwise VALID only"
        (self.width,) = kernel_size
        self.kernel = Param(rngs.normal((self.width, 1, out_features), self.width ** -0.5))
        self.bias = Param(rngs.normal((out_features,), 0.1)) if use_bias else None

    def __call__(self, x):
        x, w, b = _compute(x, self.kernel.value, None if self.bias is None else self.bias.value)
        T = x.shape[1] - self.width + 1
        y = sum(x[:, i:i + T] * w[i, 0] for i in range(self.width))
        return wrap(y if b is None else y + b)


class Sequential(Module):
    def __init__(self, *layers):
        self.layers = list(layers)

    def __call__(self, x):
        for layer in self.layers:
            x = layer(x)
        return x
