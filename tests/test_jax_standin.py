"""The numpy-backed stand-in for jax (tests/golden/jax_standin) keeps the jax semantics the reference fixtures
depend on.  Runs in a child process: putting the stand-in on `sys.path` here would shadow a real jax for every
later test of the session."""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))

SCRIPT = r'''
import numpy as np
import jax, jax.numpy as jnp
from jax import lax

a = jnp.arange(6, dtype=jnp.float32).reshape(2, 3)
assert isinstance(a, jax.Array) and isinstance(a.T, jax.Array) and isinstance(a[0], jax.Array)

# python scalars are weak: they never widen an array, also not the half types
b = a.astype(jnp.bfloat16)
assert (b * 1.5).dtype == jnp.bfloat16 and (b + 1).dtype == jnp.bfloat16 and (a * 2.0).dtype == jnp.float32
# ... and the scalar is rounded to the array's dtype before the operation: bf16(q) * bf16(scale)
q = jnp.asarray(np.float32(1.0)).astype(jnp.bfloat16)
s = 32 ** -0.5
assert float(q * s) == float(np.asarray(s, dtype=jnp.bfloat16)) != float(np.float32(s))
# integer arrays take the floating operand's dtype (numpy would give float64)
assert (a * jnp.arange(3)).dtype == jnp.float32
# half * float32 array -> float32
assert (b * a).dtype == jnp.float32

# no float64 / int64 unless x64 is switched on
assert jnp.zeros((2,)).dtype == jnp.float32 and a.astype(jnp.float64).dtype == jnp.float32
assert jnp.arange(3).dtype == jnp.int32 and jnp.asarray(np.float64(1.0) * np.ones(2)).dtype == jnp.float32
jax.config.update("jax_enable_x64", True)
assert a.astype(jnp.float64).dtype == jnp.float64 and jnp.zeros(2).dtype == jnp.float64
jax.config.update("jax_enable_x64", False)

# functional updates
z = jnp.zeros((3, 3))
z2 = z.at[1, :2].set(5.0).at[1, 0].add(1.0)
assert float(z.sum()) == 0.0 and float(z2[1, 0]) == 6.0 and float(z2[1, 1]) == 5.0

# dynamic_slice clamps its start so that the slice fits, and refuses a slice larger than the operand
x = jnp.arange(10, dtype=jnp.float32)
assert np.asarray(lax.dynamic_slice(x, (8,), (4,))).tolist() == [6.0, 7.0, 8.0, 9.0]
assert np.asarray(lax.dynamic_update_slice(x, jnp.ones(4), (8,))).tolist()[5:] == [5.0, 1.0, 1.0, 1.0, 1.0]
try:
    lax.dynamic_slice(x, (0,), (11,))
    raise SystemExit("slice larger than the operand was accepted")
except TypeError:
    pass

# loops and maps
carry, ys = lax.scan(lambda c, v: (c + v, c * v), jnp.asarray(0.0), jnp.arange(4, dtype=jnp.float32))
assert float(carry) == 6.0 and np.asarray(ys).tolist() == [0.0, 0.0, 2.0, 9.0]
carry, ys = lax.scan(lambda c, v: (c + v, c), jnp.asarray(0.0), jnp.arange(4, dtype=jnp.float32), reverse=True)
assert np.asarray(ys).tolist() == [6.0, 5.0, 3.0, 0.0]
assert float(lax.fori_loop(0, 5, lambda i, v: v + i, jnp.asarray(0.0))) == 10.0
assert float(lax.cond(jnp.asarray(3) > 2, lambda u: u + 1, lambda u: u - 1, jnp.asarray(1.0))) == 2.0
m = jax.vmap(lambda row, w: (row * w).sum(), in_axes=(0, None))(a, jnp.ones(3))
assert np.asarray(m).tolist() == [3.0, 12.0]
pair = jax.vmap(lambda row: (row.sum(), row * 2))(a)
assert pair[0].shape == (2,) and pair[1].shape == (2, 3)

# contraction with a requested result type computes in that type
e = jnp.einsum("ij,kj->ik", b, b, preferred_element_type=jnp.float32)
assert e.dtype == jnp.float32 and float(e[1, 1]) == 50.0
assert jnp.repeat(jnp.arange(2), jnp.asarray([1, 2]), total_repeat_length=3).tolist() == [0, 1, 1]
print("ok")
'''


def test_standin_semantics():
    env = dict(os.environ, PYTHONPATH=os.path.join(HERE, "golden", "jax_standin"))
    out = subprocess.run([sys.executable, "-c", SCRIPT], env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0 and out.stdout.strip().endswith("ok"), out.stdout + out.stderr
