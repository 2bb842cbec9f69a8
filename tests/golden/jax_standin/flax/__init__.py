"""Stand-in for the few `flax.nnx` names the reference's layer and modules use (see ../jax/__init__.py)."""
from . import nnx  # noqa: F401
