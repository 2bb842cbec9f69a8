"""tops_b200 — B200 (sm_100a) kernels for the gated-linear-attention hot path
of `tops`, behind the reference's Python signatures.

    from tops_b200.ops.gla import chunk_gla, fused_chunk_gla, fused_recurrent_gla
    from tops_b200.ops.simple_gla import simple_gla, chunk_simple_gla

Importing the package loads libtops_b200.so (built by
`python pallas-kernel_b200/build.py`); there is no CPU or eager fallback.
"""
from . import _lib  # noqa: F401  (fails loudly when the library is missing)
from . import ops  # noqa: F401

__all__ = ["ops"]
