"""CPU oracle for the gated-linear-attention hot path.

TEST INFRASTRUCTURE ONLY.  This package restates, in torch-on-CPU, the
algorithms of the reference's `tops/cpu/ops/**` "gold" implementation
(pure `jax.numpy`; JAX is not installable where this repository is built, so
the reference cannot be imported at test time and these functions stand in for it).  It is
imported by `tests/`, by `__graft_entry__.smoke()` and by the `cpu_baseline` /
`--impl reference` legs of `bench.py`, and by nothing else: the product
package never imports it and has no CPU fallback.

How the restatement is pinned: (1) against outputs of the reference's own,
unmodified source files, imported over a numpy-backed stand-in for the part
of the jax API they use and frozen as `tests/golden/ref_*.pt`
(`tests/golden/make_reference_golden.py`; checked in
`tests/test_reference_golden.py`: fp64 to 1e-12, fp32 to 2e-5, half
precision to rounding, every dtype equal); (2) by the equivalences the
reference's own tests use (chunked form == token-by-token recurrence in fp64
at 1e-10, explicit backward == autodiff of the naive recurrence at 1e-8,
state-split == single pass, dtype contracts), re-enacted in
`tests/test_oracle_*.py`; (3) by frozen vectors of this package itself.
Each function's docstring cites the reference file:line it follows.
"""
from .common import (  # noqa: F401
    acc_dtype,
    chunk_bwd_dh,
    chunk_fwd_h,
    chunk_local_cumsum,
    dot,
    prepare_chunk_indices,
)
