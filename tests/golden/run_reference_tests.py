"""Run the reference's own CPU-only test files over the jax stand-in (a check of the stand-in, not of this
library): the relational tests the reference keeps for `tops/cpu/ops/**` (chunked == naive, packed == per
sequence, gather / scatter round trips, properties of the KDA intra-chunk backward) must pass when its
source runs on `tests/golden/jax_standin`, or the fixtures made with it would mean little.

    python -m tests.golden.run_reference_tests --reference <checkout of Fred33146/pallas-kernel> [pytest args]

Tests that need automatic differentiation (`jax.grad` / `jax.vjp`) or another GPU library are deselected;
nothing is written into the checkout (no cache, no bytecode).
"""
import argparse
import os
import sys
import types

HERE = os.path.dirname(os.path.abspath(__file__))

FILES = [
    "tests/ref/common/test_varlen_cumsum.py",
    "tests/ref/common/test_varlen_utils.py",
    "tests/ref/common/test_varlen_chunk_h.py",
    "tests/ref/gla/test_naive_gla.py",
    "tests/ref/gla/test_chunk_gla_varlen.py",
    "tests/ref/simple_gla/test_chunk_simple_gla_varlen.py",
    "tests/ref/kda/test_chunk_kda.py",
    "tests/ref/kda/test_naive_kda.py",
    "tests/ref/kda/test_fused_recurrent_kda.py",
    "tests/ref/gla/test_chunk_gla.py",
    "tests/ref/gla/test_fused_recurrent_gla.py",
    "tests/ref/simple_gla/test_chunk_simple_gla.py",
    "tests/ref/simple_gla/test_fused_recurrent_simple_gla.py",
]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    args, rest = ap.parse_known_args()
    ref = os.path.abspath(args.reference)
    sys.dont_write_bytecode = True
    sys.path.insert(0, ref)
    sys.path.insert(0, os.path.join(HERE, "jax_standin"))
    import tops  # noqa: F401
    pkg = types.ModuleType("tops.ops")          # tops/ops/__init__.py imports the Pallas kernels (real JAX only)
    pkg.__path__ = [os.path.join(ref, "tops", "ops")]
    sys.modules["tops.ops"] = pkg
    import jax
    import pytest

    def needs_autodiff(*a, **k):
        pytest.skip("needs jax.grad / jax.vjp, which the stand-in does not provide")
    jax.grad = jax.vjp = jax.value_and_grad = needs_autodiff
    # the reference's tests import their own `tests` package: forget this repository's
    root = os.path.dirname(os.path.dirname(HERE))
    sys.path[:] = [p for p in sys.path if os.path.abspath(p or os.getcwd()) != root]
    for name in [m for m in sys.modules if m == "tests" or m.startswith("tests.")]:
        del sys.modules[name]
    os.chdir(ref)
    sys.exit(pytest.main(["-q", "-p", "no:cacheprovider", "--rootdir", ref, "-k", "not grad and not triton and not fla",
                          *[os.path.join(ref, f) for f in FILES], *rest]))


if __name__ == "__main__":
    main()
