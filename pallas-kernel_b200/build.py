"""Build libtops_b200.so (sm_100a) in-tree with nvcc.

Usage: python pallas-kernel_b200/build.py [--force]
Objects go to pallas-kernel_b200/build/, the shared library next to the
Python package (tops_b200/libtops_b200.so) so that it travels with the tree.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "tops_b200", "libtops_b200.so")
OBJ = os.path.join(HERE, "build")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-extended-lambda", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC",
    "-I" + os.path.join(ROOT, "include"), "-I" + CSRC,
]


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _deps_mtime():
    files = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    files.append(os.path.join(ROOT, "include", "tops_b200.h"))
    return max(os.path.getmtime(f) for f in files)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= _deps_mtime():
        return OUT
    os.makedirs(OBJ, exist_ok=True)
    extra = ["-Xptxas", "-v"] if verbose else []

    def compile_one(src):
        obj = os.path.join(OBJ, src[:-3] + ".o")
        cmd = [NVCC, *FLAGS, *extra, "-c", os.path.join(CSRC, src), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            print(r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=8) as ex:
        objs = list(ex.map(compile_one, _sources()))
    cmd = [NVCC, "-shared", "-o", OUT, *objs, "-lcudart"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return OUT


def build_jax_shim() -> str | None:
    """libtops_b200_jax.so: the XLA FFI handlers of jax_ffi/jax_ffi_shim.cc, compiled against
    jax.ffi.include_dir().  Only where JAX is installed; returns None (and says so) otherwise."""
    try:
        import jax  # noqa: F401
        inc = jax.ffi.include_dir()
    except Exception as exc:
        print(f"jax not found ({type(exc).__name__}: {exc}) - the jax.ffi shim is skipped")
        return None
    lib = build()
    out = os.path.join(HERE, "tops_b200", "libtops_b200_jax.so")
    cmd = [NVCC, "-std=c++17", "-O2", "-shared", "-Xcompiler", "-fPIC", "-I" + inc, "-I" + os.path.join(ROOT, "include"),
           os.path.join(HERE, "jax_ffi", "jax_ffi_shim.cc"), "-o", out, "-L" + os.path.dirname(lib), "-l:libtops_b200.so",
           "-Xlinker", "-rpath=$ORIGIN", "-lcudart"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"jax.ffi shim failed to build:\n{r.stdout}\n{r.stderr}")
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    if "--jax" in sys.argv:
        print(build_jax_shim())
