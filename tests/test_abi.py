"""The C-ABI library loads and exports every symbol include/tops_b200.h
declares; argument validation runs without a GPU."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "tops_b200.h")).read()
    return sorted(set(re.findall(r"\b(tops_b200_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from tops_b200 import _lib
    names = _declared_symbols()
    assert len(names) >= 10
    for n in names:
        assert hasattr(_lib.lib, n), f"{n} is declared in tops_b200.h but not exported"


def test_error_codes_without_gpu():
    from tops_b200 import _lib as L
    assert L.lib.tops_b200_strerror(0) == b"ok"
    assert b"shape" in L.lib.tops_b200_strerror(-1)
    p = L.ChunkFwdParams()
    assert L.lib.tops_b200_chunk_gla_fwd(ctypes.byref(p), None, 0, None) == -3      # NULL tensors
    p.q = p.k = p.v = p.o = 256
    assert L.lib.tops_b200_chunk_gla_fwd(ctypes.byref(p), None, 0, None) == -1      # zero dims
    p.pb.B, p.pb.T, p.pb.H, p.pb.K, p.pb.V, p.pb.chunk = 1, 64, 1, 64, 64, 48
    assert L.lib.tops_b200_chunk_gla_fwd(ctypes.byref(p), None, 0, None) == -1      # chunk not 16/32/64
    p.pb.chunk = 64
    p.pb.dtype = 7
    assert L.lib.tops_b200_chunk_gla_fwd(ctypes.byref(p), None, 0, None) == -2      # dtype
    p.pb.dtype = L.BF16
    assert L.lib.tops_b200_chunk_fwd_workspace_bytes(ctypes.byref(p)) > 0
    assert L.lib.tops_b200_chunk_gla_fwd(ctypes.byref(p), None, 0, None) == -4      # workspace
    assert L.launch_count() == 0


def test_python_front_end_rejects_cpu_tensors():
    import pytest
    import torch
    from tops_b200.ops.gla import chunk_gla
    x = torch.zeros(1, 16, 1, 16)
    with pytest.raises(AssertionError):
        chunk_gla(x, x, x, x)
