"""Shared chunk primitives, mirroring `tops/cpu/ops/common/{chunk_h,chunk_o}.py`:
`chunk_local_cumsum`, `chunk_fwd_h`, `chunk_bwd_dh`.  All take CUDA tensors in
the reference layout `[B, T, H, D]`; every function is one C-ABI call.
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _lib as L


def cdiv(a: int, b: int) -> int:
    return -(-a // b)


def _is_pow2(x: int) -> bool:
    return x >= 1 and (x & (x - 1)) == 0


def make_problem(B, T, H, K, V, chunk, dtype, gate_dtype, gate_kind, scale, impl=L.IMPL_AUTO,
                 cu_seqlens=None, keep=None):
    """Fill a ChunkProblem.  `cu_seqlens` may be a list / CPU tensor / CUDA
    tensor; both a device and a host copy are handed to the library and are
    kept alive through `keep`."""
    pb = L.ChunkProblem()
    pb.B, pb.T, pb.H, pb.K, pb.V, pb.chunk = B, T, H, K, V, chunk
    pb.dtype, pb.gate_dtype, pb.gate_kind, pb.impl = dtype, gate_dtype, gate_kind, impl
    pb.scale = float(scale)
    if cu_seqlens is not None:
        host = torch.as_tensor(cu_seqlens).to("cpu", torch.int32).contiguous()
        dev = host.to(torch.device("cuda", torch.cuda.current_device()))
        keep.extend([host, dev])
        pb.cu_seqlens, pb.cu_seqlens_host, pb.N = dev.data_ptr(), host.data_ptr(), host.numel() - 1
    return pb


def total_chunks(B, T, chunk, cu_seqlens=None) -> int:
    if cu_seqlens is None:
        return B * cdiv(T, chunk)
    cu = [int(x) for x in cu_seqlens]
    return sum(cdiv(cu[i + 1] - cu[i], chunk) for i in range(len(cu) - 1))


@L.on_tensor_device
def chunk_local_cumsum(g: torch.Tensor, chunk_size: int, reverse: bool = False,
                       cu_seqlens=None) -> torch.Tensor:
    """Chunk-local inclusive cumsum of log-gates along T, fp32 out
    (reference `tops/cpu/ops/common/chunk_o.py:18-112`).  `g` is `[B,T,H]` or
    `[B,T,H,K]`; `reverse=True` gives suffix sums.  With `cu_seqlens` (packed, B == 1) chunks restart at every
    sequence start: one launch per sequence on its slice (the fused chunk ops do their own packed cumsum in one)."""
    assert g.ndim in (3, 4), f"g must be [B,T,H] or [B,T,H,K], got {tuple(g.shape)}"
    assert _is_pow2(chunk_size), f"chunk_size must be a power of 2, got {chunk_size}"
    g = g.contiguous()
    if cu_seqlens is not None:
        cu = [int(c) for c in cu_seqlens]
        assert g.shape[0] == 1, f"cu_seqlens requires B=1, got B={g.shape[0]}"
        assert cu[0] == 0 and cu[-1] == g.shape[1] and all(b > a for a, b in zip(cu[:-1], cu[1:])), \
            f"cu_seqlens {cu} must rise from 0 to T={g.shape[1]}"
        out = torch.empty(g.shape, dtype=torch.float32, device=g.device)
        for a, b in zip(cu[:-1], cu[1:]):
            out[:, a:b] = chunk_local_cumsum(g[:, a:b], chunk_size, reverse)
        return out
    B, T, H = g.shape[:3]
    D = g.shape[3] if g.ndim == 4 else 1
    out = torch.empty(g.shape, dtype=torch.float32, device=g.device)
    p = L.CumsumParams(B, T, H, D, chunk_size, L.dtype_code(g.dtype), int(reverse), L.ptr(g), L.ptr(out), None, 0)
    L.check(L.lib.tops_b200_chunk_local_cumsum(C.byref(p), L.stream_ptr(g.device)), "chunk_local_cumsum")
    return out


def _gate_args(g, g_gamma, gk):
    given = [x is not None for x in (g, g_gamma, gk)]
    assert sum(given) <= 1, "pass at most one of g, g_gamma, gk"
    if gk is not None:
        return L.GATE_PER_CHANNEL, gk.float().contiguous()
    if g is not None:
        return L.GATE_SCALAR, g.float().contiguous()
    if g_gamma is not None:
        return L.GATE_GAMMA, g_gamma.float().contiguous()
    return L.GATE_NONE, None


@L.on_tensor_device
def chunk_fwd_h(k, v, *, g=None, g_gamma=None, gk=None, h0=None, output_final_state=False,
                states_in_fp32=False, chunk_size=64):
    """Chunk-start states of h <- h*exp(gate_last) + k~^T v~
    (reference `tops/cpu/ops/common/chunk_h.py:31-226`).  `g`/`gk` are
    chunk-local cumsums (fp32).  Returns (h `[B,NT,H,K,V]`, ht fp32 or None)."""
    assert k.ndim == 4 and v.ndim == 4 and k.shape[:3] == v.shape[:3]
    B, T, H, K = k.shape
    V = v.shape[-1]
    assert T % chunk_size == 0, f"T ({T}) must be a multiple of chunk_size ({chunk_size})"
    kind, gate = _gate_args(g, g_gamma, gk)
    k, v = k.contiguous(), v.contiguous()
    h0c = None if h0 is None else h0.float().contiguous()
    if h0c is not None:
        assert h0c.shape == (B, H, K, V)
    NT = T // chunk_size
    h = torch.empty(B, NT, H, K, V, dtype=torch.float32 if states_in_fp32 else k.dtype, device=k.device)
    ht = torch.empty(B, H, K, V, dtype=torch.float32, device=k.device) if output_final_state else None
    keep = []
    p = L.FwdHParams()
    p.pb = make_problem(B, T, H, K, V, chunk_size, L.dtype_code(k.dtype), L.F32, kind, 1.0, keep=keep)
    p.k, p.v, p.g_cumsum, p.h0, p.h, p.ht = L.ptr(k), L.ptr(v), L.ptr(gate), L.ptr(h0c), L.ptr(h), L.ptr(ht)
    p.h_dtype = L.dtype_code(h.dtype)
    L.check(L.lib.tops_b200_chunk_fwd_h(C.byref(p), L.stream_ptr(k.device)), "chunk_fwd_h")
    return h, ht


@L.on_tensor_device
def chunk_bwd_dh(q, do, *, g=None, g_gamma=None, gk=None, h0=None, dht=None, scale=1.0, chunk_size=64):
    """Reverse state-gradient scan (reference `tops/cpu/ops/common/chunk_h.py:229-427`).
    Returns (dh `[B,NT,H,K,V]` fp32, dh0 fp32 or None — only when h0 is given)."""
    assert q.ndim == 4 and do.ndim == 4 and q.shape[:3] == do.shape[:3]
    B, T, H, K = q.shape
    V = do.shape[-1]
    assert T % chunk_size == 0, f"T ({T}) must be a multiple of chunk_size ({chunk_size})"
    kind, gate = _gate_args(g, g_gamma, gk)
    q, do = q.contiguous(), do.contiguous()
    assert do.dtype == q.dtype
    dhtc = None if dht is None else dht.float().contiguous()
    NT = T // chunk_size
    dh = torch.empty(B, NT, H, K, V, dtype=torch.float32, device=q.device)
    dh0 = torch.empty(B, H, K, V, dtype=torch.float32, device=q.device) if h0 is not None else None
    keep = []
    p = L.BwdDhParams()
    p.pb = make_problem(B, T, H, K, V, chunk_size, L.dtype_code(q.dtype), L.F32, kind, scale, keep=keep)
    p.q, p.do_, p.g_cumsum, p.dht, p.dh, p.dh0 = L.ptr(q), L.ptr(do), L.ptr(gate), L.ptr(dhtc), L.ptr(dh), L.ptr(dh0)
    L.check(L.lib.tops_b200_chunk_bwd_dh(C.byref(p), L.stream_ptr(q.device)), "chunk_bwd_dh")
    return dh, dh0
