"""Row normalisations next to the attention kernels:

* `l2norm(x, eps=1e-6)`: `x / sqrt(sum(x^2) + eps)` over the last dimension, the q/k normalisation of
  KDA (`tops/cpu/ops/kda/fused_recurrent.py:14-18`);
* `FusedRMSNormGated`: `RMSNorm(x) * weight * silu(g)` (`tops/modules/fused_norm_gate.py:6-37`), the norm
  the reference applies to the attention output.

Both are differentiable; each direction is one kernel (plus a small fixed-order sum for the weight
gradient).  The last dimension must be a multiple of 4 and at most 1024.
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _lib as L


def _params(x, eps):
    D = x.shape[-1]
    assert D % 4 == 0 and D <= 1024, f"last dimension must be a multiple of 4 and <= 1024, got {D}"
    p = L.NormParams()
    p.rows, p.D, p.dtype, p.eps = x.numel() // D, D, L.dtype_code(x.dtype), float(eps)
    return p


@L.on_tensor_device
def _l2norm_fwd(x, eps):
    x = x.contiguous()
    y = torch.empty_like(x)
    p = _params(x, eps)
    p.x, p.y = L.ptr(x), L.ptr(y)
    L.check(L.lib.tops_b200_l2norm_fwd(C.byref(p), L.stream_ptr(x.device)), "l2norm_fwd")
    return y


@L.on_tensor_device
def _l2norm_bwd(x, dy, eps):
    x, dy = x.contiguous(), dy.to(x.dtype).contiguous()
    dx = torch.empty_like(x)
    p = _params(x, eps)
    p.x, p.dy, p.dx = L.ptr(x), L.ptr(dy), L.ptr(dx)
    L.check(L.lib.tops_b200_l2norm_bwd(C.byref(p), L.stream_ptr(x.device)), "l2norm_bwd")
    return dx


class _L2Norm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, eps):
        ctx.save_for_backward(x)
        ctx.eps = eps
        return _l2norm_fwd(x, eps)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        return _l2norm_bwd(x, dy, ctx.eps), None


def l2norm(x, eps=1e-6):
    """x / sqrt(sum(x^2, -1) + eps), in x's dtype (fp32 arithmetic)."""
    return _L2Norm.apply(x, float(eps))


@L.on_tensor_device
def _rms_fwd(x, g, w, eps):
    x, g = x.contiguous(), g.contiguous()
    y = torch.empty_like(x)
    p = _params(x, eps)
    p.x, p.gate, p.weight, p.y = L.ptr(x), L.ptr(g), L.ptr(w), L.ptr(y)
    L.check(L.lib.tops_b200_rmsnorm_gated_fwd(C.byref(p), L.stream_ptr(x.device)), "rmsnorm_gated_fwd")
    return y


@L.on_tensor_device
def _rms_bwd(x, g, w, dy, eps):
    x, g, dy = x.contiguous(), g.contiguous(), dy.to(x.dtype).contiguous()
    dx, dg = torch.empty_like(x), torch.empty_like(g)
    dw = None if w is None else torch.empty(x.shape[-1], dtype=torch.float32, device=x.device)
    p = _params(x, eps)
    p.x, p.gate, p.weight, p.dy, p.dx, p.dgate, p.dweight = (L.ptr(x), L.ptr(g), L.ptr(w), L.ptr(dy), L.ptr(dx), L.ptr(dg),
                                                             L.ptr(dw))
    ws = L.workspace(L.lib.tops_b200_rmsnorm_gated_bwd_workspace_bytes(C.byref(p)), x.device)
    L.check(L.lib.tops_b200_rmsnorm_gated_bwd(C.byref(p), ws.data_ptr(), ws.numel(), L.stream_ptr(x.device)),
            "rmsnorm_gated_bwd")
    return dx, dg, dw


class _RmsNormGated(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, g, weight, eps):
        w = None if weight is None else weight.float().contiguous()
        ctx.save_for_backward(x, g, weight)
        ctx.eps = eps
        return _rms_fwd(x, g, w, eps)

    @staticmethod
    def backward(ctx, dy):
        x, g, weight = ctx.saved_tensors
        w = None if weight is None else weight.float().contiguous()
        dx, dg, dw = _rms_bwd(x, g, w, dy, ctx.eps)
        return dx, dg, (None if weight is None else dw.to(weight.dtype)), None


def rmsnorm_gated(x, g, weight=None, eps=1e-5):
    """x * rsqrt(mean(x^2, -1) + eps) * weight * silu(g) in x's dtype (fp32 arithmetic)."""
    assert g.shape == x.shape, f"g shape {tuple(g.shape)} != x shape {tuple(x.shape)}"
    return _RmsNormGated.apply(x, g, weight, float(eps))


class FusedRMSNormGated(torch.nn.Module):
    """RMSNorm + SiLU gate (`tops/modules/fused_norm_gate.py:6-37`): `output = RMSNorm(x) * silu(g)`."""

    def __init__(self, hidden_size: int, elementwise_affine: bool = True, eps: float = 1e-5, device=None):
        super().__init__()
        self.hidden_size, self.eps = hidden_size, eps
        self.weight = torch.nn.Parameter(torch.ones(hidden_size, device=device)) if elementwise_affine else None

    def forward(self, x, g):
        return rmsnorm_gated(x, g, self.weight, self.eps)
