"""Out-of-bounds writes, checked without a sanitizer: every buffer the front-ends allocate for a kernel
(outputs, saved states, workspaces) is carved out of a larger allocation with a band of a known bit pattern on
both sides; after forward and backward of every kernel family, on ragged and on tile-aligned shapes, all bands
must be untouched.  A stray store of a few hundred elements past either end of a buffer lands in a band."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

BAND = 1024            # bytes on each side
PATTERN = 0x5A


class Arena:
    """Stands in for torch.empty / torch.zeros / *_like while a test runs."""

    def __init__(self):
        self.blocks = []
        self._empty, self._zeros = torch.empty, torch.zeros

    def _carve(self, shape, dtype, device, zero):
        if len(shape) == 1 and isinstance(shape[0], (tuple, list, torch.Size)):
            shape = tuple(shape[0])
        dtype = dtype or torch.float32
        nbytes = math.prod(shape) * torch.empty((), dtype=dtype).element_size()
        padded = (nbytes + 255) // 256 * 256          # keeps the inner buffer's start 256-byte aligned
        raw = torch.full((BAND + padded + BAND,), PATTERN, dtype=torch.uint8, device=device)
        self.blocks.append((raw, nbytes))
        inner = raw[BAND:BAND + nbytes].view(dtype).reshape(tuple(shape))
        if zero:
            inner.zero_()
        return inner

    def empty(self, *shape, dtype=None, device=None, **kw):
        if device is None or torch.device(device).type != "cuda":
            return self._empty(*shape, dtype=dtype, device=device, **kw)
        return self._carve(shape, dtype, device, False)

    def zeros(self, *shape, dtype=None, device=None, **kw):
        if device is None or torch.device(device).type != "cuda":
            return self._zeros(*shape, dtype=dtype, device=device, **kw)
        return self._carve(shape, dtype, device, True)

    def empty_like(self, t, **kw):
        return self.empty(tuple(t.shape), dtype=kw.get("dtype", t.dtype), device=t.device)

    def zeros_like(self, t, **kw):
        return self.zeros(tuple(t.shape), dtype=kw.get("dtype", t.dtype), device=t.device)

    def check(self):
        torch.cuda.synchronize()
        assert self.blocks, "no buffer went through the arena"
        for i, (raw, nbytes) in enumerate(self.blocks):
            assert bool((raw[:BAND] == PATTERN).all()), f"buffer {i} ({nbytes} bytes): bytes before it were written"
            assert bool((raw[BAND + nbytes:] == PATTERN).all()), f"buffer {i} ({nbytes} bytes): bytes after it were written"
        return len(self.blocks)


@pytest.fixture
def arena(monkeypatch):
    a = Arena()
    for name in ("empty", "zeros", "empty_like", "zeros_like"):
        monkeypatch.setattr(torch, name, getattr(a, name))
    return a


def _cuda_inputs(seed, B, T, H, K, V, dtype, **kw):
    from tops_b200.synth import make_inputs
    return {k: v.cuda() for k, v in make_inputs(seed, B, T, H, K, V, dtype=dtype, with_h0=True, with_grads=True, **kw).items()}


@pytest.mark.parametrize("B,T,H,K,V,C,dtype", [
    (1, 128, 2, 128, 128, 64, torch.bfloat16),     # tensor-core kernels: scan + chunk outputs
    (4, 64, 12, 128, 128, 64, torch.bfloat16),     # tensor-core kernels: fused forward
    (1, 1024, 2, 128, 128, 64, torch.bfloat16),    # time segments: summary scans + join
    (2, 37, 3, 8, 24, 16, torch.float32),          # generic kernels, ragged T, small K != V
    (1, 100, 2, 96, 80, 64, torch.float16),        # generic kernels, K and V not multiples of the tiles
])
def test_gla_kernels_stay_inside_their_buffers(arena, B, T, H, K, V, C, dtype):
    from tops_b200.ops.gla import chunk_gla_bwd, chunk_gla_fwd
    from tops_b200.ops._chunk import chunk_fwd_call
    from tops_b200 import _lib as L
    x = _cuda_inputs(51, B, T, H, K, V, dtype)
    scale = K ** -0.5
    chunk_fwd_call(x["q"], x["k"], x["v"], x["g"], L.GATE_PER_CHANNEL, scale, x["h0"], True, C, want_saved=True)
    chunk_gla_fwd(x["q"], x["k"], x["v"], x["g"], None, scale, x["h0"], True, chunk_size=C)
    chunk_gla_bwd(x["q"], x["k"], x["v"], x["g"], None, scale, x["h0"], None, None, x["do"], x["dht"], chunk_size=C)
    assert arena.check() >= 5


@pytest.mark.parametrize("B,T,H,K,V,dtype,gate", [
    (1, 256, 2, 128, 128, torch.bfloat16, "g"),      # scalar-gate tensor-core kernels
    (2, 50, 3, 32, 16, torch.float32, "g"),
    (1, 70, 2, 32, 48, torch.float32, "gamma"),
])
def test_simple_gla_kernels_stay_inside_their_buffers(arena, B, T, H, K, V, dtype, gate):
    from tops_b200.ops.simple_gla import chunk_simple_gla, chunk_simple_gla_bwd
    x = _cuda_inputs(52, B, T, H, K, V, dtype, gate="scalar")
    g = x["g"] if gate == "g" else None
    gam = -(0.05 + 0.1 * torch.rand(H)).cuda() if gate == "gamma" else None
    chunk_simple_gla(x["q"], x["k"], x["v"], g, gam, None, x["h0"], True, chunk_size=64)
    chunk_simple_gla_bwd(x["q"], x["k"], x["v"], g, gam, x["h0"], x["do"], x["dht"], K ** -0.5, chunk_size=64)
    assert arena.check() >= 4


@pytest.mark.parametrize("B,T,H,K,V,dtype", [
    (1, 128, 2, 128, 128, torch.bfloat16),       # chunked tensor-core kernels
    (2, 192, 3, 128, 128, torch.bfloat16),
    (2, 19, 2, 24, 40, torch.float32),           # token-serial kernels
])
def test_kda_kernels_stay_inside_their_buffers(arena, B, T, H, K, V, dtype):
    from tops_b200.ops import kda
    x = _cuda_inputs(53, B, T, H, K, V, dtype, with_beta=True, l2norm_qk=True)
    scale = K ** -0.5
    if kda.chunk_kernels_take(x["q"], x["k"], x["v"], x["g"], x["beta"], 64):
        kda.chunk_kda_fwd(x["q"], x["k"], x["v"], x["g"], x["beta"], scale, x["h0"], True)
        kda.chunk_kda_bwd(x["q"], x["k"], x["v"], x["g"], x["beta"], x["do"], scale, x["h0"], x["dht"])
    else:
        kda.kda_fwd(x["q"], x["k"], x["v"], x["g"], x["beta"], scale, x["h0"], True)
        kda.kda_bwd(x["q"], x["k"], x["v"], x["g"], x["beta"], x["do"], scale, x["h0"], x["dht"])
    assert arena.check() >= 4


def test_recurrent_cumsum_gate_and_norm_kernels_stay_inside_their_buffers(arena):
    from tops_b200.ops import gate, gla, norm
    from tops_b200.ops.common import chunk_local_cumsum
    x = _cuda_inputs(54, 2, 21, 3, 40, 24, torch.float32)
    o, ht = gla.fused_recurrent_fwd(x["q"], x["k"], x["v"], x["g"], None, None, x["h0"], True)
    gla.fused_recurrent_bwd(x["q"], x["k"], x["v"], x["g"], None, o, x["do"], x["dht"], None, x["h0"])
    chunk_local_cumsum(x["g"], 16)
    chunk_local_cumsum(x["g"][..., 0].contiguous(), 16, reverse=True)
    chunk_local_cumsum(x["g"][:1], 16, cu_seqlens=[0, 5, 21])
    A_log, bias = torch.randn(3).cuda(), torch.randn(3 * 40).cuda()
    gate.kda_gate_fwd(x["g"], A_log, bias)
    gate.gla_gate(x["g"])
    gnorm = torch.randn(2, 21, 3, 24).cuda()
    norm.FusedRMSNormGated(24).cuda()(x["v"], gnorm)
    assert arena.check() >= 8
