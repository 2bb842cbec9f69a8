"""tops_b200_chunk_gla_fwd_static: the forward pass for hosts that cannot hand
the library any scratch memory (a runtime that owns the device heap and passes
a custom call only operands and results; a server with a fixed memory pool).
Its scratch is a 32 MiB device array inside the library image, so the call
allocates nothing.  Checked here through the C ABI against the ordinary entry
point, twice in a row because every call reuses the same array."""
import ctypes as C

import pytest
import torch

from tests.util import assert_close

pytestmark = pytest.mark.gpu


def _params(x, o, ht, chunk, dtype):
    from tops_b200 import _lib as L
    from tops_b200.ops.common import make_problem
    B, T, H, K = x["q"].shape
    V = x["v"].shape[-1]
    p = L.ChunkFwdParams()
    p.pb = make_problem(B, T, H, K, V, chunk, L.dtype_code(dtype), L.dtype_code(x["g"].dtype), L.GATE_PER_CHANNEL,
                        K ** -0.5, keep=[])
    p.q, p.k, p.v, p.g, p.h0 = (x[n].data_ptr() for n in ("q", "k", "v", "g", "h0"))
    p.o, p.ht = o.data_ptr(), ht.data_ptr()
    return p


@pytest.mark.parametrize("dtype,B,T,H,K,V,chunk", [
    (torch.float32, 2, 200, 2, 64, 48, 32),        # generic kernels, ragged T
    (torch.bfloat16, 1, 256, 2, 128, 128, 64),     # tcgen05 kernels: state scan + chunk outputs
    (torch.bfloat16, 4, 1024, 16, 128, 128, 64),   # tcgen05 kernels: one fused pass over two time segments
])
def test_static_scratch_forward_matches_workspace_forward(dtype, B, T, H, K, V, chunk):
    from tops_b200 import _lib as L
    from tops_b200.synth import make_inputs
    dev = torch.device("cuda", torch.cuda.current_device())
    stream = L.stream_ptr(dev)
    for call, seed in enumerate((41, 42)):          # two calls in a row on the shared array
        x = {n: t.cuda().contiguous() for n, t in make_inputs(seed, B, T, H, K, V, dtype=dtype, with_h0=True).items()}
        o_ref = torch.empty(B, T, H, V, dtype=dtype, device=dev)
        ht_ref = torch.empty(B, H, K, V, dtype=torch.float32, device=dev)
        p = _params(x, o_ref, ht_ref, chunk, dtype)
        ws = L.workspace(L.lib.tops_b200_chunk_fwd_workspace_bytes(C.byref(p)), dev)
        L.check(L.lib.tops_b200_chunk_gla_fwd(C.byref(p), ws.data_ptr(), ws.numel(), stream), "chunk_gla_fwd")
        o = torch.full_like(o_ref, float("nan"))
        ht = torch.full_like(ht_ref, float("nan"))
        p2 = _params(x, o, ht, chunk, dtype)
        # The claim itself: the device has exactly as much free memory after the call as before.  The
        # ordinary call above has already loaded every kernel the static call launches; the first static
        # call on a device is the set-up call, which makes the CUDA runtime load the part of the library
        # image that holds the 32 MiB array (once, by the runtime, not by an allocation call), so the
        # check starts with the second call.
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        L.check(L.lib.tops_b200_chunk_gla_fwd_static(C.byref(p2), stream), "chunk_gla_fwd_static")
        torch.cuda.synchronize()
        if call > 0:
            assert torch.cuda.mem_get_info()[0] == free_before
        assert_close("o", o, o_ref, dtype)
        assert_close("ht", ht, ht_ref, dtype)
        assert L.device_error() == 0


def test_fused_forward_needs_no_state_scratch():
    """The one-pass tcgen05 forward keeps its chunk-start states on chip, so its scratch is the
    segment bookkeeping only — far less than the bf16 [B,NT,H,K,V] states of the two-kernel form."""
    from tops_b200 import _lib as L
    from tops_b200.ops.common import make_problem
    B, T, H = 8, 4096, 16
    p = L.ChunkFwdParams()
    p.pb = make_problem(B, T, H, 128, 128, 64, L.BF16, L.BF16, L.GATE_PER_CHANNEL, 0.1, keep=[])
    p.q = p.k = p.v = p.g = p.o = 256
    if L.lib.tops_b200_chunk_selected_impl(C.byref(p.pb)) != L.IMPL_SM100:
        pytest.skip("needs the tcgen05 kernels")
    states = B * (T // 64) * H * 128 * 128 * 2
    assert L.lib.tops_b200_chunk_fwd_workspace_bytes(C.byref(p)) < states // 100
    assert L.lib.tops_b200_chunk_fwd_workspace_bytes(C.byref(p)) <= L.STATIC_SCRATCH_BYTES


def test_static_scratch_refuses_problems_beyond_its_size():
    from tops_b200 import _lib as L
    from tops_b200.ops.common import make_problem
    n0 = L.launch_count()
    p = L.ChunkFwdParams()
    # fp32 cumulative gates alone need B*T*H*K*4 = 64 MiB here
    p.pb = make_problem(4, 4096, 8, 128, 128, 64, L.F32, L.F32, L.GATE_PER_CHANNEL, 0.1, keep=[])
    p.q = p.k = p.v = p.g = p.o = 256                # never dereferenced: the size check comes first
    assert L.lib.tops_b200_chunk_fwd_workspace_bytes(C.byref(p)) > L.STATIC_SCRATCH_BYTES
    rc = L.lib.tops_b200_chunk_gla_fwd_static(C.byref(p), None)
    assert rc == L.E_STATIC_LIMIT
    assert b"static" in L.lib.tops_b200_strerror(rc)
    assert L.launch_count() == n0
