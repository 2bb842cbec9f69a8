"""ctypes binding of libtops_b200.so (the C ABI declared in include/tops_b200.h).

There is no fallback: importing this module fails when the shared library has
not been built, and every op raises when the library reports an error.
"""
from __future__ import annotations

import ctypes as C
import functools
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_PATH = os.path.join(_HERE, "libtops_b200.so")
if not os.path.exists(_PATH):
    raise ImportError(
        f"{_PATH} is missing: build it with `python pallas-kernel_b200/build.py` "
        "(tops_b200 has no CPU or eager fallback)")
lib = C.CDLL(_PATH)

F32, BF16, F16 = 0, 1, 2
GATE_NONE, GATE_PER_CHANNEL, GATE_SCALAR, GATE_GAMMA = 0, 1, 2, 3
IMPL_AUTO, IMPL_GENERIC, IMPL_SM100 = 0, 1, 2

_DT = {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16}
_i32, _f32, _vp, _sz = C.c_int32, C.c_float, C.c_void_p, C.c_size_t


def dtype_code(dt: torch.dtype) -> int:
    assert dt in _DT, f"unsupported dtype {dt} (fp32, bf16, fp16 only)"
    return _DT[dt]


class CumsumParams(C.Structure):
    _fields_ = [("B", _i32), ("T", _i32), ("H", _i32), ("D", _i32), ("chunk", _i32), ("dtype", _i32),
                ("reverse", _i32), ("g", _vp), ("out", _vp), ("cu_seqlens", _vp), ("N", _i32)]


class ChunkProblem(C.Structure):
    _fields_ = [("B", _i32), ("T", _i32), ("H", _i32), ("K", _i32), ("V", _i32), ("chunk", _i32),
                ("dtype", _i32), ("gate_dtype", _i32), ("gate_kind", _i32), ("impl", _i32),
                ("scale", _f32), ("cu_seqlens", _vp), ("cu_seqlens_host", _vp), ("N", _i32)]


class FwdHParams(C.Structure):
    _fields_ = [("pb", ChunkProblem), ("k", _vp), ("v", _vp), ("g_cumsum", _vp), ("h0", _vp), ("h", _vp),
                ("h_dtype", _i32), ("ht", _vp)]


class BwdDhParams(C.Structure):
    _fields_ = [("pb", ChunkProblem), ("q", _vp), ("do_", _vp), ("g_cumsum", _vp), ("dht", _vp), ("dh", _vp),
                ("dh0", _vp)]


class ChunkFwdParams(C.Structure):
    _fields_ = [("pb", ChunkProblem), ("q", _vp), ("k", _vp), ("v", _vp), ("g", _vp), ("h0", _vp), ("o", _vp),
                ("ht", _vp), ("g_cumsum_out", _vp), ("A_out", _vp), ("h_out", _vp), ("saved_out", _vp), ("segments", _vp)]


class ChunkBwdParams(C.Structure):
    _fields_ = [("pb", ChunkProblem), ("q", _vp), ("k", _vp), ("v", _vp), ("g", _vp), ("h0", _vp), ("do_", _vp),
                ("dht", _vp), ("dq", _vp), ("dk", _vp), ("grad_dtype", _i32), ("dv", _vp), ("dg", _vp),
                ("dh0", _vp), ("h_saved", _vp), ("dg_dtype", _i32), ("rev_segments", _vp)]


class RecurrentFwdParams(C.Structure):
    _fields_ = [("B", _i32), ("T", _i32), ("H", _i32), ("K", _i32), ("V", _i32), ("dtype", _i32),
                ("gate_dtype", _i32), ("o_dtype", _i32), ("reverse", _i32), ("scale", _f32), ("q", _vp),
                ("k", _vp), ("v", _vp), ("gk", _vp), ("gv", _vp), ("state_in", _vp), ("state_out", _vp),
                ("o", _vp), ("cu_seqlens", _vp), ("N", _i32)]


class RecurrentBwdParams(C.Structure):
    _fields_ = [("B", _i32), ("T", _i32), ("H", _i32), ("K", _i32), ("V", _i32), ("dtype", _i32),
                ("gate_dtype", _i32), ("reverse", _i32), ("scale", _f32), ("q", _vp), ("k", _vp), ("v", _vp),
                ("gk", _vp), ("gv", _vp), ("o", _vp), ("do_", _vp), ("h0", _vp), ("dht", _vp), ("dq", _vp),
                ("dk", _vp), ("dv", _vp), ("dgk", _vp), ("dgv", _vp), ("dh0", _vp), ("cu_seqlens", _vp),
                ("N", _i32)]


class KdaFwdParams(C.Structure):
    _fields_ = [("B", _i32), ("T", _i32), ("H", _i32), ("K", _i32), ("V", _i32), ("dtype", _i32),
                ("gate_dtype", _i32), ("scale", _f32), ("q", _vp), ("k", _vp), ("v", _vp), ("g", _vp),
                ("beta", _vp), ("h0", _vp), ("o", _vp), ("ht", _vp)]


class KdaBwdParams(C.Structure):
    _fields_ = [("B", _i32), ("T", _i32), ("H", _i32), ("K", _i32), ("V", _i32), ("dtype", _i32),
                ("gate_dtype", _i32), ("scale", _f32), ("q", _vp), ("k", _vp), ("v", _vp), ("g", _vp),
                ("beta", _vp), ("h0", _vp), ("do_", _vp), ("dht", _vp), ("dq", _vp), ("dk", _vp), ("dv", _vp),
                ("dg", _vp), ("dbeta", _vp), ("dh0", _vp)]


class ChunkKdaFwdParams(C.Structure):
    _fields_ = [("B", _i32), ("T", _i32), ("H", _i32), ("K", _i32), ("V", _i32), ("chunk", _i32), ("dtype", _i32),
                ("gate_dtype", _i32), ("scale", _f32), ("q", _vp), ("k", _vp), ("v", _vp), ("g", _vp), ("beta", _vp),
                ("h0", _vp), ("o", _vp), ("ht", _vp), ("Aqk_out", _vp), ("Akk_out", _vp), ("saved_h", _vp),
                ("saved_vnew", _vp), ("saved_T", _vp), ("saved_R", _vp)]


_i64 = C.c_int64
GATE_ACT_KDA, GATE_ACT_KDA_LOWER_BOUND, GATE_ACT_LOG_SIGMOID = 0, 1, 2


class GateActParams(C.Structure):
    _fields_ = [("rows", _i64), ("H", _i32), ("K", _i32), ("kind", _i32), ("dtype", _i32), ("out_dtype", _i32),
                ("g", _vp), ("A_log", _vp), ("dt_bias", _vp), ("lower_bound", _f32), ("normalizer", _f32),
                ("clamp_min", _f32), ("has_clamp_min", _i32), ("out", _vp)]


class GateActBwdParams(C.Structure):
    _fields_ = [("fwd", GateActParams), ("dy", _vp), ("dy_dtype", _i32), ("dg", _vp), ("dA_log", _vp), ("dbias", _vp)]


class NormParams(C.Structure):
    _fields_ = [("rows", _i64), ("D", _i32), ("dtype", _i32), ("eps", _f32), ("x", _vp), ("gate", _vp), ("weight", _vp),
                ("y", _vp), ("rstd", _vp), ("dy", _vp), ("dx", _vp), ("dgate", _vp), ("dweight", _vp)]


class ChunkKdaBwdParams(C.Structure):
    _fields_ = [("B", _i32), ("T", _i32), ("H", _i32), ("K", _i32), ("V", _i32), ("chunk", _i32), ("dtype", _i32),
                ("gate_dtype", _i32), ("scale", _f32), ("q", _vp), ("k", _vp), ("v", _vp), ("g", _vp), ("beta", _vp),
                ("do_", _vp), ("dht", _vp), ("saved_h", _vp), ("saved_vnew", _vp), ("saved_T", _vp), ("saved_R", _vp),
                ("dq", _vp), ("dk", _vp), ("dg", _vp), ("dbeta", _vp), ("grad_dtype", _i32), ("dv", _vp), ("dh0", _vp)]


class StatePackParams(C.Structure):
    _fields_ = [("pb", ChunkProblem), ("reverse", _i32), ("x", _vp), ("g", _vp), ("y", _vp), ("state_out", _vp)]


class StateApplyParams(C.Structure):
    _fields_ = [("R", _i32), ("rank", _i32), ("reverse", _i32), ("BH", _i64), ("K", _i32), ("V", _i32), ("first", _vp),
                ("P", _vp), ("S", _vp), ("out_in", _vp), ("out_all", _vp)]


lib.tops_b200_strerror.restype = C.c_char_p
lib.tops_b200_strerror.argtypes = [C.c_int]
lib.tops_b200_launch_count.restype = C.c_int64
lib.tops_b200_launch_count.argtypes = []
lib.tops_b200_chunk_selected_impl.restype = C.c_int
lib.tops_b200_chunk_selected_impl.argtypes = [C.POINTER(ChunkProblem)]
lib.tops_b200_device_error.restype = C.c_int
lib.tops_b200_device_error.argtypes = [C.POINTER(C.c_int)]
lib.tops_b200_device_error_reset.restype = C.c_int
lib.tops_b200_device_error_reset.argtypes = []
lib.tops_b200_device_error_set.restype = C.c_int
lib.tops_b200_device_error_set.argtypes = [C.c_int]
lib.tops_b200_test_skip_load.restype = C.c_int
lib.tops_b200_test_skip_load.argtypes = [C.c_int]
lib.tops_b200_profile_enable.restype = C.c_int
lib.tops_b200_profile_enable.argtypes = [C.c_int]
lib.tops_b200_profile_read.restype = C.c_int
lib.tops_b200_profile_read.argtypes = [C.c_char_p, _sz]
for _name, _ptype, _ws in [
    ("tops_b200_chunk_local_cumsum", CumsumParams, False),
    ("tops_b200_chunk_fwd_h", FwdHParams, False),
    ("tops_b200_chunk_bwd_dh", BwdDhParams, False),
    ("tops_b200_chunk_gla_fwd", ChunkFwdParams, True),
    ("tops_b200_chunk_gla_bwd", ChunkBwdParams, True),
    ("tops_b200_fused_recurrent_gla_fwd", RecurrentFwdParams, False),
    ("tops_b200_fused_recurrent_gla_bwd", RecurrentBwdParams, True),
    ("tops_b200_kda_fwd", KdaFwdParams, False),
    ("tops_b200_kda_bwd", KdaBwdParams, True),
]:
    _f = getattr(lib, _name)
    _f.restype = C.c_int
    _f.argtypes = [C.POINTER(_ptype), _vp, _sz, _vp] if _ws else [C.POINTER(_ptype), _vp]
lib.tops_b200_chunk_kda_supported.restype = C.c_int
lib.tops_b200_chunk_kda_supported.argtypes = [C.POINTER(ChunkKdaFwdParams)]
lib.tops_b200_chunk_kda_fwd.restype = C.c_int
lib.tops_b200_chunk_kda_fwd.argtypes = [C.POINTER(ChunkKdaFwdParams), _vp]
for _name, _ptype, _ws in [
    ("tops_b200_gate_act_fwd", GateActParams, False),
    ("tops_b200_gate_act_bwd", GateActBwdParams, True),
    ("tops_b200_l2norm_fwd", NormParams, False),
    ("tops_b200_l2norm_bwd", NormParams, False),
    ("tops_b200_rmsnorm_gated_fwd", NormParams, False),
    ("tops_b200_rmsnorm_gated_bwd", NormParams, True),
]:
    _f = getattr(lib, _name)
    _f.restype = C.c_int
    _f.argtypes = [C.POINTER(_ptype), _vp, _sz, _vp] if _ws else [C.POINTER(_ptype), _vp]
lib.tops_b200_gate_act_bwd_workspace_bytes.restype = _sz
lib.tops_b200_gate_act_bwd_workspace_bytes.argtypes = [C.POINTER(GateActBwdParams)]
lib.tops_b200_rmsnorm_gated_bwd_workspace_bytes.restype = _sz
lib.tops_b200_rmsnorm_gated_bwd_workspace_bytes.argtypes = [C.POINTER(NormParams)]
lib.tops_b200_chunk_kda_bwd.restype = C.c_int
lib.tops_b200_chunk_kda_bwd.argtypes = [C.POINTER(ChunkKdaBwdParams), _vp, _sz, _vp]
lib.tops_b200_chunk_kda_bwd_workspace_bytes.restype = _sz
lib.tops_b200_chunk_kda_bwd_workspace_bytes.argtypes = [C.POINTER(ChunkKdaBwdParams)]
lib.tops_b200_chunk_state_exchange_pack.restype = C.c_int
lib.tops_b200_chunk_state_exchange_pack.argtypes = [C.POINTER(StatePackParams), _vp, _sz, _vp]
lib.tops_b200_chunk_state_exchange_pack_workspace_bytes.restype = _sz
lib.tops_b200_chunk_state_exchange_pack_workspace_bytes.argtypes = [C.POINTER(StatePackParams)]
lib.tops_b200_chunk_state_exchange_apply.restype = C.c_int
lib.tops_b200_chunk_state_exchange_apply.argtypes = [C.POINTER(StateApplyParams), _vp]
lib.tops_b200_chunk_gla_fwd_static.restype = C.c_int
lib.tops_b200_chunk_gla_fwd_static.argtypes = [C.POINTER(ChunkFwdParams), _vp]
STATIC_SCRATCH_BYTES = 32 * 1024 * 1024
E_STATIC_LIMIT = -8
for _name, _ptype in [
    ("tops_b200_chunk_fwd_workspace_bytes", ChunkFwdParams),
    ("tops_b200_chunk_bwd_workspace_bytes", ChunkBwdParams),
    ("tops_b200_fused_recurrent_gla_bwd_workspace_bytes", RecurrentBwdParams),
    ("tops_b200_kda_bwd_workspace_bytes", KdaBwdParams),
]:
    _f = getattr(lib, _name)
    _f.restype = _sz
    _f.argtypes = [C.POINTER(_ptype)]


class TopsError(RuntimeError):
    pass


lib.tops_b200_last_cuda_error.restype = C.c_int
lib.tops_b200_last_cuda_error.argtypes = [C.c_char_p, _sz]
E_CUDA = -5


def check(rc: int, what: str) -> None:
    if rc != 0:
        detail = ""
        if rc == E_CUDA:
            buf = C.create_string_buffer(256)
            lib.tops_b200_last_cuda_error(buf, len(buf))
            detail = f" [{buf.value.decode()}]"
        raise TopsError(f"{what}: {lib.tops_b200_strerror(rc).decode()} (code {rc}){detail}")


def ptr(t) -> int | None:
    """Device pointer of a tensor (None stays NULL)."""
    if t is None:
        return None
    assert t.is_cuda, "tops_b200 ops take CUDA tensors; there is no CPU path"
    assert t.is_contiguous(), "tensor must be contiguous"
    return t.data_ptr()


def stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def launch_count() -> int:
    return int(lib.tops_b200_launch_count())


def device_error() -> int:
    """Code of the first bounded device-side wait that gave up (0 = none); synchronises."""
    out = C.c_int(0)
    check(lib.tops_b200_device_error(C.byref(out)), "device_error")
    return out.value


def device_error_reset() -> None:
    check(lib.tops_b200_device_error_reset(), "device_error_reset")


def raise_on_device_error(what: str = "tops_b200") -> None:
    """Synchronise and raise TopsError when a kernel of this library gave up on a bounded wait
    since the word was last cleared (its outputs are then poisoned with NaN, not valid results).
    The word is cleared before raising so that one failure does not mark every later call."""
    code = device_error()
    if code != 0:
        device_error_reset()
        raise TopsError(f"{what}: a kernel gave up on a bounded device-side wait (code {code}); "
                        "its outputs are invalid")


# TOPS_B200_CHECK_DEVICE=1 makes every differentiable op check the device error word after its
# backward pass (one synchronisation per step); off by default, the word stays readable at any time.
CHECK_DEVICE = os.environ.get("TOPS_B200_CHECK_DEVICE", "0") not in ("", "0")


def on_tensor_device(fn):
    """Run `fn(t, ...)` with the CUDA device of its first argument current: kernel selection,
    workspace sizes and launches all follow the current device."""
    @functools.wraps(fn)
    def wrapped(t, *args, **kwargs):
        if not (isinstance(t, torch.Tensor) and t.is_cuda):
            return fn(t, *args, **kwargs)   # the op's own assertions reject it
        with torch.cuda.device(t.device):
            return fn(t, *args, **kwargs)
    return wrapped


def workspace(nbytes: int, device) -> torch.Tensor:
    return torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)
