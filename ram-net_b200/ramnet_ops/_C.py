"""Native module of ramnet_ops: loads libramnet_b200.so (C ABI, see include/ramnet_b200.h) and
defines the ``torch.ops.ramnet_ops.*`` operator schemas with their CUDA implementations.

Plays the role of the reference's compiled ``ramnet_ops._C``
(packages/ramnet-ops/csrc/ram_attn_bind.cpp:27-129): importing it registers the operators and
exposes ``INT_BITS``.  There is no CPU implementation behind these operators and no fallback:
if the shared library is missing, importing this module raises.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

import torch

_LIB_PATH = Path(__file__).resolve().parent / "libramnet_b200.so"
if not _LIB_PATH.exists():
    raise ImportError(
        f"{_LIB_PATH} is missing: build it with `python ram-net_b200/build.py` (needs nvcc); "
        "ramnet_ops has no CPU fallback for its CUDA operators.")

lib = ctypes.CDLL(str(_LIB_PATH))

_i64, _i32, _f64, _ptr = ctypes.c_int64, ctypes.c_int, ctypes.c_double, ctypes.c_void_p
_i64p = ctypes.POINTER(ctypes.c_int64)

lib.rn_int_bits.restype = ctypes.c_int
lib.rn_last_error.restype = ctypes.c_char_p
lib.rn_version.restype = ctypes.c_char_p

lib.rn_addr_fwd.restype = ctypes.c_int
lib.rn_addr_fwd.argtypes = [_ptr, _ptr, _i32, _i64p, _ptr, _i64p, _ptr, _ptr, _i64p,
                            _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _f64, _f64, _i32, _i32, _i32, _i32, _ptr]
lib.rn_addr_bwd.restype = ctypes.c_int
lib.rn_addr_bwd.argtypes = [_ptr, _ptr, _i64p, _ptr, _i64p, _ptr, _ptr, _i32, _i64p, _ptr, _i64p, _ptr, _ptr, _i64p,
                            _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _f64, _f64, _i32, _i32, _i32, _ptr]
lib.rn_decode_step.restype = ctypes.c_int
lib.rn_decode_step.argtypes = [_ptr, _ptr, _ptr, _ptr, _i32, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _f64,
                               _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _f64, _f64, _i32, _f64, _i32, _ptr]
lib.rn_decode_step_scaled.restype = ctypes.c_int
lib.rn_decode_step_scaled.argtypes = [_ptr, _ptr, _ptr, _ptr, _i32, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _f64, _ptr, _ptr, _i64p,
                                      _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _f64, _f64, _i32, _f64, _i32, _ptr]
lib.rn_decode_scales_supported.restype = ctypes.c_int
lib.rn_decode_scales_supported.argtypes = [_i32, _i64, _i64, _i64, _i64, _i64]

lib.rn_gsu_workspace_bytes.restype = ctypes.c_int64
lib.rn_gsu_workspace_bytes.argtypes = [_i64] * 7 + [_i32]
lib.rn_gsu_fwd_workspace_bytes.restype = ctypes.c_int64
lib.rn_gsu_fwd_workspace_bytes.argtypes = [_i32, _i32] + [_i64] * 7 + [_i32]
lib.rn_gsu_fwd_path.restype = ctypes.c_int
lib.rn_gsu_fwd_path.argtypes = [_i32, _i32] + [_i64] * 7 + [_i32]
lib.rn_gsu_owner_enable.restype = ctypes.c_int
lib.rn_gsu_owner_enable.argtypes = [_i32]
lib.rn_gsu_owner_profile.restype = ctypes.c_int
lib.rn_gsu_owner_profile.argtypes = [_ptr]
lib.rn_gsu_plan_info.restype = ctypes.c_int
lib.rn_gsu_plan_info.argtypes = [_i64] * 7 + [_i32, _i32, ctypes.POINTER(ctypes.c_int32), _i32]
lib.rn_gsu_fwd.restype = ctypes.c_int
lib.rn_gsu_fwd.argtypes = [_ptr, _ptr, _i64p, _ptr, _i64p, _ptr, _i64p, _i32, _ptr, _i64p, _ptr, _ptr, _ptr, _ptr, _ptr,
                           _i64p, _ptr, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i32, _f64, _i32, _ptr]

lib.rn_gsu_bwd_workspace_bytes.restype = ctypes.c_int64
lib.rn_gsu_bwd_workspace_bytes.argtypes = [_i64] * 7 + [_i32]
lib.rn_gsu_bwd.restype = ctypes.c_int
lib.rn_gsu_bwd.argtypes = [_ptr, _ptr, _i64p, _ptr, _i64p, _ptr, _i64p, _i32, _ptr, _i64p, _ptr, _ptr,
                           _ptr, _i64p, _ptr, _ptr, _ptr, _i64p, _ptr, _i64p, _ptr, _ptr, _ptr, _ptr, _i64,
                           _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i32, _f64, _i32, _ptr]
lib.rn_device_status.restype = ctypes.c_int
lib.rn_device_status.argtypes = [_i32, _ptr, _i32, ctypes.POINTER(ctypes.c_int)]
lib.rn_selftest_wait_timeout.restype = ctypes.c_int
lib.rn_selftest_wait_timeout.argtypes = [_i32, _i32, _i32, _ptr]
lib.rn_prof_enable.argtypes = [_i32]
lib.rn_prof_read.argtypes = [ctypes.POINTER(ctypes.c_float), _i32]

INT_BITS: int = int(lib.rn_int_bits())

DTYPE_CODE = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def check(rc: int) -> None:
    """Turn a non-zero C-ABI return code into RuntimeError (the reference raises the same type
    from its TORCH_CHECKs, packages/ramnet-ops/csrc/torch_compat.h:19-22)."""
    if rc != 0:
        raise RuntimeError(lib.rn_last_error().decode())


def device_status(device: torch.device | int | None = None, reset: bool = True) -> int:
    """Status word of ``device`` (0 = no kernel reported a failure since the last reset).  Synchronises the
    current stream of that device."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    index = dev.index if dev.index is not None else torch.cuda.current_device()
    out = ctypes.c_int(0)
    check(lib.rn_device_status(index, ctypes.c_void_p(torch.cuda.current_stream(index).cuda_stream), int(reset),
                               ctypes.byref(out)))
    return int(out.value)


CHECK_STATUS = os.environ.get("RAMNET_CHECK_STATUS", "0") not in ("", "0")


def check_device(t: torch.Tensor) -> None:
    """Debug mode (environment variable RAMNET_CHECK_STATUS=1): after a kernel launch, synchronise and turn a
    device-side failure report into RuntimeError.  Off by default: the operators never synchronise."""
    if CHECK_STATUS and not torch.cuda.is_current_stream_capturing():
        code = device_status(t.device)
        if code != 0:
            raise RuntimeError(f"ramnet_ops kernel reported device status {code} (1 = a bounded wait on an "
                               "asynchronous copy ran out); results of the last calls on this device are incomplete")


def gsu_plan_info(B, H, T, A, C, Kw, Kr, reverse=False, device=0) -> dict:
    """Launch plan of a prefill call (see rn_gsu_plan_info in include/ramnet_b200.h)."""
    out = (ctypes.c_int32 * 8)()
    check(lib.rn_gsu_plan_info(B, H, T, A, C, Kw, Kr, int(reverse), device, out, 8))
    names = ("fast", "cs", "ev", "nslices", "L", "state_in_smem", "ev_bwd", "smem_tables")
    info = dict(zip(names, (int(v) for v in out)))
    # forward of 16-bit values with 16-byte aligned rows: 1 when the slot-owner cluster kernel takes the call
    # (it needs no workspace), 0 when the channel-slice kernels do
    info["owner_16bit"] = int(lib.rn_gsu_fwd_workspace_bytes(DTYPE_CODE[torch.bfloat16], 1, B, H, T, A, C, Kw, Kr, device) == 0)
    # 0 general, 1 channel-slice kernels with chains, 2 slot-owner cluster kernel
    info["fwd_path_16bit"] = int(lib.rn_gsu_fwd_path(DTYPE_CODE[torch.bfloat16], 1, B, H, T, A, C, Kw, Kr, device))
    return info


def strides(t: torch.Tensor):
    return (ctypes.c_int64 * t.dim())(*t.stride())


def ptr(t: torch.Tensor | None):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def stream_of(t: torch.Tensor):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def dtype_code(t: torch.Tensor) -> int:
    try:
        return DTYPE_CODE[t.dtype]
    except KeyError:
        raise RuntimeError(f"ramnet_ops CUDA kernels support float32/float16/bfloat16, got {t.dtype}") from None


from . import _ops  # noqa: E402,F401  (defines torch.ops.ramnet_ops.* on import)
