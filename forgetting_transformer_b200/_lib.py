"""ctypes binding of ``libfox_b200.so`` (the C ABI declared in include/fox_b200.h).

There is no fallback: if the library is missing or a call fails, an exception is
raised.  The library is looked up next to this file; it is built in-tree by
``python -m forgetting_transformer_b200.build``.
"""
from __future__ import annotations

import ctypes
import os
import threading
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_int32, c_int64, c_void_p

import torch

from . import build as _build

_ERRORS = {
    -1: "FOX_ERR_BAD_ARG", -2: "FOX_ERR_HEAD_DIM", -3: "FOX_ERR_ALIGNMENT", -4: "FOX_ERR_DRIVER",
    -5: "FOX_ERR_TENSORMAP", -6: "FOX_ERR_LAUNCH", -7: "FOX_ERR_DEVICE", -8: "FOX_ERR_TOO_LARGE",
    -9: "FOX_ERR_THRESHOLD", -10: "FOX_ERR_NO_MEMORY",
}

FOX_DTYPE_FP16, FOX_DTYPE_BF16, FOX_DTYPE_FP32 = 0, 1, 2


class FoxError(RuntimeError):
    pass


class Tensor4(Structure):
    """Mirror of ``fox_tensor4``: base pointer + element strides of the B, H, T axes."""
    _fields_ = [("ptr", c_void_p), ("sb", c_int64), ("sh", c_int64), ("st", c_int64)]


_T4P = POINTER(Tensor4)
_F = c_void_p  # device pointers are passed as integers

_SIGNATURES = {
    "fox_version": (c_char_p, []),
    "fox_cumsum_fwd": (c_int, [c_int, c_void_p, c_int64, c_int64, c_int64, _F, c_int64, c_int64, c_int64, _F, _F, _F, _F]),
    "fox_gate_prefix_fwd": (c_int, [c_int, c_void_p, c_int, c_int64, c_int64, c_int64, _F, c_int64, c_int64, c_int64, _F, _F, _F]),
    "fox_gate_prefix_bwd": (c_int, [c_int, c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, _F, _F, _F, c_int64, c_int64,
                                    c_int64, _F]),
    "fox_revcumsum": (c_int, [c_int, c_void_p, c_int64, c_int64, c_int64, c_int64, _F, _F, _F, _F, _F]),
    "fox_find_index": (c_int, [c_int, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, _F, _F, c_int64, c_int64, _F, _F]),
    "fox_max_row_norm": (c_int, [c_int, c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, _T4P, _F]),
    "fox_bwd_delta": (c_int, [c_int, c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, _T4P, _T4P, _F]),
    "fox_dq_convert": (c_int, [c_int, c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, _F, c_float, _T4P]),
    "fox_attn_fwd": (c_int, [c_int, c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, c_int64, _T4P, _T4P, _T4P,
                             _F, _F, _F, c_float, _T4P, _F, _F, _F]),
    "fox_attn_decode": (c_int, [c_int, c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, _T4P, _T4P, _T4P, _F, _F, _F,
                                c_float, _T4P, _F, _F, c_int64]),
    "fox_attn_decode_workspace_floats": (c_int64, [c_int64, c_int64, c_int64, c_int64]),
    "fox_attn_bwd": (c_int, [c_int, c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, c_int64, _T4P, _T4P, _T4P,
                             _T4P, _F, _F, _F, _F, _F, c_float, _F, _F, _F, _T4P, _T4P, _F]),
    "fox_attn_bwd_dq": (c_int, [c_int, c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, c_int64, _T4P, _T4P, _T4P,
                                _T4P, _F, _F, _F, _F, _F, c_float, _T4P, _F, _F]),
    "fox_attn_bwd_noalloc": (c_int, [c_int, c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, c_int64, _T4P, _T4P,
                                     _T4P, _T4P, _F, _F, _F, _F, _F, c_float, _T4P, _T4P, _T4P, _F, _F, _F]),
    "fox_noalloc_scratch_floats": (c_int64, []),
    "fox_normgate_fwd": (c_int, [c_int, c_void_p, c_int, c_int64, c_int64, c_int64, _F, _F, _F, c_float, _F, _F]),
    "fox_normgate_bwd": (c_int, [c_int, c_void_p, c_int, c_int64, c_int64, c_int64, _F, _F, _F, _F, _F, _F, _F, _F, c_int64]),
    "fox_rmsnorm_fwd": (c_int, [c_int, c_void_p, c_int, c_int64, c_int64, _F, _F, _F, c_float, _F, _F, _F]),
    "fox_rmsnorm_bwd": (c_int, [c_int, c_void_p, c_int, c_int64, c_int64, _F, _F, _F, _F, _F, _F, _F, c_int64]),
    "fox_swiglu_fwd": (c_int, [c_int, c_void_p, c_int, c_int64, c_int64, _F, c_int64, _F, c_int64, _F, c_int64]),
    "fox_swiglu_bwd": (c_int, [c_int, c_void_p, c_int, c_int64, c_int64, _F, c_int64, _F, c_int64, _F, c_int64, _F,
                               c_int64, _F, c_int64, _F, c_int64]),
    "fox_cross_entropy_fwd": (c_int, [c_int, c_void_p, c_int, c_int64, c_int64, _F, c_int64, _F, c_float, c_float,
                                      c_float, c_int64, _F, _F, _F]),
    "fox_cross_entropy_bwd": (c_int, [c_int, c_void_p, c_int, c_int64, c_int64, _F, c_int64, _F, _F, _F, c_int64,
                                      c_float, c_float, c_float, c_int64, _F, c_int64]),
    "fox_cross_entropy_fwd_split": (c_int, [c_int, c_void_p, c_int, c_int64, c_int64, _F, c_int64, _F, c_float, c_float,
                                            c_int64, c_int64, c_int64, _F, _F]),
    "fox_cross_entropy_bwd_split": (c_int, [c_int, c_void_p, c_int, c_int64, c_int64, _F, c_int64, _F, _F, _F, c_int64,
                                            c_float, c_float, c_float, c_int64, c_int64, c_int64, _F, c_int64]),
    "fox_token_shift_fwd": (c_int, [c_int, c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, _F, c_int64, c_int64,
                                    c_int64, _F, _F, c_int64, c_int64, c_int64, _F]),
    "fox_token_shift_bwd": (c_int, [c_int, c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, _F, c_int64, c_int64,
                                    c_int64, _F, _F, c_int64, c_int64, c_int64, _F, _F, _F, _F]),
}

_lock = threading.Lock()
_lib = None


def lib_path() -> str:
    return _build.LIB_PATH


def load() -> ctypes.CDLL:
    """Load the shared library (building it first when the file is absent).
    Raises FoxError when it cannot be loaded."""
    global _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = lib_path()
        if not os.path.exists(path) and os.environ.get("FOX_B200_NO_BUILD") != "1":
            try:
                _build.build()
            except Exception as exc:
                raise FoxError(f"cannot build {path}: {exc}") from exc
        if not os.path.exists(path):
            raise FoxError(f"{path} is missing; run `python -m forgetting_transformer_b200.build`")
        lib = ctypes.CDLL(path)
        for name, (res, args) in _SIGNATURES.items():
            try:
                fn = getattr(lib, name)
            except AttributeError:
                continue
            fn.restype = res
            fn.argtypes = args
        _lib = lib
        return lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise FoxError(f"{what} failed: {_ERRORS.get(rc, rc)}")


def t4(x: torch.Tensor) -> Tensor4:
    """fox_tensor4 view of a (B, H, T, D) tensor with unit stride on D."""
    assert x.dim() == 4 and x.stride(3) == 1
    return Tensor4(x.data_ptr(), x.stride(0), x.stride(1), x.stride(2))


def ptr(x):
    return None if x is None else x.data_ptr()


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.bfloat16:
        return FOX_DTYPE_BF16
    if dt == torch.float16:
        return FOX_DTYPE_FP16
    raise FoxError(f"unsupported dtype {dt}")


def tma_ready(x: torch.Tensor) -> bool:
    """True when the view can be addressed by TMA as it is: unit inner stride,
    16-byte aligned base and byte strides."""
    if x.stride(-1) != 1 or x.data_ptr() % 16:
        return False
    es = x.element_size()
    return all((x.stride(i) * es) % 16 == 0 and x.stride(i) > 0 or x.shape[i] == 1 for i in range(x.dim() - 1))


# ------------------------------------------------------------------ status words
_status = {}


def status_buffer(device: torch.device) -> torch.Tensor:
    """Per-device int32[4] the attention kernels report a failed bounded wait in."""
    key = (device.index if device.index is not None else torch.cuda.current_device())
    buf = _status.get(key)
    if buf is None:
        buf = torch.zeros(4, dtype=torch.int32, device=device)
        _status[key] = buf
    return buf


_readback = {}   # device ordinal -> (pinned int32[4], event of the last queued copy)


def queue_status_readback(device: torch.device) -> None:
    """Queue, on the current stream, a copy of the device's status words to pinned host memory (no
    synchronisation); ``poll_status`` looks at it once it has landed.  Skipped while a CUDA graph is being
    captured."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    buf = _status.get(key)
    if buf is None or torch.cuda.is_current_stream_capturing():
        return
    slot = _readback.get(key)
    if slot is None:
        slot = (torch.zeros(4, dtype=torch.int32).pin_memory(), torch.cuda.Event())
        _readback[key] = slot
    slot[0].copy_(buf, non_blocking=True)
    slot[1].record()


def poll_status(device: torch.device) -> None:
    """Non-synchronising check: raises FoxError when the last status readback that has completed shows that a
    bounded wait inside a kernel ran out (the results of that step are incomplete)."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    slot = _readback.get(key)
    if slot is None or torch.cuda.is_current_stream_capturing() or not slot[1].query():
        return
    vals = slot[0].tolist()
    if vals[0] != 0:
        slot[0].zero_()
        _status[key].zero_()
        raise FoxError(f"kernel wait timed out in an earlier step: site={vals[0]} cta={vals[1]} thread={vals[2]} "
                       f"detail={vals[3]}")


def check_status(device=None) -> None:
    """Synchronising check of the kernels' status words; raises if a wait ran out."""
    for key, buf in list(_status.items()):
        if device is not None and torch.device(device).index not in (None, key):
            continue
        vals = buf.tolist()
        if vals[0] != 0:
            buf.zero_()
            raise FoxError(f"kernel wait timed out: site={vals[0]} cta={vals[1]} thread={vals[2]} detail={vals[3]}")
