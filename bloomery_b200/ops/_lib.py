"""ctypes loader for the two native libraries.

The CUDA library is mandatory whenever a CUDA device is visible: a missing or stale
``libbloomery_cuda.so`` raises, it never falls back to eager PyTorch.
"""
from __future__ import annotations

import ctypes
import os
import threading
from typing import Optional

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_CDIR = os.path.join(os.path.dirname(_HERE), "_C")
_lock = threading.Lock()
_cuda: Optional[ctypes.CDLL] = None
_host: Optional[ctypes.CDLL] = None


class NativeMissing(RuntimeError):
    pass


def _load(name: str, builder: str) -> ctypes.CDLL:
    path = os.path.join(_CDIR, name)
    if not os.path.exists(path):
        from .. import build
        getattr(build, builder)()
    if not os.path.exists(path):
        raise NativeMissing(f"{path} is missing and could not be built")
    return ctypes.CDLL(path)


def host() -> ctypes.CDLL:
    global _host
    with _lock:
        if _host is None:
            lib = _load("libbloomery_host.so", "build_host")
            lib.blh_resident_row_bytes.restype = ctypes.c_long
            _host = lib
        return _host


def cuda() -> ctypes.CDLL:
    global _cuda
    with _lock:
        if _cuda is None:
            lib = _load("libbloomery_cuda.so", "build_cuda")
            lib.bl_error_string.restype = ctypes.c_char_p
            _cuda = lib
        return _cuda


class KernelError(RuntimeError):
    pass


def check(code: int, what: str) -> None:
    if code != 0:
        msg = cuda().bl_error_string(ctypes.c_int(code)).decode()
        raise KernelError(f"{what}: {msg} (code {code})")


def p(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    """Device (or host) pointer of a tensor, NULL for None."""
    if t is None:
        return ctypes.c_void_p(0)
    return ctypes.c_void_p(t.data_ptr())


def stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


I = ctypes.c_int
L = ctypes.c_long
F = ctypes.c_float
