"""Logistic-regression loss kernel binding (``csrc/logreg.cu``)."""
from __future__ import annotations

import ctypes

import torch

from . import _lib


def logreg_loss(A: torch.Tensor, y: torch.Tensor, x: torch.Tensor, lam: float) -> float:
    """mean log(1 + exp(-y A x)) + lam/2 ||x||^2 with A fp32 [N, d] on the device, x fp64 [d]."""
    lib = _lib.load()
    if not getattr(lib, "_lr_declared", False):
        lib.logreg_loss.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int,
                                    ctypes.c_double, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
        lib.logreg_loss.restype = ctypes.c_int
        lib.logreg_loss_blocks.restype = ctypes.c_int
        lib._lr_declared = True
    assert A.is_cuda and A.dtype == torch.float32 and A.is_contiguous() and y.dtype == torch.float32
    assert x.dtype == torch.float64 and x.is_contiguous()
    n, d = A.shape
    scratch = torch.empty(lib.logreg_loss_blocks() + 2, dtype=torch.float64, device=A.device)
    out = torch.empty(1, dtype=torch.float64, device=A.device)
    _lib.check(lib.logreg_loss(_lib.ptr(A), _lib.ptr(y), _lib.ptr(x), n, d, float(lam), _lib.ptr(scratch), _lib.ptr(out),
                               _lib.stream_ptr()), "logreg_loss")
    return float(out)
