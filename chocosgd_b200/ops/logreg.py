"""Bindings of the convex-simulator kernels (``csrc/logreg.cu``): the full-data loss and one whole
simulator iteration (stochastic gradient of every node + gossip step + column compressor) per launch."""
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


class LogregIterArgsC(ctypes.Structure):
    _fields_ = [(n, ctypes.c_void_p) for n in ("A", "y", "rows", "x_in", "xh_in", "x_out", "xh_out", "W")] + [
        ("lr", ctypes.c_double), ("lam", ctypes.c_double), ("gamma", ctypes.c_double), ("t", ctypes.c_longlong),
        ("n", ctypes.c_int), ("d", ctypes.c_int), ("method", ctypes.c_int), ("quant", ctypes.c_int),
        ("k", ctypes.c_int), ("levels", ctypes.c_int), ("seed", ctypes.c_uint32)]


METHODS = {"plain": 0, "choco": 1, "dcd-psgd": 2, "ecd-psgd": 3}
QUANTS = {"full": 0, "top": 1, "random-biased": 2, "random-unbiased": 3, "qsgd-biased": 4, "qsgd-unbiased": 5}


def iter_supported(n_nodes: int, d: int) -> bool:
    return 1 <= n_nodes <= 64 and 1 <= d <= 12288


class LogregIterator:
    """One simulator iteration per call: state ``x``, ``x_hat`` are ``[n, d]`` fp64 device tensors
    (node-major); two copies of each are kept and swapped (neighbours read the old state while a
    node writes its new one)."""

    def __init__(self, A32, y32, W, x0, method, quantization, k=None, levels=None, lam=0.0, gamma=0.0, seed=0):
        lib = _lib.load()
        if not getattr(lib, "_lri_declared", False):
            lib.logreg_iter.argtypes = [ctypes.POINTER(LogregIterArgsC), ctypes.c_void_p]
            lib.logreg_iter.restype = ctypes.c_int
            lib.logreg_iter_args_size.restype = ctypes.c_int
            assert lib.logreg_iter_args_size() == ctypes.sizeof(LogregIterArgsC), "LogregIterArgs layout mismatch"
            lib._lri_declared = True
        self.lib = lib
        self.A, self.y = A32.contiguous(), y32.contiguous()
        self.W = W.to(torch.float64).contiguous()
        n, d = x0.shape
        assert iter_supported(n, d) and self.A.shape[1] == d
        self.x = [x0.to(torch.float64).contiguous().clone(), torch.empty_like(x0, dtype=torch.float64)]
        self.xh = [self.x[0].clone(), torch.empty_like(self.x[0])]
        self.cur = 0
        a = LogregIterArgsC()
        a.A, a.y, a.W = self.A.data_ptr(), self.y.data_ptr(), self.W.data_ptr()
        a.n, a.d, a.method, a.quant = n, d, METHODS[method], QUANTS[quantization]
        a.k, a.levels = int(k or 0), int(levels or 0)
        a.lam, a.gamma, a.seed = float(lam), float(gamma), int(seed) & 0xFFFFFFFF
        self.args = a

    @property
    def state(self):
        return self.x[self.cur], self.xh[self.cur]

    def step(self, rows: torch.Tensor, lr: float, t: int):
        a, c = self.args, self.cur
        a.rows = rows.data_ptr()
        a.x_in, a.xh_in = self.x[c].data_ptr(), self.xh[c].data_ptr()
        a.x_out, a.xh_out = self.x[1 - c].data_ptr(), self.xh[1 - c].data_ptr()
        a.lr, a.t = float(lr), int(t)
        _lib.check(self.lib.logreg_iter(ctypes.byref(a), _lib.stream_ptr()), "logreg_iter")
        _lib.count(1)
        self.cur = 1 - c
