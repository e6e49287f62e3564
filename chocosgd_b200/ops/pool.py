"""3x3 / stride 2 / pad 1 max pooling on channels_last tensors (``csrc/maxpool_nhwc.cu``): the layer behind
the ImageNet ResNet stem (``dl_code/pcode/models/resnet.py:196, 223``).  The forward keeps one byte per output
element (position of the maximum inside its window) instead of the library's 64-bit indices; the backward is a
gather (every input-gradient element written once, no atomics, no zero fill)."""
from __future__ import annotations

import ctypes

import torch

from . import _lib


def _declare():
    lib = _lib.load()
    if not getattr(lib, "_pool_declared", False):
        vp, i = ctypes.c_void_p, ctypes.c_int
        lib.maxpool3x3s2_supported.argtypes = [i, i, i, i, i]
        lib.maxpool3x3s2_forward.argtypes = [vp, vp, vp, i, i, i, i, i, vp]
        lib.maxpool3x3s2_backward.argtypes = [vp, vp, vp, i, i, i, i, i, vp]
        for n in ("maxpool3x3s2_supported", "maxpool3x3s2_forward", "maxpool3x3s2_backward"):
            getattr(lib, n).restype = i
        lib._pool_declared = True
    return lib


_DTYPES = {torch.float32: 0, torch.bfloat16: 1}


def maxpool_supported(m, x) -> bool:
    def pair(v):
        return tuple(v) if isinstance(v, (tuple, list)) else (v, v)

    if not (x.is_cuda and x.dim() == 4 and x.dtype in _DTYPES and x.is_contiguous(memory_format=torch.channels_last)):
        return False
    if pair(m.kernel_size) != (3, 3) or pair(m.stride) != (2, 2) or pair(m.padding) != (1, 1) or pair(m.dilation) != (1, 1):
        return False
    if m.ceil_mode or m.return_indices or x.numel() >= 2 ** 31:
        return False
    n, c, h, w = x.shape
    return bool(_declare().maxpool3x3s2_supported(n, h, w, c, _DTYPES[x.dtype]))


class _MaxPoolFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        lib = _declare()
        n, c, h, w = x.shape
        ho, wo = (h + 1) // 2, (w + 1) // 2
        y = torch.empty((n, c, ho, wo), dtype=x.dtype, device=x.device, memory_format=torch.channels_last)
        idx = torch.empty((n, ho, wo, c), dtype=torch.uint8, device=x.device)
        _lib.check(lib.maxpool3x3s2_forward(_lib.ptr(x), _lib.ptr(y), _lib.ptr(idx), n, h, w, c, _DTYPES[x.dtype],
                                            _lib.stream_ptr()), "maxpool3x3s2_forward")
        _lib.count(1)
        ctx.save_for_backward(idx)
        ctx.shape = (n, c, h, w)
        return y

    @staticmethod
    def backward(ctx, dy):
        lib = _declare()
        (idx,) = ctx.saved_tensors
        n, c, h, w = ctx.shape
        dy = dy.contiguous(memory_format=torch.channels_last)
        dx = torch.empty((n, c, h, w), dtype=dy.dtype, device=dy.device, memory_format=torch.channels_last)
        _lib.check(lib.maxpool3x3s2_backward(_lib.ptr(dy), _lib.ptr(idx), _lib.ptr(dx), n, h, w, c, _DTYPES[dy.dtype],
                                             _lib.stream_ptr()), "maxpool3x3s2_backward")
        _lib.count(1)
        return dx


def maxpool_native(x):
    return _MaxPoolFn.apply(x)
