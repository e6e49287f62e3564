"""Fused classifier head: global average pooling + linear layer + softmax cross-entropy + top-1 / top-5,
one kernel forward and one backward (``csrc/head.cu``).

``head_loss(feat, weight, bias, target) -> (loss, stats)`` where ``feat`` is the last feature map
(``[B, C, H, W]`` in channels_last memory).  ``stats = [loss, top-1 %, top-5 %, counted rows]``.
The reference runs ``AvgPool2d(8)`` -> ``Linear`` -> ``CrossEntropyLoss`` plus the ``topk`` metric
(``dl_code/pcode/models/resnet.py:286-294``, ``dl_code/pcode/create_metrics.py:31-48``)."""
from __future__ import annotations

import ctypes

import torch

from . import _lib

_SCRATCH = {}


def _declare():
    lib = _lib.load()
    if not getattr(lib, "_head_declared", False):
        vp, i = ctypes.c_void_p, ctypes.c_int
        lib.head_supported.argtypes = [i, i, i]
        lib.head_forward.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, i, i, i, i, vp]
        lib.head_backward.argtypes = [vp, vp, vp, vp, vp, vp, vp, i, i, i, i, vp]
        for n in ("head_supported", "head_forward", "head_backward"):
            getattr(lib, n).restype = i
        lib._head_declared = True
    return lib


def supported(feat, weight, target) -> bool:
    if not (feat.is_cuda and feat.dtype == torch.float32 and feat.dim() == 4 and weight.dtype == torch.float32):
        return False
    if not feat.is_contiguous(memory_format=torch.channels_last) or not weight.is_contiguous():
        return False
    b, c, h, w = feat.shape
    return (target.dim() == 1 and target.dtype == torch.int64 and target.numel() == b and weight.shape[1] == c
            and bool(_declare().head_supported(h * w, c, weight.shape[0])))


class _HeadFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, feat, weight, bias, target):
        lib = _declare()
        b, c, h, w = feat.shape
        k = weight.shape[0]
        dev = feat.device
        pooled = torch.empty((b, c), dtype=torch.float32, device=dev)
        dz = torch.empty((b, k), dtype=torch.float32, device=dev)
        scratch = _SCRATCH.get((dev, b))
        if scratch is None:  # zeroed once: the arrival counter resets itself
            scratch = _SCRATCH[(dev, b)] = torch.zeros(2 * b + 4, dtype=torch.int32, device=dev)
        stats = torch.empty(4, dtype=torch.float32, device=dev)
        loss = torch.empty((), dtype=torch.float32, device=dev)
        _lib.check(lib.head_forward(_lib.ptr(feat), _lib.ptr(weight), _lib.ptr(bias), _lib.ptr(target.contiguous()),
                                    _lib.ptr(pooled), _lib.ptr(dz), _lib.ptr(scratch), _lib.ptr(stats), _lib.ptr(loss),
                                    b, h * w, c, k, _lib.stream_ptr()), "head_forward")
        _lib.count(1)
        ctx.save_for_backward(weight, pooled, dz)
        ctx.shape, ctx.has_bias = (b, c, h, w), bias is not None
        ctx.set_materialize_grads(False)
        ctx.mark_non_differentiable(stats)
        return loss, stats

    @staticmethod
    def backward(ctx, g_loss, _g_stats):
        if g_loss is None:
            return None, None, None, None
        lib = _declare()
        weight, pooled, dz = ctx.saved_tensors
        b, c, h, w = ctx.shape
        k = weight.shape[0]
        dfeat = torch.empty((b, c, h, w), dtype=torch.float32, device=weight.device, memory_format=torch.channels_last)
        dw = torch.empty_like(weight)
        db = torch.empty(k, dtype=torch.float32, device=weight.device) if ctx.has_bias else None
        g = g_loss.contiguous().float()
        _lib.check(lib.head_backward(_lib.ptr(weight), _lib.ptr(pooled), _lib.ptr(dz), _lib.ptr(g), _lib.ptr(dfeat),
                                     _lib.ptr(dw), _lib.ptr(db), b, h * w, c, k, _lib.stream_ptr()), "head_backward")
        _lib.count(1)
        return dfeat, dw, db, None


def head_loss(feat, weight, bias, target):
    return _HeadFn.apply(feat, weight, bias, target)
