"""Fused softmax cross-entropy + gradient + top-1 / top-5 accuracy (``csrc/cross_entropy.cu``).

``cross_entropy(logits, target)`` returns ``(loss, stats)``: the mean loss (differentiable, 0-d)
and a 4-vector ``[loss, top1 %, top5 %, counted rows]`` on the device.  The gradient with
respect to the logits is produced by the forward kernel; the backward pass only scales it by
the incoming gradient.  Replaces ``log_softmax`` + ``nll_loss`` + ``topk`` + comparisons + sums of
the criterion and metric calls of the reference's loop
(``dl_code/pcode/distributed_running_cv.py:52-56``, ``dl_code/pcode/create_metrics.py:31-48``)."""
from __future__ import annotations

import ctypes

import torch

from . import _lib


_SCRATCH = {}


def _declare():
    lib = _lib.load()
    if not getattr(lib, "_ce_declared", False):
        vp, i = ctypes.c_void_p, ctypes.c_int
        lib.cross_entropy_fused.argtypes = [vp, vp, vp, vp, vp, vp, i, i, i, vp]
        lib.cross_entropy_fused.restype = i
        lib.cross_entropy_fused_ld.argtypes = [vp, vp, vp, vp, vp, vp, i, i, ctypes.c_longlong, i, vp]
        lib.cross_entropy_fused_ld.restype = i
        lib._ce_declared = True
    return lib


def supported(logits: torch.Tensor, target: torch.Tensor) -> bool:
    return (logits.is_cuda and logits.dtype == torch.float32 and logits.dim() == 2 and target.dim() == 1
            and target.dtype == torch.int64 and target.numel() == logits.shape[0] and logits.numel() > 0)


class _CrossEntropyFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, target, may_ignore):
        lib = _declare()
        # rows may be padded (the output of the native GEMM has 16-byte aligned rows): no copy then,
        # and the gradient gets the same row pitch so that it can go back into the GEMMs as it is
        z = logits if (logits.stride(1) == 1 and logits.stride(0) >= logits.shape[1]) else logits.contiguous()
        B, C = z.shape
        ld = z.stride(0)
        dz = torch.empty_strided((B, C), (ld, 1), dtype=z.dtype, device=z.device) if ld != C else torch.empty_like(z)
        key = (z.device, B)
        scratch = _SCRATCH.get(key)
        if scratch is None:  # zeroed once: the arrival counter resets itself
            scratch = _SCRATCH[key] = torch.zeros(2 * B + 4, dtype=torch.int32, device=z.device)
        stats = torch.empty(4, dtype=torch.float32, device=z.device)
        loss = torch.empty((), dtype=torch.float32, device=z.device)
        _lib.check(lib.cross_entropy_fused_ld(_lib.ptr(z), _lib.ptr(target.contiguous()), _lib.ptr(dz),
                                              _lib.ptr(scratch), _lib.ptr(stats), _lib.ptr(loss), B, C, ld,
                                              int(bool(may_ignore)), _lib.stream_ptr()), "cross_entropy_fused")
        _lib.count(2 if may_ignore else 1)
        ctx.save_for_backward(dz)
        ctx.set_materialize_grads(False)  # no zero tensor for the statistics output
        ctx.mark_non_differentiable(stats)
        return loss, stats

    @staticmethod
    def backward(ctx, g_loss, _g_stats):
        (dz,) = ctx.saved_tensors
        if g_loss is None:
            return None, None, None
        return dz * g_loss, None, None


def cross_entropy(logits, target, may_ignore: bool = False):
    return _CrossEntropyFn.apply(logits, target, may_ignore)


def criterion_is_plain_ce(criterion) -> bool:
    """True for ``nn.CrossEntropyLoss`` with mean reduction, no class weights, no label smoothing."""
    return (isinstance(criterion, torch.nn.CrossEntropyLoss) and criterion.reduction == "mean"
            and criterion.weight is None and getattr(criterion, "label_smoothing", 0.0) == 0.0)
