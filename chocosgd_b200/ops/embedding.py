"""Embedding lookup and gradient (``csrc/embedding.cu``), the language model's input layer
(``dl_code/pcode/models/rnn_lm.py:29, 53``).

Forward is a row gather.  The gradient is scattered, in a reproducible order and without a sort, into a
``[V, D]`` tensor.  With tied weights (the decoder shares the matrix) the module runs in *deferred* mode:
the autograd function hands back no gradient of its own; a post-accumulate hook on the shared parameter adds
the looked-up rows' gradients in place into the gradient the decoder produced, so the dense tensor of zeros,
the scatter into it and the 2 x 86 MB add of the two gradients never happen."""
from __future__ import annotations

import ctypes

import torch

from . import _lib


def _declare():
    lib = _lib.load()
    if not getattr(lib, "_emb_declared", False):
        vp, i = ctypes.c_void_p, ctypes.c_int
        lib.embedding_forward.argtypes = [vp, vp, vp, i, i, i, vp]
        lib.embedding_backward_accumulate.argtypes = [vp, vp, vp, i, i, i, vp]
        for n in ("embedding_forward", "embedding_backward_accumulate", "embedding_last_error"):
            getattr(lib, n).restype = i
        lib._emb_declared = True
    return lib


def embedding_supported(m, idx) -> bool:
    w = m.weight
    return (idx.is_cuda and idx.dtype == torch.int64 and w.is_cuda and w.dtype == torch.float32 and w.is_contiguous()
            and m.padding_idx is None and m.max_norm is None and not m.sparse and not m.scale_grad_by_freq
            and 0 < idx.numel() <= 65536)


def last_error() -> int:
    return _declare().embedding_last_error()


def scatter_add_rows(grad: torch.Tensor, idx: torch.Tensor, dy: torch.Tensor):
    """``grad[idx[i]] += dy[i]`` for all i, in place, in a fixed order."""
    lib = _declare()
    v, d = grad.shape
    _lib.check(lib.embedding_backward_accumulate(_lib.ptr(idx), _lib.ptr(dy), _lib.ptr(grad), idx.numel(), d, v,
                                                 _lib.stream_ptr()), "embedding_backward_accumulate")
    _lib.count(1)


class _Pending:
    """Gradients of look-ups waiting for the shared parameter's gradient (deferred mode), per parameter."""

    def __init__(self):
        self.items = {}

    def add(self, weight, idx, dy):
        self.items.setdefault(id(weight), []).append((idx, dy))

    def flush_into(self, weight):
        todo = self.items.pop(id(weight), None)
        if not todo:
            return
        if weight.grad is None:
            weight.grad = torch.zeros_like(weight)
        g = weight.grad
        if not (g.dtype == torch.float32 and g.is_contiguous()):
            raise RuntimeError("deferred embedding gradient needs a contiguous fp32 .grad")
        for idx, dy in todo:
            scatter_add_rows(g, idx, dy)


PENDING = _Pending()


class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, idx, weight, deferred):
        lib = _declare()
        v, d = weight.shape
        flat = idx.reshape(-1).contiguous()
        out = torch.empty(flat.numel(), d, dtype=torch.float32, device=weight.device)
        _lib.check(lib.embedding_forward(_lib.ptr(flat), _lib.ptr(weight), _lib.ptr(out), flat.numel(), d, v,
                                         _lib.stream_ptr()), "embedding_forward")
        _lib.count(1)
        ctx.save_for_backward(flat)
        ctx.weight, ctx.deferred, ctx.shape = weight, bool(deferred), (v, d)
        return out.view(*idx.shape, d)

    @staticmethod
    def backward(ctx, dy):
        (flat,) = ctx.saved_tensors
        v, d = ctx.shape
        dy2 = dy.reshape(-1, d).contiguous()
        if ctx.deferred:
            PENDING.add(ctx.weight, flat, dy2)      # added into the shared gradient by the parameter's hook
            return None, None, None
        grad = torch.zeros(v, d, dtype=torch.float32, device=dy.device)
        scatter_add_rows(grad, flat, dy2)
        return None, grad, None


def embedding_native(m, idx):
    return _EmbeddingFn.apply(idx, m.weight, bool(getattr(m, "deferred_grad", False)))


def enable_deferred_grad(m):
    """Tied weights: ``m.weight`` also receives a gradient from another layer in every backward pass.  Registers
    the hook that adds the look-ups' gradients into that gradient in place."""
    if getattr(m, "_deferred_hook", None) is None:
        w = m.weight
        m._deferred_hook = w.register_post_accumulate_grad_hook(lambda p: PENDING.flush_into(p))
    m.deferred_grad = True
