"""Layer classes used by the model zoo.

Each class is a drop-in subclass of the ``torch.nn`` layer (same parameters, same
``state_dict`` keys).  ``set_native(True)`` routes the forward/backward of supported
shapes on CUDA tensors to the hand-written kernels; everything else (CPU, unsupported
shapes, ``set_native(False)``) runs the stock PyTorch op, which also serves as the numerics
reference in the tests."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

_NATIVE = {"linear": False, "conv": False, "lstm": False, "bn": False, "wgrad": False, "ce": False, "pool": False, "embed": False}


def set_native(enabled: bool = True, which=("linear", "conv", "lstm", "bn")):
    for k in which:
        _NATIVE[k] = bool(enabled)


def available_kinds():
    """Kinds of layers whose native kernels are built into this tree."""
    import importlib.util

    kinds = ["bn", "linear", "wgrad", "ce", "pool", "embed"]
    for kind, mod in (("conv", "conv"), ("lstm", "lstm")):
        if importlib.util.find_spec(f"{__package__}.{mod}") is not None:
            kinds.append(kind)
    return tuple(kinds)


#: kinds switched on by ``auto``: the ones measured faster than the library op inside a training
#: step.  ``linear`` takes only layers large enough to fill the machine (the language model's
#: decoder: fp32-grade products on the TF32 tensor cores against the library's fp32 FMA GEMM);
#: ``lstm`` (persistent recurrence kernels) is opt-in through ``set_native`` / ``--native_layers all``.
AUTO_KINDS = ("bn", "conv", "wgrad", "ce", "linear", "pool", "embed")


def configure_native(mode: str = "auto"):
    """Apply a ``--native_layers`` choice: auto = batch-norm + 3x3 convolution forward / input /
    weight gradient, all = every kind built into the tree, bn = batch-norm + linear, conv = bn +
    convolution forward / input gradient, off = library ops only."""
    set_native(False, which=tuple(_NATIVE))
    if mode in ("off", None) or not torch.cuda.is_available():
        return
    if mode == "bn":
        set_native(True, which=("bn", "linear", "ce"))
    elif mode == "conv":
        set_native(True, which=("bn", "linear", "conv", "ce"))
    elif mode == "all":
        set_native(True, which=available_kinds())
    else:
        set_native(True, which=tuple(k for k in AUTO_KINDS if k in available_kinds()))


def native_enabled(kind: str) -> bool:
    return _NATIVE[kind]


class Linear(nn.Linear):
    def forward(self, x):
        if _NATIVE["linear"] and x.is_cuda and x.dtype == torch.float32 and not torch.is_autocast_enabled():
            from .gemm import linear_native, linear_supported

            if linear_supported(x, self.weight):
                return linear_native(x, self.weight, self.bias)
        return F.linear(x, self.weight, self.bias)


class Conv2d(nn.Conv2d):
    def forward(self, x):
        if _NATIVE["conv"] and x.is_cuda:
            from .conv import any_conv_supported, conv2d_native, conv_stem_native, stem_conv_supported

            if any_conv_supported(self, x):
                return conv2d_native(self, x)
            if self.in_channels == 3 and stem_conv_supported(self, x):
                return conv_stem_native(self, x)
        return super().forward(x)


class Embedding(nn.Embedding):
    """``tie_to_other_gradient()``: the weight is shared with a layer that produces a dense gradient of it in
    every backward pass (tied decoder); the look-ups' gradient is then added into that gradient in place."""

    def tie_to_other_gradient(self):
        self._wants_deferred = True

    def forward(self, idx):
        if _NATIVE["embed"] and idx.is_cuda and torch.is_grad_enabled() == self.weight.requires_grad:
            from .embedding import embedding_native, embedding_supported, enable_deferred_grad

            if embedding_supported(self, idx):
                if getattr(self, "_wants_deferred", False) and self.training and not getattr(self, "deferred_grad", False):
                    enable_deferred_grad(self)
                return embedding_native(self, idx)
        return super().forward(idx)


class MaxPool2d(nn.MaxPool2d):
    def forward(self, x):
        if _NATIVE["pool"] and x.is_cuda:
            from .pool import maxpool_native, maxpool_supported

            if maxpool_supported(self, x):
                return maxpool_native(x)
        return super().forward(x)


class BatchNorm2d(nn.BatchNorm2d):
    def forward(self, x):
        from .bn import bn_act, stock_forward

        if _NATIVE["bn"] and x.is_cuda:
            return bn_act(self, x, None, relu=False)
        return stock_forward(self, x)


class LSTM(nn.LSTM):
    def forward(self, input, hx=None):
        if _NATIVE["lstm"] and input.is_cuda and input.dtype == torch.float32:
            from .lstm import lstm_native, lstm_supported

            if lstm_supported(self, input):
                return lstm_native(self, input, hx)
        if input.is_cuda:
            self.flatten_parameters()
        return super().forward(input, hx)
