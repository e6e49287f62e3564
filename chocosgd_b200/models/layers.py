"""Layer factory shared by all model definitions.

Models never instantiate ``torch.nn`` compute layers directly: they ask this module, which
returns the framework's layer classes (``ops/nn.py``).  Those run the hand-written sm_100a
kernels when the native path is enabled and the tensors live on a CUDA device, and the
plain PyTorch ops otherwise (CPU tests, unsupported shapes)."""
from __future__ import annotations

import math

import torch.nn as nn

from ..ops import nn as native_nn

Conv2d = native_nn.Conv2d
BatchNorm2d = native_nn.BatchNorm2d
BatchNorm1d = nn.BatchNorm1d
Linear = native_nn.Linear
ReLU = nn.ReLU
MaxPool2d = native_nn.MaxPool2d
AvgPool2d = nn.AvgPool2d
Dropout = nn.Dropout
Embedding = native_nn.Embedding
LSTM = native_nn.LSTM


def bn_act(bn, x, residual=None, relu=True):
    """relu(bn(x) + residual): one fused kernel pair on the native path."""
    from ..ops.bn import bn_act as _f

    return _f(bn, x, residual, relu)


def conv_bn_act(conv, bn, x, residual=None, relu=True, fold_res=False, fold_ds=False):
    """relu(bn(conv(x)) + residual); on the native path the convolution epilogue also yields the
    batch statistics, so no reduction pass runs over the activation."""
    from ..ops.bn import conv_bn_act as _f

    return _f(conv, bn, x, residual, relu, fold_res, fold_ds)


def fold_shortcut_ok(conv, shortcut, x) -> bool:
    """Whether a down-sampling block's strided convolution ``conv`` can compute the input gradient of the
    block's (1x1 convolution, batch-norm) ``shortcut`` in the same launch as its own."""
    import torch.nn as nn

    if not (x.is_cuda and isinstance(shortcut, nn.Sequential) and len(shortcut) == 2
            and isinstance(shortcut[0], nn.Conv2d) and isinstance(shortcut[1], nn.BatchNorm2d)):
        return False
    from ..ops.conv import fold_shortcut_ok as _f

    return _f(conv, shortcut[0], x)


def fold_residual_ok(conv, x) -> bool:
    """Whether a residual block whose skip connection is ``x`` can hand the skip gradient to ``conv``'s
    input-gradient kernel (native kernels on, shape covered)."""
    if not x.is_cuda:
        return False
    from ..ops.bn import fold_residual_ok as _f

    return _f(conv, x)


def conv3x3(in_planes, out_planes, stride=1):
    return Conv2d(in_planes, out_planes, kernel_size=3, stride=stride, padding=1, bias=False)


def he_init(module: nn.Module, zero_linear_bias: bool = False):
    """conv ~ N(0, sqrt(2 / (kh kw c_out))), BN gamma = 1 beta = 0
    (``dl_code/pcode/models/resnet.py:130-140``)."""
    for m in module.modules():
        if isinstance(m, nn.Conv2d):
            n = m.kernel_size[0] * m.kernel_size[1] * m.out_channels
            m.weight.data.normal_(0, math.sqrt(2.0 / n))
        elif isinstance(m, nn.BatchNorm2d):
            m.weight.data.fill_(1)
            m.bias.data.zero_()
        elif zero_linear_bias and isinstance(m, nn.Linear) and m.bias is not None:
            m.bias.data.zero_()


def num_classes_of(dataset: str) -> int:
    if dataset in ("cifar10", "svhn", "mnist", "stl10") or dataset.startswith("synthetic_cifar10"):
        return 10
    if dataset == "cifar100":
        return 100
    if "imagenet" in dataset:
        return 1000
    if dataset in ("epsilon", "rcv1"):
        return 2
    if dataset.startswith("synthetic"):
        return 10
    raise ValueError(f"unknown dataset {dataset!r}")


def is_small_input(dataset: str) -> bool:
    return "imagenet" not in dataset or "downsampled" in dataset
