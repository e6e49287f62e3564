"""Fused training-mode BatchNorm (+ residual add) (+ ReLU) on NHWC fp32 tensors
(``csrc/bn_nhwc.cu``).  ``bn_act(bn_module, x, residual=None, relu=True)`` is what the model
blocks call; it uses the fused kernels for channels_last CUDA fp32 tensors in training mode
when the native path is enabled and the plain PyTorch composition otherwise."""
from __future__ import annotations

import ctypes

import torch
import torch.nn.functional as F

from . import _lib


class BnArgsC(ctypes.Structure):
    _fields_ = [(n, ctypes.c_void_p) for n in (
        "x", "dy", "y", "residual", "gamma", "beta", "out", "out2", "mean", "invstd", "running_mean", "running_var",
        "dgamma", "dbeta", "partial", "counter")] + [
        ("P", ctypes.c_int), ("C", ctypes.c_int), ("relu", ctypes.c_int), ("eps", ctypes.c_float),
        ("momentum", ctypes.c_float), ("n_partials", ctypes.c_int), ("fused_finalize", ctypes.c_int)]


_scratch = {}


def _lib_bn():
    lib = _lib.load()
    if not getattr(lib, "_bn_declared", False):
        for name in ("bn_forward", "bn_backward"):
            fn = getattr(lib, name)
            fn.argtypes = [ctypes.POINTER(BnArgsC), ctypes.c_void_p]
            fn.restype = ctypes.c_int
        lib.bn_forward_partials.argtypes = [ctypes.POINTER(BnArgsC), ctypes.c_int, ctypes.c_void_p]
        lib.bn_forward_partials.restype = ctypes.c_int
        lib.bn_backward_partials.argtypes = [ctypes.POINTER(BnArgsC), ctypes.c_int, ctypes.c_void_p]
        lib.bn_backward_partials.restype = ctypes.c_int
        lib.bn_reduce_grid.argtypes = [ctypes.c_int, ctypes.c_int]
        lib.bn_reduce_grid.restype = ctypes.c_int
        lib.bn_last_error.restype = ctypes.c_int
        lib.bn_args_size.restype = ctypes.c_int
        assert lib.bn_args_size() == ctypes.sizeof(BnArgsC)
        for name in ("bn16_forward", "bn16_backward"):
            fn = getattr(lib, name)
            fn.argtypes = [ctypes.POINTER(BnArgsC), ctypes.c_void_p]
            fn.restype = ctypes.c_int
        for name in ("bn16_supported", "bn16_reduce_grid"):
            fn = getattr(lib, name)
            fn.argtypes = [ctypes.c_int, ctypes.c_int]
            fn.restype = ctypes.c_int
        lib.bn16_last_error.argtypes = []
        lib.bn16_last_error.restype = ctypes.c_int
        lib._bn_declared = True
    return lib


def _get_scratch(device, P, C, lib):
    """Per-device scratch for the partial sums (one stream at a time uses it: kernels of one
    training step are ordered on a single stream)."""
    need = lib.bn_reduce_grid(P, C) * 2 * C
    key = device.index
    buf = _scratch.get(key)
    if buf is None or buf[0].numel() < need:
        buf = (torch.empty(max(need, 1 << 16), dtype=torch.float32, device=device),
               torch.zeros(1, dtype=torch.int32, device=device))
        _scratch[key] = buf
    return buf


def _get_scratch16(device, lib):
    """Partial-sum rows of the bf16 kernels: allocated once per device at the largest size the kernels can
    ask for (4 CTAs per SM x 2 x 2048 channels), so that a captured graph never sees it replaced."""
    key = (device.index, "bf16")
    buf = _scratch.get(key)
    if buf is None:
        sms = torch.cuda.get_device_properties(device).multi_processor_count
        buf = _scratch[key] = torch.empty(4 * sms * 2 * 2048, dtype=torch.float32, device=device)
    return buf


def supported16(x, C) -> bool:
    """bf16 activations (an autocast ImageNet ResNet): ``csrc/bn_nhwc_bf16.cu``."""
    return (x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 4 and x.numel() < 2 ** 31
            and x.is_contiguous(memory_format=torch.channels_last) and x.data_ptr() % 16 == 0
            and bool(_lib_bn().bn16_supported(x.numel() // C, C)))


class _BnAct16Fn(torch.autograd.Function):
    """``relu(bn(x) + residual)`` on bf16 NHWC tensors: three kernels each way (partial sums, finalize,
    elementwise) instead of the library's statistics / transform kernels plus add and ReLU kernels."""

    @staticmethod
    def forward(ctx, x, gamma, beta, residual, running_mean, running_var, relu, momentum, eps):
        lib = _lib_bn()
        N, C, H, W = x.shape
        y = torch.empty_like(x)
        mean = torch.empty(C, dtype=torch.float32, device=x.device)
        invstd = torch.empty_like(mean)
        a = BnArgsC()
        a.x, a.gamma, a.beta, a.out = x.data_ptr(), gamma.data_ptr(), beta.data_ptr(), y.data_ptr()
        a.residual = residual.data_ptr() if residual is not None else 0
        a.mean, a.invstd = mean.data_ptr(), invstd.data_ptr()
        a.running_mean = running_mean.data_ptr() if running_mean is not None else 0
        a.running_var = running_var.data_ptr() if running_var is not None else 0
        a.partial = _get_scratch16(x.device, lib).data_ptr()
        a.P, a.C, a.relu, a.eps, a.momentum = N * H * W, C, int(relu), float(eps), float(momentum)
        rc = lib.bn16_forward(ctypes.byref(a), _lib.stream_ptr())
        if rc != 0:
            raise RuntimeError(f"bn16_forward failed ({rc})")
        _lib.count(3)
        ctx.save_for_backward(x, y, gamma, beta, mean, invstd)
        ctx.relu, ctx.has_res = bool(relu), residual is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        lib = _lib_bn()
        x, y, gamma, beta, mean, invstd = ctx.saved_tensors
        N, C, H, W = x.shape
        if dy.dtype != x.dtype:
            dy = dy.to(x.dtype)
        dy = dy.contiguous(memory_format=torch.channels_last)
        dx = torch.empty_like(x)
        dres = torch.empty_like(x) if (ctx.has_res and ctx.relu) else None
        dgamma = torch.empty(C, dtype=torch.float32, device=x.device)
        dbeta = torch.empty_like(dgamma)
        a = BnArgsC()
        a.x, a.dy, a.y, a.gamma = x.data_ptr(), dy.data_ptr(), y.data_ptr(), gamma.data_ptr()
        a.out, a.out2 = dx.data_ptr(), dres.data_ptr() if dres is not None else 0
        a.mean, a.invstd, a.dgamma, a.dbeta = mean.data_ptr(), invstd.data_ptr(), dgamma.data_ptr(), dbeta.data_ptr()
        a.partial = _get_scratch16(x.device, lib).data_ptr()
        a.beta = beta.data_ptr()
        # ReLU without a residual: the kernels recompute the mask from x and never read y
        a.P, a.C, a.relu = N * H * W, C, (2 if (ctx.relu and not ctx.has_res) else int(ctx.relu))
        rc = lib.bn16_backward(ctypes.byref(a), _lib.stream_ptr())
        if rc != 0:
            raise RuntimeError(f"bn16_backward failed ({rc})")
        _lib.count(3)
        if ctx.has_res and dres is None:
            dres = dy   # no ReLU: the skip gradient is the incoming gradient itself
        return dx, dgamma.to(gamma.dtype), dbeta.to(gamma.dtype), dres, None, None, None, None, None


def last_error() -> int:
    """Non-zero when a grid barrier of the one-kernel backward ran out of its wait budget."""
    return _lib_bn().bn_last_error()


def last_error16() -> int:
    """1 when a wait on the copy ring of a bf16 kernel ran out since the last call."""
    return _lib_bn().bn16_last_error()


def supported(x, C) -> bool:
    return (x.is_cuda and x.dtype == torch.float32 and x.dim() == 4 and C % 4 == 0 and (C // 4) <= 256
            and 256 % (C // 4) == 0 and x.is_contiguous(memory_format=torch.channels_last))


class _BnActFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gamma, beta, residual, running_mean, running_var, relu, momentum, eps, stats=None,
                fold_res=False):
        lib = _lib_bn()
        N, C, H, W = x.shape
        P = N * H * W
        y = torch.empty_like(x)  # channels_last preserved
        mean = torch.empty(C, dtype=torch.float32, device=x.device)
        invstd = torch.empty_like(mean)
        partial, counter = _get_scratch(x.device, P, C, lib)
        a = BnArgsC()
        a.x, a.gamma, a.beta, a.out = x.data_ptr(), gamma.data_ptr(), beta.data_ptr(), y.data_ptr()
        a.residual = residual.data_ptr() if residual is not None else 0
        a.mean, a.invstd = mean.data_ptr(), invstd.data_ptr()
        a.running_mean = running_mean.data_ptr() if running_mean is not None else 0
        a.running_var = running_var.data_ptr() if running_var is not None else 0
        a.partial, a.counter = partial.data_ptr(), counter.data_ptr()
        a.P, a.C, a.relu, a.eps, a.momentum = P, C, int(relu), float(eps), float(momentum)
        if stats is not None:
            # per-CTA (sum, sum of squares) rows left by the producing convolution's epilogue
            a.partial = stats.data_ptr()
            rc = lib.bn_forward_partials(ctypes.byref(a), stats.shape[0], _lib.stream_ptr())
            _lib.count(1)
        else:
            rc = lib.bn_forward(ctypes.byref(a), _lib.stream_ptr())
            _lib.count(2)
        if rc != 0:
            raise RuntimeError(f"bn_forward failed ({rc})")
        ctx.save_for_backward(x, y, gamma, mean, invstd)
        ctx.relu, ctx.has_res = bool(relu), residual is not None
        # the skip gradient is handed to the block's first convolution (added in its epilogue)
        ctx.fold_res = bool(fold_res) and residual is not None
        ctx.res_key = residual.data_ptr() if ctx.fold_res else None
        if relu:
            # the consumer of y may fold this layer's backward sums into its input-gradient epilogue
            from .conv import FUSION

            if FUSION.enabled:
                FUSION.bn_of_output[y.data_ptr()] = (y, x, mean, invstd)
        return y

    @staticmethod
    def backward(ctx, dy):
        lib = _lib_bn()
        x, y, gamma, mean, invstd = ctx.saved_tensors
        N, C, H, W = x.shape
        P = N * H * W
        from .conv import FUSION

        dy = dy.contiguous(memory_format=torch.channels_last)
        hint = FUSION.masked.pop(dy.data_ptr(), None) if ctx.relu else None
        if hint is not None and hint[0].shape != dy.shape:
            hint = None
        dx = torch.empty_like(x)
        dgamma = torch.empty(C, dtype=torch.float32, device=x.device)
        dbeta = torch.empty_like(dgamma)
        partial, counter = _get_scratch(x.device, P, C, lib)
        a = BnArgsC()
        a.x, a.dy, a.y, a.gamma = x.data_ptr(), dy.data_ptr(), y.data_ptr(), gamma.data_ptr()
        a.out = dx.data_ptr()
        a.mean, a.invstd, a.dgamma, a.dbeta = mean.data_ptr(), invstd.data_ptr(), dgamma.data_ptr(), dbeta.data_ptr()
        a.partial, a.counter = partial.data_ptr(), counter.data_ptr()
        a.P, a.C, a.relu = P, C, int(ctx.relu)
        if hint is not None:
            # dy comes from an input-gradient epilogue that applied this layer's ReLU mask and left the
            # two backward sums as per-CTA rows: one elementwise kernel; the skip gradient is dy itself
            dres = dy if ctx.has_res else None
            a.partial = hint[1].data_ptr()
            rc = lib.bn_backward_partials(ctypes.byref(a), hint[1].shape[0], _lib.stream_ptr())
            _lib.count(1)
        else:
            dres = torch.empty_like(x) if ctx.has_res else None
            a.out2 = dres.data_ptr() if dres is not None else 0
            rc = lib.bn_backward(ctypes.byref(a), _lib.stream_ptr())
            _lib.count(2)
        if rc != 0:
            raise RuntimeError(f"bn_backward failed ({rc})")
        if ctx.fold_res:
            FUSION.pending_res[ctx.res_key] = (dy, dres)
            FUSION.clear_after_backward()
            dres = None
        return dx, dgamma, dbeta, dres, None, None, None, None, None, None, None


def bn_act(bn, x, residual=None, relu=True, stats=None, fold_res=False):
    """``relu(bn(x) + residual)`` with one fused kernel pair when possible.  ``stats``: rows of
    per-channel (sum, sum of squares) partials of ``x`` from its producer (``conv_bn_act``)."""
    from . import nn as native_nn

    if (native_nn.native_enabled("bn") and bn.training and bn.track_running_stats is not None
            and supported(x, bn.num_features) and bn.affine
            and (residual is None or (residual.shape == x.shape and residual.is_contiguous(memory_format=torch.channels_last)))):
        if bn.track_running_stats and bn.num_batches_tracked is not None and not getattr(bn, "_fused_counter", False):
            bn.num_batches_tracked.add_(1)
        mom = bn.momentum if bn.momentum is not None else 0.1
        rm = bn.running_mean if bn.track_running_stats else None
        rv = bn.running_var if bn.track_running_stats else None
        return _BnActFn.apply(x, bn.weight, bn.bias, residual, rm, rv, relu, mom, bn.eps, stats, fold_res)
    if (native_nn.native_enabled("bn") and bn.training and bn.track_running_stats is not None and bn.affine
            and stats is None and not fold_res and bn.weight.dtype == torch.float32 and supported16(x, bn.num_features)
            and (residual is None or (residual.shape == x.shape and residual.dtype == x.dtype
                                      and residual.is_contiguous(memory_format=torch.channels_last)))):
        if bn.track_running_stats and bn.num_batches_tracked is not None and not getattr(bn, "_fused_counter", False):
            bn.num_batches_tracked.add_(1)
        mom = bn.momentum if bn.momentum is not None else 0.1
        rm = bn.running_mean if bn.track_running_stats else None
        rv = bn.running_var if bn.track_running_stats else None
        return _BnAct16Fn.apply(x, bn.weight, bn.bias, residual, rm, rv, relu, mom, bn.eps)
    out = stock_forward(bn, x)
    if residual is not None:
        out = out + residual
    return F.relu(out, inplace=True) if relu else out


def fold_residual_ok(conv, x) -> bool:
    """True when ``conv`` (the first convolution of a residual block whose skip connection is ``x``
    itself) will run the native kernels and can add the skip gradient in its input-gradient epilogue."""
    from . import nn as native_nn

    if not (native_nn.native_enabled("conv") and native_nn.native_enabled("bn") and x.is_cuda and x.requires_grad
            and torch.is_grad_enabled()):
        return False
    from .conv import FUSION, conv_supported

    if not FUSION.enabled:
        return False

    return conv.in_channels != 3 and conv_supported(conv, x)


def conv_bn_act(conv, bn, x, residual=None, relu=True, fold_res=False, fold_ds=False):
    """``relu(bn(conv(x)) + residual)``.  When both layers run their native kernels the convolution
    epilogue also produces the batch statistics, so the batch-norm needs no reduction pass.
    ``fold_res`` (decided by the block with ``fold_residual_ok``): the gradient of the skip connection
    travels from this block's last batch-norm to its first convolution outside autograd.  ``fold_ds``
    (``fold_shortcut_ok``): the 1x1 shortcut's input gradient is computed by the block's strided 3x3
    convolution."""
    from . import nn as native_nn

    if (native_nn.native_enabled("conv") and native_nn.native_enabled("bn") and bn.training and x.is_cuda
            and bn.affine and bn.track_running_stats is not None and torch.is_grad_enabled()):
        from .conv import any_conv_supported, conv2d_native

        if (any_conv_supported(conv, x) and (conv.out_channels // 4) <= 256
                and 256 % (conv.out_channels // 4) == 0):
            y, stats = conv2d_native(conv, x, want_stats=True, fold_res=fold_res and residual is None, fold_ds=fold_ds)
            return bn_act(bn, y, residual, relu, stats=stats, fold_res=fold_res)
    if fold_res or fold_ds:
        raise RuntimeError("a backward fusion was requested for a layer pair that does not run the native kernels")
    return bn_act(bn, conv(x), residual, relu)


def stock_forward(bn, x):
    """The library batch-norm of a module (also for our subclass, whose ``forward`` routes here)."""
    out = torch.nn.modules.batchnorm._BatchNorm.forward(bn, x)
    if getattr(bn, "_fused_counter", False) and bn.training and bn.track_running_stats:
        bn.num_batches_tracked.sub_(1)  # the library op counted this batch; BnCounters.tick() counts it too
    return out


class BnCounters:
    """The ``num_batches_tracked`` buffers of every batch-norm layer of a model as views of ONE
    int64 tensor, advanced by a single add per training step (the stock module launches one
    increment kernel per layer per step).  ``state_dict`` / ``load_state_dict`` keep working on
    the per-layer views."""

    def __init__(self, model):
        self.model = model
        self.flat = None
        self._fuse()

    def _fuse(self):
        from .nn import BatchNorm2d  # only our subclass: its forward compensates on the library path

        self.mods = [m for m in self.model.modules()
                     if isinstance(m, BatchNorm2d) and m.track_running_stats and m.num_batches_tracked is not None]
        if not self.mods:
            self.flat = None
            return
        self.flat = torch.stack([m.num_batches_tracked.detach() for m in self.mods])
        for i, m in enumerate(self.mods):
            m._buffers["num_batches_tracked"] = self.flat[i]
            m._fused_counter = True

    def tick(self):
        if self.flat is None:
            return
        if self.mods[0].num_batches_tracked.data_ptr() != self.flat.data_ptr():
            self._fuse()  # the module was moved / reloaded: its buffers are no longer our views
        self.flat.add_(1)

    def release(self):
        for m in self.mods:
            m._fused_counter = False
