"""Native convolution path: 3x3 / stride 1 / pad 1 NHWC fp32 convolutions run the persistent
tcgen05 implicit-GEMM kernel (``csrc/conv_sm100.cu``) for the forward pass (optionally with the
batch-norm statistics of its output) and for the input gradient (same kernel on dy with the flipped
filter).  Weight gradients: ``csrc/conv_wgrad16.cu`` for 16 channels, ``csrc/conv_wgrad_gen.cu`` for 32 / 64
channels and for the strided layers (``csrc/conv_wgrad_sm100.cu``, tcgen05, is opt-in), forked onto a
second stream.  The 3-channel first layer runs ``csrc/conv_first.cu``.  Strided 3x3 and 1x1
convolutions (first convolution of a stage, down-sampling shortcut) run the same persistent kernel
through a tensor map with element strides."""
from __future__ import annotations

import ctypes
import os

import torch

from . import _lib


def _declare():
    lib = _lib.load()
    if not getattr(lib, "_conv_declared", False):
        vp, i = ctypes.c_void_p, ctypes.c_int
        lib.conv3x3_tf32.argtypes = [vp, vp, vp, i, i, i, i, i, i, vp]
        lib.conv3x3_tf32.restype = i
        lib.conv3x3_supported.argtypes = [i, i, i, i, i]
        lib.conv3x3_supported.restype = i
        lib.conv_flip_weights.argtypes = [vp, vp, i, i, vp]
        lib.conv_flip_weights.restype = i
        lib.conv3x3_last_error.restype = i
        lib.conv3x3_wgrad_tf32.argtypes = [vp, vp, vp, vp, i, i, i, i, vp]
        lib.conv3x3_wgrad_parts.argtypes = [i, i, i]
        lib.conv3x3_wgrad_parts.restype = i
        lib.conv3x3_wgrad_tf32.restype = i
        lib.conv3x3_wgrad_supported.argtypes = [i, i, i, i, i]
        lib.conv3x3_wgrad_supported.restype = i
        lib.conv3x3_wgrad_last_error.restype = i
        lib.conv_flip_weights_multi.argtypes = [vp, i, i, vp]
        lib.conv_flip_weights_multi.restype = i
        lib.conv3x3_tf32_stats.argtypes = [vp, vp, vp, vp, i, i, i, i, i, vp]
        lib.conv3x3_tf32_stats.restype = i
        lib.conv3x3_grid.argtypes = [i, i, i, i]
        lib.conv3x3_grid.restype = i
        lib.conv3x3_wgrad16.argtypes = [vp, vp, vp, vp, i, i, i, vp]
        lib.conv3x3_wgrad16.restype = i
        lib.conv3x3_wgrad16_parts.argtypes = [i, i, i]
        lib.conv3x3_wgrad16_parts.restype = i
        lib.conv3x3_wgrad16_supported.argtypes = [i, i, i]
        lib.conv3x3_wgrad16_supported.restype = i
        lib.conv3x3_dgrad_fused.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, i, i, i, i, i, vp]
        lib.conv3x3_dgrad_fused.restype = i
        lib.conv_fwd_supported.argtypes = [i, i, i, i, i, i, i]
        lib.conv_fwd_supported.restype = i
        lib.conv_fwd_tf32.argtypes = [vp, vp, vp, vp, i, i, i, i, i, i, i, vp]
        lib.conv_fwd_tf32.restype = i
        lib.conv_wgrad_gen_parts.argtypes = [i, i, i, i, i, i, i]
        lib.conv_wgrad_gen_parts.restype = i
        lib.conv_wgrad_gen.argtypes = [vp, vp, vp, vp, i, i, i, i, i, i, i, vp]
        lib.conv_wgrad_gen.restype = i
        lib.conv3x3s2_dgrad_supported.argtypes = [i, i, i, i, i, i]
        lib.conv3x3s2_dgrad_supported.restype = i
        lib.conv3x3s2_dgrad_grid.argtypes = [i, i, i, i]
        lib.conv3x3s2_dgrad_grid.restype = i
        lib.conv3x3s2_dgrad_fused.argtypes = [vp] * 11 + [i] * 6 + [vp]
        lib.conv3x3s2_dgrad_fused.restype = i
        lib.conv_flip_entry_size.restype = i
        lib._conv_declared = True
    return lib


def conv_supported(m, x) -> bool:
    if not (x.is_cuda and x.dtype == torch.float32 and x.dim() == 4 and m.weight.dtype == torch.float32):
        return False
    if m.kernel_size != (3, 3) or m.stride != (1, 1) or m.padding != (1, 1) or m.dilation != (1, 1):
        return False
    if m.groups != 1 or m.bias is not None or m.padding_mode != "zeros":
        return False
    if not (x.is_contiguous(memory_format=torch.channels_last) and m.weight.is_contiguous(memory_format=torch.channels_last)):
        return False
    n, c, h, w = x.shape
    return bool(_declare().conv3x3_supported(n, h, w, c, m.out_channels)) and bool(
        _declare().conv3x3_supported(n, h, w, m.out_channels, c))


def conv3x3(x, w_krsc_ptr_tensor, cout, relu=False):
    """x: [N, Cin, H, W] channels_last; weight tensor whose memory is [Cout, 3, 3, Cin]."""
    lib = _declare()
    n, cin, h, w = x.shape
    y = torch.empty((n, cout, h, w), dtype=torch.float32, device=x.device, memory_format=torch.channels_last)
    rc = lib.conv3x3_tf32(_lib.ptr(x), _lib.ptr(w_krsc_ptr_tensor), _lib.ptr(y), n, h, w, cin, cout, int(relu),
                          _lib.stream_ptr())
    if rc != 0:
        raise RuntimeError(f"conv3x3_tf32 failed ({rc})")
    _lib.count(1)
    return y


def conv3x3_with_stats(x, weight, cout):
    """``(y, stats)``: the convolution and, from the same kernel's epilogue, one row per CTA of
    per-channel (sum, sum of squares) of ``y`` - the batch statistics of the layer that follows."""
    lib = _declare()
    n, cin, h, w = x.shape
    y = torch.empty((n, cout, h, w), dtype=torch.float32, device=x.device, memory_format=torch.channels_last)
    stats = torch.empty((lib.conv3x3_grid(n, h, w, cout), 2 * cout), dtype=torch.float32, device=x.device)
    rc = lib.conv3x3_tf32_stats(_lib.ptr(x), _lib.ptr(weight), _lib.ptr(y), _lib.ptr(stats), n, h, w, cin, cout,
                                _lib.stream_ptr())
    if rc != 0:
        raise RuntimeError(f"conv3x3_tf32_stats failed ({rc})")
    _lib.count(1)
    return y, stats


def last_error() -> int:
    lib = _declare()
    return lib.conv3x3_last_error() | lib.conv3x3_wgrad_last_error()


def _wgrad_tcgen05() -> bool:
    # 32 / 64 channels: the tcgen05 weight-gradient kernel is opt-in (CHOCO_WGRAD_TCGEN05=1); it
    # measures 34 / 27 us against 26 / 23 us of the library kernels on the ResNet-20 shapes
    return os.environ.get("CHOCO_WGRAD_TCGEN05", "0") == "1"


def wgrad_supported(n, h, w, cin, cout) -> bool:
    """True when a native weight-gradient kernel covers a 3x3 / stride 1 shape: the warp-level
    tensor-core kernels (``conv_wgrad16.cu`` for 16 channels, ``conv_wgrad_gen.cu`` for 32 / 64) or,
    opt-in, the tcgen05 kernel."""
    lib = _declare()
    if cin == cout == 16:
        return bool(lib.conv3x3_wgrad16_supported(n, h, w))
    if _wgrad_tcgen05():
        return bool(lib.conv3x3_wgrad_supported(n, h, w, cin, cout))
    return lib.conv_wgrad_gen_parts(n, h, w, cin, cout, 3, 1) > 0


def conv_wgrad_gen(x, dy, weight, ks, stride):
    """dW of a 3x3 (pad 1) or 1x1 (pad 0) convolution of stride 1 or 2 (``csrc/conv_wgrad_gen.cu``)."""
    lib = _declare()
    n, cin = x.shape[0], x.shape[1]
    cout, ho, wo = dy.shape[1], dy.shape[2], dy.shape[3]
    parts = lib.conv_wgrad_gen_parts(n, ho, wo, cin, cout, ks, stride)
    if parts <= 0:
        raise RuntimeError("conv_wgrad_gen: shape not covered")
    dw = torch.empty_like(weight)
    scratch = torch.empty(parts * weight.numel(), dtype=torch.float32, device=x.device)
    rc = lib.conv_wgrad_gen(_lib.ptr(x), _lib.ptr(dy), _lib.ptr(dw), _lib.ptr(scratch), n, ho, wo, cin, cout, ks, stride,
                            _lib.stream_ptr())
    if rc != 0:
        raise RuntimeError(f"conv_wgrad_gen failed ({rc})")
    _lib.count(2)
    return dw


def conv3x3_wgrad(x, dy, weight):
    """dW (same memory order as ``weight``: [C_out, 3, 3, C_in]) by the native kernels."""
    lib = _declare()
    n, c, h, w = x.shape
    dw = torch.empty_like(weight)
    if c == 16:
        scratch = torch.empty(lib.conv3x3_wgrad16_parts(n, h, w) * 2304, dtype=torch.float32, device=x.device)
        rc = lib.conv3x3_wgrad16(_lib.ptr(x), _lib.ptr(dy), _lib.ptr(dw), _lib.ptr(scratch), n, h, w, _lib.stream_ptr())
        if rc != 0:
            raise RuntimeError(f"conv3x3_wgrad16 failed ({rc})")
        _lib.count(2)
        return dw
    if not _wgrad_tcgen05():
        return conv_wgrad_gen(x, dy, weight, 3, 1)
    scratch = torch.empty(lib.conv3x3_wgrad_parts(n, h, w) * 9 * c * c, dtype=torch.float32, device=x.device)
    rc = lib.conv3x3_wgrad_tf32(_lib.ptr(x), _lib.ptr(dy), _lib.ptr(dw), _lib.ptr(scratch), n, h, w, c,
                                _lib.stream_ptr())
    if rc != 0:
        raise RuntimeError(f"conv3x3_wgrad_tf32 failed ({rc})")
    _lib.count(2)
    return dw


class _Fusion:
    """Hand-over between neighbouring layers of one training step, so that work of the batch-norm
    backward and of the skip connection can ride in the epilogue of the input-gradient convolution:

    * ``bn_of_output``: a batch-norm + ReLU output -> (its pre-normalisation input, mean, invstd);
      looked up by the convolution that consumes that output;
    * ``pending_res``: a tensor used as a block's skip connection -> the gradient that arrived
      over the skip; the block's first convolution adds it in its input-gradient epilogue (no add
      kernel, and its batch-norm sums then cover the whole gradient);
    * ``masked``: a gradient the epilogue already multiplied with the ReLU mask -> the per-CTA rows
      of batch-norm backward sums it produced; the batch-norm backward then skips its reduction;
    * ``pending_ds``: the input of a down-sampling block -> (gradient of the 1x1 shortcut's output,
      transposed shortcut filter); the block's strided 3x3 convolution computes both input gradients
      in one launch.

    Keys are data pointers; every entry keeps its tensors alive so that the address cannot be reused
    while the entry exists.  ``clear()`` runs at the start of a step and when a backward pass ends."""

    def __init__(self):
        self.bn_of_output, self.pending_res, self.masked, self.pending_ds = {}, {}, {}, {}
        self._callback_queued = False
        #: CHOCO_BWD_FUSION=0 keeps every layer's backward self-contained (A/B switch, tests)
        self.enabled = os.environ.get("CHOCO_BWD_FUSION", "1") != "0"

    def clear(self):
        self.bn_of_output.clear()
        self.pending_res.clear()
        self.masked.clear()
        self.pending_ds.clear()
        self._callback_queued = False

    def clear_after_backward(self):
        if not self._callback_queued:
            torch.autograd.Variable._execution_engine.queue_callback(self.clear)
            self._callback_queued = True


FUSION = _Fusion()


def conv3x3_dgrad_fused(dy, flipped, cin, add=None, mask=None, bn=None):
    """``(dx, stats)``: input gradient with the skip gradient added, the ReLU mask applied and the
    batch-norm backward sums of the producing layer accumulated, all in the epilogue."""
    lib = _declare()
    n, cout, h, w = dy.shape
    dx = torch.empty((n, cin, h, w), dtype=torch.float32, device=dy.device, memory_format=torch.channels_last)
    stats = bnx = mean = invstd = None
    if bn is not None:
        bnx, mean, invstd = bn
        stats = torch.empty((lib.conv3x3_grid(n, h, w, cin), 2 * cin), dtype=torch.float32, device=dy.device)
    rc = lib.conv3x3_dgrad_fused(_lib.ptr(dy), _lib.ptr(flipped), _lib.ptr(dx), _lib.ptr(add), _lib.ptr(mask),
                                 _lib.ptr(bnx), _lib.ptr(mean), _lib.ptr(invstd), _lib.ptr(stats), n, h, w, cout, cin,
                                 _lib.stream_ptr())
    if rc != 0:
        raise RuntimeError(f"conv3x3_dgrad_fused failed ({rc})")
    _lib.count(1)
    return dx, stats


class FlippedWeights:
    """Filters of all native convolutions of a model in the layout of their input-gradient kernels
    (3x3: taps reversed, channel roles exchanged; 1x1 shortcut: transposed), refreshed by ONE kernel
    per step.

    ``refresh()`` is called at the start of a training step (the weights do not change between the
    forward and the backward of a step); ``get(weight)`` returns the buffer for the input-gradient
    convolution, or None when the cache is not valid (the layer then flips its own filter)."""

    def __init__(self, model):
        import numpy as np

        self.entries = {}
        rows = []
        for m in model.modules():
            if (isinstance(m, torch.nn.Conv2d) and m.kernel_size in ((3, 3), (1, 1)) and m.stride in ((1, 1), (2, 2))
                    and m.weight.is_cuda and m.weight.dtype == torch.float32 and m.bias is None and m.groups == 1
                    and m.weight.is_contiguous(memory_format=torch.channels_last)
                    and m.in_channels % 16 == 0 and m.out_channels % 16 == 0):
                buf = torch.empty(m.weight.numel(), dtype=torch.float32, device=m.weight.device)
                self.entries[m.weight.data_ptr()] = buf
                rows.append((m.weight.data_ptr(), buf.data_ptr(), m.out_channels, m.in_channels,
                             m.kernel_size[0] * m.kernel_size[1], 0))
        self.n = len(rows)
        self.valid = False
        if self.n:
            dt = np.dtype([("w", np.uint64), ("out", np.uint64), ("cout", np.int32), ("cin", np.int32),
                           ("taps", np.int32), ("pad", np.int32)])
            assert dt.itemsize == _declare().conv_flip_entry_size(), "FlipEntry layout mismatch"
            host = np.array(rows, dtype=dt)
            dev = next(iter(self.entries.values())).device
            self.table = torch.from_numpy(host.view(np.uint8).copy()).to(dev)
            self.max_elems = max(r[2] * r[3] * r[4] for r in rows)

    def refresh(self):
        if not self.n:
            return
        rc = _declare().conv_flip_weights_multi(_lib.ptr(self.table), self.n, self.max_elems, _lib.stream_ptr())
        if rc != 0:
            raise RuntimeError(f"conv_flip_weights_multi failed ({rc})")
        _lib.count(1)
        self.valid = True

    def get(self, weight):
        return self.entries.get(weight.data_ptr()) if self.valid else None


_ACTIVE_FLIPS = None


def set_active_flips(f):
    global _ACTIVE_FLIPS
    _ACTIVE_FLIPS = f


def _flipped_filter(weight):
    """The filter in input-gradient layout: from the per-step cache, else computed here."""
    flipped = _ACTIVE_FLIPS.get(weight) if _ACTIVE_FLIPS is not None else None
    if flipped is not None:
        return flipped
    cout, cin, kh, kw = weight.shape
    if kh == 1:
        return weight.detach().reshape(cout, cin).t().contiguous()
    flipped = torch.empty(weight.numel(), dtype=torch.float32, device=weight.device)
    rc = _declare().conv_flip_weights(_lib.ptr(weight), _lib.ptr(flipped), cout, cin, _lib.stream_ptr())
    if rc != 0:
        raise RuntimeError(f"conv_flip_weights failed ({rc})")
    return flipped


def conv3x3s2_dgrad_fused(dy, flipped, cx, ds=None, mask=None, bn=None):
    """``(dx, stats)`` of a 3x3 / stride 2 convolution; ``ds = (dy2, w2_t)`` adds the input gradient of
    the 1x1 / stride 2 shortcut; mask / bn as in ``conv3x3_dgrad_fused``."""
    lib = _declare()
    n, cdy, ho, wo = dy.shape
    dx = torch.empty((n, cx, 2 * ho, 2 * wo), dtype=torch.float32, device=dy.device, memory_format=torch.channels_last)
    stats = bnx = mean = invstd = None
    if bn is not None:
        bnx, mean, invstd = bn
        stats = torch.empty((lib.conv3x3s2_dgrad_grid(n, ho, wo, cx), 2 * cx), dtype=torch.float32, device=dy.device)
    dy2, w2t = ds if ds is not None else (None, None)
    rc = lib.conv3x3s2_dgrad_fused(_lib.ptr(dy), _lib.ptr(flipped), _lib.ptr(dy2), _lib.ptr(w2t), _lib.ptr(dx), None,
                                   _lib.ptr(mask), _lib.ptr(bnx), _lib.ptr(mean), _lib.ptr(invstd), _lib.ptr(stats),
                                   n, ho, wo, cdy, cx, dy2.shape[1] if dy2 is not None else 0, _lib.stream_ptr())
    if rc != 0:
        raise RuntimeError(f"conv3x3s2_dgrad_fused failed ({rc})")
    _lib.count(1)
    return dx, stats


class _Conv3x3Fn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, want_stats=False, fold_res=False):
        # x is the output of a batch-norm + ReLU of this step: its backward sums can be produced by
        # this convolution's input-gradient epilogue
        ent = FUSION.bn_of_output.get(x.data_ptr()) if FUSION.enabled else None
        ctx.bn_in = ent is not None and ent[0].shape == x.shape
        ctx.fold_res = bool(fold_res)
        if ctx.bn_in:
            ctx.save_for_backward(x, weight, ent[1], ent[2], ent[3])
        else:
            ctx.save_for_backward(x, weight)
        ctx.set_materialize_grads(False)  # no zero-filled gradient tensor for the statistics output
        if want_stats:
            y, stats = conv3x3_with_stats(x, weight, weight.shape[0])
            ctx.mark_non_differentiable(stats)
            return y, stats
        return conv3x3(x, weight, weight.shape[0])

    @staticmethod
    def backward(ctx, dy, _dstats=None):
        if dy is None:
            return None, None, None, None
        dx, dw = _Conv3x3Fn._backward(ctx, dy)
        return dx, dw, None, None

    @staticmethod
    def _backward(ctx, dy):
        x, weight = ctx.saved_tensors[:2]
        lib = _declare()
        dy = dy.contiguous(memory_format=torch.channels_last)
        cout, cin = weight.shape[0], weight.shape[1]
        dx = dw = None
        n, _, h, w = x.shape
        from . import nn as native_nn

        # the weight gradient is forked first so that it does not wait for this layer's dgrad
        if ctx.needs_input_grad[1]:
            if native_nn.native_enabled("wgrad") and wgrad_supported(n, h, w, cin, cout):
                fn = lambda: conv3x3_wgrad(x, dy, weight)
            else:
                fn = lambda: torch.ops.aten.convolution_backward(
                    dy, x, weight, None, (1, 1), (1, 1), (1, 1), False, (0, 0), 1, (False, True, False))[1]
            # Side stream only when autograd will take the result over as the new .grad without
            # touching it (no accumulate / copy kernel on the launching stream before the join).
            fork = _WGRAD_STREAM.enabled and weight.grad is None and not torch.is_grad_enabled()
            dw = _WGRAD_STREAM.run(fn, (x, dy), x.device) if fork else fn()
        if ctx.needs_input_grad[0]:
            flipped = _flipped_filter(weight)
            add = FUSION.pending_res.pop(x.data_ptr(), None) if ctx.fold_res else None
            if ctx.bn_in or add is not None:
                bn = ctx.saved_tensors[2:5] if ctx.bn_in else None
                dx, stats = conv3x3_dgrad_fused(dy, flipped, cin, add=add[1] if add is not None else None,
                                                mask=x if ctx.bn_in else None, bn=bn)
                if stats is not None:
                    FUSION.masked[dx.data_ptr()] = (dx, stats)
                    FUSION.clear_after_backward()
            else:
                dx = conv3x3(dy, flipped, cin)
        return dx, dw


def gen_conv_supported(m, x) -> bool:
    """Strided 3x3 (pad 1) and 1x1 (pad 0) convolutions between 16 / 32 / 64 / 128 channels: the first
    convolution of a ResNet stage and its down-sampling shortcut."""
    if not (x.is_cuda and x.dtype == torch.float32 and x.dim() == 4 and m.weight.dtype == torch.float32):
        return False
    ks, st = m.kernel_size[0], m.stride[0]
    if m.kernel_size != (ks, ks) or m.stride != (st, st) or ks not in (1, 3) or st not in (1, 2) or (ks == 3 and st == 1):
        return False
    if m.padding != (ks // 2, ks // 2) or m.dilation != (1, 1) or m.groups != 1 or m.bias is not None:
        return False
    if m.padding_mode != "zeros":
        return False
    if not (x.is_contiguous(memory_format=torch.channels_last) and m.weight.is_contiguous(memory_format=torch.channels_last)):
        return False
    n, c, h, w = x.shape
    if h % st or w % st:
        return False
    return bool(_declare().conv_fwd_supported(n, h // st, w // st, c, m.out_channels, ks, st))


class _ConvGenFn(torch.autograd.Function):
    """Strided 3x3 / 1x1 convolution: forward on the persistent tcgen05 kernel (strided tensor map),
    weight gradient on ``conv_wgrad_gen.cu``, input gradient of the 3x3 / stride 2 form on the same
    persistent kernel (four parity classes of the result).  ``fold_ds``: this layer and the block's
    other strided convolution read the same tensor; the 1x1 shortcut then hands its output gradient to
    the 3x3 convolution, which produces the sum of both input gradients in one launch."""

    @staticmethod
    def forward(ctx, x, weight, ks, stride, want_stats=False, fold_ds=False):
        lib = _declare()
        n, cin, h, w = x.shape
        cout, ho, wo = weight.shape[0], h // stride, w // stride
        ent = FUSION.bn_of_output.get(x.data_ptr()) if (FUSION.enabled and ks == 3) else None
        ctx.bn_in = ent is not None and ent[0].shape == x.shape
        if ctx.bn_in:
            ctx.save_for_backward(x, weight, ent[1], ent[2], ent[3])
        else:
            ctx.save_for_backward(x, weight)
        ctx.geom = (ks, stride)
        ctx.fold_ds = bool(fold_ds)
        ctx.set_materialize_grads(False)
        y = torch.empty((n, cout, ho, wo), dtype=torch.float32, device=x.device, memory_format=torch.channels_last)
        stats = None
        if want_stats:
            stats = torch.empty((lib.conv3x3_grid(n, ho, wo, cout), 2 * cout), dtype=torch.float32, device=x.device)
        rc = lib.conv_fwd_tf32(_lib.ptr(x), _lib.ptr(weight), _lib.ptr(y), _lib.ptr(stats), n, ho, wo, cin, cout, ks,
                               stride, _lib.stream_ptr())
        if rc != 0:
            raise RuntimeError(f"conv_fwd_tf32 failed ({rc})")
        _lib.count(1)
        if want_stats:
            ctx.mark_non_differentiable(stats)
            return y, stats
        return y

    @staticmethod
    def backward(ctx, dy, _dstats=None):
        if dy is None:
            return None, None, None, None, None, None
        x, weight = ctx.saved_tensors[:2]
        ks, stride = ctx.geom
        lib = _declare()
        dy = dy.contiguous(memory_format=torch.channels_last)
        n, cin, h, w = x.shape
        cout, ho, wo = weight.shape[0], h // stride, w // stride
        geom = ((stride, stride), (ks // 2, ks // 2), (1, 1), False, (0, 0), 1)
        dx = dw = None
        from . import nn as native_nn

        if ctx.needs_input_grad[1]:
            if native_nn.native_enabled("wgrad") and lib.conv_wgrad_gen_parts(n, ho, wo, cin, cout, ks, stride) > 0:
                fn = lambda: conv_wgrad_gen(x, dy, weight, ks, stride)
            else:
                fn = lambda: torch.ops.aten.convolution_backward(dy, x, weight, None, *geom, (False, True, False))[1]
            fork = _WGRAD_STREAM.enabled and weight.grad is None and not torch.is_grad_enabled()
            dw = _WGRAD_STREAM.run(fn, (x, dy), x.device) if fork else fn()
        if ctx.needs_input_grad[0]:
            if ks == 1 and ctx.fold_ds:
                # handed to the block's 3x3 / stride 2 convolution, whose backward runs after this one
                FUSION.pending_ds[x.data_ptr()] = (x, dy, _flipped_filter(weight))
                FUSION.clear_after_backward()
            elif ks == 3 and stride == 2 and lib.conv3x3s2_dgrad_supported(n, ho, wo, cout, cin, 0):
                ds = FUSION.pending_ds.pop(x.data_ptr(), None) if ctx.fold_ds else None
                if ctx.fold_ds and ds is None:
                    raise RuntimeError("the shortcut's gradient was not handed over before the strided convolution's backward")
                bn = ctx.saved_tensors[2:5] if ctx.bn_in else None
                dx, stats = conv3x3s2_dgrad_fused(dy, _flipped_filter(weight), cin, ds=ds[1:] if ds is not None else None,
                                                  mask=x if ctx.bn_in else None, bn=bn)
                if stats is not None:
                    FUSION.masked[dx.data_ptr()] = (dx, stats)
                    FUSION.clear_after_backward()
            else:
                dx = torch.ops.aten.convolution_backward(dy, x, weight, None, *geom, (True, False, False))[0]
        return dx, dw, None, None, None, None


def fold_shortcut_ok(conv, shortcut_conv, x) -> bool:
    """True when a down-sampling block's strided 3x3 convolution can take over the input gradient of its
    1x1 / stride 2 shortcut (both read ``x``; both run the native kernels)."""
    from . import nn as native_nn

    if not (native_nn.native_enabled("conv") and FUSION.enabled and x.is_cuda and x.requires_grad
            and torch.is_grad_enabled()):
        return False
    if conv.kernel_size != (3, 3) or conv.stride != (2, 2) or shortcut_conv.kernel_size != (1, 1):
        return False
    if shortcut_conv.stride != (2, 2) or not (gen_conv_supported(conv, x) and gen_conv_supported(shortcut_conv, x)):
        return False
    n, c, h, w = x.shape
    return bool(_declare().conv3x3s2_dgrad_supported(n, h // 2, w // 2, conv.out_channels, c, shortcut_conv.out_channels))


class _WgradStream:
    """Weight gradients on a second stream.

    The critical path of the backward pass is dgrad -> BN backward -> dgrad ...; the weight
    gradient of a layer is needed only by the update at the end.  Each wgrad kernel is forked onto
    a side stream (which first waits for everything enqueued so far on the launching stream), and
    joined either when more than ``depth`` of them are pending or by a callback at the end of the
    backward pass.  The operands stay referenced until the join, so the allocator cannot hand
    their memory to later kernels of the launching stream.  Nothing on the launching stream may
    read the result before the join: the fork is used only when the parameter has no ``.grad``
    yet, so that autograd adopts the new tensor without launching a kernel on it.  Works the same under CUDA-graph
    capture (the fork / join become graph dependencies)."""

    depth = 4

    def __init__(self):
        self.enabled = True
        self._streams = {}
        self._pending = []
        self._callback_queued = False

    def _side(self, device):
        st = self._streams.get(device)
        if st is None:
            st = self._streams[device] = torch.cuda.Stream(device=device)
        return st

    def run(self, fn, keep, device):
        main = torch.cuda.current_stream(device)
        side = self._side(device)
        side.wait_stream(main)
        with torch.cuda.stream(side):
            out = fn()
            ev = torch.cuda.Event()
            ev.record(side)
        # the result itself is NOT kept: a second reference would make autograd copy it (on the
        # launching stream, before the join) instead of adopting it as the parameter's .grad
        self._pending.append((ev, main, keep))
        if not self._callback_queued:
            torch.autograd.Variable._execution_engine.queue_callback(self.join)
            self._callback_queued = True
        while len(self._pending) > self.depth:
            self._join_one()
        return out

    def _join_one(self):
        ev, main, _keep = self._pending.pop(0)
        main.wait_event(ev)

    def join(self):
        """Make the launching stream wait for every pending weight gradient."""
        while self._pending:
            self._join_one()
        self._callback_queued = False


_WGRAD_STREAM = _WgradStream()


def wgrad_side_stream(device):
    """The stream weight gradients are forked onto (None before its first use or when switched off)."""
    if not _WGRAD_STREAM.enabled:
        return None
    device = torch.device(device)
    index = device.index if device.index is not None else torch.cuda.current_device()
    for d, st in _WGRAD_STREAM._streams.items():
        if d.type == device.type and (d.index if d.index is not None else torch.cuda.current_device()) == index:
            return st
    return None


def set_wgrad_side_stream(on: bool):
    _WGRAD_STREAM.join()
    _WGRAD_STREAM.enabled = bool(on)


def _declare_first():
    lib = _lib.load()
    if not getattr(lib, "_conv_first_declared", False):
        vp, i = ctypes.c_void_p, ctypes.c_int
        lib.conv_first_supported.argtypes = [i, i]
        lib.conv_first_grid.argtypes = [i, i, i, i]
        lib.conv_first_wgrad_parts.argtypes = [i, i, i, i]
        lib.conv_first_forward.argtypes = [vp, vp, vp, vp, i, i, i, i, vp]
        lib.conv_first_wgrad.argtypes = [vp, vp, vp, vp, i, i, i, i, vp]
        for n in ("conv_first_supported", "conv_first_grid", "conv_first_wgrad_parts", "conv_first_forward",
                  "conv_first_wgrad"):
            getattr(lib, n).restype = i
        lib._conv_first_declared = True
    return lib


def first_conv_supported(m, x) -> bool:
    """3x3 / stride 1 / pad 1 convolution of a 3-channel NHWC image (``csrc/conv_first.cu``)."""
    if not (x.is_cuda and x.dtype == torch.float32 and x.dim() == 4 and m.weight.dtype == torch.float32):
        return False
    if m.kernel_size != (3, 3) or m.stride != (1, 1) or m.padding != (1, 1) or m.dilation != (1, 1):
        return False
    if m.groups != 1 or m.bias is not None or m.padding_mode != "zeros" or x.requires_grad:
        return False
    if not (x.is_contiguous(memory_format=torch.channels_last) and m.weight.is_contiguous(memory_format=torch.channels_last)):
        return False
    return bool(_declare_first().conv_first_supported(x.shape[1], m.out_channels))


class _ConvFirstFn(torch.autograd.Function):
    """First-layer convolution: fp32 FMA kernels, weight gradient only (the input is the image)."""

    @staticmethod
    def forward(ctx, x, weight, want_stats=False):
        lib = _declare_first()
        n, _, h, w = x.shape
        cout = weight.shape[0]
        ctx.save_for_backward(x, weight)
        ctx.set_materialize_grads(False)
        y = torch.empty((n, cout, h, w), dtype=torch.float32, device=x.device, memory_format=torch.channels_last)
        stats = None
        if want_stats:
            stats = torch.empty((lib.conv_first_grid(n, h, w, cout), 2 * cout), dtype=torch.float32, device=x.device)
        rc = lib.conv_first_forward(_lib.ptr(x), _lib.ptr(weight), _lib.ptr(y), _lib.ptr(stats) if want_stats else None,
                                    n, h, w, cout, _lib.stream_ptr())
        if rc != 0:
            raise RuntimeError(f"conv_first_forward failed ({rc})")
        _lib.count(1)
        if want_stats:
            ctx.mark_non_differentiable(stats)
            return y, stats
        return y

    @staticmethod
    def backward(ctx, dy, _dstats=None):
        if dy is None or not ctx.needs_input_grad[1]:
            return None, None, None
        x, weight = ctx.saved_tensors
        dy = dy.contiguous(memory_format=torch.channels_last)

        def fn():
            lib = _declare_first()
            n, _, h, w = x.shape
            cout = weight.shape[0]
            dw = torch.empty_like(weight)
            scratch = torch.empty(lib.conv_first_wgrad_parts(n, h, w, cout) * cout * 27, dtype=torch.float32,
                                  device=x.device)
            rc = lib.conv_first_wgrad(_lib.ptr(x), _lib.ptr(dy), _lib.ptr(dw), _lib.ptr(scratch), n, h, w, cout,
                                      _lib.stream_ptr())
            if rc != 0:
                raise RuntimeError(f"conv_first_wgrad failed ({rc})")
            _lib.count(2)
            return dw

        # not forked to the weight-gradient stream: this is the last gradient of a backward pass, nothing is
        # left on the main stream for it to overlap with, and there it runs beside whatever the second stream
        # still has queued instead of behind it
        return None, fn(), None


def _declare_stem():
    lib = _lib.load()
    if not getattr(lib, "_conv_stem_declared", False):
        i, vp = ctypes.c_int, ctypes.c_void_p
        lib.conv_stem_supported.argtypes = [i, i, i, i, i]
        lib.conv_stem_grid.argtypes = [i, i, i]
        lib.conv_stem_last_error.argtypes = []
        lib.conv_stem_forward.argtypes = [vp, vp, vp, vp, i, i, i, vp]
        lib.conv_stem_wgrad.argtypes = [vp, vp, vp, vp, i, i, i, vp]
        for n in ("conv_stem_supported", "conv_stem_grid", "conv_stem_last_error", "conv_stem_forward", "conv_stem_wgrad"):
            getattr(lib, n).restype = i
        lib._conv_stem_declared = True
    return lib


def stem_conv_supported(m, x) -> bool:
    """7x7 / stride 2 / pad 3 convolution of a 3-channel fp32 NHWC image into 64 bf16 channels under bf16
    autocast (``csrc/conv_stem_bf16.cu``): the first layer of the ImageNet ResNets."""
    if not (x.is_cuda and x.dtype == torch.float32 and x.dim() == 4 and m.weight.dtype == torch.float32):
        return False
    if not (torch.is_autocast_enabled("cuda") and torch.get_autocast_dtype("cuda") == torch.bfloat16):
        return False
    if m.kernel_size != (7, 7) or m.stride != (2, 2) or m.padding != (3, 3) or m.dilation != (1, 1):
        return False
    if m.groups != 1 or m.bias is not None or m.padding_mode != "zeros" or x.requires_grad:
        return False
    if not (x.is_contiguous(memory_format=torch.channels_last) and m.weight.is_contiguous(memory_format=torch.channels_last)):
        return False
    n, c, h, w = x.shape
    return bool(_declare_stem().conv_stem_supported(n, h, w, c, m.out_channels))


def stem_last_error() -> int:
    """1 when a bounded wait inside one of the stem kernels ran out since the last call."""
    return _declare_stem().conv_stem_last_error()


class _ConvStemFn(torch.autograd.Function):
    """ImageNet stem: tcgen05 bf16 kernels that read the fp32 image directly; weight gradient only."""

    @staticmethod
    def forward(ctx, x, weight):
        lib = _declare_stem()
        n, _, h, w = x.shape
        ctx.save_for_backward(x, weight)
        ctx.set_materialize_grads(False)
        y = torch.empty((n, 64, h // 2, w // 2), dtype=torch.bfloat16, device=x.device, memory_format=torch.channels_last)
        rc = lib.conv_stem_forward(_lib.ptr(x), _lib.ptr(weight), _lib.ptr(y), None, n, h, w, _lib.stream_ptr())
        if rc != 0:
            raise RuntimeError(f"conv_stem_forward failed ({rc})")
        _lib.count(1)
        return y

    @staticmethod
    def backward(ctx, dy):
        if dy is None or not ctx.needs_input_grad[1]:
            return None, None
        x, weight = ctx.saved_tensors
        if dy.dtype != torch.bfloat16:
            dy = dy.to(torch.bfloat16)
        dy = dy.contiguous(memory_format=torch.channels_last)
        lib = _declare_stem()
        n, _, h, w = x.shape
        dw = torch.empty_like(weight)
        scratch = torch.empty(lib.conv_stem_grid(n, h, w) * 64 * 176, dtype=torch.float32, device=x.device)
        rc = lib.conv_stem_wgrad(_lib.ptr(x), _lib.ptr(dy), _lib.ptr(dw), _lib.ptr(scratch), n, h, w, _lib.stream_ptr())
        if rc != 0:
            raise RuntimeError(f"conv_stem_wgrad failed ({rc})")
        _lib.count(2)
        return None, dw


def conv_stem_native(m, x):
    return _ConvStemFn.apply(x, m.weight)


def conv2d_native(m, x, want_stats=False, fold_res=False, fold_ds=False):
    if m.in_channels == 3:
        return _ConvFirstFn.apply(x, m.weight, want_stats)
    if m.stride != (1, 1) or m.kernel_size != (3, 3):
        return _ConvGenFn.apply(x, m.weight, m.kernel_size[0], m.stride[0], want_stats, fold_ds)
    return _Conv3x3Fn.apply(x, m.weight, want_stats, fold_res)


def any_conv_supported(m, x) -> bool:
    """True when one of the native convolution kernels covers the layer for this input."""
    return conv_supported(m, x) or first_conv_supported(m, x) or gen_conv_supported(m, x)
