"""tcgen05 / TMEM GEMM bindings (``csrc/gemm_sm100.cu``) and the native ``Linear`` path.

``gemm(a, b, a_mn=False, b_mn=False)`` computes ``A . B^T`` in TF32 with fp32 accumulation:
``a`` is ``[M, K]`` (K-major) or ``[K, M]`` when ``a_mn``; ``b`` is ``[N, K]`` or ``[K, N]``
when ``b_mn``.  A linear layer then needs no transposes:

    forward   y  = gemm(x, W)                        x [M,K], W [N,K]
    dgrad     dx = gemm(dy, W, b_mn=True)            dy [M,N], W read as [N(k), K(n)]
    wgrad     dW = gemm(dy, x, a_mn=True, b_mn=True) reduction over the batch, split-K

TMA needs 16-byte aligned row strides; ``split_pad`` re-lays any fp32 matrix with padded rows while
it splits it into an exact-TF32 part and the fp32 remainder, and ``gemm_x3`` multiplies such pairs
with three tensor-core passes (fp32-grade accuracy).  The native ``Linear`` layer is built on those
two: its forward, input-gradient and weight-gradient GEMMs all run on the tcgen05 kernel."""
from __future__ import annotations

import ctypes

import torch

from . import _lib


def _declare():
    lib = _lib.load()
    if not getattr(lib, "_gemm_declared", False):
        import ctypes

        vp, i = ctypes.c_void_p, ctypes.c_int
        lib.gemm_tf32.argtypes = [vp, vp, vp, vp, i, i, i, i, i, i, i, i, i, i, vp]
        lib.gemm_tf32.restype = i
        lib.gemm_tf32_last_error.argtypes = []
        lib.gemm_tf32_last_error.restype = i
        lib.gemm_tf32x3.argtypes = [vp, vp, vp, vp, vp, vp, i, i, i, i, i, i, i, i, i, i, vp]
        lib.gemm_tf32x3.restype = i
        lib.tf32_split_pad.argtypes = [vp, ctypes.c_longlong, i, ctypes.c_longlong, vp, vp, i, vp]
        lib.tf32_split_pad.restype = i
        lib._gemm_declared = True
    return lib


def gemm(a, b, bias=None, a_mn=False, b_mn=False, split_k=1, relu=False, out=None):
    lib = _declare()
    assert a.is_cuda and b.is_cuda and a.dtype == torch.float32 and b.dtype == torch.float32
    assert a.dim() == 2 and b.dim() == 2 and a.stride(1) == 1 and b.stride(1) == 1
    M, K = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    N, Kb = (b.shape[1], b.shape[0]) if b_mn else (b.shape[0], b.shape[1])
    assert K == Kb, (a.shape, b.shape, a_mn, b_mn)
    if out is None:
        out = (torch.zeros if split_k > 1 else torch.empty)((M, N), dtype=torch.float32, device=a.device)
    elif split_k > 1:
        out.zero_()
    rc = lib.gemm_tf32(_lib.ptr(a), _lib.ptr(b), _lib.ptr(out), _lib.ptr(bias), M, N, K, a.stride(0), b.stride(0),
                       out.stride(0), int(a_mn), int(b_mn), int(split_k), int(relu), _lib.stream_ptr())
    if rc != 0:
        raise RuntimeError(f"gemm_tf32 failed with code {rc}")
    return out


def pad4(n: int) -> int:
    return (n + 3) // 4 * 4


def split_pad(x: torch.Tensor):
    """``(hi, lo)`` of a 2-d fp32 tensor with unit inner stride: ``hi`` holds the values with their 13
    low mantissa bits cleared (exact TF32 numbers), ``lo = x - hi``; both have ``pad4(cols)`` floats per
    row (16-byte aligned rows, as TMA needs) and are returned as ``[rows, cols]`` views."""
    lib = _declare()
    assert x.is_cuda and x.dtype == torch.float32 and x.dim() == 2 and x.stride(1) == 1
    rows, cols = x.shape
    ld = pad4(cols)
    hi = torch.empty((rows, ld), dtype=torch.float32, device=x.device)
    lo = torch.empty((rows, ld), dtype=torch.float32, device=x.device)
    rc = lib.tf32_split_pad(_lib.ptr(x), rows, cols, x.stride(0), _lib.ptr(hi), _lib.ptr(lo), ld, _lib.stream_ptr())
    if rc != 0:
        raise RuntimeError(f"tf32_split_pad failed with code {rc}")
    _lib.count(1)
    return hi[:, :cols], lo[:, :cols]


def gemm_x3(a, b, bias=None, a_mn=False, b_mn=False, split_k=1, out=None):
    """``A . B^T`` with fp32-grade products on the TF32 tensor cores: ``a`` and ``b`` are ``(hi, lo)``
    pairs from ``split_pad``; three passes accumulate hi.hi + hi.lo + lo.hi in one TMEM accumulator
    (relative error per product 2^-21 instead of 2^-10).  The result has 16-byte aligned rows and is
    returned as an ``[M, N]`` view."""
    lib = _declare()
    (ah, al), (bh, bl) = a, b
    M, K = (ah.shape[1], ah.shape[0]) if a_mn else (ah.shape[0], ah.shape[1])
    N, Kb = (bh.shape[1], bh.shape[0]) if b_mn else (bh.shape[0], bh.shape[1])
    assert K == Kb and ah.stride(0) == al.stride(0) and bh.stride(0) == bl.stride(0), (ah.shape, bh.shape)
    if out is None:
        ldd = pad4(N)
        buf = (torch.zeros if split_k > 1 else torch.empty)((M, ldd), dtype=torch.float32, device=ah.device)
        out = buf[:, :N]
    elif split_k > 1:
        out.zero_()
    rc = lib.gemm_tf32x3(_lib.ptr(ah), _lib.ptr(al), _lib.ptr(bh), _lib.ptr(bl), _lib.ptr(out), _lib.ptr(bias), M, N, K,
                         ah.stride(0), bh.stride(0), out.stride(0), int(a_mn), int(b_mn), int(split_k), 0,
                         _lib.stream_ptr())
    if rc != 0:
        raise RuntimeError(f"gemm_tf32x3 failed with code {rc}")
    _lib.count(1)
    return out


def last_error() -> int:
    """0, or the code recorded by a kernel whose bounded wait expired (synchronises)."""
    return _declare().gemm_tf32_last_error()


def _aligned(*dims):
    return all(d % 4 == 0 for d in dims)


#: below this many multiply-adds the library GEMM is the better choice (one tile per SM is not reached)
MIN_NATIVE_WORK = 1 << 30


def linear_supported(x, weight) -> bool:
    """Layers the tcgen05 GEMM takes: fp32, and large enough to fill the machine (the language
    model's decoder; small classifiers stay on the library).  Any row length works: operands are
    re-laid with 16-byte aligned rows on the way in."""
    n, k = weight.shape
    m = x.numel() // max(k, 1)
    return (weight.dtype == torch.float32 and weight.stride(-1) == 1 and x.shape[-1] == k and m >= 1
            and m * n * k >= MIN_NATIVE_WORK)


def strict_fp32() -> bool:
    """PyTorch's own switch for linear layers: when TF32 is not allowed the native path keeps fp32-grade
    accuracy with split operands (three tensor-core passes), otherwise it runs one TF32 pass."""
    return not torch.backends.cuda.matmul.allow_tf32


class _LinearFn(torch.autograd.Function):
    """y = x W^T + b on the tcgen05 GEMM.  Operands are split into exact-TF32 and remainder parts once
    per use (x and W in forward, dy in backward; W's parts are kept for the input gradient), all three
    GEMMs run without a transpose pass and in fp32-grade precision."""

    @staticmethod
    def forward(ctx, x2, weight, bias):
        xs, ws = split_pad(x2), split_pad(weight)
        ctx.save_for_backward(*xs, *ws)
        ctx.has_bias = bias is not None
        ctx.shapes = (x2.shape, weight.shape)
        return gemm_x3(xs, ws, bias)

    @staticmethod
    def backward(ctx, dy):
        xh, xl, wh, wl = ctx.saved_tensors
        (m, k), (n, _) = ctx.shapes
        if dy.stride(1) != 1:
            dy = dy.contiguous()
        dys = split_pad(dy)
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            # dx [m, k] = dy [m, n] . W [n, k]: few output tiles, long reduction -> split K over the SMs
            tiles = -(-m // 128) * -(-k // 128)
            split = max(1, min(16, 296 // max(tiles, 1)))
            dx = gemm_x3(dys, (wh, wl), b_mn=True, split_k=split,
                         out=torch.empty((m, k), dtype=torch.float32, device=dy.device))
        if ctx.needs_input_grad[1]:
            # written straight into a tensor of the parameter's own layout (the optimizer reads it there)
            dw = gemm_x3(dys, (xh, xl), a_mn=True, b_mn=True,
                         out=torch.empty((n, k), dtype=torch.float32, device=dy.device))
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy.sum(dim=0)
        return dx, dw, db


def linear_native(x, weight, bias=None):
    shape = x.shape
    x2 = x.reshape(-1, shape[-1])
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    y = _LinearFn.apply(x2, weight, bias)      # [M, N] view of a buffer with 16-byte aligned rows
    return y.view(*shape[:-1], weight.shape[0]) if len(shape) > 2 else y
