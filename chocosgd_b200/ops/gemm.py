"""tcgen05 / TMEM GEMM bindings (``csrc/gemm_sm100.cu``) and the native ``Linear`` path.

``gemm(a, b, a_mn=False, b_mn=False)`` computes ``A . B^T`` in TF32 with fp32 accumulation:
``a`` is ``[M, K]`` (K-major) or ``[K, M]`` when ``a_mn``; ``b`` is ``[N, K]`` or ``[K, N]``
when ``b_mn``.  A linear layer then needs no transposes:

    forward   y  = gemm(x, W)                        x [M,K], W [N,K]
    dgrad     dx = gemm(dy, W, b_mn=True)            dy [M,N], W read as [N(k), K(n)]
    wgrad     dW = gemm(dy, x, a_mn=True, b_mn=True) reduction over the batch, split-K

TMA needs 16-byte aligned row strides, i.e. every leading dimension a multiple of 4 floats;
``linear_supported`` checks that and the layer falls back to the library GEMM otherwise."""
from __future__ import annotations

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


def last_error() -> int:
    """0, or the code recorded by a kernel whose bounded wait expired (synchronises)."""
    return _declare().gemm_tf32_last_error()


def _aligned(*dims):
    return all(d % 4 == 0 for d in dims)


def linear_supported(x, weight) -> bool:
    n, k = weight.shape
    return (weight.dtype == torch.float32 and weight.is_contiguous() and _aligned(n, k) and x.shape[-1] == k
            and x.numel() // k >= 1)


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x2, weight, bias):
        ctx.save_for_backward(x2, weight)
        ctx.has_bias = bias is not None
        return gemm(x2, weight, bias)

    @staticmethod
    def backward(ctx, dy):
        x2, weight = ctx.saved_tensors
        dy = dy.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy, weight, b_mn=True)
        if ctx.needs_input_grad[1]:
            m = x2.shape[0]
            dw = gemm(dy, x2, a_mn=True, b_mn=True, split_k=max(1, min(32, m // 512)))
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy.sum(dim=0)
        return dx, dw, db


def linear_native(x, weight, bias=None):
    shape = x.shape
    x2 = x.reshape(-1, shape[-1]).contiguous()
    y = _LinearFn.apply(x2, weight, bias)
    return y.view(*shape[:-1], weight.shape[0])
