"""Native LSTM layer stack: gate GEMMs + recurrent kernels (``csrc/lstm_persistent.cu``,
``csrc/lstm_cell.cu``).

Per layer the input projection of all time steps is ONE GEMM (the tcgen05 kernel when the
dimensions are multiples of 4, the library GEMM otherwise, e.g. hidden size 650); the recurrence over
the time steps is ONE persistent kernel per direction for batch <= 32 and hidden sizes whose
weight slices fit in shared memory, else one recurrent GEMM plus one fused pointwise kernel per step.  Backward runs the cell kernel in reverse and
forms dW_ih, dW_hh and dX with three GEMMs over the whole sequence.  Same parameters, gate order and
results as ``torch.nn.LSTM`` (``dl_code/pcode/models/rnn_lm.py:29,53-61``); dropout between layers as there."""
from __future__ import annotations

import ctypes

import torch
import torch.nn.functional as F

from . import _lib
from .gemm import gemm, gemm_x3, split_pad


def _declare():
    lib = _lib.load()
    if not getattr(lib, "_lstm_declared", False):
        vp, i = ctypes.c_void_p, ctypes.c_int
        lib.lstm_cell_fwd.argtypes = [vp, vp, vp, vp, i, i, vp]
        lib.lstm_cell_bwd.argtypes = [vp, vp, vp, vp, vp, i, i, vp]
        lib.lstm_cell_fwd.restype = lib.lstm_cell_bwd.restype = i
        lib.lstm_rec_supported.argtypes = [i, i, i]
        lib.lstm_rec_forward.argtypes = [vp, vp, vp, vp, i, i, i, vp]
        lib.lstm_rec_backward.argtypes = [vp, vp, vp, vp, vp, vp, vp, i, i, i, vp]
        lib.lstm_rec_bwd_scratch.argtypes = [i]
        lib.lstm_rec_bwd_scratch.restype = ctypes.c_longlong
        lib.lstm_rec_supported.restype = lib.lstm_rec_forward.restype = lib.lstm_rec_backward.restype = i
        lib.lstm_rec_last_error.restype = i
        lib._lstm_declared = True
    return lib


#: one persistent kernel per layer and direction (``csrc/lstm_persistent.cu``) when the shape fits
PERSISTENT = [True]


def last_error() -> int:
    """Non-zero when a grid barrier of the persistent kernels ran out of its wait budget."""
    return _declare().lstm_rec_last_error()


#: the four large GEMMs of a layer (input projection; dX, dW_ih, dW_hh over the whole sequence) on the
#: tcgen05 GEMM with split operands (fp32-grade products); False: library GEMMs
NATIVE_GEMM = [True]
MIN_GEMM_WORK = 1 << 28   # multiply-adds below which the library GEMM is used


def _big(m, n, k) -> bool:
    return NATIVE_GEMM[0] and m * n * k >= MIN_GEMM_WORK


def _mm_nt(a, b, bias=None):
    """a [M, K] @ b[N, K]^T (+ bias)."""
    if _big(a.shape[0], b.shape[0], a.shape[1]):
        return gemm_x3(split_pad(a), split_pad(b), bias)
    out = a @ b.t()
    return out.add_(bias) if bias is not None else out


class _LSTMLayerFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, h0, c0, w_ih, w_hh, b_ih, b_hh):
        lib = _declare()
        T, B, _ = x.shape
        H = w_hh.shape[1]
        gates = _mm_nt(x.reshape(T * B, -1).contiguous(), w_ih, b_ih + b_hh)
        if gates.stride(0) != 4 * H:
            gates = gates.contiguous()
        gates = gates.view(T, B, 4 * H)
        hs = torch.empty(T + 1, B, H, dtype=x.dtype, device=x.device)
        cs = torch.empty(T + 1, B, H, dtype=x.dtype, device=x.device)
        hs[0].copy_(h0)
        cs[0].copy_(c0)
        sp = _lib.stream_ptr()
        w_hh_c = w_hh.contiguous()
        if PERSISTENT[0] and lib.lstm_rec_supported(T, B, H):
            # all T steps in one persistent kernel (grid barrier per step)
            _lib.check(lib.lstm_rec_forward(_lib.ptr(gates), _lib.ptr(w_hh_c), _lib.ptr(hs), _lib.ptr(cs), T, B, H, sp),
                       "lstm_rec_forward")
            _lib.count(1)
        else:
            for t in range(T):
                gates[t].addmm_(hs[t], w_hh.t())
                _lib.check(lib.lstm_cell_fwd(_lib.ptr(gates[t]), _lib.ptr(cs[t]), _lib.ptr(cs[t + 1]),
                                             _lib.ptr(hs[t + 1]), B, H, sp), "lstm_cell_fwd")
        ctx.save_for_backward(x, w_ih, w_hh, gates, hs, cs)
        return hs[1:], hs[T].clone(), cs[T].clone()

    @staticmethod
    def backward(ctx, d_out, d_hn, d_cn):
        lib = _declare()
        x, w_ih, w_hh, gates, hs, cs = ctx.saved_tensors
        T, B, _ = x.shape
        H = w_hh.shape[1]
        dgates = gates.clone()  # activations in, d(pre-activations) out
        dh = d_hn.clone() if d_hn is not None else torch.zeros(B, H, dtype=x.dtype, device=x.device)
        dc = d_cn.clone() if d_cn is not None else torch.zeros(B, H, dtype=x.dtype, device=x.device)
        d_out = d_out.contiguous() if d_out is not None else None
        sp = _lib.stream_ptr()
        if PERSISTENT[0] and lib.lstm_rec_supported(T, B, H):
            scratch = torch.zeros(lib.lstm_rec_bwd_scratch(H), dtype=torch.float32, device=x.device)
            dh, dc = dh.contiguous(), dc.contiguous()
            _lib.check(lib.lstm_rec_backward(_lib.ptr(dgates), _lib.ptr(w_hh.contiguous()), _lib.ptr(cs), _lib.ptr(d_out),
                                             _lib.ptr(dh), _lib.ptr(dc), _lib.ptr(scratch), T, B, H, sp),
                       "lstm_rec_backward")
            _lib.count(1)
        else:
            for t in range(T - 1, -1, -1):
                if d_out is not None:
                    dh = dh + d_out[t]
                _lib.check(lib.lstm_cell_bwd(_lib.ptr(dgates[t]), _lib.ptr(cs[t]), _lib.ptr(cs[t + 1]), _lib.ptr(dh),
                                             _lib.ptr(dc), B, H, sp), "lstm_cell_bwd")
                dh = dgates[t] @ w_hh
        dg2 = dgates.view(T * B, 4 * H)
        x2, h2 = x.reshape(T * B, -1), hs[:-1].reshape(T * B, H)
        if _big(T * B, 4 * H, x2.shape[1]):
            dgs = split_pad(dg2)
            m, k = x2.shape
            # (no split-K: its partial sums meet in atomics, and this layer promises run-to-run identical bits)
            dx = gemm_x3(dgs, split_pad(w_ih), b_mn=True,
                         out=torch.empty((m, k), dtype=torch.float32, device=x.device)).view_as(x)
            # weight gradients: the reduction runs over the T * B rows
            dw_ih = gemm_x3(dgs, split_pad(x2), a_mn=True, b_mn=True,
                            out=torch.empty_like(w_ih, memory_format=torch.contiguous_format))
            dw_hh = gemm_x3(dgs, split_pad(h2), a_mn=True, b_mn=True,
                            out=torch.empty_like(w_hh, memory_format=torch.contiguous_format))
        else:
            dx = (dg2 @ w_ih).view_as(x)
            dw_ih = dg2.t() @ x2
            dw_hh = dg2.t() @ h2
        db = dg2.sum(dim=0)
        return dx, dh, dc, dw_ih, dw_hh, db, db.clone()


def lstm_supported(m, x) -> bool:
    return (x.dim() == 3 and not m.bidirectional and not m.batch_first and m.bias and m.proj_size == 0
            and x.dtype == torch.float32 and x.is_cuda)


def lstm_native(m, x, hx=None):
    T, B, _ = x.shape
    L, H = m.num_layers, m.hidden_size
    if hx is None:
        z = x.new_zeros(L, B, H)
        hx = (z, z.clone())
    h0, c0 = hx
    out, hn, cn = x, [], []
    for l in range(L):
        w_ih, w_hh = getattr(m, f"weight_ih_l{l}"), getattr(m, f"weight_hh_l{l}")
        b_ih, b_hh = getattr(m, f"bias_ih_l{l}"), getattr(m, f"bias_hh_l{l}")
        out, h, c = _LSTMLayerFn.apply(out.contiguous(), h0[l], c0[l], w_ih, w_hh, b_ih, b_hh)
        hn.append(h)
        cn.append(c)
        if m.dropout > 0 and m.training and l < L - 1:
            out = F.dropout(out, p=m.dropout, training=True)
    return out, (torch.stack(hn), torch.stack(cn))
