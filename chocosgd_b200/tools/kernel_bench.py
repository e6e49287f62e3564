"""Run one hand-written kernel a few times on a small, fixed case: the program that is put under
``ncu`` for the committed profile summaries, and a quick CUDA-event timing of the same case.

    python -m chocosgd_b200.tools.kernel_bench --case sign --elements 67108864
    python -m chocosgd_b200.tools.kernel_bench --case gemm --m 4096 --n 4096 --k 4096
    python -m chocosgd_b200.tools.kernel_bench --case conv --batch 128 --hw 32 --channels 16
    python -m chocosgd_b200.tools.kernel_bench --case wgrad --batch 128 --hw 32 --channels 16
    python -m chocosgd_b200.tools.kernel_bench --case bn --batch 128 --hw 32 --channels 16
    python -m chocosgd_b200.tools.kernel_bench --case bn16 --batch 64 --hw 112 --channels 64        # bf16, forward + backward
    python -m chocosgd_b200.tools.kernel_bench --case wgrad_gen --batch 128 --hw 16 --channels 32   # also --ks 1|3 --stride 2
    python -m chocosgd_b200.tools.kernel_bench --case conv_s2 --batch 128 --hw 32 --channels 16    # strided forward + input gradient
    python -m chocosgd_b200.tools.kernel_bench --case maxpool --batch 64 --hw 112 --channels 64
    python -m chocosgd_b200.tools.kernel_bench --case stem --batch 64 --hw 224                     # 7x7 / 2 bf16 stem, forward and wgrad
"""
from __future__ import annotations

import argparse
import json

import torch


def timed(fn, iters):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    flush = torch.empty(64 * 1024 * 1024, dtype=torch.float32, device="cuda")  # 256 MB > L2
    ms = []
    for _ in range(iters):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ms.append(e0.elapsed_time(e1))
    ms.sort()
    return ms[len(ms) // 2]


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--case", required=True, choices=("sign", "topk", "qsgd", "randk", "gemm", "conv", "wgrad", "bn", "bn16", "wgrad_gen",
                                                    "conv_s2", "maxpool", "stem"))
    p.add_argument("--ks", type=int, default=3)
    p.add_argument("--stride", type=int, default=1)
    p.add_argument("--elements", type=int, default=64 * 1024 * 1024)
    p.add_argument("--m", type=int, default=4096)
    p.add_argument("--n", type=int, default=4096)
    p.add_argument("--k", type=int, default=4096)
    p.add_argument("--batch", type=int, default=128)
    p.add_argument("--hw", type=int, default=32)
    p.add_argument("--channels", type=int, default=16)
    p.add_argument("--iters", type=int, default=5)
    a = p.parse_args(argv)
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    out = {"case": a.case}
    if a.case in ("sign", "topk", "qsgd", "randk"):
        from ..compress.segments import Segments
        from ..ops.gossip import ChocoEngine, RankBuffers
        from ..parallel.symm import LoopbackMailbox

        op = {"sign": "sign", "topk": "compress_top_k", "qsgd": "quantize_qsgd", "randk": "compress_random_k"}[a.case]
        seg = Segments.from_sizes([a.elements])
        mk = lambda: torch.zeros(seg.total, device=dev)
        x = torch.randn(seg.total, device=dev)
        bufs = {0: RankBuffers(x, mk(), mk(), mk(), mk())}
        kw = dict(compress_ratio=0.99) if "compress" in op else (dict(qsgd_levels=16) if op == "quantize_qsgd" else {})
        eng = ChocoEngine([0], bufs, {0: {0: 1.0}}, seg, [0.0], op, lambda pw: LoopbackMailbox({0: []}, pw, dev), dev, **kw)
        eng.set_hyper(0.0, 0.0, 0.5, False)
        ms = timed(eng.launch_step, a.iters)
        eng.flush()
        out.update(elements=a.elements, ms=ms, bytes_per_elem_model=32 + 3 / 8.0,
                   achieved_GBps=(32 + 3 / 8.0) * a.elements / ms / 1e6, kernels=eng.launches_per_step)
    elif a.case == "gemm":
        from ..ops.gemm import gemm, last_error

        A = torch.randn(a.m, a.k, device=dev)
        B = torch.randn(a.n, a.k, device=dev)
        C = torch.empty(a.m, a.n, device=dev)
        ms = timed(lambda: gemm(A, B, out=C), a.iters)
        torch.backends.cuda.matmul.allow_tf32 = True
        ms_lib = timed(lambda: torch.matmul(A, B.t(), out=C), a.iters)
        out.update(m=a.m, n=a.n, k=a.k, ms=ms, tflops=2.0 * a.m * a.n * a.k / ms / 1e9, ms_cublas_tf32=ms_lib,
                   tflops_cublas_tf32=2.0 * a.m * a.n * a.k / ms_lib / 1e9, error=last_error())
    elif a.case == "conv":
        import torch.nn.functional as F

        from ..ops.conv import conv3x3, last_error

        c = a.channels
        x = torch.randn(a.batch, c, a.hw, a.hw, device=dev).contiguous(memory_format=torch.channels_last)
        w = torch.randn(c, c, 3, 3, device=dev).contiguous(memory_format=torch.channels_last)
        ms = timed(lambda: conv3x3(x, w, c), a.iters)
        torch.backends.cudnn.benchmark = True
        ms_lib = timed(lambda: F.conv2d(x, w, padding=1), a.iters)
        flops = 2.0 * a.batch * a.hw * a.hw * c * c * 9
        out.update(batch=a.batch, hw=a.hw, channels=c, ms=ms, tflops=flops / ms / 1e9, ms_cudnn=ms_lib,
                   io_GBps=2 * x.numel() * 4 / ms / 1e6, error=last_error())
    elif a.case == "wgrad":
        import os

        from ..ops.conv import conv3x3_wgrad, last_error, wgrad_supported

        os.environ["CHOCO_WGRAD_TCGEN05"] = "1"
        c = a.channels
        assert wgrad_supported(a.batch, a.hw, a.hw, c, c)
        x = torch.randn(a.batch, c, a.hw, a.hw, device=dev).contiguous(memory_format=torch.channels_last)
        dy = torch.randn(a.batch, c, a.hw, a.hw, device=dev).contiguous(memory_format=torch.channels_last)
        w = torch.randn(c, c, 3, 3, device=dev).contiguous(memory_format=torch.channels_last)
        ms = timed(lambda: conv3x3_wgrad(x, dy, w), a.iters)
        torch.backends.cudnn.benchmark = True
        ms_lib = timed(lambda: torch.ops.aten.convolution_backward(
            dy, x, w, None, (1, 1), (1, 1), (1, 1), False, (0, 0), 1, (False, True, False)), a.iters)
        out.update(batch=a.batch, hw=a.hw, channels=c, ms=ms, ms_cudnn=ms_lib, io_GBps=2 * x.numel() * 4 / ms / 1e6,
                   error=last_error())
    elif a.case == "bn16":
        from ..ops import nn as nnn
        from ..ops.bn import bn_act

        c = a.channels
        x = torch.randn(a.batch, c, a.hw, a.hw, device=dev).bfloat16().contiguous(memory_format=torch.channels_last)
        x.requires_grad_()
        g = torch.randn_like(x)
        bn = torch.nn.BatchNorm2d(c).cuda().train()
        nnn.set_native(True, which=("bn",))

        def both():
            y = bn_act(bn, x, None, True)
            y.backward(g)
            x.grad = None

        def lib():
            y = torch.relu(bn(x))
            y.backward(g)
            x.grad = None

        ms = timed(both, a.iters)
        nnn.set_native(False)
        ms_lib = timed(lib, a.iters)
        nbytes = x.numel() * 2
        out.update(batch=a.batch, hw=a.hw, channels=c, ms=ms, ms_library=ms_lib, tensor_MB=nbytes / 1e6,
                   # tensors moved: reduce 1, apply 2, backward reduce 2, backward apply 3 (ReLU without a
                   # residual: the backward recomputes the mask from x and never reads y)
                   io_GBps=(1 + 2 + 2 + 3) * nbytes / ms / 1e6)
    elif a.case == "wgrad_gen":
        from ..ops.conv import conv_wgrad_gen, last_error

        cin = a.channels
        cout = cin if a.stride == 1 else 2 * cin
        ho = a.hw // a.stride
        x = torch.randn(a.batch, cin, a.hw, a.hw, device=dev).contiguous(memory_format=torch.channels_last)
        dy = torch.randn(a.batch, cout, ho, ho, device=dev).contiguous(memory_format=torch.channels_last)
        w = torch.randn(cout, cin, a.ks, a.ks, device=dev).contiguous(memory_format=torch.channels_last)
        ms = timed(lambda: conv_wgrad_gen(x, dy, w, a.ks, a.stride), a.iters)
        torch.backends.cudnn.benchmark = True
        geom = ((a.stride, a.stride), (a.ks // 2, a.ks // 2), (1, 1), False, (0, 0), 1)
        ms_lib = timed(lambda: torch.ops.aten.convolution_backward(dy, x, w, None, *geom, (False, True, False)), a.iters)
        out.update(batch=a.batch, hw=a.hw, cin=cin, cout=cout, ks=a.ks, stride=a.stride, ms=ms, ms_library=ms_lib,
                   io_GBps=(x.numel() + dy.numel()) * 4 / ms / 1e6, error=last_error())
    elif a.case == "conv_s2":
        import torch.nn.functional as F

        from ..ops.conv import _ConvGenFn, last_error

        cin, cout = a.channels, 2 * a.channels
        x = torch.randn(a.batch, cin, a.hw, a.hw, device=dev).contiguous(memory_format=torch.channels_last).requires_grad_()
        w = torch.randn(cout, cin, 3, 3, device=dev).contiguous(memory_format=torch.channels_last)
        g = torch.randn(a.batch, cout, a.hw // 2, a.hw // 2, device=dev).contiguous(memory_format=torch.channels_last)

        def ours():
            y = _ConvGenFn.apply(x, w, 3, 2, False)
            (gx,) = torch.autograd.grad(y, x, g)
            return gx

        def lib():
            y = F.conv2d(x, w, stride=2, padding=1)
            (gx,) = torch.autograd.grad(y, x, g)
            return gx

        ms = timed(ours, a.iters)
        torch.backends.cudnn.benchmark = True
        ms_lib = timed(lib, a.iters)
        out.update(batch=a.batch, hw=a.hw, cin=cin, cout=cout, ms_fwd_plus_dgrad=ms, ms_library=ms_lib, error=last_error())
    elif a.case == "stem":
        from ..ops.conv import _ConvStemFn, stem_last_error

        x = torch.randn(a.batch, 3, a.hw, a.hw, device=dev).contiguous(memory_format=torch.channels_last)
        w = (0.05 * torch.randn(64, 3, 7, 7, device=dev)).contiguous(memory_format=torch.channels_last).requires_grad_()
        g = torch.randn(a.batch, 64, a.hw // 2, a.hw // 2, device=dev).bfloat16().contiguous(memory_format=torch.channels_last)
        state = {}

        def fwd():
            state["y"] = _ConvStemFn.apply(x, w)

        def bwd():
            state["y"].backward(g, retain_graph=True)
            w.grad = None

        def lib_fwd():
            with torch.autocast("cuda", dtype=torch.bfloat16):
                state["yl"] = torch.nn.functional.conv2d(x, w, None, 2, 3)

        def lib_bwd():
            state["yl"].backward(g, retain_graph=True)
            w.grad = None

        torch.backends.cudnn.benchmark = True
        ms_f = timed(fwd, a.iters)
        ms_b = timed(bwd, a.iters)
        ms_lf = timed(lib_fwd, a.iters)
        ms_lb = timed(lib_bwd, a.iters)
        byt_f = x.numel() * 4 + g.numel() * 2
        out.update(batch=a.batch, hw=a.hw, ms_fwd=ms_f, ms_wgrad=ms_b, ms_library_fwd=ms_lf, ms_library_wgrad=ms_lb,
                   fwd_GBps=byt_f / ms_f / 1e6, wgrad_GBps=byt_f / ms_b / 1e6, error=stem_last_error())
    elif a.case == "maxpool":
        from ..ops.pool import maxpool_native

        c = a.channels
        x = torch.randn(a.batch, c, a.hw, a.hw, device=dev).bfloat16().contiguous(memory_format=torch.channels_last)
        x.requires_grad_()
        g = torch.randn(a.batch, c, (a.hw + 1) // 2, (a.hw + 1) // 2, device=dev).bfloat16().contiguous(
            memory_format=torch.channels_last)

        def ours():
            maxpool_native(x).backward(g)
            x.grad = None

        def lib():
            torch.nn.functional.max_pool2d(x, 3, 2, 1).backward(g)
            x.grad = None

        out.update(batch=a.batch, hw=a.hw, channels=c, ms=timed(ours, a.iters), ms_library=timed(lib, a.iters))
    else:
        from ..ops import nn as nnn
        from ..ops.bn import bn_act

        c = a.channels
        x = torch.randn(a.batch, c, a.hw, a.hw, device=dev).contiguous(memory_format=torch.channels_last)
        bn = torch.nn.BatchNorm2d(c).cuda().train()
        nnn.set_native(True, which=("bn",))
        with torch.no_grad():
            ms = timed(lambda: bn_act(bn, x, None, True), a.iters)
        out.update(batch=a.batch, hw=a.hw, channels=c, ms=ms, io_GBps=3 * x.numel() * 4 / ms / 1e6)
    print(json.dumps(out))


if __name__ == "__main__":
    main()
