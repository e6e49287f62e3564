"""Run one hand-written kernel a few times on a small, fixed case: the program that is put under
``ncu`` for the committed profile summaries, and a quick CUDA-event timing of the same case.

    python -m chocosgd_b200.tools.kernel_bench --case sign --elements 67108864
    python -m chocosgd_b200.tools.kernel_bench --case gemm --m 4096 --n 4096 --k 4096
    python -m chocosgd_b200.tools.kernel_bench --case conv --batch 128 --hw 32 --channels 16
    python -m chocosgd_b200.tools.kernel_bench --case wgrad --batch 128 --hw 32 --channels 16
    python -m chocosgd_b200.tools.kernel_bench --case bn --batch 128 --hw 32 --channels 16
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
    p.add_argument("--case", required=True, choices=("sign", "topk", "qsgd", "randk", "gemm", "conv", "wgrad", "bn"))
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
