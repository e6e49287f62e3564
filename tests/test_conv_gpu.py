"""tcgen05 implicit-GEMM 3x3 convolution (forward and input gradient) against PyTorch fp32."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

SHAPES = [(4, 16, 32, 32, 16), (2, 32, 16, 16, 32), (4, 64, 8, 8, 64), (8, 32, 32, 32, 64), (2, 64, 16, 16, 32),
          (128, 16, 32, 32, 16)]


@pytest.mark.parametrize("wgrad", [False, True])
@pytest.mark.parametrize("n,cin,h,w,cout", SHAPES)
def test_conv3x3_forward_and_dgrad(n, cin, h, w, cout, wgrad, monkeypatch):
    from chocosgd_b200.ops import nn as nnn

    monkeypatch.setenv("CHOCO_WGRAD_TCGEN05", "1")  # exercise the tcgen05 weight-gradient kernel too
    from chocosgd_b200.ops.conv import conv_supported, last_error

    torch.manual_seed(0)
    torch.backends.cudnn.allow_tf32 = False
    conv = nnn.Conv2d(cin, cout, 3, padding=1, bias=False).cuda().to(memory_format=torch.channels_last)
    x = torch.randn(n, cin, h, w, device="cuda").contiguous(memory_format=torch.channels_last).requires_grad_()
    assert conv_supported(conv, x)
    ref = F.conv2d(x, conv.weight, padding=1)
    g = torch.randn_like(ref)
    gx_ref, gw_ref = torch.autograd.grad(ref, (x, conv.weight), g)
    nnn.set_native(True, which=("conv", "wgrad") if wgrad else ("conv",))
    try:
        out = conv(x)
        gx, gw = torch.autograd.grad(out, (x, conv.weight), g)
    finally:
        nnn.set_native(False)
        torch.backends.cudnn.allow_tf32 = True
    torch.cuda.synchronize()
    assert last_error() == 0
    for a, b in ((out, ref), (gx, gx_ref), (gw, gw_ref)):
        err = (a - b).abs().max().item()
        assert err <= 5e-3 * b.abs().max().item() + 1e-3, (err, b.abs().max().item())


def test_unsupported_shapes_fall_back():
    from chocosgd_b200.ops import nn as nnn
    from chocosgd_b200.ops.conv import conv_supported

    conv = nnn.Conv2d(3, 16, 3, padding=1, bias=False).cuda().to(memory_format=torch.channels_last)
    x = torch.randn(2, 3, 32, 32, device="cuda").contiguous(memory_format=torch.channels_last)
    assert not conv_supported(conv, x)
    s2 = nnn.Conv2d(16, 32, 3, stride=2, padding=1, bias=False).cuda().to(memory_format=torch.channels_last)
    assert not conv_supported(s2, torch.randn(2, 16, 32, 32, device="cuda").contiguous(memory_format=torch.channels_last))
    from chocosgd_b200.ops.conv import any_conv_supported

    odd = nnn.Conv2d(24, 32, 3, padding=1, bias=False).cuda().to(memory_format=torch.channels_last)
    assert not any_conv_supported(odd, torch.randn(2, 24, 32, 32, device="cuda").contiguous(memory_format=torch.channels_last))


@pytest.mark.parametrize("n,cin,h,w,cout", SHAPES + [(128, 32, 16, 16, 32), (128, 64, 8, 8, 64)])
def test_conv_epilogue_statistics(n, cin, h, w, cout):
    """The persistent kernel's per-CTA (sum, sum of squares) rows add up to the statistics of y."""
    from chocosgd_b200.ops.conv import conv3x3_with_stats, last_error

    torch.manual_seed(1)
    x = torch.randn(n, cin, h, w, device="cuda").contiguous(memory_format=torch.channels_last)
    wt = (torch.randn(cout, cin, 3, 3, device="cuda") * 0.1).contiguous(memory_format=torch.channels_last)
    y, stats = conv3x3_with_stats(x, wt, cout)
    torch.cuda.synchronize()
    assert last_error() == 0
    torch.backends.cudnn.allow_tf32 = False
    try:
        ref = F.conv2d(x, wt, padding=1)
    finally:
        torch.backends.cudnn.allow_tf32 = True
    assert (y - ref).abs().max() <= 5e-3 * ref.abs().max() + 1e-3
    assert stats.shape[1] == 2 * cout and stats.shape[0] * 2 * cout <= 8192
    tot = stats.double().sum(0)
    s0 = y.double().sum(dim=(0, 2, 3))
    s1 = (y.double() ** 2).sum(dim=(0, 2, 3))
    torch.testing.assert_close(tot[:cout], s0, rtol=1e-4, atol=1e-2)
    torch.testing.assert_close(tot[cout:], s1, rtol=1e-4, atol=1e-2)


def _conv_bn_setup(seed=2):
    from chocosgd_b200.ops import nn as nnn

    torch.manual_seed(seed)
    conv = nnn.Conv2d(32, 32, 3, padding=1, bias=False).cuda().to(memory_format=torch.channels_last)
    bn = nnn.BatchNorm2d(32).cuda()
    bn.weight.data.uniform_(0.5, 1.5)
    bn.bias.data.uniform_(-0.5, 0.5)
    x = torch.randn(16, 32, 16, 16, device="cuda").contiguous(memory_format=torch.channels_last).requires_grad_()
    res = torch.randn(16, 32, 16, 16, device="cuda").contiguous(memory_format=torch.channels_last)
    return conv, bn, x, res


@pytest.mark.parametrize("residual", [False, True])
def test_conv_bn_matches_library_composition(residual):
    """conv -> batch-norm with the statistics taken from the convolution epilogue (+ residual),
    forward and backward, against the library ops.  No ReLU here: a TF32-sized difference in a
    pre-activation near zero flips its mask and changes the gradients by O(1) in either path."""
    from chocosgd_b200.ops import nn as nnn
    from chocosgd_b200.ops.bn import conv_bn_act

    conv, bn, x, res = _conv_bn_setup()
    res = res if residual else None
    bn_ref = torch.nn.BatchNorm2d(32).cuda()
    bn_ref.load_state_dict(bn.state_dict())
    torch.backends.cudnn.allow_tf32 = False
    try:
        r = bn_ref(F.conv2d(x, conv.weight, padding=1))
        r = r + res if residual else r
        g = torch.randn_like(r)
        ref = torch.autograd.grad(r, (x, conv.weight, bn_ref.weight, bn_ref.bias), g)
        nnn.set_native(True, which=("conv", "wgrad", "bn"))
        out = conv_bn_act(conv, bn, x, res, relu=False)
        got = torch.autograd.grad(out, (x, conv.weight, bn.weight, bn.bias), g)
    finally:
        nnn.set_native(False)
        torch.backends.cudnn.allow_tf32 = True
    pairs = [(out, r)] + list(zip(got, ref)) + [(bn.running_var, bn_ref.running_var), (bn.running_mean, bn_ref.running_mean)]
    for a, b in pairs:
        err = (a - b).abs().max().item()
        assert err <= 5e-3 * b.abs().max().item() + 1e-3, (err, b.abs().max().item())


def test_conv_bn_act_fused_equals_unfused_native():
    """With ReLU and residual: statistics from the convolution epilogue against the batch-norm
    kernel's own reduction over the same convolution output."""
    from chocosgd_b200.ops import nn as nnn
    from chocosgd_b200.ops.bn import bn_act, conv_bn_act

    conv, bn, x, res = _conv_bn_setup(3)
    g = torch.randn(16, 32, 16, 16, device="cuda").contiguous(memory_format=torch.channels_last)
    nnn.set_native(True, which=("conv", "wgrad", "bn"))
    try:
        a = conv_bn_act(conv, bn, x, res, relu=True)
        ga = torch.autograd.grad(a, (x, conv.weight, bn.weight, bn.bias), g)
        b = bn_act(bn, conv(x), res, True)
        gb = torch.autograd.grad(b, (x, conv.weight, bn.weight, bn.bias), g)
    finally:
        nnn.set_native(False)
    for u, v in [(a, b)] + list(zip(ga, gb)):
        assert (u - v).abs().max().item() <= 1e-4 * v.abs().max().item() + 1e-5


@pytest.mark.parametrize("n,h,w,cout", [(4, 32, 32, 16), (128, 32, 32, 16), (3, 17, 9, 32), (2, 8, 8, 64)])
def test_first_layer_convolution(n, h, w, cout):
    """3-channel first convolution (fp32 FMA kernels): forward, statistics rows, weight gradient."""
    from chocosgd_b200.ops import nn as nnn
    from chocosgd_b200.ops.conv import conv2d_native, first_conv_supported

    torch.manual_seed(4)
    conv = nnn.Conv2d(3, cout, 3, padding=1, bias=False).cuda().to(memory_format=torch.channels_last)
    x = torch.randn(n, 3, h, w, device="cuda").contiguous(memory_format=torch.channels_last)
    assert first_conv_supported(conv, x)
    torch.backends.cudnn.allow_tf32 = False
    try:
        ref = F.conv2d(x, conv.weight, padding=1)
        g = torch.randn_like(ref)
        (gw_ref,) = torch.autograd.grad(ref, (conv.weight,), g)
    finally:
        torch.backends.cudnn.allow_tf32 = True
    y, stats = conv2d_native(conv, x, want_stats=True)
    (gw,) = torch.autograd.grad(y, (conv.weight,), g)
    torch.testing.assert_close(y, ref, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(gw, gw_ref, rtol=1e-3, atol=1e-3 * float(gw_ref.abs().max()))
    tot = stats.double().sum(0)
    torch.testing.assert_close(tot[:cout], y.double().sum(dim=(0, 2, 3)), rtol=1e-4, atol=1e-2)
    torch.testing.assert_close(tot[cout:], (y.double() ** 2).sum(dim=(0, 2, 3)), rtol=1e-4, atol=1e-2)
    assert stats.shape[0] * 2 * cout <= 8192


def test_residual_blocks_with_fused_backward_epilogues():
    """Two identity blocks behind a stem: with the hand-over between layers (skip gradient added,
    ReLU mask applied and batch-norm backward sums taken in the input-gradient epilogue) every
    gradient equals the one of the same native kernels with self-contained layer backwards."""
    from chocosgd_b200.models.resnet import BasicBlock
    from chocosgd_b200.models import layers as L
    from chocosgd_b200.ops import _lib
    from chocosgd_b200.ops import nn as nnn
    from chocosgd_b200.ops.conv import FUSION, last_error

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.conv1 = L.Conv2d(16, 32, 3, padding=1, bias=False)
            self.bn1 = L.BatchNorm2d(32)
            self.b1, self.b2 = BasicBlock(32, 32), BasicBlock(32, 32)

        def forward(self, x):
            return self.b2(self.b1(L.conv_bn_act(self.conv1, self.bn1, x)))

    torch.manual_seed(5)
    net = Net().cuda().to(memory_format=torch.channels_last)
    for m in net.modules():
        if isinstance(m, torch.nn.BatchNorm2d):
            m.weight.data.uniform_(0.5, 1.5)
            m.bias.data.uniform_(-0.3, 0.3)
    x = torch.randn(32, 16, 16, 16, device="cuda").contiguous(memory_format=torch.channels_last).requires_grad_()
    g = torch.randn(32, 32, 16, 16, device="cuda").contiguous(memory_format=torch.channels_last)
    params = [p for p in net.parameters()]
    nnn.set_native(True, which=("conv", "wgrad", "bn"))
    results = {}
    try:
        for fused in (True, False):
            FUSION.enabled = fused
            FUSION.clear()
            net.train()
            n0 = _lib.LAUNCHES[0]
            out = net(x)
            grads = torch.autograd.grad(out, [x] + params, g)
            torch.cuda.synchronize()
            results[fused] = (out, grads, _lib.LAUNCHES[0] - n0)
    finally:
        FUSION.enabled = True
        FUSION.clear()
        nnn.set_native(False)
    assert last_error() == 0
    (out_f, gf, n_f), (out_u, gu, n_u) = results[True], results[False]
    assert torch.equal(out_f, out_u)
    for a, b in zip(gf, gu):
        assert (a - b).abs().max().item() <= 2e-4 * b.abs().max().item() + 1e-6
    # 5 batch-norm reductions (stem, b1.bn1, b1.bn2, b2.bn1; b2.bn2 has no native consumer: 4) fold away
    assert n_u - n_f == 4, (n_u, n_f)


@pytest.mark.parametrize("cin,hw,n", [(16, 32, 8), (32, 16, 6), (16, 32, 128)])
def test_downsampling_block_with_shortcut_gradient_in_the_strided_dgrad(cin, hw, n):
    """A stage's first block (3x3 / 2 convolution + 1x1 / 2 shortcut): the strided convolution's
    input-gradient launch also produces the shortcut's input gradient, applies the ReLU mask and
    leaves the batch-norm backward sums; compared with self-contained layer backwards (same native
    kernels) and with the library composition."""
    from chocosgd_b200.models import layers as L
    from chocosgd_b200.models.resnet import BasicBlock
    from chocosgd_b200.ops import nn as nnn
    from chocosgd_b200.ops.conv import FUSION, last_error

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.conv1 = L.Conv2d(cin, cin, 3, padding=1, bias=False)
            self.bn1 = L.BatchNorm2d(cin)
            ds = torch.nn.Sequential(L.Conv2d(cin, 2 * cin, kernel_size=1, stride=2, bias=False), L.BatchNorm2d(2 * cin))
            self.b1 = BasicBlock(cin, 2 * cin, 2, ds)

        def forward(self, x):
            return self.b1(L.conv_bn_act(self.conv1, self.bn1, x))

    torch.manual_seed(6)
    net = Net().cuda().to(memory_format=torch.channels_last)
    for m in net.modules():
        if isinstance(m, torch.nn.BatchNorm2d):
            m.weight.data.uniform_(0.5, 1.5)
            m.bias.data.uniform_(-0.3, 0.3)
    x = torch.randn(n, cin, hw, hw, device="cuda").contiguous(memory_format=torch.channels_last).requires_grad_()
    g = torch.randn(n, 2 * cin, hw // 2, hw // 2, device="cuda").contiguous(memory_format=torch.channels_last)
    params = [p for p in net.parameters()]
    results = {}
    torch.backends.cudnn.allow_tf32 = False
    try:
        for mode in ("fused", "unfused", "library"):
            nnn.set_native(mode != "library", which=("conv", "wgrad", "bn"))
            FUSION.enabled = mode == "fused"
            FUSION.clear()
            net.train()
            out = net(x)
            grads = torch.autograd.grad(out, [x] + params, g)
            torch.cuda.synchronize()
            results[mode] = (out, grads)
    finally:
        FUSION.enabled = True
        FUSION.clear()
        nnn.set_native(False)
        torch.backends.cudnn.allow_tf32 = True
    assert last_error() == 0
    assert torch.equal(results["fused"][0], results["unfused"][0])
    for a, b in zip(results["fused"][1], results["unfused"][1]):
        assert (a - b).abs().max().item() <= 2e-3 * b.abs().max().item() + 1e-5
    # against the library (fp32 convolutions): TF32 rounding flips a few ReLU decisions, which moves single
    # gradient entries by O(1); the bulk must agree
    for a, b in zip((results["fused"][0],) + tuple(results["fused"][1]), (results["library"][0],) + tuple(results["library"][1])):
        assert (a - b).norm().item() <= 6e-2 * b.norm().item() + 1e-4   # (0.1 % flipped entries = 3 % in L2)


GEN_SHAPES = [  # n, cin, h, w (input), cout, ks, stride
    (8, 16, 32, 32, 32, 3, 2), (128, 16, 32, 32, 32, 3, 2), (8, 32, 16, 16, 64, 3, 2), (128, 32, 16, 16, 64, 3, 2),
    (8, 16, 32, 32, 32, 1, 2), (128, 16, 32, 32, 32, 1, 2), (6, 32, 16, 16, 64, 1, 2), (128, 32, 16, 16, 64, 1, 2),
]


@pytest.mark.parametrize("n,cin,h,w,cout,ks,stride", GEN_SHAPES)
def test_strided_and_1x1_convolutions(n, cin, h, w, cout, ks, stride):
    """First convolution of a stage (3x3 / 2) and the down-sampling shortcut (1x1 / 2): forward with the
    batch statistics, weight gradient and input gradient against PyTorch fp32."""
    from chocosgd_b200.ops import nn as nnn
    from chocosgd_b200.ops.conv import _ConvGenFn, gen_conv_supported, last_error

    torch.manual_seed(3)
    torch.backends.cudnn.allow_tf32 = False
    conv = nnn.Conv2d(cin, cout, ks, stride=stride, padding=ks // 2, bias=False).cuda().to(memory_format=torch.channels_last)
    x = torch.randn(n, cin, h, w, device="cuda").contiguous(memory_format=torch.channels_last).requires_grad_()
    assert gen_conv_supported(conv, x)
    ref = F.conv2d(x, conv.weight, stride=stride, padding=ks // 2)
    g = torch.randn_like(ref)
    gx_ref, gw_ref = torch.autograd.grad(ref, (x, conv.weight), g)
    nnn.set_native(True, which=("conv", "wgrad"))
    try:
        out, stats = _ConvGenFn.apply(x, conv.weight, ks, stride, True)
        gx, gw = torch.autograd.grad(out, (x, conv.weight), g)
    finally:
        nnn.set_native(False)
        torch.backends.cudnn.allow_tf32 = True
    torch.cuda.synchronize()
    assert last_error() == 0
    for a, b in ((out, ref), (gx, gx_ref), (gw, gw_ref)):
        err = (a - b).abs().max().item()
        assert err <= 5e-3 * b.abs().max().item() + 1e-3, (err, b.abs().max().item())
    tot = stats.sum(0)
    torch.testing.assert_close(tot[:cout], out.sum((0, 2, 3)), rtol=1e-3, atol=1e-2)
    torch.testing.assert_close(tot[cout:], (out * out).sum((0, 2, 3)), rtol=1e-3, atol=1e-2)


@pytest.mark.parametrize("n,c,hw", [(8, 32, 16), (128, 32, 16), (8, 64, 8), (128, 64, 8), (3, 64, 8)])
def test_wgrad_warp_kernel_32_64_channels(n, c, hw):
    from chocosgd_b200.ops.conv import conv_wgrad_gen

    torch.manual_seed(4)
    x = torch.randn(n, c, hw, hw, device="cuda").contiguous(memory_format=torch.channels_last)
    dy = torch.randn(n, c, hw, hw, device="cuda").contiguous(memory_format=torch.channels_last)
    w = torch.zeros(c, c, 3, 3, device="cuda").contiguous(memory_format=torch.channels_last)
    torch.backends.cudnn.allow_tf32 = False
    try:
        ref = torch.ops.aten.convolution_backward(dy, x, w, None, (1, 1), (1, 1), (1, 1), False, (0, 0), 1,
                                                  (False, True, False))[1]
    finally:
        torch.backends.cudnn.allow_tf32 = True
    a = conv_wgrad_gen(x, dy, w, 3, 1)
    b = conv_wgrad_gen(x, dy, w, 3, 1)
    assert torch.equal(a, b)                      # fixed-order reduction: bitwise reproducible
    err = (a - ref).abs().max().item()
    assert err <= 5e-3 * ref.abs().max().item() + 1e-3, (err, ref.abs().max().item())


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(4, 64, 64), (3, 40, 56), (2, 224, 224)])
def test_stem_conv_bf16_matches_fp32_reference(shape):
    """7x7 / stride 2 stem on tcgen05 (bf16 operands, fp32 accumulation) against an fp32 convolution of the
    same bf16-rounded operands; the second shape has a ragged last tile."""
    from chocosgd_b200.ops import nn as nnn
    from chocosgd_b200.ops.conv import _ConvStemFn, stem_conv_supported, stem_last_error

    n, h, w = shape
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device="cpu").manual_seed(5)
    x = torch.randn(n, 3, h, w, generator=gen).to(dev).contiguous(memory_format=torch.channels_last)
    conv = nnn.Conv2d(3, 64, kernel_size=7, stride=2, padding=3, bias=False).to(dev).to(memory_format=torch.channels_last)
    g = torch.randn(n, 64, h // 2, w // 2, generator=gen).to(dev).bfloat16().contiguous(memory_format=torch.channels_last)
    nnn.set_native(True, which=("conv",))
    try:
        with torch.autocast("cuda", dtype=torch.bfloat16):
            assert stem_conv_supported(conv, x)
            y = conv(x)
    finally:
        nnn.set_native(False, which=("conv",))
    assert type(y.grad_fn).__name__.startswith("_ConvStemFn")
    assert y.dtype == torch.bfloat16 and y.is_contiguous(memory_format=torch.channels_last)
    y.backward(g)
    dw = conv.weight.grad.clone()
    assert stem_last_error() == 0

    old = torch.backends.cudnn.allow_tf32
    torch.backends.cudnn.allow_tf32 = False
    try:
        xr = x.bfloat16().float()
        wr = conv.weight.detach().bfloat16().float().requires_grad_()
        yr = F.conv2d(xr, wr, None, 2, 3)
        yr.backward(g.float())
    finally:
        torch.backends.cudnn.allow_tf32 = old
    # the result is rounded to bf16 once: half a unit in the last of 8 bits
    assert (y.float() - yr).abs().max().item() <= 2.0 ** -8 * yr.abs().max().item() + 1e-6
    rel = ((dw - wr.grad).norm() / wr.grad.norm()).item()
    assert rel < 1e-4, rel
    # bit-reproducible (fixed-order slice reduction)
    conv.weight.grad = None
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y2 = _ConvStemFn.apply(x, conv.weight)
    y2.backward(g)
    assert torch.equal(y2, y) and torch.equal(conv.weight.grad, dw)
