"""tcgen05 implicit-GEMM 3x3 convolution (forward and input gradient) against PyTorch fp32."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

SHAPES = [(4, 16, 32, 32, 16), (2, 32, 16, 16, 32), (4, 64, 8, 8, 64), (8, 32, 32, 32, 64), (2, 64, 16, 16, 32),
          (128, 16, 32, 32, 16)]


@pytest.mark.parametrize("wgrad", [False, True])
@pytest.mark.parametrize("n,cin,h,w,cout", SHAPES)
def test_conv3x3_forward_and_dgrad(n, cin, h, w, cout, wgrad):
    from chocosgd_b200.ops import nn as nnn
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
