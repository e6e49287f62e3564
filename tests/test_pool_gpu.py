"""Native 3x3 / stride 2 / pad 1 max pooling (NHWC, bf16 and fp32) against torch.nn.MaxPool2d."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(4, 64, 112, 112), (3, 16, 9, 7), (2, 8, 5, 6), (2, 24, 33, 32)])
def test_maxpool_forward_and_backward(shape, dtype):
    from chocosgd_b200.ops import nn as nnn
    from chocosgd_b200.ops.pool import _MaxPoolFn, maxpool_supported

    torch.manual_seed(0)
    m = nnn.MaxPool2d(kernel_size=3, stride=2, padding=1)
    x = torch.randn(shape, device="cuda").to(dtype).contiguous(memory_format=torch.channels_last).requires_grad_()
    # ties inside windows (bf16 has few distinct values; force some more)
    with torch.no_grad():
        x[:, :, ::3, ::2] = 0.5
    ref = torch.nn.functional.max_pool2d(x, 3, 2, 1)
    g = torch.randn_like(ref)
    (gx_ref,) = torch.autograd.grad(ref, x, g)
    assert maxpool_supported(m, x)
    nnn.set_native(True, which=("pool",))
    try:
        out = m(x)
        assert isinstance(out.grad_fn, _MaxPoolFn._backward_cls)
        (gx,) = torch.autograd.grad(out, x, g)
    finally:
        nnn.set_native(False)
    assert torch.equal(out, ref)
    torch.testing.assert_close(gx.float(), gx_ref.float(), rtol=1e-2 if dtype == torch.bfloat16 else 1e-6, atol=1e-2 if dtype == torch.bfloat16 else 1e-6)


def test_unsupported_pooling_falls_back():
    from chocosgd_b200.ops import nn as nnn

    m = nnn.MaxPool2d(kernel_size=2, stride=2)
    x = torch.randn(2, 8, 8, 8, device="cuda").contiguous(memory_format=torch.channels_last)
    nnn.set_native(True, which=("pool",))
    try:
        assert torch.equal(m(x), torch.nn.functional.max_pool2d(x, 2, 2))
    finally:
        nnn.set_native(False)
