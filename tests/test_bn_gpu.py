"""Fused BatchNorm(+residual)(+ReLU) kernels against the PyTorch composition (fp32, NHWC)."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape,use_res,relu", [((8, 16, 32, 32), False, True), ((128, 16, 32, 32), True, True),
                                                ((16, 64, 8, 8), True, True), ((4, 32, 16, 16), False, False),
                                                ((3, 128, 5, 7), True, True), ((128, 32, 16, 16), True, True),
                                                ((256, 64, 32, 32), False, True)])
def test_bn_act_matches_torch(shape, use_res, relu):
    from chocosgd_b200.ops import nn as nnn
    from chocosgd_b200.ops.bn import bn_act

    torch.manual_seed(0)
    C = shape[1]
    x = (torch.randn(shape, device="cuda") * 2 + 0.5).contiguous(memory_format=torch.channels_last).requires_grad_()
    res = torch.randn(shape, device="cuda").contiguous(memory_format=torch.channels_last).requires_grad_() if use_res else None
    bn_a, bn_b = torch.nn.BatchNorm2d(C).cuda(), torch.nn.BatchNorm2d(C).cuda()
    with torch.no_grad():
        bn_a.weight.uniform_(0.5, 1.5)
        bn_a.bias.uniform_(-0.5, 0.5)
        bn_b.load_state_dict(bn_a.state_dict())
    bn_a.train(), bn_b.train()
    ref = bn_a(x)
    if use_res:
        ref = ref + res
    if relu:
        ref = F.relu(ref)
    g = torch.randn_like(ref)
    ins = (x, bn_a.weight, bn_a.bias) + ((res,) if use_res else ())
    grads_ref = torch.autograd.grad(ref, ins, g)
    nnn.set_native(True, which=("bn",))
    try:
        out = bn_act(bn_b, x, res, relu)
        ins_b = (x, bn_b.weight, bn_b.bias) + ((res,) if use_res else ())
        grads = torch.autograd.grad(out, ins_b, g)
    finally:
        nnn.set_native(False)
    torch.testing.assert_close(out, ref, rtol=1e-4, atol=1e-4)
    for a, b in zip(grads, grads_ref):
        torch.testing.assert_close(a, b, rtol=2e-3, atol=2e-3 * float(b.abs().max()))
    torch.testing.assert_close(bn_b.running_mean, bn_a.running_mean, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(bn_b.running_var, bn_a.running_var, rtol=1e-4, atol=1e-5)
    assert int(bn_b.num_batches_tracked) == 1
    from chocosgd_b200.ops.bn import last_error

    assert last_error() == 0  # the grid barrier of the one-kernel backward never gave up


def test_one_kernel_backward_opt_in():
    """The grid-barrier backward (CHOCO_BN_BWD_FUSED=1, read once per process) against PyTorch."""
    import os
    import subprocess
    import sys

    code = r"""
import torch, torch.nn.functional as F
from chocosgd_b200.ops import nn as nnn
from chocosgd_b200.ops.bn import bn_act, last_error
torch.manual_seed(0)
for shape in ((128, 16, 32, 32), (64, 32, 16, 16), (16, 64, 8, 8)):
    C = shape[1]
    x = (torch.randn(shape, device="cuda") * 2 + 0.5).contiguous(memory_format=torch.channels_last).requires_grad_()
    res = torch.randn(shape, device="cuda").contiguous(memory_format=torch.channels_last).requires_grad_()
    a, b = torch.nn.BatchNorm2d(C).cuda(), torch.nn.BatchNorm2d(C).cuda()
    ref = F.relu(a(x) + res)
    g = torch.randn_like(ref)
    gr = torch.autograd.grad(ref, (x, a.weight, a.bias, res), g)
    nnn.set_native(True, which=("bn",))
    for _ in range(2):
        out = bn_act(b, x, res, True)
        gn = torch.autograd.grad(out, (x, b.weight, b.bias, res), g)
    nnn.set_native(False)
    for u, v in zip(gn, gr):
        torch.testing.assert_close(u, v, rtol=2e-3, atol=2e-3 * float(v.abs().max()))
assert last_error() == 0
print("ok")
"""
    env = dict(os.environ, CHOCO_BN_BWD_FUSED="1")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", code], env=env, cwd=root, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "ok" in r.stdout, r.stderr[-2000:]


@pytest.mark.parametrize("shape,use_res,relu", [((8, 64, 56, 56), False, True), ((4, 256, 28, 28), True, True),
                                                ((2, 2048, 7, 7), True, True), ((3, 512, 14, 14), True, False),
                                                ((16, 64, 112, 112), False, True), ((5, 1024, 9, 7), False, False)])
def test_bf16_bn_act_matches_fp32_reference(shape, use_res, relu):
    """bf16 activations (autocast ImageNet models): against the same composition computed in fp32 from
    the bf16 inputs; differences are the bf16 rounding of the stored outputs only."""
    from chocosgd_b200.ops import nn as nnn
    from chocosgd_b200.ops.bn import _BnAct16Fn, bn_act

    torch.manual_seed(0)
    C = shape[1]
    x = (torch.randn(shape, device="cuda") * 2 + 0.5).bfloat16().contiguous(memory_format=torch.channels_last).requires_grad_()
    res = None
    if use_res:
        res = torch.randn(shape, device="cuda").bfloat16().contiguous(memory_format=torch.channels_last).requires_grad_()
    bn_a, bn_b = torch.nn.BatchNorm2d(C).cuda(), torch.nn.BatchNorm2d(C).cuda()
    with torch.no_grad():
        bn_a.weight.uniform_(0.5, 1.5)
        bn_a.bias.uniform_(-0.5, 0.5)
        bn_b.load_state_dict(bn_a.state_dict())
    bn_a.train(), bn_b.train()
    xf = x.detach().float().requires_grad_()
    rf = res.detach().float().requires_grad_() if use_res else None
    ref = bn_a(xf)
    if use_res:
        ref = ref + rf
    if relu:
        ref = F.relu(ref)
    g = torch.randn_like(ref).bfloat16()
    ins_ref = (xf, bn_a.weight, bn_a.bias) + ((rf,) if use_res else ())
    grads_ref = torch.autograd.grad(ref, ins_ref, g.float())
    nnn.set_native(True, which=("bn",))
    try:
        out = bn_act(bn_b, x, res, relu)
        assert out.dtype == torch.bfloat16 and isinstance(out.grad_fn, _BnAct16Fn._backward_cls)
        ins = (x, bn_b.weight, bn_b.bias) + ((res,) if use_res else ())
        grads = torch.autograd.grad(out, ins, g)
    finally:
        nnn.set_native(False)
    from chocosgd_b200.ops.bn import last_error16

    assert last_error16() == 0
    torch.testing.assert_close(out.float(), ref, rtol=1e-2, atol=1e-2)            # bf16 has 8 bits of mantissa
    # a ReLU decision can differ where the pre-activation rounds to zero in bf16: compare in bulk
    for a, b in zip(grads, grads_ref):
        a, b = a.float(), b.float()
        assert (a - b).norm() <= 1e-2 * b.norm() + 1e-3, ((a - b).norm().item(), b.norm().item())
    torch.testing.assert_close(bn_b.running_mean, bn_a.running_mean, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(bn_b.running_var, bn_a.running_var, rtol=1e-4, atol=1e-5)
    assert int(bn_b.num_batches_tracked) == 1


_PDL_CODE = """
import sys, torch
from chocosgd_b200.ops import nn as nnn
from chocosgd_b200.ops.bn import bn_act, last_error16
from chocosgd_b200.ops.conv import stem_last_error
nnn.set_native(True, which=("conv", "bn", "pool"))
torch.manual_seed(0)
x = torch.randn(8, 3, 64, 64, device="cuda").contiguous(memory_format=torch.channels_last)
conv = nnn.Conv2d(3, 64, kernel_size=7, stride=2, padding=3, bias=False).cuda().to(memory_format=torch.channels_last)
bn, bn2, pool = nnn.BatchNorm2d(64).cuda(), nnn.BatchNorm2d(64).cuda(), nnn.MaxPool2d(3, 2, 1)
with torch.autocast("cuda", dtype=torch.bfloat16):
    y = pool(bn_act(bn, conv(x), None, True))
    z = bn_act(bn2, y, y, True)
z.float().square().mean().backward()
torch.cuda.synchronize()
assert last_error16() == 0 and stem_last_error() == 0
out = torch.cat([z.float().flatten(), conv.weight.grad.flatten(), bn.weight.grad, bn.bias.grad, bn2.weight.grad])
torch.save(out.cpu(), sys.argv[1])
"""


def test_bf16_chain_is_bitwise_the_same_with_programmatic_dependent_launch(tmp_path):
    """Stem convolution -> batch-norm -> max pooling -> batch-norm with residual, forward and backward, with
    the kernels launched in plain stream order and with programmatic dependencies (each kernel may become
    resident while its predecessor drains): same bits."""
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    outs = []
    for pdl in ("0", "1"):
        path = str(tmp_path / f"pdl{pdl}.pt")
        r = subprocess.run([sys.executable, "-c", _PDL_CODE, path], env=dict(os.environ, CHOCO_PDL=pdl), cwd=root,
                           capture_output=True, text=True, timeout=300)
        assert r.returncode == 0, r.stderr[-2000:]
        outs.append(torch.load(path))
    assert torch.isfinite(outs[0]).all() and torch.equal(outs[0], outs[1])
