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
