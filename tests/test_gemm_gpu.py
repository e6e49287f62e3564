"""tcgen05 / TMEM GEMM against an fp32 PyTorch reference (TF32 inputs: ~1e-3 relative)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b, a_mn, b_mn):
    A = a.t() if a_mn else a
    B = b.t() if b_mn else b
    return A.double() @ B.double().t()


def _check(M, N, K, a_mn, b_mn, split_k=1, bias=False):
    from chocosgd_b200.ops.gemm import gemm, last_error

    g = torch.Generator(device="cuda").manual_seed(M * 7 + N * 3 + K)
    a = torch.randn((K, M) if a_mn else (M, K), device="cuda", generator=g)
    b = torch.randn((K, N) if b_mn else (N, K), device="cuda", generator=g)
    bv = torch.randn(N, device="cuda", generator=g) if bias else None
    out = gemm(a, b, bv, a_mn=a_mn, b_mn=b_mn, split_k=split_k)
    torch.cuda.synchronize()
    assert last_error() == 0
    ref = _ref(a, b, a_mn, b_mn) + (bv.double() if bias else 0)
    err = (out.double() - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= 4e-3 * scale + 1e-3, (M, N, K, a_mn, b_mn, split_k, err, scale)


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
def test_gemm_layouts(a_mn, b_mn):
    _check(128, 64, 64, a_mn, b_mn)
    _check(256, 128, 96, a_mn, b_mn)
    _check(384, 32, 32, a_mn, b_mn)


def test_gemm_ragged_edges_and_bias():
    _check(200, 72, 100, False, False, bias=True)   # M, N, K tails
    _check(132, 260, 36, False, True)
    _check(100, 40, 1000, True, True)


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
def test_gemm_wide_tiles(a_mn, b_mn):
    """Shapes large enough for the 128 x 256 tiles (at least 120 of them), ragged N and K included."""
    _check(2048, 2048, 256, a_mn, b_mn)
    _check(1920, 2300, 200, a_mn, b_mn, bias=True)


def test_gemm_split_k():
    _check(64, 144, 8192, True, True, split_k=8)
    _check(128, 128, 4096, False, False, split_k=4)


def test_linear_native_matches_torch(monkeypatch):
    """Native Linear (forward, input gradient, weight gradient on the tcgen05 GEMM with split operands):
    row lengths that are not multiples of four, ragged tiles, fp32-grade accuracy against float64."""
    from chocosgd_b200.ops import gemm as G
    from chocosgd_b200.ops import nn as nnn

    monkeypatch.setattr(G, "MIN_NATIVE_WORK", 0)
    torch.manual_seed(0)
    for (m, k, n) in ((96, 512, 256), (1120, 650, 1330), (35, 70, 333)):
        lin = nnn.Linear(k, n).cuda()
        x = torch.randn(m, k, device="cuda", requires_grad=True)
        g = torch.randn(m, n, device="cuda")
        xd, wd, bd = x.detach().double().requires_grad_(), lin.weight.detach().double().requires_grad_(), \
            lin.bias.detach().double().requires_grad_()
        y_ref = torch.nn.functional.linear(xd, wd, bd)
        gx_ref, gw_ref, gb_ref = torch.autograd.grad(y_ref, (xd, wd, bd), g.double())
        nnn.set_native(True, which=("linear",))
        try:
            y = lin(x)
            assert y.shape == (m, n)
            gx, gw, gb = torch.autograd.grad(y, (x, lin.weight, lin.bias), g)
        finally:
            nnn.set_native(False)
        assert gw.is_contiguous() and gx.is_contiguous()
        for a, b in ((y, y_ref), (gx, gx_ref), (gw, gw_ref), (gb, gb_ref)):
            assert (a.double() - b).abs().max() <= 2e-5 * b.abs().max() + 1e-6, (m, k, n)
    assert G.last_error() == 0


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
def test_gemm_split_operands_reach_fp32_accuracy(a_mn, b_mn):
    from chocosgd_b200.ops.gemm import gemm, gemm_x3, last_error, split_pad

    g = torch.Generator(device="cuda").manual_seed(11)
    # (the two large cases run the persistent kernel, whose three passes share one load of each operand tile)
    for (M, N, K, split_k) in ((300, 270, 650, 1), (2048, 2304, 332, 1), (130, 70, 4099, 4), (4736, 2560, 650, 1),
                               (4700, 2300, 333, 1)):
        a = torch.randn((K, M) if a_mn else (M, K), device="cuda", generator=g)
        b = torch.randn((K, N) if b_mn else (N, K), device="cuda", generator=g)
        ah, al = split_pad(a)
        assert torch.equal(ah + al, a) and ah.stride(0) % 4 == 0
        out = gemm_x3((ah, al), split_pad(b), a_mn=a_mn, b_mn=b_mn, split_k=split_k)
        ref = _ref(a, b, a_mn, b_mn)
        err = (out.double() - ref).abs().max().item()
        # products carry 2^-21; the tensor core adds them in fp32 without rounding to nearest, so the
        # error grows with K (1.4e-5 of the largest entry at K = 4099)
        assert err <= 5e-5 * ref.abs().max().item(), (M, N, K, err)
        if M % 4 == 0 and N % 4 == 0 and K % 4 == 0:     # one TF32 pass is three orders less accurate
            err1 = (gemm(a, b, a_mn=a_mn, b_mn=b_mn).double() - ref).abs().max().item()
            assert err1 > 20 * err
    torch.cuda.synchronize()
    assert last_error() == 0


def test_gemm_persistent_variant():
    """The persistent kernel (default for large tile counts; CHOCO_GEMM_PERSISTENT is read once per process): all four operand
    layouts, ragged M / N / K, bias, 128- and 256-wide tiles, against float64."""
    import os
    import subprocess
    import sys

    code = r"""
import torch
from chocosgd_b200.ops.gemm import gemm, last_error
g = torch.Generator(device="cuda").manual_seed(5)
for (M, N, K, bias) in ((4736, 2080, 160, False), (4700, 2300, 100, True), (9600, 200, 72, True)):
    for a_mn in (False, True):
        for b_mn in (False, True):
            a = torch.randn((K, M) if a_mn else (M, K), device="cuda", generator=g)
            b = torch.randn((K, N) if b_mn else (N, K), device="cuda", generator=g)
            bv = torch.randn(N, device="cuda", generator=g) if bias else None
            out = gemm(a, b, bv, a_mn=a_mn, b_mn=b_mn)
            out2 = gemm(a, b, bv, a_mn=a_mn, b_mn=b_mn)
            A = (a.t() if a_mn else a).double(); B = (b.t() if b_mn else b).double()
            ref = A @ B.t() + (bv.double() if bias else 0)
            err = (out.double() - ref).abs().max().item()
            assert err <= 4e-3 * ref.abs().max().item() + 1e-3, (M, N, K, a_mn, b_mn, err)
            assert torch.equal(out, out2)
torch.cuda.synchronize()
assert last_error() == 0
print("ok")
"""
    env = dict(os.environ, CHOCO_GEMM_PERSISTENT="1")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", code], env=env, cwd=root, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "ok" in r.stdout, (r.stdout[-500:], r.stderr[-2000:])
