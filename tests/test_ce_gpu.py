"""Fused cross-entropy / accuracy kernel against the PyTorch fp32 ops."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(z, t):
    z = z.detach().clone().requires_grad_(True)
    loss = torch.nn.functional.cross_entropy(z, t)
    loss.backward()
    valid = t >= 0
    zt = z.detach()[valid].gather(1, t[valid].view(-1, 1))
    rank = (z.detach()[valid] > zt).sum(1)
    n = max(int(valid.sum()), 1)
    return loss.detach(), z.grad, 100.0 * float((rank < 1).sum()) / n, 100.0 * float((rank < 5).sum()) / n


@pytest.mark.parametrize("B,C", [(128, 10), (64, 1000), (35, 33278), (1, 7)])
def test_fused_cross_entropy_matches_torch(B, C):
    from chocosgd_b200.ops.ce import cross_entropy

    g = torch.Generator().manual_seed(B + C)
    z = (torch.randn(B, C, generator=g) * 3).cuda().requires_grad_(True)
    t = torch.randint(0, C, (B,), generator=g).cuda()
    for _ in range(2):  # second call: the arrival counter reset itself
        z.grad = None
        loss, stats = cross_entropy(z, t)
        (loss * 2.0).backward()
    l_ref, g_ref, top1, top5 = _ref(z, t)
    torch.testing.assert_close(loss.detach(), l_ref, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(z.grad, 2.0 * g_ref, rtol=1e-4, atol=1e-7)
    assert abs(float(stats[1]) - top1) < 1e-3 and abs(float(stats[2]) - top5) < 1e-3
    assert float(stats[3]) == B


def test_fused_cross_entropy_skips_ignored_rows():
    from chocosgd_b200.ops.ce import cross_entropy

    g = torch.Generator().manual_seed(3)
    z = torch.randn(40, 12, generator=g).cuda().requires_grad_(True)
    t = torch.randint(0, 12, (40,), generator=g).cuda()
    t[::4] = -100
    loss, stats = cross_entropy(z, t, True)
    loss.backward()
    l_ref, g_ref, top1, top5 = _ref(z, t)
    torch.testing.assert_close(loss.detach(), l_ref, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(z.grad, g_ref, rtol=1e-4, atol=1e-7)
    assert float(stats[3]) == 30 and abs(float(stats[1]) - top1) < 1e-3
