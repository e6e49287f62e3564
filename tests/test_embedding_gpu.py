"""Embedding lookup / gradient kernels against torch, stand-alone and with tied weights (deferred mode)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_lookup_and_gradient_match_torch():
    from chocosgd_b200.ops import nn as nnn
    from chocosgd_b200.ops.embedding import last_error

    torch.manual_seed(0)
    m = nnn.Embedding(500, 130).cuda()
    idx = torch.randint(0, 500, (35, 32), device="cuda")
    idx[:, :4] = 7                                  # many repeats of one token
    g = torch.randn(35, 32, 130, device="cuda")
    ref = torch.nn.functional.embedding(idx, m.weight)
    (gw_ref,) = torch.autograd.grad(ref, m.weight, g)
    nnn.set_native(True, which=("embed",))
    try:
        out = m(idx)
        (gw,) = torch.autograd.grad(out, m.weight, g)
        (gw2,) = torch.autograd.grad(m(idx), m.weight, g)
    finally:
        nnn.set_native(False)
    assert last_error() == 0
    assert torch.equal(out, ref)
    torch.testing.assert_close(gw, gw_ref, rtol=1e-5, atol=1e-5)
    assert torch.equal(gw, gw2)                     # fixed summation order


def test_tied_language_model_gradients_match_stock():
    """Tied encoder / decoder: the look-ups' gradient is added into the decoder's weight gradient by the
    parameter hook; compared with the stock layers on the same model."""
    from chocosgd_b200.models.rnn_lm import RNNLM
    from chocosgd_b200.ops import nn as nnn

    torch.manual_seed(1)
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    model = RNNLM(300, 64, 64, 2, dropout=0.0, tie_weights=True).cuda()
    model.train()
    idx = torch.randint(0, 300, (12, 8), device="cuda")
    tgt = torch.randint(0, 300, (12 * 8,), device="cuda")
    h = model.init_hidden(8)

    def grads():
        out, _ = model(idx, h)
        loss = torch.nn.functional.cross_entropy(out.view(-1, 300), tgt)
        for p in model.parameters():
            p.grad = None
        loss.backward()
        return float(loss), [p.grad.clone() for p in model.parameters()]

    try:
        l_ref, g_ref = grads()
        nnn.set_native(True, which=("embed",))
        l_a, g_a = grads()
        l_b, g_b = grads()
    finally:
        nnn.set_native(False)
        torch.backends.cuda.matmul.allow_tf32 = True
        torch.backends.cudnn.allow_tf32 = True
    assert abs(l_a - l_ref) < 1e-6
    for a, b, r in zip(g_a, g_b, g_ref):
        torch.testing.assert_close(a, r, rtol=1e-4, atol=1e-6)
    assert torch.equal(g_a[0], g_b[0])
    from chocosgd_b200.ops.embedding import PENDING

    assert not PENDING.items                        # nothing left waiting for a gradient
