"""Native LSTM (gate GEMMs + fused cell kernels) against torch.nn.LSTM, forward and backward."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("inp,hid,layers", [(64, 64, 2), (50, 30, 1), (650, 650, 2)])
def test_lstm_matches_torch(inp, hid, layers):
    from chocosgd_b200.ops import nn as nnn

    torch.manual_seed(0)
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    T, B = 7, 4
    m = nnn.LSTM(inp, hid, layers, dropout=0.0).cuda()
    x = torch.randn(T, B, inp, device="cuda", requires_grad=True)
    h0 = torch.randn(layers, B, hid, device="cuda") * 0.1
    c0 = torch.randn(layers, B, hid, device="cuda") * 0.1
    params = [x] + list(m.parameters())
    out_ref, (hn_ref, cn_ref) = m(x, (h0, c0))
    g = torch.randn_like(out_ref)
    loss_ref = (out_ref * g).sum() + hn_ref.sum() * 0.3 + cn_ref.sum() * 0.2
    grads_ref = torch.autograd.grad(loss_ref, params)
    nnn.set_native(True, which=("lstm",))
    try:
        out, (hn, cn) = m(x, (h0, c0))
        loss = (out * g).sum() + hn.sum() * 0.3 + cn.sum() * 0.2
        grads = torch.autograd.grad(loss, params)
    finally:
        nnn.set_native(False)
        torch.backends.cuda.matmul.allow_tf32 = True
        torch.backends.cudnn.allow_tf32 = True
    tol = 5e-3 if inp % 4 == 0 else 1e-4  # the tcgen05 GEMM rounds its inputs to TF32
    for a, b in [(out, out_ref), (hn, hn_ref), (cn, cn_ref)] + list(zip(grads, grads_ref)):
        assert (a - b).abs().max() <= tol * (b.abs().max() + 1e-3), (a - b).abs().max()
