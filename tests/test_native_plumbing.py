"""Host-side plumbing around the native kernels that can be checked without a GPU: layer selection,
fused batch-norm step counters, fall-backs of the fused layer calls."""
import torch
import torch.nn.functional as F


def test_configure_native_without_cuda_disables_everything():
    from chocosgd_b200.ops import nn as nnn

    nnn.configure_native("auto")
    if not torch.cuda.is_available():
        assert not any(nnn.native_enabled(k) for k in ("bn", "conv", "wgrad", "ce", "linear", "lstm"))
    nnn.configure_native("off")
    assert not any(nnn.native_enabled(k) for k in ("bn", "conv", "wgrad", "ce", "linear", "lstm"))
    assert set(nnn.AUTO_KINDS) <= set(nnn.available_kinds())


def test_bn_counters_advance_once_per_step_and_survive_state_dict():
    from chocosgd_b200.models import layers as L
    from chocosgd_b200.ops.bn import BnCounters

    torch.manual_seed(0)
    net = torch.nn.Sequential(L.Conv2d(3, 8, 3, padding=1, bias=False), L.BatchNorm2d(8), torch.nn.ReLU(),
                              L.Conv2d(8, 8, 3, padding=1, bias=False), L.BatchNorm2d(8))
    counters = BnCounters(net)
    bns = [m for m in net.modules() if isinstance(m, torch.nn.BatchNorm2d)]
    x = torch.randn(4, 3, 6, 6)
    net.train()
    for step in range(1, 4):
        counters.tick()          # one add for all layers ...
        net(x)                   # ... and the library forward's own increment is compensated
        assert [int(b.num_batches_tracked) for b in bns] == [step, step]
    sd = net.state_dict()
    assert int(sd["1.num_batches_tracked"]) == 3
    net.load_state_dict(sd)
    counters.tick()
    net(x)
    assert [int(b.num_batches_tracked) for b in bns] == [4, 4]
    net.eval()
    net(x)
    assert [int(b.num_batches_tracked) for b in bns] == [4, 4]
    counters.release()


def test_conv_bn_act_falls_back_to_the_library_composition():
    from chocosgd_b200.models import layers as L

    torch.manual_seed(1)
    conv, bn = L.Conv2d(4, 6, 3, padding=1, bias=False), L.BatchNorm2d(6)
    bn_ref = torch.nn.BatchNorm2d(6)
    bn_ref.load_state_dict(bn.state_dict())
    x, res = torch.randn(2, 4, 5, 5), torch.randn(2, 6, 5, 5)
    out = L.conv_bn_act(conv, bn, x, residual=res, relu=True)
    ref = F.relu(bn_ref(F.conv2d(x, conv.weight, padding=1)) + res)
    torch.testing.assert_close(out, ref)
    torch.testing.assert_close(bn.running_var, bn_ref.running_var)


def test_plain_cross_entropy_detection():
    from chocosgd_b200.ops.ce import criterion_is_plain_ce

    assert criterion_is_plain_ce(torch.nn.CrossEntropyLoss())
    assert not criterion_is_plain_ce(torch.nn.CrossEntropyLoss(reduction="sum"))
    assert not criterion_is_plain_ce(torch.nn.CrossEntropyLoss(label_smoothing=0.1))
    assert not criterion_is_plain_ce(torch.nn.CrossEntropyLoss(weight=torch.ones(3)))
    assert not criterion_is_plain_ce(torch.nn.MSELoss())


def test_pdl_choice_follows_the_dtype_unless_the_environment_says_otherwise(monkeypatch):
    from chocosgd_b200.config import get_args
    from chocosgd_b200.ops import _lib

    assert get_args([]).pdl == "auto"
    for mode, bf16, want in (("auto", False, "0"), ("auto", True, "1"), ("on", False, "1"), ("off", True, "0")):
        monkeypatch.delenv("CHOCO_PDL", raising=False)
        assert _lib.configure_pdl(mode, bf16=bf16) == (want == "1")
        import os

        assert os.environ["CHOCO_PDL"] == want
    monkeypatch.setenv("CHOCO_PDL", "0")
    assert _lib.configure_pdl("on", bf16=True) is False          # an explicit environment setting wins


def test_stem_and_bf16_kernels_are_not_chosen_on_cpu():
    from chocosgd_b200.ops import nn as nnn
    from chocosgd_b200.ops.conv import stem_conv_supported

    conv = nnn.Conv2d(3, 64, kernel_size=7, stride=2, padding=3, bias=False)
    x = torch.randn(2, 3, 32, 32)
    assert not stem_conv_supported(conv, x)
    y = conv(x)                                                    # library path
    assert y.shape == (2, 64, 16, 16)
