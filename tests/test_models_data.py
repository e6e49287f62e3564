import numpy as np
import pytest
import torch

from chocosgd_b200.config import RunState, get_args
from chocosgd_b200.data import DataPartitioner, SyntheticImages, define_dataset
from chocosgd_b200.models import define_model
from chocosgd_b200.parallel.topology import Graph
from chocosgd_b200.train.metrics import Metrics, accuracy

COUNTS = {"resnet20": (272474, 65), "resnet50": (25557032, 161)}


@pytest.mark.parametrize("arch,data,shape", [
    ("resnet20", "cifar10", (2, 3, 32, 32)), ("resnet56", "cifar100", (2, 3, 32, 32)),
    ("resnet18", "imagenet", (1, 3, 224, 224)), ("resnet50", "imagenet", (1, 3, 224, 224)),
    ("densenet40", "cifar10", (2, 3, 32, 32)), ("wideresnet16", "cifar10", (2, 3, 32, 32)),
    ("vgg11_bn", "cifar10", (2, 3, 32, 32)), ("vgg13", "cifar100", (2, 3, 32, 32)), ("lenet", "cifar10", (2, 3, 32, 32)),
    ("mlp", "cifar10", (4, 3, 32, 32)),
])
def test_model_zoo_forward(arch, data, shape):
    conf = get_args(["--arch", arch, "--data", data])
    m = define_model(conf, consistent=False, verbose=False)
    m.eval()
    y = m(torch.randn(shape))
    assert y.shape == (shape[0], m.num_classes)
    if arch in COUNTS:
        n, t = COUNTS[arch]
        assert sum(p.numel() for p in m.parameters()) == n and len(list(m.parameters())) == t


def test_resnet20_bn_naming_rule():
    """38 of the 42 BatchNorm tensors carry 'bn' in their name (no weight decay); the 4 shortcut ones do not."""
    from chocosgd_b200.optim.base import build_param_groups

    m = define_model(get_args(["--arch", "resnet20"]), consistent=False, verbose=False)
    groups = build_param_groups(m, 1e-4)
    assert len(groups) == 65
    assert sum(1 for g in groups if g["weight_decay"] == 0.0) == 38
    assert all(g["weight_decay"] == 1e-4 for g in groups if "downsample" in g["name"])


def test_rnn_lm():
    conf = get_args(["--arch", "rnn_lm", "--rnn_n_hidden", "650", "--rnn_n_layers", "2", "--drop_rate", "0.4"])
    m = define_model(conf, data_loader={"n_tokens": 33278}, consistent=False, verbose=False)
    assert sum(p.numel() for p in m.parameters()) == 28434378 and len(list(m.parameters())) == 10
    assert m.decoder.weight is m.encoder.weight
    h = m.init_hidden(3)
    out, h2 = m(torch.randint(0, 33278, (5, 3)), h)
    assert out.shape == (5, 3, 33278) and h2[0].shape == (2, 3, 650)
    assert not m.repackage_hidden(h2)[0].requires_grad


def test_partitioner_random_and_sorted():
    ds = SyntheticImages((3, 4, 4), 10, 100, seed=0)
    part = DataPartitioner(ds, [0.25] * 4, "random", seed=5)
    idx = [set(part.use(r).indices) for r in range(4)]
    assert all(len(i) == 25 for i in idx) and len(set.union(*idx)) == 100
    again = DataPartitioner(ds, [0.25] * 4, "random", seed=5)
    assert list(again.use(2).indices) == list(part.use(2).indices)
    srt = DataPartitioner(ds, [0.25] * 4, "sorted", seed=5)
    labels = [int(ds.targets[i]) for i in srt.use(0).indices]
    assert max(labels) <= min(int(ds.targets[i]) for i in srt.use(3).indices)
    x, y = part.use(1)[0]
    assert x.shape == (3, 4, 4) and 0 <= y < 10


def test_define_dataset_epoch_length():
    conf = get_args(["--data", "synthetic_cifar10", "--synthetic_size", "256", "--batch_size", "16", "--num_workers", "0",
                     "--partition_data", "random", "--on_cuda", "False"])
    run = RunState()
    dl = define_dataset(conf, Graph("ring", 4, 1, on_cuda=False), run)
    assert run.num_batches_train_per_device_per_epoch == 4 and len(dl["train_loader"]) == 4
    conf2 = conf.replace(partition_data=None)
    run2 = RunState()
    define_dataset(conf2, Graph("ring", 4, 1, on_cuda=False), run2)
    assert run2.num_batches_train_per_device_per_epoch == 16 // 4


def test_bptt_iterator_and_nlp_dataset():
    conf = get_args(["--arch", "rnn_lm", "--data", "synthetic_wikitext2", "--synthetic_size", "20000", "--batch_size", "4",
                     "--rnn_bptt_len", "35", "--on_cuda", "False"])
    run = RunState()
    dl = define_dataset(conf, Graph("ring", 2, 0, on_cuda=False), run)
    x, y = next(iter(dl["train_loader"]))
    assert x.shape == (35, 8) and torch.equal(x[1:], y[:-1]) and dl["n_tokens"] == 33278
    assert run.num_batches_train_per_device_per_epoch == len(dl["train_loader"])


def test_metrics():
    out = torch.tensor([[0.1, 0.9, 0.0, 0.0, 0.0, 0.0], [0.8, 0.1, 0.05, 0.03, 0.01, 0.01]])
    tgt = torch.tensor([1, 5])
    top1, top5 = accuracy(out, tgt, (1, 5))
    assert float(top1) == 50.0 and float(top5) == 50.0

    class M:
        num_classes = 3

    assert Metrics(M()).metric_names == ["top1"]
    m = Metrics(M(), task="language_modeling")
    assert abs(float(m.evaluate(torch.tensor(2.0), None, None)[0]) - np.exp(2.0)) < 1e-4
