"""Model zoo and the ``define_model`` factory (``dl_code/pcode/create_model.py:8-102``)."""
from __future__ import annotations

import torch

from .densenet import DenseNet, densenet
from .lenet import LeNet, lenet
from .mlp import MLP, mlp
from .resnet import ResNetCifar, ResNetImagenet, resnet
from .rnn_lm import RNNLM
from .vgg import VGG, vgg
from .wideresnet import WideResNet, wideresnet

MODEL_NAMES = ("resnet", "wideresnet", "densenet", "vgg", "lenet", "mlp", "rnn_lm")


def define_cv_model(conf):
    arch = conf.arch
    if "wideresnet" in arch:
        return wideresnet(conf)
    if "resnet" in arch:
        return resnet(conf)
    if "densenet" in arch:
        return densenet(conf)
    if "vgg" in arch:
        return vgg(conf)
    if "lenet" in arch:
        return lenet(conf)
    if "mlp" in arch:
        return mlp(conf)
    raise NotImplementedError(arch)


def define_nlp_model(conf, n_tokens, emb_size=None, pretrained=None):
    emb = emb_size if emb_size is not None else conf.rnn_n_hidden
    model = RNNLM(
        ntoken=n_tokens,
        ninp=emb,
        nhid=conf.rnn_n_hidden,
        nlayers=conf.rnn_n_layers,
        tie_weights=conf.rnn_tie_weights,
        dropout=conf.drop_rate,
        weight_norm=conf.rnn_weight_norm,
    )
    if pretrained is not None:
        model.encoder.weight.data.copy_(pretrained)
    return model


def define_model(conf, graph=None, data_loader=None, device=None, consistent=True, verbose=True):
    """Build the model, move it to the device and give all ranks rank-0's weights."""
    from ..parallel.comm import consistent_model

    if "rnn_lm" in conf.arch:
        n_tokens = data_loader["n_tokens"]
        conf.n_tokens = n_tokens
        model = define_nlp_model(conf, n_tokens, data_loader.get("emb_size"), data_loader.get("vectors"))
    else:
        model = define_cv_model(conf)
    if device is not None:
        model = model.to(device)
        if getattr(conf, "channels_last", False) and str(device).startswith("cuda") and "rnn_lm" not in conf.arch:
            model = model.to(memory_format=torch.channels_last)
    if consistent:
        consistent_model(model, on_cuda=device is not None and str(device).startswith("cuda"))
    if verbose:
        rank = graph.rank if graph is not None else 0
        print(
            "=> creating model '{}'. total params for process {}: {}M".format(
                conf.arch, rank, sum(p.numel() for p in model.parameters() if p.requires_grad) / 1e6
            )
        )
    return model
