"""MLP: (Linear + BatchNorm1d + ReLU + Dropout) x L, bias-free classifier
(``dl_code/pcode/models/mlp.py:8-58``; its two size flags exist in this framework's parser)."""
from __future__ import annotations

import torch.nn as nn

from . import layers as L


FEATURE_SIZES = {"epsilon": 2000, "rcv1": 47236}   # LIBSVM feature sets (feature vectors, two classes)


class MLP(nn.Module):
    def __init__(self, dataset, num_layers, hidden_size, drop_rate):
        super().__init__()
        self.dataset, self.num_layers = dataset, num_layers
        self.num_classes = L.num_classes_of(dataset)
        if "mnist" in dataset:
            input_size = 28 * 28
        elif dataset in FEATURE_SIZES:
            input_size = FEATURE_SIZES[dataset]
        else:
            input_size = 32 * 32 * 3
        for i in range(1, num_layers + 1):
            layer = nn.Sequential(
                L.Linear(input_size if i == 1 else hidden_size, hidden_size),
                L.BatchNorm1d(hidden_size),
                L.ReLU(),
                L.Dropout(p=drop_rate),
            )
            setattr(self, "layer{}".format(i), layer)
        self.fc = L.Linear(hidden_size, self.num_classes, bias=False)

    def forward(self, x):
        out = x.reshape(x.size(0), -1)
        for i in range(1, self.num_layers + 1):
            out = getattr(self, "layer{}".format(i))(out)
        return self.fc(out)


def mlp(conf):
    return MLP(conf.data, conf.mlp_num_layers, conf.mlp_hidden_size, conf.drop_rate)
