"""LeNet-5 style network: 3 conv (5x5) + 2 FC (``dl_code/pcode/models/lenet.py:9-93``)."""
from __future__ import annotations

from collections import OrderedDict

import torch.nn as nn

from . import layers as L


class LeNet(nn.Module):
    def __init__(self, dataset="cifar10"):
        super().__init__()
        self.dataset = dataset
        self.num_classes = L.num_classes_of(dataset)
        c_in = 1 if dataset == "mnist" else 3
        self.convnet = nn.Sequential(
            OrderedDict(
                [
                    ("conv1", L.Conv2d(c_in, 6, kernel_size=(5, 5))),
                    ("relu1", L.ReLU()),
                    ("s2", L.MaxPool2d(kernel_size=(2, 2), stride=2)),
                    ("conv3", L.Conv2d(6, 16, kernel_size=(5, 5))),
                    ("relu3", L.ReLU()),
                    ("s4", L.MaxPool2d(kernel_size=(2, 2), stride=2)),
                    ("conv5", L.Conv2d(16, 120, kernel_size=(5, 5))),
                    ("relu5", L.ReLU()),
                ]
            )
        )
        self.fc = nn.Sequential(
            OrderedDict([("fc6", L.Linear(120, 84)), ("relu6", L.ReLU()), ("fc7", L.Linear(84, self.num_classes))])
        )

    def forward(self, x):
        out = self.convnet(x)
        return self.fc(out.reshape(x.size(0), -1))


def lenet(conf):
    return LeNet(dataset=conf.data)
