"""VGG-11/13/16/19 with optional BatchNorm and a 512-512-C classifier for 32x32 inputs
(``dl_code/pcode/models/vgg.py:10-96``)."""
from __future__ import annotations

import torch.nn as nn

from . import layers as L

ARCHITECTURES = {
    "A": [64, "M", 128, "M", 256, 256, "M", 512, 512, "M", 512, 512, "M"],
    "B": [64, 64, "M", 128, 128, "M", 256, 256, "M", 512, 512, "M", 512, 512, "M"],
    "D": [64, 64, "M", 128, 128, "M", 256, 256, 256, "M", 512, 512, 512, "M", 512, 512, 512, "M"],
    "E": [64, 64, "M", 128, 128, "M", 256, 256, 256, 256, "M", 512, 512, 512, 512, "M", 512, 512, 512, 512, "M"],
}


class VGG(nn.Module):
    def __init__(self, nn_arch, dataset, use_bn=True):
        super().__init__()
        self.use_bn, self.nn_arch, self.dataset = use_bn, nn_arch, dataset
        self.num_classes = L.num_classes_of(dataset)
        mods, c_in = [], 3
        for v in ARCHITECTURES[nn_arch]:
            if v == "M":
                mods.append(L.MaxPool2d(kernel_size=2, stride=2))
            else:
                mods.append(L.Conv2d(c_in, v, kernel_size=3, padding=1))
                if use_bn:
                    mods.append(L.BatchNorm2d(v))
                mods.append(L.ReLU(inplace=True))
                c_in = v
        self.features = nn.Sequential(*mods)
        self.classifier = nn.Sequential(
            L.Dropout(), L.Linear(512, 512), L.ReLU(True), L.Dropout(), L.Linear(512, 512), L.ReLU(True),
            L.Linear(512, self.num_classes),
        )
        L.he_init(self)

    def forward(self, x):
        x = self.features(x)
        return self.classifier(x.reshape(x.size(0), -1))


def vgg(conf):
    use_bn = "bn" in conf.arch
    for key, arch in (("11", "A"), ("13", "B"), ("16", "D"), ("19", "E")):
        if key in conf.arch:
            return VGG(arch, conf.data, use_bn)
    raise NotImplementedError(conf.arch)
