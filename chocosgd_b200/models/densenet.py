"""DenseNet / DenseNet-BC (``dl_code/pcode/models/densenet.py:12-208``): growth rate k,
three dense blocks for small inputs, optional bottleneck (BC) layers and channel compression
in the transitions."""
from __future__ import annotations

import math
from collections import OrderedDict

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import layers as L


class BasicLayer(nn.Module):
    def __init__(self, num_channels, growth_rate, drop_rate=0.0):
        super().__init__()
        self.bn1 = L.BatchNorm2d(num_channels)
        self.relu = L.ReLU(inplace=True)
        self.conv1 = L.Conv2d(num_channels, growth_rate, kernel_size=3, padding=1, bias=False)
        self.droprate = drop_rate

    def forward(self, x):
        out = self.conv1(self.relu(self.bn1(x)))
        if self.droprate > 0:
            out = F.dropout(out, p=self.droprate, training=self.training)
        return torch.cat((x, out), 1)


class Bottleneck(nn.Module):
    def __init__(self, num_channels, growth_rate, drop_rate=0.0):
        super().__init__()
        inter = 4 * growth_rate
        self.bn1 = L.BatchNorm2d(num_channels)
        self.relu = L.ReLU(inplace=True)
        self.conv1 = L.Conv2d(num_channels, inter, kernel_size=1, bias=False)
        self.bn2 = L.BatchNorm2d(inter)
        self.conv2 = L.Conv2d(inter, growth_rate, kernel_size=3, padding=1, bias=False)
        self.droprate = drop_rate

    def forward(self, x):
        out = self.conv1(self.relu(self.bn1(x)))
        if self.droprate > 0:
            out = F.dropout(out, p=self.droprate, training=self.training)
        out = self.conv2(self.relu(self.bn2(out)))
        if self.droprate > 0:
            out = F.dropout(out, p=self.droprate, training=self.training)
        return torch.cat((x, out), 1)


class Transition(nn.Module):
    def __init__(self, num_channels, num_out_channels, drop_rate=0.0):
        super().__init__()
        self.bn1 = L.BatchNorm2d(num_channels)
        self.relu = L.ReLU(inplace=True)
        self.conv1 = L.Conv2d(num_channels, num_out_channels, kernel_size=1, bias=False)
        self.droprate = drop_rate

    def forward(self, x):
        out = self.conv1(self.relu(self.bn1(x)))
        if self.droprate > 0:
            out = F.dropout(out, p=self.droprate, training=self.training)
        return F.avg_pool2d(out, 2)


class DenseNet(nn.Module):
    IMAGENET_BLOCKS = {121: [6, 12, 24, 16], 169: [6, 12, 32, 32], 201: [6, 12, 48, 32], 264: [6, 12, 64, 48]}

    def __init__(self, dataset, net_depth, growth_rate, bc_mode, compression, drop_rate):
        super().__init__()
        assert 0 < compression <= 1, "compression should be between 0 and 1."
        self.dataset = dataset
        self.num_classes = L.num_classes_of(dataset)
        small = L.is_small_input(dataset)
        self.avgpool_size = 8 if small else 7
        if small:
            per_block = (net_depth - 4) // 3
            if bc_mode:
                per_block //= 2
            block_config = [per_block] * 3
        else:
            block_config = self.IMAGENET_BLOCKS[net_depth]
        ch = 2 * growth_rate
        if small:
            self.features = nn.Sequential(OrderedDict([("conv0", L.Conv2d(3, ch, 3, 1, 1, bias=False))]))
        else:
            self.features = nn.Sequential(
                OrderedDict(
                    [
                        ("conv0", L.Conv2d(3, ch, kernel_size=7, stride=2, padding=3, bias=False)),
                        ("norm0", L.BatchNorm2d(ch)),
                        ("relu0", L.ReLU(inplace=True)),
                        ("pool0", L.MaxPool2d(kernel_size=3, stride=2, padding=1)),
                    ]
                )
            )
        for ind, num_layers in enumerate(block_config):
            layers_ = []
            for _ in range(int(num_layers)):
                layers_.append((Bottleneck if bc_mode else BasicLayer)(ch, growth_rate, drop_rate))
                ch += growth_rate
            self.features.add_module("denseblock%d" % (ind + 1), nn.Sequential(*layers_))
            if ind != len(block_config) - 1:
                out_ch = int(math.floor(ch * compression))
                self.features.add_module("transition%d" % (ind + 1), Transition(ch, out_ch, drop_rate))
                ch = out_ch
        self.features.add_module("norm_final", L.BatchNorm2d(ch))
        self.classifier = L.Linear(ch, self.num_classes)
        L.he_init(self, zero_linear_bias=True)

    def forward(self, x):
        f = self.features(x)
        out = F.relu(f, inplace=True)
        out = F.avg_pool2d(out, kernel_size=self.avgpool_size).reshape(f.size(0), -1)
        return self.classifier(out)


def densenet(conf):
    return DenseNet(
        conf.data,
        int(conf.arch.replace("densenet", "")),
        conf.densenet_growth_rate,
        conf.densenet_bc_mode,
        conf.densenet_compression,
        conf.drop_rate,
    )
