"""Pre-activation Wide ResNet (``dl_code/pcode/models/wideresnet.py:11-144``): depth 6n+4,
widths 16 / 16k / 32k / 64k."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import layers as L


class BasicBlock(nn.Module):
    def __init__(self, in_planes, out_planes, stride, drop_rate=0.0):
        super().__init__()
        self.bn1 = L.BatchNorm2d(in_planes)
        self.relu1 = L.ReLU(inplace=True)
        self.conv1 = L.Conv2d(in_planes, out_planes, kernel_size=3, stride=stride, padding=1, bias=False)
        self.bn2 = L.BatchNorm2d(out_planes)
        self.relu2 = L.ReLU(inplace=True)
        self.conv2 = L.Conv2d(out_planes, out_planes, kernel_size=3, stride=1, padding=1, bias=False)
        self.droprate = drop_rate
        self.equal_in_out = in_planes == out_planes
        self.conv_shortcut = (
            None if self.equal_in_out else L.Conv2d(in_planes, out_planes, kernel_size=1, stride=stride, bias=False)
        )

    def forward(self, x):
        act = self.relu1(self.bn1(x))
        if not self.equal_in_out:
            x = act
        out = self.relu2(self.bn2(self.conv1(act)))
        if self.droprate > 0:
            out = F.dropout(out, p=self.droprate, training=self.training)
        out = self.conv2(out)
        return torch.add(x if self.equal_in_out else self.conv_shortcut(x), out)


class NetworkBlock(nn.Module):
    def __init__(self, nb_layers, in_planes, out_planes, block, stride, drop_rate=0.0):
        super().__init__()
        self.layer = nn.Sequential(
            *[
                block(in_planes if i == 0 else out_planes, out_planes, stride if i == 0 else 1, drop_rate)
                for i in range(nb_layers)
            ]
        )

    def forward(self, x):
        return self.layer(x)


class WideResNet(nn.Module):
    def __init__(self, dataset, net_depth, widen_factor, drop_rate):
        super().__init__()
        assert (net_depth - 4) % 6 == 0
        self.dataset = dataset
        ch = [16, 16 * widen_factor, 32 * widen_factor, 64 * widen_factor]
        n = (net_depth - 4) // 6
        self.num_classes = L.num_classes_of(dataset)
        self.conv1 = L.Conv2d(3, ch[0], kernel_size=3, stride=1, padding=1, bias=False)
        self.block1 = NetworkBlock(n, ch[0], ch[1], BasicBlock, 1, drop_rate)
        self.block2 = NetworkBlock(n, ch[1], ch[2], BasicBlock, 2, drop_rate)
        self.block3 = NetworkBlock(n, ch[2], ch[3], BasicBlock, 2, drop_rate)
        self.bn1 = L.BatchNorm2d(ch[3])
        self.relu = L.ReLU(inplace=True)
        self.num_channels = ch[3]
        self.fc = L.Linear(ch[3], self.num_classes)
        L.he_init(self, zero_linear_bias=True)

    def forward(self, x):
        out = self.block3(self.block2(self.block1(self.conv1(x))))
        out = self.relu(self.bn1(out))
        out = F.avg_pool2d(out, 8)
        return self.fc(out.reshape(-1, self.num_channels))


def wideresnet(conf):
    if L.is_small_input(conf.data):
        return WideResNet(
            conf.data, int(conf.arch.replace("wideresnet", "")), conf.wideresnet_widen_factor, conf.drop_rate
        )
    raise NotImplementedError("wideresnet is defined for 32x32 inputs")
