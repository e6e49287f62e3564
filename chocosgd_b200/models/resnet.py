"""ResNets for CIFAR-sized inputs (6n+2 layers) and ImageNet (18/34/50/101/152).

Architecture and parameter names follow ``dl_code/pcode/models/resnet.py:16-294`` (so the
``"bn" in name`` weight-decay rule and checkpoints carry over): CIFAR nets use widths
16/32/64 with ``(size-2)/6`` blocks per stage and bottlenecks from size 44; stride-2 stages
have a 1x1-conv + BN shortcut; AvgPool(8) + Linear."""
from __future__ import annotations

import torch.nn as nn

from . import layers as L


def _shortcut(downsample, x, fold_ds=False):
    """The skip connection: identity, or the (1x1 convolution, batch-norm) pair run as one fused pair
    (the convolution's epilogue yields the batch statistics)."""
    if downsample is None:
        return x
    if isinstance(downsample, nn.Sequential) and len(downsample) == 2 and isinstance(downsample[1], nn.BatchNorm2d):
        return L.conv_bn_act(downsample[0], downsample[1], x, relu=False, fold_ds=fold_ds)
    return downsample(x)


class BasicBlock(nn.Module):
    expansion = 1

    def __init__(self, in_planes, out_planes, stride=1, downsample=None):
        super().__init__()
        self.conv1 = L.conv3x3(in_planes, out_planes, stride)
        self.bn1 = L.BatchNorm2d(out_planes)
        self.relu = L.ReLU(inplace=True)
        self.conv2 = L.conv3x3(out_planes, out_planes)
        self.bn2 = L.BatchNorm2d(out_planes)
        self.downsample = downsample
        self.stride = stride

    def forward(self, x):
        # identity blocks on the native kernels: the skip gradient is added inside conv1's
        # input-gradient kernel instead of by a separate add
        fold = self.downsample is None and self.training and L.fold_residual_ok(self.conv1, x) \
            and L.fold_residual_ok(self.conv2, x)
        # down-sampling blocks: conv1's input-gradient kernel also computes the shortcut's
        fold_ds = self.downsample is not None and self.training and L.fold_shortcut_ok(self.conv1, self.downsample, x)
        out = L.conv_bn_act(self.conv1, self.bn1, x, fold_res=fold, fold_ds=fold_ds)
        # (the shortcut is evaluated after conv1: autograd then runs its backward before conv1's)
        residual = _shortcut(self.downsample, x, fold_ds)
        return L.conv_bn_act(self.conv2, self.bn2, out, residual=residual, fold_res=fold)


class Bottleneck(nn.Module):
    expansion = 4

    def __init__(self, in_planes, out_planes, stride=1, downsample=None):
        super().__init__()
        self.conv1 = L.Conv2d(in_planes, out_planes, kernel_size=1, bias=False)
        self.bn1 = L.BatchNorm2d(out_planes)
        self.conv2 = L.Conv2d(out_planes, out_planes, kernel_size=3, stride=stride, padding=1, bias=False)
        self.bn2 = L.BatchNorm2d(out_planes)
        self.conv3 = L.Conv2d(out_planes, out_planes * 4, kernel_size=1, bias=False)
        self.bn3 = L.BatchNorm2d(out_planes * 4)
        self.relu = L.ReLU(inplace=True)
        self.downsample = downsample
        self.stride = stride

    def forward(self, x):
        residual = _shortcut(self.downsample, x)
        out = L.conv_bn_act(self.conv1, self.bn1, x)
        out = L.conv_bn_act(self.conv2, self.bn2, out)
        return L.conv_bn_act(self.conv3, self.bn3, out, residual=residual)


class _ResNetBase(nn.Module):
    def _make_block(self, block_fn, planes, block_num, stride=1):
        downsample = None
        if stride != 1 or self.inplanes != planes * block_fn.expansion:
            downsample = nn.Sequential(
                L.Conv2d(self.inplanes, planes * block_fn.expansion, kernel_size=1, stride=stride, bias=False),
                L.BatchNorm2d(planes * block_fn.expansion),
            )
        blocks = [block_fn(self.inplanes, planes, stride, downsample)]
        self.inplanes = planes * block_fn.expansion
        blocks += [block_fn(self.inplanes, planes) for _ in range(1, block_num)]
        return nn.Sequential(*blocks)


class ResNetCifar(_ResNetBase):
    def __init__(self, dataset, resnet_size):
        super().__init__()
        if resnet_size % 6 != 2:
            raise ValueError("resnet_size must be 6n + 2:", resnet_size)
        n = (resnet_size - 2) // 6
        block_fn = Bottleneck if resnet_size >= 44 else BasicBlock
        self.dataset = dataset
        self.num_classes = L.num_classes_of(dataset)
        self.inplanes = 16
        self.conv1 = L.Conv2d(3, 16, kernel_size=3, stride=1, padding=1, bias=False)
        self.bn1 = L.BatchNorm2d(16)
        self.relu = L.ReLU(inplace=True)
        self.layer1 = self._make_block(block_fn, 16, n)
        self.layer2 = self._make_block(block_fn, 32, n, stride=2)
        self.layer3 = self._make_block(block_fn, 64, n, stride=2)
        self.avgpool = L.AvgPool2d(kernel_size=8)
        self.fc = L.Linear(64 * block_fn.expansion, self.num_classes)
        L.he_init(self)

    def forward_features(self, x):
        """The last feature map (before pooling); ``forward`` = ``classify(forward_features(x))``."""
        x = L.conv_bn_act(self.conv1, self.bn1, x)
        return self.layer3(self.layer2(self.layer1(x)))

    def classify(self, feat):
        x = self.avgpool(feat)
        return self.fc(x.reshape(x.size(0), -1))

    def forward(self, x):
        return self.classify(self.forward_features(x))

    def head_loss(self, feat, target):
        """Pooling + classifier + mean cross-entropy (+ top-1 / top-5) of a feature map in one kernel:
        ``(loss, stats)``, or None when the fused kernel does not cover the shapes / device."""
        from ..ops import head

        pool_all = feat.shape[-1] == feat.shape[-2] == self.avgpool.kernel_size
        if pool_all and head.supported(feat, self.fc.weight, target):
            return head.head_loss(feat, self.fc.weight, self.fc.bias, target)
        return None


class ResNetImagenet(_ResNetBase):
    CONFIGS = {
        18: (BasicBlock, [2, 2, 2, 2]),
        34: (BasicBlock, [3, 4, 6, 3]),
        50: (Bottleneck, [3, 4, 6, 3]),
        101: (Bottleneck, [3, 4, 23, 3]),
        152: (Bottleneck, [3, 8, 36, 3]),
    }

    def __init__(self, dataset, resnet_size):
        super().__init__()
        block_fn, nums = self.CONFIGS[resnet_size]
        self.dataset = dataset
        self.num_classes = L.num_classes_of(dataset)
        self.inplanes = 64
        self.conv1 = L.Conv2d(3, 64, kernel_size=7, stride=2, padding=3, bias=False)
        self.bn1 = L.BatchNorm2d(64)
        self.relu = L.ReLU(inplace=True)
        self.maxpool = L.MaxPool2d(kernel_size=3, stride=2, padding=1)
        self.layer1 = self._make_block(block_fn, 64, nums[0])
        self.layer2 = self._make_block(block_fn, 128, nums[1], stride=2)
        self.layer3 = self._make_block(block_fn, 256, nums[2], stride=2)
        self.layer4 = self._make_block(block_fn, 512, nums[3], stride=2)
        self.avgpool = L.AvgPool2d(kernel_size=7, stride=1)
        self.fc = L.Linear(512 * block_fn.expansion, self.num_classes)
        L.he_init(self)

    def forward(self, x):
        x = self.maxpool(L.conv_bn_act(self.conv1, self.bn1, x))
        x = self.layer4(self.layer3(self.layer2(self.layer1(x))))
        x = self.avgpool(x)
        return self.fc(x.reshape(x.size(0), -1))


def resnet(conf):
    size = int(conf.arch.replace("resnet", ""))
    if "imagenet" in conf.data and "downsampled" not in conf.data:
        return ResNetImagenet(conf.data, size)
    return ResNetCifar(conf.data, size)
