"""DenseNets for CIFAR (reference: models/densenet.py:9-104): BN-ReLU-1x1 / BN-ReLU-3x3 bottlenecks whose
outputs are concatenated in front of their inputs, halving transitions with 2x2 average pooling."""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops.bn import bn_act, defer_batch_counters
from .layers import bn, conv, linear


class Bottleneck(nn.Module):
    def __init__(self, in_planes, growth_rate):
        super().__init__()
        self.bn1, self.conv1 = bn(in_planes), conv(in_planes, 4 * growth_rate, 1)
        self.bn2, self.conv2 = bn(4 * growth_rate), conv(4 * growth_rate, growth_rate, 3, padding=1)

    def forward(self, x):
        y = self.conv1(bn_act(self.bn1, x))
        y = self.conv2(bn_act(self.bn2, y))
        return torch.cat([y, x], 1)


class Transition(nn.Module):
    def __init__(self, in_planes, out_planes):
        super().__init__()
        self.bn, self.conv = bn(in_planes), conv(in_planes, out_planes, 1)

    def forward(self, x):
        return F.avg_pool2d(self.conv(bn_act(self.bn, x)), 2)


class DenseNet(nn.Module):
    def __init__(self, block, nblocks, growth_rate=12, reduction=0.5, num_classes=10):
        super().__init__()
        self.growth_rate = growth_rate
        planes = 2 * growth_rate
        self.conv1 = conv(3, planes, 3, padding=1)
        for i, depth in enumerate(nblocks, start=1):
            layers = []
            for _ in range(depth):
                layers.append(block(planes, growth_rate))
                planes += growth_rate
            setattr(self, f"dense{i}", nn.Sequential(*layers))
            if i < len(nblocks):
                out_planes = int(math.floor(planes * reduction))
                setattr(self, f"trans{i}", Transition(planes, out_planes))
                planes = out_planes
        self.bn = bn(planes)
        self.linear = linear(planes, num_classes)
        defer_batch_counters(self)

    def forward(self, x):
        x = self.conv1(x)
        x = self.trans1(self.dense1(x))
        x = self.trans2(self.dense2(x))
        x = self.trans3(self.dense3(x))
        x = self.dense4(x)
        x = F.avg_pool2d(bn_act(self.bn, x), 4)
        return self.linear(x.flatten(1))


def DenseNet121():
    return DenseNet(Bottleneck, [6, 12, 24, 16], growth_rate=32)


def DenseNet169():
    return DenseNet(Bottleneck, [6, 12, 32, 32], growth_rate=32)


def DenseNet201():
    return DenseNet(Bottleneck, [6, 12, 48, 32], growth_rate=32)


def DenseNet161():
    return DenseNet(Bottleneck, [6, 12, 36, 24], growth_rate=48)


def densenet_cifar():
    return DenseNet(Bottleneck, [6, 12, 24, 16], growth_rate=12)
