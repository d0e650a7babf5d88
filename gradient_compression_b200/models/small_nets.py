"""LeNet, GoogLeNet, MobileNet and MobileNetV2 for CIFAR (reference: models/lenet.py:6, googlenet.py:8-56,
mobilenet.py:11-35, mobilenetv2.py:12-56)."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops.bn import bn_act
from .layers import bn, conv, head_pool, linear


class LeNet(nn.Module):
    def __init__(self):
        super().__init__()
        self.conv1, self.conv2 = conv(3, 6, 5, bias=True), conv(6, 16, 5, bias=True)
        self.fc1, self.fc2, self.fc3 = linear(16 * 5 * 5, 120), linear(120, 84), linear(84, 10)

    def forward(self, x):
        x = F.max_pool2d(F.relu(self.conv1(x)), 2)
        x = F.max_pool2d(F.relu(self.conv2(x)), 2).flatten(1)
        return self.fc3(F.relu(self.fc2(F.relu(self.fc1(x)))))


class _ConvBNReLU(nn.Sequential):
    """Sequential of [conv, bn, relu]* (+ optional leading pool) evaluated with the fused BN+ReLU."""

    def forward(self, x):
        mods = list(self)
        i = 0
        while i < len(mods):
            m = mods[i]
            if isinstance(m, nn.BatchNorm2d) and i + 1 < len(mods) and isinstance(mods[i + 1], nn.ReLU):
                x, i = bn_act(m, x), i + 2
            else:
                x, i = m(x), i + 1
        return x


def _cbr(cin, cout, k, padding=0):
    return [conv(cin, cout, k, padding=padding, bias=True), bn(cout), nn.ReLU(True)]


class Inception(nn.Module):
    def __init__(self, in_planes, n1x1, n3x3red, n3x3, n5x5red, n5x5, pool_planes):
        super().__init__()
        self.b1 = _ConvBNReLU(*_cbr(in_planes, n1x1, 1))
        self.b2 = _ConvBNReLU(*_cbr(in_planes, n3x3red, 1), *_cbr(n3x3red, n3x3, 3, 1))
        self.b3 = _ConvBNReLU(*_cbr(in_planes, n5x5red, 1), *_cbr(n5x5red, n5x5, 3, 1), *_cbr(n5x5, n5x5, 3, 1))
        self.b4 = _ConvBNReLU(nn.MaxPool2d(3, stride=1, padding=1), *_cbr(in_planes, pool_planes, 1))

    def forward(self, x):
        return torch.cat([self.b1(x), self.b2(x), self.b3(x), self.b4(x)], 1)


class GoogLeNet(nn.Module):
    def __init__(self):
        super().__init__()
        self.pre_layers = _ConvBNReLU(*_cbr(3, 192, 3, 1))
        self.a3 = Inception(192, 64, 96, 128, 16, 32, 32)
        self.b3 = Inception(256, 128, 128, 192, 32, 96, 64)
        self.maxpool = nn.MaxPool2d(3, stride=2, padding=1)
        self.a4 = Inception(480, 192, 96, 208, 16, 48, 64)
        self.b4 = Inception(512, 160, 112, 224, 24, 64, 64)
        self.c4 = Inception(512, 128, 128, 256, 24, 64, 64)
        self.d4 = Inception(512, 112, 144, 288, 32, 64, 64)
        self.e4 = Inception(528, 256, 160, 320, 32, 128, 128)
        self.a5 = Inception(832, 256, 160, 320, 32, 128, 128)
        self.b5 = Inception(832, 384, 192, 384, 48, 128, 128)
        self.avgpool = nn.AvgPool2d(8, stride=1)
        self.linear = linear(1024, 10)

    def forward(self, x):
        x = self.b3(self.a3(self.pre_layers(x)))
        x = self.maxpool(x)
        x = self.e4(self.d4(self.c4(self.b4(self.a4(x)))))
        x = self.maxpool(x)
        x = self.avgpool(self.b5(self.a5(x)))
        return self.linear(x.flatten(1))


class _DWBlock(nn.Module):
    """depthwise 3x3 + pointwise 1x1, BN + ReLU after each (MobileNet v1)."""

    def __init__(self, in_planes, out_planes, stride=1):
        super().__init__()
        self.conv1, self.bn1 = conv(in_planes, in_planes, 3, stride, 1, groups=in_planes), bn(in_planes)
        self.conv2, self.bn2 = conv(in_planes, out_planes, 1), bn(out_planes)

    def forward(self, x):
        return bn_act(self.bn2, self.conv2(bn_act(self.bn1, self.conv1(x))))


class MobileNet(nn.Module):
    cfg = [64, (128, 2), 128, (256, 2), 256, (512, 2), 512, 512, 512, 512, 512, (1024, 2), 1024]

    def __init__(self, num_classes=10):
        super().__init__()
        self.conv1, self.bn1 = conv(3, 32, 3, 1, 1), bn(32)
        layers, cin = [], 32
        for item in self.cfg:
            cout, stride = (item, 1) if isinstance(item, int) else item
            layers.append(_DWBlock(cin, cout, stride))
            cin = cout
        self.layers = nn.Sequential(*layers)
        self.linear = linear(1024, num_classes)

    def forward(self, x):
        x = self.layers(bn_act(self.bn1, self.conv1(x)))
        return self.linear(head_pool(x, 2))


class _InvertedResidual(nn.Module):
    """expand 1x1 + depthwise 3x3 + linear 1x1 (MobileNetV2)."""

    def __init__(self, in_planes, out_planes, expansion, stride):
        super().__init__()
        self.stride = stride
        planes = expansion * in_planes
        self.conv1, self.bn1 = conv(in_planes, planes, 1), bn(planes)
        self.conv2, self.bn2 = conv(planes, planes, 3, stride, 1, groups=planes), bn(planes)
        self.conv3, self.bn3 = conv(planes, out_planes, 1), bn(out_planes)
        self.shortcut = nn.Sequential()
        if stride == 1 and in_planes != out_planes:
            self.shortcut = nn.Sequential(conv(in_planes, out_planes, 1), bn(out_planes))

    def forward(self, x):
        y = bn_act(self.bn1, self.conv1(x))
        y = bn_act(self.bn2, self.conv2(y))
        if self.stride == 1:
            return bn_act(self.bn3, self.conv3(y), residual=self.shortcut(x), relu=False)
        return bn_act(self.bn3, self.conv3(y), relu=False)


class MobileNetV2(nn.Module):
    # (expansion, out_planes, num_blocks, stride); the second stage keeps stride 1 for 32x32 inputs
    cfg = [(1, 16, 1, 1), (6, 24, 2, 1), (6, 32, 3, 2), (6, 64, 4, 2), (6, 96, 3, 1), (6, 160, 3, 2), (6, 320, 1, 1)]

    def __init__(self, num_classes=10):
        super().__init__()
        self.conv1, self.bn1 = conv(3, 32, 3, 1, 1), bn(32)
        layers, cin = [], 32
        for expansion, cout, n, stride in self.cfg:
            for s in [stride] + [1] * (n - 1):
                layers.append(_InvertedResidual(cin, cout, expansion, s))
                cin = cout
        self.layers = nn.Sequential(*layers)
        self.conv2, self.bn2 = conv(320, 1280, 1), bn(1280)
        self.linear = linear(1280, num_classes)

    def forward(self, x):
        x = self.layers(bn_act(self.bn1, self.conv1(x)))
        x = bn_act(self.bn2, self.conv2(x))
        return self.linear(head_pool(x, 4))
