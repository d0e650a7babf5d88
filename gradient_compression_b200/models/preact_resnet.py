"""Pre-activation ResNets for CIFAR (reference: models/preact_resnet.py:12-128): BN + ReLU precede every
convolution, shortcuts are a bare 1x1 convolution taken from the activated input."""
from __future__ import annotations

import torch.nn as nn

from ..ops.bn import bn_act, defer_batch_counters
from .layers import bn, conv, head_pool, linear


class PreActBlock(nn.Module):
    expansion = 1

    def __init__(self, in_planes, planes, stride=1):
        super().__init__()
        self.bn1, self.conv1 = bn(in_planes), conv(in_planes, planes, 3, stride, 1)
        self.bn2, self.conv2 = bn(planes), conv(planes, planes, 3, 1, 1)
        if stride != 1 or in_planes != self.expansion * planes:
            self.shortcut = nn.Sequential(conv(in_planes, self.expansion * planes, 1, stride))

    def forward(self, x):
        a = bn_act(self.bn1, x)
        skip = self.shortcut(a) if hasattr(self, "shortcut") else x
        y = self.conv2(bn_act(self.bn2, self.conv1(a)))
        return y + skip


class PreActBottleneck(nn.Module):
    expansion = 4

    def __init__(self, in_planes, planes, stride=1):
        super().__init__()
        self.bn1, self.conv1 = bn(in_planes), conv(in_planes, planes, 1)
        self.bn2, self.conv2 = bn(planes), conv(planes, planes, 3, stride, 1)
        self.bn3, self.conv3 = bn(planes), conv(planes, self.expansion * planes, 1)
        if stride != 1 or in_planes != self.expansion * planes:
            self.shortcut = nn.Sequential(conv(in_planes, self.expansion * planes, 1, stride))

    def forward(self, x):
        a = bn_act(self.bn1, x)
        skip = self.shortcut(a) if hasattr(self, "shortcut") else x
        y = self.conv2(bn_act(self.bn2, self.conv1(a)))
        y = self.conv3(bn_act(self.bn3, y))
        return y + skip


class PreActResNet(nn.Module):
    def __init__(self, block, num_blocks, num_classes=10):
        super().__init__()
        self.in_planes = 64
        self.conv1 = conv(3, 64, 3, 1, 1)
        for i, (width, depth, stride) in enumerate(zip((64, 128, 256, 512), num_blocks, (1, 2, 2, 2)), start=1):
            blocks = []
            for s in [stride] + [1] * (depth - 1):
                blocks.append(block(self.in_planes, width, s))
                self.in_planes = width * block.expansion
            setattr(self, f"layer{i}", nn.Sequential(*blocks))
        self.linear = linear(512 * block.expansion, num_classes)
        defer_batch_counters(self)

    def forward(self, x):
        x = self.layer4(self.layer3(self.layer2(self.layer1(self.conv1(x)))))
        return self.linear(head_pool(x, 4))


def PreActResNet18():
    return PreActResNet(PreActBlock, [2, 2, 2, 2])


def PreActResNet34():
    return PreActResNet(PreActBlock, [3, 4, 6, 3])


def PreActResNet50():
    return PreActResNet(PreActBottleneck, [3, 4, 6, 3])


def PreActResNet101():
    return PreActResNet(PreActBottleneck, [3, 4, 23, 3])


def PreActResNet152():
    return PreActResNet(PreActBottleneck, [3, 8, 36, 3])
