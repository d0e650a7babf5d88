"""CIFAR ResNets: 3x3 stem at stride 1, no max-pool, four stages of widths 64/128/256/512 with
strides 1/2/2/2, 4x4 average pool and a 10-way linear head (reference: models/resnet.py:14-129).
Attribute names match the reference so ``state_dict`` keys are interchangeable."""
from __future__ import annotations

import torch.nn as nn

from ..ops.bn import defer_batch_counters, flush_batch_counters
from ..ops.conv import GradLink, conv_bn_act
from ..ops.head import head_loss
from .layers import bn, conv, head_pool, linear


def _projection(cin, cout, stride):
    if stride == 1 and cin == cout:
        return nn.Sequential()
    return _Projection(conv(cin, cout, 1, stride=stride), bn(cout))


class _Projection(nn.Sequential):
    """1x1 convolution + batch norm of a shortcut; children are named "0" and "1" as in the reference."""

    def forward(self, x, donate=None):
        return conv_bn_act(self[0], self[1], x, relu=False, donate=donate)


class BasicBlock(nn.Module):
    expansion = 1

    def __init__(self, in_planes, planes, stride=1):
        super().__init__()
        self.conv1, self.bn1 = conv(in_planes, planes, 3, stride, 1), bn(planes)
        self.conv2, self.bn2 = conv(planes, planes, 3, 1, 1), bn(planes)
        self.shortcut = _projection(in_planes, planes * self.expansion, stride)

    def forward(self, x):
        identity = len(self.shortcut) == 0
        link = GradLink()
        y = conv_bn_act(self.conv1, self.bn1, x, link=link)
        return conv_bn_act(self.conv2, self.bn2, y, residual=link.residual(x) if identity else self.shortcut(x, donate=link))


class Bottleneck(nn.Module):
    expansion = 4

    def __init__(self, in_planes, planes, stride=1):
        super().__init__()
        self.conv1, self.bn1 = conv(in_planes, planes, 1), bn(planes)
        self.conv2, self.bn2 = conv(planes, planes, 3, stride, 1), bn(planes)
        self.conv3, self.bn3 = conv(planes, planes * self.expansion, 1), bn(planes * self.expansion)
        self.shortcut = _projection(in_planes, planes * self.expansion, stride)

    def forward(self, x):
        # every convolution: tensor-core kernel with BN statistics in its epilogue.  Two gradients meet at x: conv1's input
        # gradient and the skip connection's (identity block) or the projection shortcut's; the link lets conv1's GEMM add
        # onto the other one instead of autograd summing them in a pass of its own.
        identity = len(self.shortcut) == 0
        link = GradLink()
        y = conv_bn_act(self.conv1, self.bn1, x, link=link)
        y = conv_bn_act(self.conv2, self.bn2, y)
        return conv_bn_act(self.conv3, self.bn3, y, residual=link.residual(x) if identity else self.shortcut(x, donate=link))


class ResNet(nn.Module):
    def __init__(self, block, num_blocks, num_classes=10):
        super().__init__()
        self.in_planes = 64
        self.conv1, self.bn1 = conv(3, 64, 3, 1, 1), bn(64)
        for i, (width, depth, stride) in enumerate(zip((64, 128, 256, 512), num_blocks, (1, 2, 2, 2)), start=1):
            setattr(self, f"layer{i}", self._stage(block, width, depth, stride))
        self.linear = linear(512 * block.expansion, num_classes)
        defer_batch_counters(self)

    def _stage(self, block, planes, depth, stride):
        blocks = []
        for s in [stride] + [1] * (depth - 1):
            blocks.append(block(self.in_planes, planes, s))
            self.in_planes = planes * block.expansion
        return nn.Sequential(*blocks)

    def features(self, x):
        x = conv_bn_act(self.conv1, self.bn1, x)
        return self.layer4(self.layer3(self.layer2(self.layer1(x))))

    def forward(self, x):
        return self.linear(head_pool(self.features(x), 4))

    def forward_loss(self, x, labels):
        """``(loss, logits, [cross-entropy, top-1, top-5])``: pooling, the linear layer, the loss and the batch metrics in
        one kernel when the final map is 4 x 4 (``F.avg_pool2d(out, 4)`` then covers it whole, models/resnet.py:106)."""
        f = self.features(x)
        flush_batch_counters()          # (the forward hook that batches the BN step counters only fires for __call__)
        if f.shape[2] == 4 and f.shape[3] == 4:
            return head_loss(f, self.linear, labels)
        return head_loss(head_pool(f, 4)[:, :, None, None], self.linear, labels)


def ResNet18():
    return ResNet(BasicBlock, [2, 2, 2, 2])


def ResNet34():
    return ResNet(BasicBlock, [3, 4, 6, 3])


def ResNet50():
    return ResNet(Bottleneck, [3, 4, 6, 3])


def ResNet101():
    return ResNet(Bottleneck, [3, 4, 23, 3])


def ResNet152():
    return ResNet(Bottleneck, [3, 8, 36, 3])
