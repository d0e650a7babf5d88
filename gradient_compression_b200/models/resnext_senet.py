"""ResNeXt-29, SENet-18, RegNet-X/Y and PNASNet for CIFAR (reference: models/resnext.py:10-105,
senet.py:10-110, regnet.py:12-147, pnasnet.py:12-125)."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops.bn import bn_act, defer_batch_counters
from .layers import bn, conv, head_pool, linear


def _proj(cin, cout, stride):
    return nn.Sequential(conv(cin, cout, 1, stride), bn(cout))


def _shortcut(seq, x):
    """Evaluate a (conv, bn) shortcut with the fused BN, or pass x through an empty one."""
    if len(seq) == 0:
        return x
    return bn_act(seq[1], seq[0](x), relu=False)


# ---------------------------------------------------------------------------------- ResNeXt
class _XBlock(nn.Module):
    expansion = 2

    def __init__(self, in_planes, cardinality=32, bottleneck_width=4, stride=1):
        super().__init__()
        gw = cardinality * bottleneck_width
        self.conv1, self.bn1 = conv(in_planes, gw, 1), bn(gw)
        self.conv2, self.bn2 = conv(gw, gw, 3, stride, 1, groups=cardinality), bn(gw)
        self.conv3, self.bn3 = conv(gw, self.expansion * gw, 1), bn(self.expansion * gw)
        self.shortcut = nn.Sequential()
        if stride != 1 or in_planes != self.expansion * gw:
            self.shortcut = _proj(in_planes, self.expansion * gw, stride)

    def forward(self, x):
        y = bn_act(self.bn1, self.conv1(x))
        y = bn_act(self.bn2, self.conv2(y))
        return bn_act(self.bn3, self.conv3(y), residual=_shortcut(self.shortcut, x))


class ResNeXt(nn.Module):
    def __init__(self, num_blocks, cardinality, bottleneck_width, num_classes=10):
        super().__init__()
        self.cardinality, self.bottleneck_width, self.in_planes = cardinality, bottleneck_width, 64
        self.conv1, self.bn1 = conv(3, 64, 1), bn(64)
        for i, (depth, stride) in enumerate(zip(num_blocks, (1, 2, 2)), start=1):
            blocks = []
            for s in [stride] + [1] * (depth - 1):
                blocks.append(_XBlock(self.in_planes, self.cardinality, self.bottleneck_width, s))
                self.in_planes = _XBlock.expansion * self.cardinality * self.bottleneck_width
            self.bottleneck_width *= 2
            setattr(self, f"layer{i}", nn.Sequential(*blocks))
        self.linear = linear(cardinality * bottleneck_width * 8, num_classes)
        defer_batch_counters(self)

    def forward(self, x):
        x = bn_act(self.bn1, self.conv1(x))
        x = self.layer3(self.layer2(self.layer1(x)))
        return self.linear(head_pool(x, 8))


def ResNeXt29_2x64d():
    return ResNeXt([3, 3, 3], 2, 64)


def ResNeXt29_4x64d():
    return ResNeXt([3, 3, 3], 4, 64)


def ResNeXt29_8x64d():
    return ResNeXt([3, 3, 3], 8, 64)


def ResNeXt29_32x4d():
    return ResNeXt([3, 3, 3], 32, 4)


# ---------------------------------------------------------------------------------- SENet
class _SEPreActBlock(nn.Module):
    """Pre-activation basic block with a squeeze-and-excitation gate (two 1x1 convolutions)."""

    def __init__(self, in_planes, planes, stride=1):
        super().__init__()
        self.bn1, self.conv1 = bn(in_planes), conv(in_planes, planes, 3, stride, 1)
        self.bn2, self.conv2 = bn(planes), conv(planes, planes, 3, 1, 1)
        if stride != 1 or in_planes != planes:
            self.shortcut = nn.Sequential(conv(in_planes, planes, 1, stride))
        self.fc1, self.fc2 = conv(planes, planes // 16, 1, bias=True), conv(planes // 16, planes, 1, bias=True)

    def forward(self, x):
        a = bn_act(self.bn1, x)
        skip = self.shortcut(a) if hasattr(self, "shortcut") else x
        y = self.conv2(bn_act(self.bn2, self.conv1(a)))
        gate = torch.sigmoid(self.fc2(F.relu(self.fc1(F.avg_pool2d(y, y.size(2))))))
        return y * gate + skip


class _SEBasicBlock(nn.Module):
    def __init__(self, in_planes, planes, stride=1):
        super().__init__()
        self.conv1, self.bn1 = conv(in_planes, planes, 3, stride, 1), bn(planes)
        self.conv2, self.bn2 = conv(planes, planes, 3, 1, 1), bn(planes)
        self.shortcut = nn.Sequential()
        if stride != 1 or in_planes != planes:
            self.shortcut = _proj(in_planes, planes, stride)
        self.fc1, self.fc2 = conv(planes, planes // 16, 1, bias=True), conv(planes // 16, planes, 1, bias=True)

    def forward(self, x):
        y = bn_act(self.bn1, self.conv1(x))
        y = bn_act(self.bn2, self.conv2(y), relu=False)
        gate = torch.sigmoid(self.fc2(F.relu(self.fc1(F.avg_pool2d(y, y.size(2))))))
        return F.relu(y * gate + _shortcut(self.shortcut, x))


class SENet(nn.Module):
    def __init__(self, block, num_blocks, num_classes=10):
        super().__init__()
        self.in_planes = 64
        self.conv1, self.bn1 = conv(3, 64, 3, 1, 1), bn(64)
        for i, (width, depth, stride) in enumerate(zip((64, 128, 256, 512), num_blocks, (1, 2, 2, 2)), start=1):
            blocks = []
            for s in [stride] + [1] * (depth - 1):
                blocks.append(block(self.in_planes, width, s))
                self.in_planes = width
            setattr(self, f"layer{i}", nn.Sequential(*blocks))
        self.linear = linear(512, num_classes)
        defer_batch_counters(self)

    def forward(self, x):
        x = bn_act(self.bn1, self.conv1(x))
        x = self.layer4(self.layer3(self.layer2(self.layer1(x))))
        return self.linear(head_pool(x, 4))


def SENet18():
    return SENet(_SEPreActBlock, [2, 2, 2, 2])


# ---------------------------------------------------------------------------------- RegNet
class _SE(nn.Module):
    def __init__(self, in_planes, se_planes, act=F.relu):
        super().__init__()
        self.se1, self.se2 = conv(in_planes, se_planes, 1, bias=True), conv(se_planes, in_planes, 1, bias=True)
        self._act = act

    def forward(self, x):
        gate = torch.sigmoid(self.se2(self._act(self.se1(F.adaptive_avg_pool2d(x, (1, 1))))))
        return x * gate


class _RegBlock(nn.Module):
    def __init__(self, w_in, w_out, stride, group_width, bottleneck_ratio, se_ratio):
        super().__init__()
        w_b = int(round(w_out * bottleneck_ratio))
        self.conv1, self.bn1 = conv(w_in, w_b, 1), bn(w_b)
        self.conv2, self.bn2 = conv(w_b, w_b, 3, stride, 1, groups=w_b // group_width), bn(w_b)
        self.with_se = se_ratio > 0
        if self.with_se:
            self.se = _SE(w_b, int(round(w_in * se_ratio)))
        self.conv3, self.bn3 = conv(w_b, w_out, 1), bn(w_out)
        self.shortcut = nn.Sequential()
        if stride != 1 or w_in != w_out:
            self.shortcut = _proj(w_in, w_out, stride)

    def forward(self, x):
        y = bn_act(self.bn1, self.conv1(x))
        y = bn_act(self.bn2, self.conv2(y))
        if self.with_se:
            y = self.se(y)
        return bn_act(self.bn3, self.conv3(y), residual=_shortcut(self.shortcut, x))


class RegNet(nn.Module):
    def __init__(self, cfg, num_classes=10):
        super().__init__()
        self.cfg, self.in_planes = cfg, 64
        self.conv1, self.bn1 = conv(3, 64, 3, 1, 1), bn(64)
        for i in range(4):
            blocks = []
            for j in range(cfg["depths"][i]):
                blocks.append(_RegBlock(self.in_planes, cfg["widths"][i], cfg["strides"][i] if j == 0 else 1,
                                        cfg["group_width"], cfg["bottleneck_ratio"], cfg["se_ratio"]))
                self.in_planes = cfg["widths"][i]
            setattr(self, f"layer{i + 1}", nn.Sequential(*blocks))
        self.linear = linear(cfg["widths"][-1], num_classes)
        defer_batch_counters(self)

    def forward(self, x):
        x = bn_act(self.bn1, self.conv1(x))
        x = self.layer4(self.layer3(self.layer2(self.layer1(x))))
        return self.linear(F.adaptive_avg_pool2d(x, (1, 1)).flatten(1))


def _reg(depths, widths, gw, se):
    return RegNet({"depths": depths, "widths": widths, "strides": [1, 1, 2, 2], "group_width": gw,
                   "bottleneck_ratio": 1, "se_ratio": se})


def RegNetX_200MF():
    return _reg([1, 1, 4, 7], [24, 56, 152, 368], 8, 0)


def RegNetX_400MF():
    return _reg([1, 2, 7, 12], [32, 64, 160, 384], 16, 0)


def RegNetY_400MF():
    return _reg([1, 2, 7, 12], [32, 64, 160, 384], 16, 0.25)


# ---------------------------------------------------------------------------------- PNASNet
class _SepConv(nn.Module):
    """depthwise k x k convolution that also changes the width (groups = in_planes), then BN."""

    def __init__(self, in_planes, out_planes, kernel_size, stride):
        super().__init__()
        self.conv1 = conv(in_planes, out_planes, kernel_size, stride, (kernel_size - 1) // 2, groups=in_planes)
        self.bn1 = bn(out_planes)

    def forward(self, x, residual=None, relu=False):
        return bn_act(self.bn1, self.conv1(x), residual=residual, relu=relu)


class _CellA(nn.Module):
    def __init__(self, in_planes, out_planes, stride=1):
        super().__init__()
        self.stride = stride
        self.sep_conv1 = _SepConv(in_planes, out_planes, 7, stride)
        if stride == 2:
            self.conv1, self.bn1 = conv(in_planes, out_planes, 1), bn(out_planes)

    def forward(self, x):
        y2 = F.max_pool2d(x, kernel_size=3, stride=self.stride, padding=1)
        if self.stride == 2:
            y2 = bn_act(self.bn1, self.conv1(y2), relu=False)
        return self.sep_conv1(x, residual=y2, relu=True)


class _CellB(nn.Module):
    def __init__(self, in_planes, out_planes, stride=1):
        super().__init__()
        self.stride = stride
        self.sep_conv1 = _SepConv(in_planes, out_planes, 7, stride)
        self.sep_conv2 = _SepConv(in_planes, out_planes, 3, stride)
        self.sep_conv3 = _SepConv(in_planes, out_planes, 5, stride)
        if stride == 2:
            self.conv1, self.bn1 = conv(in_planes, out_planes, 1), bn(out_planes)
        self.conv2, self.bn2 = conv(2 * out_planes, out_planes, 1), bn(out_planes)

    def forward(self, x):
        b1 = self.sep_conv1(x, residual=self.sep_conv2(x), relu=True)
        y3 = F.max_pool2d(x, kernel_size=3, stride=self.stride, padding=1)
        if self.stride == 2:
            y3 = bn_act(self.bn1, self.conv1(y3), relu=False)
        b2 = self.sep_conv3(x, residual=y3, relu=True)
        return bn_act(self.bn2, self.conv2(torch.cat([b1, b2], 1)))


class PNASNet(nn.Module):
    def __init__(self, cell_type, num_cells, num_planes):
        super().__init__()
        self.in_planes, self.cell_type = num_planes, cell_type
        self.conv1, self.bn1 = conv(3, num_planes, 3, 1, 1), bn(num_planes)
        self.layer1 = self._stage(num_planes, num_cells)
        self.layer2 = self._down(num_planes * 2)
        self.layer3 = self._stage(num_planes * 2, num_cells)
        self.layer4 = self._down(num_planes * 4)
        self.layer5 = self._stage(num_planes * 4, num_cells)
        self.linear = linear(num_planes * 4, 10)
        defer_batch_counters(self)

    def _stage(self, planes, n):
        cells = []
        for _ in range(n):
            cells.append(self.cell_type(self.in_planes, planes, stride=1))
            self.in_planes = planes
        return nn.Sequential(*cells)

    def _down(self, planes):
        cell = self.cell_type(self.in_planes, planes, stride=2)
        self.in_planes = planes
        return cell

    def forward(self, x):
        x = bn_act(self.bn1, self.conv1(x))
        x = self.layer5(self.layer4(self.layer3(self.layer2(self.layer1(x)))))
        return self.linear(head_pool(x, 8))


def PNASNetA():
    return PNASNet(_CellA, num_cells=6, num_planes=44)


def PNASNetB():
    return PNASNet(_CellB, num_cells=6, num_planes=32)
