"""Dual-path networks for CIFAR (reference: models/dpn.py:7-104): a grouped-3x3 bottleneck whose output is
split into a residual part (added) and a dense part (concatenated)."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops.bn import bn_act, defer_batch_counters
from .layers import bn, conv, head_pool, linear


class Bottleneck(nn.Module):
    def __init__(self, last_planes, in_planes, out_planes, dense_depth, stride, first_layer):
        super().__init__()
        self.out_planes, self.dense_depth = out_planes, dense_depth
        self.conv1, self.bn1 = conv(last_planes, in_planes, 1), bn(in_planes)
        self.conv2, self.bn2 = conv(in_planes, in_planes, 3, stride, 1, groups=32), bn(in_planes)
        self.conv3, self.bn3 = conv(in_planes, out_planes + dense_depth, 1), bn(out_planes + dense_depth)
        self.shortcut = nn.Sequential()
        if first_layer:
            self.shortcut = nn.Sequential(conv(last_planes, out_planes + dense_depth, 1, stride), bn(out_planes + dense_depth))

    def forward(self, x):
        y = bn_act(self.bn1, self.conv1(x))
        y = bn_act(self.bn2, self.conv2(y))
        y = self.bn3(self.conv3(y))
        x = self.shortcut(x)
        d = self.out_planes
        return F.relu(torch.cat([x[:, :d] + y[:, :d], x[:, d:], y[:, d:]], 1))


class DPN(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.conv1, self.bn1 = conv(3, 64, 3, 1, 1), bn(64)
        self.last_planes = 64
        for i in range(4):
            layers = []
            stride = 1 if i == 0 else 2
            for j, s in enumerate([stride] + [1] * (cfg["num_blocks"][i] - 1)):
                layers.append(Bottleneck(self.last_planes, cfg["in_planes"][i], cfg["out_planes"][i],
                                         cfg["dense_depth"][i], s, j == 0))
                self.last_planes = cfg["out_planes"][i] + (j + 2) * cfg["dense_depth"][i]
            setattr(self, f"layer{i + 1}", nn.Sequential(*layers))
        self.linear = linear(cfg["out_planes"][3] + (cfg["num_blocks"][3] + 1) * cfg["dense_depth"][3], 10)
        defer_batch_counters(self)

    def forward(self, x):
        x = bn_act(self.bn1, self.conv1(x))
        x = self.layer4(self.layer3(self.layer2(self.layer1(x))))
        return self.linear(head_pool(x, 4))


def _cfg(num_blocks):
    return {"in_planes": (96, 192, 384, 768), "out_planes": (256, 512, 1024, 2048), "num_blocks": num_blocks,
            "dense_depth": (16, 32, 24, 128)}


def DPN26():
    return DPN(_cfg((2, 2, 2, 2)))


def DPN92():
    return DPN(_cfg((3, 4, 20, 3)))
