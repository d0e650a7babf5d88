"""Layer factories of the model zoo.

Models build their convolutions, batch norms and linear layers through ``conv`` / ``bn`` / ``linear`` so that every
file of the zoo spells the same defaults (no convolution bias unless asked for); the modules are plain ``torch.nn``
ones -- same parameters, buffers and ``state_dict`` keys as the reference's -- and the hand-written kernels are applied
to them functionally (``ops.conv_bn_act``, ``ops.bn_act``, ``ops.head``).
"""
from __future__ import annotations

import torch.nn as nn
import torch.nn.functional as F


def conv(cin, cout, k, stride=1, padding=0, groups=1, bias=False):
    return nn.Conv2d(cin, cout, kernel_size=k, stride=stride, padding=padding, groups=groups, bias=bias)


def bn(c):
    return nn.BatchNorm2d(c)


def linear(cin, cout):
    return nn.Linear(cin, cout)


def head_pool(x, k):
    """``F.avg_pool2d(x, k).flatten(1)`` of the network head.  When the window covers the whole feature map (every
    CIFAR model here) this is a mean over H and W: one reduction forward, and backward a broadcast that the next fused
    kernel reads directly."""
    if x.dim() == 4 and x.shape[2] == k and x.shape[3] == k:
        return x.mean((2, 3))
    return F.avg_pool2d(x, k).flatten(1)
