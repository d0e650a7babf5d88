"""Layer factories of the model zoo.

Models never instantiate ``torch.nn.Conv2d`` / ``BatchNorm2d`` directly: they call ``conv`` / ``bn``
here, so the hand-written sm_100a implementations (``nn_b200``) can be swapped in per layer while the
parameter names -- and therefore ``state_dict`` keys -- stay those of ``torch.nn`` modules.
"""
from __future__ import annotations

import torch.nn as nn
import torch.nn.functional as F

_IMPL = {"conv": None, "bn": None, "linear": None}


def set_layer_impl(conv=None, bn=None, linear=None):
    """Install alternative layer classes (signature-compatible with their torch.nn counterparts)."""
    _IMPL.update(conv=conv, bn=bn, linear=linear)


def conv(cin, cout, k, stride=1, padding=0, groups=1, bias=False):
    cls = _IMPL["conv"] or nn.Conv2d
    return cls(cin, cout, kernel_size=k, stride=stride, padding=padding, groups=groups, bias=bias)


def bn(c):
    cls = _IMPL["bn"] or nn.BatchNorm2d
    return cls(c)


def linear(cin, cout):
    cls = _IMPL["linear"] or nn.Linear
    return cls(cin, cout)


def head_pool(x, k):
    """``F.avg_pool2d(x, k).flatten(1)`` of the network head.  When the window covers the whole feature map (every
    CIFAR model here) this is a mean over H and W: one reduction forward, and backward a broadcast that the next fused
    kernel reads directly -- torch's NHWC average-pool backward kernel took 61 us for 16 MB on a B200."""
    if x.dim() == 4 and x.shape[2] == k and x.shape[3] == k:
        return x.mean((2, 3))
    return F.avg_pool2d(x, k).flatten(1)
