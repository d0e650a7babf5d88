"""Layer factories of the model zoo.

Models never instantiate ``torch.nn.Conv2d`` / ``BatchNorm2d`` directly: they call ``conv`` / ``bn``
here, so the hand-written sm_100a implementations (``nn_b200``) can be swapped in per layer while the
parameter names -- and therefore ``state_dict`` keys -- stay those of ``torch.nn`` modules.
"""
from __future__ import annotations

import torch.nn as nn

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
