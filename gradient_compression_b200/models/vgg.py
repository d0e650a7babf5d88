"""CIFAR VGG family: 3x3 convolutions with bias + BN + ReLU, 2x2 max-pools, a 512 -> 10 linear head
(reference: models/vgg.py:6-110).  ``features.N`` / ``classifier`` key names match the reference
(including the parameter-free ``AvgPool2d(1, 1)`` that closes ``features``)."""
from __future__ import annotations

import torch.nn as nn

from ..ops.bn import defer_batch_counters, flush_batch_counters
from ..ops.conv import conv_bn_act
from ..ops.head import head_loss
from .layers import bn, conv, linear

CFG = {
    "VGG11": [64, "M", 128, "M", 256, 256, "M", 512, 512, "M", 512, 512, "M"],
    "VGG13": [64, 64, "M", 128, 128, "M", 256, 256, "M", 512, 512, "M", 512, 512, "M"],
    "VGG16": [64, 64, "M", 128, 128, "M", 256, 256, 256, "M", 512, 512, 512, "M", 512, 512, 512, "M"],
    "VGG19": [64, 64, "M", 128, 128, "M", 256, 256, 256, 256, "M", 512, 512, 512, 512, "M", 512, 512, 512, 512, "M"],
}


class VGG(nn.Module):
    def __init__(self, vgg_name="VGG16"):
        super().__init__()
        layers, cin = [], 3
        for item in CFG[vgg_name]:
            if item == "M":
                layers.append(nn.MaxPool2d(kernel_size=2, stride=2))
            else:
                layers += [conv(cin, item, 3, padding=1, bias=True), bn(item), nn.ReLU(inplace=True)]
                cin = item
        layers.append(nn.AvgPool2d(kernel_size=1, stride=1))
        self.features = nn.Sequential(*layers)
        self.classifier = linear(512, 10)
        defer_batch_counters(self)

    def forward(self, x):
        return self.classifier(self._features(x).flatten(1))

    def forward_loss(self, x, labels):
        """``(loss, logits, [cross-entropy, top-1, top-5])`` with the linear layer, the loss and the batch metrics in one kernel
        (the feature map is 1 x 1 after the fifth max-pool: models/vgg.py:88,109 of the reference)."""
        f = self._features(x)
        flush_batch_counters()          # (the forward hook that batches the BN step counters only fires for __call__)
        if f.shape[2] * f.shape[3] != 1:
            f = f.flatten(1)[:, :, None, None]
        return head_loss(f, self.classifier, labels)

    def _features(self, x):
        mods = list(self.features)
        i = 0
        while i < len(mods):
            m = mods[i]
            if (isinstance(m, nn.Conv2d) and i + 2 < len(mods) and isinstance(mods[i + 1], nn.BatchNorm2d)
                    and isinstance(mods[i + 2], nn.ReLU)):
                # convolution with BN statistics in its epilogue, BN + ReLU in one pass; a 2x2 max-pool that follows is
                # folded into that pass (the full-resolution activation is never written)
                nxt = mods[i + 3] if i + 3 < len(mods) else None
                pool = (isinstance(nxt, nn.MaxPool2d) and nxt.kernel_size in (2, (2, 2)) and nxt.stride in (2, (2, 2))
                        and nxt.padding in (0, (0, 0)) and nxt.dilation in (1, (1, 1)) and not nxt.ceil_mode
                        and x.shape[2] % 2 == 0 and x.shape[3] % 2 == 0)
                x = conv_bn_act(m, mods[i + 1], x, pool=pool)
                i += 4 if pool else 3
            else:
                x = m(x)
                i += 1
        return x


def VGG11():
    return VGG("VGG11")


def VGG13():
    return VGG("VGG13")


def VGG16():
    return VGG("VGG16")


def VGG19():
    return VGG("VGG19")
