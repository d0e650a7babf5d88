"""ShuffleNet (G2/G3), ShuffleNetV2 and EfficientNet-B0 for CIFAR (reference: models/shufflenet.py:10-108,
shufflenetv2.py:10-150, efficientnet.py:12-166).  Integer channel arithmetic throughout (the reference's
ShuffleNet divides with ``/`` and fails on Python 3), and zero-argument ShuffleNetV2 factories."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops.bn import bn_act
from .layers import bn, conv, head_pool, linear


def channel_shuffle(x, groups):
    """[N, C, H, W] -> [N, g, C/g, H, W] -> transpose the two group axes -> [N, C, H, W]."""
    n, c, h, w = x.shape
    return x.view(n, groups, c // groups, h, w).permute(0, 2, 1, 3, 4).reshape(n, c, h, w)


class ShuffleBlock(nn.Module):
    def __init__(self, groups=2):
        super().__init__()
        self.groups = groups

    def forward(self, x):
        return channel_shuffle(x, self.groups)


class _ShuffleBottleneck(nn.Module):
    def __init__(self, in_planes, out_planes, stride, groups):
        super().__init__()
        self.stride = stride
        mid = out_planes // 4
        g = 1 if in_planes == 24 else groups
        self.conv1, self.bn1 = conv(in_planes, mid, 1, groups=g), bn(mid)
        self.shuffle1 = ShuffleBlock(groups=g)
        self.conv2, self.bn2 = conv(mid, mid, 3, stride, 1, groups=mid), bn(mid)
        self.conv3, self.bn3 = conv(mid, out_planes, 1, groups=groups), bn(out_planes)
        self.shortcut = nn.Sequential()
        if stride == 2:
            self.shortcut = nn.Sequential(nn.AvgPool2d(3, stride=2, padding=1))

    def forward(self, x):
        y = self.shuffle1(bn_act(self.bn1, self.conv1(x)))
        y = bn_act(self.bn2, self.conv2(y))
        res = self.shortcut(x)
        if self.stride == 2:
            return F.relu(torch.cat([bn_act(self.bn3, self.conv3(y), relu=False), res], 1))
        return bn_act(self.bn3, self.conv3(y), residual=res)


class ShuffleNet(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.conv1, self.bn1 = conv(3, 24, 1), bn(24)
        self.in_planes = 24
        for i, (planes, depth) in enumerate(zip(cfg["out_planes"], cfg["num_blocks"]), start=1):
            blocks = []
            for j in range(depth):
                cat_planes = self.in_planes if j == 0 else 0
                blocks.append(_ShuffleBottleneck(self.in_planes, planes - cat_planes, 2 if j == 0 else 1, cfg["groups"]))
                self.in_planes = planes
            setattr(self, f"layer{i}", nn.Sequential(*blocks))
        self.linear = linear(cfg["out_planes"][2], 10)

    def forward(self, x):
        x = bn_act(self.bn1, self.conv1(x))
        x = self.layer3(self.layer2(self.layer1(x)))
        return self.linear(head_pool(x, 4))


def ShuffleNetG2():
    return ShuffleNet({"out_planes": [200, 400, 800], "num_blocks": [4, 8, 4], "groups": 2})


def ShuffleNetG3():
    return ShuffleNet({"out_planes": [240, 480, 960], "num_blocks": [4, 8, 4], "groups": 3})


# ---------------------------------------------------------------------------------- ShuffleNetV2
class SplitBlock(nn.Module):
    def __init__(self, ratio):
        super().__init__()
        self.ratio = ratio

    def forward(self, x):
        c = int(x.size(1) * self.ratio)
        return x[:, :c], x[:, c:]


class _V2Basic(nn.Module):
    def __init__(self, in_channels, split_ratio=0.5):
        super().__init__()
        self.split = SplitBlock(split_ratio)
        c = int(in_channels * split_ratio)
        self.conv1, self.bn1 = conv(c, c, 1), bn(c)
        self.conv2, self.bn2 = conv(c, c, 3, 1, 1, groups=c), bn(c)
        self.conv3, self.bn3 = conv(c, c, 1), bn(c)
        self.shuffle = ShuffleBlock()

    def forward(self, x):
        x1, x2 = self.split(x)
        y = bn_act(self.bn1, self.conv1(x2.contiguous(memory_format=torch.channels_last) if x2.is_cuda else x2))
        y = bn_act(self.bn2, self.conv2(y), relu=False)
        y = bn_act(self.bn3, self.conv3(y))
        return self.shuffle(torch.cat([x1, y], 1))


class _V2Down(nn.Module):
    def __init__(self, in_channels, out_channels):
        super().__init__()
        mid = out_channels // 2
        self.conv1, self.bn1 = conv(in_channels, in_channels, 3, 2, 1, groups=in_channels), bn(in_channels)
        self.conv2, self.bn2 = conv(in_channels, mid, 1), bn(mid)
        self.conv3, self.bn3 = conv(in_channels, mid, 1), bn(mid)
        self.conv4, self.bn4 = conv(mid, mid, 3, 2, 1, groups=mid), bn(mid)
        self.conv5, self.bn5 = conv(mid, mid, 1), bn(mid)
        self.shuffle = ShuffleBlock()

    def forward(self, x):
        left = bn_act(self.bn2, self.conv2(bn_act(self.bn1, self.conv1(x), relu=False)))
        right = bn_act(self.bn3, self.conv3(x))
        right = bn_act(self.bn5, self.conv5(bn_act(self.bn4, self.conv4(right), relu=False)))
        return self.shuffle(torch.cat([left, right], 1))


V2_CONFIGS = {
    0.5: {"out_channels": (48, 96, 192, 1024), "num_blocks": (3, 7, 3)},
    1: {"out_channels": (116, 232, 464, 1024), "num_blocks": (3, 7, 3)},
    1.5: {"out_channels": (176, 352, 704, 1024), "num_blocks": (3, 7, 3)},
    2: {"out_channels": (224, 488, 976, 2048), "num_blocks": (3, 7, 3)},
}


class ShuffleNetV2(nn.Module):
    def __init__(self, net_size=0.5):
        super().__init__()
        oc, nb = V2_CONFIGS[net_size]["out_channels"], V2_CONFIGS[net_size]["num_blocks"]
        self.conv1, self.bn1 = conv(3, 24, 3, 1, 1), bn(24)
        self.in_channels = 24
        for i in range(3):
            layers = [_V2Down(self.in_channels, oc[i])]
            for _ in range(nb[i]):
                layers.append(_V2Basic(oc[i]))
                self.in_channels = oc[i]
            setattr(self, f"layer{i + 1}", nn.Sequential(*layers))
        self.conv2, self.bn2 = conv(oc[2], oc[3], 1), bn(oc[3])
        self.linear = linear(oc[3], 10)

    def forward(self, x):
        x = bn_act(self.bn1, self.conv1(x))
        x = self.layer3(self.layer2(self.layer1(x)))
        x = bn_act(self.bn2, self.conv2(x))
        return self.linear(head_pool(x, 4))


def ShuffleNetV2_x0_5():
    return ShuffleNetV2(0.5)


def ShuffleNetV2_x1():
    return ShuffleNetV2(1)


def ShuffleNetV2_x1_5():
    return ShuffleNetV2(1.5)


def ShuffleNetV2_x2():
    return ShuffleNetV2(2)


# ---------------------------------------------------------------------------------- EfficientNet
def swish(x):
    return x * torch.sigmoid(x)


def drop_connect(x, drop_ratio):
    """Zero whole samples with probability ``drop_ratio`` and rescale the survivors."""
    keep = 1.0 - drop_ratio
    mask = torch.empty([x.shape[0], 1, 1, 1], dtype=x.dtype, device=x.device).bernoulli_(keep)
    return x / keep * mask


class _SESwish(nn.Module):
    def __init__(self, in_channels, se_channels):
        super().__init__()
        self.se1, self.se2 = conv(in_channels, se_channels, 1, bias=True), conv(se_channels, in_channels, 1, bias=True)

    def forward(self, x):
        gate = torch.sigmoid(self.se2(swish(self.se1(F.adaptive_avg_pool2d(x, (1, 1))))))
        return x * gate


class _MBConv(nn.Module):
    def __init__(self, in_channels, out_channels, kernel_size, stride, expand_ratio=1, se_ratio=0.0, drop_rate=0.0):
        super().__init__()
        self.stride, self.drop_rate, self.expand_ratio = stride, drop_rate, expand_ratio
        ch = expand_ratio * in_channels
        self.conv1, self.bn1 = conv(in_channels, ch, 1), bn(ch)
        self.conv2 = conv(ch, ch, kernel_size, stride, 1 if kernel_size == 3 else 2, groups=ch)
        self.bn2 = bn(ch)
        self.se = _SESwish(ch, int(in_channels * se_ratio))
        self.conv3, self.bn3 = conv(ch, out_channels, 1), bn(out_channels)
        self.has_skip = stride == 1 and in_channels == out_channels

    def forward(self, x):
        y = x if self.expand_ratio == 1 else swish(bn_act(self.bn1, self.conv1(x), relu=False))
        y = swish(bn_act(self.bn2, self.conv2(y), relu=False))
        y = bn_act(self.bn3, self.conv3(self.se(y)), relu=False)
        if self.has_skip:
            if self.training and self.drop_rate > 0:
                y = drop_connect(y, self.drop_rate)
            y = y + x
        return y


class EfficientNet(nn.Module):
    def __init__(self, cfg, num_classes=10):
        super().__init__()
        self.cfg = cfg
        self.conv1, self.bn1 = conv(3, 32, 3, 1, 1), bn(32)
        layers, cin, b = [], 32, 0
        total = sum(cfg["num_blocks"])
        for expansion, cout, n, k, stride in zip(cfg["expansion"], cfg["out_channels"], cfg["num_blocks"],
                                                  cfg["kernel_size"], cfg["stride"]):
            for s in [stride] + [1] * (n - 1):
                layers.append(_MBConv(cin, cout, k, s, expansion, se_ratio=0.25,
                                      drop_rate=cfg["drop_connect_rate"] * b / total))
                cin = cout
        self.layers = nn.Sequential(*layers)
        self.linear = linear(cfg["out_channels"][-1], num_classes)

    def forward(self, x):
        x = swish(bn_act(self.bn1, self.conv1(x), relu=False))
        x = F.adaptive_avg_pool2d(self.layers(x), 1).flatten(1)
        if self.training and self.cfg["dropout_rate"] > 0:
            x = F.dropout(x, p=self.cfg["dropout_rate"])
        return self.linear(x)


def EfficientNetB0():
    return EfficientNet({"num_blocks": [1, 2, 2, 3, 3, 4, 1], "expansion": [1, 6, 6, 6, 6, 6, 6],
                         "out_channels": [16, 24, 40, 80, 112, 192, 320], "kernel_size": [3, 3, 5, 3, 5, 5, 3],
                         "stride": [1, 2, 2, 2, 1, 2, 1], "dropout_rate": 0.2, "drop_connect_rate": 0.2})
