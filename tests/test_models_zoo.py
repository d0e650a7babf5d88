"""Model zoo: every factory builds, maps 3x32x32 to 10 logits, and (where the reference's module runs)
shares parameter names, shapes and -- with the same weights -- outputs with the reference's model."""
import importlib
import os
import sys

import pytest
import torch

from gradient_compression_b200 import models

from .conftest import reference_dir

REF = reference_dir() or ""
LIGHT = ["LeNet", "ResNet18", "PreActResNet18", "densenet_cifar", "MobileNet", "MobileNetV2", "SENet18", "PNASNetA",
         "PNASNetB", "EfficientNetB0", "RegNetX_200MF", "RegNetY_400MF", "ShuffleNetG2", "ShuffleNetG3",
         "ShuffleNetV2_x0_5", "ResNeXt29_32x4d", "GoogLeNet", "DPN26", "VGG11"]


def test_every_name_of_the_reference_zoo_is_a_zero_arg_factory():
    expected = {"VGG16", "ResNet18", "ResNet34", "ResNet50", "ResNet101", "ResNet152", "PreActResNet18",
                "PreActResNet34", "PreActResNet50", "PreActResNet101", "PreActResNet152", "DenseNet121", "DenseNet169",
                "DenseNet201", "DenseNet161", "densenet_cifar", "DPN26", "DPN92", "GoogLeNet", "LeNet", "MobileNet",
                "MobileNetV2", "ResNeXt29_2x64d", "ResNeXt29_4x64d", "ResNeXt29_8x64d", "ResNeXt29_32x4d", "SENet18",
                "PNASNetA", "PNASNetB", "EfficientNetB0", "RegNetX_200MF", "RegNetX_400MF", "RegNetY_400MF",
                "ShuffleNetG2", "ShuffleNetG3"}
    assert expected <= set(models.available())
    assert all(callable(getattr(models, n)) for n in models.available())


@pytest.mark.parametrize("name", LIGHT)
def test_forward_backward_shapes(name):
    torch.manual_seed(0)
    net = getattr(models, name)()
    y = net(torch.randn(2, 3, 32, 32))
    assert y.shape == (2, 10) and torch.isfinite(y).all()
    y.sum().backward()
    unused = {"layers.0.conv1.weight", "layers.0.bn1.weight", "layers.0.bn1.bias"} if name == "EfficientNetB0" else set()
    # (EfficientNet's first block has expansion 1 and, as in the reference, never touches its conv1 / bn1)
    assert all(p.grad is not None for n_, p in net.named_parameters() if n_ not in unused)


@pytest.mark.skipif(not os.path.exists(os.path.join(REF, "models", "resnet.py")), reason="reference sources not mounted")
@pytest.mark.parametrize("name", ["ResNet18", "PreActResNet18", "densenet_cifar", "MobileNetV2", "SENet18", "PNASNetB",
                                  "RegNetY_400MF", "ShuffleNetV2_x0_5", "ResNeXt29_32x4d", "DPN26", "VGG11", "GoogLeNet"])
def test_same_weights_same_outputs_as_reference(name):
    sys.path.insert(0, REF)
    try:
        for mod in [m for m in sys.modules if m == "models" or m.startswith("models.")]:
            del sys.modules[mod]
        ref_models = importlib.import_module("models")
        if name.startswith("ShuffleNetV2"):
            ref = ref_models.ShuffleNetV2(0.5)
        elif name == "VGG11":
            ref = ref_models.VGG("VGG11")
        else:
            ref = getattr(ref_models, name)()
    finally:
        sys.path.remove(REF)
        for mod in [m for m in sys.modules if m == "models" or m.startswith("models.")]:
            del sys.modules[mod]
    ours = getattr(models, name)()
    sd = ref.state_dict()
    assert list(sd) == list(ours.state_dict())
    ours.load_state_dict(sd)
    x = torch.randn(4, 3, 32, 32)
    for mode in ("train", "eval"):
        getattr(ref, mode)()
        getattr(ours, mode)()
        ref.load_state_dict(sd)
        ours.load_state_dict(sd)
        assert torch.allclose(ours(x), ref(x), atol=1e-4, rtol=1e-4), (name, mode)
