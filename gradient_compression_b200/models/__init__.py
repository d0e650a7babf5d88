"""CIFAR-sized model zoo (3x32x32 -> 10 logits); every public name is a zero-argument factory so
``getattr(models, architecture)()`` works for all of them (reference: models/__init__.py,
model_dispatcher.py:58-64)."""
from .densenet import DenseNet, DenseNet121, DenseNet161, DenseNet169, DenseNet201, densenet_cifar
from .dpn import DPN, DPN26, DPN92
from .preact_resnet import (PreActResNet, PreActResNet18, PreActResNet34, PreActResNet50, PreActResNet101,
                            PreActResNet152)
from .resnet import ResNet, ResNet18, ResNet34, ResNet50, ResNet101, ResNet152
from .resnext_senet import (PNASNet, PNASNetA, PNASNetB, RegNet, RegNetX_200MF, RegNetX_400MF, RegNetY_400MF, ResNeXt,
                            ResNeXt29_2x64d, ResNeXt29_4x64d, ResNeXt29_8x64d, ResNeXt29_32x4d, SENet, SENet18)
from .shuffle_efficient import (EfficientNet, EfficientNetB0, ShuffleNet, ShuffleNetG2, ShuffleNetG3, ShuffleNetV2,
                                ShuffleNetV2_x0_5, ShuffleNetV2_x1, ShuffleNetV2_x1_5, ShuffleNetV2_x2)
from .small_nets import GoogLeNet, LeNet, MobileNet, MobileNetV2
from .vgg import VGG, VGG11, VGG13, VGG16, VGG19

FACTORIES = [
    "VGG11", "VGG13", "VGG16", "VGG19", "ResNet18", "ResNet34", "ResNet50", "ResNet101", "ResNet152",
    "PreActResNet18", "PreActResNet34", "PreActResNet50", "PreActResNet101", "PreActResNet152",
    "DenseNet121", "DenseNet169", "DenseNet201", "DenseNet161", "densenet_cifar", "DPN26", "DPN92", "GoogLeNet", "LeNet",
    "MobileNet", "MobileNetV2", "ResNeXt29_2x64d", "ResNeXt29_4x64d", "ResNeXt29_8x64d", "ResNeXt29_32x4d", "SENet18",
    "PNASNetA", "PNASNetB", "EfficientNetB0", "RegNetX_200MF", "RegNetX_400MF", "RegNetY_400MF", "ShuffleNetG2",
    "ShuffleNetG3", "ShuffleNetV2_x0_5", "ShuffleNetV2_x1", "ShuffleNetV2_x1_5", "ShuffleNetV2_x2",
]


def available():
    return list(FACTORIES)
