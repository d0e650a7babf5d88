"""CIFAR-sized model zoo (3x32x32 -> 10 logits); every public name is a zero-argument factory so
``getattr(models, architecture)()`` works for all of them (reference: models/__init__.py,
model_dispatcher.py:58-64)."""
from .layers import set_layer_impl
from .resnet import ResNet, ResNet18, ResNet34, ResNet50, ResNet101, ResNet152
from .vgg import VGG, VGG11, VGG13, VGG16, VGG19


def available():
    import inspect
    import sys

    mod = sys.modules[__name__]
    return sorted(n for n, f in vars(mod).items()
                  if inspect.isfunction(f) and n[0].isupper() or n == "densenet_cifar")
