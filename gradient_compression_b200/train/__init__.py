from .config import TrainConfig
from .task import CIFAR
from .trainer import initiate_distributed, train

__all__ = ["TrainConfig", "CIFAR", "initiate_distributed", "train"]
