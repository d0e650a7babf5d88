from .logger import Logger
from .metrics import AverageMeter
from .seed import set_seed
from .timer import NullTimer, Timer

__all__ = ["Logger", "AverageMeter", "set_seed", "Timer", "NullTimer"]
