"""gradient_compression_b200 -- compressed data-parallel SGD for B200 (sm_100a).

Public surface (names follow vineeths96/Gradient-Compression): ``reducers`` (25 Reducer classes +
``make_reducer``), ``compressors``, ``models`` (CIFAR zoo), ``train`` (``CIFAR`` task, ``train()``
loop, config), ``utils`` (Timer, Logger, AverageMeter, set_seed, plots), ``ops`` (native kernels and
their CPU oracles) and ``parallel`` (flat arenas, symmetric memory, fused collectives).
"""
__version__ = "0.1.0"

from . import compressors, ops, reducers, utils  # noqa: F401
from .reducers import make_reducer  # noqa: F401
