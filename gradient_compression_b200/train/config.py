"""Training configuration (reference: the module-level ``config`` dict, trainer.py:44-62).

The same keys, as a dataclass with argparse / YAML overrides.  ``as_dict()`` gives the mapping the
Logger dumps into ``success.txt`` (the reference's plots parse that file)."""
from __future__ import annotations

import argparse
import dataclasses
from dataclasses import dataclass, field
from typing import List, Optional


@dataclass
class TrainConfig:
    runs: int = 5
    distributed_backend: str = "nccl"
    num_epochs: int = 150
    batch_size: int = 128
    architecture: str = "ResNet50"
    local_steps: int = 1
    K: int = 10000
    compression: float = 1 / 1000
    quantization_level: int = 8
    higher_quantization_level: int = 12
    quantization_levels: List[int] = field(default_factory=lambda: [6, 10, 16])
    rank: int = 1
    reducer: str = "NoneAllReducer"
    seed: int = 42
    log_verbosity: int = 2
    lr: float = 0.1
    # --- additions of this library -------------------------------------------------------
    momentum: float = 0.9
    weight_decay: float = 5e-4
    nesterov: bool = True
    backend: str = "auto"             # reducer backend: auto | fused | dist
    reference_compat: bool = False
    broadcast_parameters: bool = True  # the reference never synchronises replicas
    data: str = "cifar10"             # cifar10 | synthetic | cifar10_device | synthetic_device
    data_path: str = "./data"
    synthetic_train_size: int = 50000
    synthetic_test_size: int = 10000
    max_steps_per_epoch: Optional[int] = None
    timer_mode: str = "event"         # event | sync
    log_root: str = "./logs"
    resume: Optional[str] = None
    save_training_state: bool = False
    device: Optional[str] = None
    heartbeat_timeout_s: float = 0.0  # > 0 enables the step watchdog
    graph: bool = True                # CUDA devices: run the whole step as one callable replayed from a CUDA graph
    norm_scope: str = "global"        # global: one reduce after backward (the reference) | bucket: per-bucket reduces
                                      # overlapped with backward, each bucket normalised by its own max-norm
    bucket_mb: float = 25.0           # bucket size for norm_scope = bucket
    reduce_max_blocks: int = 32       # grid cap of a fused reduce that runs beside backward kernels
    on_collective_timeout: str = "raise"   # raise | dist: after a device-side timeout continue on torch.distributed

    def as_dict(self):
        return dataclasses.asdict(self)

    def __getitem__(self, k):
        return getattr(self, k)

    @classmethod
    def from_mapping(cls, mapping):
        names = {f.name for f in dataclasses.fields(cls)}
        return cls(**{k: v for k, v in mapping.items() if k in names})

    @classmethod
    def from_yaml(cls, path):
        import yaml

        with open(path) as f:
            return cls.from_mapping(yaml.safe_load(f) or {})

    @classmethod
    def parser(cls):
        p = argparse.ArgumentParser(description="compressed data-parallel CIFAR training")
        p.add_argument("--config", type=str, default=None, help="YAML file with TrainConfig keys")
        p.add_argument("--local_rank", "--local-rank", type=int, default=None)
        p.add_argument("--local_world_size", "--local-world-size", type=int, default=1)
        for f in dataclasses.fields(cls):
            if f.type in ("int", "float", "str", "Optional[str]", "Optional[int]"):
                typ = {"int": int, "float": float, "str": str, "Optional[str]": str, "Optional[int]": int}[f.type]
                p.add_argument(f"--{f.name}", type=typ, default=None)
            elif f.type == "bool":
                p.add_argument(f"--{f.name}", type=lambda s: s.lower() in ("1", "true", "yes"), default=None)
            elif f.type == "List[int]":
                p.add_argument(f"--{f.name}", type=int, nargs="+", default=None)
        return p

    @classmethod
    def from_args(cls, argv=None):
        args = cls.parser().parse_args(argv)
        cfg = cls.from_yaml(args.config) if args.config else cls()
        for f in dataclasses.fields(cls):
            v = getattr(args, f.name, None)
            if v is not None:
                setattr(cfg, f.name, v)
        return cfg, args
