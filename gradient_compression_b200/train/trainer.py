"""Training driver (reference: trainer.py:65-244).

``python -m gradient_compression_b200.train.trainer --architecture VGG16 --reducer QSGDMaxNormReducer
--quantization_level 4`` under ``torchrun`` (or alone: one worker).  The loop structure, timer labels,
log artefacts and the per-epoch evaluation / best-checkpoint rule are the reference's; the hot loop
itself has no host synchronisation: no ``.item()``, no per-tensor copies, one kernel for the
optimiser, event-based timing.
"""
from __future__ import annotations

import datetime
import os

import torch
import torch.distributed as dist

from ..parallel.arena import CosineSchedule, FlatSGD
from ..reducers import make_reducer
from ..utils import AverageMeter, Logger, Timer, set_seed
from . import checkpoint as ckpt
from .config import TrainConfig
from .task import CIFAR


def initiate_distributed(backend="nccl", timeout_s=1800):
    """``init_process_group(env://)`` when launched under a distributed launcher (trainer.py:65-75).

    Falls back to gloo when CUDA is absent; sets a finite collective timeout so a dead peer surfaces
    as an error instead of a hang."""
    if "RANK" not in os.environ or "WORLD_SIZE" not in os.environ:
        return False
    if dist.is_initialized():
        return True
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    if backend == "nccl" and not torch.cuda.is_available():
        backend = "gloo"
    env = {k: os.environ.get(k) for k in ("MASTER_ADDR", "MASTER_PORT", "RANK", "WORLD_SIZE")}
    print(f"[{os.getpid()}] Initializing Process Group with: {env}")
    kwargs = {}
    if backend == "nccl":
        local_rank = int(os.environ.get("LOCAL_RANK", 0))
        torch.cuda.set_device(local_rank)
        kwargs["device_id"] = torch.device("cuda", local_rank)
    dist.init_process_group(backend=backend, init_method="env://", timeout=datetime.timedelta(seconds=timeout_s),
                            **kwargs)
    print(f"[{os.getpid()}] Initialized Process Group with: RANK = {dist.get_rank()}, "
          f"WORLD_SIZE = {dist.get_world_size()}, backend={dist.get_backend()}")
    return True


def _global_rank():
    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


def _device_for(config, local_rank):
    if config.device:
        return torch.device(config.device)
    if torch.cuda.is_available():
        return torch.device(f"cuda:{local_rank}")
    return torch.device("cpu")


def train(local_rank=0, config=None, logger=None):
    config = config or TrainConfig()
    if isinstance(config, dict):
        config = TrainConfig.from_mapping(config)
    cfg_dict = config.as_dict()
    logger = logger or Logger(cfg_dict, local_rank, root=config.log_root)
    best_accuracy = {"top1": [0] * config.runs, "top5": [0] * config.runs}
    device = _device_for(config, local_rank)
    if device.type == "cuda":
        torch.cuda.set_device(device)
    watchdog = None
    if config.heartbeat_timeout_s > 0:
        from ..parallel.watchdog import StepWatchdog
        watchdog = StepWatchdog.from_env(timeout_s=config.heartbeat_timeout_s)

    resume_state = torch.load(config.resume, map_location="cpu", weights_only=False) if config.resume else None
    timer, bits_communicated = None, 0

    for run in range(config.runs):
        if resume_state is not None and run < resume_state["run"]:
            continue
        set_seed(config.seed)
        timer = Timer(verbosity_level=config.log_verbosity, mode=config.timer_mode, quiet=local_rank != 0)
        bits_communicated = 0
        global_iteration_count = 0
        model_seed = config.seed if config.broadcast_parameters else config.seed + local_rank
        model = CIFAR(device, timer, config.architecture, model_seed, data=config.data, data_path=config.data_path,
                      synthetic_train_size=config.synthetic_train_size,
                      synthetic_test_size=config.synthetic_test_size,
                      broadcast_parameters=config.broadcast_parameters, reference_compat=config.reference_compat)
        optimizer = FlatSGD(model.arena, lr=config.lr, momentum=config.momentum, weight_decay=config.weight_decay,
                            nesterov=config.nesterov)
        scheduler = CosineSchedule(optimizer, T_max=config.num_epochs, eta_min=0)
        if config.norm_scope == "bucket":
            from ..parallel.bucketed import BucketedReducer
            reducer = BucketedReducer(model.parameters, config.reducer, device, timer, cfg_dict, bucket_mb=config.bucket_mb,
                                      max_blocks=config.reduce_max_blocks)
        else:
            reducer = make_reducer(config.reducer, device, timer, cfg_dict)
        # CUDA: the whole step (forward, backward, reduce, update, batch metrics) is one callable, replayed from a CUDA
        # graph when config.graph; the labelled eager path below remains for CPU runs and for per-phase timings
        step = None
        if device.type == "cuda" and (config.graph or config.norm_scope == "bucket"):
            from ..parallel.graph import GraphedStep
            step = GraphedStep(model, reducer, optimizer, enabled=config.graph,
                               fallback="dist" if config.on_collective_timeout == "dist" else None)
        elif config.norm_scope == "bucket":
            reducer.attach()
        start_epoch = 0
        if resume_state is not None and run == resume_state["run"]:
            _, start_epoch, bits_communicated, best_accuracy = ckpt.restore_training_state(
                resume_state, model, optimizer, scheduler, reducer,
                rank_state=ckpt.load_rank_state(config.resume, _global_rank()))
            resume_state = None

        for epoch in range(start_epoch, config.num_epochs):
            if local_rank == 0:
                logger.log_info("epoch info", {"Progress": epoch / config.num_epochs, "Current_epoch": epoch},
                                {"lr": scheduler.get_last_lr()})
            epoch_metrics = AverageMeter(device, reference_compat=config.reference_compat)
            for i, batch in enumerate(model.train_dataloader(config.batch_size)):
                if config.max_steps_per_epoch is not None and i >= config.max_steps_per_epoch:
                    break
                global_iteration_count += 1
                epoch_frac = epoch + i / model.len_train_loader
                if watchdog is not None:
                    watchdog.beat(global_iteration_count)
                with timer("batch", epoch_frac):
                    reduce_now = global_iteration_count % config.local_steps == 0
                    if step is not None and reduce_now:
                        step(batch)
                        epoch_metrics.add(step.metrics)
                        bits_communicated += step.bits_per_step
                        continue
                    if config.norm_scope == "bucket" and reduce_now:
                        reducer.start_step()
                    _, grads, metrics = model.batch_loss_with_gradients(batch)
                    epoch_metrics.add(metrics)
                    if reduce_now:
                        # gradients already live in the flat arena: the reducer works in place, so the
                        # reference's "batch.accumulate" copy into send buffers has nothing left to do
                        with timer("batch.reduce", epoch_frac):
                            bits_communicated += reducer.finish() if config.norm_scope == "bucket" else reducer.reduce(grads, grads)
                    with timer("batch.step", epoch_frac, verbosity=2):
                        optimizer.step()
            scheduler.step()
            if step is not None:
                step.check()                  # a reduce that timed out on the device surfaces here at the latest

            with timer("epoch_metrics.collect", epoch, verbosity=2):
                epoch_metrics.reduce()
                if local_rank == 0:
                    for key, value in epoch_metrics.values().items():
                        logger.log_info(key, {"value": value, "epoch": epoch, "bits": bits_communicated},
                                        tags={"split": "train"})
            with timer("test.last", epoch):
                test_stats = model.test()
                if local_rank == 0:
                    for key, value in test_stats.values().items():
                        logger.log_info(key, {"value": value, "epoch": epoch, "bits": bits_communicated},
                                        tags={"split": "test"})
                        if key == "top1_accuracy" and value > best_accuracy["top1"][run]:
                            best_accuracy["top1"][run] = value
                            logger.save_model(model)
                        if key == "top5_accuracy" and value > best_accuracy["top5"][run]:
                            best_accuracy["top5"][run] = value
            if local_rank == 0:
                logger.epoch_update(run, epoch, epoch_metrics, test_stats)
            if config.save_training_state:
                if step is not None:
                    step.sync_host_counters()
                # the reducer's state (error memories, noise counters) differs per worker: every rank writes its own
                logger.save_training_state(ckpt.rank_state(reducer, epoch), name=ckpt.rank_state_name(_global_rank()))
                if local_rank == 0:
                    logger.save_training_state(ckpt.training_state(model, optimizer, scheduler, reducer, run, epoch,
                                                                   bits_communicated, best_accuracy))
        if local_rank == 0:
            print(timer.summary())

    if watchdog is not None:
        watchdog.stop()
    logger.summary_writer(timer, best_accuracy, bits_communicated)
    return logger


def main(argv=None):
    config, args = TrainConfig.from_args(argv)
    local_rank = args.local_rank if args.local_rank is not None else int(os.environ.get("LOCAL_RANK", 0))
    initiate_distributed(config.distributed_backend)
    train(local_rank, config)
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
