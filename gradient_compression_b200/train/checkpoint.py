"""Checkpoints.  ``model.pt`` is the model ``state_dict`` exactly as the reference saves it
(logger.py:65-66, keys like ``layer1.0.conv1.weight`` / ``features.0.weight``).  The optional full
training state adds what the reference never saves: momentum, schedule position, reducer error
memories / index-queue position / Philox counters, epoch, run and the bit counter."""
from __future__ import annotations

import torch


def training_state(task, optimizer, scheduler, reducer, run, epoch, bits, best_accuracy):
    return {
        "model": task.state_dict(),
        "optimizer": optimizer.state_dict(),
        "scheduler": scheduler.state_dict(),
        "reducer": reducer.state_dict(),
        "reducer_class": type(reducer).__name__,
        "run": run, "epoch": epoch, "bits": bits, "best_accuracy": best_accuracy,
        "task_epoch": task._epoch,
        "torch_rng": torch.get_rng_state(),
    }


def restore_training_state(state, task, optimizer, scheduler, reducer):
    task.load_state_dict(state["model"])
    optimizer.load_state_dict(state["optimizer"])
    scheduler.load_state_dict(state["scheduler"])
    if state.get("reducer_class") == type(reducer).__name__:
        reducer.load_state_dict(state["reducer"])
    task._epoch = state.get("task_epoch", state["epoch"] + 1)
    torch.set_rng_state(state["torch_rng"])
    return state["run"], state["epoch"] + 1, state["bits"], state["best_accuracy"]
