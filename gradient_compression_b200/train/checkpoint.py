"""Checkpoints.  ``model.pt`` is the model ``state_dict`` exactly as the reference saves it
(logger.py:65-66, keys like ``layer1.0.conv1.weight`` / ``features.0.weight``).  The optional full
training state adds what the reference never saves: momentum, schedule position, reducer error
memories / index-queue position / Philox counters, epoch, run and the bit counter.

Rank 0 writes ``train_state.pt`` (model, optimiser, schedule, its own reducer state); the reducer's state differs per
worker (error-feedback memories, rounding-noise counters), so every rank also writes ``train_state.rank<r>.pt`` next
to it and, on resume from ``<name>.pt``, loads its own ``<name>.rank<r>.pt`` -- never rank 0's."""
from __future__ import annotations

import os

import torch


def rank_state_name(rank, base="train_state.pt"):
    stem = base[:-3] if base.endswith(".pt") else base
    return f"{stem}.rank{int(rank)}.pt"


def rank_state(reducer, epoch=None):
    return {"reducer": reducer.state_dict(), "reducer_class": type(reducer).__name__, "epoch": epoch}


def load_rank_state(resume_path, rank):
    """This rank's reducer state saved beside ``resume_path``, or None (single-worker checkpoints, older layouts)."""
    if not resume_path:
        return None
    path = rank_state_name(rank, os.path.abspath(resume_path))
    if not os.path.exists(path):
        return None
    return torch.load(path, map_location="cpu", weights_only=False)


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


def restore_training_state(state, task, optimizer, scheduler, reducer, rank_state=None):
    """``rank_state``: this rank's own reducer state (``load_rank_state``); without it the reducer state inside
    ``state`` (rank 0's) is used, which is only right for rank 0."""
    task.load_state_dict(state["model"])
    optimizer.load_state_dict(state["optimizer"])
    scheduler.load_state_dict(state["scheduler"])
    red = rank_state if rank_state is not None else state
    if red.get("reducer_class") == type(reducer).__name__:
        reducer.load_state_dict(red["reducer"])
    task._epoch = state.get("task_epoch", state["epoch"] + 1)
    torch.set_rng_state(state["torch_rng"])
    return state["run"], state["epoch"] + 1, state["bits"], state["best_accuracy"]
