"""Run logger (reference: logger.py:12-84).

Writes the same artefacts as the reference into ``<root>/<timestamp rounded to 30 s>_<arch>/``:
``model.pt`` (best state_dict), ``success.txt`` (completion time, best accuracies, every config
key, total bits), ``log_dict.npy`` (per-[run, epoch] metric arrays, pickled dict) and one
``timer_summary_<rank>.json`` per rank.
"""
from __future__ import annotations

import datetime
import os

import numpy as np
import torch

METRICS = ("train_top1_accuracy", "train_top5_accuracy", "test_top1_accuracy", "test_top5_accuracy",
           "train_loss", "test_loss", "time")


class Logger:
    def __init__(self, config, local_rank, root="./logs", log_path=None):
        cfg = dict(config) if not isinstance(config, dict) else config
        stamp = self.get_log_path().strftime("%Y_%m_%d_%H_%M_%S")
        self._log_path = log_path or os.path.join(root, f"{stamp}_{cfg['architecture']}")
        if local_rank == 0:
            os.makedirs(self._log_path, exist_ok=True)
        self._local_rank = local_rank
        self._config = cfg
        self._start = datetime.datetime.now()
        self._log_dict = {m: np.zeros([cfg["runs"], cfg["num_epochs"]]) for m in METRICS}

    @property
    def log_path(self):
        return self._log_path

    @staticmethod
    def get_log_path(dt=None, roundTo=30):
        """Now, rounded to ``roundTo`` seconds so that every rank derives the same directory."""
        dt = dt or datetime.datetime.now()
        seconds = (dt.replace(tzinfo=None) - dt.min).seconds
        rounding = (seconds + roundTo / 2) // roundTo * roundTo
        return dt + datetime.timedelta(0, rounding - seconds, -dt.microsecond)

    @staticmethod
    def log_info(name, values, tags={}):
        def fmt(v):
            if isinstance(v, (list, tuple)):
                return "[" + ", ".join(f"{float(x):7.3f}" for x in v) + "]"
            return f"{float(v):7.3f}"

        vals = ", ".join(f"{k}:{fmt(values[k])}" for k in sorted(values))
        tgs = ", ".join(f"{k}:{t}" for k, t in tags.items())
        print("{name:20s} - {values} ({tags})".format(name=name, values=vals, tags=tgs))

    def epoch_update(self, run, epoch, epoch_metrics, test_stats):
        nan = float("nan")
        tr = {k: epoch_metrics.values().get(k, nan) for k in ("top1_accuracy", "top5_accuracy", "cross_entropy_loss")}
        te = {k: test_stats.values().get(k, nan) for k in ("top1_accuracy", "top5_accuracy", "cross_entropy_loss")}
        d = self._log_dict
        d["train_top1_accuracy"][run, epoch] = tr["top1_accuracy"]
        d["train_top5_accuracy"][run, epoch] = tr["top5_accuracy"]
        d["test_top1_accuracy"][run, epoch] = te["top1_accuracy"]
        d["test_top5_accuracy"][run, epoch] = te["top5_accuracy"]
        d["train_loss"][run, epoch] = tr["cross_entropy_loss"]
        d["test_loss"][run, epoch] = te["cross_entropy_loss"]
        d["time"][run, epoch] = (datetime.datetime.now() - self._start).total_seconds()

    def save_model(self, model):
        torch.save(model.state_dict(), os.path.join(self._log_path, "model.pt"))

    def save_training_state(self, state, name="train_state.pt"):
        os.makedirs(self._log_path, exist_ok=True)
        torch.save(state, os.path.join(self._log_path, name))

    def summary_writer(self, timer, best_accuracy, bits_communicated):
        os.makedirs(self._log_path, exist_ok=True)
        timer.save_summary(os.path.join(self._log_path, f"timer_summary_{self._local_rank}.json"))
        if self._local_rank != 0:
            return
        with open(os.path.join(self._log_path, "success.txt"), "w") as f:
            f.write(f"Training completed at {datetime.datetime.now()}\n\n")
            f.write(f"Best Top 1 Accuracy: {sum(best_accuracy['top1']) / len(best_accuracy['top1'])}\n")
            f.write(f"Best Top 5 Accuracy: {sum(best_accuracy['top5']) / len(best_accuracy['top5'])}\n\n")
            f.write("Training parameters\n")
            for key, value in self._config.items():
                f.write(f"{key} : {value}\n")
            f.write(f"Bits communicated: {bits_communicated}")
        np.save(os.path.join(self._log_path, "log_dict.npy"), self._log_dict)
