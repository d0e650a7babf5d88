"""Labelled timing of training phases (reference: timer.py:22-163).

Two modes:

* ``mode="sync"``  -- the reference's method: ``torch.cuda.synchronize()`` on both
  sides of the region and host wall clock.  Comparable with the published logs, but
  each label costs two device syncs and forbids overlap.
* ``mode="event"`` -- a pair of CUDA events recorded on the current stream; durations
  are resolved lazily (at ``summary()``/``save_summary()`` or every ``resolve_every``
  regions) so the hot loop never blocks the host.  On CPU both modes use wall clock.

The label taxonomy, the skip-first rule, the 1/count print sampling and the JSON
summary layout ``{label: {label, average_duration, n_events, total_time}}`` follow
the reference so its plotting inputs keep working.
"""
from __future__ import annotations

import json
import time
from contextlib import contextmanager
from io import StringIO

import numpy as np
import torch

try:  # NVTX ranges are best-effort (present in CUDA builds of torch)
    from torch.cuda import nvtx as _nvtx
except Exception:  # pragma: no cover
    _nvtx = None


class Timer:
    def __init__(self, verbosity_level=1, skip_first=True, on_cuda=True, mode="sync", log_fn=None,
                 resolve_every=256, nvtx=False, quiet=False):
        if mode not in ("sync", "event"):
            raise ValueError("mode must be 'sync' or 'event'")
        self.verbosity_level = verbosity_level
        self.skip_first = skip_first
        self.cuda_available = torch.cuda.is_available() and on_cuda
        self.mode = mode if self.cuda_available else "sync"
        self.log_fn = log_fn or self.log_info
        self.quiet = quiet
        self.nvtx = bool(nvtx and _nvtx is not None and self.cuda_available)
        self.resolve_every = resolve_every
        self.reduce_times = []
        self._pending = []  # (label, epoch, start_event, end_event, host_start, host_end)
        self.reset()

    def reset(self):
        self.totals = {}
        self.first_time = {}
        self.last_time = {}
        self.call_counts = {}
        self._pending = []

    # ------------------------------------------------------------------ regions
    @contextmanager
    def __call__(self, label, epoch=-1.0, verbosity=1):
        if verbosity > self.verbosity_level:
            yield
            return
        if self.nvtx:
            _nvtx.range_push(label)
        if self.mode == "event":
            start_ev = torch.cuda.Event(enable_timing=True)
            end_ev = torch.cuda.Event(enable_timing=True)
            host_start = time.time()
            start_ev.record()
            try:
                yield
            finally:
                end_ev.record()
                if self.nvtx:
                    _nvtx.range_pop()
            self._pending.append((label, epoch, start_ev, end_ev, host_start, time.time()))
            if len(self._pending) >= self.resolve_every:
                self.resolve()
            return

        self._cuda_sync()
        start = time.time()
        try:
            yield
        finally:
            self._cuda_sync()
            end = time.time()
            if self.nvtx:
                _nvtx.range_pop()
        self._account(label, epoch, start, end, end - start)

    def resolve(self):
        """Turn recorded event pairs into durations (one device sync for all of them)."""
        if not self._pending:
            return
        self._pending[-1][3].synchronize()
        pending, self._pending = self._pending, []
        for label, epoch, s_ev, e_ev, h0, h1 in pending:
            self._account(label, epoch, h0, h1, s_ev.elapsed_time(e_ev) * 1e-3)

    def _account(self, label, epoch, start, end, duration):
        if label == "batch.reduce":
            self.reduce_times.append(duration)
        if label not in self.first_time:
            self.first_time[label] = start
        self.last_time[label] = end
        if label not in self.totals and self.skip_first:
            self.totals[label] = 0.0
            del self.first_time[label]
            self.call_counts[label] = 0
        elif label not in self.totals:
            self.totals[label] = duration
            self.call_counts[label] = 1
        else:
            self.totals[label] += duration
            self.call_counts[label] += 1
        count = self.call_counts[label]
        if count > 0 and not self.quiet and np.random.rand() < 1 / count:
            self.log_fn("timer", {"epoch": epoch, "value": duration}, {"event": label})

    # ---------------------------------------------------------------- reporting
    def average(self, label):
        self.resolve()
        count = self.call_counts.get(label, 0)
        return self.totals[label] / count if count else float("nan")

    def summary(self):
        self.resolve()
        if not self.totals:
            return ""
        with StringIO() as buf:
            total_time = 0.0
            count = 0
            print("--- Timer summary -----------------------------------------------", file=buf)
            print("  Event                          |  Count | Average time |  Frac.", file=buf)
            for label in sorted(self.totals):
                total, count = self.totals[label], self.call_counts[label]
                if count == 0:
                    continue
                span = max(self.last_time[label] - self.first_time[label], 1e-12)
                if label == "batch":
                    total_time += total
                print(f"- {label:30s} | {count:6d} | {total / count:11.5f}s | {100 * total / span:5.1f}%", file=buf)
            print("-----------------------------------------------------------------", file=buf)
            print(f"- {'total_time':30s} | {count:6d} | {total_time:11.5f}s |", file=buf)
            print("-----------------------------------------------------------------", file=buf)
            return buf.getvalue()

    def summary_dict(self, include_reduce_times=False):
        self.resolve()
        data = {}
        for label in sorted(self.totals):
            total, count = self.totals[label], self.call_counts[label]
            if count == 0:
                continue
            data[label] = {"label": label, "average_duration": total / count, "n_events": count, "total_time": total}
        if include_reduce_times:
            data["reduce_times"] = list(self.reduce_times)
        return data

    def save_summary(self, json_file_path, include_reduce_times=False):
        with open(json_file_path, "w") as fp:
            json.dump(self.summary_dict(include_reduce_times), fp)

    def _cuda_sync(self):
        if self.cuda_available:
            torch.cuda.synchronize()

    @staticmethod
    def log_info(name, values, tags={}):
        vals = ", ".join(f"{k}:{values[k]:7.3f}" for k in sorted(values))
        tgs = ", ".join(f"{k}:{t}" for k, t in tags.items())
        print("{name:20s} - {values} ({tags})".format(name=name, values=vals, tags=tgs))


class NullTimer(Timer):
    """A timer that measures nothing; used inside graph-captured or fused hot paths."""

    def __init__(self):
        super().__init__(verbosity_level=-1, on_cuda=False, quiet=True)

    @contextmanager
    def __call__(self, label, epoch=-1.0, verbosity=1):
        yield
