"""Host-side failure detection (the reference has none: a dead rank hangs NCCL forever).

``StepWatchdog``: every rank publishes "I reached step s" in a key-value store (the process group's
TCPStore, or any object with ``set`` / ``get``) and a background thread checks how stale the slowest
peer is.  When a peer has not advanced for ``timeout_s`` the watchdog records a ``PeerStalled`` error
that ``beat()`` / ``check()`` re-raise in the training thread *before the next launch*, so no kernel is
left waiting on a rank that is gone.  Device-side waits are bounded separately (``CollectiveTimeout``).
"""
from __future__ import annotations

import threading
import time


class PeerStalled(RuntimeError):
    def __init__(self, rank, last_step, age_s):
        super().__init__(f"rank {rank} has not advanced past step {last_step} for {age_s:.1f} s")
        self.rank, self.last_step, self.age_s = rank, last_step, age_s


class DictStore:
    """In-process stand-in for a TCPStore (tests, single-process runs)."""

    def __init__(self):
        self._d, self._lock = {}, threading.Lock()

    def set(self, key, value):
        with self._lock:
            self._d[key] = value if isinstance(value, bytes) else str(value).encode()

    def get(self, key):
        with self._lock:
            return self._d[key]

    def check(self, keys):
        with self._lock:
            return all(k in self._d for k in keys)


class StepWatchdog:
    def __init__(self, store, rank, world, timeout_s=60.0, poll_s=None, prefix="gcb200/hb", clock=time.monotonic):
        self.store, self.rank, self.world = store, rank, world
        self.timeout_s = float(timeout_s)
        self.poll_s = poll_s if poll_s is not None else max(min(self.timeout_s / 4, 5.0), 0.01)
        self.prefix, self.clock = prefix, clock
        self.error = None
        self._seen = {r: (-1, clock()) for r in range(world)}   # rank -> (last step, time it changed)
        self._stop = threading.Event()
        self._thread = None
        self.beat(0)

    @classmethod
    def from_env(cls, timeout_s=60.0):
        import torch.distributed as dist

        if dist.is_available() and dist.is_initialized():
            from torch.distributed.distributed_c10d import _get_default_store
            wd = cls(_get_default_store(), dist.get_rank(), dist.get_world_size(), timeout_s)
        else:
            wd = cls(DictStore(), 0, 1, timeout_s)
        wd.start()
        return wd

    def _key(self, r):
        return f"{self.prefix}/{r}"

    def beat(self, step):
        """Publish progress; raises if a peer was found stalled since the last call."""
        self.store.set(self._key(self.rank), str(int(step)))
        self.check()

    def check(self):
        if self.error is not None:
            raise self.error

    def poll_once(self):
        now = self.clock()
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                if hasattr(self.store, "check") and not self.store.check([self._key(r)]):
                    step = -1
                else:
                    step = int(self.store.get(self._key(r)).decode())
            except Exception:
                step = -1
            last, since = self._seen[r]
            if step != last:
                self._seen[r] = (step, now)
            elif now - since > self.timeout_s and self.error is None:
                self.error = PeerStalled(r, last, now - since)

    def _run(self):
        while not self._stop.wait(self.poll_s):
            self.poll_once()

    def start(self):
        if self.world > 1 and self._thread is None:
            self._thread = threading.Thread(target=self._run, daemon=True, name="gcb200-watchdog")
            self._thread.start()
        return self

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.poll_s + 1)
            self._thread = None
