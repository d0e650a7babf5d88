"""Symmetric arenas: one device allocation per rank with the same layout everywhere, mapped into
every peer with CUDA IPC, plus the flag / epoch words the fused kernels synchronise on.

``SymmetricArena``  -- one rank of a real multi-GPU group (handles exchanged through
                       ``torch.distributed``; any backend works for the exchange).
``LocalGroup``      -- all ranks of a group on ONE device, wired to each other directly.  The fused
                       kernels then run every rank side by side inside a single cooperative launch,
                       which is how the multi-rank protocols are tested on a single GPU.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ..ops import _native as nat

STATUS_OK, STATUS_TIMEOUT, STATUS_BOUNDS = 0, 1, 3


class CollectiveTimeout(RuntimeError):
    """A bounded device-side wait ran out: some peer never signalled.  The context stays usable."""

    def __init__(self, rank, phase, peer):
        super().__init__(f"rank {rank}: fused collective timed out in phase 0x{phase:x} waiting for "
                         f"{'a local block' if peer == 0xfffe else f'rank {peer}'}")
        self.rank, self.phase, self.peer = rank, phase, peer


class IndexOutOfBounds(RuntimeError):
    """A kernel met an index outside its tensor (an index list handed to the sparse exchange, or -- in the debug-bounds
    build -- any computed gather / scatter index).  The access was skipped; ``index`` is the first such value."""

    def __init__(self, rank, index):
        super().__init__(f"rank {rank}: index {index} is outside the tensor; the access was skipped")
        self.rank, self.index = rank, index


def _ck(err, what):
    if err != 0:
        raise nat.NativeError(f"{what}: CUDA error {err}")


class _Ctx:
    def __init__(self, world, rank, nbytes, device):
        self.world, self.rank, self.bytes, self.device = world, rank, int(nbytes), device
        h = ctypes.c_void_p()
        with torch.cuda.device(device):
            _ck(nat.cuda().gc_comm_create(world, rank, self.bytes, ctypes.byref(h)), "comm_create")
        self.handle = h

    def arena_ptr(self):
        return nat.cuda().gc_comm_arena_ptr(self.handle)

    def status(self):
        out = (ctypes.c_uint32 * 2)()
        with torch.cuda.device(self.device):
            _ck(nat.cuda().gc_comm_status(self.handle, out, nat.stream_ptr()), "comm_status")
        return int(out[0]), int(out[1])

    def clear_status(self):
        with torch.cuda.device(self.device):
            _ck(nat.cuda().gc_comm_clear_status(self.handle, nat.stream_ptr()), "comm_clear_status")

    def destroy(self):
        if self.handle:
            nat.cuda().gc_comm_destroy(self.handle)
            self.handle = None


class _ArenaBase:
    ctxs = ()

    def _launch_arrays(self, ins, outs):
        n = len(self.ctxs)
        ctx_arr = (ctypes.c_void_p * n)(*[c.handle for c in self.ctxs])
        in_arr = (ctypes.c_void_p * n)(*[t.data_ptr() for t in ins])
        out_arr = (ctypes.c_void_p * n)(*[t.data_ptr() for t in outs])
        return ctx_arr, n, in_arr, out_arr

    def check(self):
        """Raise ``CollectiveTimeout`` / ``IndexOutOfBounds`` if a kernel recorded a failure; synchronises the stream.  Every
        rank's status word is read and cleared before the first failure is raised, so the next launch starts clean."""
        first = None
        for c in self.ctxs:
            status, detail = c.status()
            if status == STATUS_OK:
                continue
            c.clear_status()
            if first is not None:
                continue
            if status == STATUS_TIMEOUT:
                first = CollectiveTimeout(c.rank, detail >> 16, detail & 0xFFFF)
            elif status == STATUS_BOUNDS:
                first = IndexOutOfBounds(c.rank, detail - (1 << 32) if detail >= (1 << 31) else detail)
            else:
                first = nat.NativeError(f"fused kernel reported status {status} (detail {detail})")
        if first is not None:
            raise first

    def close(self):
        for c in self.ctxs:
            c.destroy()
        self.ctxs = ()


class SymmetricArena(_ArenaBase):
    def __init__(self, nbytes, device=None, group=None):
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if self.world > nat.cuda().gc_comm_max_world():
            raise ValueError("fused collectives cover one NVSwitch domain (<= 8 ranks)")
        self.device = torch.device(device if device is not None else torch.cuda.current_device())
        self.bytes = int(nbytes)
        ctx = _Ctx(self.world, self.rank, nbytes, self.device)
        self.ctxs = (ctx,)
        if self.world > 1:
            buf = (ctypes.c_uint8 * 64)()
            _ck(nat.cuda().gc_comm_ipc_handle(ctx.handle, buf), "ipc_handle")
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(buf), group=group)
            blob = b"".join(handles)
            with torch.cuda.device(self.device):
                _ck(nat.cuda().gc_comm_open_peers(ctx.handle, blob), "open_peers")
            dist.barrier(group=group)


class LocalGroup(_ArenaBase):
    """W ranks emulated on one device (tests / single-GPU development)."""

    def __init__(self, world, nbytes, device=None):
        self.world, self.rank = world, 0
        self.device = torch.device(device if device is not None else torch.cuda.current_device())
        self.bytes = int(nbytes)
        self.ctxs = tuple(_Ctx(world, r, nbytes, self.device) for r in range(world))
        for c in self.ctxs:
            for r, other in enumerate(self.ctxs):
                _ck(nat.cuda().gc_comm_set_peer(c.handle, r, other.arena_ptr()), "set_peer")


def required_bytes(n):
    return int(nat.cuda().gc_comm_required_bytes(int(n)))


def oneshot_bytes(region_bytes):
    """Arena size for the one-shot kernels when each of the two parity regions must hold ``region_bytes``."""
    return int(nat.cuda().gc_comm_oneshot_bytes(int(region_bytes)))
