"""Reducer framework (reference: reducer.py:26-68).

A reducer turns the per-worker gradient lists into their cross-worker average:
``reduce(grad_in, grad_out) -> bits`` where ``grad_in`` are send buffers (may be mutated for error
feedback) and ``grad_out`` the live ``param.grad`` tensors to overwrite.

Differences from the reference, by design:

* no process group is required: without ``torch.distributed`` the reducer runs with one worker;
* when the tensors of a list are consecutive views of one flat allocation (as handed out by
  ``parallel.FlatArena``) flattening is a zero-copy view and the write-back is a single kernel;
  otherwise one ``torch.cat`` / one ``_foreach_copy_`` replaces the per-tensor Python loops;
* the 1/W average is folded into the dequantisation scale (the reference zero-fills and then
  ``add_(alpha=1/W)`` per tensor);
* ``bits`` returned by ``reduce`` follow the reference's accounting (8 * nelement * element_size
  of the arrays it hands to the collectives) so logs stay comparable; ``last_wire_bits`` holds what
  the packed wire format of this library actually moves per worker.
"""
from __future__ import annotations

import functools

import torch
import torch.distributed as dist

from ..utils.timer import NullTimer


def _dist_on():
    return dist.is_available() and dist.is_initialized()


class TensorBuffer:
    """Flat view of a list of tensors with per-tensor access (reference: reducer.py:46-68).

    Zero-copy when the tensors already sit back to back in one allocation."""

    def __init__(self, tensors, copy=None):
        sizes = [t.numel() for t in tensors]
        self._start_idx, self._end_idx, off = [], [], 0
        for n in sizes:
            self._start_idx.append(off)
            off += n
            self._end_idx.append(off)
        self._len_tensors = len(tensors)
        self._tensor_shapes = [t.size() for t in tensors]
        self.total = off
        alias = self._aliased_flat(tensors) if copy is not True else None
        if alias is not None and copy is None:
            self.buffer, self.is_view = alias, True
        else:
            self.buffer = torch.cat([t.reshape(-1) for t in tensors]) if tensors else torch.empty(0)
            self.is_view = False

    @staticmethod
    def _aliased_flat(tensors):
        if not tensors:
            return None
        t0 = tensors[0]
        if not all(t.is_contiguous() and t.dtype == t0.dtype and t.device == t0.device for t in tensors):
            return None
        try:
            storage_ptr = t0.untyped_storage().data_ptr()
            if any(t.untyped_storage().data_ptr() != storage_ptr for t in tensors):
                return None
        except Exception:
            return None
        off = t0.storage_offset()
        for t in tensors:
            if t.storage_offset() != off:
                return None
            off += t.numel()
        total = off - t0.storage_offset()
        return torch.as_strided(t0, (total,), (1,), t0.storage_offset())

    def __getitem__(self, index):
        return self.buffer[self._start_idx[index]: self._end_idx[index]].view(self._tensor_shapes[index])

    def __len__(self):
        return self._len_tensors

    def __iter__(self):
        for i in range(self._len_tensors):
            yield self[i]

    def scatter_to(self, outs):
        """outs[i][:] = self[i] for all i with the fewest kernels possible."""
        alias = self._aliased_flat(outs)
        if alias is not None and alias.numel() == self.buffer.numel():
            if alias.data_ptr() != self.buffer.data_ptr():
                alias.copy_(self.buffer)
            return
        torch._foreach_copy_(list(outs), [self[i] for i in range(self._len_tensors)])


def n_bits(tensor):
    return 8 * tensor.nelement() * tensor.element_size()


def physical(t):
    """The contiguous view of ``t`` in the order its elements lie in memory.  Only 4-D channels-last tensors differ
    from themselves: [N, C, H, W] strided as NHWC becomes the contiguous [N, H, W, C] view.  Reducers work on element
    vectors and on matrices whose rows are dim 0, so the order inside a row is theirs to choose; taking the memory
    order keeps a flat gradient arena zero-copy for channels-last weights."""
    if t.dim() == 4 and not t.is_contiguous() and t.is_contiguous(memory_format=torch.channels_last):
        return t.permute(0, 2, 3, 1)
    return t


def _physical_args(reduce_fn):
    @functools.wraps(reduce_fn)
    def reduce(self, grad_in, grad_out):
        return reduce_fn(self, [physical(t) for t in grad_in], [physical(t) for t in grad_out])

    reduce._physical_wrapped = True
    return reduce


class Reducer:
    """Base class of all reducers.

    ``backend``: ``"dist"`` = native ops + ``torch.distributed`` collectives (NCCL on GPU, gloo on
    CPU); ``"fused"`` = one hand-written kernel per step that compresses and reduces over peer memory
    (CUDA only); ``"auto"`` = fused when a fused implementation and a symmetric arena are available.
    """

    fused_capable = False

    def __init_subclass__(cls, **kwargs):
        super().__init_subclass__(**kwargs)
        fn = cls.__dict__.get("reduce")
        if fn is not None and not getattr(fn, "_physical_wrapped", False):
            cls.reduce = _physical_args(fn)         # every reduce() sees contiguous tensors in memory order

    def __init__(self, device, timer=None, backend="auto", seed=0, group=None, reference_compat=False):
        if _dist_on():
            self.n_workers = dist.get_world_size(group)
            self.rank = dist.get_rank(group)
        else:
            self.n_workers, self.rank = 1, 0
        self._device = torch.device(device) if not isinstance(device, torch.device) else device
        self._timer = timer if timer is not None else NullTimer()
        self._group = group
        self._seed = seed
        self._compat = reference_compat
        self.backend = backend
        self.last_wire_bits = 0
        self._fused = None

    # -- collectives ------------------------------------------------------------------------
    def _all_reduce(self, tensor, op=None):
        if self.n_workers > 1:
            dist.all_reduce(tensor, op=op if op is not None else dist.ReduceOp.SUM, group=self._group)
        return tensor

    def _all_reduce_levels(self, levels):
        """Sum of integer quantisation levels over the workers.  Levels of fewer than 8 bits travel in int8 containers, and
        a sum of W of them leaves int8 as soon as s * W > 127 (the reference all-reduces the int8 tensor and wraps,
        reducer.py:537): the collective therefore runs on an int32 copy (neither gloo nor NCCL sums int16).
        ``reference_compat=True`` keeps the container, wrap included."""
        if self.n_workers > 1 and levels.dtype == torch.int8 and not self._compat:
            levels = levels.to(torch.int32)
        return self._all_reduce(levels)

    def _all_gather(self, tensor):
        if self.n_workers == 1:
            return [tensor]
        outs = [torch.empty_like(tensor) for _ in range(self.n_workers)]
        dist.all_gather(outs, tensor, group=self._group)
        return outs

    def _global_max(self, local):
        """max over workers of a 1-element tensor, as one MAX all-reduce (the reference all-gathers
        W scalars and takes a host-side max: reducer.py:519-523)."""
        if self.n_workers > 1:
            local = local.clone()
            dist.all_reduce(local, op=dist.ReduceOp.MAX, group=self._group)
        return local

    # -- helpers ----------------------------------------------------------------------------
    def _use_fused(self):
        if self.backend == "dist" or not self.fused_capable or self._device.type != "cuda":
            return False
        return True

    def reduce(self, grad_in, grad_out):
        raise NotImplementedError()

    @staticmethod
    def n_bits(tensor):
        return n_bits(tensor)

    def state_dict(self):
        return {}

    def load_state_dict(self, sd):
        pass
