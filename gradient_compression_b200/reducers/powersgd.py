"""PowerSGD rank-r reducer with error feedback (reference: reducer.py:1718-1858).

Per matrix M (a >= 2-D gradient viewed as out_ch x rest): P = M Q, all-reduce P, Gram-Schmidt,
Q = M^T P, all-reduce Q and divide by W, gradient = P Q^T, memory = M - P Q^T.  Tensors with one
dimension or less are plainly averaged.

Differences from the reference, by design: the query matrices come from a shared-seed Philox normal
stream so that every worker multiplies by the same Q (the reference draws from each rank's own
generator, reducer.py:1780-1784); rank-1 tensors get a plain mean (the reference divides by W twice
and adds onto the un-zeroed local gradient, reducer.py:1836-1842); the three all-reduces are issued
on single flat buffers; W = 1 works.
"""
from __future__ import annotations

import torch

from .. import ops
from ..ops import philox
from .base import Reducer, TensorBuffer, n_bits


class RankKReducer(Reducer):
    fused_capable = True

    def __init__(self, device, timer=None, n_power_iterations=0, reuse_query=False, rank=1, seed=0, **kw):
        super().__init__(device, timer, seed=seed, **kw)
        assert n_power_iterations == 0
        self.rank_r = rank
        self.reuse_query = reuse_query
        self.p_memory = None
        self.q_memory = None
        self._memory = None
        self._step = 0
        self._step_dev = None     # device copy of the step counter of the query stream (fused path)
        self._layout = None

    def _device_step(self):
        if self._step_dev is None:
            self._step_dev = torch.tensor([self._step], dtype=torch.int32, device=self._device)
        return self._step_dev

    def graph_safe(self):
        """Replayable from a CUDA graph: the query stream's step counter lives on the device.  With ``reuse_query`` the
        first step differs from the later ones (it draws Q), so capture must come after it -- which the eager warm-up
        steps of ``GraphedStep`` guarantee."""
        return True

    # the reference stores the approximation rank in ``self.rank`` (shadowing the worker rank)
    def _plan(self, grad_in):
        key = tuple(tuple(t.shape) for t in grad_in)
        if self._layout is not None and self._layout["key"] == key:
            return self._layout
        # every matrix's P and Q block starts on a 16-byte boundary of p_memory / q_memory (the kernels read them in
        # quads); p_total / q_total are the sizes of those buffers, p_elems / q_elems the floats that carry information
        hi, lo, p_off, q_off, p_elems, q_elems = [], [], 0, 0, 0, 0
        for i, t in enumerate(grad_in):
            if t.dim() <= 1:
                lo.append(i)
                continue
            n, m = t.shape[0], t.numel() // t.shape[0]
            r = min(n, m, self.rank_r)
            hi.append((i, n, m, r, p_off, q_off))
            p_off += (n * r + 3) // 4 * 4
            q_off += (m * r + 3) // 4 * 4
            p_elems += n * r
            q_elems += m * r
        self._layout = {"key": key, "hi": hi, "lo": lo, "p_total": p_off, "q_total": q_off, "p_elems": p_elems,
                        "q_elems": q_elems}
        return self._layout

    def reduce(self, grad_in, grad_out):
        flat = TensorBuffer(grad_in)
        dev = flat.buffer.device
        plan = self._plan(grad_in)
        with self._timer("reduce.allocate_memory", verbosity=2):
            fresh = self.p_memory is None
            if fresh:
                self.p_memory = torch.zeros(plan["p_total"], device=dev)
                self.q_memory = torch.zeros(plan["q_total"], device=dev)
            if self._memory is None:
                self._memory = torch.zeros_like(flat.buffer)
        if self._use_fused():
            from ..parallel import engine as fused
            bits = fused.powersgd(self, flat, grad_out, plan, fresh)   # adds the error memory inside its first kernel
            if bits is not None:
                self._step += 1
                return bits
        with self._timer("reduce.memory", verbosity=2):
            flat.buffer.add_(self._memory)
        mats = [flat[i].view(n, m) for (i, n, m, r, _, _) in plan["hi"]]
        ps = [self.p_memory[po: po + n * r].view(n, r) for (_, n, m, r, po, qo) in plan["hi"]]
        qs = [self.q_memory[qo: qo + m * r].view(m, r) for (_, n, m, r, po, qo) in plan["hi"]]
        with self._timer("reduce.prepare.q", verbosity=2):
            if not (self.reuse_query and not fresh):
                philox.normal(plan["q_total"], self._seed, philox.stream_id(0, philox.PURPOSE_QINIT), self._step,
                              device=dev, out=self.q_memory)
        with self._timer("reduce.compute.p", verbosity=2):
            for M, q, p in zip(mats, qs, ps):
                torch.matmul(M, q, out=p)
        with self._timer("reduce.p", verbosity=2):
            self._all_reduce(self.p_memory)
        bits = 32 * plan["p_elems"]
        with self._timer("reduce.rank1.pack", verbosity=2):
            rank1 = torch.cat([flat[i].reshape(-1) for i in plan["lo"]]) if plan["lo"] else flat.buffer.new_zeros(0)
        with self._timer("reduce.rank1.all_reduce", verbosity=2):
            self._all_reduce(rank1)
        bits += n_bits(rank1)
        with self._timer("reduce.normalize.p", verbosity=2):
            for p in ps:
                ops.gram_schmidt_(p)
        with self._timer("reduce.compute.q", verbosity=2):
            for M, q, p in zip(mats, qs, ps):
                torch.matmul(M.t(), p, out=q)
        with self._timer("reduce.q", verbosity=2):
            self._all_reduce(self.q_memory)
            self.q_memory.mul_(1.0 / self.n_workers)
        bits += 32 * plan["q_elems"]
        self.last_wire_bits = bits
        with self._timer("reduce.outerprod", verbosity=2):
            self._memory.copy_(flat.buffer)
            for (i, n, m, r, _, _), p, q in zip(plan["hi"], ps, qs):
                approx = torch.matmul(p, q.t())
                s, e = flat._start_idx[i], flat._end_idx[i]
                self._memory[s:e].sub_(approx.view(-1))
                grad_out[i].copy_(approx.view(grad_out[i].shape))
        with self._timer("reduce.rank1.unpack", verbosity=2):
            off = 0
            for i in plan["lo"]:
                k = grad_in[i].numel()
                s, e = flat._start_idx[i], flat._end_idx[i]
                self._memory[s:e].zero_()
                grad_out[i].copy_((rank1[off: off + k] / self.n_workers).view(grad_out[i].shape))
                off += k
        self._step += 1
        return bits

    def state_dict(self):
        if self._step_dev is not None:
            self._step = int(self._step_dev.item())
        sd = {"step": self._step}
        for k in ("_memory", "p_memory", "q_memory"):
            if getattr(self, k) is not None:
                sd[k] = getattr(self, k)
        return sd

    def load_state_dict(self, sd):
        self._step = int(sd["step"])
        if self._step_dev is not None:
            self._step_dev.fill_(self._step)
        for k in ("_memory", "p_memory", "q_memory"):
            if k in sd:
                setattr(self, k, sd[k].to(self._device).clone())
