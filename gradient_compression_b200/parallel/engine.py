"""Python front end of the fused compress+collective kernels (``csrc/gc_fused.cu``).

``FusedOps`` wraps the launches for a ``SymmetricArena`` (one rank per process) or a ``LocalGroup``
(all ranks in one launch).  ``FusedEngine`` adapts them to the reducers' ``reduce(grad_in, grad_out)``
contract.  The module-level functions at the end are what the reducers call: each returns ``None`` (or
``False``) when the fused path does not apply, in which case the reducer continues on its collective
(``dist``) backend; otherwise it performs the whole reduce and returns the reference-accounting bit count.
"""
from __future__ import annotations

import os

import torch

from ..ops import _native as nat
from . import comm


class FusedOps:
    def __init__(self, arena, timeout_ms=None, max_blocks=0):
        self.arena = arena
        self.timeout_ms = int(timeout_ms if timeout_ms is not None else os.environ.get("GCB200_TIMEOUT_MS", 30000))
        self.max_blocks = int(max_blocks)

    def _prep(self, ins, outs):
        ins = [ins] if torch.is_tensor(ins) else list(ins)
        outs = [outs] if torch.is_tensor(outs) else list(outs)
        assert len(ins) == len(outs) == len(self.arena.ctxs)
        for t in ins + outs:
            assert t.is_cuda and t.dtype == torch.float32 and t.is_contiguous()
        return ins, outs, self.arena._launch_arrays(ins, outs)

    def _run(self, what, err):
        nat.check(err, what)

    def qsgd(self, ins, outs, bits, seed, step):
        ins, outs, (ctxs, nv, ia, oa) = self._prep(ins, outs)
        with torch.cuda.device(self.arena.device):
            self._run("fused_qsgd", nat.cuda().gc_fused_qsgd(ctxs, nv, ia, oa, ins[0].numel(), int(bits), int(seed),
                                                            int(step), self.timeout_ms, self.max_blocks,
                                                            nat.stream_ptr()))

    def twoscale(self, ins, outs, bits_lo, bits_hi, seed, step):
        ins, outs, (ctxs, nv, ia, oa) = self._prep(ins, outs)
        with torch.cuda.device(self.arena.device):
            self._run("fused_twoscale", nat.cuda().gc_fused_twoscale(ctxs, nv, ia, oa, ins[0].numel(), int(bits_lo),
                                                                    int(bits_hi), int(seed), int(step),
                                                                    self.timeout_ms, self.max_blocks,
                                                                    nat.stream_ptr()))

    def multiscale(self, ins, outs, levels, seed, step):
        import ctypes
        ins, outs, (ctxs, nv, ia, oa) = self._prep(ins, outs)
        lv = (ctypes.c_int * len(levels))(*[int(b) for b in levels])
        with torch.cuda.device(self.arena.device):
            self._run("fused_multiscale", nat.cuda().gc_fused_multiscale(ctxs, nv, ia, oa, ins[0].numel(), lv, len(levels),
                                                                        int(seed), int(step), self.timeout_ms,
                                                                        self.max_blocks, nat.stream_ptr()))

    def allreduce(self, ins, outs):
        ins, outs, (ctxs, nv, ia, oa) = self._prep(ins, outs)
        with torch.cuda.device(self.arena.device):
            self._run("fused_allreduce", nat.cuda().gc_fused_allreduce(ctxs, nv, ia, oa, ins[0].numel(),
                                                                      self.timeout_ms, self.max_blocks,
                                                                      nat.stream_ptr()))

    def small_sum(self, ins, outs, alpha=1.0):
        ins, outs, (ctxs, nv, ia, oa) = self._prep(ins, outs)
        with torch.cuda.device(self.arena.device):
            self._run("fused_small_sum", nat.cuda().gc_fused_small_sum(ctxs, nv, ia, oa, ins[0].numel(), float(alpha),
                                                                      self.timeout_ms, self.max_blocks,
                                                                      nat.stream_ptr()))

    def randk(self, ins, outs, seed, npass, start, k, bits_lo, bits_hi=0, zero_unselected=False, step=0, window=None):
        """``window`` (one int64 on the device): the kernel takes the window's start from it and advances it, so that
        a replayed CUDA graph selects new coordinates every step; ``k`` is then the nominal window length K."""
        ins, outs, (ctxs, nv, ia, oa) = self._prep(ins, outs)
        assert window is None or (window.is_cuda and window.dtype == torch.int64)
        with torch.cuda.device(self.arena.device):
            self._run("fused_randk", nat.cuda().gc_fused_randk(ctxs, nv, ia, oa, ins[0].numel(), int(seed), int(npass),
                                                              int(start), int(k), int(bits_lo), int(bits_hi),
                                                              int(bool(zero_unselected)), int(step), nat.ptr(window),
                                                              self.timeout_ms, self.max_blocks, nat.stream_ptr()))

    def sparse(self, vals, outs, idxs, alpha):
        vals, outs, (ctxs, nv, ia, oa) = self._prep(vals, outs)
        idxs = [idxs] if torch.is_tensor(idxs) else list(idxs)
        import ctypes
        xa = (ctypes.c_void_p * nv)(*[t.data_ptr() for t in idxs])
        with torch.cuda.device(self.arena.device):
            self._run("fused_sparse", nat.cuda().gc_fused_sparse(ctxs, nv, ia, oa, xa, outs[0].numel(), vals[0].numel(),
                                                                float(alpha), self.timeout_ms, self.max_blocks,
                                                                nat.stream_ptr()))

    def check(self):
        self.arena.check()


_shared_arena = {}

# One-shot arenas are created at least this large, so that buckets or reducers of different sizes do not regrow them.
ONESHOT_MIN_BYTES = 8 << 20


def _drain_group(device, group):
    """Every rank's kernels on the arena have finished: local synchronise, then a barrier over the group."""
    import torch.distributed as dist

    torch.cuda.synchronize(device)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.barrier(group=group)


def shared_arena(nbytes, device, group=None, family="twoshot", make=None, drain=None):
    """One arena per (device, group, kernel family), replaced collectively when a larger one is needed.

    ``family``: the two-shot kernels (QSGD, multi-scale, all-reduce; closing round, whole arena) and the one-shot
    kernels (small sum, sparse exchange, Rand-K; no closing round, two parity regions) never share an arena, so a
    rank that has moved on to the next kernel of the other family cannot write where a slower peer still reads.
    Replacing an arena frees memory that peers have mapped: all ranks reach this call with the same sizes, and the old
    arena is closed only after every rank's kernels have drained (``drain``: local synchronise + group barrier) --
    the one-shot kernels have no closing round, so a local synchronise alone would not do.
    ``make`` / ``drain`` are injection points for tests."""
    key = (str(device), id(group), family)
    cur = _shared_arena.get(key)
    if cur is None or cur.bytes < nbytes:
        if cur is not None:
            (drain or _drain_group)(device, group)
            cur.close()
        cur = (make or comm.SymmetricArena)(nbytes, device, group)
        _shared_arena[key] = cur
    return cur


def _align256(x):
    return (int(x) + 255) // 256 * 256


class FusedEngine:
    """Glue between a reducer and ``FusedOps``: arena sizing, in/out aliasing, bit accounting."""

    def __init__(self, reducer):
        self.device = reducer._device
        self.group = reducer._group
        self._owner = reducer       # its ``fused_max_blocks`` attribute (optional) caps the grid of every launch
        self.ops = None             # FusedOps of the family used last (what status checks look at)
        self._ops = {}              # family -> FusedOps
        self._n = 0

    @classmethod
    def for_reducer(cls, reducer):
        if reducer._device.type != "cuda":
            return None
        return cls(reducer)

    def _ensure(self, n, oneshot_region_bytes=None):
        """``FusedOps`` on the shared arena of the right family: two-shot kernels on an ``n``-element gradient, or
        (``oneshot_region_bytes`` given) one-shot kernels whose parity regions hold that many bytes each."""
        # the arena is shared by every reducer of this device / group and may have been regrown by another
        # one since the last call: always go through the registry, never keep a stale handle
        if oneshot_region_bytes is None:
            # an owner that knows its largest gradient (a bucketed reducer: its largest bucket) says so, and the arena is
            # sized once instead of being replaced when a larger bucket shows up
            family, nbytes = "twoshot", comm.required_bytes(max(n, int(getattr(self._owner, "fused_arena_elements", 0) or 0)))
        else:
            family, nbytes = "oneshot", max(comm.oneshot_bytes(oneshot_region_bytes), ONESHOT_MIN_BYTES)
        arena = shared_arena(nbytes, self.device, self.group, family)
        ops = self._ops.get(family)
        if ops is None or ops.arena is not arena:
            ops = self._ops[family] = FusedOps(arena)
        ops.max_blocks = int(getattr(self._owner, "fused_max_blocks", 0) or 0)
        self.ops = ops
        self._n = max(self._n, n)
        return ops

    def arenas(self):
        """Every arena this engine has launched on (status words to check, graphs to arm)."""
        return [o.arena for o in self._ops.values()]

    @staticmethod
    def _out_flat(flat, grad_out):
        """The flat destination: the aliased flat view of grad_out when it has one."""
        from ..reducers.base import TensorBuffer

        alias = TensorBuffer._aliased_flat(grad_out)
        if alias is not None and alias.numel() == flat.buffer.numel():
            return alias, None
        tmp = torch.empty_like(flat.buffer)
        return tmp, tmp

    def _finish(self, flat, grad_out, dest, tmp):
        if tmp is not None:
            buf = flat.buffer
            flat.buffer = tmp
            flat.is_view = False
            flat.scatter_to(grad_out)
            flat.buffer = buf

    def qsgd_maxnorm(self, reducer, flat, grad_out):
        n = flat.buffer.numel()
        ops = self._ensure(n)
        dest, tmp = self._out_flat(flat, grad_out)
        with reducer._timer("reduce.fused", verbosity=2):
            ops.qsgd(flat.buffer, dest, reducer._quantization_level, reducer._noise.seed, reducer._noise.next_step())
        self._finish(flat, grad_out, dest, tmp)
        container = 8 if reducer._quantization_level < 8 else 32
        reducer.last_wire_bits = reducer._wire_bits(n)
        return 32 + container * n

    def qsgd_twoscale(self, reducer, flat, grad_out):
        n = flat.buffer.numel()
        ops = self._ensure(n)
        dest, tmp = self._out_flat(flat, grad_out)
        with reducer._timer("reduce.fused", verbosity=2):
            ops.twoscale(flat.buffer, dest, reducer._lower_quantization_level, reducer._higher_quantization_level,
                         reducer._noise.seed, reducer._noise.next_step())
        self._finish(flat, grad_out, dest, tmp)
        container = 8 if reducer._lower_quantization_level < 8 else 32
        return 32 + 8 * n + container * n

    def qsgd_multiscale(self, reducer, flat, grad_out):
        levels = reducer._quantization_levels
        if not (2 <= len(levels) <= 4):
            return None
        n = flat.buffer.numel()
        ops = self._ensure(n)
        dest, tmp = self._out_flat(flat, grad_out)
        with reducer._timer("reduce.fused", verbosity=2):
            ops.multiscale(flat.buffer, dest, levels, reducer._noise.seed, reducer._noise.next_step())
        self._finish(flat, grad_out, dest, tmp)
        container = 8 if levels[0] < 8 else 32
        return 32 + 8 * n + container * n

    def allreduce_mean(self, reducer, flat, grad_out):
        n = flat.buffer.numel()
        ops = self._ensure(n)
        dest, tmp = self._out_flat(flat, grad_out)
        ops.allreduce(flat.buffer, dest)
        self._finish(flat, grad_out, dest, tmp)
        return True

    def randk(self, reducer, flat, grad_out, start, k, npass):
        n = flat.buffer.numel()
        ops = self._ensure(n, 3 * _align256(4 * k))
        dest, tmp = self._out_flat(flat, grad_out)
        lo = reducer._quantization_level
        hi = getattr(reducer, "_higher_quantization_level", 0)
        window = reducer._device_window(start)
        with reducer._timer("reduce.fused", verbosity=2):
            ops.randk(flat.buffer, dest, reducer._queue.seed, npass, start, reducer._K if window is not None else k, lo, hi,
                      reducer._unselected == "zero", reducer._noise.next_step(), window=window)
        self._finish(flat, grad_out, dest, tmp)
        container = 8 if lo < 8 else 32
        return 32 + container * k + (8 * k if hi else 0)

    def sparse(self, reducer, flat, grad_out, idx, vals):
        n = flat.buffer.numel()
        ops = self._ensure(n, 2 * _align256(4 * vals.numel()))
        dest, tmp = self._out_flat(flat, grad_out)
        with reducer._timer("reduce.fused", verbosity=2):
            ops.sparse(vals, dest, idx, 1.0 / reducer.n_workers)
        self._finish(flat, grad_out, dest, tmp)
        return True

    def _psgd_tables(self, reducer, flat, plan):
        cache = getattr(reducer, "_psgd_cache", None)
        if cache is not None and cache["key"] == plan["key"]:
            return cache
        rows, tiles, mats = 0, 0, []
        for (i, n, m, r, po, qo) in plan["hi"]:
            mats.append([flat._start_idx[i], n, m, r, po, qo, rows, tiles])
            rows += n
            tiles += int(nat.cuda().gc_cuda_psgd_q_blocks(n, m))        # 128-column tiles x row chunks of this matrix
        vecs, voff = [], 0
        for i in plan["lo"]:
            ln = flat._end_idx[i] - flat._start_idx[i]
            vecs.append([flat._start_idx[i], ln, voff])
            voff += ln
        dev = flat.buffer.device
        cache = {"key": plan["key"], "rows": rows, "tiles": tiles, "n_mats": len(mats), "n_vecs": len(vecs),
                 "v_total": voff,
                 "tab": torch.tensor(mats or [[0] * 8], dtype=torch.int64, device=dev),
                 "vtab": torch.tensor(vecs or [[0] * 3], dtype=torch.int64, device=dev),
                 "stage": torch.zeros(plan["p_total"] + voff, device=dev),       # zeroed: the alignment gaps are never written
                 "reduced": torch.zeros(plan["p_total"] + voff, device=dev),
                 "max_rows": max([n for (_, n, _, _, _, _) in plan["hi"]] or [1]),
                 "q_local": torch.zeros(max(plan["q_total"], 1) * nat.cuda().gc_cuda_psgd_q_chunks(
                     max([n for (_, n, _, _, _, _) in plan["hi"]] or [1])), device=dev)}
        reducer._psgd_cache = cache
        return cache

    def powersgd(self, reducer, flat, grad_out, plan, fresh):
        """The whole PowerSGD step with the kernels of ``csrc/gc_powersgd.cu`` and two one-shot sums."""
        from ..ops import philox

        lib = nat.cuda()
        if reducer.rank_r > lib.gc_cuda_psgd_max_rank():
            return None
        n = flat.buffer.numel()
        c = self._psgd_tables(reducer, flat, plan)
        ops = self._ensure(n, 4 * max(plan["p_total"] + c["v_total"], plan["q_total"], 1))
        dest, tmp = self._out_flat(flat, grad_out)
        g, e = flat.buffer, reducer._memory
        p_total, q_total = plan["p_total"], plan["q_total"]
        with reducer._timer("reduce.prepare.q", verbosity=2):
            if not (reducer.reuse_query and not fresh):
                # the step counter of the query stream lives on the device (a replayed graph draws a new Q every step)
                philox.normal(q_total, reducer._seed, philox.stream_id(0, philox.PURPOSE_QINIT), 0,
                              device=g.device, out=reducer.q_memory, step_offset=reducer._device_step())
                reducer._step_dev.add_(1)
        st = nat.stream_ptr
        with torch.cuda.device(g.device):
            with reducer._timer("reduce.compute.p", verbosity=2):
                nat.check(lib.gc_cuda_psgd_p(g.data_ptr(), e.data_ptr(), c["tab"].data_ptr(), c["n_mats"], c["rows"],
                                             reducer.q_memory.data_ptr(), c["stage"].data_ptr(), c["vtab"].data_ptr(),
                                             c["n_vecs"], p_total, st()), "psgd_p")
            with reducer._timer("reduce.p", verbosity=2):
                ops.small_sum(c["stage"], c["reduced"], alpha=1.0)
            with reducer._timer("reduce.normalize.p", verbosity=2):
                nat.check(lib.gc_cuda_psgd_gs(c["reduced"].data_ptr(), c["tab"].data_ptr(), c["n_mats"], 1e-8, st()),
                          "psgd_gs")
            with reducer._timer("reduce.compute.q", verbosity=2):
                nat.check(lib.gc_cuda_psgd_q(e.data_ptr(), c["tab"].data_ptr(), c["n_mats"], c["tiles"],
                                             c["reduced"].data_ptr(), c["q_local"].data_ptr(), q_total, c["max_rows"],
                                             st()), "psgd_q")
            with reducer._timer("reduce.q", verbosity=2):
                ops.small_sum(c["q_local"][:max(q_total, 1)], reducer.q_memory[:max(q_total, 1)] if q_total else c["q_local"],
                              alpha=1.0 / reducer.n_workers)
            with reducer._timer("reduce.outerprod", verbosity=2):
                nat.check(lib.gc_cuda_psgd_out(dest.data_ptr(), e.data_ptr(), c["tab"].data_ptr(), c["n_mats"], c["rows"],
                                               c["reduced"].data_ptr(), reducer.q_memory.data_ptr(),
                                               c["vtab"].data_ptr(), c["n_vecs"],
                                               c["reduced"][p_total:].data_ptr() if c["v_total"] else None,
                                               1.0 / reducer.n_workers, st()), "psgd_out")
        reducer.p_memory = c["reduced"][:p_total]
        self._finish(flat, grad_out, dest, tmp)
        bits = 32 * (plan["p_elems"] + plan["q_elems"] + c["v_total"])
        reducer.last_wire_bits = bits
        return bits


# ---------------------------------------------------------------------------------------------------------------
# dispatch from the reducers

def _engine(reducer):
    eng = getattr(reducer, "_fused", None)
    if eng is None:
        eng = FusedEngine.for_reducer(reducer)
        reducer._fused = eng if eng is not None else False
    return eng or None


def allreduce_mean(reducer, flat, grad_out):
    eng = _engine(reducer)
    return eng.allreduce_mean(reducer, flat, grad_out) if eng else False


def qsgd_maxnorm(reducer, flat, grad_out):
    eng = _engine(reducer)
    return eng.qsgd_maxnorm(reducer, flat, grad_out) if eng else None


def qsgd_twoscale(reducer, flat, grad_out):
    eng = _engine(reducer)
    return eng.qsgd_twoscale(reducer, flat, grad_out) if eng else None


def qsgd_multiscale(reducer, flat, grad_out):
    eng = _engine(reducer)
    return eng.qsgd_multiscale(reducer, flat, grad_out) if eng else None


def randk(reducer, flat, grad_out, start, k, npass):
    eng = _engine(reducer)
    return eng.randk(reducer, flat, grad_out, start, k, npass) if eng else None


def powersgd(reducer, flat, grad_out, plan, fresh):
    eng = _engine(reducer)
    return eng.powersgd(reducer, flat, grad_out, plan, fresh) if eng else None


def sparse(reducer, flat, grad_out, idx, vals):
    eng = _engine(reducer)
    return eng.sparse(reducer, flat, grad_out, idx, vals) if eng else False
