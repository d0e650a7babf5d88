"""Host-side model checkers: the flag / epoch protocol of the fused collectives (``csrc/gc_comm.cuh``), the per-rank grid
barrier, and the mbarrier pipeline of the persistent tensor-core GEMM (``csrc/gc_gemm_tc.cu``).

The fused kernels synchronise ranks with monotonically increasing epochs: ``signal_all(phase, epoch)`` stores the
epoch into ``flag[phase][me]`` of every peer, ``wait_all(phase, epoch)`` spins until every ``flag[phase][*]`` of the
own header has reached it, and ``exchange_max`` writes ``(epoch, value)`` into a slot chosen by the epoch's parity.
Nothing is ever reset between steps, so correctness rests on ordering arguments of the kind "rank A can only overwrite
buffer X in step e + 1 after rank B, which reads X in step e, has signalled something that A waits for".  This module
checks those arguments mechanically: every kernel is written down as the sequence of its remotely visible actions
(writes into the own or a peer's arena, reads from them, signals, waits), each rank runs that sequence for a number of
steps, and ALL interleavings of the ranks' actions are explored (depth-first, with memoised states).  Every value
carries the epoch it was written in; a read that finds any other epoch than its own step's is a violation (a stale read
is a missing wait, a too-new one is an overwrite that came too early), and a state in which no rank can move is a
deadlock.

The model treats a rank as one sequential agent: inside a rank the per-rank grid barrier of the kernels makes every
phase complete before the next signal is sent.  Memory is sequentially consistent, which is what the system-scope
release stores / acquire loads of the flags provide for data written before a signal and read after the matching wait.

The reference has no counterpart (it blocks on one NCCL collective after the other: reducer.py:520-549).
"""
from __future__ import annotations

# A kernel = list of operations of ONE step, executed by every rank with its own rank id r and the step's epoch e:
#   ("write_own", region)    r writes its part of `region` in its own arena
#   ("write_peers", region)  r writes its part of `region` in EVERY rank's arena (a push), one action per target
#   ("read_peers", region)   r reads, from every rank q's arena, the part of `region` that q wrote itself
#   ("read_own", region)     r reads, from its own arena, the parts of `region` every rank pushed there
#   ("signal", phase)        flag[phase][r] := e in every rank's header, one action per target
#   ("wait", phase)          blocks until flag[phase][q] >= e for every q in the own header
#   ("norm",)                exchange_max: slot[e & 1][r] := e in every header, then block until every own slot[e & 1][q] == e
#                            (("norm", "single") models one slot per source instead of two: a seeded fault for the tests)
# A region name may contain "{p}", replaced by the epoch's parity (buffers double-buffered by parity).
KERNELS = {
    # quantise + pack -> READY -> owner-pull reduce of the peers' packed rows, push of the sums -> DONE -> dequantise
    "qsgd": [("norm",), ("write_own", "packed"), ("signal", "READY"), ("wait", "READY"), ("read_peers", "packed"),
             ("write_peers", "sums"), ("signal", "DONE"), ("wait", "DONE"), ("read_own", "sums")],
    # the two-scale / multi-scale kernels add the vote round: votes -> MASK -> read everybody's votes
    "twoscale": [("norm",), ("write_own", "votes"), ("signal", "MASK"), ("wait", "MASK"), ("read_peers", "votes"),
                 ("write_own", "packed"), ("signal", "READY"), ("wait", "READY"), ("read_peers", "packed"),
                 ("write_peers", "sums"), ("signal", "DONE"), ("wait", "DONE"), ("read_own", "sums")],
    # two-shot fp32 all-reduce
    "allreduce": [("write_own", "stage"), ("signal", "STAGE"), ("wait", "STAGE"), ("read_peers", "stage"),
                  ("write_peers", "result"), ("signal", "DONE"), ("wait", "DONE"), ("read_own", "result")],
    # one-shot sum of a short vector: no closing round, the buffer is double-buffered by epoch parity instead
    "small_sum": [("write_own", "buf{p}"), ("signal", "AUX"), ("wait", "AUX"), ("read_peers", "buf{p}")],
    # shared-index Rand-K (two-scale form): votes and quantised levels are one-shot and parity double-buffered; the norm
    # exchange at the start of the next launches is what keeps a fast rank from lapping a slow one
    "randk": [("norm",), ("write_own", "mask{p}"), ("signal", "MASK"), ("wait", "MASK"), ("read_peers", "mask{p}"),
              ("write_own", "levels{p}"), ("signal", "READY"), ("wait", "READY"), ("read_peers", "levels{p}")],
    # sparse (index, value) exchange of the Top-K reducers: lists published once, read by everybody
    "sparse": [("write_own", "lists{p}"), ("signal", "AUX"), ("wait", "AUX"), ("read_peers", "lists{p}")],
}


class ProtocolViolation(AssertionError):
    pass


def oneshot_schedule(sizes, half=None):
    """Launches of a one-shot kernel (publish, signal, wait, read everybody's; no closing round) whose buffers have
    different sizes, with the arena modelled as numbered cells so that overlaps between launches show up.

    ``sizes[i]`` cells are published by launch ``i`` (epoch ``i + 1``) in the region of the epoch's parity.
    ``half=None``: the regions of a launch lie back to back, ``[parity * size, (parity + 1) * size)`` -- the layout
    whose parity-1 region moves with the size of the call, so that a larger launch's parity-0 region covers what the
    previous, smaller launch published (the fault).  ``half=H``: parity ``p`` starts at cell ``p * H`` whatever the
    size (``gc_fused.cu::parity_half_bytes``)."""
    schedule = []
    for i, size in enumerate(sizes):
        par = (i + 1) & 1
        first = par * (size if half is None else half)
        assert half is None or size <= half
        cells = [f"cell{c}" for c in range(first, first + size)]
        schedule.append([("write_own", c) for c in cells] + [("signal", "AUX"), ("wait", "AUX")] +
                        [("read_peers", c) for c in cells])
    return schedule


def _expand(kernel_ops, world, rank, epoch):
    """Micro-actions of one step of one rank: (kind, target rank, name, epoch)."""
    acts = []
    for op in kernel_ops:
        kind = op[0]
        name = op[1].replace("{p}", str(epoch & 1)) if len(op) > 1 else ""
        if kind == "write_own":
            acts.append(("write", rank, name, epoch))
        elif kind == "write_peers":
            acts += [("write", q, name, epoch) for q in range(world)]
        elif kind == "read_peers":
            acts += [("read_self_written", q, name, epoch) for q in range(world)]
        elif kind == "read_own":
            acts += [("read_pushed", q, name, epoch) for q in range(world)]          # q = the rank that pushed the part
        elif kind == "signal":
            acts += [("flag", q, name, epoch) for q in range(world)]
        elif kind == "wait":
            acts.append(("wait", rank, name, epoch))
        elif kind == "norm":
            slot = "0" if name == "single" else str(epoch & 1)      # ("norm", "single"): what would happen without the parity
            acts += [("slot", q, slot, epoch) for q in range(world)]
            acts.append(("wait_slots", rank, slot, epoch))
        else:
            raise ValueError(f"unknown operation {op!r}")
    return acts


def _program(schedule, world, rank):
    """All micro-actions of a rank for a schedule = list of kernel names or operation lists, one launch per entry."""
    acts = []
    for step, k in enumerate(schedule):
        acts += _expand(KERNELS[k] if isinstance(k, str) else k, world, rank, step + 1)
    return acts


def check(schedule, world=2, max_states=2_000_000):
    """Explore every interleaving of ``world`` ranks running ``schedule`` (launch i uses epoch i + 1 on every rank).
    Returns the number of distinct states visited; raises ``ProtocolViolation`` with a witness trace otherwise."""
    programs = [_program(schedule, world, r) for r in range(world)]
    # memory: data[(owner, region, writer)] = epoch; flags[(owner, phase, source)] = epoch; slots[(owner, parity, source)] = epoch
    start = (tuple(0 for _ in range(world)), (), (), ())
    seen = {start}
    stack = [(start, ())]
    while stack:
        (pcs, data_t, flags_t, slots_t), trace = stack.pop()
        data, flags, slots = dict(data_t), dict(flags_t), dict(slots_t)
        moved = False
        for r in range(world):
            if pcs[r] >= len(programs[r]):
                continue
            kind, q, name, e = programs[r][pcs[r]]
            nd, nf, ns = data, flags, slots
            if kind == "wait":
                if any(flags.get((r, name, s), 0) < e for s in range(world)):
                    continue                                            # blocked
            elif kind == "wait_slots":
                if any(slots.get((r, name, s), 0) != e for s in range(world)):
                    if any(slots.get((r, name, s), 0) > e for s in range(world)):
                        raise ProtocolViolation(f"rank {r}, epoch {e}: a norm slot was overwritten before it was read\n"
                                                + _format(trace))
                    continue
            elif kind == "write":
                nd = dict(data)
                nd[(q, name, r)] = e
            elif kind == "flag":
                nf = dict(flags)
                nf[(q, name, r)] = e
            elif kind == "slot":
                ns = dict(slots)
                ns[(q, name, r)] = e
            elif kind in ("read_self_written", "read_pushed"):
                key = (q, name, q) if kind == "read_self_written" else (r, name, q)
                got = data.get(key, 0)
                if got != e:
                    what = "stale data (a wait is missing)" if got < e else "data of a later step (overwritten too early)"
                    raise ProtocolViolation(f"rank {r}, epoch {e}: read of {name!r} "
                                            f"{'written by' if kind == 'read_self_written' else 'pushed by'} rank {q} "
                                            f"found epoch {got}: {what}\n" + _format(trace + ((r, kind, q, name, e),)))
            moved = True
            npcs = pcs[:r] + (pcs[r] + 1,) + pcs[r + 1:]
            state = (npcs, tuple(sorted(nd.items())), tuple(sorted(nf.items())), tuple(sorted(ns.items())))
            if state not in seen:
                if len(seen) >= max_states:
                    raise RuntimeError("state budget exhausted: use fewer ranks or steps")
                seen.add(state)
                stack.append((state, trace + ((r, kind, q, name, e),)))
        if not moved and any(pcs[r] < len(programs[r]) for r in range(world)):
            raise ProtocolViolation("deadlock: no rank can move\n" + _format(trace))
    return len(seen)


def _format(trace, last=24):
    lines = [f"  rank {r}: {kind} {name!r} -> rank {q} (epoch {e})" for (r, kind, q, name, e) in trace[-last:]]
    return "last actions of one violating interleaving:\n" + "\n".join(lines)


def check_grid_barrier(nblocks=3, rounds=3, reset_before_release=True):
    """All interleavings of ``nblocks`` blocks passing ``rounds`` consecutive per-rank grid barriers
    (``gc_comm.cuh::grid_barrier``): read the generation; add one to the arrival count; the last arriver resets the
    count and THEN bumps the generation, everybody else spins until the generation moves.  Checked: no block leaves
    barrier k before every block has arrived at barrier k, and nobody is stuck.  ``reset_before_release=False`` swaps
    the last arriver's two stores -- the fault the order of those stores guards against (a released block re-enters
    and its arrival is wiped out by the late reset)."""
    # per block: (round, pc) with pc 0 = read gen, 1 = atomic add, 2 / 3 = the last arriver's two stores, 4 = spin
    start = (tuple((0, 0, 0, False) for _ in range(nblocks)), 0, 0, tuple(0 for _ in range(nblocks)))
    seen, stack = {start}, [start]
    while stack:
        blocks, count, gen, arrived = stack.pop()
        moved = False
        for b, (rnd, pc, my_gen, last) in enumerate(blocks):
            if rnd >= rounds:
                continue
            n_count, n_gen, n_arr = count, gen, arrived
            if pc == 0:
                nb = (rnd, 1, gen, False)
            elif pc == 1:
                n_arr = arrived[:b] + (rnd + 1,) + arrived[b + 1:]
                n_count = count + 1
                nb = (rnd, 2, my_gen, True) if count == nblocks - 1 else (rnd, 4, my_gen, False)
            elif pc == 2:
                if reset_before_release:
                    n_count = 0
                else:
                    n_gen = gen + 1
                nb = (rnd, 3, my_gen, True)
            elif pc == 3:
                if reset_before_release:
                    n_gen = gen + 1
                else:
                    n_count = 0
                nb = None                                     # leaves the barrier
            else:
                if gen == my_gen:
                    continue                                  # still spinning
                nb = None
            if nb is None:
                if any(a < rnd + 1 for a in arrived):
                    raise ProtocolViolation(f"block {b} left barrier {rnd} before every block had arrived: {arrived}")
                nb = (rnd + 1, 0, 0, False)
            moved = True
            state = (blocks[:b] + (nb,) + blocks[b + 1:], n_count, n_gen, n_arr)
            if state not in seen:
                seen.add(state)
                stack.append(state)
        if not moved and any(rnd < rounds for (rnd, _, _, _) in blocks):
            raise ProtocolViolation(f"deadlock in the grid barrier: blocks {blocks}, count {count}, generation {gen}")
    return len(seen)


class _MBarrier:
    """mbarrier with an arrival count: the phase completes (its parity flips) when `count` arrivals have been seen;
    ``passes(parity)`` is ``mbarrier.try_wait.parity``: true once the phase with that parity has completed."""

    def __init__(self, count):
        self.count, self.pending, self.phase = count, count, 0

    def arrive(self):
        self.pending -= 1
        if self.pending == 0:
            self.pending, self.phase = self.count, self.phase ^ 1

    def passes(self, parity):
        return self.phase != parity

    def key(self):
        return (self.pending, self.phase)


def check_gemm_pipeline(tiles=5, kblocks=3, stages=3, epilogue_threads=2, acc_buffers=2, empty_parity_offset=1,
                        acc_empty_count=None):
    """All interleavings of the three roles of ``gemm_tf32_persistent_kernel`` (``csrc/gc_gemm_tc.cu``) over ``tiles``
    output tiles of ``kblocks`` k-blocks each: the TMA producer (waits ``empty[s]`` with parity ``phase ^ 1``, fills
    stage s, which completes ``full[s]``), the MMA issuer (waits ``acc_empty[buf]`` with parity ``aphase ^ 1``, then per
    k-block waits ``full[s]`` with parity ``phase``, reads the stage, commits ``empty[s]``; after the last k-block
    commits ``acc_full[buf]``) and the epilogue threads (wait ``acc_full[buf]`` with parity ``aphase``, read the
    accumulator, arrive on ``acc_empty[buf]``), with ``phase = (it / stages) & 1`` for the running k-block counter
    ``it`` and ``buf = tile & 1``, ``aphase = (tile >> 1) & 1``.  Checked: a stage is never refilled before it was read
    nor read before it was filled, an accumulator is never overwritten before every epilogue thread drained it nor
    drained before it is complete, and nobody is stuck.  Seeded faults for the tests: ``empty_parity_offset=0`` (waiting
    for the wrong parity of a fresh ``empty`` barrier) and ``acc_empty_count`` smaller than the number of epilogue threads
    (the accumulator is handed back while somebody still reads it)."""
    total = tiles * kblocks

    def initial():
        return {"full": [_MBarrier(1) for _ in range(stages)], "empty": [_MBarrier(1) for _ in range(stages)],
                "acc_full": [_MBarrier(1) for _ in range(acc_buffers)],
                "acc_empty": [_MBarrier(acc_empty_count or epilogue_threads) for _ in range(acc_buffers)]}

    # state: producer it, mma (tile, k, waited_acc), epilogue tiles (per thread), stage contents, accumulator contents, barriers
    def freeze(st):
        return (st["p"], st["m"], tuple(st["e"]), tuple(st["stage"]), tuple(st["acc"]), tuple(st["drained"]),
                tuple(tuple(b.key() for b in st["bars"][k]) for k in ("full", "empty", "acc_full", "acc_empty")))

    import copy

    st0 = {"p": 0, "m": (0, 0, False), "e": [0] * epilogue_threads, "stage": [-1] * stages, "acc": [-1] * acc_buffers,
           "drained": [0] * acc_buffers, "bars": initial()}
    seen, stack = {freeze(st0)}, [st0]
    while stack:
        st = stack.pop()
        succ = []
        # producer: k-block `it` goes into stage it % stages
        it = st["p"]
        if it < total:
            s, phase = it % stages, (it // stages) & 1
            if st["bars"]["empty"][s].passes(phase ^ empty_parity_offset):
                n = copy.deepcopy(st)
                if n["stage"][s] != -1:
                    raise ProtocolViolation(f"producer refills stage {s} (k-block {it}) before k-block {n['stage'][s]} was read")
                n["stage"][s] = it
                n["bars"]["full"][s].arrive()
                n["p"] = it + 1
                succ.append(n)
        # MMA issuer
        tile, k, waited = st["m"]
        if tile < tiles:
            buf, aphase = tile % acc_buffers, (tile // acc_buffers) & 1
            if not waited:
                if st["bars"]["acc_empty"][buf].passes(aphase ^ 1):
                    n = copy.deepcopy(st)
                    if n["acc"][buf] != -1 and n["drained"][buf] < epilogue_threads:
                        raise ProtocolViolation(f"MMA starts tile {tile} in accumulator {buf} before tile {n['acc'][buf]} was drained")
                    n["acc"][buf], n["drained"][buf] = -1, 0
                    n["m"] = (tile, 0, True)
                    succ.append(n)
            else:
                mit = tile * kblocks + k
                s, phase = mit % stages, (mit // stages) & 1
                if st["bars"]["full"][s].passes(phase):
                    n = copy.deepcopy(st)
                    if n["stage"][s] != mit:
                        raise ProtocolViolation(f"MMA reads stage {s} expecting k-block {mit}, found {n['stage'][s]}")
                    n["stage"][s] = -1
                    n["bars"]["empty"][s].arrive()
                    if k + 1 == kblocks:
                        n["acc"][buf] = tile
                        n["bars"]["acc_full"][buf].arrive()
                        n["m"] = (tile + 1, 0, False)
                    else:
                        n["m"] = (tile, k + 1, True)
                    succ.append(n)
        # epilogue threads
        for t in range(epilogue_threads):
            et = st["e"][t]
            if et < tiles:
                buf, aphase = et % acc_buffers, (et // acc_buffers) & 1
                if st["bars"]["acc_full"][buf].passes(aphase):
                    n = copy.deepcopy(st)
                    if n["acc"][buf] != et:
                        raise ProtocolViolation(f"epilogue thread {t} drains accumulator {buf} expecting tile {et}, found {n['acc'][buf]}")
                    n["drained"][buf] += 1
                    n["bars"]["acc_empty"][buf].arrive()
                    n["e"][t] = et + 1
                    succ.append(n)
        done = st["p"] >= total and st["m"][0] >= tiles and all(e >= tiles for e in st["e"])
        if not succ and not done:
            raise ProtocolViolation(f"pipeline deadlock: producer at {st['p']}, MMA at {st['m']}, epilogue at {st['e']}")
        for n in succ:
            key = freeze(n)
            if key not in seen:
                seen.add(key)
                stack.append(n)
    return len(seen)
