"""Compressed-reduce microbenchmark: one fp32 gradient tensor ~ N(0, 1e-3) of 1 K .. 64 M elements pushed
through each compressor at W ranks, three implementations side by side:

  fused      one hand-written kernel per step over peer memory (this library's product path)
  dist       this library's quantise / dequantise kernels + torch.distributed (NCCL) collectives
  reference  the reference's reducer classes from ``baseline/_ref`` (torch ops + NCCL), when installed

Run under torchrun (one process per GPU) or alone (W = 1).  Times are CUDA-event times on the launching
stream, max over ranks, median of ``--iters`` after ``--warmup``; between iterations a 256 MB buffer is
rewritten to flush the 126 MB L2.  Reported per row: microseconds, effective bus bandwidth in the NCCL
convention (2 (W-1)/W x 4N bytes / t, i.e. what an fp32 all-reduce of the same tensor would have to
sustain), and the fused kernel's fraction of its roofline = max(bytes over NVLink / 770 GB/s measured per
direction, HBM bytes / measured copy bandwidth) / t.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m gradient_compression_b200.benchmarks.reduce_micro --sizes 1024 1048576 67108864
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

import torch
import torch.distributed as dist

NVLINK_GBS = 770.0       # measured peer copy, per direction per GPU
HBM_GBS_FALLBACK = 6650.0


def hbm_gbs():
    path = os.path.join(os.path.dirname(__file__), "..", "..", "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return HBM_GBS_FALLBACK, "fallback"


METHODS = {
    "allreduce": ("NoneAllReducer", {}),
    "qsgd-mn-2": ("QSGDMaxNormReducer", {"quantization_level": 2}),
    "qsgd-mn-4": ("QSGDMaxNormReducer", {"quantization_level": 4}),
    "qsgd-mn-8": ("QSGDMaxNormReducer", {"quantization_level": 8}),
    "qsgd-mn-ts-2-6": ("QSGDMaxNormTwoScaleReducer", {"lower_quantization_level": 2, "higher_quantization_level": 6}),
    "grandk-mn-8": ("GlobalRandKMaxNormReducer", {"K": 10000, "quantization_level": 8, "seed": 1}),
    "grandk-mn-ts-2-6": ("GlobalRandKMaxNormTwoScaleReducer", {"K": 10000, "lower_quantization_level": 2,
                                                               "higher_quantization_level": 6, "seed": 1}),
    "topk-1pct": ("TopKReducerRatio", {"compression": 0.01}),
    "powersgd-r1": ("RankKReducer", {"rank": 1}),
    "powersgd-r2": ("RankKReducer", {"rank": 2}),
}


def roofline_seconds(method, n, world, hbm):
    """(time bound, NVLink bytes per GPU, HBM bytes per GPU) of the fused path for one step."""
    from .. import ops

    w = world
    frac = (w - 1) / w if w > 1 else 0.0
    if method == "allreduce":
        link = 2 * frac * 4 * n
        mem = (4 * n * 2) + (4 * n / max(w, 1)) * (w + w) + 4 * n * 2 if w > 1 else 8 * n
    elif method.startswith("qsgd-mn-ts"):
        mb, pb = ops.packed_sizes(n, 2)
        sumb = 1
        link = frac * (mb + pb) + frac * n * sumb + (w - 1) * pb
        mem = 4 * n * 3 + 2 * (mb + 3 * pb) + 2 * n * sumb + 4 * n
    elif method.startswith("qsgd-mn"):
        bits = int(method.rsplit("-", 1)[1])
        mb, pb = ops.packed_sizes(n, bits)
        s = (1 << bits) - 1
        sumb = 1 if s * w <= 127 else (2 if s * w <= 32767 else 4)
        link = frac * (mb + pb) + frac * n * sumb
        mem = 4 * n * 2 + 2 * (mb + pb) + 2 * n * sumb + 4 * n if w > 1 else 4 * n * 3
    elif method.startswith("grandk"):
        k = min(10000, n)
        link = (w - 1) * k * 5
        mem = 8 * n
    elif method.startswith("powersgd"):
        r = int(method[-1])
        side = int(n ** 0.5)
        link = (w - 1) * 4 * 2 * side * r
        mem = 4 * n * 3 + 4 * n + 4 * n * 3
    else:
        return None, None, None
    t = max(link / (NVLINK_GBS * 1e9), mem / (hbm * 1e9))
    return t, link, mem


def make_tensors(method, n, device, rank):
    g = torch.Generator(device=device).manual_seed(1234 + rank)
    if method.startswith("powersgd"):
        side = max(int(n ** 0.5), 1)       # a square matrix view plus its bias vector
        return [torch.randn(side, side, device=device, generator=g) * 1e-3,
                torch.randn(side, device=device, generator=g) * 1e-3]
    return [torch.randn(n, device=device, generator=g) * 1e-3]


def time_reducer(red, tensors, iters, warmup, flush, device, spin_cycles=1_500_000):
    outs = [torch.empty_like(t) for t in tensors]
    times = []
    for i in range(warmup + iters):
        send = [t.clone() for t in tensors]
        flush.add_(1.0)                      # rewrites 256 MB: nothing of the inputs is left in L2
        if dist.is_initialized():
            dist.barrier()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda._sleep(spin_cycles)       # the host runs ahead while the device spins: launch latency and
        s.record()                           # Python overhead of reduce() stay out of the device-timed interval
        red.reduce(send, outs)
        e.record()
        torch.cuda.synchronize()
        if i >= warmup:
            times.append(s.elapsed_time(e) * 1e-3)
    t = torch.tensor(times, dtype=torch.float64, device=device)
    if dist.is_initialized():
        dist.all_reduce(t, op=dist.ReduceOp.MAX)     # per-iteration max over ranks
    return statistics.median(t.tolist())


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes", type=int, nargs="+", default=[1 << 10, 1 << 14, 1 << 17, 1 << 20, 1 << 23, 1 << 26])
    ap.add_argument("--methods", nargs="+", default=list(METHODS))
    ap.add_argument("--impls", nargs="+", default=["fused", "dist", "reference"])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--out", default=None, help="write the rows as JSON lines to this file (rank 0)")
    args = ap.parse_args(argv)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29541")
    dist.init_process_group("nccl", rank=int(os.environ.get("RANK", "0")), world_size=world, device_id=device)
    rank = dist.get_rank()

    from .. import reducers as ours
    ref_mod = None
    if "reference" in args.impls:
        ref_dir = os.path.join(os.path.dirname(__file__), "..", "..", "baseline", "_ref")
        if os.path.exists(os.path.join(ref_dir, "reducer.py")):
            sys.path.insert(0, ref_dir)
            import reducer as ref_mod
            from timer import Timer as RefTimer

    hbm, hbm_src = hbm_gbs()
    flush = torch.zeros(64 << 20, device=device)
    rows = []
    for method in args.methods:
        cls_name, kw = METHODS[method]
        for n in args.sizes:
            tensors = make_tensors(method, n, device, rank)
            n_eff = sum(t.numel() for t in tensors)
            row = {"method": method, "n": n_eff, "world": world}
            for impl in args.impls:
                try:
                    if impl == "reference":
                        if ref_mod is None:
                            continue
                        if world == 1 and cls_name == "RankKReducer":
                            row["reference_us"] = None      # the reference's PowerSGD fails with one worker
                            continue
                        t = RefTimer(verbosity_level=0)
                        t.log_fn = lambda *a, **k: None
                        red = getattr(ref_mod, cls_name)(device, t, **kw)
                    else:
                        red = getattr(ours, cls_name)(device, None, backend=impl, **kw)
                        if impl == "fused" and not red.fused_capable:
                            continue
                    sec = time_reducer(red, tensors, args.iters, args.warmup, flush, device)
                    row[f"{impl}_us"] = sec * 1e6
                    row[f"{impl}_bus_gbs"] = (2 * (world - 1) / world * 4 * n_eff / sec / 1e9) if world > 1 else None
                    if impl == "fused":
                        tb, link, mem = roofline_seconds(method, n_eff, world, hbm)
                        if tb:
                            row["fused_roofline_frac"] = tb / sec
                            row["fused_link_bytes"], row["fused_hbm_bytes"] = link, mem
                except Exception as exc:     # keep the sweep going; the failure is part of the record
                    row[f"{impl}_error"] = repr(exc)[:200]
            rows.append(row)
            if rank == 0:
                print(json.dumps(row), flush=True)
    if rank == 0 and args.out:
        with open(args.out, "w") as f:
            f.write(json.dumps({"hbm_gbs": hbm, "hbm_source": hbm_src, "nvlink_gbs": NVLINK_GBS}) + "\n")
            for row in rows:
                f.write(json.dumps(row) + "\n")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
