#!/usr/bin/env python
"""Headline benchmark: training throughput (images/s, whole job) of the CIFAR ResNet-50 with the
QSGD-MaxNorm 8-bit reducer at batch 128 per GPU on N GPUs of one node, synthetic data.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 20 --warmup 5
    python bench.py --impl reference ...        # the unmodified reference from baseline/_ref

Two measurements per run, both the max over ranks:
* ``value``  -- K steps timed with CUDA events on the launching stream, batches already on the device;
* ``e2e``    -- K steps through the public API (loader -> pinned host batch -> H2D -> forward/backward ->
                reduce -> optimiser step -> loss read back to the host), wall clock between device syncs.
Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.abspath(__file__))
# published reference figure for this config: ResNet-50, QSGD-MaxNorm 8 bit, 2 GPUs, 905 img/s
# (logs/2021_05_20_08_16_00_ResNet50/timer_summary_0.json) -> per GPU, scaled weakly to N
PUBLISHED_IMG_S_PER_GPU = {("ResNet50", "QSGDMaxNormReducer", 8): 905.0 / 2, ("ResNet50", "NoneAllReducer", 0): 959.0 / 2,
                           ("VGG16", "QSGDMaxNormReducer", 8): 3777.0 / 2, ("VGG16", "NoneAllReducer", 0): 4220.0 / 2}


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=20)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--model", default="ResNet50")
    p.add_argument("--reducer", default="QSGDMaxNormReducer")
    p.add_argument("--bits", type=int, default=8)
    p.add_argument("--higher-bits", type=int, default=10)
    p.add_argument("--K", type=int, default=10000)
    p.add_argument("--rank", type=int, default=1)
    p.add_argument("--batch", type=int, default=128)
    p.add_argument("--backend", default="auto", choices=["auto", "fused", "dist"])
    p.add_argument("--graph", type=int, default=1, help="capture the training step in a CUDA graph (ours)")
    p.add_argument("--channels-last", type=int, default=1)
    p.add_argument("--cudnn-benchmark", type=int, default=1, help="let cuDNN autotune its convolution algorithms (ours)")
    p.add_argument("--cudnn-benchmark-limit", type=int, default=-1, help="algorithms cuDNN's autotuner tries (0 = all; -1 = torch default)")
    p.add_argument("--norm-scope", default="global", choices=["global", "bucket"],
                   help="global: one reduce after backward with one max-norm (the reference); bucket: per-bucket reduces "
                        "on a side stream while backward runs, each with its own max-norm (ours)")
    p.add_argument("--bucket-mb", type=float, default=25.0)
    p.add_argument("--reduce-max-blocks", type=int, default=32, help="grid cap of a fused reduce that overlaps backward (ours)")
    p.add_argument("--sustained-seconds", type=float, default=3.0, help="0 = skip the sustained measurement")
    p.add_argument("--no-e2e", action="store_true")
    return p.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index):
        self.idx = device_index
        self.proc = None
        self.lines = []
        self.first = 0

    def wait_ready(self, timeout=3.0):
        """Returns once nvidia-smi has printed its first sample (its start-up takes a few hundred milliseconds)."""
        t0 = time.perf_counter()
        while self.proc is not None and not self.lines and time.perf_counter() - t0 < timeout:
            time.sleep(0.01)

    def mark(self):
        """The timed region starts here: samples taken before (the sampler is started ahead of the warm-up steps, so that the
        process is up and printing when the clock starts) are not counted, unless the region is too short to catch one."""
        self.first = len(self.lines)

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", str(self.idx)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        lines = self.lines[self.first:] or self.lines[-1:]        # a region shorter than the 50 ms period: the sample just before it
        for line in lines:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 8:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
                power.append(float(parts[3]))
            except ValueError:
                continue
            for name, val in zip(names, parts[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def setup_dist(n):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local_rank)
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        return world, dist.get_rank(), local_rank
    if n > 1:
        raise SystemExit("launch with torch.distributed.run for --gpus > 1")
    torch.cuda.set_device(0)
    return 1, 0, 0


def max_over_ranks(x, device):
    if dist.is_initialized():
        t = torch.tensor([x], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())
    return x


def barrier_sync():
    if dist.is_initialized():
        dist.barrier()
    torch.cuda.synchronize()


def measure_sustained(one_step, args, world, rank, local_rank, device):
    """The same timed region (``args.steps`` steps between CUDA events) repeated until the GPU has been under load for
    ``args.sustained_seconds``: the median block says what a step costs once clocks have settled under the power cap.
    ``value`` / ``steps`` of the bench line stay the K-step burst; this is reported beside them."""
    if args.sustained_seconds <= 0:
        return None
    barrier_sync()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    per_block, t_begin = [], time.perf_counter()
    while True:
        s_ev, e_ev = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s_ev.record()
        for i in range(args.steps):
            one_step(i)
        e_ev.record()
        e_ev.synchronize()
        per_block.append(s_ev.elapsed_time(e_ev) / args.steps)
        more = torch.tensor([1.0 if time.perf_counter() - t_begin < args.sustained_seconds else 0.0], device=device)
        if dist.is_initialized():
            dist.all_reduce(more, op=dist.ReduceOp.MAX)      # every rank runs the same number of blocks
        if float(more.item()) == 0.0:
            break
    seconds = time.perf_counter() - t_begin
    barrier_sync()
    clocks = sampler.stop() if rank == 0 else None
    med = max_over_ranks(statistics.median(per_block), device)
    out = {"ms_per_step": med, "value": args.batch * world / (med * 1e-3), "unit": "images/s", "blocks": len(per_block),
           "steps_per_block": args.steps, "seconds": max_over_ranks(seconds, device)}
    if clocks is not None:
        out["clocks"] = clocks
        if clocks.get("sm_mhz"):
            out["ms_times_sm_mhz"] = med * clocks["sm_mhz"]
    return out


def reducer_config(args):
    return dict(quantization_level=args.bits, higher_quantization_level=args.higher_bits, K=args.K, rank=args.rank,
                seed=42, backend=args.backend, compression=0.01, quantization_levels=[args.bits, args.higher_bits])


# ------------------------------------------------------------------------------------------ ours
def run_ours(args, world, rank, local_rank):
    sys.path.insert(0, ROOT)
    from gradient_compression_b200 import make_reducer, ops
    from gradient_compression_b200.parallel import FlatSGD
    from gradient_compression_b200.parallel.graph import GraphedStep
    from gradient_compression_b200.train import CIFAR
    from gradient_compression_b200.utils import set_seed

    device = torch.device("cuda", local_rank)
    set_seed(42)
    torch.backends.cudnn.benchmark = bool(args.cudnn_benchmark)
    if args.cudnn_benchmark_limit >= 0:
        torch.backends.cudnn.benchmark_limit = args.cudnn_benchmark_limit
    steps_needed = args.steps + args.warmup + 10
    task = CIFAR(device, None, args.model, seed=42, data="synthetic",
                 synthetic_train_size=args.batch * world * steps_needed, synthetic_test_size=args.batch,
                 broadcast_parameters=True, channels_last=bool(args.channels_last))
    opt = FlatSGD(task.arena, lr=0.1, momentum=0.9, weight_decay=5e-4, nesterov=True)
    if args.norm_scope == "bucket":
        from gradient_compression_b200.parallel.bucketed import BucketedReducer
        reducer = BucketedReducer(task.parameters, args.reducer, device, None, reducer_config(args), bucket_mb=args.bucket_mb,
                                  max_blocks=args.reduce_max_blocks)
    else:
        reducer = make_reducer(args.reducer, device, None, reducer_config(args))
    # the step evaluates cross-entropy, top-1 and top-5 of the batch on the device, as the reference's step does
    step_fn = GraphedStep(task, reducer, opt, enabled=bool(args.graph))

    # device-resident batches for the device-timed loop
    gen = torch.Generator(device=device).manual_seed(1234 + rank)
    dev_batches = []
    for _ in range(4):
        x = torch.randn(args.batch, 3, 32, 32, device=device, generator=gen)
        if args.channels_last:
            x = x.contiguous(memory_format=torch.channels_last)
        dev_batches.append((x, torch.randint(0, 10, (args.batch,), device=device, generator=gen)))

    # set-up, not part of the measurement: cuDNN autotuning, arena mapping and the graph capture happen in the
    # first calls of the step function; run them before the W official warm-up steps
    for i in range(6 if args.graph else 2):
        step_fn(dev_batches[i % 4])
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        sampler.wait_ready()
    for i in range(args.warmup):
        step_fn(dev_batches[i % 4])
    barrier_sync()
    sampler.mark()
    launches0 = ops.launches()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(args.steps):
        loss = step_fn(dev_batches[i % 4])
    end.record()
    barrier_sync()
    dev_ms = max_over_ranks(start.elapsed_time(end), device) / args.steps
    launches = (ops.launches() - launches0) if not step_fn.graphed else step_fn.kernels_per_step * args.steps
    clocks = sampler.stop() if rank == 0 else None
    assert torch.isfinite(loss).all(), "loss is not finite"

    sustained = measure_sustained(lambda i: step_fn(dev_batches[i % 4]), args, world, rank, local_rank, device)

    e2e = None
    if not args.no_e2e:
        from gradient_compression_b200.train.data import LaggedReadback
        loader = task.train_dataloader(args.batch)        # pinned host batches; the copy of the next ones runs on a side stream
        it = iter(loader)
        reader = LaggedReadback(device, lag=1)
        for _ in range(2):
            float(step_fn(next(it)).item())
        barrier_sync()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            batch = next(it)                      # host -> device copy of this step's inputs (issued one step ahead)
            step_fn(batch)
            v = reader.push(step_fn.metrics_vec)  # device -> host read of this step's loss / top-1 / top-5, collected one step later
            if v is not None:
                loss_host = v[0]
        loss_host = reader.drain()[-1][0]         # the last step's result is read before the clock stops
        barrier_sync()
        e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3, device) / args.steps
        e2e = {"value": args.batch * world / (e2e_ms * 1e-3), "unit": "images/s", "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": args.batch * 3 * 32 * 32 * 4 + args.batch * 8, "d2h_bytes_per_step": 12,
               "last_loss": loss_host,
               "pipelining": "every step copies one batch host->device (issued two steps ahead on a side stream) and reads its "
                             "cross-entropy, top-1 and top-5 device->host (collected one step late); the last step's are read "
                             "before the clock stops"}
    from gradient_compression_b200.ops import conv as conv_ops
    conv_path = ("own tcgen05 TF32 kernels (paths: %s; >= %d output positions) with BN statistics in the epilogue: forward, "
                 "input gradient (stride 1) and weight gradient; input gradients of strided convolutions: cuDNN"
                 % (",".join(sorted(conv_ops.PATHS)), conv_ops.MIN_ROWS)) if conv_ops.ENABLED \
        else "cuDNN (torch); own tcgen05 paths off (GCB200_TC_CONV=0)"
    first = reducer.reducers[0] if hasattr(reducer, "reducers") else reducer
    extra = {"graph": step_fn.graphed, "backend": getattr(first, "backend", "auto"), "norm_scope": args.norm_scope,
             "buckets": len(reducer.buckets) if hasattr(reducer, "buckets") else 1,
             "fused": bool(getattr(first, "_fused", None)), "channels_last": bool(args.channels_last), "cudnn_benchmark": bool(args.cudnn_benchmark),
             "conv_path": conv_path, "wire_bits_per_step": getattr(first, "last_wire_bits", None),
             "step_evaluates": "cross-entropy, top-1, top-5 on the device (as the reference's step)",
             "capture_error": step_fn.capture_error}
    return dev_ms, launches, clocks, e2e, extra, sustained


# ------------------------------------------------------------------------------------------ reference
def run_reference(args, world, rank, local_rank):
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.exists(os.path.join(ref_dir, "reducer.py")):
        return {"impl": "reference", "unavailable": "baseline/_ref is not installed"}
    sys.path.insert(0, ref_dir)
    import torchvision

    n_items = args.batch * world * (args.steps + args.warmup + 6)

    class SyntheticCIFAR10(torch.utils.data.Dataset):
        """Stands in for the CIFAR-10 download: fp32 N(0,1) images, uniform labels (no network here)."""

        def __init__(self, root=None, train=True, download=False, transform=None):
            g = torch.Generator().manual_seed(1 if train else 2)
            n = n_items if train else args.batch * world * 2
            self.x = torch.randn(n, 3, 32, 32, generator=g)
            self.y = torch.randint(0, 10, (n,), generator=g)

        def __len__(self):
            return self.x.shape[0]

        def __getitem__(self, i):
            return self.x[i], int(self.y[i])

    torchvision.datasets.CIFAR10 = SyntheticCIFAR10
    if not dist.is_initialized():      # the reference's reducers query the world size unconditionally
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", local_rank))
    import reducer as ref_reducer
    from model_dispatcher import CIFAR as RefCIFAR
    from seed import set_seed as ref_set_seed
    from timer import Timer as RefTimer

    device = torch.device(f"cuda:{local_rank}")
    ref_set_seed(42)
    timer = RefTimer(verbosity_level=2)
    timer.log_fn = lambda *a, **k: None
    cls = getattr(ref_reducer, args.reducer)
    if args.reducer in ("NoneAllReducer", "NoneReducer"):
        red = cls(device, timer)
    elif args.reducer == "GlobalRandKMaxNormReducer":
        red = cls(device, timer, K=args.K, quantization_level=args.bits, seed=42)
    elif args.reducer == "QSGDMaxNormTwoScaleReducer":
        red = cls(device, timer, lower_quantization_level=args.bits, higher_quantization_level=args.higher_bits)
    elif args.reducer == "GlobalRandKMaxNormTwoScaleReducer":
        red = cls(device, timer, lower_quantization_level=args.bits, higher_quantization_level=args.higher_bits, seed=42)
    elif args.reducer == "RankKReducer":
        red = cls(device, timer, rank=args.rank)
    elif args.reducer in ("TopKReducer", "GlobalTopKReducer"):
        red = cls(device, timer, K=args.K)
    elif args.reducer in ("TopKReducerRatio", "GlobalTopKReducerRatio"):
        red = cls(device, timer)                 # compression 1 / 100, the reference's default (reducer.py:1234)
    else:
        red = cls(device, timer, quantization_level=args.bits)
    model = RefCIFAR(device, timer, args.model, 42 + local_rank)
    send_buffers = [torch.zeros_like(p) for p in model.parameters]
    optimizer = torch.optim.SGD(params=model.parameters, lr=0.1, momentum=0.9, weight_decay=5e-4, nesterov=True)

    def ref_step(batch):   # the body of the reference's hot loop (trainer.py:183-196), its objects only
        with timer("batch", 0.0):
            _, grads, metrics = model.batch_loss_with_gradients(batch)
            with timer("batch.accumulate", 0.0, verbosity=2):
                for grad, send_buffer in zip(grads, send_buffers):
                    send_buffer[:] = grad
            with timer("batch.reduce", 0.0):
                red.reduce(send_buffers, grads)
            with timer("batch.step", 0.0, verbosity=2):
                optimizer.step()
        return metrics

    gen = torch.Generator(device=device).manual_seed(1234 + rank)
    dev_batches = [(torch.randn(args.batch, 3, 32, 32, device=device, generator=gen),
                    torch.randint(0, 10, (args.batch,), device=device, generator=gen)) for _ in range(4)]
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        sampler.wait_ready()
    for i in range(args.warmup):
        ref_step(dev_batches[i % 4])
    barrier_sync()
    sampler.mark()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(args.steps):
        ref_step(dev_batches[i % 4])
    end.record()
    barrier_sync()
    dev_ms = max_over_ranks(start.elapsed_time(end), device) / args.steps
    clocks = sampler.stop() if rank == 0 else None
    sustained = measure_sustained(lambda i: ref_step(dev_batches[i % 4]), args, world, rank, local_rank, device)

    e2e = None
    if not args.no_e2e:
        it = iter(model.train_dataloader(args.batch))   # the reference's own DataLoader (pinned) + .to(device)
        for _ in range(2):
            ref_step(next(it))
        barrier_sync()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            metrics = ref_step(next(it))                # its step reads loss / top-1 / top-5 back with .item()
        barrier_sync()
        e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3, device) / args.steps
        e2e = {"value": args.batch * world / (e2e_ms * 1e-3), "unit": "images/s", "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": args.batch * 3 * 32 * 32 * 4 + args.batch * 8, "d2h_bytes_per_step": 12,
               "last_loss": metrics["cross_entropy_loss"]}
    extra = {"reduce_ms": timer.totals.get("batch.reduce", 0.0) / max(timer.call_counts.get("batch.reduce", 1), 1) * 1e3,
             "cudnn_allow_tf32": torch.backends.cudnn.allow_tf32, "matmul_allow_tf32": torch.backends.cuda.matmul.allow_tf32}
    return dev_ms, 0, clocks, e2e, extra, sustained


def main():
    args = parse_args()
    # libraries (NCCL's version banner) write to stdout; keep fd 1 clean for the one JSON line
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    def emit(obj):
        sys.stdout.flush()
        os.write(real_stdout, (json.dumps(obj) + "\n").encode())

    if not torch.cuda.is_available():
        if args.impl == "reference":
            emit({"impl": "reference", "unavailable": "no CUDA device in this process"})
            return
        raise SystemExit("bench.py needs a CUDA device")
    world, rank, local_rank = setup_dist(args.gpus)
    try:
        out = (run_ours if args.impl == "ours" else run_reference)(args, world, rank, local_rank)
    except Exception as exc:
        if args.impl != "reference":
            raise
        # a failure inside the reference's own code (e.g. its PowerSGD reducer with one worker) is reported,
        # not hidden: the arm is unavailable for this configuration
        out = {"impl": "reference", "unavailable": f"the reference's code raised {type(exc).__name__}: {str(exc)[:160]}"}
    if isinstance(out, dict):
        if rank == 0:
            emit(out)
        return
    sustained = None
    if len(out) == 6:
        dev_ms, launches, clocks, e2e, extra, sustained = out
    else:
        dev_ms, launches, clocks, e2e, extra = out
    if rank == 0:
        value = args.batch * world / (dev_ms * 1e-3)
        key = (args.model, args.reducer, args.bits if "QSGD" in args.reducer else 0)
        base = PUBLISHED_IMG_S_PER_GPU.get(key)
        line = {
            "metric": "training images/sec (whole job, device-timed, max over ranks)", "value": value,
            "unit": "images/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": (value / (base * world)) if base else None,
            "dtype": "fp32 params/activations, TF32 tensor cores in convolutions (torch default, as the reference)",
            "data": "synthetic 3x32x32 N(0,1) inputs, uniform labels, random-init weights",
            "impl": args.impl,
            "config": {"model": f"{args.model} (CIFAR variant)", "global_batch": args.batch * world, "seq_len": None,
                       "batch_per_gpu": args.batch, "parallelism": f"dp{world}", "reducer": args.reducer,
                       "quantization_level": args.bits, "optimizer": "SGD lr 0.1 momentum 0.9 nesterov wd 5e-4",
                       "l2": "step working set (activations + 94 MB gradient + parameters) far exceeds the 126 MB L2",
                       "published_baseline": "reference logs, 2 GPUs of unnamed hardware, scaled per GPU", **extra},
            "clocks": clocks, "e2e": e2e, "sustained": sustained, "gpu_launches": launches,
        }
        emit(line)
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
