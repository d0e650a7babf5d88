"""Per-kernel device time of one training step under CUDA-graph replay (torch profiler / CUPTI timeline, real
cache conditions -- unlike ncu, nothing is flushed or serialised).

    python -m gradient_compression_b200.benchmarks.step_profile --model ResNet50 [--eager-ops]
"""
import argparse
import collections
import re

import torch


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="ResNet50")
    ap.add_argument("--reducer", default="QSGDMaxNormReducer")
    ap.add_argument("--batch", type=int, default=128)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--norm-scope", default="global", choices=["global", "bucket"],
                    help="bucket: per-bucket reduces on a side stream beside backward")
    ap.add_argument("--bucket-mb", type=float, default=25.0)
    ap.add_argument("--timeline", type=int, default=0,
                    help="also print, with their start times inside the last step, its first N kernels and every reducer / optimiser kernel")
    ap.add_argument("--eager-ops", action="store_true",
                    help="run the step eagerly and list the torch operators by device time (which op launches which kernels)")
    args = ap.parse_args(argv)

    from .. import make_reducer
    from ..parallel import FlatSGD
    from ..parallel.graph import GraphedStep
    from ..train import CIFAR
    from torch.profiler import ProfilerActivity, profile

    torch.backends.cudnn.benchmark = True
    dev = torch.device("cuda:0")
    task = CIFAR(dev, None, args.model, seed=0, data="synthetic", synthetic_train_size=2 * args.batch,
                 synthetic_test_size=args.batch)
    opt = FlatSGD(task.arena, lr=0.1)
    if args.norm_scope == "bucket":
        from ..parallel.bucketed import BucketedReducer
        red = BucketedReducer(task.parameters, args.reducer, dev, None, {"quantization_level": 8, "seed": 1}, bucket_mb=args.bucket_mb)
    else:
        red = make_reducer(args.reducer, dev, None, {"quantization_level": 8, "seed": 1})
    step = GraphedStep(task, red, opt, enabled=not args.eager_ops)
    x = torch.randn(args.batch, 3, 32, 32, device=dev).contiguous(memory_format=torch.channels_last)
    y = torch.randint(0, 10, (args.batch,), device=dev)
    for _ in range(8):
        step((x, y))
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
        for _ in range(args.steps):
            step((x, y))
        torch.cuda.synchronize()
    if args.eager_ops:
        rows = [(e.key, e.count // args.steps, e.self_device_time_total / args.steps) for e in prof.key_averages()
                if e.self_device_time_total > 0]
        for key, cnt, t in sorted(rows, key=lambda r: -r[2])[:40]:
            print(f"{t:9.1f} us {cnt:4d}  {key[:90]}")
        return
    agg = collections.defaultdict(lambda: [0, 0.0])
    for ev in prof.events():
        if ev.device_type == torch.autograd.DeviceType.CUDA:
            name = re.sub(r"<.*", "", ev.name)[:80]
            agg[name][0] += 1
            agg[name][1] += ev.device_time
    total = sum(v[1] for v in agg.values())
    print(f"graphed: {step.graphed}; device time per step: {total / args.steps:.1f} us")
    for name, (cnt, t) in sorted(agg.items(), key=lambda kv: -kv[1][1])[:40]:
        print(f"{t / args.steps:9.1f} us {cnt // args.steps:4d}  {name}")
    if args.timeline:
        evs = sorted((ev for ev in prof.events() if ev.device_type == torch.autograd.DeviceType.CUDA),
                     key=lambda e: e.time_range.start)
        per_step = len(evs) // args.steps
        one = evs[-per_step:]
        t0 = one[0].time_range.start
        print(f"timeline of the last step ({per_step} kernels): start us, duration us, name")
        picked = [e for e in one if "fused" in e.name or "sgd" in e.name or "multi_tensor" in e.name]
        picked = sorted(set(picked + one[: args.timeline]), key=lambda e: e.time_range.start)
        for e in picked:
            print(f"{e.time_range.start - t0:10.1f} {e.device_time:8.1f}  {e.name[:70]}")
        print(f"{one[-1].time_range.end - t0:10.1f} end of step")


if __name__ == "__main__":
    main()
