"""Both arms of ``bench.py`` back to back on one box over the benchmark configurations: CIFAR ResNet-50 and VGG-16 at
batch 128 per GPU under the reference's reducers, the reference arm (``--impl reference``: the unmodified reference from
``baseline/_ref``) right before this library's arm for every row.

    python -m gradient_compression_b200.benchmarks.sweep --gpus 8 --group resnet vgg powersgd \
        --out profiles/bench_matrix_8gpu            # writes <out>.md and <out>.json

Every row is one ``bench.py`` process group per arm (``torch.distributed.run`` for more than one GPU); the numbers are
bench.py's own (CUDA events, max over ranks).  ``exposed reduce`` is this library's step time minus the same step at
one GPU when ``--one-gpu-json`` names an earlier sweep at one GPU (weak scaling: the difference is what communication
and compression add on the critical path).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

# name -> (model, reducer, extra bench.py flags, label)
ROWS = {
    "resnet": [("ResNet50", "NoneAllReducer", [], "AllReduce-SGD"),
               ("ResNet50", "QSGDMaxNormReducer", ["--bits", "8"], "QSGD-MN 8 bit"),
               ("ResNet50", "QSGDMaxNormReducer", ["--bits", "4"], "QSGD-MN 4 bit"),
               ("ResNet50", "QSGDMaxNormReducer", ["--bits", "2"], "QSGD-MN 2 bit"),
               ("ResNet50", "QSGDMaxNormTwoScaleReducer", ["--bits", "2", "--higher-bits", "6"], "QSGD-MN-TS (2, 6)")],
    "vgg": [("VGG16", "GlobalRandKMaxNormReducer", ["--bits", "8", "--K", "10000"], "GRandK-MN 8 bit K=10000"),
            ("VGG16", "GlobalRandKMaxNormTwoScaleReducer", ["--bits", "2", "--higher-bits", "6", "--K", "10000"],
             "GRandK-MN-TS (2, 6) K=10000"),
            ("VGG16", "QSGDMaxNormReducer", ["--bits", "8"], "QSGD-MN 8 bit")],
    "powersgd": [("ResNet50", "RankKReducer", ["--rank", "1"], "PowerSGD rank 1"),
                 ("ResNet50", "RankKReducer", ["--rank", "2"], "PowerSGD rank 2"),
                 ("VGG16", "RankKReducer", ["--rank", "1"], "PowerSGD rank 1"),
                 ("VGG16", "RankKReducer", ["--rank", "2"], "PowerSGD rank 2")],
    "topk": [("ResNet50", "TopKReducerRatio", [], "TopK 1 %")],
}


def run_bench(gpus, model, reducer, flags, impl, steps, warmup, port, timeout, extra):
    cmd = [sys.executable]
    if gpus > 1:
        cmd += ["-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(gpus), "--master-addr", "127.0.0.1",
                "--master-port", str(port)]
    cmd += [os.path.join(ROOT, "bench.py"), "--gpus", str(gpus), "--steps", str(steps), "--warmup", str(warmup), "--model", model,
            "--reducer", reducer, "--impl", impl] + list(flags) + list(extra)
    t0 = time.time()
    try:
        out = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, cwd=ROOT)
    except subprocess.TimeoutExpired:
        return {"impl": impl, "unavailable": f"no result within {timeout} s"}
    line = None
    for cand in reversed(out.stdout.strip().splitlines()):
        if cand.startswith("{"):
            line = cand
            break
    if line is None:
        return {"impl": impl, "unavailable": f"exit code {out.returncode}: {out.stderr.strip().splitlines()[-1][:200] if out.stderr.strip() else 'no output'}"}
    rec = json.loads(line)
    rec["wall_s"] = round(time.time() - t0, 1)
    return rec


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--group", nargs="+", default=["resnet", "vgg", "powersgd"], choices=sorted(ROWS))
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--timeout", type=int, default=600)
    ap.add_argument("--arms", nargs="+", default=["reference", "ours"], choices=["reference", "ours"])
    ap.add_argument("--e2e", action="store_true", help="also take bench.py's end-to-end measurement (slower)")
    ap.add_argument("--sustained-seconds", type=float, default=0.0)
    ap.add_argument("--one-gpu-json", default=None, help="an earlier sweep at one GPU: adds the exposed reduce time per row")
    ap.add_argument("--only", nargs="+", default=None, help="keep the rows whose label contains one of these strings")
    ap.add_argument("--out", default=os.path.join(ROOT, "profiles", "bench_matrix"))
    args = ap.parse_args(argv)
    extra = ["--sustained-seconds", str(args.sustained_seconds)] + ([] if args.e2e else ["--no-e2e"])
    base = {}
    if args.one_gpu_json and os.path.exists(args.one_gpu_json):
        with open(args.one_gpu_json) as f:
            for r in json.load(f)["rows"]:
                if "ours" in r and "ms_per_step" in r["ours"]:
                    base[(r["model"], r["label"])] = r["ours"]["ms_per_step"]
    rows, port = [], 29600
    for group in args.group:
        for model, reducer, flags, label in ROWS[group]:
            if args.only and not any(o in label for o in args.only):
                continue
            row = {"group": group, "model": model, "reducer": reducer, "label": label, "gpus": args.gpus}
            for impl in args.arms:                       # the reference first, this library right after it
                port += 1
                rec = run_bench(args.gpus, model, reducer, flags, impl, args.steps, args.warmup, port, args.timeout, extra)
                row[impl] = {k: rec.get(k) for k in ("ms_per_step", "value", "unavailable", "clocks", "e2e", "sustained", "wall_s")
                             if rec.get(k) is not None}
                print(json.dumps({"row": label, "model": model, "impl": impl, **row[impl]}), flush=True)
            if "ms_per_step" in row.get("ours", {}) and "ms_per_step" in row.get("reference", {}):
                row["ratio"] = row["reference"]["ms_per_step"] / row["ours"]["ms_per_step"]
            if (model, label) in base and "ms_per_step" in row.get("ours", {}):
                row["exposed_reduce_ms"] = row["ours"]["ms_per_step"] - base[(model, label)]
            rows.append(row)
    os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
    with open(args.out + ".json", "w") as f:
        json.dump({"gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "rows": rows}, f, indent=1)
    with open(args.out + ".md", "w") as f:
        f.write(f"# Training throughput, both arms on one box: {args.gpus} x B200, batch 128 per GPU, synthetic data\n\n")
        f.write("command: `python -m gradient_compression_b200.benchmarks.sweep " + " ".join(sys.argv[1:] if argv is None else argv) + "`\n\n")
        f.write("Each row: `bench.py --impl reference` (the unmodified reference, torch ops + NCCL) and then `bench.py` (this library) with "
                f"the same model, reducer and batch; {args.steps} timed steps after {args.warmup} warm-up steps, CUDA events, max over ranks.\n\n")
        f.write("| model | reducer | reference ms/step | reference img/s | this library ms/step | this library img/s | ratio | exposed reduce ms |\n")
        f.write("|---|---|---|---|---|---|---|---|\n")
        for r in rows:
            ref, ours = r.get("reference", {}), r.get("ours", {})

            def cell(d, k, fmt):
                return fmt.format(d[k]) if k in d else ("n/a: " + d.get("unavailable", "not run")[:60] if k == "ms_per_step" else "")
            f.write(f"| {r['model']} | {r['label']} | {cell(ref, 'ms_per_step', '{:.2f}')} | {cell(ref, 'value', '{:.0f}')} | "
                    f"{cell(ours, 'ms_per_step', '{:.2f}')} | {cell(ours, 'value', '{:.0f}')} | "
                    f"{('%.2fx' % r['ratio']) if 'ratio' in r else ''} | "
                    f"{('%.3f' % r['exposed_reduce_ms']) if 'exposed_reduce_ms' in r else ''} |\n")
        throttled = [r["label"] for r in rows for arm in ("reference", "ours")
                     if any(x in (r.get(arm, {}).get("clocks") or {}).get("reasons", []) for x in ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown"))]
        f.write("\nClock records: " + ("slow-down reasons seen in " + ", ".join(throttled) if throttled else
                                        "no hw_slowdown / thermal slow-down reason in any run") + ".\n")
    print(f"wrote {args.out}.md and {args.out}.json")


if __name__ == "__main__":
    main()
