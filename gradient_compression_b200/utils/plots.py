"""Offline analysis: convergence curves, time breakdowns, scalability bars and the analytic
performance model (reference: utils.py:42-1001, which drives matplotlib and calls ``plt.show()``).

Headless by design: figures are written as SVG files, never shown.  matplotlib (Agg backend) is used
when importable; otherwise a small built-in SVG writer draws the same line and bar charts, so the
analysis works on machines without any plotting stack.

Inputs are the Logger's artefacts: ``success.txt`` (config + results), ``log_dict.npy`` (per-[run, epoch]
metrics) and ``timer_summary_<rank>.json`` (or the legacy single-GPU ``timer_summary.json``).
"""
from __future__ import annotations

import glob
import json
import math
import os

import numpy as np

# labels of the reduce-phase breakdown, in drawing order (reference: utils.py:539-547)
TIME_LABELS = ["batch.forward", "batch.backward", "batch.evaluate", "batch.accumulate", "batch.reduce", "batch.step"]
MODEL_SIZE_MB = {"ResNet50": 89.72, "VGG16": 56.18}          # fp32 gradient sizes (23 520 842 / 14 728 266 params)
MODEL_PARAMS = {"ResNet50": 23520842, "VGG16": 14728266}


# ------------------------------------------------------------------------------------------ parsing
def parse_success(path):
    """``success.txt`` -> dict of the config keys plus best accuracies and total bits."""
    out = {}
    with open(path) as f:
        for line in f:
            line = line.strip()
            if line.startswith("Best Top 1 Accuracy:"):
                out["best_top1"] = float(line.split(":")[1])
            elif line.startswith("Best Top 5 Accuracy:"):
                out["best_top5"] = float(line.split(":")[1])
            elif line.startswith("Bits communicated:"):
                out["bits"] = float(line.split(":")[1])
            elif " : " in line:
                k, v = line.split(" : ", 1)
                out[k.strip()] = v.strip()
    return out


def run_label(cfg):
    """Legend label of a run from its config, in the paper's vocabulary."""
    red = cfg.get("reducer", "?")
    q, hq, k, r = cfg.get("quantization_level"), cfg.get("higher_quantization_level"), cfg.get("K"), cfg.get("rank")
    names = {"NoneAllReducer": "AllReduce-SGD", "QSGDMaxNormReducer": f"QSGD-MN-{q}",
             "GlobalRandKMaxNormReducer": f"GRandK-MN-{q} (K={k})",
             "QSGDMaxNormTwoScaleReducer": f"QSGD-MN-TS-({q},{hq})",
             "GlobalRandKMaxNormTwoScaleReducer": f"GRandK-MN-TS-({q},{hq}) (K={k})",
             "QSGDMaxNormMultiScaleReducer": f"QSGD-MN-MS-{cfg.get('quantization_levels')}",
             "RankKReducer": f"PowerSGD rank {r}", "TopKReducer": f"TopK (K={k})",
             "TopKReducerRatio": f"TopK ({cfg.get('compression')})", "GlobalTopKReducer": f"GlobalTopK (K={k})"}
    return names.get(red, red)


def load_run(log_dir):
    run = {"dir": log_dir, "config": {}, "log": None, "timers": {}}
    sp = os.path.join(log_dir, "success.txt")
    if os.path.exists(sp):
        run["config"] = parse_success(sp)
    lp = os.path.join(log_dir, "log_dict.npy")
    if os.path.exists(lp):
        run["log"] = np.load(lp, allow_pickle=True).item()
    for tp in sorted(glob.glob(os.path.join(log_dir, "timer_summary*.json"))):
        with open(tp) as f:
            run["timers"][os.path.basename(tp)] = json.load(f)
    run["label"] = run_label(run["config"]) if run["config"] else os.path.basename(log_dir)
    return run


def load_runs(root):
    return [load_run(d) for d in sorted(glob.glob(os.path.join(root, "*"))) if os.path.isdir(d)]


def rank0_timer(run):
    for name in ("timer_summary_0.json", "timer_summary.json"):
        if name in run["timers"]:
            return run["timers"][name]
    return next(iter(run["timers"].values()), {})


# ------------------------------------------------------------------------------------------ drawing
_PALETTE = ["#1f77b4", "#ff7f0e", "#2ca02c", "#d62728", "#9467bd", "#8c564b", "#e377c2", "#7f7f7f", "#bcbd22", "#17becf"]


def _have_matplotlib():
    try:
        import matplotlib
        matplotlib.use("Agg")
        return True
    except Exception:
        return False


def _svg_frame(title, xlabel, ylabel, w=720, h=440):
    head = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{w}" height="{h}" viewBox="0 0 {w} {h}" font-family="sans-serif" font-size="12">',
            f'<rect width="{w}" height="{h}" fill="white"/>',
            f'<text x="{w / 2}" y="20" text-anchor="middle" font-size="14">{title}</text>',
            f'<text x="{w / 2}" y="{h - 8}" text-anchor="middle">{xlabel}</text>',
            f'<text x="14" y="{h / 2}" text-anchor="middle" transform="rotate(-90 14 {h / 2})">{ylabel}</text>']
    return head, (60, 30, w - 200, h - 75)     # plot box: x0, y0, width, height


def _ticks(lo, hi, n=5):
    if hi <= lo:
        hi = lo + 1.0
    step = 10 ** math.floor(math.log10((hi - lo) / n))
    for m in (1, 2, 5, 10):
        if (hi - lo) / (step * m) <= n:
            step *= m
            break
    t = math.ceil(lo / step) * step
    out = []
    while t <= hi + 1e-12:
        out.append(t)
        t += step
    return out


def line_chart(path, series, title="", xlabel="", ylabel=""):
    """series: list of (label, xs, ys)."""
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    if _have_matplotlib():
        import matplotlib.pyplot as plt
        fig, ax = plt.subplots(figsize=(8, 5))
        for label, xs, ys in series:
            ax.plot(xs, ys, label=label)
        ax.set(title=title, xlabel=xlabel, ylabel=ylabel)
        ax.grid(True, alpha=0.3)
        ax.legend(fontsize=8)
        fig.savefig(path, format="svg", bbox_inches="tight")
        plt.close(fig)
        return path
    head, (x0, y0, pw, ph) = _svg_frame(title, xlabel, ylabel)
    allx = [x for _, xs, _ in series for x in xs] or [0, 1]
    ally = [y for _, _, ys in series for y in ys if np.isfinite(y)] or [0, 1]
    xlo, xhi, ylo, yhi = min(allx), max(allx), min(ally), max(ally)
    xhi = xhi if xhi > xlo else xlo + 1
    yhi = yhi if yhi > ylo else ylo + 1
    sx = lambda x: x0 + (x - xlo) / (xhi - xlo) * pw
    sy = lambda y: y0 + ph - (y - ylo) / (yhi - ylo) * ph
    body = [f'<rect x="{x0}" y="{y0}" width="{pw}" height="{ph}" fill="none" stroke="#444"/>']
    for t in _ticks(xlo, xhi):
        body.append(f'<text x="{sx(t):.1f}" y="{y0 + ph + 15}" text-anchor="middle">{t:g}</text>')
    for t in _ticks(ylo, yhi):
        body.append(f'<line x1="{x0}" x2="{x0 + pw}" y1="{sy(t):.1f}" y2="{sy(t):.1f}" stroke="#ddd"/>')
        body.append(f'<text x="{x0 - 5}" y="{sy(t) + 4:.1f}" text-anchor="end">{t:g}</text>')
    for i, (label, xs, ys) in enumerate(series):
        col = _PALETTE[i % len(_PALETTE)]
        pts = " ".join(f"{sx(x):.1f},{sy(y):.1f}" for x, y in zip(xs, ys) if np.isfinite(y))
        body.append(f'<polyline points="{pts}" fill="none" stroke="{col}" stroke-width="1.5"/>')
        body.append(f'<rect x="{x0 + pw + 10}" y="{y0 + 16 * i}" width="10" height="10" fill="{col}"/>')
        body.append(f'<text x="{x0 + pw + 25}" y="{y0 + 16 * i + 9}">{label}</text>')
    with open(path, "w") as f:
        f.write("\n".join(head + body + ["</svg>"]))
    return path


def bar_chart(path, groups, series, title="", ylabel="", stacked=False):
    """groups: x-axis group names; series: list of (label, values per group)."""
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    if _have_matplotlib():
        import matplotlib.pyplot as plt
        fig, ax = plt.subplots(figsize=(9, 5))
        n, x = len(series), np.arange(len(groups))
        bottom = np.zeros(len(groups))
        for i, (label, vals) in enumerate(series):
            if stacked:
                ax.bar(x, vals, 0.6, bottom=bottom, label=label)
                bottom += np.asarray(vals, dtype=float)
            else:
                ax.bar(x + (i - (n - 1) / 2) * 0.8 / n, vals, 0.8 / n, label=label)
        ax.set_xticks(x)
        ax.set_xticklabels(groups, rotation=20, ha="right", fontsize=8)
        ax.set(title=title, ylabel=ylabel)
        ax.legend(fontsize=8)
        fig.savefig(path, format="svg", bbox_inches="tight")
        plt.close(fig)
        return path
    head, (x0, y0, pw, ph) = _svg_frame(title, "", ylabel)
    totals = [sum(v[g] for _, v in series) for g in range(len(groups))] if stacked else [v for _, vals in series for v in vals]
    yhi = max(totals + [1e-12])
    sy = lambda y: y0 + ph - y / yhi * ph
    body = [f'<rect x="{x0}" y="{y0}" width="{pw}" height="{ph}" fill="none" stroke="#444"/>']
    for t in _ticks(0, yhi):
        body.append(f'<line x1="{x0}" x2="{x0 + pw}" y1="{sy(t):.1f}" y2="{sy(t):.1f}" stroke="#ddd"/>')
        body.append(f'<text x="{x0 - 5}" y="{sy(t) + 4:.1f}" text-anchor="end">{t:g}</text>')
    gw = pw / max(len(groups), 1)
    for g, name in enumerate(groups):
        base = 0.0
        for i, (label, vals) in enumerate(series):
            col = _PALETTE[i % len(_PALETTE)]
            if stacked:
                bx, bw, top, bot = x0 + g * gw + gw * 0.2, gw * 0.6, base + vals[g], base
                base += vals[g]
            else:
                bw = gw * 0.8 / len(series)
                bx, top, bot = x0 + g * gw + gw * 0.1 + i * bw, vals[g], 0.0
            body.append(f'<rect x="{bx:.1f}" y="{sy(top):.1f}" width="{bw:.1f}" height="{max(sy(bot) - sy(top), 0):.1f}" fill="{col}"/>')
        body.append(f'<text x="{x0 + (g + 0.5) * gw:.1f}" y="{y0 + ph + 15}" text-anchor="middle" font-size="10">{name}</text>')
    for i, (label, _) in enumerate(series):
        col = _PALETTE[i % len(_PALETTE)]
        body.append(f'<rect x="{x0 + pw + 10}" y="{y0 + 16 * i}" width="10" height="10" fill="{col}"/>')
        body.append(f'<text x="{x0 + pw + 25}" y="{y0 + 16 * i + 9}">{label}</text>')
    with open(path, "w") as f:
        f.write("\n".join(head + body + ["</svg>"]))
    return path


# ------------------------------------------------------------------------------------------ figures
def _mean_over_runs(log, key):
    return np.asarray(log[key]).mean(axis=0)


def plot_convergence(runs, out_dir, metric="test_top1_accuracy", versus="epoch"):
    """Metric vs epoch or vs wall time, one curve per run (reference: plot_loss_curves / plot_top1_* ,
    utils.py:42-340)."""
    series = []
    for run in runs:
        if run["log"] is None:
            continue
        ys = _mean_over_runs(run["log"], metric)
        xs = np.arange(1, len(ys) + 1) if versus == "epoch" else _mean_over_runs(run["log"], "time")
        series.append((run["label"], list(xs), list(ys)))
    name = f"{metric}_vs_{versus}.svg"
    return line_chart(os.path.join(out_dir, name), series, title=metric.replace("_", " "),
                      xlabel="epoch" if versus == "epoch" else "time (s)", ylabel=metric)


def plot_time_breakdown(runs, out_dir):
    """Stacked bars of the average per-step time of each phase (reference: utils.py:538-617)."""
    groups = [r["label"] for r in runs]
    series = []
    for label in TIME_LABELS:
        series.append((label, [rank0_timer(r).get(label, {}).get("average_duration", 0.0) for r in runs]))
    return bar_chart(os.path.join(out_dir, "time_breakdown.svg"), groups, series, "time per step", "seconds", stacked=True)


def throughput(run, n_gpus=None):
    """images/s = batch_size * GPUs / average batch time, as the reference computes it (utils.py:785)."""
    t = rank0_timer(run).get("batch", {}).get("average_duration")
    if not t:
        return float("nan")
    bs = int(float(run["config"].get("batch_size", 128)))
    return bs * (n_gpus or 1) / t


def plot_scalability(runs_by_gpus, out_dir, quantity="throughput"):
    """runs_by_gpus: {n_gpus: [runs]} -> grouped bars of step time or images/s (utils.py:620-812)."""
    gpus = sorted(runs_by_gpus)
    labels = sorted({r["label"] for rs in runs_by_gpus.values() for r in rs})
    series = []
    for lab in labels:
        vals = []
        for g in gpus:
            match = [r for r in runs_by_gpus[g] if r["label"] == lab]
            if not match:
                vals.append(0.0)
            elif quantity == "throughput":
                vals.append(throughput(match[0], g))
            else:
                vals.append(rank0_timer(match[0]).get("batch", {}).get("average_duration", 0.0))
        series.append((lab, vals))
    ylabel = "images / s" if quantity == "throughput" else "seconds / step"
    return bar_chart(os.path.join(out_dir, f"scalability_{quantity}.svg"), [f"{g} GPU" for g in gpus], series,
                     f"{quantity} scalability", ylabel)


# ------------------------------------------------------------------------------------------ performance model
def compressed_size_mb(model, method, bits=8, K=10000):
    """Gradient megabytes on the wire for the performance model.  ``wire="reference"`` factors follow
    utils.py:898-917 (QSGD-MN /4, two-scale /2, Rand-K x K/N)."""
    size, n = MODEL_SIZE_MB[model], MODEL_PARAMS[model]
    if method == "allreduce":
        return size
    if method == "qsgd-mn":
        return size / 4
    if method == "qsgd-mn-ts":
        return size / 2
    if method == "grandk-mn":
        return size * K / n / 4
    if method == "grandk-mn-ts":
        return size * K / n / 2
    if method == "packed":
        return size * (bits + 1) / 32          # this library's wire format: b magnitude bits + 1 sign bit
    raise ValueError(method)


def performance_model(t_batch_1gpu, size_mb, n_gpus, gpus_per_node=4, inter_gpu_bw=200 * 1024,
                      network_bw=1 * 1024 / 8, latency=9e-3, batch_size=128):
    """Predicted step time and images/s (reference: utils.py:819-824,925-930):
    T = t_batch(1 GPU) + S / BW_gpu * log2(gpus per node) + (latency + S / BW_net) * log2(nodes)."""
    nodes = max(n_gpus // gpus_per_node, 1)
    local = min(n_gpus, gpus_per_node)
    t = t_batch_1gpu + size_mb / inter_gpu_bw * math.log2(max(local, 1)) if local > 1 else t_batch_1gpu
    if nodes > 1:
        t += (latency + size_mb / network_bw) * math.log2(nodes)
    return t, batch_size * n_gpus / t


def nvlink_performance_model(t_batch_1gpu, payload_bytes, n_gpus, link_gbs=770.0, phases=3, phase_latency_us=8.0,
                             batch_size=128):
    """Same idea for one NVSwitch domain: two-shot exchange moves 2 (W-1)/W * payload per GPU at the measured
    per-direction peer bandwidth, plus a fixed cost per cross-GPU synchronisation phase."""
    if n_gpus <= 1:
        return t_batch_1gpu, batch_size / t_batch_1gpu
    t_comm = 2 * (n_gpus - 1) / n_gpus * payload_bytes / (link_gbs * 1e9) + phases * phase_latency_us * 1e-6
    t = t_batch_1gpu + t_comm
    return t, batch_size * n_gpus / t


def plot_performance_model(out_dir, t_batch, model="ResNet50", gpu_counts=(4, 8, 16, 32, 64), **kw):
    series = []
    for method in ("allreduce", "qsgd-mn", "qsgd-mn-ts", "grandk-mn", "grandk-mn-ts"):
        series.append((method, [performance_model(t_batch, compressed_size_mb(model, method), g, **kw)[1] for g in gpu_counts]))
    return bar_chart(os.path.join(out_dir, f"performance_model_{model}.svg"), [f"{g} GPU" for g in gpu_counts], series,
                     f"modelled throughput, {model}", "images / s")


def main(argv=None):
    import argparse

    p = argparse.ArgumentParser(description="draw the analysis figures from a directory of run logs")
    p.add_argument("logs", help="directory that holds one sub-directory per run")
    p.add_argument("--out", default="./plots")
    args = p.parse_args(argv)
    runs = load_runs(args.logs)
    made = []
    for metric in ("train_loss", "test_loss", "test_top1_accuracy", "test_top5_accuracy"):
        for versus in ("epoch", "time"):
            made.append(plot_convergence(runs, args.out, metric, versus))
    made.append(plot_time_breakdown(runs, args.out))
    for m in made:
        print(m)


if __name__ == "__main__":
    main()
