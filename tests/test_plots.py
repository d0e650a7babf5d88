"""Analysis helpers: log parsing (including the reference's committed logs), headless SVG figures and the
analytic performance model."""
import os
import time

import numpy as np
import pytest

from gradient_compression_b200.utils import plots

# the reference's committed logs are not part of its installed copy: only an explicit checkout has them
REF_LOGS = os.path.join(os.environ["GRADCOMP_REFERENCE_DIR"], "logs") if os.environ.get("GRADCOMP_REFERENCE_DIR") else ""


def test_performance_model_formula():
    t, ips = plots.performance_model(0.2, 89.72, 8, gpus_per_node=4)
    expect = 0.2 + 89.72 / (200 * 1024) * 2 + (9e-3 + 89.72 / 128) * 1
    assert t == pytest.approx(expect) and ips == pytest.approx(128 * 8 / expect)
    assert plots.performance_model(0.2, 89.72, 1)[0] == 0.2
    assert plots.compressed_size_mb("ResNet50", "qsgd-mn") == pytest.approx(89.72 / 4)
    assert plots.compressed_size_mb("VGG16", "grandk-mn") == pytest.approx(56.18 * 10000 / 14728266 / 4)
    t1, _ = plots.nvlink_performance_model(0.01, 94e6, 8)
    assert 0.01 < t1 < 0.011


def test_figures_from_synthetic_logs(tmp_path):
    from gradient_compression_b200.utils import AverageMeter, Logger, Timer

    for i, red in enumerate(["NoneAllReducer", "QSGDMaxNormReducer"]):
        cfg = {"architecture": "VGG16", "runs": 1, "num_epochs": 3, "reducer": red, "quantization_level": 4,
               "batch_size": 128}
        lg = Logger(cfg, 0, log_path=str(tmp_path / "logs" / f"run{i}"))
        t = Timer(verbosity_level=2, quiet=True, skip_first=False)
        for label in plots.TIME_LABELS + ["batch"]:
            with t(label):
                time.sleep(0.0005)          # a measurable duration whatever the clock resolution
        for ep in range(3):
            m = AverageMeter("cpu")
            m.add({"top1_accuracy": 0.1 * ep, "top5_accuracy": 0.2 * ep, "cross_entropy_loss": 2.0 - ep * 0.5})
            lg.epoch_update(0, ep, m, m)
        lg.summary_writer(t, {"top1": [0.2], "top5": [0.4]}, 10)
    runs = plots.load_runs(str(tmp_path / "logs"))
    assert [r["label"] for r in runs] == ["AllReduce-SGD", "QSGD-MN-4"]
    out = str(tmp_path / "plots")
    a = plots.plot_convergence(runs, out, "test_top1_accuracy", "epoch")
    b = plots.plot_time_breakdown(runs, out)
    c = plots.plot_scalability({1: runs, 2: runs}, out)
    d = plots.plot_performance_model(out, 0.2)
    for path in (a, b, c, d):
        txt = open(path).read()
        assert txt.lstrip().startswith("<") and "svg" in txt[:400]
    assert np.isfinite(plots.throughput(runs[0], 2))


@pytest.mark.skipif(not os.path.isdir(REF_LOGS), reason="reference logs not mounted")
def test_parses_the_reference_logs():
    run = plots.load_run(os.path.join(REF_LOGS, "2021_05_20_08_16_00_ResNet50"))
    assert run["config"]["reducer"] == "QSGDMaxNormReducer" and run["label"] == "QSGD-MN-8"
    assert run["config"]["best_top1"] == pytest.approx(0.9461, abs=1e-3)
    assert plots.throughput(run, 2) == pytest.approx(905, rel=0.01)
    assert run["log"]["test_top1_accuracy"].shape == (5, 150)
