"""T2: trainer plumbing on CPU -- timer/logger file formats, AverageMeter, models, config, the
5-step ResNet-50 + QSGD-MN-8 run on two gloo ranks, checkpoint / resume."""
import json
import os

import numpy as np
import pytest
import torch

from gradient_compression_b200 import models
from gradient_compression_b200.parallel import CosineSchedule, FlatArena, FlatSGD
from gradient_compression_b200.train import CIFAR, TrainConfig, train
from gradient_compression_b200.utils import AverageMeter, Logger, Timer, set_seed


def test_timer_sync_mode_labels_and_json(tmp_path):
    t = Timer(verbosity_level=2, quiet=True)
    for _ in range(3):
        with t("batch"):
            with t("batch.reduce"):
                pass
            with t("reduce.norm", verbosity=2):
                pass
            with t("too.verbose", verbosity=3):
                pass
    assert t.call_counts["batch"] == 2          # first occurrence skipped
    assert "too.verbose" not in t.totals and len(t.reduce_times) == 3
    path = tmp_path / "timer_summary_0.json"
    t.save_summary(str(path))
    data = json.loads(path.read_text())
    assert set(data["batch"]) == {"label", "average_duration", "n_events", "total_time"}
    assert "Timer summary" in t.summary() and "total_time" in t.summary()


def test_average_meter_modes():
    m = AverageMeter("cpu")
    m.add({"a": 1.0})
    m.add({"a": torch.tensor(3.0)})
    m.reduce()
    assert m.values()["a"] == pytest.approx(2.0)
    c = AverageMeter("cpu", reference_compat=True)   # reference keeps only the latest value
    c.add({"a": 1.0})
    c.add({"a": 3.0})
    assert c.values()["a"] == 3.0


def test_logger_artifacts(tmp_path):
    cfg = {"architecture": "VGG16", "runs": 1, "num_epochs": 2, "lr": 0.1}
    lg = Logger(cfg, 0, root=str(tmp_path))
    assert os.path.basename(lg.log_path).endswith("_VGG16")
    stamp = os.path.basename(lg.log_path)[:19]
    assert int(stamp[-2:]) % 30 == 0                 # rounded to 30 s so that ranks agree
    tr, te = AverageMeter("cpu"), AverageMeter("cpu")
    for m in (tr, te):
        m.add({"top1_accuracy": 0.5, "top5_accuracy": 0.9, "cross_entropy_loss": 1.2})
    lg.epoch_update(0, 1, tr, te)
    lg.save_model(torch.nn.Linear(2, 2))
    lg.summary_writer(Timer(quiet=True), {"top1": [0.5], "top5": [0.9]}, 1234)
    files = set(os.listdir(lg.log_path))
    assert {"model.pt", "success.txt", "log_dict.npy", "timer_summary_0.json"} <= files
    txt = open(os.path.join(lg.log_path, "success.txt")).read()
    assert "Best Top 1 Accuracy: 0.5" in txt and "architecture : VGG16" in txt and txt.endswith("Bits communicated: 1234")
    d = np.load(os.path.join(lg.log_path, "log_dict.npy"), allow_pickle=True).item()
    assert d["test_top1_accuracy"].shape == (1, 2) and d["test_top1_accuracy"][0, 1] == 0.5


def test_models_shapes_and_param_counts():
    counts = {"ResNet50": (23520842, 161), "VGG16": (14728266, 54)}
    for name, (n, k) in counts.items():
        net = getattr(models, name)()
        ps = list(net.parameters())
        assert sum(p.numel() for p in ps) == n and len(ps) == k
    net = models.ResNet18()
    assert net(torch.randn(2, 3, 32, 32)).shape == (2, 10)
    keys = list(models.ResNet50().state_dict())
    assert keys[0] == "conv1.weight" and "layer1.0.shortcut.0.weight" in keys and keys[-1] == "linear.bias"
    assert "features.0.weight" in models.VGG16().state_dict() and "classifier.bias" in models.VGG16().state_dict()


def test_flat_arena_and_sgd_match_torch():
    set_seed(0)
    net = models.VGG11()
    ref = models.VGG11()
    ref.load_state_dict(net.state_dict())
    arena = FlatArena(list(net.parameters()))
    opt = FlatSGD(arena, lr=0.1)
    sched = CosineSchedule(opt, T_max=10)
    topt = torch.optim.SGD(ref.parameters(), lr=0.1, momentum=0.9, weight_decay=5e-4, nesterov=True)
    tsched = torch.optim.lr_scheduler.CosineAnnealingLR(topt, T_max=10, eta_min=0)
    x, y = torch.randn(4, 3, 32, 32), torch.randint(0, 10, (4,))
    for _ in range(2):
        arena.zero_grad()
        topt.zero_grad()
        torch.nn.functional.cross_entropy(net(x), y).backward()
        torch.nn.functional.cross_entropy(ref(x), y).backward()
        assert all(p.grad.data_ptr() == gv.data_ptr() for p, gv in zip(arena.params, arena.grad_views))
        opt.step()
        topt.step()
        sched.step()
        tsched.step()
        assert opt.lr == pytest.approx(tsched.get_last_lr()[0])
    for a, b in zip(net.parameters(), ref.parameters()):
        assert torch.allclose(a, b, atol=1e-5)


def test_config_cli_and_yaml(tmp_path):
    cfg, args = TrainConfig.from_args(["--architecture", "VGG16", "--reducer", "RankKReducer", "--rank", "2",
                                       "--local-rank", "1", "--quantization_levels", "2", "6"])
    assert cfg.architecture == "VGG16" and cfg.rank == 2 and args.local_rank == 1 and cfg.quantization_levels == [2, 6]
    p = tmp_path / "c.yaml"
    p.write_text("architecture: ResNet18\nlr: 0.05\nK: 123\n")
    cfg, _ = TrainConfig.from_args(["--config", str(p), "--lr", "0.2"])
    assert cfg.architecture == "ResNet18" and cfg.K == 123 and cfg.lr == 0.2


def _train_body(rank, world, root):
    cfg = TrainConfig(runs=1, num_epochs=1, batch_size=4, architecture="ResNet50", reducer="QSGDMaxNormReducer",
                      quantization_level=8, data="synthetic", synthetic_train_size=8 * world * 5,
                      synthetic_test_size=8 * world, max_steps_per_epoch=5, log_root=root, log_verbosity=2,
                      lr=0.1, save_training_state=True, timer_mode="sync")
    lg = train(rank, cfg, logger=Logger(cfg.as_dict(), rank, log_path=os.path.join(root, "run")))
    assert os.path.exists(os.path.join(lg.log_path, f"timer_summary_{rank}.json"))


def test_baseline_config0_resnet50_qsgd8_two_gloo_ranks(dist_runner, tmp_path):
    dist_runner(_train_body, world=2, args=(str(tmp_path),))
    run = tmp_path / "run"
    files = set(os.listdir(run))
    assert {"model.pt", "success.txt", "log_dict.npy", "timer_summary_0.json", "timer_summary_1.json",
            "train_state.pt"} <= files
    sd = torch.load(run / "model.pt")
    net = models.ResNet50()
    net.load_state_dict(sd)                        # reference-compatible keys, bit-exact reload
    assert all(torch.equal(sd[k], v) for k, v in net.state_dict().items())
    timers = json.loads((run / "timer_summary_0.json").read_text())
    assert {"batch", "batch.forward", "batch.backward", "batch.reduce", "batch.step"} <= set(timers)
    log = np.load(run / "log_dict.npy", allow_pickle=True).item()
    assert np.isfinite(log["train_loss"]).all()
    bits = int(open(run / "success.txt").read().rsplit(":", 1)[1])
    assert bits == 5 * (32 + 32 * 23520842)         # 8-bit levels ride int32 containers in the reference's accounting


def test_resume_continues_where_it_stopped(tmp_path):
    base = dict(runs=1, batch_size=4, architecture="VGG11", reducer="GlobalRandKMaxNormReducer", K=1000,
                quantization_level=4, data="synthetic", synthetic_train_size=16, synthetic_test_size=8,
                log_verbosity=0, save_training_state=True, timer_mode="sync", lr=0.01)
    full = TrainConfig(num_epochs=2, log_root=str(tmp_path / "a"), **base)
    lg_full = train(0, full, logger=Logger(full.as_dict(), 0, log_path=str(tmp_path / "a" / "run")))
    # the twin run saves an extra copy of its state after epoch 0; resuming from that copy must reach
    # the same end state as the uninterrupted run
    first = TrainConfig(num_epochs=2, log_root=str(tmp_path / "b"), **base)
    lg_b = Logger(first.as_dict(), 0, log_path=str(tmp_path / "b" / "run"))
    real_save = Logger.save_training_state

    def capture(self, state, name="train_state.pt"):
        if state.get("epoch") == 0:
            real_save(self, state, name.replace("train_state", "epoch0"))
        real_save(self, state, name)

    Logger.save_training_state = capture
    try:
        train(0, first, logger=lg_b)
    finally:
        Logger.save_training_state = real_save
    resumed_cfg = TrainConfig(num_epochs=2, log_root=str(tmp_path / "c"), resume=str(tmp_path / "b" / "run" / "epoch0.pt"),
                              **base)
    lg_c = train(0, resumed_cfg, logger=Logger(resumed_cfg.as_dict(), 0, log_path=str(tmp_path / "c" / "run")))
    a = torch.load(os.path.join(lg_full.log_path, "train_state.pt"), weights_only=False)
    c = torch.load(os.path.join(lg_c.log_path, "train_state.pt"), weights_only=False)
    assert a["epoch"] == c["epoch"] == 1 and a["bits"] == c["bits"]
    for k in a["model"]:
        assert torch.allclose(a["model"][k].float(), c["model"][k].float(), atol=1e-6), k
    assert torch.allclose(a["optimizer"]["momentum_buf"], c["optimizer"]["momentum_buf"], atol=1e-6)


def test_trainer_with_device_resident_pipeline(tmp_path):
    cfg = TrainConfig(runs=1, num_epochs=1, batch_size=8, architecture="LeNet", reducer="NoneAllReducer",
                      data="synthetic_device", synthetic_train_size=32, synthetic_test_size=16, log_verbosity=0,
                      timer_mode="sync", lr=0.01, log_root=str(tmp_path))
    lg = train(0, cfg, logger=Logger(cfg.as_dict(), 0, log_path=str(tmp_path / "run")))
    log = np.load(os.path.join(lg.log_path, "log_dict.npy"), allow_pickle=True).item()
    assert np.isfinite(log["train_loss"]).all() and np.isfinite(log["test_loss"]).all()


def _resume_body(rank, world, root):
    """Two workers with error-feedback memories: each must get its OWN memory and noise stream back on resume."""
    base = dict(runs=1, batch_size=4, architecture="LeNet", reducer="TopKReducer", K=5, data="synthetic",
                synthetic_train_size=16 * world, synthetic_test_size=8 * world, log_verbosity=0, save_training_state=True,
                timer_mode="sync", lr=0.01, broadcast_parameters=True)
    first = TrainConfig(num_epochs=1, log_root=root, **base)
    train(rank, first, logger=Logger(first.as_dict(), rank, log_path=os.path.join(root, "run")))
    torch.distributed.barrier()                  # every rank has written its files
    mine = torch.load(os.path.join(root, "run", f"train_state.rank{rank}.pt"), weights_only=False)
    other = torch.load(os.path.join(root, "run", f"train_state.rank{1 - rank}.pt"), weights_only=False)
    mem_mine, mem_other = mine["reducer"]["memory"], other["reducer"]["memory"]
    assert not torch.equal(mem_mine, mem_other), "workers see different data: their memories differ"
    # resume: the reducer of this rank must hold this rank's memory, not rank 0's
    from gradient_compression_b200.reducers import make_reducer
    from gradient_compression_b200.train import checkpoint as ckpt

    red = make_reducer("TopKReducer", "cpu", None, {"K": 5})
    state = torch.load(os.path.join(root, "run", "train_state.pt"), weights_only=False)
    rs = ckpt.load_rank_state(os.path.join(root, "run", "train_state.pt"), rank)
    assert rs is not None
    red.load_state_dict((rs if rs["reducer_class"] == "TopKReducer" else state)["reducer"])
    assert torch.equal(red.state_dict()["memory"], mem_mine)


def test_two_rank_resume_restores_each_workers_own_reducer_state(dist_runner, tmp_path):
    dist_runner(_resume_body, world=2, args=(str(tmp_path),))


def test_noise_source_keeps_the_live_rank_on_restore():
    from gradient_compression_b200.compressors import NoiseSource

    saved = NoiseSource(seed=3, rank=0)
    saved.step = 17
    live = NoiseSource(seed=3, rank=1)
    live.load_state_dict(saved.state_dict())
    assert live.rank == 1 and live.step == 17 and live.stream(1) != saved.stream(1)
