import json
import os

import torch

from chocosgd_b200.utils.logging import Logger
from chocosgd_b200.utils.stat_tracker import AverageMeter, BestPerf, RuntimeTracker
from chocosgd_b200.utils.tensor_buffer import TensorBuffer
from chocosgd_b200.utils.timer import Timer


def test_logger_schema_and_rotation(tmp_path):
    lg = Logger(str(tmp_path))
    for i in range(1001):
        lg.log_metric("runtime", {"epoch": i, "loss": 1.0}, {"split": "train"})
    lg.save_json()
    data = json.load(open(tmp_path / "log-1.json"))
    assert len(data) == 1001 and data[0] == {"measurement": "runtime", "epoch": 0, "loss": 1.0, "split": "train"}
    assert lg.values == [] and lg.file_json.endswith("log-2.json")
    lg.log("hello")
    assert "hello" in open(tmp_path / "log.txt").read()


def test_timer_counts_and_summary():
    records = []
    t = Timer(verbosity_level=1, log_fn=lambda n, v, tags: records.append((n, v, tags)), on_cuda=False)
    for _ in range(3):
        with t("forward_pass", epoch=1.0):
            sum(range(1000))
        with t("sync.apply_grad", epoch=1.0):
            pass
    with t("hidden", verbosity=2):
        pass
    assert t.call_counts["forward_pass"] == 2  # first occurrence skipped
    assert "hidden" not in t.totals
    assert "forward_pass" in t.summary() and records and records[0][0] == "timer"


def test_trackers():
    m = AverageMeter()
    m.update(2.0, 3)
    m.update(torch.tensor(4.0), 1)
    assert abs(m.avg - 2.5) < 1e-9
    tr = RuntimeTracker(["top1"], on_cuda=False)
    tr.update_metrics([1.0, 50.0], 10)
    tr.update_metrics([3.0, 100.0], 10)
    assert tr() == {"loss": 2.0, "top1": 75.0} and tr.evaluate_global_metrics() == [75.0]
    b = BestPerf(larger_is_better=True)
    b.update(10, 1.0)
    b.update(5, 2.0)
    assert b.best_perf == 10 and b.get_best_perf_loc() == 1.0 and not b.is_best
    lo = BestPerf(larger_is_better=False)
    lo.update(10, 1.0)
    lo.update(5, 2.0)
    assert lo.best_perf == 5 and lo.is_best


def test_tensor_buffer_roundtrip():
    ts = [torch.randn(3, 4), torch.randn(5)]
    tb = TensorBuffer(ts)
    assert tb.nelement() == 17 and len(tb) == 2 and tb[0].shape == (3, 4)
    tb.buffer.mul_(2)
    out = [torch.zeros(3, 4), torch.zeros(5)]
    tb.unpack(out)
    assert torch.equal(out[0], ts[0] * 2)


def test_checkpoint_roundtrip_restores_algorithm_state(tmp_path):
    """x_hat, s, momentum and the step counter survive save / load (the reference loses them)."""
    from chocosgd_b200.config import get_args
    from chocosgd_b200.optim import define_optimizer
    from chocosgd_b200.parallel.topology import Graph

    def build():
        torch.manual_seed(0)
        model = torch.nn.Sequential(torch.nn.Linear(6, 5), torch.nn.Linear(5, 2))
        conf = get_args(["--optimizer", "parallel_choco_v", "--comm_op", "compress_top_k", "--compress_ratio", "0.5",
                         "--on_cuda", "False", "--gossip_impl", "nccl", "--lr", "0.1", "--consensus_stepsize", "0.3"])
        return model, define_optimizer(conf, model, Graph("ring", 1, 0, on_cuda=False))

    def run(opt, t0, t1):
        for t in range(t0, t1):
            g = torch.Generator().manual_seed(t)
            opt.arena.g.copy_(torch.randn(opt.seg.total, generator=g) * torch.from_numpy(opt.seg.valid_mask()))
            opt.step()

    m1, o1 = build()
    run(o1, 0, 6)
    m2, o2 = build()
    run(o2, 0, 3)
    path = tmp_path / "checkpoint.pth.tar"
    torch.save({"optimizer": o2.state_dict(), "state_dict": m2.state_dict()}, path)
    ck = torch.load(path, weights_only=False)
    m3, o3 = build()
    m3.load_state_dict(ck["state_dict"])
    o3.load_state_dict(ck["optimizer"])
    assert o3.arena.check_bound() and o3.local_index == 3
    run(o3, 3, 6)
    o1.finalize(), o3.finalize()
    torch.testing.assert_close(o3.arena.x, o1.arena.x, rtol=0, atol=0)
    torch.testing.assert_close(o3.x_hat, o1.x_hat, rtol=0, atol=0)
    assert set(ck["optimizer"].keys()) == {"state", "param_groups", "algo_state"}
