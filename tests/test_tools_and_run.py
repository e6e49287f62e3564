"""Launcher + training loop + result tools on CPU: two Gloo ranks started by the launcher train a
tiny synthetic problem, write logs and checkpoints, and the tools read them back."""
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_hostfile_and_commands(tmp_path):
    from chocosgd_b200 import run
    from chocosgd_b200.config import get_args

    hf = tmp_path / "hostfile"
    hf.write_text("localhost slots=2\nnode1 slots=3\n# comment\n")
    hosts = run.read_hostfile(str(hf))
    assert hosts == [{"host": "localhost", "slots": 2}, {"host": "node1", "slots": 3}]
    assert run.map_slot(hosts) == ["localhost"] * 2 + ["node1"] * 3
    conf = get_args(["--arch", "resnet20", "--n_mpi_process", "2", "--comm_op", "sign"])
    cmd = run.build_rank_command(conf, 1)
    assert cmd[1:3] == ["-m", "chocosgd_b200.main"] and cmd[-2:] == ["--local_rank", "1"]
    assert "--comm_op" in cmd and "sign" in cmd
    env = run.rank_env(conf, 1, 2, 1234, base={})
    assert env["RANK"] == "1" and env["WORLD_SIZE"] == "2" and env["MASTER_PORT"] == "1234"


def test_tmux_job_lines():
    from chocosgd_b200.tmux_cluster import Job

    job = Job("exp")
    job.add("localhost", "echo a")
    job.add("node1", "echo b")
    lines = job.lines()
    assert lines[0].startswith("tmux kill-session -t exp") and "ssh node1" in lines[-1] and len(lines) == 4


@pytest.mark.timeout(600)
def test_launcher_trains_two_ranks_and_tools_read_results(tmp_path):
    ck = tmp_path / "ckpt"
    cmd = [sys.executable, "-m", "chocosgd_b200.run", "--data", "synthetic_cifar10", "--synthetic_size", "128",
           "--arch", "lenet", "--batch_size", "16", "--num_epochs", "2", "--optimizer", "parallel_choco_v",
           "--comm_op", "sign", "--graph_topology", "ring", "--consensus_stepsize", "0.4", "--on_cuda", "False",
           "--backend", "gloo", "--n_mpi_process", "2", "--partition_data", "random", "--lr", "0.05",
           "--lr_schedule_scheme", "custom_multistep", "--lr_change_epochs", "1", "--num_workers", "0",
           "--checkpoint", str(ck), "--evaluate_consensus", "True", "--summary_freq", "2", "--experiment", "t",
           "--timestamp", "run1", "--manual_seed", "3"]
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""), OMP_NUM_THREADS="1")
    r = subprocess.run(cmd, env=env, cwd=ROOT, capture_output=True, text=True, timeout=560)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    root = ck / "synthetic_cifar10" / "lenet" / "t" / "run1"
    for rank in ("0", "1"):
        assert (root / rank / "checkpoint.pth.tar").exists() and (root / rank / "log-1.json").exists()
    assert (root / "arguments.pickle").exists()

    from chocosgd_b200.tools.show_results import curve, find_experiments, load_experiment, split_records, summarize

    exp = load_experiment(str(root))
    assert sorted(exp["records"]) == [0, 1] and exp["arguments"]["comm_op"] == "sign"
    parts = split_records(exp["records"][0])
    assert parts["train"] and parts["test_local"] and parts["test_averaged"] and parts["stat"]
    assert parts["stat"][0]["distance"] >= 0
    xs, ys = curve(exp, "test_local", "loss")
    assert xs == [1.0, 2.0] and all(np.isfinite(ys))
    assert len(find_experiments(str(ck), {"optimizer": "parallel_choco_v"})) == 1
    assert len(find_experiments(str(ck), {"optimizer": "sgd"})) == 0
    df = summarize([exp], metric="loss")
    assert len(df) == 1 and df["count"][0] == 1

    from chocosgd_b200 import auto_extract
    from chocosgd_b200.tools.plot import plot_curves
    from chocosgd_b200.utils.op_files import load_pickle

    out = auto_extract.main(["--in_dir", str(ck)])
    summary = load_pickle(out)
    assert len(summary) == 1 and "test_local/loss" in summary[0]["curves"]
    p = plot_curves({"loss": (xs, ys)}, str(tmp_path / "c.png"))
    assert os.path.exists(p)

    # resume: one more epoch from the checkpoint continues local_index
    cmd2 = [c for c in cmd]
    cmd2[cmd2.index("--num_epochs") + 1] = "3"
    cmd2[cmd2.index("--timestamp") + 1] = "run2"
    cmd2 += ["--resume", str(root)]
    r = subprocess.run(cmd2, env=env, cwd=ROOT, capture_output=True, text=True, timeout=560)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    import torch

    ckpt = torch.load(root / "0" / "checkpoint.pth.tar", weights_only=False)
    assert ckpt["current_epoch"] == 3 and "x_hat" in ckpt["optimizer"]["algo_state"]


def _fake_exp(tmp_path, name, opt, lr, seed, n_nodes=2, batch=32):
    import json
    import pickle

    d = tmp_path / name
    (d / "0").mkdir(parents=True)
    with open(d / "arguments.pickle", "wb") as f:
        pickle.dump({"optimizer": opt, "lr": lr, "manual_seed": seed, "n_mpi_process": n_nodes, "batch_size": batch,
                     "comm_op": "sign"}, f)
    recs = []
    for i in range(1, 7):
        recs.append({"measurement": "runtime", "split": "train", "time": "2024-01-01 00:00:%02d" % i, "rank": 0,
                     "epoch": i / 2, "local_index": i, "n_bits_to_transmit": 0.5, "loss": 2.0 / i + 0.01 * seed})
        if i % 2 == 0:
            recs.append({"measurement": "runtime", "split": "test", "type": "local_model", "rank": 0, "epoch": i / 2,
                         "local_index": i, "time": "2024-01-01 00:00:%02d" % i, "top1": 10.0 * i + seed})
    with open(d / "0" / "log-1.json", "w") as f:
        json.dump(recs, f)


def test_plot_tool_groups_legends_and_axes(tmp_path):
    from chocosgd_b200.tools import plot
    from chocosgd_b200.tools.show_results import find_experiments

    for seed in (0, 1):
        _fake_exp(tmp_path, f"a{seed}", "parallel_choco_v", 0.1, seed)
    _fake_exp(tmp_path, "b0", "sgd", 0.2, 0, n_nodes=4)
    exps = find_experiments(str(tmp_path))
    series, bands = plot.collect_series(exps, "optimizer,lr", "test_local", "top1", "epoch")
    assert set(series) == {"optimizer=parallel_choco_v, lr=0.1", "optimizer=sgd, lr=0.2"}
    xs, ys = series["optimizer=parallel_choco_v, lr=0.1"]
    assert xs == [1.0, 2.0, 3.0] and ys == [20.5, 40.5, 60.5]          # mean of the two repetitions
    assert "optimizer=parallel_choco_v, lr=0.1" in bands and "optimizer=sgd, lr=0.2" not in bands
    xs, ys = plot.series_of(exps[0], "train", "loss", "bits")
    assert xs == [0.5, 1.0, 1.5, 2.0, 2.5, 3.0]
    xs, _ = plot.series_of(exps[0], "train", "loss", "time")
    assert xs[0] == 1 and xs[-1] == 6
    assert plot.smooth([1, 2, 3, 4], 2) == [1.0, 1.5, 2.5, 3.5]
    assert plot.find_same_num_sync([(100, 4), (90, 2)]) == 25
    out = plot.plot_curve_wrt(exps, str(tmp_path / "fig.png"), x="step", split="train", metric="loss", legend="optimizer")
    assert out.endswith((".png", ".csv")) and (tmp_path / out.split("/")[-1]).exists()
    groups = plot.best_by_global_minibatch_size(exps)
    assert dict(groups)["0.1"] == [(64, 61.0)] and dict(groups)["0.2"] == [(128, 60.0)]
    assert plot.plot_by_global_minibatch_size(exps, str(tmp_path / "gb.png")).endswith((".png", ".csv"))


def test_convex_suboptimality_curves_and_bit_model(tmp_path):
    import numpy as np

    from chocosgd_b200.convex.data import synthetic_logistic
    from chocosgd_b200.convex.experiment import epsilon_final_params, run_experiment
    from chocosgd_b200.tools import plot_convex

    A, y = synthetic_logistic(180, 16, seed=2)
    params = [p for p in epsilon_final_params(n=180, d=16, n_cores=3, num_epoch=1, seeds=(1, 2), splits=("random",))
              if p.method in ("plain", "choco") and p.quantization in ("full", "top")]
    for p in params:
        if p.quantization == "top":
            p.coordinates_to_keep = 4
    run_experiment(str(tmp_path / "exp"), (A, y), params, nproc=1)
    curves = plot_convex.main([str(tmp_path / "exp"), "--out", str(tmp_path / "plots"), "--n_samples", "180",
                               "--n_features", "16"])
    assert set(curves) == {"plain-full-random", "choco-top-random", "choco-full-random"}
    c = curves["choco-top-random"]
    assert c["n_runs"] == 2 and c["epoch"][0] == 0 and len(c["bits"]) == len(c["mean"])
    # (64 + ceil(log2 16)) * 2 * 4 bits per node and iteration, 3 nodes, 6 iterations between loss evaluations
    assert np.isclose(c["bits"][1], 6 * 3 * (64 + 4) * 2 * 4)
    assert np.isclose(curves["plain-full-random"]["bits"][1], 6 * 3 * 64 * 2 * 16)
    assert (tmp_path / "plots").exists() and len(list((tmp_path / "plots").iterdir())) == 2


def test_every_example_script_parses_with_the_cli():
    """Each ``python -m chocosgd_b200.run ...`` command of the shipped example scripts is a valid
    command line of this framework (flags, choices and types)."""
    import glob
    import re
    import shlex

    from chocosgd_b200.config import get_args

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    scripts = sorted(glob.glob(os.path.join(root, "exps", "*", "*.sh")))
    assert len(scripts) >= 4
    n_cmds = 0
    for path in scripts:
        text = open(path).read().replace("\\\n", " ")
        common = re.search(r'COMMON="([^"]*)"', text)
        for line in text.splitlines():
            if "chocosgd_b200.run" not in line or line.lstrip().startswith("#"):
                continue
            argv = shlex.split(line.split("chocosgd_b200.run", 1)[1].replace("$COMMON", common.group(1) if common else ""))
            conf = get_args(argv)
            assert conf.optimizer in ("sgd", "parallel_choco", "parallel_choco_v", "dcd_psgd", "ecd_psgd",
                                      "deep_squeeze", "dgc", "ef_sign_sgd")
            assert conf.n_mpi_process in (8, 32)
            n_cmds += 1
    assert n_cmds >= 14
    hosts = open(os.path.join(root, "hostfile")).read().split()
    assert hosts[0] == "localhost" and hosts[1].startswith("slots=")


def test_kernel_bench_lists_its_cases():
    """The single-kernel bench parses its arguments without a GPU (``--help`` names every case)."""
    import subprocess
    import sys

    r = subprocess.run([sys.executable, "-m", "chocosgd_b200.tools.kernel_bench", "--help"], capture_output=True, text=True,
                       cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    assert r.returncode == 0
    for case in ("sign", "topk", "gemm", "conv", "bn16", "wgrad_gen", "conv_s2", "maxpool"):
        assert case in r.stdout
