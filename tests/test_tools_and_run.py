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
