import re
import shlex

import pytest

from chocosgd_b200.config import RunState, get_args, validate
from chocosgd_b200.parallel.topology import Graph
from chocosgd_b200.train.scheduler import Scheduler

EXAMPLE = """
python run.py --arch resnet20 --optimizer parallel_choco \
    --avg_model True --experiment demo --manual_seed 6 \
    --data cifar10 --pin_memory True --batch_size 128 --base_batch_size 64 --num_workers 2 --eval_freq 1 \
    --num_epochs 300 --partition_data random --reshuffle_per_epoch True --stop_criteria epoch \
    --n_mpi_process 8 --n_sub_process 1 --world 0,0,0,0,0,0,0,0 --on_cuda True --use_ipc False \
    --lr 0.1 --lr_scaleup True --lr_scaleup_factor graph --lr_warmup True --lr_warmup_epochs 5 \
    --lr_schedule_scheme custom_multistep --lr_change_epochs 150,225 --lr_decay 10 \
    --weight_decay 1e-4 --use_nesterov True --momentum_factor 0.9 \
    --comm_op sign --consensus_stepsize 0.45 --compress_ratio 0.9 --quantize_level 16 --is_biased True \
    --hostfile hostfile --graph_topology ring --track_time True --display_tracked_time True \
    --python_path $HOME/conda/envs/pytorch-py3.6/bin/python --mpi_path $HOME/.openmpi/
"""


def _argv(cmd):
    toks = shlex.split(cmd.replace("\\\n", " "))
    return toks[2:]


def test_reference_style_command_line_parses():
    conf = get_args(_argv(EXAMPLE))
    assert conf.arch == "resnet20" and conf.optimizer == "parallel_choco" and conf.comm_op == "sign"
    assert conf.consensus_stepsize == 0.45 and conf.graph_topology == "ring" and conf.n_mpi_process == 8
    assert conf.lr_change_epochs == "150,225" and conf.use_nesterov is True and conf.world == "0,0,0,0,0,0,0,0"
    validate(conf)
    cli = conf.to_cli()
    again = get_args(cli)
    assert again.lr == conf.lr and again.comm_op == conf.comm_op and again.lr_change_epochs == conf.lr_change_epochs


def test_unknown_legacy_flags_are_tolerated():
    with pytest.warns(UserWarning):
        conf = get_args(["--choco_consenus_stepsize", "0.5", "--graph_topology", "data_center", "--lr_milestones", "3"])
    assert conf.graph_topology == "complete"
    with pytest.raises(SystemExit):
        get_args(["--nonexistent_flag", "1"], strict=True)


def test_validate_rejects_inconsistent_settings():
    with pytest.raises(ValueError):
        validate(get_args(["--optimizer", "parallel_choco_v"]))
    with pytest.raises(ValueError):
        validate(get_args(["--optimizer", "dcd_psgd", "--comm_op", "compress_top_k"]))
    with pytest.raises(ValueError):
        validate(get_args(["--optimizer", "sgd", "--use_nesterov", "True", "--momentum_factor", "0"]))


def _sched(argv, n=8, batches=100):
    conf = get_args(argv)
    run = RunState()
    run.num_batches_train_per_device_per_epoch = batches
    return Scheduler(conf, Graph(conf.graph_topology, n, 0), run), conf


def test_multistep_with_warmup_matches_worked_example():
    s, conf = _sched(["--lr", "0.1", "--base_batch_size", "64", "--batch_size", "128", "--lr_scaleup", "True",
                      "--lr_scaleup_factor", "graph", "--lr_warmup", "True", "--lr_warmup_epochs", "5",
                      "--lr_schedule_scheme", "custom_multistep", "--lr_change_epochs", "150,225", "--num_epochs", "300",
                      "--graph_topology", "ring"])
    assert abs(s.learning_rate - 0.6) < 1e-12          # 0.1/64*128 * |neighbourhood| = 0.2 * 3
    assert abs(s.get_lr(0.0) - 0.1) < 1e-12            # warm-up starts at --lr
    assert abs(s.get_lr(2.5) - 0.35) < 1e-12
    assert abs(s.get_lr(5.0) - 0.6) < 1e-12 and abs(s.get_lr(149.99) - 0.6) < 1e-12
    assert abs(s.get_lr(150.0) - 0.06) < 1e-12 and abs(s.get_lr(225.0) - 0.006) < 1e-12
    assert s.get_lr(300.0) is None


def test_scheduler_step_updates_groups_and_progress():
    import torch

    s, conf = _sched(["--lr", "1.0", "--lr_schedule_scheme", "custom_multistep", "--lr_change_epochs", "1",
                      "--num_epochs", "2"], batches=4)
    opt = torch.optim.SGD([torch.nn.Parameter(torch.zeros(1))], lr=123.0)
    lrs = []
    for _ in range(8):
        s.step(opt)
        lrs.append(opt.param_groups[0]["lr"])
    assert lrs[:3] == [1.0, 1.0, 1.0] and abs(lrs[3] - 0.1) < 1e-12 and s.epoch == 2 and s.is_stop()
    assert s.local_index == 8 and s.run.epoch_ == 2.0


def test_other_schemes():
    s, _ = _sched(["--lr_schedule_scheme", "custom_one_cycle", "--num_epochs", "60"])
    assert abs(s.get_lr(0) - 0.15) < 1e-12 and abs(s.get_lr(23) - 3.0) < 1e-9 and abs(s.get_lr(46) - 0.15) < 1e-9
    s, _ = _sched(["--lr_schedule_scheme", "strict", "--lr_change_epochs", "10", "--lr_fields", "0.1,0.1/0.01,0.01",
                   "--lr_scale_indicators", "0,0", "--num_epochs", "20"])
    assert abs(s.get_lr(5) - 0.1) < 1e-12 and abs(s.get_lr(15) - 0.01) < 1e-12
    s, _ = _sched(["--lr_schedule_scheme", "custom_convex_decay", "--lr_gamma", "2", "--lr_mu", "0.5", "--lr_alpha", "1",
                   "--num_epochs", "10"])
    assert abs(s.get_lr(3) - 2 / (0.5 * 4)) < 1e-12
    s, _ = _sched(["--lr", "0.1", "--lr_scaleup", "True", "--lr_scaleup_type", "sqrt", "--base_batch_size", "32",
                   "--batch_size", "128"], n=4)
    assert abs(s.learning_rate - 0.1 * (4 * 128 / 32) ** 0.5) < 1e-12
