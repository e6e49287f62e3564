"""Per-rank checkpoints with the reference's layout and keys.

``<checkpoint>/<data>/<arch>/<experiment>/<timestamp>/<rank>/checkpoint.pth.tar`` holds
``{"arch", "current_epoch", "local_index", "best_perf", "optimizer", "state_dict"}``;
``model_best.pth.tar`` and ``checkpoint_epoch_N.pth.tar`` are copies; rank 0 pickles the
arguments (``dl_code/pcode/utils/checkpoint.py:59-159``).  ``optimizer`` additionally
carries the algorithm state (x_hat, s, error memories), which the reference loses on resume."""
from __future__ import annotations

import gc
import shutil
from os.path import isfile, join

import torch

from . import logging as logging_
from .op_files import write_pickle
from .op_paths import build_dirs, remove_folder


def init_checkpoint(conf, graph, run):
    run.checkpoint_root = join(
        conf.checkpoint, conf.data, conf.arch, conf.experiment if conf.experiment is not None else "", conf.timestamp
    )
    run.checkpoint_dir = join(run.checkpoint_root, str(graph.rank))
    if conf.save_some_models is not None and isinstance(conf.save_some_models, str):
        run.extras["save_some_models"] = conf.save_some_models.split(",")
    build_dirs(run.checkpoint_dir)


def save_arguments(conf, graph, run):
    if graph.rank == 0:
        write_pickle({k: v for k, v in vars(conf).items() if not k.startswith("_")},
                     path=join(run.checkpoint_root, "arguments.pickle"))


def save_to_checkpoint(run, state, is_best, dirname, filename, save_all=False):
    path = join(dirname, filename)
    torch.save(state, path)
    if is_best:
        shutil.copyfile(path, join(dirname, "model_best.pth.tar"))
    some = run.extras.get("save_some_models")
    if save_all or (some is not None and str(state["current_epoch"]) in some):
        shutil.copyfile(path, join(dirname, "checkpoint_epoch_%s.pth.tar" % state["current_epoch"]))
    return path


def maybe_resume_from_checkpoint(conf, graph, run, model, optimizer, scheduler):
    if not conf.resume:
        return False
    index = "_epoch_" + conf.checkpoint_index if conf.checkpoint_index is not None else ""
    path = join(conf.resume, str(graph.rank), "checkpoint{}.pth.tar".format(index))
    print("try to load previous model from the path:{}".format(path))
    if not isfile(path):
        print("=> no checkpoint found at '{}'".format(conf.resume))
        return False
    checkpoint = torch.load(path, map_location="cpu", weights_only=False)
    scheduler.update_from_checkpoint(checkpoint)
    if run.checkpoint_root and run.checkpoint_root != conf.resume:
        remove_folder(run.checkpoint_root)
    run.checkpoint_root = conf.resume
    run.checkpoint_dir = join(conf.resume, str(graph.rank))
    model.load_state_dict(checkpoint["state_dict"])
    optimizer.load_state_dict(checkpoint["optimizer"])
    print("=> loaded model from path '{}' checkpointed at (epoch {})".format(conf.resume, checkpoint["current_epoch"]))
    run.logger = logging_.Logger(run.checkpoint_dir)
    del checkpoint
    gc.collect()
    return True
