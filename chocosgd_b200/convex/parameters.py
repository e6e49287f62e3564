"""Experiment parameters with fail-fast validation (``convex_code/parameters.py:6-129``)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

LR_TYPES = ("constant", "epoch-decay", "decay", "bottou")
QUANTIZATIONS = ("full", "top", "random-biased", "random-unbiased", "qsgd-biased", "qsgd-unbiased")
ESTIMATES = ("final", "mean", "t+tau", "(t+tau)^2")
TOPOLOGIES = ("centralized", "ring", "torus", "disconnected")
METHODS = ("choco", "dcd-psgd", "ecd-psgd", "plain")
SPLITS = ("naive", "random", "label-sorted")


@dataclass
class Parameters:
    num_epoch: int
    lr_type: str
    initial_lr: Optional[float] = None
    regularizer: Optional[float] = None
    epoch_decay_lr: Optional[float] = None
    consensus_lr: Optional[float] = None
    quantization: str = "full"
    coordinates_to_keep: Optional[int] = None  # k of top-k / random-k
    num_levels: Optional[int] = None  # s of QSGD
    estimate: str = "final"
    name: Optional[str] = None
    n_cores: int = 1
    topology: str = "centralized"
    method: str = "choco"
    distribute_data: bool = False
    split_data_strategy: Optional[str] = None
    tau: Optional[float] = None
    real_update_every: int = 1
    random_seed: Optional[int] = None
    split_data_random_seed: Optional[int] = None

    def __post_init__(self):
        def need(cond, msg):
            if not cond:
                raise ValueError(msg)

        need(self.num_epoch >= 0, "num_epoch must be >= 0")
        need(self.lr_type in LR_TYPES, f"lr_type must be one of {LR_TYPES}")
        if self.lr_type in ("constant", "decay"):
            need(self.initial_lr is not None and self.initial_lr > 0, "initial_lr must be > 0")
        if self.lr_type == "decay":
            need(bool(self.tau) and self.regularizer is not None and self.regularizer > 0,
                 "lr_type 'decay' needs tau and a positive regularizer")
        if self.lr_type == "epoch-decay":
            need(self.epoch_decay_lr is not None, "lr_type 'epoch-decay' needs epoch_decay_lr")
        if self.method == "choco":
            need(self.consensus_lr is not None and self.consensus_lr > 0, "choco needs consensus_lr > 0")
        else:
            need(self.consensus_lr is None, "consensus_lr is only used by choco")
        need(self.quantization in QUANTIZATIONS, f"quantization must be one of {QUANTIZATIONS}")
        if self.quantization == "full":
            need(not self.coordinates_to_keep, "'full' takes no coordinates_to_keep")
        elif self.quantization in ("top", "random-biased", "random-unbiased"):
            need(self.coordinates_to_keep is not None and self.coordinates_to_keep > 0, "coordinates_to_keep must be > 0")
        else:
            need(self.num_levels is not None and self.num_levels > 0, "qsgd needs num_levels > 0")
        need(self.estimate in ESTIMATES, f"estimate must be one of {ESTIMATES}")
        need(self.n_cores > 0, "n_cores must be > 0")
        need(self.topology in TOPOLOGIES, f"topology must be one of {TOPOLOGIES}")
        need(self.method in METHODS, f"method must be one of {METHODS}")
        if self.method in ("dcd-psgd", "ecd-psgd"):
            need(self.quantization in ("random-unbiased", "qsgd-unbiased"),
                 "dcd-/ecd-psgd are defined for unbiased compressors")
        if not self.distribute_data:
            need(not self.split_data_strategy, "split_data_strategy needs distribute_data")
        else:
            need(self.split_data_strategy in SPLITS, f"split_data_strategy must be one of {SPLITS}")

    def lr_str(self):
        if self.lr_type == "constant":
            return "lr{}".format(self.initial_lr)
        if self.lr_type == "decay":
            return "lr{}/lambda*(t+{})".format(self.initial_lr, self.tau)
        if self.lr_type == "bottou":
            return "lr-bottou-{}".format(self.initial_lr)
        return "lr-{}".format(self.lr_type)

    def sparse_str(self):
        s = self.quantization
        if self.quantization in ("top", "random-biased", "random-unbiased"):
            s += str(self.coordinates_to_keep)
        elif self.quantization != "full":
            s += str(self.num_levels)
        return s

    def __str__(self):
        if self.name:
            return self.name
        reg = "-reg{}".format(self.regularizer) if self.regularizer else ""
        return "epoch{}-{}{}-{}-{}".format(self.num_epoch, self.lr_str(), reg, self.sparse_str(), self.estimate)
