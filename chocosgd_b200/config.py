"""Command-line surface and run configuration.

Every flag name, default and choice of the reference parser is accepted
(reference: ``dl_code/parameters.py:10-237``) so that the shell scripts under
``dl_code/exps`` parse unchanged.  Differences, all deliberate:

* flags that the reference scripts pass but its parser never defined
  (``--choco_consenus_stepsize``, ``--lr_scheduler``, ``--lr_milestones`` ...) are
  accepted and reported instead of aborting the run;
* the static configuration (``Config``) is separated from the mutable run state
  (``RunState``: graph, logger, timer, epoch counters) that the reference keeps
  on the same namespace (``dl_code/main.py:152-188``);
* additions for this framework are grouped at the end of the parser.
"""
from __future__ import annotations

import argparse
import time
import warnings
from dataclasses import dataclass, field
from os.path import join
from typing import Any, List, Optional, Sequence

OPTIMIZERS = (
    "sgd",
    "dgc",
    "dcd_psgd",
    "ecd_psgd",
    "parallel_choco",
    "parallel_choco_v",
    "ef_sign_sgd",
    "deep_squeeze",
)
COMM_OPS = ("compress_top_k", "compress_random_k", "quantize_qsgd", "sign")
TOPOLOGIES = (
    "complete",
    "ring",
    "torus",
    "expander",
    "margulis_expander",
    "social",
    "ring_ext",
)


def str2bool(v) -> bool:
    """Same truth table as ``dl_code/parameters.py:240-246``."""
    if isinstance(v, bool):
        return v
    if v.lower() in ("yes", "true", "t", "y", "1"):
        return True
    if v.lower() in ("no", "false", "f", "n", "0"):
        return False
    raise argparse.ArgumentTypeError("Boolean value expected.")


class Config(argparse.Namespace):
    """Parsed flags.  Attribute access like the reference's ``conf`` object."""

    def replace(self, **kw) -> "Config":
        new = Config(**vars(self))
        for k, v in kw.items():
            setattr(new, k, v)
        return new

    def to_cli(self, skip: Sequence[str] = ()) -> List[str]:
        """Serialise every non-None attribute back into ``--k v`` pairs.

        The launcher forwards the full configuration to every rank this way
        (reference: ``dl_code/run.py:54-59``)."""
        out: List[str] = []
        for k, v in sorted(vars(self).items()):
            if v is None or k in skip or k.startswith("_"):
                continue
            out += [f"--{k}", str(v)]
        return out


@dataclass
class RunState:
    """Objects and counters that change while a run is in progress."""

    graph: Any = None
    logger: Any = None
    timer: Any = None
    epoch_: float = 0.0
    epoch: int = 0
    local_index: int = 0
    best_perf: Optional[float] = None
    checkpoint_root: Optional[str] = None
    checkpoint_dir: Optional[str] = None
    num_batches_train_per_device_per_epoch: int = 1
    num_iterations_per_worker: Optional[int] = None
    learning_rate: Optional[float] = None
    init_warmup_lr: Optional[float] = None
    is_centralized: bool = False
    distributed: bool = True
    group: Any = None          # process group of the ranks currently in the run (None: the default group)
    membership: Any = None     # parallel.elastic.Membership when --elastic
    extras: dict = field(default_factory=dict)


def build_parser() -> argparse.ArgumentParser:
    root = "./"
    raw_data = join(root, "data/")
    training = join(raw_data, "checkpoint")

    p = argparse.ArgumentParser(
        description="B200-native decentralized training (CHOCO-SGD family)",
        allow_abbrev=False,
    )
    # where to run.
    p.add_argument("--work_dir", default=None, type=str)
    p.add_argument("--remote_exec", default=False, type=str2bool)

    # dataset.
    p.add_argument("--data", default="cifar10")
    p.add_argument("--data_dir", default=raw_data)
    p.add_argument("--use_lmdb_data", default=False, type=str2bool)
    p.add_argument("--partition_data", default=None, type=str)
    p.add_argument("--pin_memory", default=True, type=str2bool)

    # model.
    p.add_argument("--arch", "-a", default="resnet20")

    # training schedule.
    p.add_argument("--train_fast", type=str2bool, default=False)
    p.add_argument("--stop_criteria", type=str, default="epoch")
    p.add_argument("--num_epochs", type=int, default=90)
    p.add_argument("--num_iterations", type=int, default=32000)
    p.add_argument("--avg_model", type=str2bool, default=False)
    p.add_argument("--reshuffle_per_epoch", default=False, type=str2bool)
    p.add_argument("--batch_size", "-b", default=256, type=int)
    p.add_argument("--base_batch_size", default=None, type=int)

    # learning rate.
    p.add_argument("--lr", type=float, default=0.01)
    p.add_argument("--lr_schedule_scheme", type=str, default=None)
    p.add_argument("--lr_change_epochs", type=str, default=None)
    p.add_argument("--lr_fields", type=str, default=None)
    p.add_argument("--lr_scale_indicators", type=str, default=None)
    p.add_argument("--lr_scaleup", type=str2bool, default=False)
    p.add_argument("--lr_scaleup_type", type=str, default="linear")
    p.add_argument("--lr_scaleup_factor", type=str, default="graph")
    p.add_argument("--lr_warmup", type=str2bool, default=False)
    p.add_argument("--lr_warmup_epochs", type=int, default=5)
    p.add_argument("--lr_decay", type=float, default=10)
    p.add_argument("--lr_onecycle_low", type=float, default=0.15)
    p.add_argument("--lr_onecycle_high", type=float, default=3)
    p.add_argument("--lr_onecycle_extra_low", type=float, default=0.0015)
    p.add_argument("--lr_onecycle_num_epoch", type=int, default=46)
    p.add_argument("--lr_gamma", type=float, default=None)
    p.add_argument("--lr_mu", type=float, default=None)
    p.add_argument("--lr_alpha", type=float, default=None)

    # algorithm.
    p.add_argument("--optimizer", type=str, default="sgd", choices=OPTIMIZERS)
    p.add_argument("--adam_beta_1", default=0.9, type=float)
    p.add_argument("--adam_beta_2", default=0.999, type=float)
    p.add_argument("--adam_eps", default=1e-8, type=float)

    # topology.
    p.add_argument("--graph_topology", default="complete", type=str)

    # compression.
    p.add_argument("--comm_algo", default=None, type=str)
    p.add_argument("--comm_op", default=None, type=str, choices=COMM_OPS)
    p.add_argument("--compress_ratio", default=None, type=float)
    p.add_argument(
        "--compress_warmup_values", default="0.75,0.9375,0.984375,0.996,0.999", type=str
    )
    p.add_argument("--compress_warmup_epochs", default=0, type=int)
    p.add_argument("--quantize_level", default=None, type=int)
    p.add_argument("--is_biased", default=False, type=str2bool)
    p.add_argument("--majority_vote", default=False, type=str2bool)
    p.add_argument("--consensus_stepsize", default=0.9, type=float)
    p.add_argument("--evaluate_consensus", default=False, type=str2bool)
    p.add_argument("--mask_momentum", default=False, type=str2bool)
    p.add_argument("--clip_grad", default=False, type=str2bool)
    p.add_argument("--clip_grad_val", default=None, type=float)
    p.add_argument("--local_step", default=1, type=int)
    p.add_argument("--turn_on_local_step_from", default=0, type=int)
    p.add_argument("--local_adam_memory_treatment", default=None, type=str)

    # momentum / regularisation.
    p.add_argument("--momentum_factor", default=0.9, type=float)
    p.add_argument("--use_nesterov", default=False, type=str2bool)
    p.add_argument("--weight_decay", default=5e-4, type=float)
    p.add_argument("--drop_rate", default=0.0, type=float)

    # per-architecture.
    p.add_argument("--densenet_growth_rate", default=12, type=int)
    p.add_argument("--densenet_bc_mode", default=False, type=str2bool)
    p.add_argument("--densenet_compression", default=0.5, type=float)
    p.add_argument("--wideresnet_widen_factor", default=4, type=int)
    p.add_argument("--rnn_n_hidden", default=200, type=int)
    p.add_argument("--rnn_n_layers", default=2, type=int)
    p.add_argument("--rnn_bptt_len", default=35, type=int)
    p.add_argument("--rnn_clip", type=float, default=0.25)
    p.add_argument("--rnn_use_pretrained_emb", type=str2bool, default=True)
    p.add_argument("--rnn_tie_weights", type=str2bool, default=True)
    p.add_argument("--rnn_weight_norm", type=str2bool, default=False)
    p.add_argument("--mlp_num_layers", default=2, type=int)
    p.add_argument("--mlp_hidden_size", default=500, type=int)

    # misc.
    p.add_argument("--manual_seed", type=int, default=6)
    p.add_argument("--evaluate", "-e", dest="evaluate", type=str2bool, default=False)
    p.add_argument("--eval_freq", default=1, type=int)
    p.add_argument("--summary_freq", default=100, type=int)
    p.add_argument("--timestamp", default=None, type=str)
    p.add_argument("--track_time", default=False, type=str2bool)
    p.add_argument("--track_detailed_time", default=False, type=str2bool)
    p.add_argument("--display_tracked_time", default=False, type=str2bool)
    p.add_argument("--evaluate_avg", default=False, type=str2bool)

    # checkpoint.
    p.add_argument("--resume", default=None, type=str)
    p.add_argument("--checkpoint", "-c", default=training, type=str)
    p.add_argument("--checkpoint_index", type=str, default=None)
    p.add_argument("--save_all_models", type=str2bool, default=False)
    p.add_argument("--save_some_models", type=str, default=None)

    # meta.
    p.add_argument("--user", type=str, default="lin")
    p.add_argument("--project", type=str, default="distributed_adam_type_algorithm")
    p.add_argument("--experiment", type=str, default=None)

    # device / launch.
    p.add_argument("--backend", type=str, default="nccl")
    p.add_argument("--use_ipc", type=str2bool, default=False)
    p.add_argument("--hostfile", type=str, default=None)
    p.add_argument("--mpi_path", type=str, default="$HOME/.openmpi")
    p.add_argument("--mpi_env", type=str, default=None)
    p.add_argument("--python_path", type=str, default="python")
    p.add_argument("-j", "--num_workers", default=4, type=int)
    p.add_argument("--n_mpi_process", default=1, type=int)
    p.add_argument("--n_sub_process", default=1, type=int)
    p.add_argument("--world", default=None, type=str)
    p.add_argument("--on_cuda", type=str2bool, default=True)
    p.add_argument("--comm_device", type=str, default="cuda")
    p.add_argument("--local_rank", default=None, type=str)
    p.add_argument("--clean_python", default=False, type=str2bool)

    # additions of this framework.
    p.add_argument(
        "--gossip_impl",
        default="auto",
        choices=("auto", "fused", "nccl"),
        help="fused = in-kernel NVLink push over peer-mapped arenas; "
        "nccl = torch.distributed send/recv (baseline path, also used on CPU/gloo)",
    )
    p.add_argument("--dtype", default="fp32", choices=("fp32", "bf16"))
    p.add_argument("--pdl", default="auto", choices=("auto", "on", "off"),
                   help="programmatic dependent launch between the library's kernels (auto: on with --dtype bf16)")
    p.add_argument("--steps", default=None, type=int, help="stop after this many local steps")
    p.add_argument("--wait_budget_ms", default=2000.0, type=float,
                   help="upper bound of every in-kernel wait on a peer flag")
    p.add_argument("--gossip_bucket_mb", default=0.0, type=float,
                   help="> 0: with the sign codec the gossip step is launched per bucket of tensors of about this "
                   "size from gradient hooks, on a side stream, overlapping the rest of the backward pass")
    p.add_argument("--nvls", default="auto", choices=("auto", "off"),
                   help="all-reduce of the averaged-model evaluation inside the NVSwitch (multimem kernels) when the "
                   "system has NVLink multicast; off = the process group's all_reduce")
    p.add_argument("--elastic", default=False, type=str2bool,
                   help="keep training on the survivors when a rank leaves or goes silent (heartbeat through the "
                   "rendezvous store, survivor graph with Metropolis weights)")
    p.add_argument("--heartbeat_every", default=50, type=int, help="steps between two membership checks")
    p.add_argument("--heartbeat_stale_s", default=30.0, type=float,
                   help="a rank whose heartbeat has not advanced for this long counts as lost")
    p.add_argument("--leave_at_step", default=None, type=str,
                   help="rank:step - that rank announces an orderly exit before that step (tests of --elastic)")
    p.add_argument("--synthetic_size", default=None, type=int,
                   help="number of samples of the synthetic dataset (data=synthetic_*)")
    p.add_argument("--use_cuda_graph", default=True, type=str2bool)
    p.add_argument("--channels_last", default=True, type=str2bool,
                   help="keep 4-d activations and convolution weights in NHWC / KRSC memory order on CUDA")
    p.add_argument("--native_layers", default="auto", choices=("auto", "all", "off", "bn", "conv"),
                   help="layers routed to the hand-written sm_100a kernels on CUDA: auto = batch-norm + 3x3 "
                   "convolution fwd/dgrad/wgrad, all = auto + linear + LSTM cell, "
                   "bn = batch-norm + linear only, conv = bn + convolution fwd/dgrad, off = library ops")
    p.add_argument("--overlap_gossip", default=True, type=str2bool)
    p.add_argument("--qsgd_levels", default=None, type=int,
                   help="explicit number of QSGD levels s (convex-code spelling); "
                   "--quantize_level gives bits, s = 2^bits - 1")
    p.add_argument("--random_k_seed", default=1234, type=int)
    p.add_argument("--master_addr", default="127.0.0.1", type=str)
    p.add_argument("--master_port", default=None, type=int)
    return p


def default_timestamp(conf: Config) -> str:
    """Folder name that encodes the hyper-parameters of the run.

    Same fields, in the same order, as ``dl_code/pcode/utils/checkpoint.py:14-56``."""
    time_id = str(int(time.time()))
    if conf.comm_op is None:
        comm_info = ""
    elif "compress" in conf.comm_op:
        comm_info = "{}-{}_".format(conf.comm_op, conf.compress_ratio)
        comm_info += "warmup_epochs-{}".format(conf.compress_warmup_epochs)
        comm_info += "_mask_momentum" if conf.mask_momentum else ""
        comm_info += "_clip_grad-{}".format(conf.clip_grad_val) if conf.clip_grad else ""
    elif conf.comm_op == "quantize_qsgd":
        comm_info = "{}-{}_".format(conf.comm_op, conf.quantize_level)
    elif conf.comm_op == "sign":
        comm_info = "{}_".format(conf.comm_op)
    else:
        comm_info = ""
    if "choco" in conf.optimizer:
        optim_info = "{}-stepsize-{}".format(conf.optimizer, conf.consensus_stepsize)
    else:
        optim_info = str(conf.optimizer)
    return (
        time_id
        + "_l2-{}_lr-{}_epochs-{}_batchsize-{}_basebatchsize-{}_num_mpi_process_{}"
        "_n_sub_process-{}_topology-{}_optim-{}_comm_info-{}".format(
            conf.weight_decay,
            conf.lr,
            conf.num_epochs,
            conf.batch_size,
            conf.base_batch_size,
            conf.n_mpi_process,
            conf.n_sub_process,
            conf.graph_topology,
            optim_info,
            comm_info,
        )
    )


def get_args(argv: Optional[Sequence[str]] = None, strict: bool = False) -> Config:
    """Parse ``argv`` (default ``sys.argv[1:]``) into a :class:`Config`.

    Unknown ``--flag value`` pairs are tolerated unless ``strict`` is set: the
    reference's own example scripts pass several that its parser rejects
    (``dl_code/exps/finetune-resnet50-imagenet/example.sh:11-12``)."""
    parser = build_parser()
    conf = Config()
    _, unknown = parser.parse_known_args(argv, namespace=conf)
    if unknown:
        if strict:
            parser.error("unrecognized arguments: " + " ".join(unknown))
        warnings.warn("ignoring unrecognized arguments: " + " ".join(unknown))
    conf._unknown = list(unknown)
    if conf.graph_topology not in TOPOLOGIES:
        warnings.warn(
            f"unknown graph_topology {conf.graph_topology!r}; falling back to 'complete'"
        )
        conf.graph_topology = "complete"
    if conf.timestamp is None:
        conf.timestamp = default_timestamp(conf)
    return conf


def validate(conf: Config) -> None:
    """Fail fast on inconsistent combinations (the convex code does this with asserts,
    ``convex_code/parameters.py:34-71``; the deep-learning code does not)."""
    needs_op = ("parallel_choco", "parallel_choco_v", "dcd_psgd", "ecd_psgd", "deep_squeeze", "dgc")
    if conf.optimizer in needs_op and conf.comm_op is None:
        raise ValueError(f"--optimizer {conf.optimizer} needs --comm_op")
    if conf.comm_op in ("compress_top_k", "compress_random_k"):
        if conf.compress_ratio is None or not (0.0 <= conf.compress_ratio < 1.0):
            raise ValueError("--compress_ratio (fraction dropped) must be in [0, 1)")
    if conf.comm_op == "quantize_qsgd" and conf.quantize_level is None and conf.qsgd_levels is None:
        raise ValueError("quantize_qsgd needs --quantize_level (bits) or --qsgd_levels (s)")
    if conf.use_nesterov and conf.momentum_factor <= 0:
        raise ValueError("Nesterov momentum requires a momentum")
    if conf.n_sub_process > 1:
        # The reference gives a graph node several GPUs by wrapping its model in torch.nn.DataParallel
        # (dl_code/main.py:79-81): one process scattering batches and gathering gradients every step.
        # Here every GPU is a process with its own flat arena, captured step and peer mailboxes; use
        # n_mpi_process = number of GPUs (for 8 nodes x 4 GPUs: 32 ranks, e.g. on the torus graph).
        raise ValueError("--n_sub_process > 1 is not supported: run one rank per GPU (raise --n_mpi_process and, "
                         "to keep the global batch, leave --batch_size per GPU as it is)")
