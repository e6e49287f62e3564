"""Common machinery of the distributed optimizers.

Construction mirrors ``dl_code/pcode/create_optimizer.py:13-52``: one param-group per
parameter tensor carrying ``name``, ``weight_decay`` (0 when the name contains ``"bn"``),
``param_size`` and ``nelement``; ``lr`` / ``momentum`` / ``nesterov`` from the config.
``step(timer=..., scheduler=...)`` returns the number of bits transmitted, as in the
reference (e.g. ``dl_code/pcode/optim/sgd.py:67-122``).

Unlike the reference, all algorithm state (x_hat, s, replicas, error memories, step
counters) is part of ``state_dict()`` so a resumed run continues the same trajectory.
"""
from __future__ import annotations

import contextlib
from typing import Dict, Optional

import torch
from torch.optim.optimizer import Optimizer

from ..compress.reference import make_codec
from ..parallel.comm import CentralizedAggregation, DecentralizedAggregation
from .arena import FlatArena


class _NullTimer:
    @contextlib.contextmanager
    def __call__(self, *a, **k):
        yield


def build_param_groups(model, weight_decay: float):
    groups = []
    for name, p in model.named_parameters():
        if not p.requires_grad:
            continue
        groups.append(
            {
                "params": [p],
                "name": name,
                "weight_decay": weight_decay if "bn" not in name else 0.0,
                "param_size": p.size(),
                "nelement": p.nelement(),
            }
        )
    return groups


class DistributedOptimizer(Optimizer):
    #: labels of the timer scopes this algorithm emits (observability contract).
    timer_labels = ()

    def __init__(self, model, conf, graph, group=None):
        groups = build_param_groups(model, conf.weight_decay)
        defaults = dict(
            lr=conf.lr,
            momentum=conf.momentum_factor,
            dampening=0,
            weight_decay=conf.weight_decay,
            nesterov=conf.use_nesterov,
        )
        if conf.use_nesterov and conf.momentum_factor <= 0:
            raise ValueError("Nesterov momentum requires a momentum and zero dampening")
        super().__init__(groups, defaults)
        self.conf = conf
        self.graph = graph
        self.rank = graph.rank
        self.n_nodes = graph.n_nodes
        self.neighbors_info: Dict[int, float] = graph.get_neighborhood()
        self.param_names = list(enumerate(g["name"] for g in self.param_groups))
        self.arena = FlatArena([(g["name"], g["params"][0]) for g in self.param_groups])
        self.seg = self.arena.seg
        self.device = self.arena.device
        self.wd_vec = self.arena.per_element([g["weight_decay"] for g in self.param_groups])
        self.momentum_buf: Optional[torch.Tensor] = None  # flat, created on first use
        self.local_index = 0  # number of completed step() calls
        self.n_bits = 0
        self.world_aggregator = CentralizedAggregation(
            self.rank, graph.ranks, {r: 1.0 / graph.n_nodes for r in graph.ranks}, group
        )
        self.decentralized_aggregator = DecentralizedAggregation(self.rank, self.neighbors_info, group)
        self._epoch_override = None
        self.group = group
        self._exchange = None
        self._gather = None

    # ---- transports ----------------------------------------------------------------------
    def _mailbox_ok(self) -> bool:
        import torch.distributed as dist

        return (self.device.type == "cuda" and self.n_nodes > 1 and dist.is_available() and dist.is_initialized()
                and getattr(self.conf, "gossip_impl", "auto") != "nccl")

    def neighbor_exchange(self):
        """Transport of neighbour payloads: peer-mapped mailboxes written from inside kernels
        on NVLink, ``torch.distributed`` send/recv otherwise (CPU / Gloo, ``--gossip_impl nccl``)."""
        if self._exchange is None:
            if self._mailbox_ok() and len(self.neighbors_info) - 1 <= 16:
                from ..parallel.exchange import MailboxExchange

                self._exchange = MailboxExchange(self.graph, self.seg.total, self.device, self.group,
                                                 getattr(self.conf, "wait_budget_ms", 2000.0))
            else:
                self._exchange = self.decentralized_aggregator
        return self._exchange

    def gather_payloads(self, payload):
        """Payloads of all ranks in rank order (all-gather; by mailbox push on NVLink)."""
        if self._gather is None:
            if self._mailbox_ok() and self.n_nodes - 1 <= 16:
                from ..parallel.exchange import MailboxExchange
                from ..parallel.topology import Graph

                full = Graph("complete", self.n_nodes, self.rank)
                self._gather = MailboxExchange(full, self.seg.total, self.device, self.group,
                                               getattr(self.conf, "wait_budget_ms", 2000.0))
            else:
                self._gather = False
        if self._gather is False:
            return self.world_aggregator._agg(payload, communication_scheme="all_gather")
        return self._gather.all_gather(payload)

    # ---- fused kernels of the non-CHOCO algorithms (ops/algos.py) ------------------------
    engine = None
    gamma_for_engine = 0.0

    def fused_wanted(self) -> bool:
        """True when the step should run in the hand-written kernels: a CUDA device, not the
        ``--gossip_impl nccl`` baseline, and (for more than one node) peer mailboxes available."""
        want = getattr(self.conf, "gossip_impl", "auto")
        if self.device.type != "cuda" or want in ("nccl", "torch"):
            return False
        if self.identity_quantizer():
            return False  # 32-bit "quantization" is the identity: nothing for the packed formats to do
        return self.n_nodes == 1 or self._mailbox_ok()

    def identity_quantizer(self) -> bool:
        c = self.conf
        return (c.comm_op == "quantize_qsgd" and getattr(c, "qsgd_levels", None) is None
                and c.quantize_level is not None and int(c.quantize_level) >= 32)

    def build_algo_engine(self, algo, comm_op, complete=False, hats=None, mem=None, **kw):
        """Engine of one rank (one process per GPU).  ``complete``: the payload goes to every rank
        (all-gather by push) instead of the graph neighbours."""
        from ..ops.algos import AlgoEngine
        from ..ops.gossip import RankBuffers
        from ..parallel.symm import DistributedMailbox, LoopbackMailbox
        from ..parallel.topology import Graph

        conf, r = self.conf, self.rank
        graph = Graph("complete", self.n_nodes, r) if complete else self.graph
        nbh = {r: graph.get_neighborhood()}
        if len(nbh[r]) - 1 > 16:
            raise ValueError("the fused kernels support at most 16 peers per rank")
        if self.momentum_buf is None:
            self.momentum_buf = torch.zeros_like(self.arena.x)
        dummy = torch.zeros(32, device=self.device)
        bufs = {r: RankBuffers(self.arena.x, self.arena.g, self.momentum_buf, dummy, dummy)}
        if self.n_nodes > 1:
            mailbox = lambda pw: DistributedMailbox(graph, pw, self.device, self.group)
        else:
            mailbox = lambda pw: LoopbackMailbox({r: []}, pw, self.device)
        return AlgoEngine(
            algo, [r], bufs, nbh, self.seg, [g["weight_decay"] for g in self.param_groups], comm_op, mailbox,
            self.device, hats={r: hats} if hats is not None else None, mems={r: mem} if mem is not None else None,
            n_world=self.n_nodes, compress_ratio=conf.compress_ratio, quantize_level=conf.quantize_level,
            qsgd_levels=getattr(conf, "qsgd_levels", None), is_biased=conf.is_biased,
            seed=getattr(conf, "random_k_seed", 1234), wait_budget_ms=getattr(conf, "wait_budget_ms", 2000.0), **kw)

    @property
    def capturable(self) -> bool:
        return self.engine is not None

    def prepare_step(self):
        """Host side of a fused step: refresh the device-resident hyper-parameters, account bits."""
        self.local_index += 1
        self.engine.set_hyper(self.lr, self.momentum, self.gamma_for_engine, self.nesterov)
        self.n_bits = self.codec.n_bits() if getattr(self, "codec", None) is not None else 32 * self.seg.n_elements
        return self.n_bits

    def launch(self, stream=None):
        """Device side of a fused step: the kernels, nothing else (what a CUDA graph captures)."""
        self.engine.launch_step(stream)

    def fused_step(self, timer, ep, label):
        with timer(label, epoch=ep):
            bits = self.prepare_step()
            self.launch()
        return bits

    def check(self):
        """Raise ``GossipTimeout`` if a bounded device-side wait of any transport of this optimizer
        ran out (synchronises the device)."""
        if self.engine is not None:
            self.engine.check()
        for ex in (self._exchange, self._gather):
            if ex is not None and ex is not False and hasattr(ex, "check"):
                ex.check()

    # ---- hyper-parameters ------------------------------------------------------------
    @property
    def lr(self) -> float:
        return float(self.param_groups[0]["lr"])

    @property
    def momentum(self) -> float:
        return float(self.param_groups[0]["momentum"])

    @property
    def nesterov(self) -> bool:
        return bool(self.param_groups[0]["nesterov"])

    def make_codec(self, compress_ratio=None):
        c = self.conf
        return make_codec(
            self.seg,
            c.comm_op,
            c.compress_ratio if compress_ratio is None else compress_ratio,
            c.quantize_level,
            getattr(c, "qsgd_levels", None),
            c.is_biased,
            getattr(c, "random_k_seed", 1234),
        )

    def epoch_of(self, kargs) -> float:
        sch = kargs.get("scheduler")
        if sch is not None and hasattr(sch, "epoch_"):
            return float(sch.epoch_)
        return float(kargs.get("epoch", 0.0))

    @staticmethod
    def timer_of(kargs):
        t = kargs.get("timer")
        return t if t is not None else _NullTimer()

    # ---- local momentum-SGD direction ---------------------------------------------------
    def local_direction(self) -> torch.Tensor:
        """d' of ``apply_gradient`` on the flat buffers (``dl_code/pcode/optim/utils.py:13-47``):
        d = g + wd x; buf = d on the first call, mu buf + d later; d' = d + mu buf | buf.
        Consumes (zeroes) the gradient buffer."""
        a = self.arena
        d = torch.addcmul(a.g, self.wd_vec, a.x)
        mu = self.momentum
        if mu != 0:
            if self.momentum_buf is None:
                self.momentum_buf = d.clone()
            else:
                self.momentum_buf.mul_(mu).add_(d)
            d = d.add(self.momentum_buf, alpha=mu) if self.nesterov else self.momentum_buf.clone()
        a.g.zero_()
        return d

    def zero_grad(self, set_to_none: bool = False):
        # gradients alias the arena; they are cleared when consumed by step().
        self.arena.g.zero_()

    # ---- checkpointing ---------------------------------------------------------------
    def algo_state(self) -> dict:
        return {}

    def load_algo_state(self, state: dict):
        pass

    def state_dict(self):
        groups = []
        for i, g in enumerate(self.param_groups):
            gg = {k: v for k, v in g.items() if k != "params"}
            gg["params"] = [i]
            gg["param_size"] = tuple(g["param_size"])
            groups.append(gg)
        state = {}
        if self.momentum_buf is not None:
            for i, sl in enumerate(self.seg.slices()):
                view = self.arena._view(self.momentum_buf[sl], self.param_groups[i]["param_size"],
                                        self.arena.channels_last[i])
                state[i] = {"momentum_buffer": view.detach().clone()}
        algo = {k: (v.detach().clone() if torch.is_tensor(v) else v) for k, v in self.algo_state().items()}
        algo["local_index"] = self.local_index
        return {"state": state, "param_groups": groups, "algo_state": algo}

    def load_state_dict(self, sd):
        for g, lg in zip(self.param_groups, sd["param_groups"]):
            for k in ("lr", "momentum", "dampening", "weight_decay", "nesterov"):
                if k in lg:
                    g[k] = lg[k]
        self.wd_vec = self.arena.per_element([g["weight_decay"] for g in self.param_groups])
        st = sd.get("state", {})
        if st:
            if self.momentum_buf is None:
                self.momentum_buf = torch.zeros_like(self.arena.x)
            else:
                self.momentum_buf.zero_()  # in place: the fused kernels hold its address
            for i, sl in enumerate(self.seg.slices()):
                ent = st.get(i, st.get(str(i)))
                if ent is not None and "momentum_buffer" in ent:
                    self.arena._view(self.momentum_buf[sl], self.param_groups[i]["param_size"],
                                     self.arena.channels_last[i]).copy_(ent["momentum_buffer"])
        algo = dict(sd.get("algo_state", {}))
        self.local_index = int(algo.pop("local_index", 0))
        self.load_algo_state(algo)
        if self.engine is not None and hasattr(self.engine, "algo"):
            self.engine.reset_step(self.local_index)
        self.arena.rebind()

    def finalize(self):
        """Complete any communication still in flight (end of training / before a checkpoint)
        and surface a timed-out wait."""
        self.check()
