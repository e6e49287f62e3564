"""Fused CHOCO-SGD engine: launches the hand-written gossip kernels.

``ChocoEngine`` owns everything the kernels need besides the optimizer's flat buffers:
the chunk / segment tables, the device-resident hyper-parameters and step counters, the
outbox, the peer-mapped mailbox and the ``ChocoParams`` blocks in device memory.  One
engine drives one logical rank per GPU in production (``for_optimizer``) or all logical
ranks of a graph on one GPU (``LoopbackWorld``, used to test the very same kernels without
NVLink).

Per training step the engine launches (everything on the current stream, capturable in a
CUDA graph because the step index and learning rate live in device memory):

=========  ====================================================================================
sign       1 kernel  ``choco_sign_step`` (decode t-1, SGD, consensus, compress, push, publish)
qsgd       2 kernels ``choco_dense_prep`` + ``choco_qsgd_pack``
top-k      wait + (deg+1) sparse decodes + prep + 2 histogram passes + count + emit
random-k   wait + (deg+1) sparse decodes + prep + emit
=========  ====================================================================================

No ``torch.distributed`` call and no stand-alone elementwise kernel is on this path
(the reference: ``dl_code/pcode/optim/parallel_choco_v.py:104-155``, ~65-161 per-tensor op
sequences plus three flatten/unflatten copies and ``isend``/``irecv`` per step).
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..compress.reference import qsgd_levels_from, qsgd_nbits
from ..compress.segments import Segments
from ..parallel.symm import DistributedMailbox, LoopbackMailbox, MailboxView
from ..utils.error_handler import GossipTimeout
from . import _lib

MODE_DECODE, MODE_PUSH = 1, 2
CODEC_ID = {"sign": 3, "quantize_qsgd": 0, "compress_top_k": 1, "compress_random_k": 2, "raw": 4}
HYP_LR, HYP_MOMENTUM, HYP_GAMMA, HYP_NESTEROV, HYP_GSCALE, HYP_N = 0, 1, 2, 3, 4, 8


def pick_chunk_elems(total: int) -> int:
    """Elements per CTA: as large as possible (the per-CTA prologue / publish epilogue is a fixed
    cost) while keeping about two waves of CTAs on 148 SMs x 8 resident CTAs."""
    c = 1024
    while c < 32768 and total // (2 * c) >= 2400:
        c *= 2
    return c


class SegTables:
    """Host-built chunk / segment tables, uploaded once."""

    def __init__(self, seg: Segments, weight_decay: Sequence[float], ks: Optional[Sequence[int]], device,
                 chunk_elems: Optional[int] = None):
        self.seg = seg
        ce = chunk_elems or pick_chunk_elems(seg.total)
        chunk_seg, chunk_start, chunk_valid, first, count = [], [], [], [], []
        for t, (off, n) in enumerate(zip(seg.offsets, seg.sizes)):
            first.append(len(chunk_seg))
            done = 0
            while done < n:
                v = min(ce, n - done)
                chunk_seg.append(t)
                chunk_start.append(off + done)
                chunk_valid.append(v)
                done += v
            count.append(len(chunk_seg) - first[-1])
        ks = list(ks) if ks is not None else [0] * seg.n_segments
        koff = np.concatenate([[0], np.cumsum(ks)[:-1]]) if ks else np.zeros(0)

        def dev(a, dt):
            return torch.as_tensor(np.asarray(a, dtype=dt), device=device)

        self.chunk_elems = ce
        self.n_chunks = len(chunk_seg)
        self.sum_k = int(sum(ks))
        self.t = {
            "chunk_seg": dev(chunk_seg, np.int32),
            "chunk_start": dev(chunk_start, np.int32),
            "chunk_valid": dev(chunk_valid, np.int32),
            "seg_start": dev(seg.offsets, np.int32),
            "seg_size": dev(seg.sizes, np.int32),
            "seg_first_chunk": dev(first, np.int32),
            "seg_n_chunks": dev(count, np.int32),
            "seg_wd": dev(list(weight_decay), np.float32),
            "seg_k": dev(ks, np.int32),
            "seg_koff": dev(koff, np.int32),
        }

    def fill(self, c: _lib.SegTableC):
        for k, v in self.t.items():
            setattr(c, k, v.data_ptr())
        c.n_chunks, c.n_segments = self.n_chunks, self.seg.n_segments
        c.chunk_elems, c.total = self.chunk_elems, self.seg.total


ALLREDUCE = "allreduce"


class ArPlanC(ctypes.Structure):
    _fields_ = [("n_world", ctypes.c_int), ("my_rank", ctypes.c_int), ("shard_words", ctypes.c_int),
                ("slot_of", ctypes.c_int * (_lib.MAX_PEERS + 1))]


class RankBuffers:
    """Flat state of one logical rank (all fp32, length ``seg.total``)."""

    def __init__(self, x, g, m, x_hat, s):
        self.x, self.g, self.m, self.x_hat, self.s = x, g, m, x_hat, s


def payload_layout(comm_op: str, seg: Segments, sum_k: int, nbits: int):
    """-> (payload_words, body_off)."""
    header = (seg.n_segments + 31) // 32 * 32
    if comm_op is None:
        return 32, 0
    if comm_op == "sign":
        return header + seg.total // 32, header
    if comm_op == "quantize_qsgd":
        return header + (seg.total // 32) * (nbits + 1), header
    if comm_op == "compress_top_k":
        return 2 * sum_k, 0
    if comm_op == "compress_random_k":
        return sum_k, 0
    if comm_op == "raw":  # full-precision exchange (D-PSGD)
        return seg.total, 0
    raise NotImplementedError(comm_op)


class ChocoEngine:
    def __init__(
        self,
        ranks: List[int],
        buffers: Dict[int, RankBuffers],
        neighborhoods: Dict[int, Dict[int, float]],
        seg: Segments,
        weight_decay: Sequence[float],
        comm_op: str,
        mailbox,
        device,
        compress_ratio: Optional[float] = None,
        quantize_level: Optional[int] = None,
        qsgd_levels: Optional[int] = None,
        is_biased: bool = False,
        seed: int = 1234,
        wait_budget_ms: float = 2000.0,
        chunk_elems: Optional[int] = None,
        coop: Optional[bool] = None,
    ):
        if comm_op is not None and comm_op != ALLREDUCE and comm_op not in CODEC_ID:
            raise NotImplementedError(f"fused gossip kernels do not cover comm_op={comm_op!r}")
        self.lib = _lib.load()
        self.device = torch.device(device)
        # comm_op None: local fused SGD only (no payloads, no mailbox traffic)
        self.comm_op, self.codec = comm_op, CODEC_ID.get(comm_op, -1)
        self.ranks, self.buffers, self.seg = list(ranks), buffers, seg
        self.n_local = len(self.ranks)
        ks = seg.keep_counts(compress_ratio) if (comm_op and "compress" in comm_op) else None
        self.tables = SegTables(seg, weight_decay, ks, self.device, chunk_elems)
        self.s_levels = qsgd_levels_from(quantize_level, qsgd_levels) if comm_op == "quantize_qsgd" else 1
        self.nbits = qsgd_nbits(self.s_levels) if comm_op == "quantize_qsgd" else 0
        if not (0 <= self.nbits <= 30 and 0 < self.s_levels < 2 ** 31):
            raise ValueError(f"QSGD with {self.s_levels} levels does not fit the packed format (at most 30 bits)")
        if comm_op == ALLREDUCE:
            # two-shot all-reduce: one shard of scattered gradients + one shard of averages per slot
            self.n_world = len(neighborhoods[self.ranks[0]])
            assert all(sorted(neighborhoods[r]) == list(range(self.n_world)) for r in self.ranks), \
                "the fused all-reduce needs the complete graph over ranks 0..n-1"
            self.shard_words = -(-self.tables.n_chunks // self.n_world) * self.tables.chunk_elems
            self.payload_words, self.body_off = 2 * self.shard_words, 0
        else:
            self.payload_words, self.body_off = payload_layout(comm_op, seg, self.tables.sum_k, self.nbits)
        self.mailbox = mailbox(self.payload_words) if callable(mailbox) else mailbox
        peers_max = max(len([j for j in neighborhoods[r] if j != r]) for r in self.ranks)
        if peers_max > _lib.MAX_PEERS:
            raise ValueError(f"a rank has {peers_max} neighbours; the fused kernels support {_lib.MAX_PEERS}")
        self.max_peers = peers_max
        same = all(len([j for j in neighborhoods[r] if j != r]) == peers_max for r in self.ranks)
        self.peers_hint = peers_max if (same and peers_max in (0, 1, 2, 3, 4, 7)) else -1

        T, nc, dev = seg.n_segments, self.tables.n_chunks, self.device
        z = lambda n, dt: torch.zeros(n, dtype=dt, device=dev)
        self.hyper = z(HYP_N, torch.float32)
        # Staging for the hyper-parameter refresh: a ring of pinned slots, each guarded by an event
        # recorded after its copy, so the host never rewrites a slot whose (asynchronous) copy has
        # not run yet while it keeps enqueuing steps with a changing learning rate.
        n_slots = 16 if dev.type == "cuda" else 1
        self._hyper_ring = [torch.zeros(HYP_N, dtype=torch.float32) for _ in range(n_slots)]
        if dev.type == "cuda":
            self._hyper_ring = [t.pin_memory() for t in self._hyper_ring]
        self._hyper_events = [None] * n_slots
        self._hyper_slot = 0
        self.hyper_host = self._hyper_ring[0]
        self.hyper_host[HYP_GSCALE] = 1.0
        self.hyper.copy_(self.hyper_host)
        self._hyper_sent = None
        self.per_rank = {}
        blocks = []
        sparse = self.codec in (1, 2)
        for r in self.ranks:
            b = buffers[r]
            res = {
                "step": z(4, torch.int32),
                "seg_count": z(T, torch.int32),
                "done_count": z(8, torch.int32),
                "partial": z(nc, torch.float32),
                "status": z(4, torch.int32),
                "outbox": z(2 * self.payload_words, torch.int32),
                "scratch_d": z(seg.total, torch.float32) if self.codec in (0, 1, 2) else None,
                "hist": z(T * self.lib.choco_hist_words(), torch.int32) if self.codec == 1 else None,
                "chunk_cnt": z(2 * nc, torch.int32) if self.codec == 1 else None,
                "sel": z(4 * T, torch.int32) if self.codec == 1 else None,
            }
            self.per_rank[r] = res
            view: MailboxView = self.mailbox.view(r)
            nb = neighborhoods[r]
            c = _lib.ChocoParamsC()
            c.x, c.g, c.m, c.x_hat, c.s = (t.data_ptr() for t in (b.x, b.g, b.m, b.x_hat, b.s))
            c.scratch_d = res["scratch_d"].data_ptr() if res["scratch_d"] is not None else 0
            c.outbox = res["outbox"].data_ptr()
            for k, j in enumerate(view.peers):
                c.peer_inbox[k], c.peer_flag[k] = view.peer_inbox[k], view.peer_flag[k]
                c.my_inbox[k], c.my_flag[k] = view.my_inbox[k], view.my_flag[k]
                c.w_peer[k] = float(nb[j])
                c.peer_rank[k] = int(j)
            c.hyper = self.hyper.data_ptr()
            for name in ("step", "seg_count", "done_count", "partial", "status"):
                setattr(c, name, res[name].data_ptr())
            for name in ("hist", "chunk_cnt", "sel"):
                setattr(c, name, res[name].data_ptr() if res[name] is not None else 0)
            c.wait_budget_ns = int(wait_budget_ms * 1e6)
            self.tables.fill(c.tab)
            c.w_self = float(nb[r])
            c.n_peers = len(view.peers)
            c.payload_words, c.body_off, c.rank = self.payload_words, self.body_off, int(r)
            c.seed = (int(seed) + 7919 * int(r)) & 0xFFFFFFFF
            c.qsgd_s, c.qsgd_nbits, c.qsgd_biased = int(self.s_levels), int(self.nbits), int(bool(is_biased))
            blocks.append(c)
        self._structs = blocks
        self._grad_tables = {}
        if comm_op == ALLREDUCE:
            self._init_allreduce()
        raw = np.frombuffer(b"".join(bytes(c) for c in blocks), dtype=np.uint8).copy()
        self.params = torch.from_numpy(raw).to(dev)
        self._pp = ctypes.c_void_p(self.params.data_ptr())
        self._steps = 0
        self.sparse = sparse
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        self.entry_blocks = max(1, min(8 * sms, (self.tables.sum_k + 255) // 256)) if sparse else 1
        # Sparsifying codecs of plain CHOCO-SGD can run the whole step as ONE cooperative kernel (grid
        # barriers instead of launch boundaries): ``coop=True`` / CHOCO_SPARSE_COOP=1.  Off by default:
        # replayed from a CUDA graph the chain of kernels measured faster on B200 at every size (top-k
        # 82 us against 107 us at 1 Mi elements, 315 against 539 at 16 Mi; random-k 29 against 29 and
        # 124 against 170; the ResNet-20 step 1.003 ms against 1.028 ms) - a grid barrier costs about what a
        # graph edge costs, and a co-resident grid has far fewer CTAs in flight for the streaming phases.
        self.coop, self.coop_grid = False, 0
        if sparse and type(self) is ChocoEngine:
            want = coop
            if want is None:
                want = os.environ.get("CHOCO_SPARSE_COOP", "0") not in ("0", "off", "auto")
            if want:
                self._init_coop(sms)

    # ---- construction helpers --------------------------------------------------------------
    @classmethod
    def for_optimizer(cls, opt, group=None):
        """Engine of one rank of a distributed run (one process per GPU)."""
        conf, graph = opt.conf, opt.graph
        if opt.momentum_buf is None:
            opt.momentum_buf = torch.zeros_like(opt.arena.x)
        bufs = {graph.rank: RankBuffers(opt.arena.x, opt.arena.g, opt.momentum_buf, opt.x_hat, opt.s)}
        nbh = {graph.rank: graph.get_neighborhood()}
        wd = [g["weight_decay"] for g in opt.param_groups]
        if graph.n_nodes > 1:
            mailbox = lambda pw: DistributedMailbox(graph, pw, opt.device, group)
        else:
            mailbox = lambda pw: LoopbackMailbox({graph.rank: []}, pw, opt.device)
        return cls(
            [graph.rank], bufs, nbh, opt.seg, wd, conf.comm_op, mailbox, opt.device,
            compress_ratio=conf.compress_ratio, quantize_level=conf.quantize_level,
            qsgd_levels=getattr(conf, "qsgd_levels", None), is_biased=conf.is_biased,
            seed=getattr(conf, "random_k_seed", 1234), wait_budget_ms=getattr(conf, "wait_budget_ms", 2000.0),
        )

    def set_grad_pointers(self, rank, grads: Optional[Sequence[torch.Tensor]]):
        """Let the kernels read each tensor's gradient where autograd left it (one contiguous,
        16-byte aligned fp32 tensor per parameter) instead of a packed flat buffer.
        ``None`` switches back to the flat gradient."""
        i = self.ranks.index(rank)
        if grads is None:
            self._grad_tables.pop(rank, None)
            self._structs[i].seg_g = 0
        else:
            assert len(grads) == self.seg.n_segments
            for gt, n in zip(grads, self.seg.sizes):
                assert gt.dtype == torch.float32 and gt.numel() == n
                assert gt.data_ptr() % 16 == 0
            table = torch.tensor([gt.data_ptr() for gt in grads], dtype=torch.int64).to(self.device)
            self._grad_tables[rank] = (table, list(grads))
            self._structs[i].seg_g = table.data_ptr()
        raw = np.frombuffer(b"".join(bytes(c) for c in self._structs), dtype=np.uint8).copy()
        self.params.copy_(torch.from_numpy(raw), non_blocking=False)

    # ---- hyper-parameters ---------------------------------------------------------------------
    def set_hyper(self, lr, momentum, gamma, nesterov):
        key = (float(lr), float(momentum), float(gamma), bool(nesterov))
        if key == self._hyper_sent:
            return
        i = self._hyper_slot = (self._hyper_slot + 1) % len(self._hyper_ring)
        if self._hyper_events[i] is not None:
            self._hyper_events[i].synchronize()  # the copy that last used this slot has completed
        h = self.hyper_host = self._hyper_ring[i]
        h[HYP_LR], h[HYP_MOMENTUM], h[HYP_GAMMA], h[HYP_NESTEROV] = key[0], key[1], key[2], 1.0 if key[3] else 0.0
        # slots 0..3 only: slot 4 (gradient scale) is written by the clipping kernel
        self.hyper[:4].copy_(h[:4], non_blocking=True)
        if self.device.type == "cuda":
            ev = self._hyper_events[i] or torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.device))
            self._hyper_events[i] = ev
        self._hyper_sent = key

    # ---- launches ---------------------------------------------------------------------------------
    launches_per_step = 0
    _n_launch = 0

    def _init_coop(self, sms):
        L = self.lib
        L.choco_sparse_coop_max_grid.argtypes = [ctypes.c_int]
        L.choco_sparse_coop_max_grid.restype = ctypes.c_int
        L.choco_sparse_coop_step.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                             ctypes.c_void_p]
        L.choco_sparse_coop_step.restype = ctypes.c_int
        with torch.cuda.device(self.device):
            cap = L.choco_sparse_coop_max_grid(self.n_local)
        if cap < 1:
            return  # cannot be made co-resident (many logical ranks on one device): keep the chain
        work = max(self.tables.n_chunks, self.entry_blocks)
        # one CTA per SM at most: more CTAs make every grid barrier slower than the phase it ends
        self.coop_grid = max(1, min(work, cap, max(1, sms // self.n_local)))
        self.coop = True

    def _chk(self, code, what):
        self._n_launch += 1
        _lib.count(1)
        _lib.check(code, what)

    def launch_step(self, stream=None):
        """All kernels of one CHOCO step on ``stream`` (default: current)."""
        L, pp, nc, nr = self.lib, self._pp, self.tables.n_chunks, self.n_local
        sp = _lib.stream_ptr(stream)
        self._n_launch = 0
        if self.codec == 3:
            self._chk(L.choco_sign_step(pp, nc, nr, MODE_DECODE | MODE_PUSH, self.peers_hint, sp), "choco_sign_step")
        elif self.codec == 0:
            self._chk(L.choco_dense_prep(pp, nc, nr, MODE_DECODE, 0, sp), "choco_dense_prep")
            self._chk(L.choco_qsgd_pack_nbits(pp, nc, nr, int(self.nbits), sp), "choco_qsgd_pack")
        elif self.coop:
            self._chk(L.choco_sparse_coop_step(pp, self.coop_grid, nr, self.codec, 3, sp), "choco_sparse_coop_step")
        else:
            self._launch_sparse_decode(sp)
            self._chk(L.choco_dense_prep(pp, nc, nr, 0, self.codec, sp), "choco_dense_prep")
            if self.codec == 1:
                self._chk(L.choco_topk_hist(pp, nc, nr, 2, sp), "choco_topk_hist2")
                self._chk(L.choco_topk_hist(pp, nc, nr, 3, sp), "choco_topk_hist3")
                self._chk(L.choco_topk_count(pp, nc, nr, sp), "choco_topk_count")
                self._chk(L.choco_topk_emit(pp, nc, nr, sp), "choco_topk_emit")
            else:
                self._chk(L.choco_randk_emit(pp, self.entry_blocks, nr, sp), "choco_randk_emit")
        self._steps += 1
        self.launches_per_step = self._n_launch

    # ---- a step issued bucket by bucket (sign codec) ------------------------------------------------
    def segment_chunk_range(self, seg_first: int, seg_last: int):
        """Chunks of the segments ``seg_first .. seg_last`` (inclusive): ``(first chunk, count)``."""
        first = self.tables.t["seg_first_chunk"][seg_first:seg_last + 1].tolist()
        count = self.tables.t["seg_n_chunks"][seg_first:seg_last + 1].tolist()
        return int(first[0]), int(first[-1] + count[-1] - first[0])

    def launch_step_range(self, chunk0: int, n_chunks: int, stream=None, last: bool = False):
        """The sign-codec step for the chunks ``[chunk0, chunk0 + n_chunks)`` only.  All ranges of a step
        together must cover every chunk exactly once; the range that completes the arena publishes the
        step on the device (whichever it is), ``last=True`` closes the host-side accounting."""
        if self.codec != 3:
            raise NotImplementedError("range launches exist for the sign codec")
        self._chk(self.lib.choco_sign_step_range(self._pp, int(chunk0), int(n_chunks), self.n_local,
                                                 MODE_DECODE | MODE_PUSH, self.peers_hint, _lib.stream_ptr(stream)),
                  "choco_sign_step_range")
        if last:
            self._steps += 1
            self.launches_per_step = self._n_launch

    def _launch_sparse_decode(self, sp):
        """One launch per source payload (own, then each neighbour: sources are applied one after the other so
        that s stays reproducible); the first also waits for the neighbours' flags, the last records completion."""
        L, pp, nr = self.lib, self._pp, self.n_local
        last = self.max_peers - 1
        for src in range(-1, self.max_peers):
            flags = (1 if src == -1 else 0) | (2 if src == last else 0)
            self._chk(L.choco_sparse_decode_ex(pp, self.entry_blocks, nr, src, self.codec, flags, sp), "choco_sparse_decode")

    def launch_decode(self, stream=None):
        """Apply the payloads of the last push to x_hat / s (end of training, checkpoints)."""
        L, pp, nc, nr = self.lib, self._pp, self.tables.n_chunks, self.n_local
        sp = _lib.stream_ptr(stream)
        if self.codec == 3:
            self._chk(L.choco_sign_step(pp, nc, nr, MODE_DECODE, self.peers_hint, sp), "choco_sign_decode")
        elif self.codec == 0:
            self._chk(L.choco_qsgd_decode(pp, nc, nr, sp), "choco_qsgd_decode")
        elif self.coop:
            self._chk(L.choco_sparse_coop_step(pp, self.coop_grid, nr, self.codec, 1, sp), "choco_sparse_coop_decode")
        else:
            self._launch_sparse_decode(sp)

    def _init_allreduce(self):
        L = self.lib
        L.allreduce_sgd_step.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
        plans = []
        for r in self.ranks:
            pl = ArPlanC()
            pl.n_world, pl.my_rank, pl.shard_words = self.n_world, int(r), self.shard_words
            peers = self.mailbox.view(r).peers
            for j in range(_lib.MAX_PEERS + 1):
                pl.slot_of[j] = peers.index(j) if j in peers else -1
            plans.append(pl)
        assert L.ar_plan_size() == ctypes.sizeof(ArPlanC), "ArPlan layout mismatch"
        raw = np.frombuffer(b"".join(bytes(c) for c in plans), dtype=np.uint8).copy()
        self._plans = torch.from_numpy(raw).to(self.device)
        with torch.cuda.device(self.device):
            cap = L.allreduce_sgd_max_grid(self.n_local)
        if cap < 1:
            raise RuntimeError("the fused all-reduce kernel cannot be made co-resident on this device")
        self.ar_grid = max(1, min(self.tables.n_chunks, cap))

    def launch_allreduce_sgd(self, stream=None):
        """Gradient averaging over all ranks + momentum-SGD update, one kernel."""
        self._n_launch = 0
        self._chk(self.lib.allreduce_sgd_step(self._pp, ctypes.c_void_p(self._plans.data_ptr()), self.ar_grid,
                                              self.n_local, _lib.stream_ptr(stream)), "allreduce_sgd_step")
        self._steps += 1
        self.launches_per_step = 1

    def launch_sgd_only(self, apply=True, stream=None):
        self._chk(
            self.lib.fused_sgd_step(self._pp, self.tables.n_chunks, self.n_local, 1 if apply else 0,
                                    _lib.stream_ptr(stream)),
            "fused_sgd_step",
        )
        self.launches_per_step = 1

    # ---- optimizer-facing API ----------------------------------------------------------------------
    def step(self, opt):
        self.set_hyper(opt.lr, opt.momentum, opt.consensus_stepsize, opt.nesterov)
        self.launch_step()
        bits = opt.n_bits
        opt.n_bits = opt.codec.n_bits()
        opt.gossip_step += 1
        return bits

    def flush(self, opt=None):
        self.launch_decode()
        self.check()

    def reset_step(self, step: int):
        for r in self.ranks:
            st = self.per_rank[r]["step"]
            st[0], st[2] = int(step), int(step)
            st[1] = 1 if step > 0 else 0

    def momentum_flags(self):
        return [int(self.per_rank[r]["step"][1]) for r in self.ranks]

    def set_momentum_flags(self, flags):
        for r, f in zip(self.ranks, flags):
            self.per_rank[r]["step"][1] = int(f)

    def rebase_time(self):
        """Hook for engines whose update rule depends on the step index (see ``AlgoEngine``)."""

    def check(self):
        """Read the status words (synchronises); raise on a timed-out wait."""
        for r in self.ranks:
            code, peer, step, _ = self.per_rank[r]["status"].tolist()
            if code != 0:
                raise GossipTimeout(code, peer, step)

    def step_index(self, rank=None) -> int:
        r = self.ranks[0] if rank is None else rank
        return int(self.per_rank[r]["step"][0])

    def close(self):
        if hasattr(self.mailbox, "close"):
            self.mailbox.close()


class LoopbackWorld:
    """All ``n`` logical ranks of a graph on ONE GPU: the production kernels run with
    gridDim.y = n and "peer" pointers that are local, so flags, parities, payload layouts and
    the arithmetic are exercised without NVLink.  State tensors are ``[n, total]``."""

    def __init__(self, w: np.ndarray, seg: Segments, x0: torch.Tensor, comm_op: str, weight_decay, device="cuda",
                 **codec_kw):
        n = w.shape[0]
        self.n, self.seg, self.device = n, seg, torch.device(device)
        mk = lambda: torch.zeros(n, seg.total, dtype=torch.float32, device=self.device)
        self.x, self.g, self.m, self.x_hat, self.s = mk(), mk(), mk(), mk(), mk()
        self.x.copy_(x0.to(self.device) if x0.dim() == 2 else x0.to(self.device).repeat(n, 1))
        nbh = {i: {j: float(w[i, j]) for j in range(n) if (w[i, j] != 0 or j == i)} for i in range(n)}
        peers = {i: [j for j in nbh[i] if j != i] for i in range(n)}
        bufs = {i: RankBuffers(self.x[i], self.g[i], self.m[i], self.x_hat[i], self.s[i]) for i in range(n)}
        wd = weight_decay if hasattr(weight_decay, "__len__") else [weight_decay] * seg.n_segments
        self.engine = ChocoEngine(
            list(range(n)), bufs, nbh, seg, wd, comm_op, lambda pw: LoopbackMailbox(peers, pw, self.device),
            self.device, **codec_kw,
        )

    def step(self, grads: torch.Tensor, lr, momentum, gamma, nesterov):
        self.g.copy_(grads.to(self.device))
        self.engine.set_hyper(lr, momentum, gamma, nesterov)
        if self.engine.comm_op == ALLREDUCE:
            self.engine.launch_allreduce_sgd()
        else:
            self.engine.launch_step()

    def flush(self):
        if self.engine.comm_op == ALLREDUCE:
            return self.engine.check()
        self.engine.flush()
