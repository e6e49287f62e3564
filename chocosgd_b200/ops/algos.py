"""Engine of the fused steps of D-PSGD, DCD-PSGD, ECD-PSGD, DeepSqueeze, DGC and EF-signSGD
(``csrc/algos.cu``).

``AlgoEngine`` extends ``ChocoEngine``: same flat buffers, segment tables, wire formats,
mailboxes and device-resident step counter; the algorithm-specific state (neighbour replicas,
error memory) is described by one ``AlgoParams`` block per logical rank.  Launches per step
(all on the current stream, capturable in a CUDA graph):

=========  ==========================================================================
sign/raw   ``algo_prep`` (packs and pushes) + ``algo_apply_dense``
qsgd       ``algo_prep`` + ``choco_qsgd_pack`` + ``algo_apply_dense``
top-k      ``algo_prep`` + 2 histograms + count + emit + wait + (deg + 1) sparse applies + mark
random-k   ``algo_prep`` + emit + wait + (deg + 1) sparse applies + mark
=========  ==========================================================================

The reference runs these algorithms as per-tensor PyTorch op sequences around blocking
``isend`` / ``irecv`` (``dl_code/pcode/optim/{dcd_psgd,ecd_psgd,deep_squeeze,dgc,ef_sign_sgd}.py``).
"""
from __future__ import annotations

import ctypes
from typing import Dict, List, Optional

import numpy as np
import torch

from ..compress.segments import Segments
from ..parallel.symm import LoopbackMailbox
from . import _lib
from .gossip import ChocoEngine, RankBuffers

ALGO_ID = {"dcd_psgd": 1, "ecd_psgd": 2, "deep_squeeze": 3, "dgc": 4, "ef_sign_sgd": 5, "dpsgd": 6}
RAW = "raw"


class AlgoParamsC(ctypes.Structure):
    _fields_ = [
        ("hat", ctypes.c_void_p * (_lib.MAX_PEERS + 1)),
        ("mem", ctypes.c_void_p),
        ("inv_world", ctypes.c_float),
        ("mask_momentum", ctypes.c_int),
        ("use_memory", ctypes.c_int),
        ("t_offset", ctypes.c_int),
    ]


def _declare():
    lib = _lib.load()
    if not getattr(lib, "_algos_declared", False):
        vp, i = ctypes.c_void_p, ctypes.c_int
        lib.algo_prep.argtypes = [vp, vp, i, i, i, i, vp]
        lib.algo_apply_dense.argtypes = [vp, vp, i, i, i, i, vp]
        lib.algo_apply_sparse.argtypes = [vp, vp, i, i, i, i, i, vp]
        for n in ("algo_prep", "algo_apply_dense", "algo_apply_sparse", "algo_params_size"):
            getattr(lib, n).restype = i
        assert lib.algo_params_size() == ctypes.sizeof(AlgoParamsC), "AlgoParams layout mismatch"
        lib._algos_declared = True
    return lib


class AlgoEngine(ChocoEngine):
    def __init__(self, algo: str, ranks, buffers, neighborhoods, seg, weight_decay, comm_op, mailbox, device,
                 hats: Optional[Dict[int, Dict[int, torch.Tensor]]] = None,
                 mems: Optional[Dict[int, torch.Tensor]] = None,
                 n_world: int = 1, mask_momentum: bool = False, use_memory: bool = True, **kw):
        self.algo = ALGO_ID[algo]
        if (comm_op == RAW) != (algo == "dpsgd"):
            raise ValueError("the raw payload belongs to D-PSGD and only to it")
        if algo == "ef_sign_sgd" and comm_op != "sign":
            raise ValueError("EF-signSGD uses the sign codec")
        super().__init__(ranks, buffers, neighborhoods, seg, weight_decay, comm_op, mailbox, device, **kw)
        _declare()
        blocks = []
        for r in self.ranks:
            c = AlgoParamsC()
            peers = self.mailbox.view(r).peers
            if hats is not None:
                c.hat[0] = hats[r][r].data_ptr()
                for k, j in enumerate(peers):
                    c.hat[1 + k] = hats[r][j].data_ptr()
            c.mem = mems[r].data_ptr() if mems is not None else 0
            c.inv_world = 1.0 / float(n_world)
            c.mask_momentum, c.use_memory = int(bool(mask_momentum)), int(bool(use_memory and mems is not None))
            blocks.append(c)
        self._algo_structs, self._keep = blocks, (hats, mems)
        raw = np.frombuffer(b"".join(bytes(c) for c in blocks), dtype=np.uint8).copy()
        self.algo_params = torch.from_numpy(raw).to(self.device)
        self._ap = ctypes.c_void_p(self.algo_params.data_ptr())

    def launch_step(self, stream=None):
        L, pp, ap, nc, nr = self.lib, self._pp, self._ap, self.tables.n_chunks, self.n_local
        sp = _lib.stream_ptr(stream)
        self._n_launch = 0
        codec = self.codec
        self._chk(L.algo_prep(pp, ap, nc, nr, self.algo, codec, sp), "algo_prep")
        if codec == 0:
            self._chk(L.choco_qsgd_pack_nbits(pp, nc, nr, int(self.nbits), sp), "choco_qsgd_pack")
        elif codec == 1:
            self._chk(L.choco_topk_hist(pp, nc, nr, 2, sp), "choco_topk_hist2")
            self._chk(L.choco_topk_hist(pp, nc, nr, 3, sp), "choco_topk_hist3")
            self._chk(L.choco_topk_count(pp, nc, nr, sp), "choco_topk_count")
            self._chk(L.choco_topk_emit(pp, nc, nr, sp), "choco_topk_emit")
        elif codec == 2:
            self._chk(L.choco_randk_emit(pp, self.entry_blocks, nr, sp), "choco_randk_emit")
        if codec in (0, 3, 4):
            self._chk(L.algo_apply_dense(pp, ap, nc, nr, self.algo, codec, sp), "algo_apply_dense")
        else:
            self._chk(L.choco_wait_flags(pp, nr, sp), "choco_wait_flags")
            for src in range(-1, self.max_peers):
                self._chk(L.algo_apply_sparse(pp, ap, self.entry_blocks, nr, self.algo, src, codec, sp),
                          "algo_apply_sparse")
            self._chk(L.choco_sparse_decode(pp, 1, nr, 1000, codec, sp), "choco_mark_decoded")
        self._steps += 1
        self.launches_per_step = self._n_launch

    def rebase_time(self):
        """Make the current device step count the origin of the algorithm's own step index (ECD-PSGD
        weights its updates by t): used after warm-up steps whose effects were rolled back."""
        now = self.step_index()
        for c in self._algo_structs:
            c.t_offset = int(now)
        raw = np.frombuffer(b"".join(bytes(c) for c in self._algo_structs), dtype=np.uint8).copy()
        self.algo_params.copy_(torch.from_numpy(raw))

    def launch_decode(self, stream=None):
        return None  # the exchange of a step is applied inside the step

    def flush(self, opt=None):
        self.check()

    def reset_step(self, step: int):
        """After loading a checkpoint taken at algorithm step ``step``: the device counter keeps
        counting pushes of this process (it pairs with the mailbox flags), the offset maps it back."""
        now = self.step_index()
        for c in self._algo_structs:
            c.t_offset = int(now) - int(step)
        raw = np.frombuffer(b"".join(bytes(c) for c in self._algo_structs), dtype=np.uint8).copy()
        self.algo_params.copy_(torch.from_numpy(raw))
        for r in self.ranks:
            self.per_rank[r]["step"][1] = 1 if step > 0 else 0


class AlgoLoopbackWorld:
    """All logical ranks of a graph on ONE GPU running the fused kernels of ``algo`` (tests)."""

    def __init__(self, algo: str, w: np.ndarray, seg: Segments, x0: torch.Tensor, comm_op, weight_decay,
                 device="cuda", mask_momentum=False, **codec_kw):
        n = w.shape[0]
        self.n, self.seg, self.device, self.algo = n, seg, torch.device(device), algo
        mk = lambda: torch.zeros(n, seg.total, dtype=torch.float32, device=self.device)
        self.x, self.g, self.m = mk(), mk(), mk()
        self.x.copy_(x0.to(self.device) if x0.dim() == 2 else x0.to(self.device).repeat(n, 1))
        nbh = {i: {j: float(w[i, j]) for j in range(n) if (w[i, j] != 0 or j == i)} for i in range(n)}
        peers = {i: [j for j in nbh[i] if j != i] for i in range(n)}
        dummy = torch.zeros(32, device=self.device)
        bufs = {i: RankBuffers(self.x[i], self.g[i], self.m[i], dummy, dummy) for i in range(n)}
        self.hats = self.mems = None
        if algo in ("dcd_psgd", "ecd_psgd"):
            self.hats = {i: {j: self.x[i].clone() for j in nbh[i]} for i in range(n)}
        use_memory = True
        if algo in ("deep_squeeze", "ef_sign_sgd", "dgc"):
            use_memory = algo != "dgc" or (comm_op is not None and "compress" in comm_op)
            self.mem = mk()
            self.mems = {i: self.mem[i] for i in range(n)}
        wd = weight_decay if hasattr(weight_decay, "__len__") else [weight_decay] * seg.n_segments
        self.engine = AlgoEngine(
            algo, list(range(n)), bufs, nbh, seg, wd, comm_op, lambda pw: LoopbackMailbox(peers, pw, self.device),
            self.device, hats=self.hats, mems=self.mems, n_world=n, mask_momentum=mask_momentum,
            use_memory=use_memory, **codec_kw)

    def step(self, grads: torch.Tensor, lr, momentum, gamma, nesterov):
        self.g.copy_(grads.to(self.device))
        self.engine.set_hyper(lr, momentum, gamma, nesterov)
        self.engine.launch_step()

    def flush(self):
        self.engine.flush()
